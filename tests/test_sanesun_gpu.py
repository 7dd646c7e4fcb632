"""GPU: the Sanesun model class on the ragged step engine against the plain float64 statement in oracle/sanesun_ref.py.

Small configurations with random weights; sizes are chosen so that nothing is a multiple of a warp, a page or a key
chunk by accident (kv heads fewer than heads in attention AND in the delta rule, head sizes 12 / 20 / 33 / 72, more
heads than one pass of the attention kernel takes, convolutions of 1, 2 and 4 taps, windows of 5, 9 and 33 tokens, a
window shorter than the kept prefix, rotary over part of a head and over all of it, a layer without a feed-forward).
Where random weights would hide a fault the inputs are made so that it shows: one key among hundreds gets a score
that dominates, keys sit just inside and just outside a window or the kept prefix, the sink is made large.
"""
import math

import pytest
import torch

import dgi_b200  # noqa: F401
from oracle import sanesun_ref as R

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64


def attn(heads, kv, dim, vdim, size, keep, rot_dims, base=10000.0, scale=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim,
                                           "scale": scale or 1.0 / math.sqrt(dim), "mask": {"size": size, "keep_first": keep},
                                           "rot": {"base": base, "dims": rot_dims}}}


def latent(heads, dim, vdim, kv_rank, q_rank, scale=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank,
                                                  "q_rank": q_rank, "scale": scale or 1.0 / math.sqrt(dim)}}


def delta(heads, kv, dim, vdim, conv):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def with_mlp(layer, ff):
    layer = dict(layer)
    layer["mlp"] = {"kind": "dense", "ff": ff} if ff else None
    return layer


CFG_A = {
    "architecture": "Sanesun", "width": 56, "vocab": 53, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "layers": [
        with_mlp(delta(4, 2, 12, 20, 4), 72),
        with_mlp(attn(4, 2, 24, 20, 9, 3, 12, base=50.0, scale=0.3), None),
        with_mlp(latent(3, 10, 14, 18, 22, scale=0.4), 40),
        with_mlp(attn(6, 6, 16, 36, 33, 0, 16), 24),
        with_mlp(delta(2, 2, 40, 33, 2), 16),
    ],
}
CFG_B = {  # other order; ten heads (two passes of the attention kernel) mixed by one matrix; a one-tap convolution;
           # a window shorter than the kept prefix; a latent wider than 64
    "architecture": "Sanesun", "width": 40, "vocab": 37, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "layers": [
        with_mlp(latent(5, 6, 10, 72, 12), None),
        with_mlp(attn(10, 5, 8, 12, 5, 40, 4, base=300.0), 33),
        with_mlp(delta(3, 1, 16, 8, 1), 20),
        with_mlp(attn(2, 1, 40, 130, 17, 2, 40), 20),
    ],
}


CFG_C = {  # sizes the tensor-core attention takes in 16-bit storage: a value width below its tile (48 of 64) that is
           # turned back, twelve mixed heads over four kv heads, a latent whose one pool serves both products
    "architecture": "Sanesun", "width": 64, "vocab": 41, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
    "layers": [
        with_mlp(attn(4, 2, 32, 48, 19, 3, 16, base=200.0), 48),
        with_mlp(latent(10, 16, 24, 64, 40), 32),
        with_mlp(delta(2, 1, 32, 32, 3), None),
        with_mlp(attn(12, 4, 16, 128, 40, 0, 16), 32),
        with_mlp(latent(3, 8, 8, 80, 24), None),
    ],
}


def build(cfg_raw, dtype=torch.float32, seed=0, max_tokens=512, max_seqs=4):
    from dgi_b200 import sanesun_layer as S
    from dgi_b200.ragged_engine import RaggedStepEngine

    cfg = S.SanesunConfig.from_dict(cfg_raw)
    tensors = S.random_checkpoint(cfg, seed=seed)
    shards = S.build_shards(cfg, tensors, [(0, cfg.num_hidden_layers)], DEV, dtype)
    return RaggedStepEngine(shards, max_tokens=max_tokens, max_seqs=max_seqs), tensors


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def whole(engine, rid, toks, want=None):
    want = list(range(len(toks))) if want is None else want
    out = engine.step([(rid, toks, want)]).cpu()
    engine.finish(rid)
    return out


def close(got, ref, tol):
    err = (got.to(F64) - ref.to(F64)).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()), f"max abs error {err}"


def paged(k, v, bs=16, seed=0):
    """Pools holding ``k [n, G, dk]`` / ``v [n, G, dv]`` in shuffled blocks, and the block table that finds them."""
    n, G, dk = k.shape
    nb = (n + bs - 1) // bs
    perm = torch.randperm(nb + 3, generator=torch.Generator().manual_seed(seed))[:nb]
    kp = torch.full((nb + 3, G, bs, dk), float("nan"), dtype=k.dtype)
    vp = torch.full((nb + 3, G, bs, v.shape[2]), float("nan"), dtype=v.dtype)
    for t in range(n):
        kp[perm[t // bs], :, t % bs] = k[t]
        vp[perm[t // bs], :, t % bs] = v[t]
    # rows of the last block past the sequence are never visible; leave them NaN to prove it
    return kp.to(DEV), vp.to(DEV), perm.to(torch.int32).view(1, -1).to(DEV)


def run_attention(q, k, v, scale, rows, **kw):
    from dgi_b200 import mixer_ops as M

    n, H, _ = q.shape
    kp, vp, table = paged(k, v)
    rows_t = torch.tensor(rows, dtype=torch.int64)
    out = torch.empty((len(rows), H, v.shape[2]), dtype=q.dtype, device=DEV)
    for name in ("talk", "sink"):
        if kw.get(name) is not None:
            kw[name] = kw[name].to(torch.float32).to(DEV)
    M.mixed_paged_attention(out, q[rows_t].to(DEV), kp, vp, table, torch.zeros(len(rows), dtype=torch.int32, device=DEV),
                            rows_t.to(torch.int32).to(DEV), scale, **kw)
    return out.cpu()


# ---- mechanisms alone ----------------------------------------------------------------------------------------------

def test_norm_residual_update_and_activation():
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(1)
    x, a, b = (torch.randn(7, 50, generator=g) for _ in range(3))
    w = 1 + 0.2 * torch.randn(50, generator=g)
    for dt, tol in ((torch.float32, 2e-6), (torch.bfloat16, 1e-2)):
        wd, ad, bd = w.to(dt), a.to(dt), b.to(dt)
        close(M.rms_norm(x.to(DEV), wd.to(DEV), 1e-5).float().cpu(), R.rms_norm(x.to(F64), wd.to(F64), 1e-5), tol)
        wide = torch.cat([ad, bd], dim=1).to(DEV)                      # a column slice of a wider activation
        close(M.rms_norm(wide[:, 50:], wd.to(DEV), 1e-5).float().cpu(), R.rms_norm(bd.to(F64), wd.to(F64), 1e-5), tol)
        xd = x.to(DEV).clone()
        nxt = M.residual_add2_norm(xd, ad.to(DEV), bd.to(DEV), wd.to(DEV), 1e-5)
        ref = x.to(F64) + (ad.to(F64) + bd.to(F64))
        close(xd.cpu(), ref, 2e-6)                                     # the residual is fp32 for every storage dtype
        close(nxt.float().cpu(), R.rms_norm(ref, wd.to(F64), 1e-5), tol)
        xd = x.to(DEV).clone()
        assert M.residual_add2_norm(xd, ad.to(DEV), None, None, 1e-5) is None
        close(xd.cpu(), x.to(F64) + ad.to(F64), 2e-6)
    z = torch.randn(5, 77, generator=g) * 3
    pq = torch.tensor([0.7, -1.2])
    close(M.xielu(z.to(DEV), pq.to(DEV)).cpu(), R.xielu(z.to(F64), pq[0].to(F64), pq[1].to(F64)), 3e-6)
    small = torch.tensor([[1e-4, -1e-4, 0.0, -30.0, 12.0]])              # both branches near zero and far out
    close(M.xielu(small.to(DEV), pq.to(DEV)).cpu(), R.xielu(small.to(F64), pq[0].to(F64), pq[1].to(F64)), 1e-6)


@pytest.mark.parametrize("interleaved", [False, True])
def test_rotary_append_turns_q_k_and_values(interleaved):
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(2)
    n, H, G, dk, dv, dims, base, bs = 21, 4, 2, 20, 14, 12, 70.0, 16
    q, k, v = torch.randn(n, H * dk, generator=g), torch.randn(n, G * dk, generator=g), torch.randn(n, G * dv, generator=g)
    pos = torch.tensor([5000 + 3 * i for i in range(n)], dtype=torch.int32)    # large positions: angles need care
    kp = torch.zeros(4, G, bs, dk, device=DEV)
    vp = torch.zeros(4, G, bs, dv, device=DEV)
    slots = torch.tensor([(3 - i // bs) * bs + i % bs for i in range(n)], dtype=torch.int64)
    qd = q.to(DEV).clone()
    M.rotary_kv_append(qd, k.to(DEV), v.to(DEV), kp, vp, slots.to(DEV), pos.to(DEV), H, dims, base, True, interleaved)
    close(qd.cpu(), R.turn(q.to(F64).view(n, H, dk), pos, dims, base, interleaved=interleaved).reshape(n, -1), 2e-6)
    want_k = R.turn(k.to(F64).view(n, G, dk), pos, dims, base, interleaved=interleaved)
    want_v = R.turn(v.to(F64).view(n, G, dv), pos, dv, base, interleaved=interleaved)
    for i in range(n):
        close(kp[3 - i // bs, :, i % bs].cpu(), want_k[i], 2e-6)
        close(vp[3 - i // bs, :, i % bs].cpu(), want_v[i], 2e-6)


def test_attention_window_edges_kept_prefix_sink_and_head_mixing():
    g = torch.Generator().manual_seed(3)
    n, H, G, dk, dv, size, keep = 150, 4, 2, 24, 20, 32, 5
    q, k, v = torch.randn(n, H, dk, generator=g), torch.randn(n, G, dk, generator=g), torch.randn(n, G, dv, generator=g)
    talk = torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)
    sink = torch.randn(H, generator=g)
    # for query 140: the key just inside the window (109), just outside (108), the last kept one (4) and the first
    # that is not kept (5) are all made to dominate; only two of them may be seen
    i = 140
    for j in (i - size + 1, i - size, keep - 1, keep):
        k[j] = 6.0 * q[i].view(G, H // G, dk)[:, 0] / q[i].view(G, H // G, dk)[:, 0].norm(dim=-1, keepdim=True)
    rows = [0, 1, keep, size - 1, size, size + keep, 99, i, n - 1]
    got = run_attention(q, k, v, 0.35, rows, talk=talk, sink=sink, window=size, keep_first=keep)
    ref = R.windowed_attention(q.to(F64), k.to(F64), v.to(F64), 0.35, size, keep, talk.to(F64), sink.to(F64), rows=rows)
    close(got, ref[rows], 3e-6)
    blind = R.windowed_attention(q.to(F64), k.to(F64), v.to(F64), 0.35, size + 1, keep + 1, talk.to(F64), sink.to(F64), rows=[i])
    assert (ref[i] - blind[i]).abs().max() > 0.05          # the test would notice a window or a prefix that is one off
    # a large sink takes nearly all the weight; no sink and no mixing is plain attention
    big = torch.full((H,), 30.0)
    got = run_attention(q, k, v, 0.35, [i], sink=big, window=size, keep_first=keep)
    assert got.abs().max() < 1e-6
    got = run_attention(q, k, v, 0.35, rows)
    close(got, R.windowed_attention(q.to(F64), k.to(F64), v.to(F64), 0.35, rows=rows)[rows], 3e-6)


def test_attention_finds_one_far_key_among_hundreds():
    g = torch.Generator().manual_seed(4)
    n, H, dk = 700, 3, 72                                      # one latent "head" serves all query heads
    q, c = torch.randn(n, H, dk, generator=g), torch.randn(n, 1, dk, generator=g)
    far, i = 37, n - 1
    c[far, 0] = 9.0 * q[i, 1] / q[i, 1].norm()
    gate = torch.randn(n, H, generator=g)
    from dgi_b200 import mixer_ops as M

    kp, _, table = paged(c, c)
    rows = [far, 300, i]
    rows_t = torch.tensor(rows)
    out = torch.empty((H, len(rows), dk), device=DEV)          # head-major output, as the latent mixer asks for it
    M.mixed_paged_attention(out.transpose(0, 1), q[rows_t].to(DEV), kp, kp, table,
                            torch.zeros(len(rows), dtype=torch.int32, device=DEV), rows_t.to(torch.int32).to(DEV), 0.2,
                            gate=gate[rows_t].to(DEV))
    ref = R.windowed_attention(q.to(F64), c.to(F64), c.to(F64), 0.2, rows=rows)[rows] * torch.sigmoid(gate[rows_t].to(F64))[:, :, None]
    close(out.transpose(0, 1).cpu(), ref, 3e-6)
    w = torch.softmax((c[: i + 1, 0].to(F64) @ q[i, 1].to(F64)) * 0.2, 0)
    assert w[far] > 0.9                                        # the far key really carries the answer


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
@pytest.mark.parametrize("H,G,dk,dv,mixing", [(4, 2, 32, 48, True), (12, 4, 16, 128, True), (20, 20, 16, 64, True),
                                              (3, 1, 64, 64, False), (10, 2, 48, 256, False)])
def test_tensor_core_attention_matches_the_statement(dt, H, G, dk, dv, mixing):
    """The 16-bit kernel for portions and single tokens: window and prefix edges inside one 16-token tile, tiles that
    straddle pages and key tiles, a needle just inside and just outside, turned-back outputs, gates."""
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(8)
    n, size, keep, base = 200, 37, 5, 90.0
    q, k, v = (torch.randn(n, x, d, generator=g).to(dt) for x, d in ((H, dk), (G, dk), (G, dv)))
    i = 170
    for j in (i - size + 1, i - size):          # seen / hidden needle for head 0's group
        k[j, 0] = (5.0 * q[i, 0].float() / q[i, 0].float().norm()).to(dt)
    talk = (torch.eye(H) + 0.3 * torch.randn(H, H, generator=g) / math.sqrt(H)) if mixing else None
    sink = torch.randn(H, generator=g) if mixing else None
    gate = None if mixing else torch.randn(n, H, generator=g).to(dt)
    assert M.mixed_prompt_attention_supported(H, G, dk, dv, mixing, False, mixing, dt)
    pos = torch.arange(n)
    vt = R.turn(v.to(F64), pos, dv, base).to(dt) if mixing else v            # stored turned, as the append leaves them
    kp, vp, table = paged(k, vt)
    tab = None
    if mixing:
        ang = pos.to(F64)[:, None] * base ** (-2.0 * torch.arange(dv // 2, dtype=F64) / dv)
        tab = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().to(DEV)
    # tiles: whole 16-token runs from 0, a run cut at an odd place, single tokens at the end
    cuts = [16] * 5 + [3, 13, 16, 16, 16, 16, 7, 9] + [1] * 24
    assert sum(cuts) == n
    tiles, at = [], 0
    for c in cuts:
        tiles.append((at, c, 0))
        at += c
    out = torch.full((n, H, dv), float("nan"), dtype=dt, device=DEV)
    M.mixed_prompt_attention(out, q.to(DEV), kp, vp, table, torch.tensor(tiles, dtype=torch.int32, device=DEV),
                             pos.to(torch.int32).to(DEV), 0.3, talk=None if talk is None else talk.to(DEV),
                             sink=None if sink is None else sink.to(DEV), window=size, keep_first=keep, value_rot=tab,
                             gate=None if gate is None else gate.to(DEV))
    rows = [0, 1, keep, 15, 16, 17, size - 1, size, size + keep, 95, 96, 97, i, n - 25, n - 24, n - 1]
    ref = R.windowed_attention(q.to(F64), k.to(F64), vt.to(F64), 0.3, size, keep, None if talk is None else talk.to(F64),
                               None if sink is None else sink.to(F64), rows=rows)
    if mixing:
        ref = R.turn(ref, pos, dv, base, back=True)
    else:
        ref = ref * torch.sigmoid(gate.to(F64))[:, :, None]
    got = out.cpu().to(F64)
    assert torch.isfinite(got).all()
    err = (got[rows] - ref[rows]).abs().max().item()
    assert err <= 2e-2 * max(1.0, ref[rows].abs().max().item()), err
    # the same step with its keys divided over several CTAs and merged (what steps of few tokens do); the hint is made
    # large so that some CTAs get no key tile at all
    out3 = torch.full((n, H, dv), float("nan"), dtype=dt, device=DEV)
    M.mixed_prompt_attention(out3, q.to(DEV), kp, vp, table, torch.tensor(tiles, dtype=torch.int32, device=DEV),
                             pos.to(torch.int32).to(DEV), 0.3, talk=None if talk is None else talk.to(DEV),
                             sink=None if sink is None else sink.to(DEV), window=size, keep_first=keep, value_rot=tab,
                             gate=None if gate is None else gate.to(DEV), max_context=1 << 14)
    assert (out3.float() - out.float()).abs().max().item() <= 1e-2 * max(1.0, ref[rows].abs().max().item())
    # the row kernel is the fp32 / odd-size fallback for the same operation: both agree on every row
    out2 = torch.empty_like(out)
    M.mixed_paged_attention(out2, q.to(DEV), kp, vp, table, torch.zeros(n, dtype=torch.int32, device=DEV),
                            pos.to(torch.int32).to(DEV), 0.3, talk=None if talk is None else talk.to(DEV),
                            sink=None if sink is None else sink.to(DEV), window=size, keep_first=keep,
                            unrotate_base=base if mixing else None, gate=None if gate is None else gate.to(DEV))
    assert (out2.float() - out.float()).abs().max().item() <= 2e-2 * max(1.0, ref[rows].abs().max().item())


def test_tensor_core_latent_attention_reads_one_pool_for_keys_and_values():
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(9)
    n, H, r = 300, 5, 128
    q, c = torch.randn(n, H, r, generator=g).bfloat16(), torch.randn(n, 1, r, generator=g).bfloat16()
    far, i = 21, n - 1
    c[far, 0] = (9.0 * q[i, 2].float() / q[i, 2].float().norm()).bfloat16()
    kp, _, table = paged(c, c)
    tiles = torch.tensor([(lo, min(16, n - lo), 0) for lo in range(0, n, 16)], dtype=torch.int32, device=DEV)
    out = torch.empty((H, n, r), dtype=torch.bfloat16, device=DEV)            # head-major, as the latent mixer has it
    M.mixed_prompt_attention(out.transpose(0, 1), q.to(DEV), kp, kp, table, tiles,
                             torch.arange(n, dtype=torch.int32, device=DEV), 0.09)
    rows = [0, 15, 16, far, 150, i]
    ref = R.windowed_attention(q.to(F64), c.to(F64), c.to(F64), 0.09, rows=rows)
    got = out.transpose(0, 1).cpu().to(F64)
    assert (got[rows] - ref[rows]).abs().max().item() <= 2e-2 * ref[rows].abs().max().item()
    # three decoded tokens of long contexts: few CTAs, so the keys are split and merged
    last = torch.tensor([n - 3, n - 2, n - 1])
    out = torch.empty((H, 3, r), dtype=torch.bfloat16, device=DEV)
    M.mixed_prompt_attention(out.transpose(0, 1), q[last].to(DEV), kp, kp, table.expand(3, -1).contiguous(),
                             torch.tensor([(0, 1, 0), (1, 1, 1), (2, 1, 2)], dtype=torch.int32, device=DEV),
                             last.to(torch.int32).to(DEV), 0.09, max_context=n)
    assert M._lib_().b200_mixed_prompt_attn_splits(3, (n + 31) // 32, H, 1, r, r, 0, 1, 0, 2) > 1
    ref = R.windowed_attention(q.to(F64), c.to(F64), c.to(F64), 0.09, rows=last.tolist())
    assert (out.transpose(0, 1).cpu().to(F64) - ref[last]).abs().max().item() <= 2e-2 * ref[last].abs().max().item()
    w = torch.softmax((c[: i + 1, 0].to(F64) @ q[i, 2].to(F64)) * 0.09, 0)
    assert w[far] > 0.9


def test_value_rotation_cancels_to_the_distance():
    """Values stored turned by j and read back turned by -i: a lone visible key returns its value turned by j - i."""
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(5)
    n, H, dk, dv, base = 40, 2, 8, 12, 30.0
    q, k, v = torch.randn(n, H, dk, generator=g), torch.randn(n, H, dk, generator=g), torch.randn(n, H, dv, generator=g)
    pos = torch.arange(n)
    vt = R.turn(v.to(F64), pos, dv, base)
    rows = [0, 7, 39]
    got = run_attention(q, k, vt.float(), 0.3, rows, window=1, unrotate_base=base)     # window 1: only j = i is seen
    close(got, v[rows], 3e-6)
    got = run_attention(q, k, vt.float(), 0.3, rows, window=6, keep_first=2, unrotate_base=base)
    ref = R.turn(R.windowed_attention(q.to(F64), k.to(F64), vt, 0.3, 6, 2, rows=rows), pos, dv, base, back=True)
    close(got, ref[rows], 3e-6)


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_short_convolution_carries_its_inputs_between_steps(taps):
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(6)
    C, n = 150, 90
    x, w = torch.randn(n, C, generator=g), torch.randn(C, taps, generator=g)
    ref = R.causal_conv_silu(x.to(F64), w.to(F64))
    tail = torch.full((3, taps - 1, C), float("nan"), device=DEV)       # a fresh sequence never reads its slot
    got, at, first = [], 0, 1
    for cut in (1, 1, 2, 70, 3, 1, 12):                                 # portions shorter than the taps too
        seqs = torch.tensor([[0, cut, 2, first]], dtype=torch.int32, device=DEV)
        got.append(M.causal_conv_silu(x[at:at + cut].to(DEV), w.to(DEV), tail, seqs, cut))
        at, first = at + cut, 0
    assert at == n
    close(torch.cat(got).cpu(), ref, 3e-6)


@pytest.mark.parametrize("H,G,dk,dv", [(4, 2, 12, 20), (2, 2, 40, 33), (1, 1, 130, 64)])
def test_delta_rule_state_through_portions(H, G, dk, dv):
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(7)
    n = 75
    qkv = torch.randn(n, 2 * G * dk + H * dv, generator=g)
    beta, a = torch.randn(n, H, generator=g), torch.randn(n, H * dk, generator=g)
    dt_bias, a_log = torch.randn(H * dk, generator=g) - 1, torch.rand(H, generator=g) - 1
    q, k = qkv[:, :G * dk].to(F64).view(n, G, dk), qkv[:, G * dk:2 * G * dk].to(F64).view(n, G, dk)
    qn = (q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5).repeat_interleave(H // G, 1)
    kn = (k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(H // G, 1)
    gd = torch.exp(-torch.exp(a_log.to(F64))[None, :, None] * R.softplus((a + dt_bias).to(F64).view(n, H, dk)))
    ref = R.delta_rule(qn, kn, qkv[:, 2 * G * dk:].to(F64).view(n, H, dv), torch.sigmoid(beta.to(F64)), gd)
    state = torch.full((2, H, dk, dv), float("nan"), device=DEV)
    d = qkv.to(DEV)
    got, at, first = [], 0, 1
    for cut in (1, 2, 5, 40, 1, 1, 25):
        seqs = torch.tensor([[0, cut, 1, first]], dtype=torch.int32, device=DEV)
        s = d[at:at + cut]
        got.append(M.delta_scan(s[:, :G * dk], s[:, G * dk:2 * G * dk], s[:, 2 * G * dk:], beta[at:at + cut].to(DEV),
                                a[at:at + cut].to(DEV), dt_bias.to(DEV), a_log.to(DEV), state, seqs, G, 1e-6, dk ** -0.5))
        at, first = at + cut, 0
    close(torch.cat(got).cpu(), ref, 1e-5)
    w, gate = 1 + 0.1 * torch.randn(dv, generator=g), torch.randn(n, H * dv, generator=g)
    normed = M.head_rmsnorm_gated(torch.cat(got), w.to(DEV), gate.to(DEV), 1e-5).cpu()
    want = ref / torch.sqrt((ref * ref).mean(-1, keepdim=True) + 1e-5) * w.to(F64) * torch.sigmoid(gate.to(F64)).view(n, H, dv)
    close(normed, want.reshape(n, -1), 1e-5)


# ---- whole models ----------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("cfg", [CFG_A, CFG_B, CFG_C], ids=["A", "B", "C"])
def test_whole_prompt_fp32(cfg):
    engine, tensors = build(cfg)
    toks = tokens(90, cfg["vocab"], 11)
    close(whole(engine, "a", toks), R.forward(cfg, tensors, toks), 3e-5)
    one = tokens(1, cfg["vocab"], 12)                            # the first token alone
    close(whole(engine, "b", one), R.forward(cfg, tensors, one), 3e-5)


@pytest.mark.parametrize("cfg", [CFG_A, CFG_B, CFG_C], ids=["A", "B", "C"])
def test_whole_prompt_bf16(cfg):
    engine, tensors = build(cfg, dtype=torch.bfloat16)
    toks = tokens(70, cfg["vocab"], 13)
    ref = R.forward(cfg, tensors, toks)
    got = whole(engine, "a", toks)
    assert (got.to(F64) - ref).pow(2).mean().sqrt() <= 0.03 * ref.pow(2).mean().sqrt()


@pytest.mark.parametrize("cfg", [CFG_A, CFG_B], ids=["A", "B"])
def test_prefill_then_long_decode_matches_the_whole_prompt(cfg):
    engine, tensors = build(cfg)
    toks = tokens(120, cfg["vocab"], 14)
    ref = R.forward(cfg, tensors, toks)
    got = [engine.step([("a", toks[:30], list(range(30)))])]
    for t in range(30, len(toks)):                               # 90 decoded tokens: every window passes over them
        got.append(engine.step([("a", [toks[t]], [0])]))
    engine.finish("a")
    close(torch.cat(got).cpu(), ref, 3e-5)
    got = [engine.step([("b", [t], [0])]) for t in toks[:40]]    # decoding from the very first token
    engine.finish("b")
    close(torch.cat(got).cpu(), ref[:40], 3e-5)


@pytest.mark.parametrize("cfg", [CFG_A, CFG_B], ids=["A", "B"])
def test_portions_of_any_size_down_to_two_tokens(cfg):
    engine, tensors = build(cfg)
    toks = tokens(131, cfg["vocab"], 15)
    ref = R.forward(cfg, tensors, toks)
    for cuts in ([2, 2, 13, 3, 16, 17, 2, 31, 33, 2, 1, 9], [64, 2, 65], [15, 1, 16, 1, 31, 1, 2, 64]):
        got, at = [], 0
        for c in cuts:
            c = min(c, len(toks) - at)
            got.append(engine.step([("a", toks[at:at + c], list(range(c)))]))
            at += c
        engine.finish("a")
        close(torch.cat(got).cpu(), ref[:at], 3e-5)


def test_mixed_batches_match_each_request_alone_and_reuse_pages_and_slots():
    cfg = CFG_A
    engine, tensors = build(cfg, max_tokens=256, max_seqs=3)
    prompts = {r: tokens(n, cfg["vocab"], 20 + i) for i, (r, n) in enumerate((("a", 70), ("b", 33), ("c", 5), ("d", 90), ("e", 48)))}
    ref = {r: R.forward(cfg, tensors, t) for r, t in prompts.items()}
    at = {r: 0 for r in prompts}
    got = {r: [] for r in prompts}

    def feed(plan):
        entries = []
        for r, c in plan:
            entries.append((r, prompts[r][at[r]:at[r] + c], list(range(c))))
        out = engine.step(entries)
        o = 0
        for r, c in plan:
            got[r].append(out[o:o + c])
            o, at[r] = o + c, at[r] + c
            if at[r] == len(prompts[r]):
                engine.finish(r)

    feed([("a", 40), ("b", 2), ("c", 5)])                        # c ends: its slot and page are free again
    feed([("a", 1), ("b", 30), ("d", 17)])                       # d takes c's slot
    feed([("b", 1), ("d", 2), ("a", 1)])                         # b ends
    feed([("e", 31), ("a", 1), ("d", 1)])                        # e takes b's slot and pages
    feed([("d", 70), ("a", 27), ("e", 2)])                       # a and d end
    feed([("e", 15)])
    for r in prompts:
        assert at[r] == len(prompts[r])
        close(torch.cat(got[r]).cpu(), ref[r], 3e-5)
    assert engine.free_slots == 3 and engine.free_blocks == 256 // 16


@pytest.mark.parametrize("cfg", [CFG_A, CFG_C], ids=["A", "C"])
def test_logits_do_not_depend_on_the_batch_or_the_cut_beyond_rounding_bf16(cfg):
    engine, _ = build(cfg, dtype=torch.bfloat16)
    a, b = tokens(80, cfg["vocab"], 31), tokens(37, cfg["vocab"], 32)
    alone = whole(engine, "a", a)
    out = engine.step([("b", b[:20], []), ("a", a[:50], list(range(50)))])
    out2 = engine.step([("a", a[50:], list(range(30))), ("b", b[20:], [])])
    engine.release()
    both = torch.cat([out, out2]).cpu()
    assert (both - alone).abs().max() <= 0.02 * alone.abs().max()


def test_greedy_generation_through_the_scheduler():
    cfg = CFG_B
    engine, tensors = build(cfg, max_tokens=256, max_seqs=2)
    prompts = [tokens(n, cfg["vocab"], 40 + i) for i, n in enumerate((9, 30, 3))]     # three requests, two slots
    out = engine.generate(prompts, max_new_tokens=6, prefill_chunk=7, token_budget=12)
    for p, o in zip(prompts, out):
        want = R.greedy(cfg, tensors, p, 6)
        # a near-tie may flip a token in fp32; up to the first difference the texts must agree and it must be a near-tie
        for k, (x, y) in enumerate(zip(o, want)):
            if x != y:
                lg = R.forward(cfg, tensors, p + want[:k])[-1]
                assert abs(lg[x] - lg[y]) < 1e-4
                break
    assert engine.free_slots == 2


def test_registry_serves_a_checkpoint_folder(tmp_path):
    import json

    from dgi_b200 import model_registry, sanesun_layer as S
    from dgi_b200.ragged_engine import RaggedStepEngine
    from dgi_b200.safetensors_io import write_safetensors

    cfg = S.SanesunConfig.from_dict(CFG_B)
    tensors = S.random_checkpoint(cfg, seed=5)
    (tmp_path / "config.json").write_text(json.dumps(CFG_B))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    arch, _, shards = model_registry.load_model_dir(str(tmp_path), device=DEV, dtype=torch.float32)
    assert arch.name == "Sanesun" and arch.engine == "ragged"
    engine = RaggedStepEngine(shards, max_tokens=128, max_seqs=1)
    toks = tokens(20, CFG_B["vocab"], 50)
    close(whole(engine, "a", toks), R.forward(CFG_B, tensors, toks), 3e-5)
