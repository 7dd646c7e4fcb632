"""GPU: the Petipel model class on the ragged step engine against the plain fp32 statement in oracle/petipel_ref.py.

Small configurations with random weights, sizes chosen so that nothing is a multiple of a warp, a page or a key tile
by accident (kv heads > 1, head sizes 20 / 48 / 10 / 24, top-2 and top-3 routing, odd table sizes, a layer without a
feed-forward, layers with and without temperature and value mixing).  Where random weights would hide a fault the
inputs are made so that it shows: one key among hundreds gets a score that dominates, bias tables get large steps
at their bucket edges, the temperature coefficient is large.
"""
import math

import pytest
import torch

import dgi_b200  # noqa: F401
from oracle import petipel_ref as R

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def attn(heads, kv, dim, vdim, **kw):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": 1.0 / math.sqrt(dim), "bias_max": 40}
    m.update(kw)
    return {"type": "attention", "mixer": m}


def hgrn(heads, dim, vdim):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


def with_mlp(layer, mlp):
    layer = dict(layer)
    layer["mlp"] = mlp
    return layer


DENSE = {"kind": "dense", "ff": 80}


def moe(experts, top, ff=24, limit=1.5):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


CFG_A = {
    "architecture": "Petipel", "width": 48, "vocab": 61, "residual_mult": 0.4, "norm": {"eps": 1e-5},
    "layers": [
        with_mlp(attn(4, 2, 20, 48, v_mix=True, q_temp={"coef": 0.7, "every": 8}), moe(5, 2)),
        with_mlp(hgrn(3, 10, 24), DENSE),
        with_mlp(attn(4, 2, 20, 48, v_mix=True, q_temp={"coef": 0.3, "every": 5}), None),
        with_mlp(hgrn(2, 16, 40), moe(3, 1, ff=16, limit=0.8)),
        with_mlp(attn(2, 2, 36, 48, v_mix=True, bias_max=17), DENSE),
    ],
}
CFG_B = {  # other order, one kv head per query head, no temperature, no value mixing, wide recurrent values
    "architecture": "Petipel", "width": 40, "vocab": 37, "residual_mult": 1.0, "norm": {"eps": 1e-6},
    "layers": [
        with_mlp(hgrn(1, 8, 70), moe(7, 3, ff=8, limit=3.0)),
        with_mlp(attn(3, 3, 32, 16, bias_max=20.5), {"kind": "dense", "ff": 33}),
        with_mlp(attn(6, 1, 12, 72, v_mix=True), None),
        with_mlp(hgrn(5, 3, 5), None),
    ],
}


def build(cfg_raw, dtype=torch.float32, seed=0, bias_rows=12, max_tokens=512, max_seqs=4):
    from dgi_b200 import petipel_layer as P
    from dgi_b200.ragged_engine import RaggedStepEngine

    cfg = P.PetipelConfig.from_dict(cfg_raw)
    tensors = P.random_checkpoint(cfg, seed=seed, bias_rows=bias_rows)
    shards = P.build_shards(cfg, tensors, [(0, cfg.num_hidden_layers)], DEV, dtype)
    return RaggedStepEngine(shards, max_tokens=max_tokens, max_seqs=max_seqs), tensors


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def whole(engine, rid, toks, want=None):
    want = list(range(len(toks))) if want is None else want
    out = engine.step([(rid, toks, want)]).cpu()
    engine.finish(rid)
    return out


def close(got, ref, tol):
    err = (got - ref).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()), f"max abs error {err}"


# ---- mechanisms alone ----------------------------------------------------------------------------------------------

def test_offset_norm_and_residual_update():
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(1)
    x = torch.randn(7, 50, generator=g)
    y = torch.randn(7, 50, generator=g)
    w1, w2 = torch.randn(50, generator=g) * 0.2, torch.randn(50, generator=g) * 0.2
    for dt, tol in ((torch.float32, 2e-6), (torch.bfloat16, 1e-2)):
        wd1, wd2 = w1.to(dt), w2.to(dt)
        got = M.offset_rmsnorm(x.to(DEV), wd1.to(DEV), 1e-5).float().cpu()
        close(got, R.offset_norm(x, wd1.float(), 1e-5), tol)
        xd = x.to(DEV).clone()
        yd = y.to(dt)
        nxt = M.postnorm_residual(xd, yd.to(DEV), wd1.to(DEV), 0.3, 1e-5, w_next=wd2.to(DEV))
        ref_x = x + 0.3 * R.offset_norm(yd.float(), wd1.float(), 1e-5)
        close(xd.cpu(), ref_x, 2e-6)                      # the residual is fp32 for every storage dtype
        close(nxt.float().cpu(), R.offset_norm(ref_x, wd2.float(), 1e-5), tol)
        # fp32 sublayer output (the routed feed-forward's sum) into a 16-bit model
        xd = x.to(DEV).clone()
        assert M.postnorm_residual(xd, y.to(DEV), wd1.to(DEV), 0.3, 1e-5) is None
        close(xd.cpu(), x + 0.3 * R.offset_norm(y, wd1.float(), 1e-5), 2e-6)


def test_polynorm_and_clamped_glu():
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(2)
    z = torch.randn(5, 77, generator=g) * 2
    coef = torch.tensor([0.6, -0.3, 0.2, 0.05])
    close(M.polynorm(z.to(DEV), coef.to(DEV), 1e-5).cpu(), R.polynorm(z, coef, 1e-5), 3e-6)
    gu = torch.randn(9, 2 * 13, generator=g) * 3
    got = M.clamped_glu(gu.to(DEV), 1.5, 1.702).cpu()
    gg, uu = gu[:, :13].clamp(max=1.5), gu[:, 13:].clamp(-1.5, 1.5)
    close(got, gg * torch.sigmoid(1.702 * gg) * (uu + 1), 3e-6)


def test_router_picks_top_scores_and_scales_the_input():
    from dgi_b200 import petipel_layer as P

    g = torch.Generator().manual_seed(3)
    W, E, ff = 24, 37, 6            # more experts than a warp has lanes
    spec = moe(E, 3, ff=ff, limit=1.0)
    t = {"router": torch.randn(E, W, generator=g)}
    for e in range(E):
        t[f"e{e}.gate"], t[f"e{e}.up"] = torch.randn(ff, W, generator=g), torch.randn(ff, W, generator=g)
        t[f"e{e}.down"] = torch.randn(W, ff, generator=g)
    mod = P.SigmoidTopKMoE(spec, t, DEV, torch.float32)
    h = torch.randn(11, W, generator=g)
    close(mod(h.to(DEV)).cpu(), R.moe_ff(h, t, spec), 1e-5)


def test_distance_table_matches_the_bucket_rule():
    from dgi_b200 import petipel_layer as P

    for rows, far in ((12, 40), (7, 20.5), (32, 300), (1, 5), (2, 3)):
        rel = torch.arange(rows * 2, dtype=torch.float32).view(rows, 2)
        lut = P.distance_bias_table(rel, far)
        for d in range(0, 400):
            want = rel[R.distance_bucket(d, rows, far)]
            assert torch.equal(lut[:, min(d, lut.shape[1] - 1)], want), (rows, far, d)


def _attention_rows(q, gate, k, v, pos_q, rel, far, scale, coef, every, H, G):
    """Plain attention of query rows at positions ``pos_q`` over keys 0..len(k)-1 (fp32, vectorised per row)."""
    rows = rel.shape[0]
    out = torch.zeros(len(pos_q), H, v.shape[-1])
    for r, p in enumerate(pos_q):
        bucket = torch.tensor([R.distance_bucket(p - j, rows, far) for j in range(p + 1)])
        temp = 1.0 + coef * math.log(((p + 1) // every) + 1)
        for h in range(H):
            gi = h // (H // G)
            s = (k[: p + 1, gi] @ q[r, h]) * scale * temp + rel[bucket, h]
            out[r, h] = torch.softmax(s, 0) @ v[: p + 1, gi] * torch.sigmoid(gate[r, h])
    return out.reshape(len(pos_q), -1)


def _paged_case(n_ctx, G, dk, dv, bs=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    k, v = torch.randn(n_ctx, G, dk, generator=g), torch.randn(n_ctx, G, dv, generator=g)
    nb = (n_ctx + bs - 1) // bs
    order = torch.randperm(nb + 5, generator=g)[:nb]          # scattered pages
    k_pool, v_pool = torch.zeros(nb + 5, G, bs, dk), torch.zeros(nb + 5, G, bs, dv)
    for j in range(n_ctx):
        k_pool[order[j // bs], :, j % bs], v_pool[order[j // bs], :, j % bs] = k[j], v[j]
    return k, v, k_pool, v_pool, order.to(torch.int32)[None]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_one_key_wherever_it_lies(dtype):
    """One key gets a dominating score; the output must be its value.  Needles: far back, at page borders, at the
    borders of the 32-key tiles, the first keys, the newest key; queried from a prompt portion and as one token."""
    from dgi_b200 import mixer_ops as M

    H, G, dk, dv, n_ctx = 4, 2, 20, 48, 700
    k, v, k_pool, v_pool, table = _paged_case(n_ctx, G, dk, dv)
    rel = torch.zeros(12, H)
    lut = torch.zeros(H, 41)
    dirs = torch.nn.functional.normalize(torch.randn(64, dk, generator=torch.Generator().manual_seed(9)), dim=-1)
    needles = [0, 1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 255, 256, 300, 511, 512, 640, 671, 672, 698, 699]
    for i, j in enumerate(needles):
        k[j] = 0.05 * k[j]
        k[j, :, :] += 6.0 * dirs[i]
        k_pool[table[0, j // 16].long(), :, j % 16] = k[j]
    kp, vp = k_pool.to(DEV, dtype), v_pool.to(DEV, dtype)
    kr, vr = k.to(dtype).float(), v.to(dtype).float()
    for portion in (24, 1):                               # the last `portion` positions are the step's queries
        pos_q = list(range(n_ctx - portion, n_ctx))
        q = torch.randn(portion, H, dk, generator=torch.Generator().manual_seed(4)) * 0.1
        for r in range(portion):
            for h in range(H):
                q[r, h] += 6.0 * dirs[(r * H + h) % len(needles)]
        qd = q.reshape(portion, H * dk).to(dtype)
        gate = torch.full((portion, H), 30.0)             # gate open: sigmoid = 1
        cap = M.attn_tile_tokens(portion, H, G)
        tiles = torch.tensor([[lo, min(cap, portion - lo), 0] for lo in range(0, portion, cap)], dtype=torch.int32)
        out = M.biased_paged_attention(qd.to(DEV), gate.to(DEV, dtype), kp, vp, table.to(DEV), tiles.to(DEV), cap,
                                       torch.tensor(pos_q, dtype=torch.int32, device=DEV), lut.to(DEV), 1.0, 0.0, 1, H)
        ref = _attention_rows(qd.float().view(portion, H, dk), gate, kr, vr, pos_q, rel, 40, 1.0, 0.0, 1, H, G)
        close(out.float().cpu(), ref, 2e-5 if dtype == torch.float32 else 2e-2)
        for r in range(portion):                          # and the needle really decides the row
            for h in range(H):
                j = needles[(r * H + h) % len(needles)]
                if j <= pos_q[r]:
                    got = out[r].float().cpu().view(H, dv)[h]
                    assert (got - vr[j, h // (H // G)]).abs().max() < 0.05, (portion, r, h, j)


def test_bias_edges_and_temperature_steps():
    """A bias table with large steps makes every bucket edge visible (the last exact distance, the first logarithmic
    one, the distance where the table saturates, one beyond); a large temperature coefficient makes the positions
    where floor((p + 1) / every) steps visible.  Prompt portions and single tokens."""
    from dgi_b200 import mixer_ops as M
    from dgi_b200 import petipel_layer as P

    H, G, dk, dv, n_ctx = 2, 1, 12, 16, 90
    rows, far, every, coef = 12, 40, 8, 2.5
    k, v, k_pool, v_pool, table = _paged_case(n_ctx, G, dk, dv, seed=5)
    rel = torch.tensor([((-1.0) ** i) * (1.0 + 0.7 * i) for i in range(rows)])[:, None] * torch.tensor([[1.0, -0.5]])
    lut = P.distance_bias_table(rel, far)
    q = torch.randn(n_ctx, H, dk, generator=torch.Generator().manual_seed(6)) * 0.3
    gate = torch.randn(n_ctx, H, generator=torch.Generator().manual_seed(7))
    ref = _attention_rows(q, gate, k, v, list(range(n_ctx)), rel, far, 0.4, coef, every, H, G)
    for cuts in ([n_ctx], [1] * n_ctx, [7, 2, 30, 1, 1, 49]):
        at, outs = 0, []
        for n in cuts:
            cap = M.attn_tile_tokens(n, H, G)
            tiles = torch.tensor([[lo, min(cap, n - lo), 0] for lo in range(0, n, cap)], dtype=torch.int32)
            outs.append(M.biased_paged_attention(
                q[at:at + n].reshape(n, -1).to(DEV), gate[at:at + n].to(DEV), k_pool.to(DEV), v_pool.to(DEV),
                table.to(DEV), tiles.to(DEV), cap, torch.arange(at, at + n, dtype=torch.int32, device=DEV), lut.to(DEV),
                0.4, coef, every, H).cpu())
            at += n
        close(torch.cat(outs), ref, 2e-5)


def test_value_prep_norms_mixes_and_appends():
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(8)
    n, G, dk, dv, bs = 9, 3, 10, 24, 16
    proj = torch.randn(n, G * dk + G * dv + 5, generator=g)
    prev = torch.randn(n, G * dv, generator=g)
    k_pool, v_pool = torch.zeros(4, G, bs, dk, device=DEV), torch.zeros(4, G, bs, dv, device=DEV)
    slots = torch.tensor([3 * bs + 15, 0, 1, 2 * bs, 2 * bs + 1, 17, 18, 19, 62])
    keep = torch.empty(n, G * dv, device=DEV)
    pd = proj.to(DEV)
    M.value_prep_append(pd[:, :G * dk], pd[:, G * dk:G * (dk + dv)], k_pool, v_pool, slots.to(DEV), 1e-5,
                        v_prev=prev.to(DEV), lam=0.3, v_keep=keep)
    want_v = 0.7 * R.rms_unit(proj[:, G * dk:G * (dk + dv)].view(n, G, dv), 1e-5) + 0.3 * prev.view(n, G, dv)
    close(keep.cpu().view(n, G, dv), want_v, 2e-6)
    for i, s in enumerate(slots.tolist()):
        close(v_pool[s // bs, :, s % bs].cpu(), want_v[i], 2e-6)
        assert torch.equal(k_pool[s // bs, :, s % bs].cpu(), proj[i, :G * dk].view(G, dk))


@pytest.mark.parametrize("H,dk,dv", [(3, 10, 24), (1, 8, 70), (2, 33, 300), (1, 100, 16), (2, 130, 20), (2, 64, 128)])
@pytest.mark.parametrize("hint", [1 << 20, 1])      # long portions: state in registers; single tokens: in shared memory
def test_gated_recurrence_against_the_loop(H, dk, dv, hint):
    """Portions of unequal sequences in one launch, state carried through the slot pool, stale slots ignored when a
    sequence starts."""
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(10)
    W = 16
    t = {"q": torch.randn(H * dk, W, generator=g), "f": torch.randn(H * dk, W, generator=g),
         "v": torch.randn(H * dv, W, generator=g), "f.b": torch.randn(H * dk, generator=g),
         "lower": torch.rand(H * dk, generator=g) * 0.9, "norm": torch.ones(dv), "o": torch.eye(H * dv)}
    m = {"heads": H, "dim": dk, "vdim": dv}
    lens = [13, 1, 40]
    hs = [torch.randn(n, W, generator=g) for n in lens]
    state = torch.full((4, H, dk, dv), 7.0, device=DEV)          # stale content everywhere
    slot = [2, 0, 3]
    done = [0, 0, 0]
    got = [[] for _ in lens]
    for cuts in ([5, 1, 2], [8, 0, 38], [0, 0, 0]):
        rows, seqs, owner = [], [], []
        for b, n in enumerate(cuts):
            n = min(n, lens[b] - done[b])
            if n:
                seqs.append((sum(r.shape[0] for r in rows), n, slot[b], 1 if done[b] == 0 else 0))
                rows.append(hs[b][done[b]:done[b] + n])
                owner.append((b, n))
                done[b] += n
        if not rows:
            continue
        h = torch.cat(rows).to(DEV)
        proj = torch.nn.functional.linear(h, torch.cat([t["q"], t["f"], t["v"]]).to(DEV))
        a = H * dk
        o = M.gated_scan(proj[:, :a], proj[:, a:2 * a], proj[:, 2 * a:], t["f.b"].to(DEV), t["lower"].to(DEV), state,
                         torch.tensor(seqs, dtype=torch.int32, device=DEV), H, max_count=hint)
        on = M.head_rmsnorm(o, t["norm"].to(DEV), 1e-5).cpu().view(h.shape[0], H * dv)
        at = 0
        for b, n in owner:
            got[b].append(on[at:at + n])
            at += n
    for b, n in enumerate(lens):
        ref, S = R.hgrn2_mixer(hs[b], t, m, 1e-5)
        close(torch.cat(got[b]), ref[: sum(x.shape[0] for x in got[b])], 2e-5)
    close(state[2].cpu(), R.hgrn2_mixer(hs[0][:8 + 5], t, m, 1e-5)[1], 2e-5)


# ---- the model on the engine ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("cfg,rows", [(CFG_A, 12), (CFG_B, 7)])
def test_whole_prompt_matches_the_oracle_layer_by_layer(cfg, rows):
    eng, tensors = build(cfg, bias_rows=rows)
    toks = tokens(75, cfg["vocab"], 1)
    eng.layer_trace = []
    got = whole(eng, "a", toks)
    trace = []
    ref = R.forward(cfg, tensors, toks, trace=trace)
    for i, (x, y) in enumerate(zip(eng.layer_trace, trace)):
        err = (x.cpu() - y).abs().max().item()
        assert err < 3e-5 * max(1.0, y.abs().max().item()), f"layer {i} ({cfg['layers'][i]['type']}): {err}"
    close(got, ref, 3e-5)


@pytest.mark.parametrize("cfg,rows", [(CFG_A, 12), (CFG_B, 7)])
def test_portions_decoding_and_batches_do_not_change_a_position(cfg, rows):
    """The same three prompts: whole; token by token; in portions down to two tokens; and all three interleaved in
    mixed steps (a portion of one beside single tokens of the others).  fp32, so agreement is to rounding."""
    eng, _ = build(cfg, bias_rows=rows)
    prompts = [tokens(n, cfg["vocab"], 20 + n) for n in (70, 9, 41)]
    ref = [whole(eng, "w", p) for p in prompts]
    # token by token (the first tokens of a sequence included)
    for p, r in zip(prompts[1:], ref[1:]):
        outs = [eng.step([("d", [t], [0])]) for t in p]
        eng.finish("d")
        close(torch.cat(outs).cpu(), r, 1e-5)
    # portions of several sizes
    for sizes in ([2, 2, 3, 17, 1, 16, 2, 64], [33, 32, 5], [1, 69]):
        at, outs, k = 0, [], 0
        p = prompts[0]
        while at < len(p):
            n = min(sizes[k % len(sizes)], len(p) - at)
            outs.append(eng.step([("c", p[at:at + n], list(range(n)))]))
            at, k = at + n, k + 1
        eng.finish("c")
        close(torch.cat(outs).cpu(), ref[0], 1e-5)
    # mixed steps
    plan = [[(0, 30), (1, 1)], [(1, 1), (2, 2)], [(0, 1), (1, 7), (2, 20)], [(0, 39), (2, 1)], [(2, 18)]]
    at = [0, 0, 0]
    got = [[], [], []]
    for stepn in plan:
        entries = [(f"m{i}", prompts[i][at[i]:at[i] + n], list(range(n))) for i, n in stepn]
        out = eng.step(entries).cpu()
        o = 0
        for i, n in stepn:
            got[i].append(out[o:o + n])
            o += n
            at[i] += n
    for i in range(3):
        assert at[i] == len(prompts[i])
        eng.finish(f"m{i}")
        close(torch.cat(got[i]), ref[i], 1e-5)


def test_pages_and_slots_are_reused_cleanly():
    """A pool of 8 pages and 2 slots: requests come and go, every page and slot is used several times, by requests
    of other lengths, and the pool is full at times.  Each answer equals the request's answer in a fresh engine."""
    fresh, _ = build(CFG_A, max_tokens=512)
    eng, _ = build(CFG_A, max_tokens=128, max_seqs=2)
    assert eng.num_blocks == 8 and eng.free_slots == 2
    prompts = [tokens(n, CFG_A["vocab"], 40 + n) for n in (60, 50, 17, 64, 33, 64)]
    ref = [whole(fresh, "r", p) for p in prompts]
    a = eng.step([("p0", prompts[0][:40], list(range(40))), ("p1", prompts[1][:20], list(range(20)))]).cpu()
    b = eng.step([("p0", prompts[0][40:], list(range(20))), ("p1", prompts[1][20:], list(range(30)))]).cpu()
    assert eng.free_blocks == 0
    with pytest.raises(RuntimeError):
        eng.step([("p0", [1], [0]), ("p1", [1] * 15, [])])  # p1 would need a ninth page: refused, nothing half-done
    assert eng.requests["p0"].length == 60 and eng.requests["p1"].length == 50
    close(torch.cat([a[:40], b[:20]]), ref[0], 1e-5)
    close(torch.cat([a[40:], b[20:]]), ref[1], 1e-5)
    eng.finish("p1")
    with pytest.raises(RuntimeError):
        eng.admit("x"), eng.admit("y")                     # one slot is free, not two
    eng.finish("x")
    for i in (2, 3):                                       # reuse p1's pages and slot while p0 stays live
        close(whole(eng, f"p{i}", prompts[i]), ref[i], 1e-5)
    eng.finish("p0")
    close(whole(eng, "p4", prompts[4]), ref[4], 1e-5)
    out = eng.step([("p5", prompts[5], list(range(64))), ("p3", prompts[3], list(range(64)))]).cpu()
    close(out[:64], ref[5], 1e-5)
    close(out[64:], ref[3], 1e-5)
    eng.release()
    assert eng.free_blocks == 8 and eng.free_slots == 2


def test_long_decoding_and_far_keys_through_the_model():
    """300 tokens one at a time (the recurrence and the cache grow step by step across many pages and past the point
    where the bias table saturates) against the whole prompt in one step."""
    eng, tensors = build(CFG_B, bias_rows=7)
    toks = tokens(300, CFG_B["vocab"], 3)
    ref = whole(eng, "w", toks)
    outs = [eng.step([("d", [t], [0])]) for t in toks]
    eng.finish("d")
    close(torch.cat(outs).cpu(), ref, 2e-5)
    oracle = R.forward(CFG_B, tensors, toks[:120])
    close(ref[:120], oracle, 5e-5)


def test_bfloat16_serving_stays_close_to_fp32():
    eng16, tensors = build(CFG_A, dtype=torch.bfloat16)
    toks = tokens(64, CFG_A["vocab"], 5)
    ref = R.forward(CFG_A, tensors, toks)
    got = whole(eng16, "a", toks)
    d = (got - ref)
    rel = (d - d.mean(1, keepdim=True)).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()
    assert rel < 0.05, rel
    # and a portion split changes nothing beyond 16-bit rounding of the GEMM inputs
    parts = torch.cat([eng16.step([("b", toks[:31], list(range(31)))]), eng16.step([("b", toks[31:], list(range(33)))])]).cpu()
    eng16.finish("b")
    assert ((parts - got).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()) < 0.03


def test_greedy_generation_through_the_scheduler():
    """``generate`` — admission, chunked prompts beside decoding requests, retirement, more requests than slots —
    gives the tokens the oracle's greedy loop gives."""
    eng, tensors = build(CFG_A, max_tokens=256, max_seqs=3)
    prompts = [tokens(n, CFG_A["vocab"], 60 + n) for n in (23, 5, 40, 11, 1)]
    n_new = 6
    got = eng.generate(prompts, n_new, prefill_chunk=16, token_budget=24)
    assert eng.free_blocks == eng.num_blocks and eng.free_slots == 3
    for p, g in zip(prompts, got):
        seq = list(p)
        for _ in range(n_new):
            seq.append(int(R.forward(CFG_A, tensors, seq)[-1].argmax()))
        assert g == seq[len(p):]
    res = eng.batch_inference([{"input_ids": prompts[1], "max_new_tokens": 3}, {"input_ids": []}])
    assert res[0]["output_ids"] == got[1][:3] and isinstance(res[1], Exception)


def test_checkpoint_folder_round_trip(tmp_path):
    """config.json + model.safetensors on disk -> registry -> engine -> the same logits as the in-memory build."""
    import json

    from dgi_b200 import model_registry
    from dgi_b200 import petipel_layer as P
    from dgi_b200.ragged_engine import RaggedStepEngine
    from dgi_b200.safetensors_io import write_safetensors

    cfg = P.PetipelConfig.from_dict(CFG_B)
    tensors = P.random_checkpoint(cfg, seed=4, bias_rows=9)
    (tmp_path / "config.json").write_text(json.dumps(CFG_B))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    arch, config, shards = model_registry.load_model_dir(str(tmp_path), DEV, torch.float32, ranges=[(0, 2), (2, 4)])
    assert arch.name == "Petipel" and arch.engine == "ragged" and len(shards) == 2
    toks = tokens(30, CFG_B["vocab"], 6)
    got = whole(RaggedStepEngine(shards, max_tokens=64), "a", toks)
    close(got, R.forward(CFG_B, tensors, toks), 5e-5)


# ---- the tensor-core prompt kernel (16-bit storage, dk % 16 == 0, dv % 8 == 0) -----------------------------------------

def _prompt_tiles(spans, cap=64):
    rows = []
    for first, count, table_row in spans:
        for lo in range(0, count, cap):
            rows.append([first + lo, min(cap, count - lo), table_row])
    return torch.tensor(rows, dtype=torch.int32)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("H,G,dk,dv", [(4, 2, 32, 48), (2, 1, 96, 32), (3, 3, 16, 128), (2, 2, 48, 8)])
def test_prompt_kernel_finds_needles_and_respects_edges(dtype, H, G, dk, dv):
    """Portions that start anywhere (not at a multiple of the 64-key tile or the 16-token page), needles at tile and
    page borders and among the first and newest keys, a bias table with large steps, a strong temperature; against
    the plain fp32 attention of the same 16-bit-rounded q, k, v."""
    from dgi_b200 import mixer_ops as M
    from dgi_b200 import petipel_layer as P

    assert M.prompt_attention_supported(dk, dv, dtype)
    n_ctx, rows, far, every, coef = 333, 12, 40, 8, 1.5
    k, v, k_pool, v_pool, table = _paged_case(n_ctx, G, dk, dv, seed=11)
    dirs = torch.nn.functional.normalize(torch.randn(40, dk, generator=torch.Generator().manual_seed(12)), dim=-1)
    needles = [0, 1, 15, 16, 63, 64, 65, 127, 128, 191, 192, 200, 255, 256, 300, 319, 320, 331, 332]
    for i, j in enumerate(needles):
        k[j] = 0.05 * k[j] + 5.0 * dirs[i]
        k_pool[table[0, j // 16].long(), :, j % 16] = k[j]
    rel = torch.tensor([((-1.0) ** i) * (0.5 + 0.3 * i) for i in range(rows)])[:, None] * torch.linspace(1.0, -1.0, H)[None]
    lut = P.distance_bias_table(rel, far)
    q = torch.randn(n_ctx, H, dk, generator=torch.Generator().manual_seed(13)) * 0.2
    for r in range(n_ctx):
        for h in range(H):
            q[r, h] += 5.0 * dirs[(r * H + h) % len(needles)]
    gate = torch.randn(n_ctx, H, generator=torch.Generator().manual_seed(14))
    qd, gd = q.reshape(n_ctx, H * dk).to(dtype), gate.to(dtype)
    kr, vr = k.to(dtype).float(), v.to(dtype).float()
    ref = _attention_rows(qd.float().view(n_ctx, H, dk), gd.float(), kr, vr, list(range(n_ctx)), rel, far, 0.3, coef,
                          every, H, G)
    for lo, n in ((0, n_ctx), (0, 17), (37, 150), (250, 83), (317, 16), (332, 1), (64, 1), (0, 1), (130, 3)):
        out = torch.full((n, H * dv), 7.0, dtype=dtype, device=DEV)
        M.biased_prompt_attention(out, qd[lo:lo + n].to(DEV), gd[lo:lo + n].to(DEV), k_pool.to(DEV, dtype),
                                  v_pool.to(DEV, dtype), table.to(DEV),
                                  _prompt_tiles([(0, n, 0)], M.prompt_tile_tokens(H, G)).to(DEV),
                                  torch.arange(lo, lo + n, dtype=torch.int32, device=DEV), lut.to(DEV), 0.3, coef, every, H,
                                  max_tile_tokens=min(n, M.prompt_tile_tokens(H, G)))   # <= 16 rows: the key-split variant
        close(out.float().cpu(), ref[lo:lo + n], 2.5e-2)


def test_prompt_kernel_two_sequences_and_unaligned_rows():
    """Two sequences in one launch (their tiles must not see each other's pages) with q rows taken as column slices
    of a wider projection whose row stride is not a multiple of 16 bytes."""
    from dgi_b200 import mixer_ops as M

    H, G, dk, dv = 2, 1, 32, 16
    ka, va, kpa, vpa, ta = _paged_case(70, G, dk, dv, seed=21)
    kb, vb, kpb, vpb, tb = _paged_case(100, G, dk, dv, seed=22)
    nb = kpa.shape[0]
    k_pool, v_pool = torch.cat([kpa, kpb]), torch.cat([vpa, vpb])
    width = max(ta.shape[1], tb.shape[1])
    table = torch.zeros(2, width, dtype=torch.int32)
    table[0, :ta.shape[1]], table[1, :tb.shape[1]] = ta[0], tb[0] + nb
    g = torch.Generator().manual_seed(23)
    wide = torch.randn(170, H * dk + 5, generator=g).to(torch.bfloat16)     # 69 columns: 138-byte rows
    q = wide[:, :H * dk]
    pos = torch.cat([torch.arange(70), torch.arange(100)]).to(torch.int32)
    lut = torch.zeros(H, 5)
    out = torch.empty(170, H * dv, dtype=torch.bfloat16, device=DEV)
    M.biased_prompt_attention(out, wide.to(DEV)[:, :H * dk], None, k_pool.to(DEV, torch.bfloat16),
                              v_pool.to(DEV, torch.bfloat16), table.to(DEV),
                              _prompt_tiles([(0, 70, 0), (70, 100, 1)], M.prompt_tile_tokens(H, G)).to(DEV),
                              pos.to(DEV), lut.to(DEV), 0.2, 0.0, 1, H)
    big = torch.full((170, H), 30.0)
    rel = torch.zeros(4, H)
    qa = q.float().view(170, H, dk)
    ref = torch.cat([
        _attention_rows(qa[:70], big[:70], ka.bfloat16().float(), va.bfloat16().float(), list(range(70)), rel, 9, 0.2, 0.0, 1, H, G),
        _attention_rows(qa[70:], big[70:], kb.bfloat16().float(), vb.bfloat16().float(), list(range(100)), rel, 9, 0.2, 0.0, 1, H, G)])
    close(out.float().cpu(), ref, 2e-2)


CFG_C = {  # head sizes the tensor-core prompt kernel takes
    "architecture": "Petipel", "width": 64, "vocab": 53, "residual_mult": 0.5, "norm": {"eps": 1e-5},
    "layers": [
        with_mlp(attn(4, 2, 32, 24, v_mix=True, q_temp={"coef": 0.5, "every": 16}), DENSE),
        with_mlp(hgrn(2, 16, 32), moe(4, 2)),
        with_mlp(attn(4, 2, 32, 24, v_mix=True, bias_max=100), DENSE),
    ],
}


def test_bfloat16_model_with_tensor_core_prompts():
    """bf16 serving where long portions take the tensor-core kernel and short ones / decoded tokens the row kernel:
    whole prompt, portions and token-by-token agree with each other and with the fp32 oracle to 16-bit rounding."""
    eng, tensors = build(CFG_C, dtype=torch.bfloat16)
    assert eng.shards[0].layers[0].mixer.tensor_core_prompt
    toks = tokens(150, CFG_C["vocab"], 8)
    ref = R.forward(CFG_C, tensors, toks)
    scale = ref.pow(2).mean().sqrt()

    def rel(a, b):
        d = a - b
        return ((d - d.mean(1, keepdim=True)).pow(2).mean().sqrt() / scale).item()

    got = whole(eng, "a", toks)
    assert rel(got, ref) < 0.05
    at, outs = 0, []
    for n in (70, 3, 40, 1, 1, 20, 15):
        outs.append(eng.step([("b", toks[at:at + n], list(range(n)))]))
        at += n
    eng.finish("b")
    assert at == 150 and rel(torch.cat(outs).cpu(), ref) < 0.05 and rel(torch.cat(outs).cpu(), got) < 0.04
    eng32, _ = build(CFG_C, dtype=torch.float32)
    close(whole(eng32, "c", toks), ref, 5e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_grouped_linear_with_device_offsets(dtype):
    """Expert-sorted rows through all experts in one launch: empty experts, an expert with more rows than a row tile,
    output and inner sizes that are not multiples of the kernel's tiles."""
    from dgi_b200 import mixer_ops as M

    g = torch.Generator().manual_seed(31)
    E, N, K = 6, 328, 40
    counts = [0, 3, 37, 0, 16, 1]
    rows = sum(counts)
    xs = torch.randn(rows, K, generator=g).to(dtype)
    w = (torch.randn(E, N, K, generator=g) / K ** 0.5).to(dtype)
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32)
    assert M.grouped_linear_supported(K, dtype) and not M.grouped_linear_supported(K, torch.float32)
    assert not M.grouped_linear_supported(K + 4, dtype)
    out = M.grouped_linear(xs.to(DEV), w.to(DEV), offsets.to(DEV)).float().cpu()
    lo = 0
    for e, c in enumerate(counts):
        if c:
            close(out[lo:lo + c], xs[lo:lo + c].float() @ w[e].float().t(), 1e-2)
        lo += c


def test_routed_feed_forward_16_bit_takes_the_grouped_kernel():
    from dgi_b200 import petipel_layer as P

    g = torch.Generator().manual_seed(32)
    W, E, ff = 64, 5, 24
    spec = moe(E, 2, ff=ff, limit=1.5)
    t = {"router": torch.randn(E, W, generator=g).bfloat16()}
    for e in range(E):
        t[f"e{e}.gate"], t[f"e{e}.up"] = (torch.randn(ff, W, generator=g) / 8).bfloat16(), (torch.randn(ff, W, generator=g) / 8).bfloat16()
        t[f"e{e}.down"] = (torch.randn(W, ff, generator=g) / 5).bfloat16()
    mod = P.SigmoidTopKMoE(spec, t, DEV, torch.bfloat16)
    assert mod.grouped
    h = torch.randn(50, W, generator=g).bfloat16()
    ref = R.moe_ff(h.float(), {k: v.float() for k, v in t.items()}, spec)
    got = mod(h.to(DEV)).cpu()
    mod.GROUPED_MAX_ROWS = 0                      # the per-expert path on the same input
    loops = mod(h.to(DEV)).cpu()
    close(got, ref, 2e-2)
    close(loops, ref, 2e-2)


def test_engine_adapter_serves_a_checkpoint_folder(tmp_path):
    """The reference-shaped engine surface (load_model / inference / batch_inference) picks the ragged step engine
    for a checkpoint folder whose config.json names this model class, and answers with the oracle's greedy tokens."""
    import json

    from dgi_b200 import petipel_layer as P
    from dgi_b200.safetensors_io import write_safetensors
    from dgi_b200.worker.engines.paged_engine import PagedLLMEngine

    cfg = P.PetipelConfig.from_dict(CFG_B)
    tensors = P.random_checkpoint(cfg, seed=7, bias_rows=9)
    (tmp_path / "config.json").write_text(json.dumps(CFG_B))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    eng = PagedLLMEngine({"model_path": str(tmp_path), "device": DEV, "dtype": torch.float32, "max_batch_size": 2,
                          "max_num_batched_tokens": 256})
    eng.load_model()
    assert eng.get_backend_info()["backend"] == "ragged_b200"
    prompts = [tokens(n, CFG_B["vocab"], 70 + n) for n in (12, 30, 5)]
    res = eng.batch_inference([{"input_ids": p, "max_tokens": 4} for p in prompts] + [{"nothing": 1}])
    assert isinstance(res[3], Exception)
    for p, r in zip(prompts, res):
        seq = list(p)
        for _ in range(4):
            seq.append(int(R.forward(CFG_B, tensors, seq)[-1].argmax()))
        assert r["output_ids"] == seq[len(p):] and r["usage"]["prompt_tokens"] == len(p)
    eng.unload_model()
