"""Sanesun: a decoder whose layers read ONE norm of an fp32 residual stream and add a sequence mixer's and a
feed-forward's outputs to it together,

    h = norm(x);   x <- x + (mixer(h) + ff(h)),

with one of three mixers per layer:

  ``attention``         grouped-query softmax attention with partial rotary positions, a sliding window that also keeps
                        the sequence's first tokens, a learned sink logit per head in the softmax denominator, a
                        head-mixing matrix on the scores before the softmax, and values that are stored ROTATED by
                        their position over the whole value width (the head's output is turned back by the query's
                        position, so a value enters by its distance to the query).
  ``latent_attention``  causal softmax attention without positions whose keys and values are up-projections of one
                        normed latent row per token; only that row is cached.  Queries pass a normed latent too, and
                        the head outputs a per-head sigmoid gate.  Served in the absorbed form: the key up-projection
                        moves to the query side and the value up-projection behind the attention, so the kernel is a
                        multi-query attention over the latent pool with key size = value size = latent size.
  ``channel_delta``     gated delta rule with one decay per head and key channel.  q, k, v pass a short causal
                        convolution and SiLU, q and k are made unit vectors per head; the fp32 state ``[heads, dk,
                        dv]`` and the convolution's last inputs live in a slot pool per live sequence.

Feed-forward: ``W_down xielu(W_up h)``.

The modules follow the calling convention of ``ModelShard.forward`` (reference:
worker/distributed/model_shard.py:205-215): ``layer(h, attention_mask=, position_ids=, past_key_value=, use_cache=)
-> (h, present)`` with ``h`` the packed fp32 residual ``[n_tok, width]`` of one step and ``past_key_value`` a
``RaggedLayerCache``.  Matrix products are torch GEMMs; everything between them is a kernel of ``mixer_ops``.  There
is no dense / CPU mode.

Checkpoint names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``; linear weights
are ``[out, in]``.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import mixer_ops
from .paged_layer import RaggedLayerCache
from .petipel_layer import FloatEmbedding, _param
from .worker.distributed.model_shard import ModelShard

MIXERS = ("attention", "latent_attention", "channel_delta")
UNIT_NORM_EPS = 1e-6      # q and k of the delta rule: x / sqrt(sum(x^2) + 1e-6); fixed by the design


class SanesunConfig:
    """``config.json`` of the design, plus the attribute names the rest of the framework reads from a config."""

    def __init__(self, raw: Dict[str, Any]):
        self.raw = raw
        self.architecture = raw.get("architecture", "Sanesun")
        self.layers: List[Dict[str, Any]] = list(raw["layers"])
        self.width = int(raw["width"])
        self.vocab = int(raw["vocab"])
        self.eps = float(raw["norm"]["eps"])
        self.embed_scale = float((raw.get("embedding") or {}).get("scale", 1.0))
        for i, layer in enumerate(self.layers):
            if layer["type"] not in MIXERS:
                raise NotImplementedError(f"layer {i}: unknown mixer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise NotImplementedError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
            m = layer["mixer"]
            if layer["type"] != "latent_attention" and int(m["heads"]) % int(m.get("kv_heads", m["heads"])):
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
        # names shared with the other model classes
        self.hidden_size = self.width
        self.vocab_size = self.vocab
        self.num_hidden_layers = len(self.layers)
        self.num_attention_heads = max(int(l["mixer"]["heads"]) for l in self.layers)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "SanesunConfig":
        return cls(raw)

    def kv_shape(self, i: int) -> Optional[Tuple[int, int, int]]:
        """``(kv heads, key size, value size)`` of a layer that keeps pages; a latent layer keeps one row per token
        that serves as key and value, hence one head and no value pool."""
        kind, m = self.layers[i]["type"], self.layers[i]["mixer"]
        if kind == "attention":
            return int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])
        if kind == "latent_attention":
            return 1, int(m["kv_rank"]), 0
        return None

    def state_shape(self, i: int):
        """Per live sequence: the delta rule's state and the convolutions' last ``taps - 1`` inputs (q | k | v)."""
        kind, m = self.layers[i]["type"], self.layers[i]["mixer"]
        if kind != "channel_delta":
            return None
        H, G, dk, dv = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])
        return [(H, dk, dv), (max(int(m["conv"]) - 1, 0), 2 * G * dk + H * dv)]


class PlainRMSNorm(nn.Module):
    """``x * rsqrt(mean(x^2) + eps) * w`` over fp32 (or storage-dtype) rows; the weight's dtype out."""

    def __init__(self, width: int, eps: float, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(width, device=device, dtype=dtype), requires_grad=False)
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return mixer_ops.rms_norm(x, self.weight, self.eps)


class ScaledFloatEmbedding(FloatEmbedding):
    """Embedding rows times a constant, opening the fp32 residual stream."""

    def __init__(self, *args, scale: float = 1.0, **kwargs):
        super().__init__(*args, **kwargs)
        self.scale = scale

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        x = super().forward(ids)
        return x * self.scale if self.scale != 1.0 else x


def _pad8(w: torch.Tensor) -> torch.Tensor:
    """Zero rows up to a multiple of 8: the sections of a fused projection stay 16-byte aligned."""
    pad = -w.shape[0] % 8
    return torch.cat([w, w.new_zeros(pad, *w.shape[1:])], dim=0) if pad else w


class WindowedSinkAttention(nn.Module):
    """The ``attention`` mixer: one GEMM (with biases) produces q | k | v, one launch rotates q, k and the values and
    appends k and v to the pages, one attention launch serves prompt portions and decoded tokens alike."""

    def __init__(self, spec: Dict[str, Any], t: Dict[str, torch.Tensor], device, dtype):
        super().__init__()
        self.H, self.G = int(spec["heads"]), int(spec.get("kv_heads", spec["heads"]))
        self.dk, self.dv = int(spec["dim"]), int(spec["vdim"])
        self.scale = float(spec["scale"])
        mask, rot = spec.get("mask") or {}, spec.get("rot") or {}
        self.window, self.keep_first = int(mask.get("size", 0)), int(mask.get("keep_first", 0))
        self.rot_dims, self.rot_base = int(rot.get("dims", 0)), float(rot.get("base", 10000.0))
        self.rotate_values = bool(rot)     # the design turns the values whenever it turns q and k
        self.interleaved = False           # pairs are (i, i + half); the kernels also know (2i, 2i + 1)
        sections = [t["q"], t["k"], t["v"]]
        self.cuts = [0]
        for s in sections:
            self.cuts.append(self.cuts[-1] + s.shape[0] + (-s.shape[0] % 8))
        self.w_in = _param(torch.cat([_pad8(s) for s in sections], dim=0), device, dtype)
        zero = lambda s: torch.zeros(s.shape[0], dtype=s.dtype)  # noqa: E731
        self.b_in = _param(torch.cat([_pad8(t.get(n + ".b", zero(t[n]))) for n in ("q", "k", "v")], dim=0), device, dtype)
        self.w_o = _param(t["o"], device, dtype)
        self.talk = _param(t["talk"], device, torch.float32) if "talk" in t else None
        self.sink = _param(t["sink"], device, torch.float32) if "sink" in t else None
        self.tensor_cores = mixer_ops.mixed_prompt_attention_supported(
            self.H, self.G, self.dk, self.dv, self.talk is not None, False, self.rotate_values, self.w_in.dtype)

    def forward(self, h: torch.Tensor, cache: RaggedLayerCache) -> torch.Tensor:
        st, n = cache.state, h.shape[0]
        H, G, dk, dv = self.H, self.G, self.dk, self.dv
        proj = F.linear(h, self.w_in, self.b_in)
        c = self.cuts
        q, k, v = proj[:, c[0]:c[0] + H * dk], proj[:, c[1]:c[1] + G * dk], proj[:, c[2]:c[2] + G * dv]
        table = mixer_ops.rotary_kv_append(q, k, v, cache.k_pool, cache.v_pool, st.slot_mapping, st.tok_pos, H,
                                           self.rot_dims, self.rot_base, self.rotate_values, self.interleaved,
                                           want_table=self.tensor_cores)
        attn = torch.empty((n, H, dv), dtype=h.dtype, device=h.device)
        if self.tensor_cores:     # 16-bit storage and sizes the tensor-core kernel takes: portions and single tokens
            tiles, _ = st.prompt_tiles(1, mixer_ops.PROMPT_TILE_TOKENS)
            mixer_ops.mixed_prompt_attention(attn, q.unflatten(1, (H, dk)), cache.k_pool, cache.v_pool, st.block_tables,
                                             tiles, st.tok_pos, self.scale, talk=self.talk, sink=self.sink,
                                             window=self.window, keep_first=self.keep_first, value_rot=table,
                                             interleaved=self.interleaved, max_context=st.max_context())
        else:                     # fp32, or head sizes off the tensor-core grid: the row kernel
            mixer_ops.mixed_paged_attention(attn, q.unflatten(1, (H, dk)), cache.k_pool, cache.v_pool, st.block_tables,
                                            st.tok_row, st.tok_pos, self.scale, talk=self.talk, sink=self.sink,
                                            window=self.window, keep_first=self.keep_first,
                                            unrotate_base=self.rot_base if self.rotate_values else None,
                                            interleaved=self.interleaved)
        return F.linear(attn.view(n, H * dv), self.w_o)


class LatentAttention(nn.Module):
    """The ``latent_attention`` mixer in absorbed form.  One GEMM produces the query latent | the key/value latent |
    the gate logits; the normed key/value latent goes to a one-head pool; queries are moved into the latent space by
    the key up-projection (``q' = W_uk^T q`` per head), attend over the pool, and the per-head results are brought to
    the value size by the value up-projection before the output projection."""

    def __init__(self, spec: Dict[str, Any], t: Dict[str, torch.Tensor], eps: float, device, dtype):
        super().__init__()
        self.H, self.dk, self.dv = int(spec["heads"]), int(spec["dim"]), int(spec["vdim"])
        self.rank, self.q_rank = int(spec["kv_rank"]), t["dq"].shape[0]
        self.scale, self.eps = float(spec["scale"]), eps
        sections = [t["dq"], t["dkv"], t["g"]]
        self.cuts = [0]
        for s in sections:
            self.cuts.append(self.cuts[-1] + s.shape[0] + (-s.shape[0] % 8))
        self.w_in = _param(torch.cat([_pad8(s) for s in sections], dim=0), device, dtype)
        self.q_norm, self.c_norm = _param(t["dq.norm"], device, dtype), _param(t["dkv.norm"], device, dtype)
        self.w_uq = _param(t["uq"], device, dtype)
        self.w_uk = _param(t["uk"].reshape(self.H, self.dk, self.rank), device, dtype)                  # [H, dk, r]
        self.w_uv = _param(t["uv"].reshape(self.H, self.dv, self.rank).transpose(1, 2), device, dtype)  # [H, r, dv]
        self.w_o = _param(t["o"], device, dtype)
        self.tensor_cores = mixer_ops.mixed_prompt_attention_supported(self.H, 1, self.rank, self.rank, False, True,
                                                                       False, self.w_in.dtype)

    def forward(self, h: torch.Tensor, cache: RaggedLayerCache) -> torch.Tensor:
        st, n = cache.state, h.shape[0]
        H, r, c = self.H, self.rank, self.cuts
        proj = F.linear(h, self.w_in)
        mixer_ops.norm_append(proj[:, c[1]:c[1] + r], self.c_norm, self.eps, cache.k_pool, st.slot_mapping)
        cq = mixer_ops.rms_norm(proj[:, c[0]:c[0] + self.q_rank], self.q_norm, self.eps)
        q = F.linear(cq, self.w_uq).view(n, H, self.dk)
        q_lat = torch.bmm(q.transpose(0, 1), self.w_uk)                          # [H, n, r]
        o_lat = torch.empty((H, n, r), dtype=h.dtype, device=h.device)
        if self.tensor_cores:
            tiles, _ = st.prompt_tiles(1, mixer_ops.PROMPT_TILE_TOKENS)
            mixer_ops.mixed_prompt_attention(o_lat.transpose(0, 1), q_lat.transpose(0, 1), cache.k_pool, cache.k_pool,
                                             st.block_tables, tiles, st.tok_pos, self.scale, gate=proj[:, c[2]:c[2] + H],
                                             max_context=st.max_context())
        else:
            mixer_ops.mixed_paged_attention(o_lat.transpose(0, 1), q_lat.transpose(0, 1), cache.k_pool, cache.k_pool,
                                            st.block_tables, st.tok_row, st.tok_pos, self.scale,
                                            gate=proj[:, c[2]:c[2] + H])
        o = torch.bmm(o_lat, self.w_uv)                                          # [H, n, dv]
        return F.linear(o.transpose(0, 1).reshape(n, H * self.dv), self.w_o)


class ChannelDeltaMixer(nn.Module):
    """The ``channel_delta`` mixer: one GEMM produces q | k | v (pre-convolution) | write-strength logits | the two
    low-rank bottlenecks; one launch convolves and activates q, k and v, one runs the delta rule of every (sequence,
    head) over the step's tokens against the state pool, one norms and gates the read-outs."""

    def __init__(self, spec: Dict[str, Any], t: Dict[str, torch.Tensor], eps: float, device, dtype):
        super().__init__()
        self.H, self.G = int(spec["heads"]), int(spec.get("kv_heads", spec["heads"]))
        self.dk, self.dv, self.taps = int(spec["dim"]), int(spec["vdim"]), int(spec["conv"])
        self.eps = eps
        self.n_conv = 2 * self.G * self.dk + self.H * self.dv
        self.ra, self.rg = t["a1"].shape[0], t["g1"].shape[0]
        sections = [torch.cat([t["q"], t["k"], t["v"]], dim=0), t["b"], t["a1"], t["g1"]]
        self.cuts = [0]
        for s in sections:
            self.cuts.append(self.cuts[-1] + s.shape[0] + (-s.shape[0] % 8))
        self.w_in = _param(torch.cat([_pad8(s) for s in sections], dim=0), device, dtype)
        self.w_conv = _param(torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0), device, dtype)
        self.w_a2, self.w_g2 = _param(t["a2"], device, dtype), _param(t["g2"], device, dtype)
        self.dt_bias, self.a_log = _param(t["dt_bias"], device, dtype), _param(t["A_log"], device, dtype)
        self.norm_w = _param(t["norm"], device, dtype)
        self.w_o = _param(t["o"], device, dtype)

    def forward(self, h: torch.Tensor, cache: RaggedLayerCache) -> torch.Tensor:
        st = cache.state
        H, G, dk, dv, c = self.H, self.G, self.dk, self.dv, self.cuts
        state, tail = cache.rstate
        proj = F.linear(h, self.w_in)
        qkv = mixer_ops.causal_conv_silu(proj[:, :self.n_conv], self.w_conv, tail, st.scan_seqs,
                                         max_count=max(sp[1] for sp in st.spans))
        a_logit = F.linear(proj[:, c[2]:c[2] + self.ra], self.w_a2)
        gate = F.linear(proj[:, c[3]:c[3] + self.rg], self.w_g2)
        o = mixer_ops.delta_scan(qkv[:, :G * dk], qkv[:, G * dk:2 * G * dk], qkv[:, 2 * G * dk:], proj[:, c[1]:c[1] + H],
                                 a_logit, self.dt_bias, self.a_log, state, st.scan_seqs, G, UNIT_NORM_EPS, dk ** -0.5)
        return F.linear(mixer_ops.head_rmsnorm_gated(o, self.norm_w, gate, self.eps), self.w_o)


class XieluMLP(nn.Module):
    def __init__(self, t: Dict[str, torch.Tensor], device, dtype):
        super().__init__()
        self.w_up, self.w_down = _param(t["up"], device, dtype), _param(t["down"], device, dtype)
        self.pq = _param(t["act"], device, dtype)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return F.linear(mixer_ops.xielu(F.linear(h, self.w_up), self.pq), self.w_down)


class SanesunDecoderLayer(nn.Module):
    """One layer; see the module docstring.  ``next_norm_weight`` (set by the builder when another layer of the same
    shard follows) lets the residual update also produce that layer's normed input."""

    def __init__(self, config: SanesunConfig, layer_idx: int, t: Dict[str, torch.Tensor], device=None, dtype=None):
        super().__init__()
        spec = config.layers[layer_idx]
        self.layer_idx, self.kind, self.eps = layer_idx, spec["type"], config.eps
        mix = {k[4:]: v for k, v in t.items() if k.startswith("mix.")}
        if self.kind == "attention":
            self.mixer = WindowedSinkAttention(spec["mixer"], mix, device, dtype)
        elif self.kind == "latent_attention":
            self.mixer = LatentAttention(spec["mixer"], mix, self.eps, device, dtype)
        else:
            self.mixer = ChannelDeltaMixer(spec["mixer"], mix, self.eps, device, dtype)
        self.norm1 = PlainRMSNorm(config.width, self.eps, device, dtype)
        with torch.no_grad():
            self.norm1.weight.copy_(t["norm1"])
        self.mlp = None
        if spec.get("mlp") is not None:
            self.mlp = XieluMLP({k[4:]: v for k, v in t.items() if k.startswith("mlp.")}, device, dtype)
        self.next_norm_weight: Optional[torch.Tensor] = None

    def forward(self, hidden_states: torch.Tensor, attention_mask=None, position_ids=None,
                past_key_value: Optional[RaggedLayerCache] = None, use_cache: bool = True):
        if not isinstance(past_key_value, RaggedLayerCache):
            raise TypeError("SanesunDecoderLayer needs a RaggedLayerCache handle in past_key_value")
        x, st = hidden_states, past_key_value.state
        if x.dtype != torch.float32 or x.dim() != 2:
            raise TypeError("the residual stream is a packed fp32 [n_tok, width] tensor")
        h = st.pending_norm if st.pending_norm is not None else self.norm1(x)
        st.pending_norm = None
        y = self.mixer(h, past_key_value)
        z = self.mlp(h) if self.mlp is not None else None
        st.pending_norm = mixer_ops.residual_add2_norm(x, y, z, self.next_norm_weight, self.eps)
        return x, (past_key_value if use_cache else None)


def build_shards(config: SanesunConfig, tensors: Dict[str, torch.Tensor], ranges: Sequence[Tuple[int, int]],
                 device: str, dtype: torch.dtype) -> List[ModelShard]:
    """``ModelShard``s for layer ranges holding the weights of a checkpoint's name -> tensor dict."""
    shards = []
    total = config.num_hidden_layers
    for start, end in ranges:
        layers = []
        for i in range(start, end):
            pre = f"l{i}."
            layers.append(SanesunDecoderLayer(config, i, {k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)},
                                              device, dtype))
        for a, b in zip(layers[:-1], layers[1:]):
            a.next_norm_weight = b.norm1.weight
        embed = norm = head = None
        if start == 0:
            embed = ScaledFloatEmbedding(config.vocab, config.width, device=device, dtype=dtype, scale=config.embed_scale)
            embed.weight.requires_grad_(False)
            with torch.no_grad():
                embed.weight.copy_(tensors["embed"])
        if end == total:
            norm = PlainRMSNorm(config.width, config.eps, device, dtype)
            head = nn.Linear(config.width, config.vocab, bias=False, device=device, dtype=dtype)
            head.weight.requires_grad_(False)
            with torch.no_grad():
                norm.weight.copy_(tensors["final.norm"])
                head.weight.copy_(tensors["head"])
        shards.append(ModelShard.from_layers(config, layers, start, end, device, dtype, embed, norm, head,
                                             model_id="sanesun").eval())
    return shards


def random_checkpoint(config: SanesunConfig, seed: int = 0, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Random weights with the checkpoint's names and shapes (for tests and benchmarks; not a trained model).
    Projections ~ N(0, 1 / fan_in); norm weights, biases, sinks and the mixing matrix are chosen so that every term
    of the design contributes."""
    g = torch.Generator().manual_seed(seed)
    W = config.width

    def lin(out, inp, gain=1.0):
        return (torch.randn(out, inp, generator=g) * gain / math.sqrt(inp)).to(dtype)

    def near_one(*shape, s=0.1):
        return (1.0 + s * torch.randn(*shape, generator=g)).to(dtype)

    t: Dict[str, torch.Tensor] = {"embed": (torch.randn(config.vocab, W, generator=g) / config.embed_scale).to(dtype)}
    for i, layer in enumerate(config.layers):
        pre, m = f"l{i}.mix.", layer["mixer"]
        t[f"l{i}.norm1"] = near_one(W)
        H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        if layer["type"] == "attention":
            G = int(m.get("kv_heads", H))
            for name, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
                t[pre + name] = lin(rows, W, 1.5)
                t[pre + name + ".b"] = (0.1 * torch.randn(rows, generator=g)).to(dtype)
            t[pre + "talk"] = (torch.eye(H) + 0.3 * torch.randn(H, H, generator=g) / math.sqrt(H)).to(dtype)
            t[pre + "sink"] = torch.randn(H, generator=g).to(dtype)
            t[pre + "o"] = lin(W, H * dv)
        elif layer["type"] == "latent_attention":
            rq, r = int(m["q_rank"]), int(m["kv_rank"])
            t[pre + "dq"], t[pre + "dq.norm"], t[pre + "uq"] = lin(rq, W), near_one(rq), lin(H * dk, rq, 1.5)
            t[pre + "dkv"], t[pre + "dkv.norm"] = lin(r, W), near_one(r)
            t[pre + "uk"], t[pre + "uv"] = lin(H * dk, r, 1.5), lin(H * dv, r)
            t[pre + "g"] = lin(H, W)
            t[pre + "o"] = lin(W, H * dv)
        else:
            G, taps = int(m.get("kv_heads", H)), int(m["conv"])
            ra = rg = max(8, W // 16)
            for name, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                t[pre + name] = lin(rows, W, 1.5)
                t[pre + name + ".conv"] = (torch.randn(rows, taps, generator=g) / math.sqrt(taps)).to(dtype)
            t[pre + "b"] = lin(H, W)
            t[pre + "A_log"] = (torch.rand(H, generator=g) * 2.0 - 1.5).to(dtype)
            t[pre + "a1"], t[pre + "a2"] = lin(ra, W), lin(H * dk, ra, 2.0)
            t[pre + "dt_bias"] = (torch.randn(H * dk, generator=g) - 1.0).to(dtype)
            t[pre + "g1"], t[pre + "g2"] = lin(rg, W), lin(H * dv, rg, 2.0)
            t[pre + "norm"] = near_one(dv)
            t[pre + "o"] = lin(W, H * dv)
        mlp = layer.get("mlp")
        if mlp:
            ff = int(mlp["ff"])
            t[f"l{i}.mlp.up"], t[f"l{i}.mlp.down"] = lin(ff, W), lin(W, ff)
            t[f"l{i}.mlp.act"] = torch.tensor([0.4, -0.3]).to(dtype)
    t["final.norm"] = near_one(W)
    t["head"] = lin(config.vocab, W)
    return t
