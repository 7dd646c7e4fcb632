"""Petipel: a decoder whose layers pick one of two sequence mixers and one of two feed-forwards, over an fp32
residual stream with a norm before AND after every sublayer.

    x <- x + m * norm_b(mixer(norm_a(x)))          x <- x + m * norm_d(ff(norm_c(x)))

Mixers
  ``attention``  grouped-query softmax attention without rotation.  Position enters through a learned bias per
                 (bucketed distance, head) and a query temperature that grows with the logarithm of the position.
                 Values are unit-RMS per head, optionally blended with the values the first such layer produced
                 for the same token, and the head outputs pass a per-head sigmoid gate.  K rows and V rows have
                 their own widths, so the layer's paged pools do too.
  ``hgrn2``      gated linear recurrence: the forget gate f (bounded below per channel) also sets the write
                 strength 1 - f; the state ``[heads, dk, dv]`` is fp32 and lives in a slot pool per live sequence.
Feed-forwards
  ``dense``      up -> PolyNorm (a N(z) + b N(z^2) + c N(z^3) + e) -> down
  ``moe``        sigmoid-scored top-k routing whose score scales the expert's INPUT; experts are clamped GLUs.

The modules below follow the calling convention of ``ModelShard.forward`` (reference:
worker/distributed/model_shard.py:205-215): ``layer(h, attention_mask=, position_ids=, past_key_value=, use_cache=)
-> (h, present)``.  ``h`` is the packed fp32 residual ``[n_tok, width]`` of one step and ``past_key_value`` a
``RaggedLayerCache``.  Matrix products are torch GEMMs; everything between them is one of the kernels of
``mixer_ops``.  There is no dense / CPU mode.

Checkpoint names: ``embed``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``,
``head``; linear weights are ``[out, in]``.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import mixer_ops
from .paged_layer import RaggedLayerCache
from .worker.distributed.model_shard import ModelShard


class PetipelConfig:
    """``config.json`` of the design, plus the attribute names the rest of the framework reads from a config."""

    def __init__(self, raw: Dict[str, Any]):
        self.raw = raw
        self.architecture = raw.get("architecture", "Petipel")
        self.layers: List[Dict[str, Any]] = list(raw["layers"])
        self.width = int(raw["width"])
        self.vocab = int(raw["vocab"])
        self.eps = float(raw["norm"]["eps"])
        self.residual_mult = float(raw["residual_mult"])
        for i, layer in enumerate(self.layers):
            if layer["type"] not in ("attention", "hgrn2"):
                raise NotImplementedError(f"layer {i}: unknown mixer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp["kind"] not in ("dense", "moe"):
                raise NotImplementedError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
        # names shared with the other model classes
        self.hidden_size = self.width
        self.vocab_size = self.vocab
        self.num_hidden_layers = len(self.layers)
        self.num_attention_heads = max(int(l["mixer"]["heads"]) for l in self.layers)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PetipelConfig":
        return cls(raw)

    def first_value_mix_layer(self) -> Optional[int]:
        for i, layer in enumerate(self.layers):
            if layer["type"] == "attention" and layer["mixer"].get("v_mix"):
                return i
        return None

    def kv_shape(self, i: int) -> Optional[Tuple[int, int, int]]:
        m = self.layers[i]["mixer"]
        return (int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])) if self.layers[i]["type"] == "attention" else None

    def state_shape(self, i: int) -> Optional[Tuple[int, int, int]]:
        m = self.layers[i]["mixer"]
        return (int(m["heads"]), int(m["dim"]), int(m["vdim"])) if self.layers[i]["type"] == "hgrn2" else None


def log_distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of a ``rows``-row distance table for distance ``n``: one row per distance below ``rows // 2``, then rows
    spread evenly over ln(distance) up to ``far``; everything at or beyond ``far`` shares the last row."""
    half = rows // 2
    if n < half:
        return n
    if half == 0 or far <= half:
        return rows - 1
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_bias_table(rel: torch.Tensor, far: float) -> torch.Tensor:
    """``rel [rows, H]`` -> fp32 ``[H, L]`` with entry ``[h, d]`` the bias of distance ``d``; distances >= L - 1 use
    the last column (from ``far`` on the bucket no longer changes)."""
    rows = rel.shape[0]
    length = max(int(math.ceil(far)), rows // 2) + 1
    while log_distance_bucket(length - 1, rows, far) != rows - 1 and length < (1 << 22):
        length += 1
    idx = torch.tensor([log_distance_bucket(d, rows, far) for d in range(length)], dtype=torch.int64)
    return rel.detach().to(torch.float32).cpu()[idx].t().contiguous()


class OffsetRMSNorm(nn.Module):
    """RMS norm whose weight is stored around zero: ``x * rsqrt(mean(x^2) + eps) * (1 + w)``, fp32 in."""

    def __init__(self, width: int, eps: float, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(width, device=device, dtype=dtype), requires_grad=False)
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return mixer_ops.offset_rmsnorm(x, self.weight, self.eps)


class FloatEmbedding(nn.Embedding):
    """Embedding whose rows open an fp32 residual stream, whatever dtype the table is stored in."""

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return super().forward(ids).to(torch.float32)


def _param(t: torch.Tensor, device, dtype) -> nn.Parameter:
    return nn.Parameter(t.to(device=device, dtype=dtype).contiguous(), requires_grad=False)


class BiasedPagedAttention(nn.Module):
    """The ``attention`` mixer.  One GEMM produces q | k | v | gate logits; values are normed, mixed and appended with
    the keys in one launch; one attention launch serves prompt portions and decoded tokens alike."""

    def __init__(self, spec: Dict[str, Any], t: Dict[str, torch.Tensor], eps: float, is_first_mix: bool, device, dtype):
        super().__init__()
        self.H, self.G = int(spec["heads"]), int(spec["kv_heads"])
        self.dk, self.dv = int(spec["dim"]), int(spec["vdim"])
        if self.H % self.G:
            raise ValueError("query heads must be a multiple of key/value heads")
        self.scale = float(spec["scale"])
        qt = spec.get("q_temp") or {}
        self.temp_coef, self.temp_every = float(qt.get("coef", 0.0)), int(qt.get("every", 1))
        self.v_mix = bool(spec.get("v_mix", False))
        self.is_first_mix = is_first_mix
        self.eps = eps
        w_in = torch.cat([t["q"], t["k"], t["v"], t["g"]], dim=0)
        pad = -w_in.shape[0] % 8     # zero rows: projection rows stay 16-byte aligned for the kernels' vector loads
        self.w_in = _param(torch.cat([w_in, w_in.new_zeros(pad, w_in.shape[1])], dim=0), device, dtype)
        self.w_o = _param(t["o"], device, dtype)
        self.tensor_core_prompt = mixer_ops.prompt_attention_supported(self.dk, self.dv, self.w_in.dtype)
        self.register_buffer("bias_lut", distance_bias_table(t["rel"], float(spec["bias_max"])).to(device), persistent=False)
        self.lam = float(t["vmix"].to(torch.float32)) if "vmix" in t else 0.0

    def forward(self, h: torch.Tensor, cache: RaggedLayerCache) -> torch.Tensor:
        st = cache.state
        H, G, dk, dv = self.H, self.G, self.dk, self.dv
        proj = F.linear(h, self.w_in)
        a, b, c = H * dk, (H + G) * dk, (H + G) * dk + G * dv
        v_prev = v_keep = None
        if self.v_mix:
            if self.is_first_mix:
                v_keep = st.v_first = torch.empty((h.shape[0], G * dv), dtype=h.dtype, device=h.device)
            else:
                v_prev = st.v_first
                if v_prev is None or v_prev.shape[1] != G * dv:
                    raise RuntimeError("value mixing needs the first mixing layer's values of this step (same shape)")
        mixer_ops.value_prep_append(proj[:, a:b], proj[:, b:c], cache.k_pool, cache.v_pool, st.slot_mapping, self.eps,
                                    v_prev=v_prev, lam=self.lam, v_keep=v_keep)
        q, gate = proj[:, :a], proj[:, c:c + H]
        attn = torch.empty((h.shape[0], H * dv), dtype=h.dtype, device=h.device)
        if self.tensor_core_prompt:   # 16-bit storage and sizes the tensor-core kernel takes: portions and single tokens
            tiles, most = st.prompt_tiles(1, mixer_ops.prompt_tile_tokens(H, G))
            mixer_ops.biased_prompt_attention(attn, q, gate, cache.k_pool, cache.v_pool, st.block_tables, tiles,
                                              st.tok_pos, self.bias_lut, self.scale, self.temp_coef, self.temp_every, H,
                                              max_tile_tokens=most)
        else:                         # fp32, or head sizes off the tensor-core grid: the row kernel
            tiles, most = st.tiles_for(H, G)
            mixer_ops.biased_paged_attention(q, gate, cache.k_pool, cache.v_pool, st.block_tables, tiles, most,
                                             st.tok_pos, self.bias_lut, self.scale, self.temp_coef, self.temp_every, H,
                                             out=attn)
        return F.linear(attn, self.w_o)


class GatedLinearRecurrence(nn.Module):
    """The ``hgrn2`` mixer: one GEMM produces q | f | v pre-activations, one launch runs the recurrence of every
    (sequence, head) over the step's tokens against the state pool, one launch norms the read-outs per head."""

    def __init__(self, spec: Dict[str, Any], t: Dict[str, torch.Tensor], eps: float, device, dtype):
        super().__init__()
        self.H, self.dk, self.dv = int(spec["heads"]), int(spec["dim"]), int(spec["vdim"])
        self.eps = eps
        self.w_in = _param(torch.cat([t["q"], t["f"], t["v"]], dim=0), device, dtype)
        self.f_bias = _param(t["f.b"], device, dtype)
        self.lower = _param(t["lower"], device, dtype)
        self.norm_w = _param(t["norm"], device, dtype)
        self.w_o = _param(t["o"], device, dtype)

    def forward(self, h: torch.Tensor, cache: RaggedLayerCache) -> torch.Tensor:
        n, a = h.shape[0], self.H * self.dk
        proj = F.linear(h, self.w_in)
        o = mixer_ops.gated_scan(proj[:, :a], proj[:, a:2 * a], proj[:, 2 * a:], self.f_bias, self.lower, cache.rstate,
                                 cache.state.scan_seqs, self.H, max_count=max(sp[1] for sp in cache.state.spans))
        return F.linear(mixer_ops.head_rmsnorm(o, self.norm_w, self.eps).view(n, self.H * self.dv), self.w_o)


class PolyNormMLP(nn.Module):
    def __init__(self, t: Dict[str, torch.Tensor], eps: float, device, dtype):
        super().__init__()
        self.eps = eps
        self.w_up, self.w_down = _param(t["up"], device, dtype), _param(t["down"], device, dtype)
        self.coef = _param(t["act"], device, dtype)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return F.linear(mixer_ops.polynorm(F.linear(h, self.w_up), self.coef, self.eps), self.w_down)


class SigmoidTopKMoE(nn.Module):
    """Router in fp32; tokens are sorted by expert, scaled by their score on the way in, pushed through the experts'
    clamped GLUs and summed per token in fp32.  ``GLU_ALPHA`` is fixed by the design."""

    GLU_ALPHA = 1.702
    GROUPED_MAX_ROWS = 2048     # routed rows of a step up to which the grouped kernel beats per-expert vendor GEMMs

    def __init__(self, spec: Dict[str, Any], t: Dict[str, torch.Tensor], device, dtype):
        super().__init__()
        self.E, self.top = int(spec["router"]["experts"]), int(spec["router"]["top"])
        self.limit = float(spec["expert"]["limit"])
        self.w_router = _param(t["router"], device, torch.float32)
        self.w_gu = _param(torch.stack([torch.cat([t[f"e{e}.gate"], t[f"e{e}.up"]], dim=0) for e in range(self.E)]),
                           device, dtype)                                                    # [E, 2 ff, W]
        self.w_down = _param(torch.stack([t[f"e{e}.down"] for e in range(self.E)]), device, dtype)  # [E, W, ff]
        self.grouped = (mixer_ops.grouped_linear_supported(self.w_gu.shape[2], self.w_gu.dtype)
                        and mixer_ops.grouped_linear_supported(self.w_down.shape[2], self.w_down.dtype))

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        n, top = h.shape[0], self.top
        ids, w = mixer_ops.sigmoid_topk(F.linear(h.to(torch.float32), self.w_router), top)
        flat = ids.reshape(-1).to(torch.int64)
        order = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=self.E)
        xs = mixer_ops.scaled_gather(h, w.reshape(-1), order, top)
        if self.grouped and n * top <= self.GROUPED_MAX_ROWS:
            # all experts in one launch each way, offsets stay on the device: no host copy, no per-expert calls
            offsets = torch.zeros(self.E + 1, dtype=torch.int32, device=h.device)
            offsets[1:] = torch.cumsum(counts, 0)
            y = mixer_ops.clamped_glu(mixer_ops.grouped_linear(xs, self.w_gu, offsets), self.limit, self.GLU_ALPHA)
            ys = mixer_ops.grouped_linear(y, self.w_down, offsets)
        else:
            # long prompt steps (and fp32): one vendor GEMM per expert each way; the counts come to the host once
            counts = counts.tolist()
            gu = torch.empty((n * top, self.w_gu.shape[1]), dtype=h.dtype, device=h.device)
            lo = 0
            for e, c in enumerate(counts):
                if c:
                    torch.mm(xs[lo:lo + c], self.w_gu[e].t(), out=gu[lo:lo + c])
                    lo += c
            y = mixer_ops.clamped_glu(gu, self.limit, self.GLU_ALPHA)
            ys = torch.empty((n * top, h.shape[1]), dtype=h.dtype, device=h.device)
            lo = 0
            for e, c in enumerate(counts):
                if c:
                    torch.mm(y[lo:lo + c], self.w_down[e].t(), out=ys[lo:lo + c])
                    lo += c
        where = torch.empty_like(order)
        where[order] = torch.arange(n * top, device=h.device)
        return mixer_ops.expert_combine(ys, where, n, top)


class PetipelDecoderLayer(nn.Module):
    """One layer; see the module docstring.  ``next_norm_weight`` (set by the builder when another layer of the same
    shard follows) lets the layer's last residual update also produce that layer's normed input."""

    def __init__(self, config: PetipelConfig, layer_idx: int, t: Dict[str, torch.Tensor], device=None, dtype=None):
        super().__init__()
        spec = config.layers[layer_idx]
        self.layer_idx, self.kind = layer_idx, spec["type"]
        self.eps, self.mult = config.eps, config.residual_mult
        W = config.width
        mix = {k[4:]: v for k, v in t.items() if k.startswith("mix.")}
        if self.kind == "attention":
            self.mixer = BiasedPagedAttention(spec["mixer"], mix, self.eps, config.first_value_mix_layer() == layer_idx,
                                              device, dtype)
        else:
            self.mixer = GatedLinearRecurrence(spec["mixer"], mix, self.eps, device, dtype)
        self.norm1, self.norm1b = OffsetRMSNorm(W, self.eps, device, dtype), OffsetRMSNorm(W, self.eps, device, dtype)
        names = ["norm1", "norm1b"]
        mlp = spec.get("mlp")
        self.mlp = None
        if mlp is not None:
            ff = {k[4:]: v for k, v in t.items() if k.startswith("mlp.")}
            self.mlp = PolyNormMLP(ff, self.eps, device, dtype) if mlp["kind"] == "dense" else SigmoidTopKMoE(mlp, ff, device, dtype)
            self.norm2, self.norm2b = OffsetRMSNorm(W, self.eps, device, dtype), OffsetRMSNorm(W, self.eps, device, dtype)
            names += ["norm2", "norm2b"]
        with torch.no_grad():
            for name in names:
                getattr(self, name).weight.copy_(t[name])
        self.next_norm_weight: Optional[torch.Tensor] = None

    def forward(self, hidden_states: torch.Tensor, attention_mask=None, position_ids=None,
                past_key_value: Optional[RaggedLayerCache] = None, use_cache: bool = True):
        if not isinstance(past_key_value, RaggedLayerCache):
            raise TypeError("PetipelDecoderLayer needs a RaggedLayerCache handle in past_key_value")
        x, st = hidden_states, past_key_value.state
        if x.dtype != torch.float32 or x.dim() != 2:
            raise TypeError("the residual stream is a packed fp32 [n_tok, width] tensor")
        h = st.pending_norm if st.pending_norm is not None else self.norm1(x)
        st.pending_norm = None
        y = self.mixer(h, past_key_value)
        if self.mlp is not None:
            h = mixer_ops.postnorm_residual(x, y, self.norm1b.weight, self.mult, self.eps, w_next=self.norm2.weight)
            y = self.mlp(h)
            st.pending_norm = mixer_ops.postnorm_residual(x, y, self.norm2b.weight, self.mult, self.eps,
                                                         w_next=self.next_norm_weight)
        else:
            st.pending_norm = mixer_ops.postnorm_residual(x, y, self.norm1b.weight, self.mult, self.eps,
                                                         w_next=self.next_norm_weight)
        return x, (past_key_value if use_cache else None)


def build_shards(config: PetipelConfig, tensors: Dict[str, torch.Tensor], ranges: Sequence[Tuple[int, int]],
                 device: str, dtype: torch.dtype) -> List[ModelShard]:
    """``ModelShard``s for layer ranges holding the weights of a checkpoint's name -> tensor dict."""
    shards = []
    total = config.num_hidden_layers
    for start, end in ranges:
        layers = []
        for i in range(start, end):
            pre = f"l{i}."
            layers.append(PetipelDecoderLayer(config, i, {k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)},
                                              device, dtype))
        for a, b in zip(layers[:-1], layers[1:]):
            a.next_norm_weight = b.norm1.weight
        embed = norm = head = None
        if start == 0:
            embed = FloatEmbedding(config.vocab, config.width, device=device, dtype=dtype)
            embed.weight.requires_grad_(False)
            with torch.no_grad():
                embed.weight.copy_(tensors["embed"])
        if end == total:
            norm = OffsetRMSNorm(config.width, config.eps, device, dtype)
            head = nn.Linear(config.width, config.vocab, bias=False, device=device, dtype=dtype)
            head.weight.requires_grad_(False)
            with torch.no_grad():
                norm.weight.copy_(tensors["final.norm"])
                head.weight.copy_(tensors["head"])
        shards.append(ModelShard.from_layers(config, layers, start, end, device, dtype, embed, norm, head,
                                             model_id="petipel").eval())
    return shards


def random_checkpoint(config: PetipelConfig, seed: int = 0, dtype: torch.dtype = torch.bfloat16,
                      bias_rows: int = 32) -> Dict[str, torch.Tensor]:
    """Random weights with the checkpoint's names and shapes (for tests and benchmarks; not a trained model).
    Projections ~ N(0, 1 / fan_in); norm weights, gates' biases and table entries small and non-zero so that every
    term of the design contributes."""
    g = torch.Generator().manual_seed(seed)
    W = config.width

    def lin(out, inp, gain=1.0):
        return (torch.randn(out, inp, generator=g) * gain / math.sqrt(inp)).to(dtype)

    def small(*shape, s=0.1):
        return (torch.randn(*shape, generator=g) * s).to(dtype)

    t: Dict[str, torch.Tensor] = {"embed": (torch.randn(config.vocab, W, generator=g)).to(dtype)}
    for i, layer in enumerate(config.layers):
        pre, m = f"l{i}.", layer["mixer"]
        for name in ("norm1", "norm1b") + (("norm2", "norm2b") if layer.get("mlp") else ()):
            t[pre + name] = small(W)
        H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        if layer["type"] == "attention":
            G = int(m["kv_heads"])
            t[pre + "mix.q"], t[pre + "mix.k"], t[pre + "mix.v"] = lin(H * dk, W), lin(G * dk, W), lin(G * dv, W)
            t[pre + "mix.rel"] = small(bias_rows, H, s=0.5)
            t[pre + "mix.vmix"] = torch.tensor(0.3 + 0.05 * (i % 5)).to(dtype)
            t[pre + "mix.g"] = lin(H, W)
            t[pre + "mix.o"] = lin(W, H * dv)
        else:
            t[pre + "mix.q"], t[pre + "mix.f"], t[pre + "mix.v"] = lin(H * dk, W), lin(H * dk, W, 2.0), lin(H * dv, W)
            t[pre + "mix.f.b"] = small(H * dk, s=1.0)
            t[pre + "mix.lower"] = (torch.rand(H * dk, generator=g) * 0.9).to(dtype)
            t[pre + "mix.norm"] = (1.0 + 0.1 * torch.randn(dv, generator=g)).to(dtype)
            t[pre + "mix.o"] = lin(W, H * dv)
        mlp = layer.get("mlp")
        if mlp and mlp["kind"] == "dense":
            ff = int(mlp["ff"])
            t[pre + "mlp.up"], t[pre + "mlp.down"] = lin(ff, W), lin(W, ff)
            t[pre + "mlp.act"] = torch.tensor([0.6, 0.3, 0.2, 0.05]).to(dtype)
        elif mlp:
            ff, E = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"])
            for e in range(E):
                t[pre + f"mlp.e{e}.gate"], t[pre + f"mlp.e{e}.up"] = lin(ff, W, 2.0), lin(ff, W, 2.0)
                t[pre + f"mlp.e{e}.down"] = lin(W, ff)
            t[pre + "mlp.router"] = lin(E, W, 2.0)
    t["final.norm"] = small(W)
    t["head"] = lin(config.vocab, W)
    return t
