"""Plain, slow statement of the Petipel decoder in fp32 torch on the CPU: one function per mechanism.

Shares no code with the CUDA path.  Every function takes a whole sequence (``[T, ...]`` tensors, positions 0..T-1)
and loops where the definition loops.  ``forward`` strings them together from a config dict and a name -> tensor
dict laid out like the checkpoint (``l<i>.mix.q`` ...).

Notation: ``W`` width, ``H`` query heads, ``G`` key/value heads, ``dk`` query/key size, ``dv`` value size.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F32 = torch.float32


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight sits around zero: unit(x) * (1 + w)."""
    return rms_unit(x, eps) * (1.0 + w)


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Bucket of distance ``n`` in a table of ``rows`` rows: exact below rows/2, logarithmic up to ``far``."""
    half = rows // 2
    if n < half:
        return n
    if half == 0:
        return rows - 1
    step = math.log(n / half) / math.log(far / half) * (rows - half)
    return min(rows - 1, half + int(math.floor(step)))


def query_temperature(p: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log(((p + 1) // every) + 1)


def attention_mixer(h: torch.Tensor, t: Dict[str, torch.Tensor], m: dict, eps: float,
                    v_first: Optional[torch.Tensor]):
    """``h [T, W]`` -> ``(out [T, W], v_cached [T, G, dv])``.  ``v_first``: the values the first value-mixing layer
    cached for the same tokens (None in that layer, or when the layer does not mix)."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t["q"].T).view(T, H, dk)
    k = (h @ t["k"].T).view(T, G, dk)
    v = rms_unit((h @ t["v"].T).view(T, G, dv), eps)
    if m.get("v_mix") and v_first is not None:
        lam = t["vmix"].reshape(())
        v = (1.0 - lam) * v + lam * v_first
    gate = torch.sigmoid(h @ t["g"].T)                                   # [T, H]
    qt = m.get("q_temp")
    rel = t["rel"]                                                       # [rows, H]
    rows = rel.shape[0]
    out = torch.zeros(T, H, dv, dtype=F32)
    for i in range(T):
        temp = query_temperature(i, qt["coef"], qt["every"]) if qt else 1.0
        for hd in range(H):
            g = hd // (H // G)
            s = (k[: i + 1, g] @ (q[i, hd] * temp)) * m["scale"]
            s = s + torch.tensor([float(rel[distance_bucket(i - j, rows, m["bias_max"]), hd]) for j in range(i + 1)])
            w = torch.softmax(s, dim=0)
            out[i, hd] = (w[:, None] * v[: i + 1, g]).sum(0) * gate[i, hd]
    return out.reshape(T, H * dv) @ t["o"].T, v


def hgrn2_mixer(h: torch.Tensor, t: Dict[str, torch.Tensor], m: dict, eps: float,
                state: Optional[torch.Tensor] = None):
    """Gated linear recurrence; ``state [H, dk, dv]`` is carried (zeros at the start).  Returns ``(out, state)``."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = torch.nn.functional.silu(h @ t["q"].T).view(T, H, dk)
    v = (h @ t["v"].T).view(T, H, dv)
    low = t["lower"].view(H, dk)
    f = low + (1.0 - low) * torch.sigmoid(h @ t["f"].T + t["f.b"]).view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=F32) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=F32)
    for i in range(T):
        S = f[i][:, :, None] * S + (1.0 - f[i])[:, :, None] * v[i][:, None, :]
        o[i] = torch.einsum("hkv,hk->hv", S, q[i])
    o = rms_unit(o, eps) * t["norm"]
    return o.reshape(T, H * dv) @ t["o"].T, S


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    a, b, c, e = [float(x) for x in coef]
    return a * rms_unit(z, eps) + b * rms_unit(z * z, eps) + c * rms_unit(z * z * z, eps) + e


def dense_ff(h: torch.Tensor, t: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    return polynorm(h @ t["up"].T, t["act"], eps) @ t["down"].T


def expert_ff(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(x @ gate.T, max=limit)
    u = torch.clamp(x @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def moe_ff(h: torch.Tensor, t: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    """Sigmoid-scored top-k routing; the score scales the expert's INPUT and is not renormalised."""
    top, limit = mlp["router"]["top"], mlp["expert"]["limit"]
    s = torch.sigmoid(h @ t["router"].T)
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for e in torch.topk(s[i], top).indices.tolist():
            out[i] += expert_ff((s[i, e] * h[i])[None], t[f"e{e}.gate"], t[f"e{e}.up"], t[f"e{e}.down"], limit)[0]
    return out


def sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F32) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], states: Optional[list] = None,
            trace: Optional[list] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence from position 0.  ``trace`` (a list) receives the residual stream after
    every layer.  ``states`` (a list, one entry per layer) receives the recurrent layers' final state."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = tensors["embed"].to(F32)[torch.tensor(tokens)]
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        nrm = sub(tensors, pre)
        mix = sub(tensors, pre + "mix.")
        hin = offset_norm(x, nrm["norm1"], eps)
        if layer["type"] == "attention":
            y, v = attention_mixer(hin, mix, layer["mixer"], eps, v_first)
            if layer["mixer"].get("v_mix") and v_first is None:
                v_first = v
        elif layer["type"] == "hgrn2":
            y, S = hgrn2_mixer(hin, mix, layer["mixer"], eps)
            if states is not None:
                states.append(S)
        else:
            raise ValueError(layer["type"])
        x = x + mult * offset_norm(y, nrm["norm1b"], eps)
        if layer.get("mlp"):
            ff = sub(tensors, pre + "mlp.")
            hin = offset_norm(x, nrm["norm2"], eps)
            y = dense_ff(hin, ff, eps) if layer["mlp"]["kind"] == "dense" else moe_ff(hin, ff, layer["mlp"])
            x = x + mult * offset_norm(y, nrm["norm2b"], eps)
        if trace is not None:
            trace.append(x.clone())
    x = offset_norm(x, tensors["final.norm"].to(F32), eps)
    return x @ tensors["head"].to(F32).T
