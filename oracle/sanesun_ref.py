"""Plain statement of the Sanesun design in float64 on the CPU: one function per mechanism, whole sequences only, loops
where a loop says it most directly.  Slow on purpose; shares no code with the package.

Notation: ``h`` is a layer's normed input ``[n, width]``, positions count from 0, linear weights are ``[out, in]``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def xielu(z, p, q):
    pos = softplus(p) * z * z + z / 2
    neg = (0.5 + softplus(q)) * (torch.expm1(torch.clamp(z, max=0)) - z) + z / 2
    return torch.where(z > 0, pos, neg)


def turn(x, pos, dims, base, back=False, interleaved=False):
    """Rotate the first ``dims`` entries of the last axis of ``x [n, heads, d]``: pair i is (i, i + dims/2), or
    (2i, 2i + 1) when interleaved, turned by pos * base^(-2i/dims) (by minus that when ``back``)."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
        ang = pos.to(F64) * base ** (-2.0 * i / dims)
        if back:
            ang = -ang
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        out[..., a] = x[..., a] * c - x[..., b] * s
        out[..., b] = x[..., b] * c + x[..., a] * s
    return out


def visible(i, j, window, keep_first):
    return j <= i and (window <= 0 or i - j < window or j < keep_first)


def windowed_attention(q, k, v, scale, window=0, keep_first=0, talk=None, sink=None, rows=None):
    """``q [n, H, dk]``, ``k [n, G, dk]``, ``v [n, G, dv]`` (already rotated where the design rotates) -> ``[n, H, dv]``.
    Scores of all heads are mixed by ``talk [H, H]`` before the mask; ``sink [H]`` adds exp(sink) to the denominator.
    ``rows``: the query positions to compute (the others stay zero)."""
    n, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(n, H, v.shape[2], dtype=F64)
    for i in (range(n) if rows is None else rows):
        js = [j for j in range(n) if visible(i, j, window, keep_first)]
        raw = torch.stack([torch.stack([(q[i, h] * k[j, h // rep]).sum() * scale for j in js]) for h in range(H)])
        mixed = talk @ raw if talk is not None else raw
        for h in range(H):
            m = mixed[h].max()
            if sink is not None:
                m = torch.maximum(m, sink[h])
            e = torch.exp(mixed[h] - m)
            den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
            out[i, h] = (e[:, None] * torch.stack([v[j, h // rep] for j in js])).sum(0) / den
    return out


def attention_mixer(h, spec, t):
    n = h.shape[0]
    H, G, dk, dv = spec["heads"], spec.get("kv_heads", spec["heads"]), spec["dim"], spec["vdim"]
    pos = torch.arange(n)
    q = (h @ t["q"].T + t["q.b"]).view(n, H, dk)
    k = (h @ t["k"].T + t["k.b"]).view(n, G, dk)
    v = (h @ t["v"].T + t["v.b"]).view(n, G, dv)
    rot, mask = spec["rot"], spec["mask"]
    q, k = turn(q, pos, rot["dims"], rot["base"]), turn(k, pos, rot["dims"], rot["base"])
    v = turn(v, pos, dv, rot["base"])                     # stored turned by the key's own position
    o = windowed_attention(q, k, v, spec["scale"], mask["size"], mask["keep_first"], t["talk"], t["sink"])
    o = turn(o, pos, dv, rot["base"], back=True)          # and turned back by the query's
    return o.reshape(n, H * dv) @ t["o"].T


def latent_mixer(h, spec, t, eps):
    n = h.shape[0]
    H, dk, dv = spec["heads"], spec["dim"], spec["vdim"]
    cq = rms_norm(h @ t["dq"].T, t["dq.norm"], eps)
    q = (cq @ t["uq"].T).view(n, H, dk)
    c = rms_norm(h @ t["dkv"].T, t["dkv.norm"], eps)
    k, v = (c @ t["uk"].T).view(n, H, dk), (c @ t["uv"].T).view(n, H, dv)
    o = windowed_attention(q, k, v, spec["scale"])
    g = torch.sigmoid(h @ t["g"].T)
    return (o * g[:, :, None]).reshape(n, H * dv) @ t["o"].T


def causal_conv_silu(x, w):
    """``x [n, C]``, ``w [C, taps]`` with the last column on the current token; zeros before the start."""
    n, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for t_ in range(n):
        for i in range(taps):
            src = t_ - (taps - 1 - i)
            if src >= 0:
                y[t_] += w[:, i] * x[src]
    return y * torch.sigmoid(y)


def delta_rule(q, k, v, beta, g):
    """``q, k [n, H, dk]``, ``v [n, H, dv]``, ``beta [n, H]``, ``g [n, H, dk]`` -> read-outs ``[n, H, dv]``."""
    n, H, dk = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, dk, dv, dtype=F64)
    o = torch.zeros(n, H, dv, dtype=F64)
    for t_ in range(n):
        for h in range(H):
            S[h] = g[t_, h][:, None] * S[h]
            u = beta[t_, h] * (v[t_, h] - S[h].T @ k[t_, h])
            S[h] = S[h] + torch.outer(k[t_, h], u)
            o[t_, h] = S[h].T @ q[t_, h]
    return o


def delta_mixer(h, spec, t, eps):
    n = h.shape[0]
    H, G, dk, dv = spec["heads"], spec.get("kv_heads", spec["heads"]), spec["dim"], spec["vdim"]
    q = causal_conv_silu(h @ t["q"].T, t["q.conv"]).view(n, G, dk)
    k = causal_conv_silu(h @ t["k"].T, t["k.conv"]).view(n, G, dk)
    v = causal_conv_silu(h @ t["v"].T, t["v.conv"]).view(n, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ t["b"].T)
    a = ((h @ t["a1"].T) @ t["a2"].T + t["dt_bias"]).view(n, H, dk)
    g = torch.exp(-torch.exp(t["A_log"])[None, :, None] * softplus(a))
    o = delta_rule(q, k, v, beta, g)
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * t["norm"]
    gate = torch.sigmoid((h @ t["g1"].T) @ t["g2"].T).view(n, H, dv)
    return (o * gate).reshape(n, H * dv) @ t["o"].T


def forward(cfg: Dict, tensors: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None):
    """Logits ``[n, vocab]`` of a whole sequence; ``tensors`` in any dtype (their stored values are taken exactly)."""
    w = {k: v.to(F64) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = rms_norm(x, w[pre + "norm1"], eps)
        mix = {k[len(pre) + 4:]: v for k, v in w.items() if k.startswith(pre + "mix.")}
        if layer["type"] == "attention":
            y = attention_mixer(h, layer["mixer"], mix)
        elif layer["type"] == "latent_attention":
            y = latent_mixer(h, layer["mixer"], mix, eps)
        else:
            y = delta_mixer(h, layer["mixer"], mix, eps)
        if layer.get("mlp") is not None:
            act = w[pre + "mlp.act"]
            y = y + xielu(h @ w[pre + "mlp.up"].T, act[0], act[1]) @ w[pre + "mlp.down"].T
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(cfg, tensors, prompt: List[int], n_new: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(cfg, tensors, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
