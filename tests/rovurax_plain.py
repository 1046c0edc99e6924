"""A plain, slow restatement of the Rovurax design, one function per mechanism, on the CPU.

Nothing here is shared with the package: tensors come in as a dict name -> torch tensor, the
configuration as the dict that config.json holds, and every sequence is computed whole, position
by position where that is the clearest way to say it.  `dtype` is the arithmetic of the parts that
may run in reduced precision (float64 by default: the yardstick the GPU paths are measured with).

Notation: x is a row of the residual stream, h its normed copy, p a position counted from 0.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def clipped_glu(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    """g = min(gate h, L); u = clamp(up h, -L, L); down (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequency per pair [dims/2], the factor that multiplies cos and sin)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, scaling: Optional[dict]) -> torch.Tensor:
    """x [..., T, D]: the first `dims` values of the last axis turn, value 2i with value 2i+1."""
    f, mag = yarn_frequencies(dims, base, scaling)
    ang = positions.to(torch.float64)[:, None] * f[None, :]
    cos, sin = (torch.cos(ang) * mag).to(x.dtype), (torch.sin(ang) * mag).to(x.dtype)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def softmax_rows(scores: torch.Tensor, visible: torch.Tensor, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """scores [H, T, T], visible [T, T] bool, sink [H] or None: weights whose denominator also
    holds exp(sink) once."""
    s = scores.masked_fill(~visible[None], float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return e / den


def causal_mask(T: int, chunk: Optional[int] = None) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    vis = j <= i
    if chunk:
        vis = vis & (i // chunk == j // chunk)
    return vis


def chunked_attention(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, mix: dict, v_first: Optional[torch.Tensor]):
    """Grouped-query attention without positions, over chunks; returns (output, this layer's values
    before mixing)."""
    T = h.shape[0]
    H, G, d, dv = mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"]
    q = (h @ t[p + "q"].T).view(T, H, d).transpose(0, 1)
    k = (h @ t[p + "k"].T).view(T, G, d).transpose(0, 1)
    v_raw = (h @ t[p + "v"].T).view(T, G, dv).transpose(0, 1)
    v = v_raw
    if mix.get("v_mix") and v_first is not None:
        lam = t[p + "vmix"].to(h.dtype)
        v = (1.0 - lam) * v_raw + lam * v_first
    rep = H // G
    kk, vv = k.repeat_interleave(rep, 0), v.repeat_interleave(rep, 0)
    scores = (q @ kk.transpose(1, 2)) * mix["scale"]
    size = (mix.get("mask") or {}).get("size")
    w = softmax_rows(scores, causal_mask(T, size))
    out = (w @ vv).transpose(0, 1).reshape(T, H * dv)
    return out @ t[p + "o"].T, v_raw


def latent_attention(h: torch.Tensor, t: Dict[str, torch.Tensor], p: str, mix: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, r, dv, rank = mix["heads"], mix["dim"], mix["rot_dim"], mix["vdim"], mix["kv_rank"]
    rot = mix["rot"]
    pos = torch.arange(T)
    q = (h @ t[p + "q"].T).view(T, H, d + r).transpose(0, 1)
    dkv = h @ t[p + "dkv"].T
    c = rms_norm(dkv[:, :rank], t[p + "dkv.norm"].to(h.dtype), eps)
    k_rot = rotate_interleaved(dkv[:, rank:], pos, rot["dims"], rot["base"], rot.get("scaling"))
    k_un = (c @ t[p + "uk"].T).view(T, H, d).transpose(0, 1)
    v = (c @ t[p + "uv"].T).view(T, H, dv).transpose(0, 1)
    q_un = q[..., :d]
    q_rot = rotate_interleaved(q[..., d:], pos, rot["dims"], rot["base"], rot.get("scaling"))
    scores = (q_un @ k_un.transpose(1, 2) + q_rot @ k_rot.T[None]) * mix["scale"]
    w = softmax_rows(scores, causal_mask(T), t[p + "sink"].to(h.dtype))
    gate = torch.sigmoid(h @ t[p + "g"].T)
    out = (w @ v) * gate.T[:, :, None]
    return out.transpose(0, 1).reshape(T, H * dv) @ t[p + "o"].T


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, layers_out: Optional[list] = None):
    """Logits [T, vocab] of one sequence computed whole."""
    t = {k: v.to(dtype) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = t["embed"][torch.tensor(tokens)]
    v_first = None
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, t[p + "norm1"], eps)
        mix = layer["mixer"]
        if layer["type"] == "attention":
            m, v_raw = chunked_attention(h, t, p + "mix.", mix, v_first)
            if mix.get("v_mix") and v_first is None:
                v_first = v_raw
        elif layer["type"] == "latent_attention":
            m = latent_attention(h, t, p + "mix.", mix, eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            assert mlp["kind"] == "dense"
            m = m + clipped_glu(h, t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"], float(mlp["limit"]))
        x = x + m
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, t["final.norm"], eps) @ t["head"].T
