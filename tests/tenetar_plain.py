"""Tenetar restated in plain PyTorch on the CPU, in float32, one function per mechanism.

Nothing here is shared with the package: the functions take a config.json as a dict and the
checkpoint tensors by name (any dtype; they are widened to float32), run a whole sequence at once
with full T x T score matrices and explicit loops, and return the logits of every position.

Notation: T tokens, width W; per attention layer H query heads, G key/value heads, key width D, value
width Dv; R rotated values per head; window n, kept first positions f; E real experts, I identity
experts, k chosen per token.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import torch


PRECISION = torch.float32      # the tests set float64: the same equations, as a sharper reference


def f32(t: torch.Tensor) -> torch.Tensor:
    """The tensor on the CPU in the working precision (float32 unless PRECISION says otherwise)."""
    return t.detach().to("cpu", PRECISION)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def rotate_half_layout(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, D]: the first `dims` values of every head are rotated, value i with value
    i + dims/2 by the angle position * base^(-2i / dims); the rest passes unchanged."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims).to(torch.float32).to(PRECISION)
    ang = positions.to(PRECISION)[:, None] * freq[None, :]             # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visible(T: int, window: Optional[int], keep_first: int, start: int = 0) -> torch.Tensor:
    """bool [T, T]: query i sees key j when j <= i and (i - j < window or j < keep_first)."""
    i = torch.arange(start, start + T)[:, None]
    j = torch.arange(start, start + T)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def sink_softmax(scores: torch.Tensor, mask: torch.Tensor, sink: Optional[torch.Tensor]) -> torch.Tensor:
    """scores [H, T, T]; weights exp(s_ij) / (sum over visible j of exp(s_ij) + exp(sink_h)): the sink adds
    one term to the denominator and nothing else."""
    s = scores.masked_fill(~mask[None], float("-inf"))
    m = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return e / den


def attention_keys_values(h: torch.Tensor, mixer: Mapping, w: Mapping[str, torch.Tensor], prefix: str, eps: float,
                          positions: torch.Tensor):
    """Keys (after the norm over the whole projection and rotation) [T, G, D] and values [T, G, Dv]."""
    G, D, Dv = mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    T = h.shape[0]
    k = rms_norm(h @ f32(w[prefix + "k"]).T, f32(w[prefix + "k.norm"]), eps).view(T, G, D)
    rot = mixer.get("rot")
    if rot:
        k = rotate_half_layout(k, positions, rot["dims"], rot["base"])
    v = (h @ f32(w[prefix + "v"]).T).view(T, G, Dv)
    return k, v


def attention_mixer(h: torch.Tensor, mixer: Mapping, w: Mapping[str, torch.Tensor], prefix: str, eps: float,
                    positions: torch.Tensor, kv) -> torch.Tensor:
    """Sliding-window grouped-query attention with kept first positions and a sink, on keys and values `kv`
    (this layer's own or an earlier layer's)."""
    H, G, D, Dv = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    T = h.shape[0]
    q = rms_norm(h @ f32(w[prefix + "q"]).T, f32(w[prefix + "q.norm"]), eps).view(T, H, D)
    rot = mixer.get("rot")
    if rot:
        q = rotate_half_layout(q, positions, rot["dims"], rot["base"])
    k, v = kv
    per = H // G
    kh = k.repeat_interleave(per, dim=1)            # query head h reads kv head h // per
    vh = v.repeat_interleave(per, dim=1)
    scores = torch.einsum("thd,shd->hts", q, kh) * float(mixer["scale"])
    mask_cfg = mixer.get("mask")
    mask = visible(T, mask_cfg["size"] if mask_cfg else None, (mask_cfg or {}).get("keep_first", 0))
    p = sink_softmax(scores, mask, f32(w[prefix + "sink"]) if (prefix + "sink") in w else None)
    o = torch.einsum("hts,shd->thd", p, vh).reshape(T, H * Dv)
    return o @ f32(w[prefix + "o"]).T


def dense_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str) -> torch.Tensor:
    g = h @ f32(w[prefix + "gate"]).T
    return ((g * torch.sigmoid(g)) * (h @ f32(w[prefix + "up"]).T)) @ f32(w[prefix + "down"]).T


def relu2_expert(h: torch.Tensor, w: Mapping[str, torch.Tensor], prefix: str) -> torch.Tensor:
    return torch.relu(h @ f32(w[prefix + "up"]).T).square() @ f32(w[prefix + "down"]).T


def route(h: torch.Tensor, router: Mapping, w: Mapping[str, torch.Tensor], prefix: str, margins: Optional[list] = None,
          forced: Optional[torch.Tensor] = None):
    """(chosen [T, k] expert indices, weights [T, k]).  `margins` collects, per token, how far the choice was
    from going another way (the gap between the last group or expert taken and the first one left).  Scores are the softmax over all E + I router outputs;
    the choice is made on score + correction, among the experts of the `keep` groups whose best such value
    is largest (all others count as minus infinity); the weights are the plain scores of the chosen."""
    z = h @ f32(w[prefix + "router"]).T
    s = torch.softmax(z, dim=-1)
    choice = s + f32(w[prefix + "correction"])[None, :]
    n = choice.shape[-1]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    best = choice.view(-1, count, n // count).max(dim=-1).values          # [T, count]
    kept = torch.zeros_like(best, dtype=torch.bool)
    kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
    allowed = kept.repeat_interleave(n // count, dim=1)
    choice = choice.masked_fill(~allowed, float("-inf"))
    chosen = choice.topk(router["top"], dim=-1).indices
    if margins is not None:
        gap = torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
        if keep < count:
            b = best.sort(dim=-1, descending=True).values
            gap = torch.minimum(gap, b[:, keep - 1] - b[:, keep])
        c = choice.sort(dim=-1, descending=True).values
        if router["top"] < n:
            gap = torch.minimum(gap, c[:, router["top"] - 1] - c[:, router["top"]])
        margins.append(gap)
    if forced is not None:          # the choice is given (a run in lower precision made it); the weights stay this run's scores
        chosen = forced.to(torch.long)
    return chosen, s.gather(1, chosen)


def moe_ff(h: torch.Tensor, mlp: Mapping, w: Mapping[str, torch.Tensor], prefix: str, margins: Optional[list] = None,
           forced: Optional[torch.Tensor] = None) -> torch.Tensor:
    router = mlp["router"]
    E, I = router["experts"], router.get("identity", 0)
    chosen, weights = route(h, router, w, prefix, margins, forced)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            y = h[t] if e >= E else relu2_expert(h[t:t + 1], w, f"{prefix}e{e}.")[0]
            out[t] += g * y
    assert E + I == w[prefix + "router"].shape[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ f32(w[prefix + "shared.sg"]).T)         # [T, 1]
        out = out + gate * relu2_expert(h, w, prefix + "shared.")
    return out


def forward(config: Mapping, w: Mapping[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None,
            margins: Optional[list] = None, forced: Optional[Mapping[int, torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence; `layers_out` collects the residual stream after every layer,
    `margins` the routers' margins (see `route`); `forced` gives, for layers by index, the experts every
    token takes ([T, k]) instead of the router's own choice."""
    eps = float(config["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    x = f32(w["embed"])[torch.tensor(tokens)] * float(config["embedding"]["scale"])
    kept: Dict[int, tuple] = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        mixer = layer["mixer"]
        h = rms_norm(x, f32(w[p + "norm1"]), eps)
        if mixer.get("kv_from") is not None:
            kv = kept[mixer["kv_from"]]
        else:
            kv = kept[i] = attention_keys_values(h, mixer, w, p + "mix.", eps, positions)
        x = x + rms_norm(attention_mixer(h, mixer, w, p + "mix.", eps, positions, kv), f32(w[p + "norm1b"]), eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, f32(w[p + "norm2"]), eps)
            y = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, mlp, w, p + "mlp.", margins, (forced or {}).get(i))
            x = x + rms_norm(y, f32(w[p + "norm2b"]), eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, f32(w["final.norm"]), eps) @ f32(w["head"]).T
