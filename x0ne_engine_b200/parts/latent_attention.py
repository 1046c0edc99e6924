"""Attention over a cached latent: one low-rank row per position from which every head's keys and
values are linear maps, plus a rotated key part that all heads share."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .attention import run_attention_ex
from .base import MIXERS, CacheNeed, Mixer
from .linear import Linear


class LatentAttention(Mixer):
    """Per position the cache keeps c = rmsnorm(W_c x) (`kv_rank` values, weight `dkv_norm`) and
    r = rot(W_r x) (`rot_dim` values, rotated by the model's position encoding), both rows of the one
    matrix `dkv`.  Head h has unrotated keys K_h c, values V_h c (`uk`, `uv` laid out head by head) and
    queries [q_h | rot(q'_h)] of head_dim + rot_dim values; a score is (q_h . K_h c + rot(q'_h) . r) x
    scale.  Because q_h . K_h c = (K_h^T q_h) . c, the queries are first carried into the latent space,
    every head then reads the same cache row of kv_rank + rot_dim values as its key and the first
    kv_rank of them as its value, and V_h is applied to the attention's result: the cache is never
    expanded per head.  Optional: a learned per-head sink that joins the softmax denominator
    (`names.sink`), and a per-head output gate sigmoid(G x)_h (`names.gate`) on the head's result.
    Causal over all keys.

    Parameters: hidden_size, heads, head_dim, rot_dim, v_dim, kv_rank, scale, norm_eps, position (name
    of a rotary position encoding of the model with rotary_dim == rot_dim and interleaved pairs), sink,
    gate (booleans), names.{q, dkv, dkv_norm, uk, uv, o, sink, gate}.
    """
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        g = spec.get
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.head_dim = int(spec["head_dim"])
        self.rot_dim = int(spec["rot_dim"])
        self.v_dim = int(spec["v_dim"])
        self.rank = int(spec["kv_rank"])
        self.scale = float(spec["scale"])
        self.eps = float(spec["norm_eps"])
        self.has_sink, self.has_gate = bool(g("sink")), bool(g("gate"))
        self.position = env.positions[spec["position"]]
        rot = self.position.rotary()
        if rot is None or rot[1] != self.rot_dim or getattr(self.position, "layout", None) != "interleaved":
            raise ValueError("latent attention needs a rotary encoding of rot_dim values with interleaved pairs")
        self.q_width = self.heads * (self.head_dim + self.rot_dim)
        self.proj_width = self.q_width + self.rank + self.rot_dim + (self.heads if self.has_gate else 0)
        self.proj = self.o = self.uk_t = self.uv = self.norm_w = self.sink = None

    @staticmethod
    def cache_need(spec: PartSpec) -> CacheNeed:
        return CacheNeed("kv", 1, int(spec["kv_rank"]) + int(spec["rot_dim"]), None, v_dim=0)

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        w, H, d, r = int(spec["hidden_size"]), int(spec["heads"]), int(spec["head_dim"]), int(spec["rot_dim"])
        vd, rank, n = int(spec["v_dim"]), int(spec["kv_rank"]), spec["names"]
        needs = [TensorNeed(n["q"], (H * (d + r), w)), TensorNeed(n["dkv"], (rank + r, w)),
                 TensorNeed(n["dkv_norm"], (rank,), role="vector", init="norm"),
                 TensorNeed(n["uk"], (H * d, rank)), TensorNeed(n["uv"], (H * vd, rank)), TensorNeed(n["o"], (w, H * vd))]
        if spec.get("sink"):
            needs.append(TensorNeed(n["sink"], (H,), role="vector", init="linear"))
        if spec.get("gate"):
            needs.append(TensorNeed(n["gate"], (H, w)))
        return needs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.spec["names"]
        packed = [tensors[n["q"]], tensors[n["dkv"]]] + ([tensors[n["gate"]]] if self.has_gate else [])
        self.proj = Linear(torch.cat(packed, dim=0).contiguous())
        self.o = Linear(tensors[n["o"]])
        # K_h^T as the [out, in] matrix of a product: [heads, kv_rank, head_dim]
        self.uk_t = tensors[n["uk"]].view(self.heads, self.head_dim, self.rank).transpose(1, 2).contiguous()
        self.uv = tensors[n["uv"]].view(self.heads, self.v_dim, self.rank).contiguous()
        self.norm_w = tensors[n["dkv_norm"]]
        self.sink = tensors[n["sink"]] if self.has_sink else None

    def weight_bytes(self) -> int:
        return self.proj.weight_bytes() + self.o.weight_bytes() + \
            (self.uk_t.numel() + self.uv.numel()) * self.uk_t.element_size()

    def forward(self, ctx, entry, x, n_rows, cache_entry=None, write_cache=True):
        dt, rows = self.env.dtype, ctx.ws.max_rows
        H, d, r, rank, vd = self.heads, self.head_dim, self.rot_dim, self.rank, self.v_dim
        proj = ctx.ws.buffer("lattn.proj", (rows, self.proj_width), dt)
        q_abs = ctx.ws.buffer("lattn.q_latent", (H * rows * rank,), dt)[:H * n_rows * rank].view(H, n_rows, rank)
        q_full = ctx.ws.buffer("lattn.q", (rows, H * (rank + r)), dt)
        o_lat = ctx.ws.buffer("lattn.o_latent", (rows, H * rank), dt)
        att = ctx.ws.buffer("lattn.out", (rows, H * vd), dt)
        out = ctx.ws.buffer("delta", (rows, self.hidden), dt)
        self.proj(x, proj, n_rows)
        # queries into the latent space, head by head: q_abs[h] = q[:, h, :head_dim] K_h
        q_un = proj[:n_rows, :self.q_width].view(n_rows, H, d + r)[:, :, :d].permute(1, 0, 2)
        ops.batched_product(q_un, self.uk_t, q_abs)
        view = ctx.cache.kv_view(entry if cache_entry is None else cache_entry)
        freq, _ = self.position.rotary()
        table = self.position.cos_sin_table(self.env.max_positions) if self.env.max_positions else None
        ops.latent_prepare(proj, self.q_width, q_abs, self.norm_w, self.eps, freq, float(self.position.mag), table, q_full,
                           H, d, r, rank, view, ctx.row_slot, ctx.row_pos, n_rows, write_cache)
        gate = proj[0, self.q_width + rank + r:] if self.has_gate else None
        extra = ops.attn_extra(v_from_k=rank, sink=self.sink, gate=gate, gate_ld=self.proj_width)
        run_attention_ex(ctx, q_full, o_lat, view, n_rows, H, self.scale, 0, extra)
        # back out of the latent space: head h's values are V_h (weights . c)
        ops.batched_product(o_lat[:n_rows].view(n_rows, H, rank).permute(1, 0, 2), self.uv,
                            att[:n_rows].view(n_rows, H, vd).permute(1, 0, 2))
        self.o(att, out, n_rows)
        return out


MIXERS.register("latent_attention", LatentAttention)
