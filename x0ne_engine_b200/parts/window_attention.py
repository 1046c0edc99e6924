"""Grouped-query attention over a sliding window with kept first positions and a sink, queries and
keys normed over their whole projection, keys and values of its own or of an earlier layer."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .attention import run_attention_ex
from .base import MIXERS, CacheNeed, Mixer
from .linear import Linear


class SinkWindowAttention(Mixer):
    """q, k, v from one product on the packed [q; k; v] weight.  Queries and keys are normed by RMS over
    the whole projection (all heads together, one learned weight per projected value, `qk_norm_eps`),
    then split into heads and rotated by the model's position encoding (`position`; the encoding's
    rotary_dim may be smaller than head_dim).  Keys (after norm and rotation) and values go to the
    cache.  The query at position i sees key j <= i when i - j < `window` or j < `keep_first`
    (`window` None: every j <= i); kept keys are read at their true positions.  Softmax over the
    visible scores q.k * scale, with exp(sink_h) added to the denominator of head h when `sink` is
    set.  q head h reads kv head h // (q_heads // kv_heads); keys of `head_dim`, values of `v_dim`.

    `own_kv` False: the layer has no key and value projections or key norm; the engine's run order
    names the entry whose cache it reads (`RunEntry.reads_cache_of`), and its queries meet those
    keys and values under its own mask, scale and sink.

    The cache keeps every position of a sequence (the kept first keys live in the same pages as the
    rest), so `window` bounds what a query reads, not what a sequence holds.

    Parameters: hidden_size, q_heads, kv_heads, head_dim, v_dim, scale, window, keep_first, sink,
    qk_norm_eps, position, own_kv, names.{q, k, v, o, q_norm, k_norm, sink}.
    """
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        g = spec.get
        self.hidden = int(spec["hidden_size"])
        self.q_heads = int(spec["q_heads"])
        self.kv_heads = int(spec["kv_heads"])
        self.head_dim = int(spec["head_dim"])
        self.v_dim = int(g("v_dim") or self.head_dim)
        if self.q_heads % self.kv_heads:
            raise ValueError("q heads are not a multiple of kv heads")
        self.scale = float(spec["scale"])
        self.window = int(g("window") or 0)
        self.keep_first = int(g("keep_first") or 0) if self.window else 0
        self.eps = float(spec["qk_norm_eps"])
        self.own_kv = bool(g("own_kv", True))
        self.has_sink = bool(g("sink"))
        pos = g("position")
        self.position = env.positions[pos] if pos is not None else None
        self.q_dim = self.q_heads * self.head_dim
        self.k_dim = self.kv_heads * self.head_dim
        self.kv_v_dim = self.kv_heads * self.v_dim
        self.width = self.q_dim + (self.k_dim + self.kv_v_dim if self.own_kv else 0)
        self.proj = self.o = self.q_norm = self.k_norm = self.sink = None

    @staticmethod
    def cache_need(spec: PartSpec) -> CacheNeed:
        hd = int(spec["head_dim"])
        vd = int(spec.get("v_dim") or hd)
        return CacheNeed("kv", int(spec["kv_heads"]), hd, None, v_dim=None if vd == hd else vd)

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        h, hd = int(spec["hidden_size"]), int(spec["head_dim"])
        vd, n = int(spec.get("v_dim") or hd), spec["names"]
        qh, kvh = int(spec["q_heads"]), int(spec["kv_heads"])
        needs = [TensorNeed(n["q"], (qh * hd, h)), TensorNeed(n["q_norm"], (qh * hd,), role="vector", init="norm")]
        if spec.get("own_kv", True):
            needs += [TensorNeed(n["k"], (kvh * hd, h)), TensorNeed(n["v"], (kvh * vd, h)),
                      TensorNeed(n["k_norm"], (kvh * hd,), role="vector", init="norm")]
        if spec.get("sink"):
            needs.append(TensorNeed(n["sink"], (qh,), role="vector", init="linear"))
        needs.append(TensorNeed(n["o"], (h, qh * vd)))
        return needs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.spec["names"]
        if self.own_kv:
            self.proj = Linear(torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous())
            self.k_norm = tensors[n["k_norm"]]
        else:
            self.proj = Linear(tensors[n["q"]])
        self.q_norm = tensors[n["q_norm"]]
        self.o = Linear(tensors[n["o"]])
        self.sink = tensors[n["sink"]] if self.has_sink else None

    def weight_bytes(self) -> int:
        return self.proj.weight_bytes() + self.o.weight_bytes()

    def forward(self, ctx, entry, x, n_rows, cache_entry=None, write_cache=True):
        if write_cache != self.own_kv:
            raise ValueError("a layer without key and value projections must read another entry's cache, and only such a layer may")
        dt, rows = self.env.dtype, ctx.ws.max_rows
        proj = ctx.ws.buffer("wattn.proj", (rows, self.width), dt)
        q = ctx.ws.buffer("wattn.q", (rows, self.q_dim), dt)
        att = ctx.ws.buffer("wattn.out", (rows, self.q_heads * self.v_dim), dt)
        out = ctx.ws.buffer("delta", (rows, self.hidden), dt)
        self.proj(x, proj, n_rows)
        view = ctx.cache.kv_view(entry if cache_entry is None else cache_entry)
        if view.kv_heads != self.kv_heads or view.head_dim != self.head_dim or view.value_dim != self.v_dim:
            raise ValueError("the cache this layer reads does not have its key and value heads")
        rot = self.position.rotary() if self.position is not None else None
        freq, rot_dim = rot if rot is not None else (None, 0)
        table = None
        if rot is not None and self.env.max_positions and hasattr(self.position, "cos_sin_table"):
            table = self.position.cos_sin_table(self.env.max_positions)
        ops.whole_norm_rope_kv_write(proj, self.q_dim, self.q_dim + self.k_dim, self.q_norm, self.k_norm, self.eps, freq,
                                     rot_dim, table, q, self.q_heads, view, ctx.row_slot, ctx.row_pos, n_rows, self.own_kv)
        extra = ops.attn_extra(sink=self.sink, keep_first=self.keep_first)
        run_attention_ex(ctx, q, att, view, n_rows, self.q_heads, self.scale, self.window, extra)
        self.o(att, out, n_rows)
        return out


MIXERS.register("sink_window_attention", SinkWindowAttention)
