"""Tenetar: the typed configuration, read strictly from config.json, and its ModelSpec.

A Tenetar model scales its token embedding by a constant and runs a list of layers, each
`x += norm1b(mixer(norm1(x)))` then (unless the layer has no feed-forward)
`x += norm2b(ff(norm2(x)))`, all four RMS norms with weights of their own.  The mixer is
grouped-query attention over a sliding window that also keeps the sequence's first positions
visible, with queries and keys normed over their whole projection, rotate-half rotary positions on
the first `rot.dims` values of each head, a scale from the configuration, and a learned per-head sink
in the softmax denominator; a layer may have no keys and values of its own and read an earlier
layer's (`kv_from`).  The feed-forward is a dense SiLU-gated unit or a mixture of squared-ReLU
experts with a grouped, bias-corrected choice, identity experts and a gated shared expert.

Every size and constant comes from config.json (`embedding.scale`, `layers[i].mixer`,
`layers[i].mlp`, `norm.eps`, `vocab`, `width`); the layer list may have any order and length.
Tensor names: `embed`, `l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Mapping, Optional, Tuple

from .rovurax import UNBOUNDED_POSITIONS, _get, _num, _only, _pint, _plain
from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

ARCHITECTURE = "Tenetar"
MODEL_TYPE = "tenetar"


def _nonneg(d, key, where, default=0) -> int:
    v = d.get(key, default) if isinstance(d, Mapping) else default
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"config.json: {where}.{key} is not a non-negative integer")
    return v


@dataclass(frozen=True)
class TenetarLayer:
    type: str                       # "attention"
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]


@dataclass(frozen=True)
class TenetarConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[TenetarLayer, ...]
    dtype: str = "bfloat16"
    eos_token_ids: tuple = ()
    max_position_embeddings: int = UNBOUNDED_POSITIONS
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    # ---- reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "TenetarConfig":
        if not isinstance(d, Mapping):
            raise ConfigError("config.json: not a JSON object")
        norm = _get(d, "norm", "the model")
        _only(norm, ("eps",), "norm")
        emb = d.get("embedding") or {}
        _only(emb, ("scale",), "embedding")
        scale = _num(emb, "scale", "embedding") if "scale" in emb else 1.0
        raw_layers = _get(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: layers is not a list of at least one layer")
        layers: List[TenetarLayer] = []
        for i, l in enumerate(raw_layers):
            where = f"layers[{i}]"
            _only(l, ("type", "mixer", "mlp"), where)
            kind = _get(l, "type", where)
            if kind != "attention":
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this architecture")
            mixer = _get(l, "mixer", where)
            mw = where + ".mixer"
            _only(mixer, ("dim", "heads", "kv_heads", "kv_from", "mask", "rot", "scale", "vdim"), mw)
            for k in ("dim", "heads", "kv_heads", "vdim"):
                _pint(mixer, k, mw)
            _num(mixer, "scale", mw)
            if mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(f"config.json: {mw}: heads are not a multiple of kv_heads")
            if mixer.get("mask") is not None:
                _only(mixer["mask"], ("size", "keep_first"), mw + ".mask")
                _pint(mixer["mask"], "size", mw + ".mask")
                _nonneg(mixer["mask"], "keep_first", mw + ".mask")
            if mixer.get("rot") is not None:
                rot = mixer["rot"]
                _only(rot, ("base", "dims"), mw + ".rot")
                _num(rot, "base", mw + ".rot")
                if _pint(rot, "dims", mw + ".rot") % 2 or rot["dims"] > mixer["dim"]:
                    raise ConfigError(f"config.json: {mw}.rot.dims must be even and at most dim")
            src = mixer.get("kv_from")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                    raise ConfigError(f"config.json: {mw}.kv_from must name an earlier layer")
                other = layers[src].mixer
                if other.get("kv_from") is not None:
                    raise ConfigError(f"config.json: {mw}.kv_from names layer {src}, which has no keys and values of its own")
                for k in ("kv_heads", "dim", "vdim"):
                    if other[k] != mixer[k]:
                        raise ConfigError(f"config.json: {mw}.kv_from names layer {src}, whose {k} {other[k]} differs from {mixer[k]}")
                if _plain(other.get("rot")) != _plain(mixer.get("rot")):
                    raise ConfigError(f"config.json: {mw}.kv_from names layer {src}, whose rotation differs")
            mlp = l.get("mlp")
            if mlp is not None:
                cls._check_mlp(mlp, where + ".mlp")
            layers.append(TenetarLayer(kind, mixer, mlp))
        dtype = d.get("dtype") or "bfloat16"
        if dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"config.json: dtype {dtype!r}; bfloat16 and float32 checkpoints are served")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab=_pint(d, "vocab", "the model"), width=_pint(d, "width", "the model"),
                   norm_eps=_num(norm, "eps", "norm"), embedding_scale=scale, layers=tuple(layers), dtype=dtype,
                   eos_token_ids=eos_ids, raw=dict(d))

    @staticmethod
    def _check_mlp(mlp: Mapping[str, Any], where: str) -> None:
        kind = _get(mlp, "kind", where)
        if kind == "dense":
            _only(mlp, ("ff", "kind"), where)
            _pint(mlp, "ff", where)
            return
        if kind != "moe":
            raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this architecture")
        _only(mlp, ("kind", "expert", "router", "shared"), where)
        expert = _get(mlp, "expert", where)
        _only(expert, ("ff",), where + ".expert")
        _pint(expert, "ff", where + ".expert")
        router = _get(mlp, "router", where)
        rw = where + ".router"
        _only(router, ("experts", "groups", "identity", "top"), rw)
        n = _pint(router, "experts", rw) + _nonneg(router, "identity", rw)
        top = _pint(router, "top", rw)
        count, keep = 1, 1
        if router.get("groups") is not None:
            _only(router["groups"], ("count", "keep"), rw + ".groups")
            count, keep = _pint(router["groups"], "count", rw + ".groups"), _pint(router["groups"], "keep", rw + ".groups")
        if n % count or keep > count or top > keep * (n // count):
            raise ConfigError(f"config.json: {rw}: {n} outputs in {count} groups of which {keep} stay cannot give {top} choices")
        if mlp.get("shared") is not None:
            _only(mlp["shared"], ("ff",), where + ".shared")
            _pint(mlp["shared"], "ff", where + ".shared")

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": {"scale": self.embedding_scale},
             "layers": [{"type": l.type, "mixer": _plain(l.mixer), "mlp": _plain(l.mlp)} for l in self.layers]}
        if self.dtype != "bfloat16":
            d["dtype"] = self.dtype
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- the model as data
    def to_spec(self) -> ModelSpec:
        w, eps = self.width, self.norm_eps

        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", dict(size=w, eps=eps, names=dict(weight=name)))

        positions, layers, order = {}, [], []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}", l.mixer
            pos_name = None
            if m.get("rot") is not None:
                rot = m["rot"]
                pos_name = f"rot.{rot['dims']}.{float(rot['base'])!r}.{m['dim']}"       # layers with one rotation share its table
                positions.setdefault(pos_name, PartSpec("rope", dict(
                    head_dim=m["dim"], rotary_dim=rot["dims"], theta=float(rot["base"]), freq_in_double=True)))
            mask = m.get("mask") or {}
            own = m.get("kv_from") is None
            names = dict(q=f"{p}.mix.q", q_norm=f"{p}.mix.q.norm", sink=f"{p}.mix.sink", o=f"{p}.mix.o")
            if own:
                names.update(k=f"{p}.mix.k", v=f"{p}.mix.v", k_norm=f"{p}.mix.k.norm")
            parts = dict(
                mixer_norm=norm(f"{p}.norm1"),
                mixer=PartSpec("sink_window_attention", dict(
                    hidden_size=w, q_heads=m["heads"], kv_heads=m["kv_heads"], head_dim=m["dim"], v_dim=m["vdim"],
                    scale=float(m["scale"]), window=mask.get("size"), keep_first=mask.get("keep_first", 0), sink=True,
                    qk_norm_eps=eps, position=pos_name, own_kv=own, names=names)),
                mixer_post_norm=norm(f"{p}.norm1b"))
            if l.mlp is not None:
                parts["ffn_norm"] = norm(f"{p}.norm2")
                parts["ffn_post_norm"] = norm(f"{p}.norm2b")
                if l.mlp["kind"] == "dense":
                    parts["ffn"] = PartSpec("swiglu", dict(
                        hidden_size=w, intermediate_size=l.mlp["ff"],
                        names=dict(gate=f"{p}.mlp.gate", up=f"{p}.mlp.up", down=f"{p}.mlp.down")))
                else:
                    r, shared = l.mlp["router"], l.mlp.get("shared")
                    groups = r.get("groups") or {}
                    parts["ffn"] = PartSpec("routed_experts", dict(
                        hidden_size=w, experts=r["experts"], identity=r.get("identity", 0), top=r["top"],
                        groups=groups.get("count", 1), keep_groups=groups.get("keep", groups.get("count", 1)),
                        expert_size=l.mlp["expert"]["ff"], activation="relu2",
                        shared_size=shared["ff"] if shared else None, shared_gate=bool(shared),
                        names=dict(router=f"{p}.mlp.router", correction=f"{p}.mlp.correction", up=f"{p}.mlp.e{{e}}.up",
                                   down=f"{p}.mlp.e{{e}}.down", shared_up=f"{p}.mlp.shared.up",
                                   shared_down=f"{p}.mlp.shared.down", shared_gate=f"{p}.mlp.shared.sg")))
            layers.append(LayerSpec(block="sandwich", parts=parts))
            order.append(RunEntry(i, reads_cache_of=m.get("kv_from")))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=w,
            max_position_embeddings=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", dict(vocab_size=self.vocab, hidden_size=w, scale=self.embedding_scale,
                                                       names=dict(weight="embed"))),
            positions=positions, layers=tuple(layers), run_order=tuple(order),
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", dict(vocab_size=self.vocab, hidden_size=w, tied=False, names=dict(weight="head"))),
            stop_token_ids=tuple(self.eos_token_ids), checkpoint_dtype=self.dtype)
        spec.validate()
        return spec
