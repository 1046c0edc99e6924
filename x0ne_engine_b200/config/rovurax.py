"""Rovurax: the typed configuration, read strictly from config.json, and its ModelSpec.

A Rovurax model is a list of layers, each with one norm whose output feeds a mixer and (unless the
layer has none) a feed-forward side by side; both results are added to the residual together.  The
mixer of a layer is one of

  * `attention`: grouped-query attention without positions, every query seeing the keys of its own
    chunk of `mask.size` positions only, with values optionally blended with the values the first
    such layer computed for the same token;
  * `latent_attention`: attention over one cached latent row per position (`kv_rank` values, from
    which every head's keys and values are linear maps) plus a rotated key part shared by all heads,
    interleaved rotary pairs with YaRN-scaled frequencies, a learned per-head sink in the softmax
    denominator, and a per-head sigmoid gate on the output.

Every size and constant comes from config.json (`layers[i].mixer`, `layers[i].mlp`, `norm.eps`,
`vocab`, `width`); the layer list may have any order and length.  Tensor names: `embed`,
`l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, List, Mapping, Optional, Tuple

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

ARCHITECTURE = "Rovurax"
MODEL_TYPE = "rovurax"

# config.json gives no longest sequence: positions are unbounded by the design, the cache bounds them
UNBOUNDED_POSITIONS = 1 << 24


def _get(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping) or key not in d:
        raise ConfigError(f"config.json: {where} has no {key!r}")
    return d[key]


def _pint(d, key, where) -> int:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} is not a positive integer")
    return v


def _num(d, key, where, positive=True) -> float:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or (positive and v <= 0):
        raise ConfigError(f"config.json: {where}.{key} is not a {'positive ' if positive else ''}number")
    return float(v)


def _only(d: Mapping[str, Any], known, where: str) -> None:
    extra = sorted(set(d) - set(known))
    if extra:
        raise ConfigError(f"config.json: {where} has keys this library does not know: {extra}")


@dataclass(frozen=True)
class RovuraxLayer:
    type: str                       # "attention" | "latent_attention"
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]


@dataclass(frozen=True)
class RovuraxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[RovuraxLayer, ...]
    dtype: str = "bfloat16"
    eos_token_ids: tuple = ()
    max_position_embeddings: int = UNBOUNDED_POSITIONS
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    # ---- reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RovuraxConfig":
        if not isinstance(d, Mapping):
            raise ConfigError("config.json: not a JSON object")
        norm = _get(d, "norm", "the model")
        _only(norm, ("eps",), "norm")
        layers: List[RovuraxLayer] = []
        raw_layers = _get(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: layers is not a list of at least one layer")
        for i, l in enumerate(raw_layers):
            where = f"layers[{i}]"
            _only(l, ("type", "mixer", "mlp"), where)
            kind = _get(l, "type", where)
            mixer = _get(l, "mixer", where)
            mw = where + ".mixer"
            if kind == "attention":
                _only(mixer, ("dim", "heads", "kv_heads", "mask", "scale", "v_mix", "vdim"), mw)
                for k in ("dim", "heads", "kv_heads", "vdim"):
                    _pint(mixer, k, mw)
                _num(mixer, "scale", mw)
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"config.json: {mw}: heads are not a multiple of kv_heads")
                if mixer.get("mask") is not None:
                    _only(mixer["mask"], ("size",), mw + ".mask")
                    _pint(mixer["mask"], "size", mw + ".mask")
                if not isinstance(mixer.get("v_mix", False), bool):
                    raise ConfigError(f"config.json: {mw}.v_mix is not a boolean")
            elif kind == "latent_attention":
                _only(mixer, ("dim", "heads", "kv_rank", "rot", "rot_dim", "scale", "vdim"), mw)
                for k in ("dim", "heads", "kv_rank", "rot_dim", "vdim"):
                    _pint(mixer, k, mw)
                _num(mixer, "scale", mw)
                rot = _get(mixer, "rot", mw)
                _only(rot, ("base", "dims", "scaling"), mw + ".rot")
                _num(rot, "base", mw + ".rot")
                if _pint(rot, "dims", mw + ".rot") != mixer["rot_dim"] or rot["dims"] % 2:
                    raise ConfigError(f"config.json: {mw}: rot.dims must be even and equal rot_dim")
                if rot.get("scaling") is not None:
                    sc = rot["scaling"]
                    _only(sc, ("factor", "original", "fast", "slow"), mw + ".rot.scaling")
                    for k in ("factor", "original", "fast", "slow"):
                        _num(sc, k, mw + ".rot.scaling")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this architecture")
            mlp = l.get("mlp")
            if mlp is not None:
                _only(mlp, ("ff", "kind", "limit"), where + ".mlp")
                if _get(mlp, "kind", where + ".mlp") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not implemented")
                _pint(mlp, "ff", where + ".mlp")
                _num(mlp, "limit", where + ".mlp")
            layers.append(RovuraxLayer(kind, mixer, mlp))
        dtype = d.get("dtype") or "bfloat16"
        if dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"config.json: dtype {dtype!r}; bfloat16 and float32 checkpoints are served")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        c = cls(vocab=_pint(d, "vocab", "the model"), width=_pint(d, "width", "the model"),
                norm_eps=_num(norm, "eps", "norm"), layers=tuple(layers), dtype=dtype, eos_token_ids=eos_ids,
                raw=dict(d))
        c.check()
        return c

    def check(self) -> None:
        first = None
        for i, l in enumerate(self.layers):
            if l.type == "attention" and l.mixer.get("v_mix"):
                kv = (l.mixer["kv_heads"], l.mixer["vdim"])
                if first is None:
                    first = kv
                elif kv != first:
                    raise ConfigError(f"config.json: layers[{i}] blends its values with the first such layer's, "
                                      f"whose kv_heads x vdim {first} differ from its {kv}")

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": [{"type": l.type, "mixer": _plain(l.mixer), "mlp": _plain(l.mlp)} for l in self.layers]}
        if self.dtype != "bfloat16":
            d["dtype"] = self.dtype
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- the model as data
    def to_spec(self) -> ModelSpec:
        w, eps = self.width, self.norm_eps
        positions = {}
        layers = []
        seen_mix = False
        for i, l in enumerate(self.layers):
            p, m = f"l{i}", l.mixer
            if l.type == "attention":
                role = None
                if m.get("v_mix"):
                    role = "blend" if seen_mix else "source"
                    seen_mix = True
                names = dict(q=f"{p}.mix.q", k=f"{p}.mix.k", v=f"{p}.mix.v", o=f"{p}.mix.o")
                if role is not None:
                    names["v_blend"] = f"{p}.mix.vmix"
                mixer = PartSpec("masked_attention", dict(
                    hidden_size=w, q_heads=m["heads"], kv_heads=m["kv_heads"], head_dim=m["dim"], v_dim=m["vdim"],
                    scale=float(m["scale"]), chunk=(m.get("mask") or {}).get("size"), window=None, v_blend=role,
                    position=None, names=names))
            else:
                rot = m["rot"]
                pos_name = f"{p}.rot"
                positions[pos_name] = PartSpec("yarn_rope", dict(
                    rotary_dim=rot["dims"], theta=float(rot["base"]), scaling=_plain(rot.get("scaling")),
                    layout="interleaved"))
                mixer = PartSpec("latent_attention", dict(
                    hidden_size=w, heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_dim=m["vdim"],
                    kv_rank=m["kv_rank"], scale=float(m["scale"]), norm_eps=eps, position=pos_name, sink=True, gate=True,
                    names=dict(q=f"{p}.mix.q", dkv=f"{p}.mix.dkv", dkv_norm=f"{p}.mix.dkv.norm", uk=f"{p}.mix.uk",
                               uv=f"{p}.mix.uv", sink=f"{p}.mix.sink", gate=f"{p}.mix.g", o=f"{p}.mix.o")))
            parts = dict(norm=PartSpec("rmsnorm", dict(size=w, eps=eps, names=dict(weight=f"{p}.norm1"))), mixer=mixer)
            if l.mlp is not None:
                parts["ffn"] = PartSpec("clipped_glu", dict(
                    hidden_size=w, intermediate_size=l.mlp["ff"], limit=float(l.mlp["limit"]), slope=1.702, shift=1.0,
                    names=dict(gate=f"{p}.mlp.gate", up=f"{p}.mlp.up", down=f"{p}.mlp.down")))
            layers.append(LayerSpec(block="parallel", parts=parts))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=w,
            max_position_embeddings=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", dict(vocab_size=self.vocab, hidden_size=w, names=dict(weight="embed"))),
            positions=positions, layers=tuple(layers), run_order=tuple(RunEntry(i) for i in range(len(layers))),
            final_norm=PartSpec("rmsnorm", dict(size=w, eps=eps, names=dict(weight="final.norm"))),
            head=PartSpec("lm_head", dict(vocab_size=self.vocab, hidden_size=w, tied=False, names=dict(weight="head"))),
            stop_token_ids=tuple(self.eos_token_ids), checkpoint_dtype=self.dtype)
        spec.validate()
        return spec


def _plain(x):
    if isinstance(x, Mapping):
        return {k: _plain(v) for k, v in x.items()}
    return x
