"""Small Tenetar configurations and model folders with random weights for the tests.

Sizes lie away from powers of two and from each other (key width != value width, heads != kv heads,
rotated part smaller than the head, widths that are no multiple of 8), windows and kept first positions
that do not line up with the pages of 64 (kept keys on one page and on two, windows shorter and longer
than a page), layers that read an earlier layer's keys and values under another window, dense and
routed feed-forwards (with and without groups, identity experts, a shared expert), a layer without a
feed-forward.  Weights are drawn here, not by the package's initialiser, so that sinks, corrections
and routers take values that matter.
"""
import json
import os
import tempfile

import numpy as np
import torch

import tenetar_plain as P

P.PRECISION = torch.float64      # the reference of the tests is the plain implementation in double precision


def attention(dim=20, heads=6, kv_heads=2, vdim=12, window=37, keep=3, rot=12, base=10000.0, scale=None, kv_from=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "scale": scale or 1.3 * dim ** -0.5}
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff=100):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, identity=2, top=3, groups=(4, 2), ff=40, shared=24):
    r = {"experts": experts, "identity": identity, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def config(layers, vocab=211, width=72, eps=1e-5, scale=3.5):
    return {"architecture": "Tenetar", "embedding": {"scale": scale}, "layers": layers, "norm": {"eps": eps}, "vocab": vocab,
            "width": width}


CONFIGS = {
    # own keys, a reader of them under a longer window with more kept keys, own keys again, a reader without a feed-forward
    "mixed": lambda: config([layer(attention(), dense()), layer(attention(window=50, keep=70, kv_from=0), moe()),
                             layer(attention(dim=16, heads=4, kv_heads=4, vdim=24, window=64, keep=1, rot=16), moe(groups=None, identity=0, top=2)),
                             layer(attention(dim=16, heads=8, kv_heads=4, vdim=24, window=9, keep=0, rot=16, kv_from=2), None)]),
    # widths that are multiples of 16, as served models have; one layer without a window, one without rotation
    "even": lambda: config([layer(attention(dim=32, heads=4, kv_heads=2, vdim=32, window=None, rot=32), moe(experts=6, identity=0, top=2, groups=(3, 1), ff=64, shared=64)),
                            layer(attention(dim=32, heads=4, kv_heads=2, vdim=32, window=130, keep=64, rot=None), dense(128)),
                            layer(attention(dim=32, heads=4, kv_heads=2, vdim=32, window=100, keep=5, rot=None, kv_from=1), moe(experts=4, identity=4, top=4, groups=(2, 2), ff=32, shared=None))],
                           vocab=256, width=128, scale=1.0),
    # many q heads on one kv head, wide values, one expert chosen
    "wide": lambda: config([layer(attention(dim=16, heads=20, kv_heads=1, vdim=80, window=70, keep=2, rot=8), moe(experts=5, identity=1, top=1, groups=(3, 2), ff=24, shared=8)),
                            layer(attention(dim=16, heads=20, kv_heads=1, vdim=80, window=20, keep=66, rot=8, kv_from=0), dense(64))],
                           vocab=97, width=64),
    # nothing a multiple of 8
    "odd": lambda: config([layer(attention(dim=10, heads=3, kv_heads=3, vdim=6, window=11, keep=2, rot=6), moe(experts=3, identity=3, top=2, groups=(3, 2), ff=50, shared=14)),
                           layer(attention(dim=10, heads=3, kv_heads=3, vdim=6, window=40, keep=13, rot=6, kv_from=0), dense(50))],
                          vocab=101, width=100),
    # sizes of a small served model: heads of 64 with half of each rotated, 16 + 4 experts in 4 groups, 6 chosen
    "served": lambda: config([layer(attention(dim=64, heads=8, kv_heads=2, vdim=64, window=128, keep=8, rot=32, base=500000.0), dense(512)),
                              layer(attention(dim=64, heads=8, kv_heads=2, vdim=64, window=128, keep=8, rot=32, base=500000.0), moe(experts=16, identity=4, top=6, groups=(4, 2), ff=128, shared=192)),
                              layer(attention(dim=64, heads=8, kv_heads=2, vdim=64, window=200, keep=0, rot=32, base=500000.0, kv_from=1), moe(experts=16, identity=4, top=6, groups=(4, 2), ff=128, shared=192)),
                              layer(attention(dim=128, heads=4, kv_heads=4, vdim=128, window=96, keep=65, rot=128), moe(experts=4, identity=0, top=1, groups=None, ff=256, shared=None))],
                             vocab=1000, width=256, scale=16.0),
    "attention_only": lambda: config([layer(attention(window=9, keep=2), None)]),
    "dense_only": lambda: config([layer(attention(heads=2, kv_heads=1, dim=8, vdim=8, window=5, keep=1, rot=8), dense(160))]),
    "experts_only": lambda: config([layer(attention(heads=2, kv_heads=1, dim=8, vdim=8, window=None, rot=None), moe())]),
}

_folders = {}


def make_tensors(cfg: dict, seed: int, sharp: float = 1.0, router_scale: float = 6.0, spaced: float = 0.4):
    """Random tensors by name (float32 values that bfloat16 holds exactly).  `sharp` scales the query
    projections, which makes the softmax peaky: single keys then decide the output.  `router_scale`
    spreads the router's logits and `spaced` puts the corrections this far apart (in a random order, some
    negative; a score near 1 lands half way between two of them); spaced = 0 draws them at random.  Close
    calls between two choices are common either way: a float32 run follows the plain implementation through
    them, a bfloat16 run is compared under its own choices (`Choices`)."""
    g = torch.Generator().manual_seed(seed)

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * (s / i ** 0.5)).bfloat16().float()

    def vec(n, mean=1.0, s=0.1):
        return (mean + s * torch.randn(n, generator=g)).bfloat16().float()

    w, t = cfg["width"], {}
    t["embed"] = (torch.randn(cfg["vocab"], w, generator=g)).bfloat16().float()
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        for n in ("norm1", "norm1b"):
            t[p + n] = vec(w)
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        t[p + "mix.q"] = mat(H * d, w, sharp)
        t[p + "mix.q.norm"] = vec(H * d, s=0.3)
        if m.get("kv_from") is None:
            t[p + "mix.k"] = mat(G * d, w)
            t[p + "mix.v"] = mat(G * dv, w)
            t[p + "mix.k.norm"] = vec(G * d, mean=1.5 * sharp, s=0.3)
        t[p + "mix.sink"] = vec(H, mean=0.5, s=1.5)
        t[p + "mix.o"] = mat(w, H * dv)
        mlp = l.get("mlp")
        if mlp is None:
            continue
        for n in ("norm2", "norm2b"):
            t[p + n] = vec(w)
        if mlp["kind"] == "dense":
            t[p + "mlp.gate"] = mat(mlp["ff"], w, 1.2)
            t[p + "mlp.up"] = mat(mlp["ff"], w, 1.2)
            t[p + "mlp.down"] = mat(w, mlp["ff"])
        else:
            r = mlp["router"]
            n_out = r["experts"] + r.get("identity", 0)
            for e in range(r["experts"]):
                t[p + f"mlp.e{e}.up"] = mat(mlp["expert"]["ff"], w, 1.5)
                t[p + f"mlp.e{e}.down"] = mat(w, mlp["expert"]["ff"])
            t[p + "mlp.router"] = mat(n_out, w, router_scale)
            if spaced:
                t[p + "mlp.correction"] = ((torch.randperm(n_out, generator=g).float() - n_out / 2) * spaced).bfloat16().float()
            else:
                t[p + "mlp.correction"] = (0.4 * torch.randn(n_out, generator=g) - 0.1).bfloat16().float()
            if mlp.get("shared"):
                t[p + "mlp.shared.up"] = mat(mlp["shared"]["ff"], w, 1.5)
                t[p + "mlp.shared.down"] = mat(w, mlp["shared"]["ff"])
                t[p + "mlp.shared.sg"] = mat(1, w, 2.0)
    t["final.norm"] = vec(w)
    t["head"] = mat(cfg["vocab"], w)
    return t


def write_folder(cfg, tensors, prefix="x0ne_tnt_"):
    from x0ne_engine_b200.weights import write_file
    d = tempfile.mkdtemp(prefix=prefix)
    write_file(os.path.join(d, "model.safetensors"), {k: v.bfloat16() for k, v in tensors.items()})
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    return d


def folder(name: str, seed: int = 0, sharp: float = 1.0, soft: bool = False):
    """(folder, config, tensors) of a tiny model written once per (name, seed, sharp, soft).  soft: routers with
    ordinary logits and random corrections."""
    key = (name, seed, sharp, soft)
    if key not in _folders:
        cfg = CONFIGS[name]()
        tensors = make_tensors(cfg, seed, sharp, 6.0, 0.0) if soft else make_tensors(cfg, seed, sharp)
        _folders[key] = (write_folder(cfg, tensors, f"x0ne_tnt_{name}_"), cfg, tensors)
    return _folders[key]


def plain_logits(cfg, tensors, ids, layers_out=None, margins=None, forced=None):
    return P.forward(cfg, tensors, list(ids), layers_out, margins, forced).numpy()


class Choices:
    """Records what the routers of an engine choose, per layer and (slot, position), while it is active.  A
    bfloat16 run may take another expert than the plain implementation where two choices are within its
    rounding, and from there on the two would differ altogether; the tests give the plain implementation
    the engine's choices (`forced`) and check separately that the choices agree wherever they are clear.
    (The engine must launch its passes itself, `pass_graphs=False`: a replayed graph calls no Python.)"""

    def __init__(self, eng):
        self.eng = eng
        self.layers = [i for i, b in enumerate(eng.model.blocks) if type(getattr(b, "ffn", None)).__name__ == "RoutedExperts"]
        self.seen = {i: {} for i in self.layers}

    def __enter__(self):
        for i in self.layers:
            part = self.eng.model.blocks[i].ffn

            def forward(ctx, x, n_rows, _f=type(part).forward, _p=part, _i=i):
                out = _f(_p, ctx, x, n_rows)
                top = _p.top
                ch = ctx.ws.buffer("moe.chosen", (ctx.ws.max_rows, top), torch.int32)[:n_rows].cpu()
                slots, pos = ctx.row_slot[:n_rows].cpu().tolist(), ctx.row_pos[:n_rows].cpu().tolist()
                for r, (s, p) in enumerate(zip(slots, pos)):
                    if s >= 0:
                        self.seen[_i][(s, p)] = ch[r].clone()
                return out
            part.forward = forward
        return self

    def __exit__(self, *exc):
        for i in self.layers:
            del self.eng.model.blocks[i].ffn.forward

    def of(self, slot: int, n: int):
        """{layer: [n, k]} for positions 0..n-1 of the sequence that ran in `slot`."""
        return {i: torch.stack([self.seen[i][(slot, p)] for p in range(n)]) for i in self.layers}


def agreement(cfg, tensors, ids, forced, clear=0.25):
    """(fraction of (token, layer) whose engine choice equals the plain choice, the same among those where the
    plain margin is at least `clear`)."""
    layers = [i for i, l in enumerate(cfg["layers"]) if l.get("mlp") and l["mlp"]["kind"] == "moe"]
    same_all, same_clear, n_clear, n_all = 0, 0, 0, 0
    # the plain run follows the engine's choices, so that every router sees the inputs the engine's router saw
    hs = plain_router_inputs(cfg, tensors, ids, forced)
    for k, i in enumerate(layers):
        mlp = cfg["layers"][i]["mlp"]
        m = []
        chosen, _ = P.route(hs[i], mlp["router"], tensors, f"l{i}.mlp.", m)
        eq = (chosen.sort(-1).values == forced[i].to(torch.long).sort(-1).values).all(-1)
        ok = m[0] >= clear
        same_all += int(eq.sum()); n_all += eq.numel()
        same_clear += int((eq & ok).sum()); n_clear += int(ok.sum())
    return same_all / max(n_all, 1), same_clear / max(n_clear, 1)


def plain_router_inputs(cfg, tensors, ids, forced):
    """{layer: the normed rows its feed-forward reads} of the plain run that follows `forced`."""
    out, eps = {}, float(cfg["norm"]["eps"])
    layers_out = []
    P.forward(cfg, tensors, list(ids), layers_out, None, forced)
    # the input of layer i's feed-forward is the residual after its mixer: recomputed from the residual
    # before the layer by running the layer's mixer part again
    x = P.f32(tensors["embed"])[torch.tensor(list(ids))] * float(cfg["embedding"]["scale"])
    positions = torch.arange(len(ids))
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, mixer = f"l{i}.", layer["mixer"]
        h = P.rms_norm(x, P.f32(tensors[p + "norm1"]), eps)
        if mixer.get("kv_from") is not None:
            kv = kept[mixer["kv_from"]]
        else:
            kv = kept[i] = P.attention_keys_values(h, mixer, tensors, p + "mix.", eps, positions)
        x_mid = x + P.rms_norm(P.attention_mixer(h, mixer, tensors, p + "mix.", eps, positions, kv), P.f32(tensors[p + "norm1b"]), eps)
        if layer.get("mlp") is not None:
            out[i] = P.rms_norm(x_mid, P.f32(tensors[p + "norm2"]), eps)
        x = layers_out[i]
    return out


def clear_ids(cfg, tensors, n, seed=0, margin=0.0):
    """n token ids (drawn from `seed`, then seed + 1000, ...) for which no router of the model comes closer
    than `margin` to another choice, by the plain implementation: rounding to bfloat16 then cannot flip one."""
    for k in range(200):
        ids = [int(t) for t in np.random.default_rng(seed + 1000 * k).integers(0, cfg["vocab"], n)]
        if margin <= 0:
            return ids
        m = []
        P.forward(cfg, tensors, ids, None, m)
        if not m or min(float(x.min()) for x in m) >= margin:
            return ids
    raise AssertionError("no token sequence with clear routing found")


def plain_greedy(cfg, tensors, prompt, n_new):
    ids, out = list(prompt), []
    for _ in range(n_new):
        t = int(P.forward(cfg, tensors, ids)[-1].argmax())
        out.append(t)
        ids.append(t)
    return out
