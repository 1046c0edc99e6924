"""Small Rovurax configurations and model folders with random weights for the tests.

The sizes are chosen away from powers of two and from each other (key width != value width, heads !=
kv heads, widths that are no multiple of 8 or 16), with chunks and pages that do not line up, layers
without a feed-forward, attention layers that blend their values and ones that do not, and a latent
layer before the first attention layer.  Weights are drawn here (not by the package's initialiser), so
that blends, sinks and gates take values that matter.
"""
import json
import os
import tempfile

import torch

import rovurax_plain as R


def attention_layer(dim=20, heads=6, kv_heads=2, vdim=12, chunk=37, v_mix=True, ff=100, limit=1.5, scale=None):
    mixer = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "scale": scale or dim ** -0.5}
    if chunk:
        mixer["mask"] = {"size": chunk}
    if v_mix:
        mixer["v_mix"] = True
    return {"type": "attention", "mixer": mixer, "mlp": {"ff": ff, "kind": "dense", "limit": limit} if ff else None}


def latent_layer(dim=24, heads=3, rot_dim=6, vdim=20, kv_rank=40, base=10000.0, scaling="yarn", ff=100, limit=2.5, scale=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling == "yarn":
        rot["scaling"] = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}
    elif scaling:
        rot["scaling"] = scaling
    mixer = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "rot": rot, "rot_dim": rot_dim, "vdim": vdim,
             "scale": scale or (dim + rot_dim) ** -0.5}
    return {"type": "latent_attention", "mixer": mixer, "mlp": {"ff": ff, "kind": "dense", "limit": limit} if ff else None}


def config(layers, vocab=211, width=72, eps=1e-5):
    return {"architecture": "Rovurax", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


CONFIGS = {
    # a latent layer first, then the source of the blended values, a layer that does not blend, one that does
    "mixed": lambda: config([latent_layer(), attention_layer(), attention_layer(v_mix=False, chunk=50, ff=0),
                             attention_layer(chunk=64), latent_layer(scaling=None, ff=0, heads=5, kv_rank=24, vdim=8)]),
    # widths that are multiples of 16, as served models have; one q head per kv head; no chunks in one layer
    "even": lambda: config([attention_layer(dim=32, heads=4, kv_heads=4, vdim=48, chunk=None, ff=128),
                            latent_layer(dim=32, heads=4, rot_dim=16, vdim=32, kv_rank=64, ff=128),
                            attention_layer(dim=32, heads=4, kv_heads=4, vdim=48, chunk=130, ff=128)], vocab=256, width=128),
    # many q heads on one kv head (more than one MMA tile of heads in decoding), wide values
    "wide": lambda: config([attention_layer(dim=16, heads=20, kv_heads=1, vdim=80, chunk=70, ff=64),
                            latent_layer(dim=8, heads=18, rot_dim=4, vdim=16, kv_rank=136, ff=0)], vocab=97, width=64),
    # nothing a multiple of 8: width, key and value widths, rank, feed-forward, vocabulary
    "odd": lambda: config([attention_layer(dim=10, heads=3, kv_heads=3, vdim=6, chunk=11, ff=50),
                           latent_layer(dim=10, heads=2, rot_dim=6, vdim=14, kv_rank=22, ff=50),
                           attention_layer(dim=10, heads=3, kv_heads=3, vdim=6, chunk=40, ff=0)], vocab=101, width=100),
    "attention_only": lambda: config([attention_layer(ff=0, v_mix=False, chunk=9)]),
    "latent_only": lambda: config([latent_layer(ff=0)]),
    "ffn_heavy": lambda: config([attention_layer(heads=2, kv_heads=1, dim=8, vdim=8, chunk=5, ff=160, limit=0.3)]),
}

_folders = {}


def make_tensors(cfg: dict, seed: int, sharp: float = 1.0):
    """Random tensors by name (float32 values that bfloat16 holds exactly).  `sharp` scales the query
    projections, which makes the softmax peaky: single keys then decide the output."""
    g = torch.Generator().manual_seed(seed)

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * (s / i ** 0.5)).bfloat16().float()

    def vec(n, mean=1.0, s=0.1):
        return (mean + s * torch.randn(n, generator=g)).bfloat16().float()

    w, t = cfg["width"], {}
    t["embed"] = (torch.randn(cfg["vocab"], w, generator=g)).bfloat16().float()
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        t[p + "norm1"] = vec(w)
        if layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[p + "mix.q"] = mat(H * d, w, 1.4 * sharp)
            t[p + "mix.k"] = mat(G * d, w, 1.4)
            t[p + "mix.v"] = mat(G * dv, w)
            t[p + "mix.o"] = mat(w, H * dv)
            if m.get("v_mix"):
                t[p + "mix.vmix"] = (0.25 + 0.5 * torch.rand((), generator=g)).bfloat16().float()
        else:
            H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            t[p + "mix.q"] = mat(H * (d + r), w, 1.4 * sharp)
            t[p + "mix.dkv"] = mat(rank + r, w, 1.4)
            t[p + "mix.dkv.norm"] = vec(rank)
            t[p + "mix.uk"] = mat(H * d, rank)
            t[p + "mix.uv"] = mat(H * dv, rank)
            t[p + "mix.sink"] = vec(H, mean=0.5, s=1.5)
            t[p + "mix.g"] = mat(H, w, 2.0)
            t[p + "mix.o"] = mat(w, H * dv)
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            t[p + "mlp.gate"] = mat(ff, w, 1.2)
            t[p + "mlp.up"] = mat(ff, w, 1.2)
            t[p + "mlp.down"] = mat(w, ff)
    t["final.norm"] = vec(w)
    t["head"] = mat(cfg["vocab"], w)
    return t


def folder(name: str, seed: int = 0, sharp: float = 1.0, cfg: dict = None):
    """(folder, config, tensors) of a tiny model written once per (name, seed, sharp)."""
    from x0ne_engine_b200.weights import write_file
    key = (name, seed, sharp)
    if key not in _folders:
        cfg = cfg or CONFIGS[name]()
        tensors = make_tensors(cfg, seed, sharp)
        d = tempfile.mkdtemp(prefix=f"x0ne_rvx_{name}_")
        write_file(os.path.join(d, "model.safetensors"), {k: v.bfloat16() for k, v in tensors.items()})
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        _folders[key] = (d, cfg, tensors)
    return _folders[key]


def plain_logits(cfg, tensors, ids, layers_out=None):
    return R.forward(cfg, tensors, list(ids), torch.float64, layers_out).numpy()


def plain_greedy(cfg, tensors, prompt, n_new):
    ids, out = list(prompt), []
    for _ in range(n_new):
        t = int(R.forward(cfg, tensors, ids, torch.float64)[-1].argmax())
        out.append(t)
        ids.append(t)
    return out
