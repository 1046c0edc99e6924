"""Rovurax on the GPU against the plain implementation (tests/rovurax_plain.py), in float32 and
bfloat16: every mechanism alone, whole prompts, token-by-token decoding, portions down to two tokens,
unequal batches with slots and pages used again, chunk and page borders in prompts and in decoding,
far keys, the first tokens, long decoding, odd sizes, and greedy generation through the entry point.
Kernel-level: the general bfloat16 attention kernels against the plain kernel on random caches."""
import numpy as np
import pytest
import torch

import rovurax_helpers as H
import rovurax_plain as R
from helpers import BF16_SELF_TOL, assert_close_bf16, assert_close_f32, first_difference

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
DEV = "cuda:0"
_engines = {}


def engine(name, dtype, seed=0, sharp=1.0, max_tokens=2048, **kw):
    from x0ne_engine_b200 import Engine
    key = (name, dtype, seed, sharp, max_tokens, tuple(sorted(kw.items())))
    if key not in _engines:
        folder, cfg, tensors = H.folder(name, seed, sharp)
        _engines[key] = (Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, max_seq_len=max_tokens, **kw), cfg, tensors)
    return _engines[key]


def check(dtype, got, want, what):
    (assert_close_f32 if dtype == "float32" else assert_close_bf16)(got, want, what)


def same_cut(dtype, got, base, what):
    got, base = np.asarray(got), np.asarray(base)
    if dtype == "float32":
        assert np.array_equal(got, base), f"{what}: first difference at {first_difference(got, base)}"
    else:
        err = np.max(np.abs(got - base) / (np.max(np.abs(base), axis=-1, keepdims=True) + 1e-30))
        assert err <= BF16_SELF_TOL, f"{what}: {err:.3e}"


def ids_for(cfg, n, seed=0):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]


def whole(eng, ids):
    s = eng.new_sequence()
    try:
        return eng.step([s], [ids], [list(range(len(ids)))]).cpu().numpy()
    finally:
        eng.free_sequence(s)


def in_pieces(eng, ids, cuts):
    """The prompt cut at `cuts` (piece sizes, the last piece takes the rest); logits of all places."""
    s = eng.new_sequence()
    out, at = [], 0
    try:
        for c in list(cuts) + [len(ids)]:
            piece = ids[at:at + c]
            if not piece:
                break
            out.append(eng.step([s], [piece], [list(range(len(piece)))]).cpu().numpy())
            at += len(piece)
    finally:
        eng.free_sequence(s)
    return np.concatenate(out)


# ------------------------------------------------------------------------------------------ row-wise kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clipped_gated_unit_kernel(dtype):
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(1)
    rows, inter, limit = 5, 37, 0.7
    gu = (torch.randn(rows, 2 * inter, generator=g) * 1.5).to(dtype).to(DEV)
    out = torch.empty((rows, inter), dtype=dtype, device=DEV)
    ops.glu_clipped(gu, out, rows, limit, 1.702, 1.0)
    x = gu.double().cpu()
    gate, up = x[:, :inter].clamp(max=limit), x[:, inter:].clamp(-limit, limit)
    want = gate * torch.sigmoid(1.702 * gate) * (up + 1.0)
    assert (x[:, :inter] > limit).any() and (x[:, inter:] < -limit).any()
    tol = 1e-6 if dtype == torch.float32 else 2 ** -8
    assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [72, 128, 1000])
def test_add_norm_with_two_branches(dtype, hidden):
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    rows, eps = 6, 1e-5
    resid = torch.randn(rows, hidden, generator=g).to(DEV)
    a, b = (torch.randn(rows, hidden, generator=g).to(dtype).to(DEV) for _ in range(2))
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(DEV)
    out = torch.empty((rows, hidden), dtype=dtype, device=DEV)
    before = resid.clone()
    ops.add_rmsnorm(resid, (a, b), w, out, rows, eps)
    want_r = before + (a.float() + b.float())
    assert torch.equal(resid, want_r)                          # float32 sum of the branches, one add into the residual
    want = R.rms_norm(want_r.double(), w.double(), eps)
    tol = 1e-6 if dtype == torch.float32 else 2 ** -8
    assert (out.double() - want).abs().max() <= tol * want.abs().max()


# ------------------------------------------------------------------------------------------ the model, whole
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths", [("attention_only", [1, 2, 9, 10, 40]), ("latent_only", [1, 3, 70]),
                                          ("ffn_heavy", [1, 12]), ("mixed", [1, 2, 37, 38, 65, 150]),
                                          ("even", [64, 131, 300]), ("wide", [5, 71, 141]), ("odd", [1, 12, 90])])
def test_each_request_alone_and_whole(name, lengths, dtype):
    eng, cfg, t = engine(name, dtype)
    for k, n in enumerate(lengths):
        ids = ids_for(cfg, n, seed=k)
        check(dtype, whole(eng, ids), H.plain_logits(cfg, t, ids), f"{name} len {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,n,tail", [("mixed", 120, 60), ("wide", 100, 40), ("even", 160, 40), ("odd", 70, 30)])
def test_prefill_against_token_by_token(name, n, tail, dtype):
    eng, cfg, t = engine(name, dtype)
    ids = ids_for(cfg, n, seed=5)
    base = whole(eng, ids)
    got = in_pieces(eng, ids, [n - tail] + [1] * tail)
    same_cut(dtype, got, base, f"{name}: last {tail} one by one")
    check(dtype, got, H.plain_logits(cfg, t, ids), f"{name} decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "even"])
def test_prompt_in_portions_down_to_two_tokens(name, dtype):
    eng, cfg, t = engine(name, dtype)
    ids = ids_for(cfg, 170, seed=6)
    base = whole(eng, ids)
    for cuts in ([2] * 30, [64, 64], [63, 2, 1, 64], [37, 37, 37, 37], [3, 125, 2], [129]):
        same_cut(dtype, in_pieces(eng, ids, cuts), base, f"{name} cut {cuts[:4]}")
    check(dtype, base, H.plain_logits(cfg, t, ids), name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_unequal_batches_against_each_alone_with_slots_used_again(name, dtype):
    eng, cfg, t = engine(name, dtype)
    for round_ in range(3):                      # the second and third rounds get slots and pages that were used
        lengths, steps = [[1, 30, 77, 140], [66, 2, 129], [140, 5]][round_], [3, 9, 1, 6]
        prompts = [ids_for(cfg, n, seed=10 * round_ + k) for k, n in enumerate(lengths)]
        tails = [ids_for(cfg, steps[k], seed=50 + k) for k in range(len(lengths))]
        slots = [eng.new_sequence() for _ in lengths]
        got = [[] for _ in lengths]
        first = eng.step(slots, prompts, [list(range(n)) for n in lengths]).cpu().numpy()
        at = 0
        for k, n in enumerate(lengths):
            got[k].append(first[at:at + n])
            at += n
        live = list(range(len(lengths)))
        for step in range(max(steps)):
            live = [k for k in live if step < steps[k]]         # the shorter requests end earlier
            out = eng.step([slots[k] for k in live], [[tails[k][step]] for k in live]).cpu().numpy()
            for j, k in enumerate(live):
                got[k].append(out[j:j + 1])
        for s in slots:
            eng.free_sequence(s)
        for k, n in enumerate(lengths):
            ids = prompts[k] + tails[k]
            alone = whole(eng, ids)
            same_cut(dtype, np.concatenate(got[k]), alone, f"{name} round {round_} request {k}")
            if round_ == 0:
                check(dtype, alone, H.plain_logits(cfg, t, ids), f"{name} request {k}")


# ------------------------------------------------------------------------------------------ edges, far keys
@pytest.mark.parametrize("dtype", DTYPES)
def test_chunk_and_page_borders_with_keys_that_decide(dtype):
    """Sharp queries make single keys decide a row, so a mask or a page that is one position off
    changes the logits by far more than the tolerance.  Chunks of 37, 50 and 64 positions against
    pages of 64: every position of a 260-token sequence is checked, in a prompt and decoded alone."""
    # (bfloat16 rounds the queries and keys themselves: with the sharpest scores that alone moves the
    # logits by a tenth, so the bfloat16 run keeps ordinary scores, under which the edges still decide)
    eng, cfg, t = engine("mixed", dtype, seed=3, sharp=4.0 if dtype == "float32" else 1.0)
    ids = ids_for(cfg, 260, seed=8)
    want = H.plain_logits(cfg, t, ids)
    # the test sees what it is for: moving a chunk's edge by one position changes the plain result
    shifted = {**cfg, "layers": [dict(l, mixer=dict(l["mixer"], mask={"size": l["mixer"]["mask"]["size"] + 1}))
                                 if l["type"] == "attention" and l["mixer"].get("mask") else l for l in cfg["layers"]]}
    moved = np.abs(H.plain_logits(shifted, t, ids) - want).max(-1) / np.abs(want).max(-1)
    assert (moved > 0.2).sum() > 100
    check(dtype, whole(eng, ids), want, "prompt")
    got = in_pieces(eng, ids, [30] + [1] * 230)
    check(dtype, got, want, "decoded across chunk and page borders")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_among_hundreds_and_the_sink(dtype):
    """One early token's key is made to dominate a late query of the latent layer: one query direction of
    head 0 and one latent direction are aligned with that token's embedding (the late token is the same
    token), so the late logits hang on a key hundreds of positions back, read in a prompt and in
    decoding.  The sinks are raised until they hold a good part of the denominators.  Without the key,
    and without the sinks, the plain result differs by more than the tolerance."""
    from x0ne_engine_b200 import Engine
    from x0ne_engine_b200.weights import write_file
    import json
    import os
    import tempfile
    cfg = H.config([H.latent_layer(ff=0, heads=4), H.attention_layer(chunk=None, v_mix=False, kv_heads=3)])
    t = H.make_tensors(cfg, seed=4)
    special = 7
    u = t["embed"][special] / t["embed"][special].norm()
    t["l0.mix.q"][0] += 2.0 * u
    t["l0.mix.dkv"][0] += 2.0 * u
    t["l0.mix.uk"][0, 0] += 1.0
    t["l0.mix.uv"] *= 4.0
    t["l0.mix.sink"] += 8.0
    t = {k: v.bfloat16().float() for k, v in t.items()}
    d = tempfile.mkdtemp(prefix="x0ne_rvx_far_")
    write_file(os.path.join(d, "model.safetensors"), {k: v.bfloat16() for k, v in t.items()})
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    ids = [8 + x % (cfg["vocab"] - 8) for x in ids_for(cfg, 700, seed=9)]
    ids[130] = special
    ids[-1] = special
    want = H.plain_logits(cfg, t, ids)[-3:]
    other = list(ids)
    other[130] = 9
    assert np.abs(H.plain_logits(cfg, t, other)[-1] - want[-1]).max() > 0.07 * np.abs(want[-1]).max()
    no_sink = dict(t)
    no_sink["l0.mix.sink"] = t["l0.mix.sink"] - 40.0
    assert np.abs(H.plain_logits(cfg, no_sink, ids)[-1] - want[-1]).max() > 0.06 * np.abs(want[-1]).max()
    eng = Engine.from_folder(d, dtype=dtype, max_tokens=1024, max_seq_len=1024)
    check(dtype, whole(eng, ids)[-3:], want, "far key in a prompt")
    check(dtype, in_pieces(eng, ids, [697, 1, 1])[-3:], want, "far key decoded")


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(dtype):
    eng, cfg, t = engine("mixed", dtype)
    ids = ids_for(cfg, 6, seed=11)
    want = H.plain_logits(cfg, t, ids)
    check(dtype, in_pieces(eng, ids, [1, 1, 1, 1, 1]), want, "first tokens one by one")
    check(dtype, in_pieces(eng, ids, [2, 2]), want, "first tokens in twos")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    eng, cfg, t = engine("even", dtype)
    ids = ids_for(cfg, 420, seed=12)
    got = in_pieces(eng, ids, [20] + [1] * 400)
    check(dtype, got, H.plain_logits(cfg, t, ids), "400 decoded tokens")


# ------------------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", ["graph", "eager"])
def test_greedy_generation_through_the_entry_point(decode, dtype):
    from x0ne_engine_b200 import Model
    folder, cfg, t = H.folder("mixed")
    prompts = [ids_for(cfg, n, seed=20 + n) for n in (1, 7, 36, 64)]
    n_new = 14
    m = Model.from_folder(folder, dtype=dtype, max_batch=3, max_ctx=256, decode=decode)
    out = m.generate(prompts, max_tokens=n_new, stop_token_ids=())
    assert out.finish_reasons == ["length"] * len(prompts)
    for p, got in zip(prompts, out.tokens):
        if dtype == "float32":
            assert got == H.plain_greedy(cfg, t, p, n_new)
        else:
            ids = list(p)
            for tok in got:
                row = H.plain_logits(cfg, t, ids)[-1]
                top = np.sort(row)[-2:]
                if tok != int(np.argmax(row)):
                    assert top[1] - top[0] <= 2 * 0.05 * np.abs(row).max(), "a bfloat16 token left a clear argmax"
                    break
                ids.append(tok)
    assert m.generate(prompts, max_tokens=n_new, stop_token_ids=()).tokens == out.tokens


def test_random_model_from_a_configuration_generates():
    from x0ne_engine_b200 import Model
    from x0ne_engine_b200.config import config_from_dict
    m = Model.random(config_from_dict(H.CONFIGS["even"]()), seed=1, max_batch=2, max_ctx=128, norm_jitter=0.1)
    out = m.generate([[1, 2, 3], [4]], max_tokens=5, stop_token_ids=())
    assert [len(x) for x in out.tokens] == [5, 5] and all(0 <= x < 256 for row in out.tokens for x in row)


def test_short_prompt_passes_replayed_from_graphs_give_the_same_bits():
    eng, cfg, _ = engine("mixed", "bfloat16")
    base, _, _ = engine("mixed", "bfloat16", pass_graphs=False)
    assert eng.replayable and eng.pass_graphs and not base.pass_graphs
    before = eng.pass_graph_replays
    for k, lengths in enumerate([[100], [120], [70], [126], [20], [30], [5], [5], [100, 20], [90, 30], [100]]):
        prompts = [ids_for(cfg, n, seed=100 + 7 * k + j) for j, n in enumerate(lengths)]
        got = []
        for e in (eng, base):
            slots = [e.new_sequence() for _ in lengths]
            first = e.step(slots, prompts).cpu().numpy()
            nxt = e.step(slots, [[int(np.argmax(r))] for r in first]).cpu().numpy()
            for s in slots:
                e.free_sequence(s)
            got.append((first, nxt))
        assert np.array_equal(got[0][0], got[1][0]) and np.array_equal(got[0][1], got[1][1]), lengths
    assert eng.pass_graph_replays - before >= 4


# ------------------------------------------------------------------------------------------ attention kernels
def scattered_cache(kv_heads, dk, dv, n_slots, pages_per_slot, ring=None, seed=0):
    """A one-entry bfloat16 cache with random keys and values and a page table that scatters pages.
    dv None: values as wide as the keys; 0: no value plane."""
    from x0ne_engine_b200.csrc import ops
    vd = dk if dv is None else dv
    n_pages = n_slots * pages_per_slot + 3
    g = torch.Generator().manual_seed(seed)
    storage = (torch.randn(n_pages, kv_heads * 64 * (dk + vd), generator=g)).bfloat16().to(DEV)
    perm = torch.randperm(n_pages, generator=g)[:n_slots * pages_per_slot].reshape(n_slots, pages_per_slot)
    table = perm.to(torch.int32).to(DEV)
    view = ops.PagedCacheArg(storage.data_ptr(), table.data_ptr(), kv_heads * 64 * (dk + vd), pages_per_slot,
                             ring or pages_per_slot, 64, kv_heads, dk, n_pages, 0 if dv is None else (dv if dv > 0 else -1))
    return storage, table, view


def plain_kernel_in_float32(q, view_args, storage, table, slots, pos, q_heads, scale, window, extra_kw, vd_out):
    """The plain kernel on the same cache widened to float32 (same layout, same table)."""
    from x0ne_engine_b200.csrc import ops
    s32 = storage.float()
    v = ops.PagedCacheArg(s32.data_ptr(), table.data_ptr(), *view_args)
    kw = dict(extra_kw)
    if kw.get("gate") is not None:
        kw["gate"] = kw["gate"].float()
    q32 = q.float()
    out = torch.empty((q.shape[0], q_heads * vd_out), dtype=torch.float32, device=DEV)
    ops.attention_rows(q32, out, v, slots, pos, q.shape[0], q_heads, scale, window, ops.attn_extra(**kw))
    return out, (s32, q32, kw)


CASES = [  # q_heads, kv_heads, dk, dv, v_from_k, chunk, window, sink, gate
    (4, 2, 48, None, 0, 200, 0, False, False),
    (6, 1, 144, 0, 128, 0, 0, True, True),
    (6, 2, 20, 12, 0, 37, 0, False, False),
    (3, 3, 24, 40, 0, 0, 100, True, False),
    (20, 1, 16, 80, 0, 70, 0, False, True),
    (18, 1, 140, 0, 136, 0, 0, True, False),
    (5, 5, 72, 200, 0, 0, 0, False, False),
    (2, 1, 40, 0, 24, 64, 0, False, True),
]


@pytest.mark.parametrize("case", CASES)
def test_general_attention_kernels_against_the_plain_kernel(case):
    """Prefill tiles and decode rows of the tensor-core kernels against the plain kernel in float32 on
    the same scattered cache: unequal sequences, positions on page borders, several splits of a long row."""
    from x0ne_engine_b200.csrc import ops
    H_, G, dk, dv, vfk, chunk, window, sink, gate = case
    vd = vfk or (dk if dv is None else dv)
    pages = 12
    storage, table, view = scattered_cache(G, dk, dv, 3, pages, seed=dk)
    view_args = (view.page_stride, view.table_stride, view.ring_pages, 64, G, dk, view.n_pages, view.v_dim)
    assert ops.attention_flex_takes(view, torch.bfloat16, vfk, False) and ops.attention_flex_takes(view, torch.bfloat16, vfk, True)
    g = torch.Generator().manual_seed(5)
    scale = 1.7 * dk ** -0.5
    sink_t = (torch.randn(H_, generator=g) * 2).to(DEV) if sink else None
    # ---- prefill: three sequences bring 200, 1 and 67 rows at positions 130.., 63 and 0..
    seqs = [(0, 130, 200), (1, 63, 1), (2, 0, 67)]
    n_rows = sum(n for _, _, n in seqs)
    q = (torch.randn(n_rows, H_ * dk + 8, generator=g)).bfloat16().to(DEV)          # queries inside wider rows
    gate_t = torch.randn(n_rows, H_ + 3, generator=g).bfloat16().to(DEV) if gate else None
    slots = torch.tensor([s for s, _, n in seqs for _ in range(n)], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p0 + r for _, p0, n in seqs for r in range(n)], dtype=torch.int32, device=DEV)
    first, tiles = [0], []
    for k, (_, _, n) in enumerate(seqs):
        tiles += [(k, first[-1] + r0) for r0 in range(0, n, 128)]
        first.append(first[-1] + n)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    kw = dict(chunk=chunk, v_from_k=vfk, sink=sink_t, gate=gate_t, gate_ld=H_ + 3 if gate else 0, q_ld=H_ * dk + 8)
    out = torch.zeros((n_rows, H_ * vd), dtype=torch.bfloat16, device=DEV)
    ops.attention_flex_prefill(q, out, view, i32([t[0] for t in tiles]), i32([t[1] for t in tiles]), len(tiles), i32(first),
                               i32([s for s, _, _ in seqs]), i32([p for _, p, _ in seqs]), H_, scale, window, ops.attn_extra(**kw))
    want, keep = plain_kernel_in_float32(q, view_args, storage, table, slots, pos, H_, scale, window, kw, vd)
    err = (out.float() - want).abs().max().item()
    assert err <= 2 ** -7 * want.abs().max().item(), f"prefill {err}"
    # ---- decode: one row per sequence, at a page's last position, its first, and far out; 1, 3 and 7 splits
    rows = [(0, 63), (1, 64), (2, 64 * pages - 2)]
    q1 = (torch.randn(3, H_ * dk, generator=g)).bfloat16().to(DEV)
    gate1 = torch.randn(3, H_, generator=g).bfloat16().to(DEV) if gate else None
    kw1 = dict(chunk=chunk, v_from_k=vfk, sink=sink_t, gate=gate1, gate_ld=H_ if gate else 0)
    slots1, pos1 = i32([s for s, _ in rows]), i32([p for _, p in rows])
    want1, keep1 = plain_kernel_in_float32(q1, view_args, storage, table, slots1, pos1, H_, scale, window, kw1, vd)
    results = []
    for splits in (1, 3, 7):
        out1 = torch.zeros((3, H_ * vd), dtype=torch.bfloat16, device=DEV)
        scratch = torch.empty(ops.attention_flex_scratch_bytes(3, H_, G, vd, splits) // 4 + 1, dtype=torch.float32, device=DEV)
        ops.attention_flex_decode(q1, out1, view, slots1, pos1, 3, H_, scale, window, ops.attn_extra(**kw1), splits, scratch)
        err = (out1.float() - want1).abs().max().item()
        assert err <= 2 ** -7 * want1.abs().max().item(), f"decode, {splits} splits: {err}"
        results.append(out1.clone())
        ops.attention_flex_decode(q1, out1, view, slots1, pos1, 3, H_, scale, window, ops.attn_extra(**kw1), splits, scratch)
        assert torch.equal(out1, results[-1])                  # the same bits on every call


def test_attention_on_a_ring_that_has_lapped():
    """A windowed cache whose logical pages wrap: positions past the ring overwrite the oldest pages;
    the general kernels read the same keys as the plain kernel."""
    from x0ne_engine_b200.csrc import ops
    H_, G, dk, dv, window, ring = 4, 2, 24, 40, 100, 4
    storage, table, view = scattered_cache(G, dk, dv, 2, ring, ring=ring, seed=3)
    view_args = (view.page_stride, view.table_stride, ring, 64, G, dk, view.n_pages, view.v_dim)
    g = torch.Generator().manual_seed(6)
    q = torch.randn(2, H_ * dk, generator=g).bfloat16().to(DEV)
    slots = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    pos = torch.tensor([64 * 9 + 5, 64 * 6 + 63], dtype=torch.int32, device=DEV)     # both past the ring's 256 positions
    kw = {}
    want, _ = plain_kernel_in_float32(q, view_args, storage, table, slots, pos, H_, 0.3, window, kw, dv)
    out = torch.zeros((2, H_ * dv), dtype=torch.bfloat16, device=DEV)
    ops.attention_flex_decode(q, out, view, slots, pos, 2, H_, 0.3, window, ops.attn_extra(), 2,
                              torch.empty(ops.attention_flex_scratch_bytes(2, H_, G, dv, 2) // 4, dtype=torch.float32, device=DEV))
    assert (out.float() - want).abs().max() <= 2 ** -7 * want.abs().max()


@pytest.mark.parametrize("rows,inter,k", [(3, 96, 64), (8, 200, 72), (16, 256, 128), (40, 512, 256), (800, 384, 128)])
def test_clipped_unit_in_the_products_epilogues(rows, inter, k):
    """The gate|up product with the clipped unit in its epilogue (every kernel that takes the shape)
    against the product in float64 followed by the plain formula."""
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(rows)
    limit, slope, shift = 0.8, 1.702, 1.0
    x = torch.randn(rows, k, generator=g).bfloat16().to(DEV)
    w = (torch.randn(2 * inter, k, generator=g) * (2.0 / k ** 0.5)).bfloat16().to(DEV)
    gu = x.double() @ w.double().T
    gate, up = gu[:, :inter].clamp(max=limit), gu[:, inter:].clamp(-limit, limit)
    want = gate * torch.sigmoid(slope * gate) * (up + shift)
    assert (gu[:, :inter] > limit).any() and (gu[:, inter:].abs() > limit).any()
    ran = 0
    for name, takes, fn in [("smallm", ops.gemm_smallm_takes(w, rows, True), ops.gemm_bf16_smallm),
                            ("skinny", ops.gemm_skinny_tc_takes(w, rows), ops.gemm_bf16_skinny_tcgen05),
                            ("tc", ops.gemm_tc_takes(w, rows) and rows >= 128, ops.gemm_bf16_tcgen05)]:
        if not takes:
            continue
        y = torch.zeros((rows, inter), dtype=torch.bfloat16, device=DEV)
        fn(x, w, y, rows, swiglu=True, glu=(limit, slope, shift))
        ops.check_tc_status(torch.device(DEV))
        err = (y.double() - want).abs().max().item()
        assert err <= 2 ** -7 * want.abs().max().item(), f"{name}: {err}"
        ran += 1
    assert ran >= 1


def test_bfloat16_falls_back_to_the_plain_kernel_where_the_general_ones_do_not_take_a_shape(monkeypatch):
    """Values wider than the tensor-core kernels are compiled for go to the plain kernel, in bfloat16 too:
    forced here for every layer of a small model, prompts and decoding."""
    from x0ne_engine_b200 import Engine
    from x0ne_engine_b200.csrc import ops
    folder, cfg, t = H.folder("mixed")
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=512, max_seq_len=512)
    monkeypatch.setattr(ops, "attention_flex_takes", lambda *a, **k: False)
    ids = ids_for(cfg, 90, seed=31)
    want = H.plain_logits(cfg, t, ids)
    check("bfloat16", whole(eng, ids), want, "plain kernel, prompt")
    check("bfloat16", in_pieces(eng, ids, [70] + [1] * 20), want, "plain kernel, decoded")


def test_the_tile_height_the_engine_plans_with_is_the_kernels_own():
    from x0ne_engine_b200.csrc import ops
    assert ops.attention_prefill_tile_rows() == ops.PREFILL_TILE_ROWS
    assert int(ops._lib("flex").x0ne_attention_flex_tile_rows()) == ops.PREFILL_TILE_ROWS


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pass_rows", [64, 100])
def test_a_step_larger_than_one_pass(pass_rows, dtype):
    """A step of more rows than the engine's pass is cut wherever the pass ends, also inside a prompt: the
    later rows run from the cache the earlier pass left, and the blended values' source is that pass's own."""
    eng, cfg, t = engine("mixed", dtype, max_step_tokens=pass_rows)
    base, _, _ = engine("mixed", dtype)
    prompts = [ids_for(cfg, n, seed=40 + n) for n in (150, 31, 97)]
    slots = [eng.new_sequence() for _ in prompts]
    got = eng.step(slots, prompts, [list(range(len(p))) for p in prompts]).cpu().numpy()
    for s in slots:
        eng.free_sequence(s)
    at = 0
    for p in prompts:
        same_cut(dtype, got[at:at + len(p)], whole(base, p), f"passes of {pass_rows}")
        at += len(p)
    check(dtype, got[:150], H.plain_logits(cfg, t, prompts[0]), "first request")
