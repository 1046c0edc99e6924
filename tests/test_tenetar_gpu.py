"""Tenetar on the GPU against the plain implementation (tests/tenetar_plain.py), in float32 and bfloat16:
every mechanism alone, whole prompts, token-by-token decoding, portions down to two tokens, unequal
batches with slots and pages used again, the window's edge and the kept first keys in prompts and in
decoding, far keys, the sink, the first tokens, long decoding, odd sizes, routing with and without groups,
identity experts and a shared expert, and greedy generation through the entry point.  Token sequences
are drawn so that no router is within rounding of another choice (the margin is checked by the plain
implementation), since a choice that flips changes a row altogether."""
import numpy as np
import pytest
import torch

import tenetar_helpers as H
import tenetar_plain as P
from helpers import BF16_SELF_TOL, assert_close_bf16, assert_close_f32, first_difference

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
DEV = "cuda:0"
MARGIN = {"float32": 1e-4, "bfloat16": 0.0}
_engines = {}


def engine(name, dtype, seed=0, sharp=1.0, soft=False, max_tokens=2048, **kw):
    from x0ne_engine_b200 import Engine
    if dtype == "bfloat16":
        kw.setdefault("pass_graphs", False)          # the routers' choices are recorded by Python hooks (H.Choices)
    key = (name, dtype, seed, sharp, soft, max_tokens, tuple(sorted(kw.items())))
    if key not in _engines:
        folder, cfg, tensors = H.folder(name, seed, sharp, soft)
        _engines[key] = (Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, max_seq_len=max_tokens, **kw), cfg, tensors)
    return _engines[key]


def close_bf16(got, want, what):
    """Rows within the bfloat16 tolerance of the other tests; of many rows, one in fifty (or one) may reach twice
    that: a routed layer's weights are scores of a softmax, and a row in which two of them are close amplifies
    the rounding of its input."""
    from helpers import BF16_KL_TOL, BF16_LOGIT_TOL, kl_rows
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape and np.isfinite(got).all(), what
    err = np.max(np.abs(got - want), axis=-1) / (np.max(np.abs(want), axis=-1) + 1e-30)
    over = int((err > BF16_LOGIT_TOL).sum())
    assert err.max() <= 2 * BF16_LOGIT_TOL and over <= max(1, len(err) // 50), \
        f"{what}: worst logit error {err.max():.3e}, {over} of {len(err)} rows over {BF16_LOGIT_TOL}"
    kl = kl_rows(want, got)
    assert kl.max() <= 2 * BF16_KL_TOL and int((kl > BF16_KL_TOL).sum()) <= max(1, len(err) // 50), f"{what}: worst KL {kl.max():.3e}"


class Run:
    """Logits of one sequence and what its routers chose."""

    def __init__(self, logits, forced):
        self.logits, self.forced = logits, forced


def check(dtype, cfg, t, ids, run, what, rows=None):
    """A run against the plain implementation.  float32: the plain implementation chooses for itself.  bfloat16: it
    follows the run's choices (they may differ where two are within bfloat16's rounding), and the choices
    must agree with the plain ones wherever those are clear."""
    rows = slice(None) if rows is None else rows
    if dtype == "float32":
        assert_close_f32(run.logits[rows], H.plain_logits(cfg, t, ids)[rows], what)
        return
    close_bf16(run.logits[rows], H.plain_logits(cfg, t, ids, None, None, run.forced)[rows], what)
    if run.forced:
        overall, clear = H.agreement(cfg, t, ids, run.forced, clear=0.15)
        assert clear >= 0.98 and overall >= 0.85, f"{what}: routers agree on {overall:.3f} of all rows, {clear:.3f} of the clear ones"


def same_cut(dtype, cfg, t, ids, run, base, what):
    """Two runs of one sequence cut differently: the same bits in float32; in bfloat16 each is held against the
    plain implementation (a router may choose differently in the two)."""
    if dtype == "float32":
        got, want = np.asarray(run.logits), np.asarray(base.logits)
        assert np.array_equal(got, want), f"{what}: first difference at {first_difference(got, want)}"
    else:
        check(dtype, cfg, t, ids, run, what)


def ids_for(cfg, t, n, dtype, seed=0):
    return H.clear_ids(cfg, t, n, seed, MARGIN[dtype])


def in_pieces(eng, ids, cuts):
    """The prompt cut at `cuts` (piece sizes, the last piece takes the rest): logits of all places, and the choices."""
    with H.Choices(eng) as rec:
        s = eng.new_sequence()
        out, at = [], 0
        try:
            for c in list(cuts) + [len(ids)]:
                piece = ids[at:at + c]
                if not piece:
                    break
                out.append(eng.step([s], [piece], [list(range(len(piece)))]).cpu().numpy())
                at += len(piece)
            forced = rec.of(s, len(ids))
        finally:
            eng.free_sequence(s)
    return Run(np.concatenate(out), forced)


def whole(eng, ids):
    return in_pieces(eng, ids, [])


# ------------------------------------------------------------------------------------------ row-wise kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [72, 128, 1000, 5000])
def test_add_of_a_normed_delta_then_norm(dtype, hidden):
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(2)
    rows, eps_d, eps = 6, 1e-5, 1e-6
    resid = torch.randn(rows, hidden, generator=g).to(DEV)
    d = (3 * torch.randn(rows, hidden, generator=g)).to(dtype).to(DEV)
    wd, w = ((1 + 0.2 * torch.randn(hidden, generator=g)).to(DEV) for _ in range(2))
    out = torch.empty((rows, hidden), dtype=dtype, device=DEV)
    before = resid.clone()
    ops.add_normed_rmsnorm(resid, d, wd, eps_d, w, out, rows, eps)
    want_r = before.double() + P.rms_norm(d.double(), wd.double(), eps_d)
    assert (resid.double() - want_r).abs().max() <= 2e-6 * want_r.abs().max()       # the normed delta is never rounded
    want = P.rms_norm(want_r, w.double(), eps)
    tol = 2e-6 if dtype == torch.float32 else 2 ** -8
    assert (out.double() - want).abs().max() <= tol * want.abs().max()
    # gathered rows (the final norm of the wanted rows only)
    resid2 = before.clone()
    rows_t = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    out2 = torch.empty((2, hidden), dtype=dtype, device=DEV)
    ops.add_normed_rmsnorm(resid2, d, wd, eps_d, w, out2, 2, eps, rows_t)
    assert torch.equal(out2, out[[4, 1]]) and torch.equal(resid2[0], before[0])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scaled_embedding(dtype):
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    table = torch.randn(50, 72, generator=g).to(dtype).to(DEV)
    tok = torch.tensor([3, 49, 0, 77], dtype=torch.int32, device=DEV)
    resid = torch.empty((4, 72), dtype=torch.float32, device=DEV)
    ops.embedding(table, tok, resid, 4, 3.25)
    assert torch.equal(resid[:3], table[[3, 49, 0]].float() * 3.25) and not resid[3].any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H_,G,D,Dv,rot", [(6, 2, 20, 12, 12), (4, 4, 32, 32, 32), (3, 1, 10, 6, 0), (8, 2, 64, 64, 16)])
def test_whole_projection_norm_rotation_and_cache_write(dtype, H_, G, D, Dv, rot):
    from x0ne_engine_b200.cache import SequenceCache
    from x0ne_engine_b200.csrc import ops
    from x0ne_engine_b200.parts.base import CacheNeed
    g = torch.Generator().manual_seed(4)
    rows, eps, base = 5, 1e-5, 1000.0
    cache = SequenceCache([CacheNeed("kv", G, D, None, v_dim=None if Dv == D else Dv)], [None], 512, 512, dtype, DEV)
    slot = cache.acquire(300)
    pos = torch.tensor([0, 1, 63, 64, 200], dtype=torch.int32, device=DEV)
    slots = torch.full((rows,), slot, dtype=torch.int32, device=DEV)
    width = H_ * D + G * D + G * Dv
    src = torch.randn(rows, width, generator=g).to(dtype).to(DEV)
    wq = (1 + 0.3 * torch.randn(H_ * D, generator=g)).to(DEV)
    wk = (1 + 0.3 * torch.randn(G * D, generator=g)).to(DEV)
    freq = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1)).float().to(DEV) if rot else None
    q_out = torch.empty((rows, H_ * D), dtype=dtype, device=DEV)
    view = cache.kv_view(0)
    ops.whole_norm_rope_kv_write(src, H_ * D, H_ * D + G * D, wq, wk, eps, freq, rot, None, q_out, H_, view, slots, pos, rows, True)
    x = src.double().cpu()
    p_cpu = pos.cpu()
    q_want = P.rotate_half_layout(P.rms_norm(x[:, :H_ * D], wq.cpu().double(), eps).view(rows, H_, D), p_cpu, rot, base)
    k_want = P.rotate_half_layout(P.rms_norm(x[:, H_ * D:H_ * D + G * D], wk.cpu().double(), eps).view(rows, G, D), p_cpu, rot, base)
    tol = 3e-6 if dtype == torch.float32 else 2 ** -8
    assert (q_out.float().cpu().view(rows, H_, D) - q_want).abs().max() <= tol * q_want.abs().max()
    # read the cache back through the plain attention kernel's view of it: one-hot queries would be roundabout,
    # so the storage is read directly: page of (slot, pos), keys [kv head][64][D], then values [kv head][64][Dv]
    g0 = cache.groups[0]
    store = g0.storage[0].reshape(g0.n_pages, -1).float().cpu()
    for r in range(rows):
        page = int(g0.table_host[slot, int(p_cpu[r]) // 64])
        at = int(p_cpu[r]) % 64
        keys = store[page, :G * 64 * D].view(G, 64, D)[:, at]
        vals = store[page, G * 64 * D:].view(G, 64, Dv)[:, at]
        assert (keys - k_want[r]).abs().max() <= tol * k_want.abs().max()
        assert torch.equal(vals.double(), x[r, H_ * D + G * D:].view(G, Dv))


def plain_route(z, corr, groups, keep, top):
    cfg = {"experts": z.shape[1], "top": top, "groups": {"count": groups, "keep": keep}}
    w = {"r.router": torch.eye(z.shape[1]), "r.correction": corr}
    return P.route(z.double(), cfg, w, "r.")


@pytest.mark.parametrize("n,groups,keep,top", [(10, 5, 2, 3), (8, 1, 1, 3), (12, 4, 2, 5), (6, 3, 2, 1), (64, 8, 3, 6), (7, 7, 2, 2)])
def test_router_choice(n, groups, keep, top):
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(n)
    rows = 37
    z = torch.randn(rows, n + 1, generator=g) * 3
    corr = torch.randn(n, generator=g) * 0.3 - 0.4               # mostly negative choice values
    chosen = torch.empty((rows, top), dtype=torch.int32, device=DEV)
    weights = torch.empty((rows, top), dtype=torch.float32, device=DEV)
    sgate = torch.empty((rows,), dtype=torch.float32, device=DEV)
    ops.moe_route(z.to(DEV), corr.to(DEV), n, groups, keep, top, rows, chosen, weights, sgate, n)
    want_c, want_w = plain_route(z[:, :n], corr, groups, keep, top)
    assert torch.equal(chosen.cpu().long(), want_c)
    assert (weights.cpu() - want_w).abs().max() <= 1e-6
    assert (sgate.cpu() - torch.sigmoid(z[:, n])).abs().max() <= 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,E,I,top,hidden,ff", [(1, 4, 0, 2, 64, 32), (9, 6, 2, 3, 72, 40), (150, 3, 3, 2, 100, 50), (70, 16, 0, 4, 128, 96)])
def test_experts_over_grouped_pairs(dtype, rows, E, I, top, hidden, ff):
    """Grouping, both products and the weighted sum against a loop over rows and choices."""
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, hidden, generator=g).to(dtype)
    up = (torch.randn(E, ff, hidden, generator=g) / hidden ** 0.5).to(dtype)
    down = (torch.randn(E, hidden, ff, generator=g) / ff ** 0.5).to(dtype)
    chosen = torch.stack([torch.randperm(E + I, generator=g)[:top] for _ in range(rows)]).to(torch.int32)
    weights = torch.rand(rows, top, generator=g)
    shared = torch.randn(rows, hidden, generator=g).to(dtype)
    sgate = torch.rand(rows, generator=g)
    pairs = rows * top
    n_tiles = ops.moe_max_tiles(pairs, E)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    listed = torch.empty(pairs, dtype=torch.int32, device=DEV)
    tiles = torch.empty((n_tiles, 3), dtype=torch.int32, device=DEV)
    act = torch.empty((pairs, ff), dtype=dtype, device=DEV)
    y = torch.empty((pairs, hidden), dtype=torch.float32, device=DEV)
    out = torch.empty((rows, hidden), dtype=dtype, device=DEV)
    xd, ch = x.to(DEV), chosen.to(DEV)
    ops.moe_group(ch, pairs, E, offsets, listed, tiles)
    off = offsets.cpu().tolist()
    flat = chosen.flatten()
    assert [off[e + 1] - off[e] for e in range(E)] == [int((flat == e).sum()) for e in range(E)]
    for e in range(E):
        assert sorted(listed.cpu()[off[e]:off[e + 1]].tolist()) == torch.nonzero(flat == e).flatten().tolist()
    ops.moe_product(0, xd, up.to(DEV), listed, tiles, n_tiles, top, act)
    ops.moe_product(1, act, down.to(DEV), listed, tiles, n_tiles, top, y)
    ops.moe_combine(y, xd, ch, weights.to(DEV), top, E, shared.to(DEV), sgate.to(DEV), out, rows)
    want = torch.zeros(rows, hidden, dtype=torch.float64)
    for r in range(rows):
        for j in range(top):
            e = int(chosen[r, j])
            v = x[r].double() if e >= E else torch.relu(up[e].double() @ x[r].double()).square() @ down[e].double().T
            want[r] += weights[r, j].double() * v
        want[r] += sgate[r].double() * shared[r].double()
    tol = 1e-5 if dtype == torch.float32 else 2 ** -6
    assert (out.double().cpu() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("rows,E,I,top,hidden,ff", [(100, 5, 1, 3, 72, 40), (700, 16, 2, 4, 256, 192), (513, 3, 0, 1, 320, 600)])
def test_experts_on_the_tensor_cores(rows, E, I, top, hidden, ff):
    """Tiles of 128 listed pairs on tcgen05 (rows gathered into the listed order, activations kept in it, the down
    product written by pair) against a loop over rows and choices; widths that end inside a tile of 256 outputs
    and inside a slice of 64 inner values, experts with no pair and with more than a tile of them."""
    from x0ne_engine_b200.csrc import ops
    g = torch.Generator().manual_seed(rows)
    dtype = torch.bfloat16
    x = torch.randn(rows, hidden, generator=g).to(dtype)
    up = (torch.randn(E, ff, hidden, generator=g) / hidden ** 0.5).to(dtype)
    down = (torch.randn(E, hidden, ff, generator=g) / ff ** 0.5).to(dtype)
    n_out = E + I
    prefer = torch.rand(n_out, generator=g) ** 3                 # unequal loads; the last real expert gets no pair at all
    prefer[E - 1] = 0
    chosen = torch.stack([torch.multinomial(prefer + 1e-9 * (torch.arange(n_out) != E - 1), top, generator=g) for _ in range(rows)]).to(torch.int32)
    weights = torch.rand(rows, top, generator=g)
    pairs = rows * top
    assert ops.moe_tc_takes(dtype, pairs, hidden, ff)
    n_tiles = ops.moe_max_tiles(pairs, E, ops.MOE_TC_TILE_ROWS)
    i32 = lambda *shape: torch.empty(shape, dtype=torch.int32, device=DEV)
    offsets, listed, tiles, n_real = i32(E + 1), i32(pairs), i32(n_tiles, 3), i32(1)
    xs = torch.full((pairs, hidden), float("nan"), dtype=dtype, device=DEV)      # places that hold no pair keep whatever was there
    act = torch.empty((pairs, ff), dtype=dtype, device=DEV)
    y = torch.empty((pairs, hidden), dtype=torch.float32, device=DEV)
    out = torch.empty((rows, hidden), dtype=dtype, device=DEV)
    xd, ch = x.to(DEV), chosen.to(DEV)
    ops.moe_group(ch, pairs, E, offsets, listed, tiles, ops.MOE_TC_TILE_ROWS, n_real)
    counts = [int((chosen.flatten() == e).sum()) for e in range(E)]
    assert int(n_real[0]) == sum(-(-c // 128) for c in counts) and counts[E - 1] == 0 and (max(counts) > 128 or rows < 200)
    ops.moe_gather_rows(xd, listed, offsets, E, top, xs, pairs)
    ops.moe_product_tc(0, xs, up.to(DEV), listed, tiles, n_real, n_tiles, act)
    ops.moe_product_tc(1, act, down.to(DEV), listed, tiles, n_real, n_tiles, y)
    ops.check_tc_status(torch.device(DEV))
    ops.moe_combine(y, xd, ch, weights.to(DEV), top, E, None, None, out, rows)
    want = torch.zeros(rows, hidden, dtype=torch.float64)
    for r in range(rows):
        for j in range(top):
            e = int(chosen[r, j])
            if e >= E:
                v = x[r].double()
            else:
                a = torch.relu(up[e].double() @ x[r].double()).square().to(dtype).double()      # the activations are kept in bfloat16
                v = a @ down[e].double().T
            want[r] += weights[r, j].double() * v
    assert (out.double().cpu() - want).abs().max() <= 2 ** -7 * want.abs().max()


ATT_CASES = [  # q_heads, kv_heads, dk, dv, window, keep_first, sink
    (4, 2, 48, None, 100, 4, True),
    (6, 2, 20, 12, 37, 70, True),        # kept keys on two pages
    (3, 3, 24, 40, 64, 64, False),       # a whole page kept
    (20, 1, 16, 80, 9, 1, True),
    (8, 2, 64, 64, 48, 130, True),       # more kept keys than the window is long
    (2, 1, 40, 24, 300, 0, True),
]


@pytest.mark.parametrize("case", ATT_CASES)
def test_attention_kernels_with_kept_first_keys(case):
    """The plain kernel in float32 against explicit sums, and the tensor-core prefill and decode kernels
    against the plain kernel, on a scattered cache: unequal sequences, rows on page borders, rows whose
    window starts just before, at and just after the last kept key, several splits of a long row."""
    from test_rovurax_gpu import plain_kernel_in_float32, scattered_cache
    from x0ne_engine_b200.csrc import ops
    H_, G, dk, dv, window, keep, sink = case
    vd = dk if dv is None else dv
    pages = 12
    storage, table, view = scattered_cache(G, dk, dv, 3, pages, seed=dk + keep)
    view_args = (view.page_stride, view.table_stride, view.ring_pages, 64, G, dk, view.n_pages, view.v_dim)
    g = torch.Generator().manual_seed(7)
    scale = 1.7 * dk ** -0.5
    sink_t = (torch.randn(H_, generator=g) * 2).to(DEV) if sink else None
    seqs = [(0, 130, 200), (1, 63, 1), (2, 0, 67)]
    n_rows = sum(n for _, _, n in seqs)
    q = torch.randn(n_rows, H_ * dk, generator=g).bfloat16().to(DEV)
    slots = torch.tensor([s for s, _, n in seqs for _ in range(n)], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p0 + r for _, p0, n in seqs for r in range(n)], dtype=torch.int32, device=DEV)
    kw = dict(sink=sink_t, keep_first=keep)
    want, _ = plain_kernel_in_float32(q, view_args, storage, table, slots, pos, H_, scale, window, kw, vd)
    # the plain kernel itself, against explicit sums over the keys a row may see
    s32 = storage.float().cpu()
    per = G * 64 * (dk + vd)
    tab = table.cpu()
    for r in (0, 5, 70, 199, 200, 201, 230, 267):
        s_, p_ = int(slots[r]), int(pos[r])
        js = [j for j in range(p_ + 1) if p_ - j < window or j < keep]
        for h in (0, H_ - 1):
            kh = h // (H_ // G)
            ks = torch.stack([s32[tab[s_, j // 64]][:G * 64 * dk].view(G, 64, dk)[kh, j % 64] for j in js])
            vs = torch.stack([s32[tab[s_, j // 64]][G * 64 * dk:per].view(G, 64, vd)[kh, j % 64] for j in js])
            sc = (ks.double() @ q[r].float().cpu().view(H_, dk)[h].double()) * scale
            m = max(sc.max(), sink_t[h].cpu().double()) if sink else sc.max()
            e = torch.exp(sc - m)
            den = e.sum() + (torch.exp(sink_t[h].cpu().double() - m) if sink else 0.0)
            ref = (e[:, None] * vs.double()).sum(0) / den
            got = want[r].view(H_, vd)[h].double().cpu()
            assert (got - ref).abs().max() <= 1e-5 * max(ref.abs().max(), 1e-3), (r, h)
    assert ops.attention_flex_takes(view, torch.bfloat16, 0, False) and ops.attention_flex_takes(view, torch.bfloat16, 0, True)
    first, tiles = [0], []
    for k, (_, _, n) in enumerate(seqs):
        tiles += [(k, first[-1] + r0) for r0 in range(0, n, 128)]
        first.append(first[-1] + n)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    out = torch.zeros((n_rows, H_ * vd), dtype=torch.bfloat16, device=DEV)
    ops.attention_flex_prefill(q, out, view, i32([t[0] for t in tiles]), i32([t[1] for t in tiles]), len(tiles), i32(first),
                               i32([s for s, _, _ in seqs]), i32([p for _, p, _ in seqs]), H_, scale, window, ops.attn_extra(**kw))
    err = (out.float() - want).abs().max().item()
    assert err <= 2 ** -7 * want.abs().max().item(), f"prefill {err}"
    # decode: rows whose window starts around the last kept key, on page borders, and far out
    rows = [(0, 63), (1, 64), (2, 64 * pages - 2), (0, keep + window - 2), (1, keep + window - 1), (2, keep + window),
            (0, max(keep, 1) - 1), (1, window - 1), (2, window)]
    q1 = torch.randn(len(rows), H_ * dk, generator=g).bfloat16().to(DEV)
    slots1, pos1 = i32([s for s, _ in rows]), i32([p for _, p in rows])
    want1, _ = plain_kernel_in_float32(q1, view_args, storage, table, slots1, pos1, H_, scale, window, kw, vd)
    for splits in (1, 2, 5):
        out1 = torch.zeros((len(rows), H_ * vd), dtype=torch.bfloat16, device=DEV)
        scratch = torch.empty(ops.attention_flex_scratch_bytes(len(rows), H_, G, vd, splits) // 4 + 1, dtype=torch.float32, device=DEV)
        ops.attention_flex_decode(q1, out1, view, slots1, pos1, len(rows), H_, scale, window, ops.attn_extra(**kw), splits, scratch)
        err = (out1.float() - want1).abs().max().item()
        assert err <= 2 ** -7 * want1.abs().max().item(), f"decode, {splits} splits: {err}"


# ------------------------------------------------------------------------------------------ the model, whole
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,lengths", [("attention_only", [1, 2, 9, 10, 40]), ("dense_only", [1, 12]), ("experts_only", [1, 3, 70]),
                                          ("mixed", [1, 2, 37, 38, 65, 150]), ("even", [64, 131, 300]), ("wide", [5, 71, 141]),
                                          ("odd", [1, 12, 90]), ("served", [7, 450])])
def test_each_request_alone_and_whole(name, lengths, dtype):
    eng, cfg, t = engine(name, dtype)
    for k, n in enumerate(lengths):
        ids = ids_for(cfg, t, n, dtype, seed=k)
        check(dtype, cfg, t, ids, whole(eng, ids), f"{name} len {n}")


def test_residual_stream_after_every_layer():
    """The float32 residual after each layer (the pending normed delta added by hand) against the plain one."""
    eng, cfg, t = engine("mixed", "float32")
    ids = ids_for(cfg, t, 90, "float32", seed=3)
    want = []
    H.plain_logits(cfg, t, ids, want)
    seen = []
    for b in eng.model.blocks:
        def wrapped(ctx, entry, resid, delta, cache_entry=None, write_cache=True, _f=b.forward):
            out = _f(ctx, entry, resid, delta, cache_entry=cache_entry, write_cache=write_cache)
            d = out.delta.double()[:ctx.n_rows]
            seen.append((resid[:ctx.n_rows].double() + P.rms_norm(d, out.norm.weight.double(), out.norm.eps)).cpu())
            return out
        b.forward = wrapped
    try:
        whole(eng, ids)
    finally:
        for b in eng.model.blocks:
            del b.forward
    assert len(seen) == len(want)
    for i, (a, b) in enumerate(zip(seen, want)):
        assert (a - b.double()).abs().max() <= 1e-4 * b.abs().max(), f"layer {i}"


def test_soft_routing_in_float32():
    """Routers with ordinary logits and random corrections: many rows choose by small differences of the scores."""
    for name in ("mixed", "odd"):
        eng, cfg, t = engine(name, "float32", soft=True)
        ids = H.clear_ids(cfg, t, 120, 4, 1e-4)
        base = whole(eng, ids)
        check("float32", cfg, t, ids, base, name)
        same_cut("float32", cfg, t, ids, in_pieces(eng, ids, [50, 3] + [1] * 67), base, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,n,tail", [("mixed", 120, 60), ("wide", 100, 40), ("even", 160, 40), ("odd", 70, 30), ("served", 330, 140)])
def test_prefill_against_token_by_token(name, n, tail, dtype):
    eng, cfg, t = engine(name, dtype)
    ids = ids_for(cfg, t, n, dtype, seed=5)
    base = whole(eng, ids)
    got = in_pieces(eng, ids, [n - tail] + [1] * tail)
    same_cut(dtype, cfg, t, ids, got, base, f"{name}: last {tail} one by one")
    check(dtype, cfg, t, ids, got, f"{name} decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "even"])
def test_prompt_in_portions_down_to_two_tokens(name, dtype):
    eng, cfg, t = engine(name, dtype)
    ids = ids_for(cfg, t, 170, dtype, seed=6)
    base = whole(eng, ids)
    for cuts in ([2] * 30, [64, 64], [63, 2, 1, 64], [37, 37, 37, 37], [3, 125, 2], [129]):
        same_cut(dtype, cfg, t, ids, in_pieces(eng, ids, cuts), base, f"{name} cut {cuts[:4]}")
    check(dtype, cfg, t, ids, base, name)


def test_a_step_cut_into_passes_inside_prompts():
    eng, cfg, t = engine("mixed", "float32", max_step_tokens=64)
    ids = ids_for(cfg, t, 150, "float32", seed=7)
    assert np.array_equal(whole(eng, ids).logits, whole(engine("mixed", "float32")[0], ids).logits)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_unequal_batches_against_each_alone_with_slots_used_again(name, dtype):
    eng, cfg, t = engine(name, dtype)
    for round_ in range(3):                      # the second and third rounds get slots and pages that were used
        lengths, steps = [[1, 30, 77, 140], [66, 2, 129], [140, 5]][round_], [3, 9, 1, 6]
        full = [ids_for(cfg, t, n + steps[k], dtype, seed=10 * round_ + k) for k, n in enumerate(lengths)]
        prompts = [f[:n] for f, n in zip(full, lengths)]
        tails = [f[n:] for f, n in zip(full, lengths)]
        with H.Choices(eng) as rec:
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
            runs = [Run(np.concatenate(got[k]), rec.of(slots[k], len(full[k]))) for k in range(len(lengths))]
            for s in slots:
                eng.free_sequence(s)
        for k, n in enumerate(lengths):
            alone = whole(eng, full[k])
            same_cut(dtype, cfg, t, full[k], runs[k], alone, f"{name} round {round_} request {k}")
            if round_ == 0:
                check(dtype, cfg, t, full[k], alone, f"{name} request {k}")


# ------------------------------------------------------------------------------------------ edges, far keys
@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edges_and_kept_keys_that_decide(dtype):
    """Sharp queries make single keys decide a row, so a window or a count of kept keys that is one off, or
    a page read wrongly, changes the logits by far more than the tolerance.  Windows of 37, 50, 64 and 9
    positions and 3, 70, 1 and 0 kept keys against pages of 64; every position of a 260-token sequence is
    checked, in a prompt and decoded alone."""
    eng, cfg, t = engine("mixed", dtype, seed=3, sharp=4.0 if dtype == "float32" else 1.5)
    ids = ids_for(cfg, t, 260, dtype, seed=8)
    want = H.plain_logits(cfg, t, ids)

    def moved(change):
        layers = [dict(l, mixer=dict(l["mixer"], mask=change(dict(l["mixer"]["mask"])))) for l in cfg["layers"]]
        diff = np.abs(H.plain_logits({**cfg, "layers": layers}, t, ids) - want).max(-1) / np.abs(want).max(-1)
        return (diff > 0.1).sum()
    # the test sees what it is for: one more key in the window, or one kept key fewer, changes the plain result
    many = 60 if dtype == "float32" else 25
    assert moved(lambda m: {**m, "size": m["size"] + 1}) > many
    assert moved(lambda m: {**m, "keep_first": max(m["keep_first"] - 1, 0)}) > many
    check(dtype, cfg, t, ids, whole(eng, ids), "prompt")
    check(dtype, cfg, t, ids, in_pieces(eng, ids, [30] + [1] * 230), "decoded across window edges, kept keys and page borders")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_kept_key_far_back_and_the_sink(dtype):
    """The first token's key is made to dominate a late query: one key direction of head 0 is aligned with
    that token's embedding and the same query direction with the last token's, so the late logits hang on a
    kept key hundreds of positions back, outside every window, read in a prompt and in decoding.  The sinks
    are raised until they hold a good part of the denominators.  Without the kept key, and without the
    sinks, the plain result differs by more than the tolerance."""
    from x0ne_engine_b200 import Engine
    cfg = H.config([H.layer(H.attention(heads=4, kv_heads=2, window=30, keep=2, rot=None), None),
                    H.layer(H.attention(heads=4, kv_heads=2, window=45, keep=1, rot=None, kv_from=0), H.dense(64))])
    t = H.make_tensors(cfg, seed=4)
    special, late = 7, 11
    u = t["embed"][special] / t["embed"][special].norm()
    u2 = t["embed"][late] / t["embed"][late].norm()
    t["l0.mix.k"][0] += 6.0 * u
    t["l0.mix.q"][0] += 6.0 * u2
    t["l1.mix.q"][0] += 6.0 * u2
    for name in ("l0.mix.q.norm", "l0.mix.k.norm", "l1.mix.q.norm"):
        t[name][0] = 4.0
    t["l0.mix.v"] *= 3.0
    t["l0.mix.sink"] += 6.0
    t["l1.mix.sink"] += 6.0
    t = {k: v.bfloat16().float() for k, v in t.items()}
    d = H.write_folder(cfg, t, "x0ne_tnt_far_")
    ids = [12 + x % (cfg["vocab"] - 12) for x in H.clear_ids(cfg, t, 700, 9)]
    ids[0] = special
    ids[-1] = late
    want = H.plain_logits(cfg, t, ids)[-3:]
    other = list(ids)
    other[0] = 9
    assert np.abs(H.plain_logits(cfg, t, other)[-1] - want[-1]).max() > 0.07 * np.abs(want[-1]).max()
    no_keep = {**cfg, "layers": [dict(l, mixer=dict(l["mixer"], mask={**l["mixer"]["mask"], "keep_first": 0})) for l in cfg["layers"]]}
    assert np.abs(H.plain_logits(no_keep, t, ids)[-1] - want[-1]).max() > 0.07 * np.abs(want[-1]).max()
    no_sink = dict(t)
    for k in ("l0.mix.sink", "l1.mix.sink"):
        no_sink[k] = t[k] - 40.0
    assert np.abs(H.plain_logits(cfg, no_sink, ids)[-1] - want[-1]).max() > 0.06 * np.abs(want[-1]).max()
    eng = Engine.from_folder(d, dtype=dtype, max_tokens=1024, max_seq_len=1024)
    check(dtype, cfg, t, ids, whole(eng, ids), "kept key in a prompt", rows=slice(-3, None))
    check(dtype, cfg, t, ids, in_pieces(eng, ids, [697, 1, 1]), "kept key decoded", rows=slice(-3, None))


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(dtype):
    eng, cfg, t = engine("mixed", dtype)
    ids = ids_for(cfg, t, 6, dtype, seed=11)
    check(dtype, cfg, t, ids, in_pieces(eng, ids, [1, 1, 1, 1, 1]), "first tokens one by one")
    check(dtype, cfg, t, ids, in_pieces(eng, ids, [2, 2]), "first tokens in twos")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    eng, cfg, t = engine("even", dtype)
    ids = ids_for(cfg, t, 420, dtype, seed=12)
    check(dtype, cfg, t, ids, in_pieces(eng, ids, [20] + [1] * 400), "400 decoded tokens")


# ------------------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", ["graph", "eager"])
def test_greedy_generation_through_the_entry_point(decode, dtype):
    from x0ne_engine_b200 import Model
    folder, cfg, t = H.folder("mixed")
    prompts = [ids_for(cfg, t, n, dtype, seed=20 + n) for n in (1, 7, 36, 64)]
    n_new = 14
    m = Model.from_folder(folder, dtype=dtype, max_batch=3, max_ctx=256, decode=decode)
    out = m.generate(prompts, max_tokens=n_new, stop_token_ids=())
    assert out.finish_reasons == ["length"] * len(prompts)
    for p, got in zip(prompts, out.tokens):
        ids = list(p)
        for tok in got:
            margins = []
            row = H.plain_logits(cfg, t, ids, None, margins)[-1]
            top = np.sort(row)[-2:]
            clear_route = min(float(x.min()) for x in margins) >= (1e-4 if dtype == "float32" else 0.15)
            if tok != int(np.argmax(row)):
                tol = 1e-4 if dtype == "float32" else 2 * 0.05
                assert not clear_route or top[1] - top[0] <= tol * np.abs(row).max(), "a token left a clear argmax"
                break
            if not clear_route:
                break                       # (from a close call of a router on, the two may part)
            ids.append(tok)
    assert m.generate(prompts, max_tokens=n_new, stop_token_ids=()).tokens == out.tokens


def test_random_model_from_a_configuration_generates():
    from x0ne_engine_b200 import Model
    from x0ne_engine_b200.config import config_from_dict
    m = Model.random(config_from_dict(H.CONFIGS["even"]()), seed=1, max_batch=2, max_ctx=128, norm_jitter=0.1)
    out = m.generate([[1, 2, 3], [4]], max_tokens=5, stop_token_ids=())
    assert [len(x) for x in out.tokens] == [5, 5] and all(0 <= x < 256 for row in out.tokens for x in row)


def test_short_prompt_passes_replayed_from_graphs_give_the_same_bits():
    eng, cfg, t = engine("mixed", "bfloat16", pass_graphs=True)
    base, _, _ = engine("mixed", "bfloat16", pass_graphs=False)
    assert eng.replayable and eng.pass_graphs and not base.pass_graphs
    before = eng.pass_graph_replays
    for k, lengths in enumerate([[100], [120], [70], [126], [20], [30], [5], [5], [100, 20], [90, 30], [100]]):
        prompts = [H.clear_ids(cfg, t, n, 100 + 7 * k + j) for j, n in enumerate(lengths)]
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
