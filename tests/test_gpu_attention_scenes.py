"""The attention span scan and merge on the GPU against the CPU oracle, on the scenes of the reference's own
scan tests (Tests/SploshOracleTests/AttentionScanCandidateTests.swift:85-200, 548-637), for both head shapes the
library builds: head_dim 256 with six query heads per kv head (the 27B shape, the instantiation the benchmark runs)
and head_dim 128 with four (the tiny hybrid).

A scene: two slots with contexts [ctx * 2 // 5 + 17, ctx], the long slot first; 13 + 11 query rows = the last
tokens of each context, in blocks of 8 with a short last block; the page table shuffled by earlier traffic over a
pool with spare pages; every int8 code random; kScale = 0.04 (0.5 + u), vScale = 0.01 (0.5 + u) per token and NaN
wherever no token is stored, so a masked token that leaks shows; span limits 1 / 4 / 16; contexts that put a block
across the first page of a span or one token before a chunk boundary; one key with its scale x 50 late, early and
inside the step's own rows, and two such keys in one chunk.

The pool is written through spl_kv_import and the step runs with its KV store switched off (spl_debug_kv_store), so
the scan reads exactly what the scene wrote. The queries and output gates are the model's own (read back from the
GPU) and go to the oracle unchanged: both sides scan identical inputs, and the tolerances are the reference's
(AttentionScanCandidateTests.swift:35-40): 1/128 of the largest output on the vectors, 5e-4 on the log-sum.
"""
import numpy as np
import pytest

import splosh_b200 as S
from helpers import Pair, assert_tables_equal, observed
from oracle import tables as T

pytestmark = pytest.mark.gpu

VECTOR_TOL = 1.0 / 128.0      # of the scene's largest output magnitude
LOGSUM_TOL = 5e-4
HEADER_BYTES = 32             # the snapshot header ahead of the pages
MAX_CTX = 40011
_PAIRS = {}


def geometry_of(name):
    return S.b27_geometry(layers=4, vocab=32768) if name == "b27" else S.tiny_geometry()


def pair_for(name):
    """One engine + oracle pair per geometry, with a pool that holds the largest scene and five spare pages."""
    if name not in _PAIRS:
        pages = (MAX_CTX + 255) // 256 + (MAX_CTX * 2 // 5 + 17 + 255) // 256 + 5
        cfg = S.EngineConfig(max_slots=3, max_rows=64, kv_pages=pages, max_context=MAX_CTX + 256)
        _PAIRS[name] = Pair(geometry_of(name), cfg)
    return _PAIRS[name]


def host_only_step(pair, rows):
    """A step on the GPU engine; the oracle's host follows (pages, units) without computing anything."""
    ot = pair.ohost.build([T.Row(r.slot, r.token, r.position, r.want_logits, r.verify) for r in rows])
    pair.ohost.finish_step(ot)
    pair.engine.step(rows)


def fill_scene(pair, slot, ctx, seed, big_keys=()):
    """Write the slot's pages: random codes, per-token scales, NaN scales past the context; big_keys = [(token, factor)]."""
    g, e = pair.g, pair.engine
    hd, kvh = g.head_dim, g.kv_heads
    pages = (ctx + 255) // 256
    blob = e.export_kv(slot, ctx)
    codes, vecs = kvh * 256 * hd, kvh * 256
    per_page = 2 * codes + 2 * vecs * 4
    assert blob.size == HEADER_BYTES + pages * per_page          # one attention block in these geometries
    rng = np.random.default_rng(seed)
    body = blob[HEADER_BYTES:].reshape(pages, per_page)
    body[:, :2 * codes] = rng.integers(1, 256, (pages, 2 * codes), dtype=np.uint8)       # stored byte = code + 128, codes -127..127
    token = np.arange(pages * 256).reshape(pages, 1, 256)
    ks = (0.04 * (0.5 + rng.random((pages, kvh, 256)))).astype(np.float32)
    vs = (0.01 * (0.5 + rng.random((pages, kvh, 256)))).astype(np.float32)
    for tok, factor in big_keys:
        ks[tok // 256, :, tok % 256] *= factor
    stored = np.broadcast_to(token < ctx, ks.shape)
    ks = np.where(stored, ks, np.float32(np.nan)); vs = np.where(stored, vs, np.float32(np.nan))
    body[:, 2 * codes:2 * codes + vecs * 4] = ks.reshape(pages, -1).view(np.uint8)
    body[:, 2 * codes + vecs * 4:] = vs.reshape(pages, -1).view(np.uint8)
    e.import_kv(slot, ctx, blob)


def prepare(pair, ctx, seed, big_keys=(), compute=False):
    """Slots 0 (ctx tokens) and 1 (ctx * 2 // 5 + 17) on shuffled pages, the scene in the GPU pool and in the oracle's.
    With `compute` the oracle runs the page-taking steps too, so both sides hold the same recurrent state afterwards."""
    short = ctx * 2 // 5 + 17
    for slot in range(3):
        pair.reset(slot)
    take = pair.step if compute else (lambda rows: host_only_step(pair, rows))
    take([S.EngineRow(2, 7 + i, 700 + i, False) for i in range(3)])       # slot 2 takes three pages and frees them
    pair.reset(2)
    take([S.EngineRow(0, 5, ctx - 1, False), S.EngineRow(1, 6, short - 1, False)])
    fill_scene(pair, 0, ctx, seed, big_keys)
    fill_scene(pair, 1, short, seed + 1)
    for which in ("k_codes", "v_codes", "k_scale", "v_scale"):
        ob = pair.oengine.buffer(which, 0)
        ob[:] = pair.engine.debug_read(which, 0, ob.size, ob.dtype)
    return short


def untile_operand(cells, rows, width, rn):
    """The GEMM operand layout (row blocks of rn rows, 64-wide groups, 128-byte swizzle) back to [rows, width]."""
    blocks = (rows + rn - 1) // rn
    row = np.arange(rows)[:, None]; k = np.arange(width)[None, :]
    g, kk, rb, r = k >> 6, k & 63, row // rn, row % rn
    index = (g * blocks + rb) * (rn * 64) + (r >> 3) * 512 + (r & 7) * 64 + ((((kk >> 3) ^ (r & 7)) & 7) << 3) + (kk & 7)
    return cells[index]


def scan_both(pair, ctx, short, limit, label):
    g, e = pair.g, pair.engine
    hd, heads = g.head_dim, g.heads
    rows = [S.EngineRow(0, 11 + i, ctx - 13 + i, True) for i in range(13)] + [S.EngineRow(1, 40 + i, short - 11 + i, True) for i in range(11)]
    R = len(rows)
    ot = pair.ohost.build([T.Row(r.slot, r.token, r.position, r.want_logits, r.verify) for r in rows])
    pair.ohost.finish_step(ot)
    mine = e.host.build(rows)
    tab = e.host.last
    step_pages = int(tab.step_pages)
    pps = (step_pages + limit - 1) // limit
    spans = (step_pages + pps - 1) // pps
    tab.spans, tab.pages_per_span = spans, pps
    ot.spans, ot.pages_per_span = spans, pps
    mine["spans"], mine["pages_per_span"] = spans, pps
    assert_tables_equal(mine, ot)
    e.debug_kv_store(False)
    try:
        e.step_tables(tab, R)
    finally:
        e.debug_kv_store(True)
    e.host.finish_step()
    live = int(tab.live_rows)
    assert live == R
    att_ld = 2 * heads * hd + 2 * g.kv_heads * hd
    proj = e.debug_read("proj", 0, R * att_ld).reshape(R, att_ld)
    q = e.debug_read("q", 0, R * heads * hd, np.float16).astype(np.float32).reshape(R, heads, hd)
    got = e.debug_read("attn_partials", 0, live * heads * spans * (hd + 2)).reshape(live, heads, spans, hd + 2)
    rn = 16 if R <= 16 else 32 if R <= 32 else 64
    padded = (pair.config.max_rows + 63) // 64 * 64
    core_ld = max(g.value_dim, heads * hd)
    cells = e.debug_read("core", 0, padded * core_ld, np.uint16)
    merged_gpu = untile_operand(cells, R, heads * hd, rn).view(np.float16).astype(np.float32)
    ref, merged_ref = pair.oengine.attention_scan(ot, 0, live, q, proj[:, :2 * heads * hd].reshape(R, heads, 2 * hd))

    assert not np.isnan(got).any(), label
    empty = np.isneginf(ref[..., 0])
    # A record whose reference is -inf holds nothing: total 0 and a zero vector.
    assert np.array_equal(np.isneginf(got[..., 0]), empty), label
    assert (got[empty][:, 1:] == 0).all(), label
    with np.errstate(divide="ignore", invalid="ignore"):
        lse_got, lse_ref = got[..., 0] + np.log(got[..., 1]), ref[..., 0] + np.log(ref[..., 1])
        out_got, out_ref = got[..., 2:] / got[..., 1:2], ref[..., 2:] / ref[..., 1:2]
    full = ~empty
    assert full.any(), label
    worst_lse = float(np.abs(lse_got[full] - lse_ref[full]).max())
    scale = float(np.abs(out_ref[full]).max())
    worst_out = float(np.abs(out_got[full] - out_ref[full]).max()) / scale
    merged_scale = float(np.abs(merged_ref).max())
    worst_merged = float(np.abs(merged_gpu - merged_ref).max()) / merged_scale
    observed(f"attention scene {label}: spans {spans}, log-sum diff {worst_lse:.2e} (<= {LOGSUM_TOL:.0e}), span vectors {worst_out:.2e}, "
             f"merged output {worst_merged:.2e} of the largest (<= {VECTOR_TOL:.1e})")
    assert worst_lse <= LOGSUM_TOL, (label, worst_lse)
    assert worst_out <= VECTOR_TOL, (label, worst_out)
    assert worst_merged <= VECTOR_TOL, (label, worst_merged)
    return ref


@pytest.mark.parametrize("name", ["b27", "tiny"])
@pytest.mark.parametrize("ctx", [300, 5003, MAX_CTX])
def test_two_slots_over_shuffled_pages_under_span_limits_1_4_16(name, ctx):
    """AttentionScanCandidateTests.swift:548-570: contexts 300 / 5,003 / 40,011, each under span limits 1, 4 and 16."""
    pair = pair_for(name)
    short = prepare(pair, ctx, seed=ctx)
    for limit in (1, 4, 16):
        scan_both(pair, ctx, short, limit, f"{name} ctx {ctx} limit {limit}")


@pytest.mark.parametrize("name", ["b27", "tiny"])
@pytest.mark.parametrize("ctx", [5130, 5122, 5119])
def test_blocks_that_straddle_a_span_or_stop_short_of_a_chunk(name, ctx):
    """AttentionScanCandidateTests.swift:572-609: a full block (5,130) and a short block (5,122) across the first page
    of a span, and a block whose first position is one token before a chunk boundary (5,119)."""
    pair = pair_for(name)
    short = prepare(pair, ctx, seed=ctx)
    for limit in (4, 16):
        scan_both(pair, ctx, short, limit, f"{name} ctx {ctx} limit {limit}")


@pytest.mark.parametrize("name", ["b27", "tiny"])
@pytest.mark.parametrize("case,keys", [("late", [(5003 - 40, 50.0)]), ("early", [(37, 50.0)]), ("inside the step's rows", [(5003 - 5, 50.0)]),
                                       ("two in one chunk", [(2600, 50.0), (2610, 35.0)])])
def test_one_key_fifty_times_larger_moves_the_softmax_reference(name, case, keys):
    """AttentionScanCandidateTests.swift:571, 611-631: a key whose scale is x 50 makes scores far above the running
    reference after the first chunk, so the reference is raised and what was accumulated is rescaled; placed late,
    early, inside the step's own rows (visible to some rows of a block only), and twice in one chunk."""
    pair = pair_for(name)
    ctx = 5003
    short = prepare(pair, ctx, seed=77, big_keys=keys)
    for limit in (1, 4):
        ref = scan_both(pair, ctx, short, limit, f"{name} big key {case} limit {limit}")
    # The scene does what it is for: for some query of the long slot the large key dominates its span.
    assert np.nanmax(ref[:13, :, :, 0]) > 60.0


def test_long_context_logits_on_the_27b_shape_with_the_kv_store_on():
    """The whole step at 5,003 tokens of context on the 27B-shape slice (spl_attn_scan_kernel<256, 6>, several pages,
    the engine's own span split), keys and values of the step's rows stored by both sides: logits against the oracle."""
    from test_gpu_step import check, SLICE_TOL
    pair = pair_for("b27")
    ctx = 5003
    short = prepare(pair, ctx, seed=5, compute=True)
    rows = [S.EngineRow(0, 11 + i, ctx + i, True, True) for i in range(13)] + [S.EngineRow(1, 40 + i, short + i, True) for i in range(11)]
    gl, ol = pair.step(rows)
    worst = check(gl, ol, pair.g.vocab, "27B slice, long context", tol=SLICE_TOL)
    observed(f"27B-shape slice at {ctx} tokens: max |logit - oracle| {worst:.3e} (<= {SLICE_TOL})")
