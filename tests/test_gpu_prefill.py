"""Prompt chunks: steps of hundreds to 2,048 ordinary rows of one slot. Such a step takes the wide GEMM blocks (128 rows
per tensor-core instruction) and the chunked form of the gated delta rule (spl_gdn_chunk.cuh), neither of which the
verify-sized steps reach. Checked against the CPU oracle, whose recurrence is the reference's token-by-token one, and
against the library's own per-token kernel fed the same tokens in short steps (the reference's bound between two of its
kernels and its CPU statement: 5e-4 relative, Tests/SploshOracleTests/GdnCandidateTests.swift:41-47)."""
import numpy as np
import pytest

import splosh_b200 as S
from helpers import Pair, tokens_for, observed
from oracle import oracle as O
from test_gpu_step import check, SLICE_TOL

pytestmark = pytest.mark.gpu
STATE_TOL = 5e-4           # kernel against kernel on the same inputs
ORACLE_STATE_TOL = 3e-3    # against the oracle after thousands of tokens: the two sides' inputs differ by the bf16 roundings upstream


def test_two_2048_row_chunks_of_one_prompt_on_the_tiny_model():
    """BASELINE configuration 2's shape of work at the tiny model's size: a 4,096-token prompt fed as two 2,048-row steps;
    logits of the last token of each chunk and the recurrent state afterwards against the oracle."""
    g = S.tiny_geometry()
    pair = Pair(g, S.EngineConfig(max_slots=2, max_rows=2048, kv_pages=20, max_context=4608, max_logit_rows=8))
    toks = tokens_for(0xC0FFEE00, 4096, g.vocab)
    for chunk in range(2):
        rows = [S.EngineRow(0, toks[2048 * chunk + i], 2048 * chunk + i, i == 2047) for i in range(2048)]
        gl, ol = pair.step(rows)
        check(gl, ol, g.vocab, f"2048-row chunk {chunk}")
    for index in range(3):
        ob = pair.oengine.buffer("state", index)
        gb = pair.engine.debug_read("state", index, ob.size)
        worst = float(np.abs(gb - ob).max() / max(1.0, np.abs(ob).max()))
        observed(f"state of gated-delta block {index} after 4,096 prompt tokens in 64-token chunks: {worst:.2e} of the largest (<= {ORACLE_STATE_TOL})")
        assert worst <= ORACLE_STATE_TOL


def test_the_chunked_scan_equals_the_per_token_kernel_on_the_same_tokens():
    """One engine is fed 700 tokens as one step (chunks of 64, the last one of 60), its twin as steps of at most 63 rows
    (the per-token kernel), with three journal entries to replay in front of the long step: same state, same logits."""
    g = S.tiny_geometry()
    cfg = S.EngineConfig(max_slots=2, max_rows=768, kv_pages=8, max_context=1024, max_logit_rows=16)
    model = O.Model(O.tiny_geometry())
    a, b = S.Engine(g, cfg), S.Engine(g, cfg)
    a.load_model(model); b.load_model(model)
    toks = tokens_for(0xBEEF, 800, g.vocab)
    for e in (a, b):
        e.step([S.EngineRow(0, toks[i], i, False) for i in range(20)])
        e.step([S.EngineRow(0, toks[20 + i], 20 + i, True, True) for i in range(5)])
        e.accept_verify(0, 3, 23)                      # three journal entries wait for the next run
    a.debug_gdn_chunk_min(64)                          # the long step takes the chunked scan whatever the default threshold
    a.step([S.EngineRow(0, toks[23 + i], 23 + i, i == 699) for i in range(700)])
    fed = 0
    while fed < 700:
        n = min(63, 700 - fed)
        b.step([S.EngineRow(0, toks[23 + fed + i], 23 + fed + i, fed + i == 699) for i in range(n)])
        fed += n
    la, lb = a.all_logits(), b.all_logits()
    assert la.shape == lb.shape == (1, g.vocab)
    observed(f"chunked scan against per-token kernel, 700 tokens: max |logit difference| {float(np.abs(la - lb).max()):.3e}")
    assert np.abs(la - lb).max() <= 2e-2
    for index in range(3):
        sa = a.debug_read("state", index, 2 * g.gdn_value_heads * 128 * 128)[:g.gdn_value_heads * 128 * 128]
        sb = b.debug_read("state", index, 2 * g.gdn_value_heads * 128 * 128)[:g.gdn_value_heads * 128 * 128]
        worst = float(np.abs(sa - sb).max() / max(1.0, np.abs(sb).max()))
        # The first block's two kernels read identical inputs; the later blocks' inputs already differ by what the first left.
        bound = STATE_TOL if index == 0 else ORACLE_STATE_TOL
        observed(f"  state of block {index}: {worst:.2e} of the largest (<= {bound})")
        assert worst <= bound


def test_a_prompt_chunk_rides_with_verify_blocks_on_the_27b_shape():
    """The 27B-shape slice (head_dim 256, 48 / 16 delta heads, contractions of 5,120 to 17,408): two sessions verify 8-row
    blocks and a third feeds 136 prompt rows in the same step (two 128-row GEMM blocks, chunks of 64 + 64 + 8)."""
    g = S.b27_geometry(layers=4, vocab=32768)
    pair = Pair(g, S.EngineConfig(max_slots=3, max_rows=160, kv_pages=8, max_context=512, max_logit_rows=24))
    toks = tokens_for(0xC0FFEE00, 400, g.vocab)
    pair.engine.debug_gdn_chunk_min(64)                # the 136-row run takes the chunked scan (by default only runs of 512 rows and more do)
    pair.step([S.EngineRow(s, toks[50 * s + i], i, False) for s in range(2) for i in range(6 + s)])
    rows = [S.EngineRow(s, toks[100 + 10 * s + i], 6 + s + i, True, True) for s in range(2) for i in range(8)]
    rows += [S.EngineRow(2, toks[200 + i], i, i == 135) for i in range(136)]
    gl, ol = pair.step(rows)
    assert gl.shape == (17, g.vocab)
    check(gl, ol, g.vocab, "27B slice, prompt chunk with verify blocks", tol=SLICE_TOL)
    ob = pair.oengine.buffer("state", 0)
    gb = pair.engine.debug_read("state", 0, ob.size)
    assert np.abs(gb - ob).max() <= ORACLE_STATE_TOL * max(1.0, np.abs(ob).max())
