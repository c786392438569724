"""A wait inside a kernel that runs out: the step returns SPL_ERR_TIMEOUT, nothing faults or hangs, and the engine
takes the next step. The wait is made to run out on the host's say-so: a test switch has the q4 GEMM's weight-copy role
leave out one stage of every block's piece, so the roles that wait for that stage give up when their time budget
(shortened here) is spent, the block unwinds through its barriers, frees its tensor memory and sets the error word."""
import numpy as np
import pytest

import splosh_b200 as S
from helpers import Pair, tokens_for

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_gives_timeout_and_the_engine_stays_usable():
    g = S.tiny_geometry()
    pair = Pair(g, S.EngineConfig(max_slots=2, max_rows=32, kv_pages=4, max_context=512))
    toks = tokens_for(0xFEED, 64, g.vocab)
    rows = [S.EngineRow(0, toks[p], p, p == 11) for p in range(12)]
    engine = pair.engine
    engine.debug_wait_budget(20_000_000)            # 20 ms
    engine.debug_drop_weight_stage(1)
    try:
        with pytest.raises(S.EngineError) as caught:
            engine.step(rows)
        assert caught.value.case == "timeout" and "gave up" in str(caught.value)
    finally:
        engine.debug_drop_weight_stage(-1)
        engine.debug_wait_budget(250_000_000)
    # The slot the failed step touched starts again; the same rows now give the oracle's logits.
    engine.reset_slot(0)
    got, want = pair.step(rows)
    assert not np.isnan(got).any()
    assert np.abs(got - want).max() <= 5e-2


def test_static_gemm_reports_a_timeout_through_its_status_call():
    import torch
    from splosh_b200.engine import gemm_q4_static
    from oracle import oracle as O
    g = S.tiny_geometry()
    engine = S.Engine(g, S.EngineConfig(max_slots=1, max_rows=8, kv_pages=1, max_context=256))
    engine.load_model(O.Model(O.tiny_geometry()))
    d_a = torch.ones((4, 2816), device="cuda"); d_out = torch.zeros((4, 1024), device="cuda")
    engine.debug_wait_budget(20_000_000)
    engine.debug_drop_weight_stage(0)          # every block's first stage: this tensor's blocks have one stage each
    try:
        gemm_q4_static(engine, 0, "down", d_a.data_ptr(), 4, 0, d_out.data_ptr())
        torch.cuda.synchronize()
        with pytest.raises(S.EngineError) as caught:
            engine.static_status()
        assert caught.value.case == "timeout"
    finally:
        engine.debug_drop_weight_stage(-1)
        engine.debug_wait_budget(250_000_000)
    gemm_q4_static(engine, 0, "down", d_a.data_ptr(), 4, 0, d_out.data_ptr())
    torch.cuda.synchronize()
    engine.static_status()
