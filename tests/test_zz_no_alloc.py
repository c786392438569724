"""spl_gemm_q4_static: the GEMM for callers that cannot allocate device memory (a host that owns
the whole GPU through its own pool, or a serving loop that bans cudaMalloc and cudaFree because they
synchronise the device). It keeps its scratch in a static device array, so the test's job is to show that the
static-scratch variant computes what the ordinary entry point (spl_op_gemm_q4) computes, on two
calls in a row that share the array, and that it refuses what the array cannot hold.

This file sorts last on purpose: a run that stops at the first failure has then run everything else."""
import numpy as np
import pytest

import splosh_b200 as S
from splosh_b200.engine import gemm_q4_static

pytestmark = pytest.mark.gpu


def test_static_scratch_gemm_equals_the_ordinary_entry_point_twice_in_a_row(oracle):
    import torch
    g = S.tiny_geometry()
    engine = S.Engine(g, S.EngineConfig(max_slots=1, max_rows=8, kv_pages=1, max_context=256))
    model = oracle.Model(oracle.tiny_geometry())
    engine.load_model(model)
    rng = np.random.default_rng(5)
    # Two calls back to back on different tensors and row counts: the second reuses the array the first left dirty.
    calls = [(0, "down", "down", 37, True), (3, "out_proj", "o", 5, False), (1, "gate_up", "gate", 64, False)]
    pending = []
    for layer, which, kind, rows, with_residual in calls:
        packed, scales, biases = model.q4(layer, kind)
        n, k = packed.shape[0], packed.shape[1] * 8
        a = rng.normal(0, 1, (rows, k)).astype(np.float32)
        res = rng.normal(0, 1, (rows, n)).astype(np.float32) if with_residual else None
        want = S.gemm_q4(packed, scales, biases, a, res)                 # the existing entry point, host buffers
        ld = 2 * n if which == "gate_up" else n
        d_a = torch.from_numpy(a).cuda()
        d_out = torch.full((rows, ld), float("nan"), device="cuda")
        d_res = None
        if with_residual:
            d_out.copy_(torch.from_numpy(res))                             # residual aliased onto the output
            d_res = d_out
        gemm_q4_static(engine, layer, which, d_a.data_ptr(), rows, d_res.data_ptr() if d_res is not None else 0, d_out.data_ptr())
        pending.append((d_out, d_a, want, n))
    torch.cuda.synchronize()
    for d_out, _, want, n in pending:
        got = d_out.cpu().numpy()[:, :n]
        assert not np.isnan(got).any()
        # Same kernel, same split: the two entry points agree to the tolerance of the GEMM tests.
        assert np.abs(got - want).max() <= 4e-6 * np.abs(want).max()


def test_static_scratch_gemm_refuses_what_does_not_fit(oracle):
    import torch
    g = S.tiny_geometry()
    engine = S.Engine(g, S.EngineConfig(max_slots=1, max_rows=8, kv_pages=1, max_context=256))
    engine.load_model(oracle.Model(oracle.tiny_geometry()))
    d = torch.zeros(128 * 2816, device="cuda")
    with pytest.raises(S.EngineError) as caught:
        gemm_q4_static(engine, 0, "down", d.data_ptr(), 65, 0, d.data_ptr())
    assert caught.value.case == "invalidRows" and "64" in str(caught.value)
    with pytest.raises(S.EngineError):
        gemm_q4_static(engine, 0, "head", d.data_ptr(), 1, 0, d.data_ptr())    # the head is a model-level tensor
