"""spl_gemm_q4_static: the GEMM for callers that cannot allocate device memory (a host that owns
the whole GPU through its own pool, or a serving loop that bans cudaMalloc and cudaFree because they
synchronise the device). It keeps its scratch in a static device array, so the test's job is to show that the
static-scratch variant computes what the ordinary entry point (spl_op_gemm_q4) and the CPU oracle compute, on
calls in a row that share the array, that the calls after the first leave the device's free memory as it was, and
that it refuses what the array cannot hold.

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
        reference = oracle.gemm_q4(packed, scales, biases, a, res)       # and the CPU oracle on the same inputs
        ld = 2 * n if which == "gate_up" else n
        d_a = torch.from_numpy(a).cuda()
        d_out = torch.full((rows, ld), float("nan"), device="cuda")
        d_res = None
        if with_residual:
            d_out.copy_(torch.from_numpy(res))                             # residual aliased onto the output
            d_res = d_out
        free_before = torch.cuda.mem_get_info()[0]
        gemm_q4_static(engine, layer, which, d_a.data_ptr(), rows, d_res.data_ptr() if d_res is not None else 0, d_out.data_ptr())
        if pending:      # the first call on a device may load the module's code; no later call takes device memory
            assert torch.cuda.mem_get_info()[0] == free_before
        pending.append((d_out, d_a, want, reference, n))
    torch.cuda.synchronize()
    engine.static_status()       # no block gave up a wait
    for d_out, _, want, reference, n in pending:
        got = d_out.cpu().numpy()[:, :n]
        assert not np.isnan(got).any()
        # Same kernel, same cut of the work: the two entry points agree to the tolerance of the GEMM tests, and both with the oracle.
        assert np.abs(got - want).max() <= 4e-6 * np.abs(want).max()
        assert np.abs(got - reference).max() <= 8e-6 * np.abs(reference).max()


def test_static_scratch_gemm_at_the_limit_of_its_inner_dimension(oracle):
    """A contraction of 17,408 (the 27B shape's down projection) is the longest the array holds: accepted, and equal to the oracle."""
    import torch
    g = S.b27_geometry(layers=1, vocab=1024)
    engine = S.Engine(g, S.EngineConfig(max_slots=1, max_rows=8, kv_pages=1, max_context=256))
    model = oracle.Model(oracle.b27_geometry().with_(layers=1, vocab=1024))
    engine.load_model(model)
    packed, scales, biases = model.q4(0, "down")
    rng = np.random.default_rng(9)
    a = rng.normal(0, 1, (64, 17408)).astype(np.float32)
    want = oracle.gemm_q4(packed, scales, biases, a)
    d_a = torch.from_numpy(a).cuda()
    d_out = torch.full((64, 5120), float("nan"), device="cuda")
    gemm_q4_static(engine, 0, "down", d_a.data_ptr(), 64, 0, d_out.data_ptr())
    torch.cuda.synchronize()
    engine.static_status()
    assert np.abs(d_out.cpu().numpy() - want).max() <= 8e-6 * np.abs(want).max()


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
