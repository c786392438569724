"""The engine's primitives on device buffers: what the reference's drafter builds its passes from
(Sources/SploshRuntime/DraftModel.swift:344-357, 418-468: Engine.gemm / norm / mlpIn / embed on its own tensors, and the
target's lm_head). Each call against the oracle's (or numpy's) result on the same inputs."""
import numpy as np
import pytest
import torch

import splosh_b200 as S
from helpers import observed
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def bf16_round(x):
    return O.bf16_round(np.asarray(x, np.float32))


def bits_to_float(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


@pytest.fixture(scope="module")
def setup():
    g = S.tiny_geometry()
    model = O.Model(O.tiny_geometry())
    engine = S.Engine(g, S.EngineConfig(max_slots=1, max_rows=64, kv_pages=4, max_context=512))
    engine.load_model(model)
    return g, model, engine


def device(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def test_gemm_norm_and_mlp_in_on_a_tensor_of_the_callers(setup):
    g, model, engine = setup
    rng = np.random.default_rng(5)
    rows, inner, n = 24, 1024, 384
    w = (rng.standard_normal((n, inner)) * 0.02).astype(np.float32)
    wu = (rng.standard_normal((n, inner)) * 0.02).astype(np.float32)
    gate, up = O.quantize_mlx4(w), O.quantize_mlx4(wu)
    x = rng.standard_normal((rows, inner)).astype(np.float32)
    res = rng.standard_normal((rows, n)).astype(np.float32)
    norm_bits = (bf16_round(1.0 + 0.02 * rng.standard_normal(inner)).view(np.uint32) >> 16).astype(np.uint16)
    tg, tu, tn = engine.tensor_q4(*gate), engine.tensor_q4(*up), engine.tensor_vector(norm_bits)
    dx, dres = device(x), device(res)
    dout, dnorm = torch.empty((rows, n), device="cuda"), torch.empty((rows, inner), device="cuda")
    dact, dscratch = torch.empty((rows, n), device="cuda"), torch.empty((rows, n), device="cuda")
    engine.pass_begin()
    engine.pass_gemm(tg, dx.data_ptr(), rows, dout.data_ptr(), dres.data_ptr())
    engine.pass_norm(dx.data_ptr(), tn, rows, inner, dnorm.data_ptr())
    engine.pass_mlp_in(tg, tu, dx.data_ptr(), rows, dact.data_ptr(), dscratch.data_ptr())
    engine.pass_wait()
    want = O.gemm_q4(*gate, x, res)
    got = dout.cpu().numpy()
    scale = np.abs(want).max()
    observed(f"primitive GEMM with residual: max difference {np.abs(got - want).max() / scale:.2e} of the largest output")
    assert np.abs(got - want).max() <= 2e-5 * scale
    inv = 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + g.eps)
    want_norm = (x * inv * bits_to_float(norm_bits)).astype(np.float32)
    assert np.abs(dnorm.cpu().numpy() - want_norm).max() <= 1e-5 * np.abs(want_norm).max()
    gx, ux = O.gemm_q4(*gate, x), O.gemm_q4(*up, x)
    want_act = bf16_round(gx / (1.0 + np.exp(-gx)) * ux)
    got_act = dact.cpu().numpy()
    # bf16 results: equal except where the two sides' sums straddle a rounding boundary (one bf16 step)
    assert np.abs(got_act - want_act).max() <= 2.0 ** -7 * max(np.abs(want_act).max(), 1e-6)
    assert (got_act == want_act).mean() > 0.99
    for t in (tg, tu, tn):
        engine.tensor_destroy(t)


def test_embedding_rows_and_the_targets_head(setup):
    g, model, engine = setup
    rng = np.random.default_rng(6)
    rows = 12
    tokens = rng.integers(0, g.vocab, rows).astype(np.uint32)
    dtok = device(tokens)
    demb, dlogits = torch.empty((rows, g.hidden), device="cuda"), torch.empty((rows, g.vocab), device="cuda")
    engine.pass_begin()
    engine.pass_embed(dtok.data_ptr(), rows, demb.data_ptr())
    engine.pass_gemm_head(demb.data_ptr(), rows, dlogits.data_ptr())
    engine.pass_wait()
    packed, scales, biases = model.q4(-1, "embed")
    table = O.dequant_mlx4(packed[tokens], bits_to_float(scales[tokens]), bits_to_float(biases[tokens]), g.hidden)
    assert np.array_equal(demb.cpu().numpy(), table)          # scale * nibble + bias, one fp32 multiply-add each
    want = O.gemm_q4(*model.q4(-1, "head"), table)
    got = dlogits.cpu().numpy()
    assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()
    observed(f"primitive head GEMM on embedding rows: max difference {np.abs(got - want).max() / np.abs(want).max():.2e} of the largest logit")


def test_the_primitives_refuse_what_they_cannot_hold(setup):
    g, model, engine = setup
    rng = np.random.default_rng(7)
    w = O.quantize_mlx4((rng.standard_normal((32, 4096)) * 0.02).astype(np.float32))
    with pytest.raises(S.EngineError):
        engine.tensor_q4(*w)                                 # inner dimension beyond the engine's MLP width (2,816)
    t = engine.tensor_q4(*O.quantize_mlx4((rng.standard_normal((32, 512)) * 0.02).astype(np.float32)))
    x = torch.zeros((80, 512), device="cuda"); out = torch.zeros((80, 32), device="cuda")
    with pytest.raises(S.EngineError):
        engine.pass_gemm(t, x.data_ptr(), 80, out.data_ptr())      # more rows than the engine's max_rows
    engine.tensor_destroy(t)
