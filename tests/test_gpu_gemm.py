"""The MLX affine-4 dequant-GEMM through the C ABI (spl_op_gemm_q4, host buffers in and out)
against the CPU oracle on the same seeded inputs.

Tolerance: both sides form, per 64-group, the exact dot of bf16 activations with 4-bit codes and
add dot * scale + sum * bias; they differ only in fp32 summation order (the kernel keeps one running
accumulator per issuing warp over all of a split's groups), so |diff| <= 8e-6 of the
largest output (the reference allows relErr 1e-2 for its kernel, GemmOracleTests.swift:165)."""
import numpy as np
import pytest

import splosh_b200 as S

pytestmark = pytest.mark.gpu
TOL = 8e-6


def case(oracle, n, k, rows, seed, residual=True):
    rng = np.random.default_rng(seed)
    w = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    packed, scales, biases = oracle.quantize_mlx4(w)
    a = rng.normal(0, 1, (rows, k)).astype(np.float32)
    res = rng.normal(0, 1, (rows, n)).astype(np.float32) if residual else None
    want = oracle.gemm_q4(packed, scales, biases, a, res)
    got = S.gemm_q4(packed, scales, biases, a, res)
    assert not np.isnan(got).any()
    assert np.abs(got - want).max() <= TOL * np.abs(want).max(), (n, k, rows)


@pytest.mark.parametrize("rows", [1, 2, 3, 7, 8, 9, 16, 17, 31, 33, 48, 64, 65, 127, 130])
def test_every_row_tier_and_ragged_row_counts(oracle, rows):
    case(oracle, 1024, 1024, rows, rows)


@pytest.mark.parametrize("n,k", [(48, 1024), (8, 1024), (16, 256), (3104, 1024), (5632, 1024), (1024, 2816), (24, 5120), (1000, 512)])
def test_output_widths_that_do_not_fill_a_tile(oracle, n, k):
    """48- and 8-row projections (the a and b projections), widths that are not a multiple of 16."""
    case(oracle, n, k, 20, n + k, residual=n % 2 == 0)


@pytest.mark.parametrize("pair", [True, False])
@pytest.mark.parametrize("n,k,rows", [(3104, 1024, 300), (1024, 2816, 129), (5632, 1024, 257), (48, 1024, 200), (5120, 6144, 128), (2176, 5120, 520)])
def test_the_two_128_row_blocks(oracle, pair, n, k, rows):
    """Steps of more than 64 rows: the pair form (two tiles of the weight a block: an odd tile count, 25, whose last pair does
    its one tile twice; one row block with the contraction cut; several row blocks) and, with the switch off, the block of
    one tile."""
    S.engine.debug_pair_blocks(pair)
    try:
        case(oracle, n, k, rows, 1000 + rows)
    finally:
        S.engine.debug_pair_blocks(True)


@pytest.mark.parametrize("k", [256, 768, 1280, 2304])
@pytest.mark.parametrize("rows", [5, 64])
def test_short_contractions_with_odd_stage_counts(oracle, k, rows):
    """One, three, five and nine shared-memory stages of four groups (inner dimensions are multiples of 256): fewer
    stages than the rings hold, and counts that leave the rings' slots at every phase."""
    case(oracle, 384, k, rows, 100 + k)


@pytest.mark.parametrize("n,k", [(17408, 5120), (5120, 17408), (10240, 5120), (5120, 6144)])
def test_27b_shapes_at_64_rows(oracle, n, k):
    case(oracle, n, k, 64, 7)


def test_linearity_at_full_size(oracle):
    """A size-independent property: GEMM(a1 + a2) = GEMM(a1) + GEMM(a2) for activations exactly representable in bf16."""
    rng = np.random.default_rng(11)
    n, k, rows = 34816, 5120, 64
    packed = rng.integers(0, 2 ** 32, (n, k // 8), dtype=np.uint64).astype(np.uint32)
    scales = np.full((n, k // 64), 0x3C00, np.uint16)       # bf16 2^-7
    biases = np.full((n, k // 64), 0xBD80, np.uint16)       # bf16 -2^-4
    a1 = rng.integers(-8, 9, (rows, k)).astype(np.float32); a2 = rng.integers(-8, 9, (rows, k)).astype(np.float32)
    y1, y2, y12 = (S.gemm_q4(packed, scales, biases, a) for a in (a1, a2, a1 + a2))
    assert np.abs(y12 - (y1 + y2)).max() <= 1e-5 * np.abs(y12).max()


def test_zero_rows_and_bad_shapes_are_rejected():
    z16 = np.zeros((16, 32), np.uint32); s = np.zeros((16, 4), np.uint16)
    with pytest.raises(S.EngineError):
        S.gemm_q4(z16, s, s, np.zeros((0, 256), np.float32))
    with pytest.raises(S.EngineError):
        S.gemm_q4(np.zeros((16, 8), np.uint32), np.zeros((16, 1), np.uint16), np.zeros((16, 1), np.uint16), np.zeros((1, 64), np.float32))


def test_weights_the_tensor_cores_cannot_hold_exactly_are_refused():
    """scale * (code - 8), 512 * scale and 64 * bias must be exact in fp16: a scale of 200, a scale of 2^-20 or a bias of
    2,048 is refused when the weight is loaded, never approximated; zero scales and the largest allowed values pass."""
    packed = np.zeros((128, 32), np.uint32); a = np.ones((4, 256), np.float32)
    def run(scale_bits, bias_bits):
        return S.gemm_q4(packed, np.full((128, 4), scale_bits, np.uint16), np.full((128, 4), bias_bits, np.uint16), a)
    for scale_bits, bias_bits in ((0x4348, 0x0000), (0x3580, 0x0000), (0x3C00, 0x4500)):      # 200.0; 2^-20; bias 2,048
        with pytest.raises(S.EngineError) as caught:
            run(scale_bits, bias_bits)
        assert caught.value.case == "invalidArgument"
    out = run(0x42FE, 0xC47F)            # scale 127, bias -1,020: codes are 0, so every output is 256 * bias
    assert np.array_equal(out, np.full((4, 128), -1020.0 * 256, np.float32))
    assert np.array_equal(run(0x0000, 0x3F80), np.full((4, 128), 256.0, np.float32))      # zero scale, bias 1
