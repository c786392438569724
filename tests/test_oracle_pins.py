"""Pins of the CPU oracle against the reference's own golden vectors and known-answer tests.

Every case names the reference test it restates. Golden data comes from tests/golden/ (made by
tests/golden/make_golden.py from the reference checkout)."""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(HERE, "golden", "gguf_golden_blocks.json")) as f:
        return json.load(f)


@pytest.mark.parametrize("kind", ["Q4_K", "Q5_K", "Q6_K"])
def test_gguf_real_block_decodes_to_reference_values(oracle, golden, kind):
    """GgufTests.swift:237 'A real block of each quantised format decodes to the reference values':
    relative error <= 1e-6 per element, and two blocks decode one after the other."""
    raw = np.array(golden[kind]["bytes"], np.uint8)[None, :]
    want = np.array(golden[kind]["values"], np.float32)
    got = oracle.decode_gguf(kind, raw)[0]
    assert got.shape == want.shape == (256,)
    assert np.all(np.abs(got - want) <= 1e-6 * np.abs(want))
    twice = oracle.decode_gguf(kind, np.concatenate([raw, raw]))
    assert np.array_equal(twice[0], got) and np.array_equal(twice[1], got)


@pytest.mark.parametrize("kind", ["Q4_K", "Q5_K", "Q6_K"])
def test_gguf_random_blocks_match_reference_numpy_decoder(oracle, kind):
    """Seeded random blocks decoded by the reference's tools/gguf_check.py `decode` (run in the
    build container; outputs stored): bit-exact."""
    data = np.load(os.path.join(HERE, "golden", "gguf_check_vectors.npz"))
    got = oracle.decode_gguf(kind, data[kind + "_raw"])
    assert np.array_equal(got, data[kind + "_values"])


def test_q4k_packed_scale_contract(oracle):
    """QuantDequantOracleTests.swift:19-31: d = 1, dmin = 1, every group scale 1 and minimum 0,
    payload bytes 0x10 -> low nibbles 0 in even groups, high nibbles 1 in odd groups."""
    block = bytes([0x00, 0x3c, 0x00, 0x00]) + bytes([1] * 8 + [0] * 4) + bytes([0x10] * 128)
    values = oracle.decode_gguf("Q4_K", np.frombuffer(block, np.uint8)[None, :])[0]
    assert values[0] == 0 and values[1] == 0 and values[31] == 0
    assert values[32] == 1 and values[63] == 1


def test_mlx_affine_group64_contract(oracle):
    """QuantDequantOracleTests.swift:33-50: 65 columns, low-first nibbles c % 16, scales [2, 3],
    biases [-1, 10]: value = scale * nibble + bias with the group changing at column 64."""
    columns = 65
    words = np.zeros((1, 9), np.uint32)
    for c in range(columns):
        words[0, c // 8] |= np.uint32((c % 16) << ((c % 8) * 4))
    got = oracle.dequant_mlx4(words, np.array([[2, 3]], np.float32), np.array([[-1, 10]], np.float32), columns)[0]
    want = np.array([(2 if c < 64 else 3) * (c % 16) + (-1 if c < 64 else 10) for c in range(columns)], np.float32)
    assert np.array_equal(got, want)


def test_mlx_affine_partial_columns_second_row(oracle):
    """Q4BufferLayoutTests.swift:8-31: two rows of 65 columns with nibble (k + row) & 15, scales
    2 + i and biases -i per sidecar: row 0 k 0 -> 0, row 0 k 64 -> -1, row 1 k 64 -> 2."""
    words = np.zeros((2, 9), np.uint32)
    for row in range(2):
        for k in range(65):
            words[row, k // 8] |= np.uint32(((k + row) & 15) << ((k % 8) * 4))
    scales = np.array([[2, 3], [4, 5]], np.float32); biases = np.array([[0, -1], [-2, -3]], np.float32)
    got = oracle.dequant_mlx4(words, scales, biases, 65)
    assert got[0, 0] == 0 and got[0, 64] == -1 and got[1, 64] == 2


def test_bf16_rounding_is_nearest_even(oracle):
    """DraftModel.swift:721-724 / SwigluOracle.swift:33-44: round to nearest, ties to even."""
    lib = oracle.lib()
    assert lib.orc_bf16(1.0) == 0x3F80
    assert lib.orc_bf16(float(np.float32(1.0) + np.float32(2.0 ** -8))) == 0x3F80      # tie, even stays
    assert lib.orc_bf16(float(np.float32(1.0) + np.float32(3 * 2.0 ** -8))) == 0x3F82  # tie, rounds up to even
    x = np.array([0.1, -2.7, 3.3e-5, 1e20], np.float32)
    assert np.array_equal(oracle.bf16_round(x), np.array([oracle.bf16_bits_to_float([lib.orc_bf16(float(v))])[0] for v in x], np.float32))


def test_gdn_decode_order_hand_case(oracle):
    """GdnOracleTests.swift:7-12 'decay, delta write, then read': q = k = [1, 0], v = [2, 3],
    beta 1, log-decay 0 -> output [2, 3], state [2, 3, 0, 0]."""
    import ctypes as C
    state = np.zeros(4, np.float32); out = np.zeros(2, np.float32)
    f = lambda a: np.array(a, np.float32)
    q, k, v, b, d = f([1, 0]), f([1, 0]), f([2, 3]), f([1]), f([0])
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    oracle.lib().orc_gdn_decode(p(q), p(k), p(v), p(b), p(d), 1, 2, 2, p(state), p(out))
    assert out.tolist() == [2, 3] and state.tolist() == [2, 3, 0, 0]


def test_gdn_recurrence_carries_state(oracle):
    """GdnOracleTests.swift:14-22: second token with beta 0.5 on the carried state: output[0] = 2
    at token 0 and 3 at token 1."""
    import ctypes as C
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    f = lambda a: np.array(a, np.float32)
    state = np.zeros(4, np.float32)
    outs = []
    for v, beta in (([2, 3], 1.0), ([4, 5], 0.5)):
        out = np.zeros(2, np.float32)
        oracle.lib().orc_gdn_decode(p(f([1, 0])), p(f([1, 0])), p(f(v)), p(f([beta])), p(f([0])), 1, 2, 2, p(state), p(out))
        outs.append(out.copy())
    assert abs(outs[0][0] - 2) < 1e-6 and abs(outs[1][0] - 3) < 1e-6


def test_engine_form_of_the_update_equals_the_per_op_oracle(oracle):
    """The engine folds the key's inverse norm into raw k (engine.metal:774-786); the per-op oracle
    takes a normalised key and log-decay (GdnOracle.swift:44-64). On the 512-token generator of
    GdnPrefillChunkTests.swift:9-18 (widened to 128 dims) both leave the same state and output."""
    import ctypes as C
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    d = 128
    rng = np.random.default_rng(3)
    s_engine = rng.uniform(-0.5, 0.5, (d, d)).astype(np.float32)         # [value j][key i]
    s_oracle = np.ascontiguousarray(s_engine.T.copy())[None]             # [head][key][value]
    for t in range(64):
        q = rng.uniform(-1, 1, d).astype(np.float32); k = rng.uniform(-1, 1, d).astype(np.float32); v = rng.uniform(-1, 1, d).astype(np.float32)
        beta = np.float32(0.25 + 0.1 * (t % 4)); log_decay = np.float32(-0.01 * (t % 3))
        inv_k = np.float32(1.0 / np.sqrt(float((k.astype(np.float64) ** 2).sum()) + 1e-6)); inv_q = np.float32(1.0 / np.sqrt(float((q.astype(np.float64) ** 2).sum()) + 1e-6))
        out_e = np.zeros(d, np.float32); out_o = np.zeros(d, np.float32)
        oracle.lib().orc_gdn_engine_update(p(q), p(k), p(v), C.c_float(beta), C.c_float(np.exp(log_decay)), C.c_float(inv_q), C.c_float(inv_k), d, p(s_engine), p(out_e))
        kn = (k * inv_k).astype(np.float32); qn = (q * inv_q).astype(np.float32)
        oracle.lib().orc_gdn_decode(p(qn), p(kn), p(v), p(np.array([beta], np.float32)), p(np.array([log_decay], np.float32)), 1, d, d, p(s_oracle), p(out_o))
        assert np.abs(out_e - out_o).max() <= 2e-4 * max(1.0, np.abs(out_o).max())
    assert np.abs(s_engine - s_oracle[0].T).max() <= 2e-4 * np.abs(s_engine).max()


def test_rope_partial_dims_neox_pairing(oracle):
    """RopeOracleTests.swift:58-65 and RopeOracle.swift:15-56 for text (one position id): only the
    first 64 of 256 dims rotate; out[i] = x[i] cos - x[i+32] sin, out[i+32] = x[i+32] cos + x[i] sin
    with angle = pos * theta^(-2i/64)."""
    import ctypes as C
    x = np.array([(i + 1) / 17 for i in range(256)], np.float32)
    out = np.zeros(256, np.float32)
    oracle.lib().orc_rope(x.ctypes.data_as(C.c_void_p), 256, 64, C.c_float(1e7), 3, out.ctypes.data_as(C.c_void_p))
    assert np.array_equal(out[64:], x[64:]) and not np.array_equal(out[:64], x[:64])
    for i in range(32):
        angle = 3.0 * (1e7 ** (-2.0 * i / 64))
        assert abs(out[i] - (x[i] * np.cos(angle) - x[i + 32] * np.sin(angle))) < 1e-5
        assert abs(out[i + 32] - (x[i + 32] * np.cos(angle) + x[i] * np.sin(angle))) < 1e-5


def test_swiglu_bf16_contract(oracle):
    """SwigluOracle.swift:14-29: bf16 in, fp32 silu(gate) * up, bf16 out (nearest even)."""
    import ctypes as C
    lib = oracle.lib()
    gate = np.array([lib.orc_bf16(v) for v in (-3.0, -0.5, 0.0, 0.75, 2.0, 8.0)], np.uint16)
    up = np.array([lib.orc_bf16(v) for v in (1.5, -2.0, 4.0, 0.3, -1.25, 0.01)], np.uint16)
    out = np.zeros(6, np.uint16)
    lib.orc_swiglu_bf16(gate.ctypes.data_as(C.c_void_p), up.ctypes.data_as(C.c_void_p), 6, out.ctypes.data_as(C.c_void_p))
    g = oracle.bf16_bits_to_float(gate).astype(np.float64); u = oracle.bf16_bits_to_float(up).astype(np.float64)
    want = oracle.bf16_round((g / (1 + np.exp(-g)) * u).astype(np.float32))
    assert np.allclose(oracle.bf16_bits_to_float(out), want, rtol=2.0 ** -7, atol=0)


def test_argmax_is_first_maximum_under_the_vocab_limit(oracle):
    """Sampler.swift:11-16 (vDSP_maxvi: first index of the maximum) and :94-96 (ids past the
    tokenizer's limit are never chosen)."""
    logits = np.array([[0.5, 2.0, 2.0, 1.0, 9.0]], np.float32)
    assert oracle.argmax(logits, 5)[0] == 4
    assert oracle.argmax(logits, 4)[0] == 1


def test_quantiser_rule(oracle):
    """DraftModel.swift:634-670 'minmax': scale = bf16((max - min) / 15), bias = bf16(min), codes
    rounded against the stored parameters; a flat group takes scale 1."""
    rng = np.random.default_rng(0)
    w = rng.normal(0, 0.02, (3, 128)).astype(np.float32)
    w[2, 64:] = 0.125
    packed, scales, biases = oracle.quantize_mlx4(w)
    s = oracle.bf16_bits_to_float(scales); b = oracle.bf16_bits_to_float(biases)
    for r in range(3):
        for g in range(2):
            grp = w[r, g * 64:(g + 1) * 64]
            if grp.max() > grp.min():
                assert s[r, g] == oracle.bf16_round(np.array([(grp.max() - grp.min()) / np.float32(15)], np.float32))[0]
            else:
                assert s[r, g] == 1.0
            assert b[r, g] == oracle.bf16_round(np.array([grp.min()], np.float32))[0]
    deq = oracle.dequant_mlx4(packed, s, b, 128)
    assert np.abs(deq[:2] - w[:2]).max() <= 0.51 * s[:2].max() + 2.0 ** -8 * np.abs(w).max()
    assert np.all(deq[2, 64:] == 0.125)


@pytest.mark.parametrize("kind", ["Q4_K", "Q5_K", "Q6_K"])
def test_gguf_tile_weights_are_the_decoded_values_within_one_fp16_step(oracle, golden, kind):
    """The tile kernels' weights (one fp32 operation, then fp16: gguf_formats.h:390-438) against the exact decode on the
    reference's golden blocks: the reference's own bound is one fp16 unit in the last place (GgufKernelTests.swift:207)."""
    raw = np.array(golden[kind]["bytes"], np.uint8)[None, :]
    exact = oracle.decode_gguf(kind, raw)[0]
    tile = oracle.gguf_tile_weights(kind, raw)[0]
    assert np.array_equal(tile.astype(np.float16).astype(np.float32), tile)          # fp16-representable
    ulp = np.spacing(np.abs(exact).astype(np.float16)).astype(np.float32)
    assert np.all(np.abs(tile - exact) <= ulp)


def test_gguf_gemm_is_the_tile_weights_times_rounded_activations(oracle):
    rng = np.random.default_rng(0)
    for kind in ("Q4_K", "Q5_K", "Q6_K"):
        blocks = oracle.quantize_gguf(kind, rng.normal(0, 0.02, (24, 512)).astype(np.float32))
        a = rng.normal(0, 1, (5, 512)).astype(np.float32); res = rng.normal(0, 1, (5, 24)).astype(np.float32)
        w = oracle.gguf_tile_weights(kind, blocks.reshape(-1, blocks.shape[2])).reshape(24, 512).astype(np.float64)
        want = oracle.bf16_round(a).astype(np.float64) @ w.T + res
        got = oracle.gemm_gguf(kind, blocks, a, res)
        assert np.abs(got - want).max() <= 2e-6 * np.abs(want).max()
        # the encoder makes blocks that decode close to what went in
        assert np.abs(w).max() > 0
