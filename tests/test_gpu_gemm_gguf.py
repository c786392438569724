"""The GGUF K-quant dequant-GEMM through the C ABI (spl_op_gemm_gguf) against the CPU oracle on the same seeded blocks.

Both sides form each weight once in fp16 from one fp32 operation (fma(code, d * scale, -dmin * minimum), or
(code - 32) * (d * scale) for Q6_K: Sources/Shaders/gguf_formats.h:390-438) and multiply by bf16-rounded activations
with fp32 sums; they differ only in the order of the k fp32 additions, so |diff| <= 1e-6 * sqrt(k / 64) of the largest
output (4e-6 at k = 1024, 1.7e-5 at k = 17408). Blocks come from a
build-owned encoder (parity is defined on decoded values, so any valid encoding serves) and from raw random bytes with
finite d / dmin, which reach every code, scale and minimum value."""
import numpy as np
import pytest

import splosh_b200 as S
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def check(kind, blocks, rows, seed, residual=True):
    rng = np.random.default_rng(seed)
    n, k = blocks.shape[0], blocks.shape[1] * 256
    a = rng.normal(0, 1, (rows, k)).astype(np.float32)
    res = rng.normal(0, 1, (rows, n)).astype(np.float32) if residual else None
    want = O.gemm_gguf(kind, blocks, a, res)
    got = S.gemm_gguf(kind, blocks, a, res)
    assert not np.isnan(got).any()
    assert np.abs(got - want).max() <= 1e-6 * np.sqrt(k / 64) * max(np.abs(want).max(), 1.0), (kind, n, k, rows)


@pytest.mark.parametrize("kind", ["Q4_K", "Q5_K", "Q6_K"])
@pytest.mark.parametrize("rows", [1, 8, 17, 64, 70])
def test_encoded_weights_every_row_tier(kind, rows):
    rng = np.random.default_rng(11)
    w = rng.normal(0, 0.02, (384, 1024)).astype(np.float32)
    check(kind, O.quantize_gguf(kind, w), rows, seed=rows)


@pytest.mark.parametrize("kind", ["Q4_K", "Q5_K", "Q6_K"])
def test_random_blocks_reach_every_field_value(kind):
    rng = np.random.default_rng(5)
    n, supers, size = 200, 3, O.GGUF_BLOCK_BYTES[kind]
    raw = rng.integers(0, 256, (n, supers, size), dtype=np.uint8)
    # finite, modest fp16 d (and dmin): overwrite their bytes
    d = rng.uniform(1e-4, 2e-3, (n, supers)).astype(np.float16)
    if kind == "Q6_K":
        raw[:, :, 208:210] = d.view(np.uint8).reshape(n, supers, 2)
    else:
        raw[:, :, 0:2] = d.view(np.uint8).reshape(n, supers, 2)
        raw[:, :, 2:4] = rng.uniform(1e-4, 2e-3, (n, supers)).astype(np.float16).view(np.uint8).reshape(n, supers, 2)
    check(kind, raw, 16, seed=3)


@pytest.mark.parametrize("kind,n,k", [("Q5_K", 5120, 6144), ("Q5_K", 2048, 17408), ("Q6_K", 4096, 5120)])
def test_27b_inner_dimensions_and_split_contraction(kind, n, k):
    rng = np.random.default_rng(2)
    w = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    check(kind, O.quantize_gguf(kind, w), 64, seed=9, residual=False)
