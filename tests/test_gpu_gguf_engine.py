"""A GGUF-weighted engine (the GGUF branch of Engine.gemm, Sources/SploshRuntime/Engine.swift:1666-1695, over tensors as
Sources/SploshModel/GgufConvert.swift leaves them: Q5_K blocks, Q6_K embedding and head): the packed step through the C ABI
against the CPU oracle holding the same blocks. The oracle forms weights as the reference's tile kernels do (one fp32
operation, rounded to fp16, Sources/Shaders/gguf_formats.h:390-438), decodes the embedding exactly (:463-501) and runs
plain norms (the GGUF GEMM has no deferred form), which is the contract of the CUDA path."""
import numpy as np
import pytest

from helpers import Pair, tokens_for, observed
import splosh_b200 as S
import oracle.oracle as O

pytestmark = pytest.mark.gpu

LOGIT_TOL = 3e-2      # the MLX-weighted step's tolerance (tests/test_gpu_step.py)


def geometry():
    # hidden, inter, the mixers' inner dimensions: multiples of 256 (a K-quant super-block)
    return S.Geometry(4, 256, 512, 2048, 8, 2, 128, 32, 2, 4, 128, 1e-6, 1e7)


@pytest.fixture(scope="module")
def plain_norms():
    O.set_norm_contract(False)
    yield
    O.set_norm_contract(True)


@pytest.mark.parametrize("kinds", [("Q5_K", "Q6_K"), ("Q4_K", "Q6_K"), ("Q6_K", "Q4_K")])
def test_gguf_weighted_step_matches_the_oracle(plain_norms, kinds):
    """A prompt chunk, a second chunk, then verify blocks on two sessions with a partial acceptance: logits and arg-max."""
    g = geometry()
    cfg = S.EngineConfig(max_slots=2, max_rows=64, kv_pages=8, max_context=1024)
    pair = Pair(g, cfg, gguf=kinds)
    toks = tokens_for(0xC0FFEE00, 400, g.vocab)
    steps = [
        [S.EngineRow(0, toks[i], i, i == 39) for i in range(40)],
        [S.EngineRow(1, toks[100 + i], i, i == 23) for i in range(24)] + [S.EngineRow(0, toks[40 + i], 40 + i, True, True) for i in range(8)],
    ]
    worst = 0.0
    for rows in steps:
        glogits, ologits = pair.step(rows)
        diff = np.abs(glogits - ologits).max()
        worst = max(worst, diff)
        assert diff < LOGIT_TOL * max(1.0, np.abs(ologits).max())
        # The arg-max may differ only where the oracle's own leaders are closer than the tolerance.
        for r in np.nonzero(np.argmax(glogits, axis=1) != np.argmax(ologits, axis=1))[0]:
            assert ologits[r].max() - ologits[r, np.argmax(glogits[r])] < 2 * LOGIT_TOL
    pair.accept(0, 5, 45)
    rows = [S.EngineRow(0, toks[45 + i], 45 + i, True, True) for i in range(8)] + [S.EngineRow(1, toks[124 + i], 24 + i, True, True) for i in range(4)]
    glogits, ologits = pair.step(rows)
    worst = max(worst, np.abs(glogits - ologits).max())
    assert np.abs(glogits - ologits).max() < LOGIT_TOL * max(1.0, np.abs(ologits).max())
    observed(f"GGUF-weighted step ({kinds[0]} blocks, {kinds[1]} embedding and head): max |logit - oracle| {worst:.3e} (<= {LOGIT_TOL})")


def test_a_partly_converted_engine_refuses_to_step(plain_norms):
    g = geometry()
    cfg = S.EngineConfig(max_slots=1, max_rows=16, kv_pages=4, max_context=512)
    pair = Pair(g, cfg, gguf=("Q5_K", "Q6_K"), gpu=False)
    engine = S.Engine(g, cfg)
    engine.load_model(pair.model)                       # MLX tensors and vectors
    engine.set_gguf(-1, "head", *pair.model.gguf(-1, "head"))
    with pytest.raises(S.EngineError):
        engine.step([S.EngineRow(0, 5, 0, True)])
    with pytest.raises(S.EngineError):                  # q and qkv, z, a, b share a device tensor: one type
        engine.set_gguf(0, "qkv", *pair.model.gguf(0, "qkv"))
        kind, blocks = pair.model.gguf(0, "z")
        engine.set_gguf(0, "z", "Q4_K", O.quantize_gguf("Q4_K", np.zeros((blocks.shape[0], blocks.shape[1] * 256), np.float32)))


def test_a_gguf_file_loads_into_the_engine(plain_norms, tmp_path):
    """The synthetic GGUF-weighted model written as a llama.cpp GGUF file (value heads in the file's order, -exp(A_log), fp32
    norms, an MTP block and metadata to skip; tests/gguf_writer.py) and read back by spl_weights_load_gguf_file: the step
    equals, bit for bit, that of an engine given the same tensors one by one, and matches the oracle that holds the out
    projections in file order (Sources/SploshModel/GgufNames.swift:73-84, GgufConvert.swift:15-32)."""
    import gguf_writer
    g = geometry()
    cfg = S.EngineConfig(max_slots=2, max_rows=64, kv_pages=8, max_context=1024)
    pair = Pair(g, cfg, gguf=("Q5_K", "Q6_K"))
    pair.model.set_out_file_order(True)
    pair.engine.gguf_file_order(True)
    path = str(tmp_path / "model.gguf")
    gguf_writer.write(path, g, pair.model)
    loaded = S.Engine(g, cfg)
    loaded.load_gguf_file(path)
    toks = tokens_for(0xC0FFEE00, 200, g.vocab)
    for rows in ([S.EngineRow(0, toks[i], i, i % 7 == 0) for i in range(40)],
                 [S.EngineRow(0, toks[40 + i], 40 + i, True, True) for i in range(8)]):
        glogits, ologits = pair.step(rows)
        loaded.step(rows)
        assert np.array_equal(loaded.all_logits(), glogits)
        assert np.abs(glogits - ologits).max() < LOGIT_TOL * max(1.0, np.abs(ologits).max())
    # The head order matters: the same file with the switch off gives something else.
    loaded.gguf_file_order(False)
    loaded.reset_slot(0)
    loaded.step([S.EngineRow(0, toks[i], i, i % 7 == 0) for i in range(40)])
    pair2 = Pair(g, cfg, gguf=("Q5_K", "Q6_K"), gpu=False)
    pair2.model.set_out_file_order(True)
    _, ref = pair2.step([S.EngineRow(0, toks[i], i, i % 7 == 0) for i in range(40)])
    assert np.abs(loaded.all_logits() - ref).max() > LOGIT_TOL


def test_a_broken_gguf_file_is_refused_with_a_message(tmp_path):
    import gguf_writer
    g = geometry()
    cfg = S.EngineConfig(max_slots=1, max_rows=16, kv_pages=4, max_context=512)
    from helpers import to_oracle_geometry
    model = O.Model(to_oracle_geometry(g)).to_gguf("Q5_K", "Q6_K")
    path = str(tmp_path / "model.gguf")
    gguf_writer.write(path, g, model)
    raw = open(path, "rb").read()
    engine = S.Engine(g, cfg)
    cut = str(tmp_path / "cut.gguf"); open(cut, "wb").write(raw[: len(raw) // 2])
    with pytest.raises(S.EngineError, match="outside the file"):
        engine.load_gguf_file(cut)
    bad = str(tmp_path / "bad.gguf"); open(bad, "wb").write(b"GGUX" + raw[4:])
    with pytest.raises(S.EngineError, match="not a GGUF file"):
        engine.load_gguf_file(bad)
    other = S.Engine(S.tiny_geometry(), cfg)
    with pytest.raises(S.EngineError, match="shape|elements"):
        other.load_gguf_file(path)
