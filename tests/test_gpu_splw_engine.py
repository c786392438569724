"""An SPLW artifact into the engine (spl_weights_load_splw_file: the reference's WeightFile + ModelWeights.resolve,
Sources/SploshModel/WeightFile.swift:88-141, ModelWeights.swift:181-248, with the tiled layout of Retile.swift put back in
rows): the step of an engine loaded from the file equals, bit for bit, that of an engine given the same tensors one by one,
for the row-major and for the tiled artifact."""
import numpy as np
import pytest

from helpers import Pair, tokens_for, observed
import splosh_b200 as S
import splw_writer

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tiled", [False, True])
def test_an_splw_artifact_loads_into_the_engine(tiled, tmp_path):
    g = S.tiny_geometry()
    cfg = S.EngineConfig(max_slots=2, max_rows=64, kv_pages=8, max_context=1024)
    pair = Pair(g, cfg)
    path = str(tmp_path / "model.splw")
    header = splw_writer.write(path, g, pair.model, tiled=tiled)
    loaded = S.Engine(g, cfg)
    loaded.load_splw_file(path)
    toks = tokens_for(0xC0FFEE00, 200, g.vocab)
    worst = 0.0
    for rows in ([S.EngineRow(0, toks[i], i, i % 7 == 0) for i in range(40)],
                 [S.EngineRow(0, toks[40 + i], 40 + i, True, True) for i in range(8)] + [S.EngineRow(1, toks[100 + i], i, i == 11) for i in range(12)]):
        glogits, ologits = pair.step(rows)
        loaded.step(rows)
        assert np.array_equal(loaded.all_logits(), glogits)
        worst = max(worst, np.abs(glogits - ologits).max())
    observed(f"SPLW artifact ({header['format']}, {len(header['tensorRecords'])} records): the loaded engine's logits are the tensor-by-tensor engine's; max |logit - oracle| {worst:.3e}")


def test_artifacts_the_engine_cannot_take_are_refused_with_a_message(tmp_path):
    g = S.tiny_geometry()
    cfg = S.EngineConfig(max_slots=1, max_rows=16, kv_pages=4, max_context=512)
    import oracle.oracle as O
    from helpers import to_oracle_geometry
    model = O.Model(to_oracle_geometry(g), 0x5EED6D17)
    engine = S.Engine(g, cfg)
    path = str(tmp_path / "m.splw")
    splw_writer.write(path, g, model, bits=8)
    with pytest.raises(S.EngineError, match="mlxAffine8 is not mlxAffine4"):
        engine.load_splw_file(path)

    splw_writer.write(path, g, model)
    raw = open(path, "rb").read()
    with pytest.raises(S.EngineError, match="shape"):
        S.Engine(S.Geometry(4, 256, 512, 2048, 8, 2, 128, 32, 2, 4, 128, 1e-6, 1e7), cfg).load_splw_file(path)
    with pytest.raises(S.EngineError, match="truncated framing|weight file invalid"):
        cut = str(tmp_path / "cut.splw"); open(cut, "wb").write(raw[:8])
        engine.load_splw_file(cut)
    # A tensor the model needs under another name: the loader says which one is missing.
    import struct
    length = struct.unpack("<Q", raw[8:16])[0]
    renamed = raw[:16] + raw[16:16 + length].replace(b"layers.1.mlp.down_proj.weight", b"layers.1.mlp.down_proj.weighs") + raw[16 + length:]
    other = str(tmp_path / "renamed.splw"); open(other, "wb").write(renamed)
    with pytest.raises(S.EngineError, match="missing tensor language_model.model.layers.1.mlp.down_proj.weight"):
        engine.load_splw_file(other)


def test_a_gguf_derived_artifact_loads_into_the_engine(tmp_path):
    """The artifact the reference's GGUF converter leaves (format gguf.tiled128: every 2-D weight as the three planes of
    Sources/SploshModel/GgufPlanes.swift, padded to whole tiles; the out projections in the file's order of the value heads,
    Sources/SploshModel/GgufConvert.swift:1-33): the loaded engine steps bit for bit like one given the native blocks tensor by
    tensor with the file order switched on, and matches the oracle that holds the same blocks."""
    import oracle.oracle as O
    O.set_norm_contract(False)
    try:
        g = S.Geometry(4, 256, 512, 2048, 8, 2, 128, 32, 2, 4, 128, 1e-6, 1e7)
        cfg = S.EngineConfig(max_slots=2, max_rows=64, kv_pages=8, max_context=1024)
        pair = Pair(g, cfg, gguf=("Q5_K", "Q6_K"))
        pair.model.set_out_file_order(True)
        pair.engine.gguf_file_order(True)
        path = str(tmp_path / "model.splw")
        header = splw_writer.write_gguf_derived(path, g, pair.model)
        assert S.engine.splw_check(path) == ("gguf.tiled128", len(header["tensorRecords"]))
        loaded = S.Engine(g, cfg)
        loaded.load_splw_file(path)
        toks = tokens_for(0xC0FFEE00, 200, g.vocab)
        worst = 0.0
        for rows in ([S.EngineRow(0, toks[i], i, i % 7 == 0) for i in range(40)],
                     [S.EngineRow(0, toks[40 + i], 40 + i, True, True) for i in range(8)]):
            glogits, ologits = pair.step(rows)
            loaded.step(rows)
            assert np.array_equal(loaded.all_logits(), glogits)
            worst = max(worst, np.abs(glogits - ologits).max())
            assert np.abs(glogits - ologits).max() < 3e-2 * max(1.0, np.abs(ologits).max())
        observed(f"GGUF-derived SPLW artifact ({len(header['tensorRecords'])} records, Q5_K planes, Q6_K embedding and head): loaded engine = block-by-block engine; max |logit - oracle| {worst:.3e}")
    finally:
        O.set_norm_contract(True)
