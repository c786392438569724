"""The SPLW container's checks (Sources/SploshModel/WeightFile.swift:88-141) as spl_splw_check restates them: a file the
tests' writer produces the way the reference's converter does (Sources/SploshModel/Converter.swift:160-228) is accepted, and
each way the reference refuses a file is refused with the reference's reason. No GPU: the check needs no engine."""
import json
import struct

import numpy as np
import pytest

import splosh_b200 as S
import oracle.oracle as O
from helpers import to_oracle_geometry
import splw_writer


@pytest.fixture(scope="module")
def model():
    g = S.tiny_geometry()
    return g, O.Model(to_oracle_geometry(g), 0x5EED6D17)


def test_a_converted_artifact_passes_the_container_checks(model, tmp_path):
    g, m = model
    for tiled in (False, True):
        path = str(tmp_path / ("tiled.splw" if tiled else "rows.splw"))
        header = splw_writer.write(path, g, m, tiled=tiled)
        fmt, count = S.engine.splw_check(path)
        assert fmt == ("mlxAffine4.tiled128" if tiled else "mlxAffine4")
        assert count == len(header["tensorRecords"])
        # The framing says what the header says.
        raw = open(path, "rb").read()
        length = struct.unpack("<Q", raw[8:16])[0]
        assert json.loads(raw[16:16 + length])["headerLength"] == length
    # The tiled artifact is the row-major one with the bytes of eligible triplets permuted, nothing else.
    def parts(path):
        raw = open(path, "rb").read()
        length = struct.unpack("<Q", raw[8:16])[0]
        return json.loads(raw[16:16 + length]), raw
    (ha, a), (hb, b) = parts(str(tmp_path / "rows.splw")), parts(str(tmp_path / "tiled.splw"))
    assert ha["payloadLength"] == hb["payloadLength"] and [r["name"] for r in ha["tensorRecords"]] == [r["name"] for r in hb["tensorRecords"]]
    changed = 0
    for ra, rb in zip(ha["tensorRecords"], hb["tensorRecords"]):
        assert ra["rawByteLength"] == rb["rawByteLength"]
        xa = a[ra["payloadOffset"]: ra["payloadOffset"] + ra["rawByteLength"]]
        xb = b[rb["payloadOffset"]: rb["payloadOffset"] + rb["rawByteLength"]]
        eligible = ra["name"].startswith("language_model.") and "embed_tokens" not in ra["name"] and ra["name"].endswith((".weight", ".scales", ".biases")) \
            and len(ra["shape"]) == 2 and ra["shape"][0] % 128 == 0
        assert sorted(xa) == sorted(xb) if eligible else xa == xb
        changed += xa != xb
    assert changed > 0


def rewrite(raw, change):
    """The file with its header changed and re-framed (the payload where it was: only for changes that keep the header's length)."""
    length = struct.unpack("<Q", raw[8:16])[0]
    header = json.loads(raw[16:16 + length])
    change(header)
    encoded = json.dumps(header, sort_keys=True, separators=(",", ":")).encode()
    assert len(encoded) <= length, "the change must not lengthen the header"
    encoded += b" " * (length - len(encoded))
    return raw[:16] + encoded + raw[16 + length:]


def test_every_way_the_reference_refuses_a_container(model, tmp_path):
    g, m = model
    good = str(tmp_path / "good.splw")
    splw_writer.write(good, g, m)
    raw = open(good, "rb").read()
    length = struct.unpack("<Q", raw[8:16])[0]

    def refused(data, reason):
        path = str(tmp_path / "bad.splw")
        open(path, "wb").write(data)
        with pytest.raises(S.EngineError, match=reason):
            S.engine.splw_check(path)

    with pytest.raises(S.EngineError, match="weight file missing"):
        S.engine.splw_check(str(tmp_path / "absent.splw"))
    refused(raw[:10], "truncated framing")
    refused(b"SPLX" + raw[4:], "bad magic")
    refused(raw[:4] + struct.pack("<I", 2) + raw[8:], "unsupported version")
    refused(raw[:8] + struct.pack("<Q", len(raw)) + raw[16:], "header length overflow")
    refused(raw[:16] + b"{" + raw[17:16 + length - 1] + b"]" + raw[16 + length:], "malformed header")
    refused(rewrite(raw, lambda h: h.update(headerLength=h["headerLength"] - 1)), "contradictory header framing")
    refused(rewrite(raw, lambda h: h.update(version=2)), "contradictory header framing")
    refused(rewrite(raw, lambda h: h["quantization"].update(bits=3)), "unsupported quantization")
    refused(rewrite(raw, lambda h: h["quantization"].update(mode="gguf")), "unsupported quantization")
    refused(rewrite(raw, lambda h: h["alignment"].update(pointerAlignmentBytes=0)), "invalid alignment")
    refused(raw + b"\0" * 128, "payload size mismatch")
    refused(rewrite(raw, lambda h: h.update(payloadLength=h["payloadLength"] - 128)), "payload size mismatch")

    def rename_second(h):
        h["tensorRecords"][1]["name"] = h["tensorRecords"][0]["name"]
    refused(rewrite(raw, rename_second), "duplicate tensor")
    refused(rewrite(raw, lambda h: h["tensorRecords"][2].update(dtype="F8")), "unknown dtype")
    refused(rewrite(raw, lambda h: h["tensorRecords"][0].update(payloadOffset=0)), "tensor bounds")
    refused(rewrite(raw, lambda h: h["tensorRecords"][3].update(payloadOffset=h["tensorRecords"][3]["payloadOffset"] - 8, alignmentPadding=0)), "tensor bounds|unaligned tensor")
    refused(rewrite(raw, lambda h: h["tensorRecords"][3].update(alignmentPadding=h["tensorRecords"][3]["alignmentPadding"] + 1)), "padding mismatch")
    # A record that claims fewer bytes than lie there: the next one's padding no longer accounts for the gap.
    refused(rewrite(raw, lambda h: h["tensorRecords"][3].update(rawByteLength=h["tensorRecords"][3]["rawByteLength"] - 2)), "padding mismatch")
    # The last record dropped: its bytes are nobody's.
    refused(rewrite(raw, lambda h: h["tensorRecords"].pop()), "unaccounted payload bytes")


def test_an_alignment_other_than_128_is_honoured(model, tmp_path):
    g, m = model
    path = str(tmp_path / "a256.splw")
    splw_writer.write(path, g, m, alignment=256)
    assert S.engine.splw_check(path)[0] == "mlxAffine4"


@pytest.mark.parametrize("kind", ["Q4_K", "Q5_K", "Q6_K"])
def test_planes_unpack_to_the_native_blocks_they_were_made_of(kind):
    """GgufPlanes.unpack (Sources/SploshModel/GgufPlanes.swift:150-190) undoes the repack for every bit of a block: random
    blocks, 200 rows (two tiles, the second padded), through the tests' restatement of the repack and back through
    spl_gguf_planes_unpack."""
    rng = np.random.default_rng(7)
    block_bytes = splw_writer.PLANES[kind][1]
    blocks = rng.integers(0, 256, (200, 3, block_bytes), dtype=np.uint8)
    p0, p1, meta = splw_writer.planes_of(kind, blocks)
    assert p0.size == 256 * 24 * 16 and meta.size == 256 * 3 * splw_writer.PLANES[kind][3]
    native = S.engine.gguf_planes_unpack(kind, p0, p1, meta, 200, 768)
    assert np.array_equal(native, blocks)
    # One element of one row: its nibble is where the layout says (row 130 = tile 1, row 2; group 9; element 21 -> slot 13).
    if kind != "Q6_K":
        record = p0.reshape(2, 24, 128, 16)[1, 9, 2]
        word = int.from_bytes(bytes(record[4:8]), "little")
        codes = 48 if kind == "Q5_K" else 16
        assert (word >> (16 * (13 & 1) + 4 * ((13 & 7) >> 1))) & 15 == (int(blocks[130, 1, codes + 32 * 0 + 21]) >> 4) & 15
