"""Writes an SPLW artifact of the tests' synthetic MLX affine-4 model, row-major or tiled: what the reference's converter
and re-tiler leave on disk (Sources/SploshModel/Converter.swift:46-82 for the header and the framing, :160-228 for the
layout of the payload; Sources/SploshModel/Retile.swift:31-36, 137-153 for the tiled form). Test infrastructure."""
import json
import struct

import numpy as np

NAMES = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj",
         "qkv": "linear_attn.in_proj_qkv", "z": "linear_attn.in_proj_z", "a": "linear_attn.in_proj_a", "b": "linear_attn.in_proj_b",
         "out": "linear_attn.out_proj", "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj",
         "input_norm": "input_layernorm.weight", "post_norm": "post_attention_layernorm.weight",
         "q_norm": "self_attn.q_norm.weight", "k_norm": "self_attn.k_norm.weight", "conv": "linear_attn.conv1d.weight",
         "a_log": "linear_attn.A_log", "dt_bias": "linear_attn.dt_bias", "gdn_norm": "linear_attn.norm.weight"}


def tile(array, rows, element_bytes):
    """[row][group][element] -> [tile of 128 rows][group][row in tile][element] (Converter.tile)."""
    flat = np.ascontiguousarray(array).view(np.uint8).reshape(rows // 128, 128, -1, element_bytes)
    return np.ascontiguousarray(flat.transpose(0, 2, 1, 3))


def tensors_of(g, model):
    """(name, dtype, shape, logical shape or None, numpy array) for every tensor of the model, the reference's names."""
    out = []

    def q4(name, layer, kind):
        packed, scales, biases = model.q4(layer, kind)
        rows, words = packed.shape
        out.append((name + ".weight", "U32", [rows, words], [rows, words * 8], np.ascontiguousarray(packed, np.uint32)))
        out.append((name + ".scales", "BF16", list(scales.shape), None, np.ascontiguousarray(scales, np.uint16)))
        out.append((name + ".biases", "BF16", list(biases.shape), None, np.ascontiguousarray(biases, np.uint16)))

    def dense(name, layer, kind, shape):
        out.append((name, "BF16", shape, None, np.ascontiguousarray(model.vec(layer, kind), np.uint16)))

    C = (2 * g.gdn_key_heads + g.gdn_value_heads) * g.gdn_head_dim
    for layer in range(g.layers):
        p = f"language_model.model.layers.{layer}."
        full = layer % 4 == 3
        for kind in (["q", "k", "v", "o"] if full else ["qkv", "z", "a", "b", "out"]) + ["gate", "up", "down"]:
            q4(p + NAMES[kind], layer, kind)
        shapes = {"input_norm": [g.hidden], "post_norm": [g.hidden], "q_norm": [g.head_dim], "k_norm": [g.head_dim], "conv": [C, 4, 1],
                  "a_log": [g.gdn_value_heads], "dt_bias": [g.gdn_value_heads], "gdn_norm": [g.gdn_head_dim]}
        for kind in ["input_norm", "post_norm"] + (["q_norm", "k_norm"] if full else ["conv", "a_log", "dt_bias", "gdn_norm"]):
            dense(p + NAMES[kind], layer, kind, shapes[kind])
    q4("language_model.model.embed_tokens", -1, "embed")
    q4("language_model.lm_head", -1, "head")
    dense("language_model.model.norm.weight", -1, "final_norm", [g.hidden])
    # A tensor outside the language model, as a vision tower's would be: the loader passes it by.
    out.append(("vision_tower.patch_embed.bias", "BF16", [8], None, np.arange(8, dtype=np.uint16)))
    return sorted(out, key=lambda t: t[0])


def write(path, g, model, tiled=False, alignment=128, mutate=None, bits=4, fmt=None):
    """mutate(header dict, records list) may change the header before it is encoded (for files that are to be refused)."""
    tensors = tensors_of(g, model)
    payloads = []
    tiled_rows = {}
    for name, dtype, shape, logical, array in tensors:
        if tiled and dtype == "U32" and name.startswith("language_model.") and "embed_tokens" not in name and shape[0] % 128 == 0:
            tiled_rows[name[:-len(".weight")]] = shape[0]
    for name, dtype, shape, logical, array in tensors:
        base = name.rsplit(".", 1)[0]
        if dtype == "U32" and base in tiled_rows:
            array = tile(array, shape[0], 32)
        elif name.endswith((".scales", ".biases")) and base in tiled_rows:
            array = tile(array, tiled_rows[base], 2)
        payloads.append(array.tobytes())
    fmt = fmt or ("mlxAffine%d.tiled128" % bits if tiled else "mlxAffine%d" % bits)

    def records_for(start):
        records, cursor = [], start
        for (name, dtype, shape, logical, _), blob in zip(tensors, payloads):
            offset = (cursor + alignment - 1) // alignment * alignment
            row_bytes = shape[1] * 4 if dtype == "U32" else (shape[1] * 2 if len(shape) == 2 else len(blob))
            record = {"name": name, "dtype": dtype, "shape": shape, "physicalShape": shape, "payloadOffset": offset, "rawByteLength": len(blob),
                      "rowStride": (row_bytes + 127) // 128 * 128, "alignmentPadding": offset - cursor, "sourceShard": "model.safetensors"}
            if logical is not None:
                record["logicalShape"] = logical
            records.append(record)
            cursor = offset + len(blob)
        return records, cursor

    header_bytes = b""
    for _ in range(8):        # the header's length depends on the offsets it holds: to a fixed point, as the converter does
        start = (16 + len(header_bytes) + alignment - 1) // alignment * alignment
        records, end = records_for(start)
        header = {"magic": "SPLW", "version": 1, "format": fmt, "dtype": "MIXED", "quantization": {"bits": bits, "groupSize": 64, "mode": "affine"},
                  "alignment": {"rowStrideBytes": 128, "pointerAlignmentBytes": alignment, "padded": True}, "configHash": "0" * 64, "tokenizerHash": "1" * 64,
                  "tensorRecords": records, "headerLength": len(header_bytes), "payloadLength": end - start}
        if mutate:
            mutate(header, records)
        encoded = json.dumps(header, sort_keys=True, separators=(",", ":")).encode()
        if encoded == header_bytes:
            break
        header_bytes = encoded
    start = (16 + len(header_bytes) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(b"SPLW" + struct.pack("<IQ", 1, len(header_bytes)) + header_bytes)
        f.write(b"\0" * (start - 16 - len(header_bytes)))
        at = start
        for record, blob in zip(records, payloads):
            f.write(b"\0" * (record["payloadOffset"] - at))
            f.write(blob)
            at = record["payloadOffset"] + len(blob)
    return header


# ---- a GGUF-derived artifact: every 2-D weight as three planes (Sources/SploshModel/GgufPlanes.swift:1-20, 214-262) ----
PLANES = {"Q4_K": (12, 144, 0, 16), "Q5_K": (13, 176, 4, 16), "Q6_K": (14, 210, 8, 20)}      # ggml type, block bytes, plane 1 and meta record bytes
SLOT = np.array([8 * ((e >> 2) & 3) + 4 * (e >> 4) + (e & 3) for e in range(32)])


def planes_of(kind, blocks):
    """Native blocks uint8 [rows][inner / 256][block bytes] -> (plane0, plane1 or None, meta), rows padded to whole tiles of 128
    with zero blocks: per (row, group of 32) a 16-byte record of low nibbles in slot order and a record of the bits above
    them; per (row, native block) the block's scale fields; records of the same group of a tile's 128 rows side by side."""
    _, block_bytes, plane1_bytes, meta_bytes = PLANES[kind]
    blocks = np.asarray(blocks, np.uint8)
    rows, per_row, _ = blocks.shape
    stored = (rows + 127) // 128 * 128
    padded = np.zeros((stored, per_row, block_bytes), np.uint8)
    padded[:rows] = blocks
    groups = per_row * 8
    low = np.zeros((stored, groups, 32), np.uint32)        # [row][group][element]
    high = np.zeros((stored, groups, 32), np.uint32)
    for j in range(8):
        if kind == "Q6_K":
            half, quarter = j // 4, j % 4
            ql = padded[:, :, 64 * half + 32 * (quarter & 1): 64 * half + 32 * (quarter & 1) + 32]
            qh = padded[:, :, 128 + 32 * half: 128 + 32 * half + 32]
            low[:, j::8] = (ql >> (4 * (quarter >> 1))) & 15
            high[:, j::8] = (qh >> (2 * quarter)) & 3
        else:
            codes = 48 if kind == "Q5_K" else 16
            qs = padded[:, :, codes + 32 * (j // 2): codes + 32 * (j // 2) + 32]
            low[:, j::8] = (qs >> (4 * (j % 2))) & 15
            if kind == "Q5_K":
                high[:, j::8] = (padded[:, :, 16:48] >> j) & 1
    by_slot = np.zeros_like(low); by_slot[:, :, SLOT] = low            # slot s holds element e with SLOT[e] == s
    top_slot = np.zeros_like(high); top_slot[:, :, SLOT] = high
    s = np.arange(32)
    words = np.zeros((stored, groups, 4), np.uint32)
    for c in range(4):
        for i in range(8):
            words[:, :, c] |= by_slot[:, :, 8 * c + i] << np.uint32((i & 1) * 16 + 4 * (i >> 1))
    plane0 = words.view(np.uint8).reshape(stored, groups, 16)
    plane1 = None
    if plane1_bytes:
        width = 1 if kind == "Q5_K" else 2
        per_word = 32 // width
        hw = np.zeros((stored, groups, width), np.uint32)
        for w in range(width):
            for i in range(per_word):
                hw[:, :, w] |= top_slot[:, :, w * per_word + i] << np.uint32(width * i)
        plane1 = hw.view(np.uint8).reshape(stored, groups, plane1_bytes)
    meta = np.zeros((stored, per_row, meta_bytes), np.uint8)
    if kind == "Q6_K":
        meta[:, :, :16] = padded[:, :, 192:208]; meta[:, :, 16:18] = padded[:, :, 208:210]
    else:
        meta[:, :, :16] = padded[:, :, :16]

    def tiled(plane):          # [row][record][bytes] -> [tile][record][row in tile][bytes]
        n, per, width = plane.shape
        return np.ascontiguousarray(plane.reshape(n // 128, 128, per, width).transpose(0, 2, 1, 3))
    return tiled(plane0), None if plane1 is None else tiled(plane1), tiled(meta)


def write_gguf_derived(path, g, model, alignment=128):
    """The artifact GgufConvert.convertGguf leaves (Sources/SploshModel/GgufConvert.swift:1-33, 118-146): the MLX pack's names,
    dense tensors as they are in the engine (bf16), every 2-D weight as <base>.weight (plane 0, with `ggufType` and
    `logicalShape`), <base>.plane1 and <base>.meta. model: the oracle Model after to_gguf(); its out projections are then in
    the file's order of the value heads by definition (set_out_file_order)."""
    records = []          # (name, dtype, shape, logical, gguf type, bytes)

    def weight(name, layer, kind):
        gguf_kind, blocks = model.gguf(layer, kind)
        blocks = np.asarray(blocks, np.uint8)
        rows, inner = blocks.shape[0], blocks.shape[1] * 256
        p0, p1, meta = planes_of(gguf_kind, blocks)
        stored = (rows + 127) // 128 * 128
        records.append((name + ".weight", "U8", [stored, p0.size // stored], [rows, inner], PLANES[gguf_kind][0], p0.tobytes()))
        if p1 is not None:
            records.append((name + ".plane1", "U8", [stored, p1.size // stored], None, None, p1.tobytes()))
        records.append((name + ".meta", "U8", [stored, meta.size // stored], None, None, meta.tobytes()))

    def dense(name, layer, kind, shape):
        records.append((name, "BF16", shape, None, None, np.ascontiguousarray(model.vec(layer, kind), np.uint16).tobytes()))

    C = (2 * g.gdn_key_heads + g.gdn_value_heads) * g.gdn_head_dim
    for layer in range(g.layers):
        p = f"language_model.model.layers.{layer}."
        full = layer % 4 == 3
        for kind in (["q", "k", "v", "o"] if full else ["qkv", "z", "a", "b", "out"]) + ["gate", "up", "down"]:
            weight(p + NAMES[kind], layer, kind)
        shapes = {"input_norm": [g.hidden], "post_norm": [g.hidden], "q_norm": [g.head_dim], "k_norm": [g.head_dim], "conv": [C, 4, 1],
                  "a_log": [g.gdn_value_heads], "dt_bias": [g.gdn_value_heads], "gdn_norm": [g.gdn_head_dim]}
        for kind in ["input_norm", "post_norm"] + (["q_norm", "k_norm"] if full else ["conv", "a_log", "dt_bias", "gdn_norm"]):
            dense(p + NAMES[kind], layer, kind, shapes[kind])
    weight("language_model.model.embed_tokens", -1, "embed")
    weight("language_model.lm_head", -1, "head")
    dense("language_model.model.norm.weight", -1, "final_norm", [g.hidden])
    records.sort(key=lambda r: r[0])

    header_bytes = b""
    for _ in range(8):
        start = (16 + len(header_bytes) + alignment - 1) // alignment * alignment
        entries, cursor = [], start
        for name, dtype, shape, logical, gguf_type, blob in records:
            offset = (cursor + alignment - 1) // alignment * alignment
            entry = {"name": name, "dtype": dtype, "shape": shape, "physicalShape": shape, "payloadOffset": offset, "rawByteLength": len(blob),
                     "rowStride": (len(blob) // max(shape[0], 1) + 127) // 128 * 128, "alignmentPadding": offset - cursor, "sourceShard": "model.gguf"}
            if logical is not None:
                entry["logicalShape"] = logical
            if gguf_type is not None:
                entry["ggufType"] = gguf_type
            entries.append(entry)
            cursor = offset + len(blob)
        header = {"magic": "SPLW", "version": 1, "format": "gguf.tiled128", "dtype": "MIXED", "quantization": {"bits": 0, "groupSize": 32, "mode": "gguf"},
                  "alignment": {"rowStrideBytes": 128, "pointerAlignmentBytes": alignment, "padded": True}, "configHash": "2" * 64, "tokenizerHash": "1" * 64,
                  "tensorRecords": entries, "headerLength": len(header_bytes), "payloadLength": cursor - start}
        encoded = json.dumps(header, sort_keys=True, separators=(",", ":")).encode()
        if encoded == header_bytes:
            break
        header_bytes = encoded
    start = (16 + len(header_bytes) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(b"SPLW" + struct.pack("<IQ", 1, len(header_bytes)) + header_bytes)
        f.write(b"\0" * (start - 16 - len(header_bytes)))
        at = start
        for entry, record in zip(entries, records):
            f.write(b"\0" * (entry["payloadOffset"] - at))
            f.write(record[5])
            at = entry["payloadOffset"] + len(record[5])
    return header
