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
