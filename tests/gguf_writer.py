"""Writes a llama.cpp GGUF file (version 3) of the tests' synthetic GGUF-weighted model: the inverse of what the library's
reader does (Sources/SploshModel/GgufNames.swift:13-44 for the names, :73-84 for the order of the gated-delta value heads;
GgufConvert.swift:25-28 for the dense tensors). Test infrastructure."""
import struct

import numpy as np

GGML = {"F32": 0, "F16": 1, "Q4_K": 12, "Q5_K": 13, "Q6_K": 14}


def bits_to_float(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def engine_head(g, file_head):
    ratio = g.gdn_value_heads // g.gdn_key_heads
    return ratio * (file_head % g.gdn_key_heads) + file_head // g.gdn_key_heads


def to_file_order(g, array, first, span):
    """Units [first, first + heads x span) of the leading axis, from the engine's head order to the file's."""
    out = np.array(array, copy=True)
    for i in range(g.gdn_value_heads):
        e = engine_head(g, i)
        out[first + i * span: first + (i + 1) * span] = array[first + e * span: first + (e + 1) * span]
    return out


def string(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write(path, g, model, mtp_block=True, tied_head=False):
    """model: oracle Model after to_gguf(). The out projection is written as the model holds it: its columns are then in the
    file's order by definition, and the model is to be told so (set_out_file_order)."""
    tensors = []                           # (name, extents fastest first, ggml type, bytes)
    D, KH, VH = g.gdn_head_dim, g.gdn_key_heads, g.gdn_value_heads

    def packed(name, layer, kind, first=None, span=0):
        gguf_kind, blocks = model.gguf(layer, kind)
        blocks = np.asarray(blocks)
        if first is not None:
            blocks = to_file_order(g, blocks, first, span)
        tensors.append((name, [blocks.shape[1] * 256, blocks.shape[0]], GGML[gguf_kind], blocks.tobytes()))

    def dense(name, values, extents=None, as_f16=False):
        values = np.ascontiguousarray(values, np.float32)
        if as_f16:
            tensors.append((name, extents or [values.size], GGML["F16"], values.astype(np.float16).tobytes()))
        else:
            tensors.append((name, extents or [values.size], GGML["F32"], values.tobytes()))

    for layer in range(g.layers):
        b = f"blk.{layer}."
        dense(b + "attn_norm.weight", bits_to_float(model.vec(layer, "input_norm")))
        dense(b + "post_attention_norm.weight", bits_to_float(model.vec(layer, "post_norm")))
        if layer % 4 == 3:
            packed(b + "attn_q.weight", layer, "q"); packed(b + "attn_k.weight", layer, "k")
            packed(b + "attn_v.weight", layer, "v"); packed(b + "attn_output.weight", layer, "o")
            dense(b + "attn_q_norm.weight", bits_to_float(model.vec(layer, "q_norm")))
            dense(b + "attn_k_norm.weight", bits_to_float(model.vec(layer, "k_norm")))
        else:
            packed(b + "attn_qkv.weight", layer, "qkv", 2 * KH * D, D)
            packed(b + "attn_gate.weight", layer, "z", 0, D)
            packed(b + "ssm_alpha.weight", layer, "a", 0, 1)
            packed(b + "ssm_beta.weight", layer, "b", 0, 1)
            packed(b + "ssm_out.weight", layer, "out")
            conv = bits_to_float(model.vec(layer, "conv")).reshape(-1, 4)
            dense(b + "ssm_conv1d.weight", to_file_order(g, conv, 2 * KH * D, D), [4, conv.shape[0]])
            a_log = bits_to_float(model.vec(layer, "a_log"))
            dense(b + "ssm_a", to_file_order(g, -np.exp(a_log.astype(np.float64)).astype(np.float32), 0, 1))
            dense(b + "ssm_dt.bias", to_file_order(g, bits_to_float(model.vec(layer, "dt_bias")), 0, 1))
            dense(b + "ssm_norm.weight", bits_to_float(model.vec(layer, "gdn_norm")))
        packed(b + "ffn_gate.weight", layer, "gate"); packed(b + "ffn_up.weight", layer, "up"); packed(b + "ffn_down.weight", layer, "down")
    packed("token_embd.weight", -1, "embed")
    if not tied_head:
        packed("output.weight", -1, "head")
    dense("output_norm.weight", bits_to_float(model.vec(-1, "final_norm")))
    if mtp_block:                          # an MTP head the engine does not run: the last block of a file with .nextn. tensors
        b = f"blk.{g.layers}."
        dense(b + "nextn.eh_proj.weight", np.ones(64, np.float32))
        dense(b + "attn_norm.weight", np.full(g.hidden, 7.0, np.float32))

    alignment = 32
    meta = [("general.architecture", 8, "qwen35"), ("general.alignment", 4, alignment), ("general.file_type", 4, 17),
            ("tokenizer.ggml.tokens", 9, ["a", "bc", "def"]), ("some.scale", 6, 1.5), ("some.flag", 7, True)]
    out = bytearray(struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(meta)))
    for key, kind, value in meta:
        out += string(key) + struct.pack("<I", kind)
        if kind == 8:
            out += string(value)
        elif kind == 4:
            out += struct.pack("<I", value)
        elif kind == 6:
            out += struct.pack("<f", value)
        elif kind == 7:
            out += struct.pack("<B", 1 if value else 0)
        elif kind == 9:
            out += struct.pack("<IQ", 8, len(value)) + b"".join(string(v) for v in value)
    offset, offsets = 0, []
    for _, _, _, data in tensors:
        offsets.append(offset)
        offset = (offset + len(data) + alignment - 1) // alignment * alignment
    for (name, extents, kind, _), at in zip(tensors, offsets):
        out += string(name) + struct.pack("<I", len(extents)) + b"".join(struct.pack("<Q", e) for e in extents) + struct.pack("<IQ", kind, at)
    out += b"\0" * ((-len(out)) % alignment)
    start = len(out)
    for (_, _, _, data), at in zip(tensors, offsets):
        out += b"\0" * (start + at - len(out)) + data
    with open(path, "wb") as f:
        f.write(bytes(out))
