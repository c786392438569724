"""ctypes binding of the CPU oracle (oracle/splosh_oracle.cpp). TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may import this.
"""
import ctypes as C
import os
import subprocess
import numpy as np

from .tables import Tables

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class Geometry(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("layers", "hidden", "inter", "vocab", "heads", "kv_heads", "head_dim", "rotary_dim",
                                         "gdn_key_heads", "gdn_value_heads", "gdn_head_dim")] + [("eps", C.c_float), ("rope_theta", C.c_float)]

    @property
    def channels(self):
        return (2 * self.gdn_key_heads + self.gdn_value_heads) * self.gdn_head_dim

    @property
    def value_dim(self):
        return self.gdn_value_heads * self.gdn_head_dim

    def with_(self, **kw):
        out = Geometry.from_buffer_copy(bytes(self))
        for k, v in kw.items():
            setattr(out, k, v)
        return out


def tiny_geometry():
    """The 4-layer hybrid of the first benchmark configuration."""
    return Geometry(4, 1024, 2816, 32000, 8, 2, 128, 32, 4, 8, 128, 1e-6, 1e7)


def b27_geometry():
    """The 27B shape (Sources/SploshModel/ModelWeights.swift:66-88)."""
    return Geometry(64, 5120, 17408, 248320, 24, 4, 256, 64, 16, 48, 128, 1e-6, 1e7)


class _CTables(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("rows", "run_count", "logit_rows", "attn_block_count", "step_pages", "live_rows",
                                          "spans", "pages_per_span")] + \
               [(n, C.POINTER(C.c_uint32)) for n in ("tokens", "row_slot", "row_pos", "runs", "run_info", "row_read", "row_write",
                                                     "gather_index", "attn_blocks", "page_table")]


def build():
    subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.orc_splitmix_at.restype = C.c_uint64; L.orc_splitmix_at.argtypes = [C.c_uint64, C.c_uint64]
        L.orc_uniform_at.restype = C.c_float; L.orc_uniform_at.argtypes = [C.c_uint64, C.c_uint64]
        L.orc_normal_at.restype = C.c_float; L.orc_normal_at.argtypes = [C.c_uint64, C.c_uint64, C.c_float]
        L.orc_fnv1a64.restype = C.c_uint64; L.orc_fnv1a64.argtypes = [C.c_char_p]
        L.orc_bf16.restype = C.c_uint16; L.orc_bf16.argtypes = [C.c_float]
        L.orc_f16_round.restype = C.c_float; L.orc_f16_round.argtypes = [C.c_float]
        L.orc_argmax.restype = C.c_int32; L.orc_argmax.argtypes = [C.c_void_p, C.c_int]
        L.orc_model_create.restype = C.c_void_p; L.orc_model_create.argtypes = [C.POINTER(Geometry), C.c_uint64]
        L.orc_model_destroy.argtypes = [C.c_void_p]
        L.orc_tensor_seed.restype = C.c_uint64; L.orc_tensor_seed.argtypes = [C.c_uint64, C.c_int, C.c_int, C.c_int]
        L.orc_engine_create.restype = C.c_void_p; L.orc_engine_create.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]
        L.orc_engine_destroy.argtypes = [C.c_void_p]
        L.orc_engine_reset_slot.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.orc_engine_buffer.restype = C.c_void_p; L.orc_engine_buffer.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_size_t)]
        L.orc_set_norm_contract.argtypes = [C.c_int]
        L.orc_model_set_out_file_order.argtypes = [C.c_void_p, C.c_int]
        L.orc_model_set_gguf.restype = C.c_int; L.orc_model_set_gguf.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.orc_step.restype = C.c_int; L.orc_step.argtypes = [C.c_void_p, C.POINTER(_CTables), C.c_void_p, C.c_void_p, C.c_int]
        L.orc_attention_scan.restype = C.c_int
        L.orc_attention_scan.argtypes = [C.c_void_p, C.c_int, C.POINTER(_CTables), C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_model_q4.restype = C.c_int
        L.orc_model_q4.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)] + [C.POINTER(C.c_void_p)] * 3
        L.orc_model_vec.restype = C.c_int
        L.orc_model_vec.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_int)]
        L.orc_threads.restype = C.c_int
        _LIB = L
    return _LIB


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


Q4_KINDS = ["qkv", "z", "a", "b", "out", "q", "k", "v", "o", "gate", "up", "down", "embed", "head"]
VEC_KINDS = ["input_norm", "post_norm", "conv", "a_log", "dt_bias", "gdn_norm", "q_norm", "k_norm", "final_norm"]


def bf16_round(x):
    """Round an fp32 array to bf16 (nearest even) and back."""
    bits = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return (((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def bf16_bits_to_float(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def quantize_mlx4(w):
    w = np.ascontiguousarray(w, np.float32)
    rows, inner = w.shape
    packed = np.zeros((rows, inner // 8), np.uint32); scales = np.zeros((rows, inner // 64), np.uint16); biases = np.zeros_like(scales)
    lib().orc_quantize_mlx4(_ptr(w), rows, inner, _ptr(packed), _ptr(scales), _ptr(biases))
    return packed, scales, biases


def dequant_mlx4(packed, scales, biases, columns):
    packed = np.ascontiguousarray(packed, np.uint32); rows = packed.shape[0]
    scales = np.ascontiguousarray(scales, np.float32); biases = np.ascontiguousarray(biases, np.float32)
    out = np.zeros((rows, columns), np.float32)
    lib().orc_dequant_mlx4(_ptr(packed), _ptr(scales), _ptr(biases), rows, columns, _ptr(out))
    return out


def decode_gguf(kind, raw):
    """raw: uint8 [blocks, block_bytes] -> float32 [blocks, 256]."""
    raw = np.ascontiguousarray(raw, np.uint8)
    out = np.zeros((raw.shape[0], 256), np.float32)
    if kind == "Q6_K":
        assert raw.shape[1] == 210
        lib().orc_decode_q6k(_ptr(raw), raw.shape[0], _ptr(out))
    else:
        assert raw.shape[1] == {"Q4_K": 144, "Q5_K": 176}[kind]
        lib().orc_decode_q45k(_ptr(raw), raw.shape[0], 1 if kind == "Q5_K" else 0, _ptr(out))
    return out


GGUF_TYPE = {"Q4_K": 12, "Q5_K": 13, "Q6_K": 14}
GGUF_BLOCK_BYTES = {"Q4_K": 144, "Q5_K": 176, "Q6_K": 210}


def gguf_tile_weights(kind, raw):
    """The weights as the GGUF tile kernels form them (gguf_formats.h:390-438): raw uint8 [blocks, bytes] -> float32 [blocks, 256]
    of fp16-representable values."""
    raw = np.ascontiguousarray(raw, np.uint8)
    assert raw.shape[1] == GGUF_BLOCK_BYTES[kind]
    out = np.zeros((raw.shape[0], 256), np.float32)
    lib().orc_gguf_tile_weights(GGUF_TYPE[kind], _ptr(raw), raw.shape[0], _ptr(out))
    return out


def gemm_gguf(kind, blocks, activations, residual=None):
    """blocks: uint8 [n, k / 256, block bytes] native GGUF super-blocks, row-major; activations fp32 [rows, k]."""
    blocks = np.ascontiguousarray(blocks, np.uint8)
    n, per_row = blocks.shape[0], blocks.shape[1]
    a = np.ascontiguousarray(activations, np.float32)
    out = np.zeros((a.shape[0], n), np.float32)
    res = None if residual is None else np.ascontiguousarray(residual, np.float32)
    lib().orc_gemm_gguf(GGUF_TYPE[kind], _ptr(blocks), n, per_row * 256, _ptr(a), a.shape[0], None if res is None else _ptr(res), _ptr(out))
    return out


def quantize_gguf(kind, weights, seed=0):
    """A build-owned K-quant encoder, good enough to make valid blocks (parity is defined on the DECODED values, so any
    valid encoding serves): per 32 (Q4_K, Q5_K) or 16 (Q6_K) elements a min/max scale against per-256 fp16 d / dmin.
    weights: fp32 [n, k] -> uint8 [n, k / 256, block bytes]."""
    w = np.ascontiguousarray(weights, np.float32)
    n, k = w.shape
    assert k % 256 == 0
    blocks = w.reshape(n * (k // 256), 256)
    nb = blocks.shape[0]
    out = np.zeros((nb, GGUF_BLOCK_BYTES[kind]), np.uint8)
    if kind == "Q6_K":
        sub = blocks.reshape(nb, 16, 16)
        amax = np.abs(sub).max(axis=2)                          # [nb, 16]
        d = (amax.max(axis=1) / (127.0 * 31.0)).astype(np.float16)
        d32 = np.where(d.astype(np.float32) == 0, 1.0, d.astype(np.float32))
        sc = np.clip(np.rint(amax / 31.0 / d32[:, None]), -128, 127).astype(np.int8)
        step = d32[:, None] * sc.astype(np.float32)
        step = np.where(step == 0, 1.0, step)
        q = np.clip(np.rint(sub / step[:, :, None]) + 32, 0, 63).astype(np.uint8).reshape(nb, 256)
        for half in range(2):
            for quarter in range(4):
                e = q[:, 128 * half + 32 * quarter: 128 * half + 32 * quarter + 32]
                low, high = e & 15, e >> 4
                ql = out[:, 64 * half + 32 * (quarter & 1): 64 * half + 32 * (quarter & 1) + 32]
                ql |= (low << (4 * (quarter >> 1))).astype(np.uint8)
                qh = out[:, 128 + 32 * half: 128 + 32 * half + 32]
                qh |= (high << (2 * quarter)).astype(np.uint8)
        out[:, 192:208] = sc.view(np.uint8)
        out[:, 208:210] = d.view(np.uint8).reshape(nb, 2)
        return out.reshape(n, k // 256, 210)
    levels = 31 if kind == "Q5_K" else 15
    sub = blocks.reshape(nb, 8, 32)
    lo = np.minimum(sub.min(axis=2), 0.0); hi = sub.max(axis=2)
    step = (hi - lo) / levels                                   # [nb, 8]
    d = (step.max(axis=1) / 63.0).astype(np.float16); dmin = ((-lo).max(axis=1) / 63.0).astype(np.float16)
    d32 = np.where(d.astype(np.float32) == 0, 1.0, d.astype(np.float32)); m32 = np.where(dmin.astype(np.float32) == 0, 1.0, dmin.astype(np.float32))
    sc = np.clip(np.rint(step / d32[:, None]), 0, 63).astype(np.uint8); mn = np.clip(np.rint(-lo / m32[:, None]), 0, 63).astype(np.uint8)
    s = d.astype(np.float32)[:, None] * sc; m = dmin.astype(np.float32)[:, None] * mn
    q = np.clip(np.rint((sub + m[:, :, None]) / np.where(s == 0, 1.0, s)[:, :, None]), 0, levels).astype(np.uint8)      # [nb, 8, 32]
    out[:, 0:2] = d.view(np.uint8).reshape(nb, 2); out[:, 2:4] = dmin.view(np.uint8).reshape(nb, 2)
    for j in range(4):
        out[:, 4 + j] = (sc[:, j] & 63) | ((sc[:, j + 4] >> 4) << 6)
        out[:, 8 + j] = (mn[:, j] & 63) | ((mn[:, j + 4] >> 4) << 6)
        out[:, 12 + j] = (sc[:, j + 4] & 15) | ((mn[:, j + 4] & 15) << 4)
    codes = 48 if kind == "Q5_K" else 16
    for j in range(8):
        nib = (q[:, j] & 15).astype(np.uint8)
        out[:, codes + 32 * (j // 2): codes + 32 * (j // 2) + 32] |= (nib << (4 * (j % 2))).astype(np.uint8)
        if kind == "Q5_K":
            out[:, 16:48] |= ((q[:, j] >> 4) << j).astype(np.uint8)
    return out.reshape(n, k // 256, GGUF_BLOCK_BYTES[kind])


def gemm_q4(packed, scales, biases, activations, residual=None):
    n, k = packed.shape[0], packed.shape[1] * 8
    a = np.ascontiguousarray(activations, np.float32)
    out = np.zeros((a.shape[0], n), np.float32)
    res = None if residual is None else np.ascontiguousarray(residual, np.float32)
    lib().orc_gemm_q4(_ptr(np.ascontiguousarray(packed)), _ptr(np.ascontiguousarray(scales)), _ptr(np.ascontiguousarray(biases)),
                      n, k, _ptr(a), a.shape[0], None if res is None else _ptr(res), _ptr(out))
    return out


class Model:
    """A seeded synthetic model: projection weights ~N(0, 0.02) quantised to MLX affine-4, norm
    weights bf16(1 + N(0, 0.02)), conv / A_log / dt_bias in the ranges of the reference's tests."""

    def __init__(self, geometry, seed=0x5EED6D17):
        self.g, self.seed = geometry, seed
        self.handle = lib().orc_model_create(C.byref(geometry), seed)

    def __del__(self):
        if getattr(self, "handle", None):
            lib().orc_model_destroy(self.handle); self.handle = None

    def full(self, layer):
        return layer % 4 == 3

    def q4(self, layer, kind):
        """(packed u32 [rows, inner/8], scales u16 [rows, inner/64], biases) as views of the oracle's memory."""
        rows, inner = C.c_int(), C.c_int()
        p, s, b = C.c_void_p(), C.c_void_p(), C.c_void_p()
        if lib().orc_model_q4(self.handle, layer, Q4_KINDS.index(kind), C.byref(rows), C.byref(inner), C.byref(p), C.byref(s), C.byref(b)):
            return None
        r, k = rows.value, inner.value
        packed = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint32)), (r, k // 8))
        scales = np.ctypeslib.as_array(C.cast(s, C.POINTER(C.c_uint16)), (r, k // 64))
        biases = np.ctypeslib.as_array(C.cast(b, C.POINTER(C.c_uint16)), (r, k // 64))
        return packed, scales, biases

    def set_gguf(self, layer, kind, gguf_kind, blocks):
        """The tensor as native GGUF super-blocks from now on (uint8 [rows, inner / 256, block bytes])."""
        blocks = np.ascontiguousarray(blocks, np.uint8)
        if lib().orc_model_set_gguf(self.handle, layer, Q4_KINDS.index(kind), GGUF_TYPE[gguf_kind], _ptr(blocks)):
            raise ValueError(f"tensor {kind} of layer {layer} cannot hold {gguf_kind} blocks")
        if not hasattr(self, "_gguf"):
            self._gguf = {}
        self._gguf[(layer, kind)] = (gguf_kind, blocks)

    def gguf(self, layer, kind):
        return self._gguf[(layer, kind)]

    def set_out_file_order(self, enabled=True):
        """The gated-delta out projections hold their columns in a GGUF file's order of the value heads."""
        lib().orc_model_set_out_file_order(self.handle, 1 if enabled else 0)
        self.out_file_order = bool(enabled)

    def to_gguf(self, block_kind="Q5_K", head_kind="Q6_K"):
        """Re-quantise every tensor from its MLX affine-4 values to GGUF K-quants: the synthetic GGUF-weighted model
        (all 2-D tensors `block_kind`, embedding and head `head_kind`). Parity is defined on the decoded blocks."""
        def convert(layer, kind, gguf_kind):
            packed, scales, biases = self.q4(layer, kind)
            to_float = lambda bits: (bits.astype(np.uint32) << 16).view(np.float32)
            values = dequant_mlx4(packed, to_float(scales), to_float(biases), packed.shape[1] * 8)
            self.set_gguf(layer, kind, gguf_kind, quantize_gguf(gguf_kind, values))
        for layer in range(self.g.layers):
            for kind in (["q", "k", "v", "o"] if self.full(layer) else ["qkv", "z", "a", "b", "out"]) + ["gate", "up", "down"]:
                convert(layer, kind, block_kind)
        convert(-1, "embed", head_kind)
        convert(-1, "head", head_kind)
        return self

    def vec(self, layer, kind):
        p, n = C.c_void_p(), C.c_int()
        if lib().orc_model_vec(self.handle, layer, VEC_KINDS.index(kind), C.byref(p), C.byref(n)):
            return None
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint16)), (n.value,))


class Engine:
    """The oracle's device-state stand-in: KV pools, recurrent state, conv history, journal."""

    def __init__(self, model, max_slots, kv_pages, max_pages, state_units):
        self.model = model
        self.shape = (max_slots, kv_pages, max_pages, state_units)
        self.handle = lib().orc_engine_create(model.handle, max_slots, kv_pages, max_pages, state_units)

    def __del__(self):
        if getattr(self, "handle", None):
            lib().orc_engine_destroy(self.handle); self.handle = None

    def reset_slot(self, slot, unit):
        lib().orc_engine_reset_slot(self.handle, slot, unit)

    def buffer(self, which, index):
        names = ["state", "conv", "journal", "k_codes", "v_codes", "k_scale", "v_scale"]
        n = C.c_size_t()
        p = lib().orc_engine_buffer(self.handle, names.index(which), index, C.byref(n))
        dtype = np.int8 if which in ("k_codes", "v_codes") else np.float32
        count = n.value // np.dtype(dtype).itemsize
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_int8 if dtype == np.int8 else C.c_float)), (count,))

    @staticmethod
    def _ctables(t):
        keep = [np.ascontiguousarray(getattr(t, n), np.uint32) for n in
                ("tokens", "row_slot", "row_pos", "runs", "run_info", "row_read", "row_write", "gather_index", "attn_blocks", "page_table")]
        ct = _CTables(t.rows, t.run_count, t.logit_rows, t.attn_block_count, t.step_pages, t.live_rows, t.spans, t.pages_per_span,
                      *[a.ctypes.data_as(C.POINTER(C.c_uint32)) for a in keep])
        return ct, keep

    def attention_scan(self, t: Tables, full_index, live, q, qproj):
        """The span scan and merge of one attention layer over the pool as it stands: q [live, heads, head_dim] prepared
        queries, qproj [rows, heads, 2 head_dim]. Returns (partials [live, heads, spans, head_dim + 2], merged [live, heads * head_dim])."""
        g = self.model.g
        ct, keep = self._ctables(t)
        q = np.ascontiguousarray(q, np.float32); qproj = np.ascontiguousarray(qproj, np.float32)
        partials = np.zeros((live, g.heads, t.spans, g.head_dim + 2), np.float32)
        merged = np.zeros((live, g.heads * g.head_dim), np.float32)
        rc = lib().orc_attention_scan(self.handle, full_index, C.byref(ct), live, _ptr(q), _ptr(qproj), _ptr(partials), _ptr(merged))
        assert rc == 0
        return partials, merged

    def step(self, t: Tables, taps=False, max_layers=-1):
        g = self.model.g
        ct, keep = self._ctables(t)
        logits = np.zeros((t.logit_rows, g.vocab), np.float32)
        hidden = np.zeros((g.layers, t.rows, g.hidden), np.float32) if taps else None
        rc = lib().orc_step(self.handle, C.byref(ct), _ptr(logits), None if hidden is None else _ptr(hidden), max_layers)
        assert rc == 0
        return (logits, hidden) if taps else logits


def set_norm_contract(deferred):
    """True (the default): norms after the first are the reference's deferred form (Sources/Shaders/engine_na.metal:365-415:
    the operand is bf16(h w), the consumer multiplies its sums by the row's rsqrt). False: the plain RMSNorm before rounding
    (Sources/Shaders/engine.metal:159-178)."""
    lib().orc_set_norm_contract(1 if deferred else 0)


def argmax(logits, limit):
    logits = np.ascontiguousarray(logits, np.float32)
    return np.array([lib().orc_argmax(_ptr(logits[i]), limit) for i in range(logits.shape[0])], np.int32)
