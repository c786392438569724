"""The DFlash 2 block-diffusion drafter (Sources/SploshRuntime/DraftModel.swift) over libsploshcuda's spl_draft_* entry points:
the same names and argument meaning as the reference's DraftModel (DraftRequest, DraftProposal, pushContext, propose,
resetSlot, truncate, contextLength). No CPU fallback: the passes run on the engine's device."""
import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from .engine import EngineError, lib, _ptr


class _Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("layers", "heads", "kv_heads", "group_size", "rank", "window", "ring_capacity", "block_size", "max_block",
                                        "candidates", "mask_token", "minmax_ranges")]


class _Request(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("slot", "anchor", "start", "block", "isolate_prefix")]


class _Entry(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("slot", "position", "engine_row")]


@dataclass
class DraftConfig:
    """The reference's constants (DraftModel.swift:67-82) as defaults."""
    layers: int = 5
    heads: int = 32
    kv_heads: int = 8
    group_size: int = 16
    rank: int = 256
    window: int = 2048
    ring_capacity: int = 2304
    block_size: int = 8
    max_block: int = 16
    candidates: int = 16
    mask_token: int = 248070
    minmax_ranges: bool = False


@dataclass
class DraftRequest:
    """DraftRequest (DraftModel.swift:29-42): `block - 1` tokens after `anchor`, which sits at position `start`."""
    slot: int
    anchor: int
    start: int
    block: int = 8
    isolate_prefix: bool = False


@dataclass
class DraftProposal:
    """DraftProposal (DraftModel.swift:44-64)."""
    tokens: List[int]
    candidates: List[List[int]]
    probabilities: Optional[List[List[float]]] = None


def quantize_q4(bf16_bits, fitted=True):
    """DraftModel.quantize (:635-680) on row-major bf16 bits [rows][inner]: packed words, scales and biases (bf16 bits)."""
    src = np.ascontiguousarray(bf16_bits, np.uint16)
    rows, inner = src.shape
    packed = np.empty((rows, inner // 8), np.uint32); scales = np.empty((rows, inner // 64), np.uint16); biases = np.empty((rows, inner // 64), np.uint16)
    status = lib().spl_draft_quantize_q4(_ptr(src), rows, inner, int(fitted), _ptr(packed), _ptr(scales), _ptr(biases))
    if status:
        raise EngineError(status, "spl_draft_quantize_q4")
    return packed, scales, biases


def select(ids, values, hidden_rows, hidden_projection, predecessor, successor, anchor, temperature=0.0, random_state=0):
    """CandidateSelector.select (:479-531) for one request. Returns (tokens, probabilities or None, the advanced random state)."""
    ids = np.ascontiguousarray(ids, np.int32); values = np.ascontiguousarray(values, np.float32)
    hidden_rows = np.ascontiguousarray(hidden_rows, np.float32); hidden_projection = np.ascontiguousarray(hidden_projection, np.float32)
    predecessor = np.ascontiguousarray(predecessor, np.uint16); successor = np.ascontiguousarray(successor, np.uint16)
    drafted, k = ids.shape
    rank, hidden = hidden_projection.shape
    tokens = np.empty(drafted, np.int32)
    probabilities = np.empty((drafted, k), np.float32) if temperature > 0 else None
    state = C.c_uint64(random_state)
    status = lib().spl_draft_select(drafted, k, rank, hidden, anchor, _ptr(ids), _ptr(values), _ptr(hidden_rows), _ptr(hidden_projection), _ptr(predecessor),
                                    _ptr(successor), C.c_float(temperature), C.cast(C.byref(state), C.c_void_p), _ptr(tokens),
                                    _ptr(probabilities) if probabilities is not None else None)
    if status:
        raise EngineError(status, "spl_draft_select")
    return tokens, probabilities, state.value


class DraftModel:
    def __init__(self, engine, config=None):
        self.engine = engine
        self.config = config or DraftConfig()
        c = self.config
        cfg = _Config(c.layers, c.heads, c.kv_heads, c.group_size, c.rank, c.window, c.ring_capacity, c.block_size, c.max_block, c.candidates, c.mask_token,
                      int(c.minmax_ranges))
        handle = C.c_void_p()
        engine._check(lib().spl_draft_create(engine.handle, C.byref(cfg), C.byref(handle)))
        self.handle = handle
        self.random_state = 0

    def close(self):
        if getattr(self, "handle", None):
            lib().spl_draft_destroy(self.handle); self.handle = None

    def __del__(self):
        self.close()

    def set_tensor(self, name, bf16_bits):
        """One tensor of the checkpoint by its safetensors name, as bf16 bits (a vector, or [rows][inner])."""
        bits = np.ascontiguousarray(bf16_bits, np.uint16)
        rows, inner = (1, bits.size) if bits.ndim == 1 else (bits.shape[0], int(np.prod(bits.shape[1:])))
        self.engine._check(lib().spl_draft_set_tensor(self.handle, name.encode(), _ptr(bits), rows, inner))

    def load_safetensors(self, path):
        """DraftModel.init(engine:safetensorsURL:): every tensor of the bf16 checkpoint at `path`."""
        message = C.create_string_buffer(512)
        status = lib().spl_draft_load_safetensors(self.handle, str(path).encode(), message, len(message))
        if status:
            raise EngineError(status, message.value.decode())

    def expected_tensors(self):
        """(name, shape) of every tensor the drafter asks for, in the reference's order."""
        out = []
        for index in range(lib().spl_draft_tensor_count(self.handle)):
            name = C.create_string_buffer(160); shape = (C.c_int64 * 4)(); nd = C.c_int32()
            self.engine._check(lib().spl_draft_tensor_expected(self.handle, index, name, len(name), C.cast(shape, C.c_void_p), C.cast(C.byref(nd), C.c_void_p)))
            out.append((name.value.decode(), tuple(shape[i] for i in range(nd.value))))
        return out

    def export_context(self, slot, token_count):
        """DraftModel.exportContext: (first, end, rings) for a prefix of `token_count` tokens, or None when nothing useful is held."""
        rings = np.empty(lib().spl_draft_context_bytes(self.handle), np.uint8)
        first, end = C.c_int32(), C.c_int32()
        self.engine._check(lib().spl_draft_export_context(self.handle, slot, token_count, C.cast(C.byref(first), C.c_void_p), C.cast(C.byref(end), C.c_void_p), _ptr(rings)))
        return None if first.value < 0 else (first.value, end.value, rings)

    def import_context(self, slot, snapshot):
        first, end, rings = snapshot
        rings = np.ascontiguousarray(rings, np.uint8)
        self.engine._check(lib().spl_draft_import_context(self.handle, slot, first, end, _ptr(rings), rings.nbytes))

    def reset_slot(self, slot):
        self.engine._check(lib().spl_draft_reset_slot(self.handle, slot))

    def truncate(self, slot, token_count):
        self.engine._check(lib().spl_draft_truncate(self.handle, slot, token_count))

    def context_length(self, slot, start):
        return lib().spl_draft_context_length(self.handle, slot, start)

    def push_context(self, entries):
        """DraftModel.pushContext: entries are (slot, position, engine_row) of the step that has just run."""
        arr = (_Entry * max(len(entries), 1))()
        for i, (slot, position, engine_row) in enumerate(entries):
            arr[i].slot, arr[i].position, arr[i].engine_row = slot, position, engine_row
        self.engine._check(lib().spl_draft_push_context(self.handle, C.cast(arr, C.c_void_p), len(entries)))

    def propose(self, requests, temperature=0.0, vocab_limit=None):
        """DraftModel.propose: one DraftProposal per request."""
        if not requests:
            return []
        arr = (_Request * len(requests))()
        for i, r in enumerate(requests):
            arr[i].slot, arr[i].anchor, arr[i].start, arr[i].block, arr[i].isolate_prefix = r.slot, r.anchor, r.start, r.block, int(r.isolate_prefix)
        k = self.config.candidates
        drafted = sum(max(r.block - 1, 0) for r in requests)
        tokens = np.zeros(max(drafted, 1), np.int32); candidates = np.zeros((max(drafted, 1), k), np.int32); probabilities = np.zeros((max(drafted, 1), k), np.float32)
        state = C.c_uint64(self.random_state)
        limit = vocab_limit if vocab_limit is not None else self.engine.g.vocab
        self.engine._check(lib().spl_draft_propose(self.handle, C.cast(arr, C.c_void_p), len(requests), C.c_float(temperature), limit, C.cast(C.byref(state), C.c_void_p),
                                                   _ptr(tokens), _ptr(candidates), _ptr(probabilities)))
        self.random_state = state.value
        out, at = [], 0
        for r in requests:
            n = r.block - 1
            out.append(DraftProposal(tokens[at:at + n].tolist(), candidates[at:at + n].tolist(), probabilities[at:at + n].tolist() if temperature > 0 else None))
            at += n
        return out

    def debug_read(self, what, shape, dtype=np.float32, index=0):
        out = np.empty(shape, dtype)
        self.engine._check(lib().spl_draft_debug_read(self.handle, what, index, _ptr(out), out.nbytes))
        return out
