"""ctypes host over libsploshcuda.so, mirroring the reference's `Engine` API
(Sources/SploshRuntime/Engine.swift:19-108 types, :810-868 slot lifecycle, :1316 step,
:1202-1205 logits) so tests read like the reference's own drivers
(Sources/SploshCLI/GenerateCommand.swift:375-469)."""
import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def library_path():
    return os.path.join(_HERE, "libsploshcuda.so")


class Geometry(C.Structure):
    """ModelGeometry (Sources/SploshModel/ModelWeights.swift:66-88) as a parameter."""
    _fields_ = [(n, C.c_int32) for n in ("layers", "hidden", "inter", "vocab", "heads", "kv_heads", "head_dim", "rotary_dim",
                                         "gdn_key_heads", "gdn_value_heads", "gdn_head_dim")] + [("eps", C.c_float), ("rope_theta", C.c_float)]

    @property
    def channels(self):
        return (2 * self.gdn_key_heads + self.gdn_value_heads) * self.gdn_head_dim

    @property
    def value_dim(self):
        return self.gdn_value_heads * self.gdn_head_dim


def tiny_geometry():
    return Geometry(4, 1024, 2816, 32000, 8, 2, 128, 32, 4, 8, 128, 1e-6, 1e7)


def b27_geometry(layers=64, vocab=248320):
    return Geometry(layers, 5120, 17408, vocab, 24, 4, 256, 64, 16, 48, 128, 1e-6, 1e7)


class _Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("device", "max_slots", "max_rows", "kv_pages", "max_context", "state_units",
                                         "max_logit_rows", "span_target")]


class _Row(C.Structure):
    _fields_ = [("slot", C.c_int32), ("token", C.c_int32), ("position", C.c_int32), ("want_logits", C.c_uint8),
                ("verify", C.c_uint8), ("reserved", C.c_uint8 * 2)]


class _Tables(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("rows", "run_count", "logit_rows", "attn_block_count", "step_pages", "live_rows",
                                          "spans", "pages_per_span")] + \
               [(n, C.POINTER(C.c_uint32)) for n in ("tokens", "row_slot", "row_pos", "runs", "run_info", "row_read", "row_write",
                                                     "gather_index", "attn_blocks", "page_table")]


class _Session(C.Structure):
    _fields_ = [("slot", C.c_int32), ("evaluated", C.c_int32), ("pending", C.c_int32), ("proposal", C.POINTER(C.c_int32)), ("proposal_count", C.c_int32),
                ("prompt", C.POINTER(C.c_int32)), ("prompt_count", C.c_int32), ("fed", C.c_int32), ("marks", C.POINTER(C.c_int32)),
                ("mark_count", C.c_int32), ("block_yield", C.c_double)]


class _PackConfig(C.Structure):
    _fields_ = [("block", C.c_int32), ("max_verify_rows", C.c_int32), ("speculate", C.c_int32), ("prefill_rows_while_decoding", C.c_int32),
                ("decode_weight", C.c_double), ("costs", C.c_void_p)]


class _Planned(C.Structure):
    _fields_ = [("kind", C.c_int32), ("session", C.c_int32), ("count", C.c_int32), ("complete", C.c_int32)]


@dataclass
class PackSession:
    """What the row packer reads of a session (BatchScheduler.swift:1323-1442)."""
    slot: int
    evaluated: int
    pending: int = None            # None while the prompt is being fed
    proposal: tuple = ()
    prompt: tuple = ()
    fed: int = 0
    marks: tuple = ()
    block_yield: float = 0.0


class _Stats(C.Structure):
    _fields_ = [("rows", C.c_int32), ("launches", C.c_int32), ("gpu_seconds", C.c_double), ("wall_seconds", C.c_double)]


class _Memory(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("weight_bytes", "kv_pool_bytes", "kv_bytes_per_page", "kv_pages_total", "kv_pages_used",
                                         "state_bytes_per_slot", "state_bytes_total", "state_units_used", "scratch_bytes",
                                         "device_total_bytes", "device_free_bytes")]


STATUS_NAMES = ["ok", "kvPoolExhausted", "contextExceeded", "unsupportedDevice", "allocationFailed", "invalidRows",
                "snapshotMismatch", "invalidKernelChoice", "device", "timeout", "invalidArgument"]
Q4_KINDS = ["qkv", "z", "a", "b", "out", "q", "k", "v", "o", "gate", "up", "down", "embed", "head"]
VEC_KINDS = ["input_norm", "post_norm", "conv", "a_log", "dt_bias", "gdn_norm", "q_norm", "k_norm", "final_norm"]


class EngineError(Exception):
    """EngineError (Engine.swift:88-108): `.case` holds the Swift case name."""

    def __init__(self, status, message):
        self.status = status
        self.case = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"{self.case}: {message}")


@dataclass
class EngineConfig:
    max_slots: int = 8
    max_rows: int = 64
    kv_pages: int = 256
    max_context: int = 32768
    state_units: int = 0
    max_logit_rows: int = 0
    span_target: int = 0
    device: int = 0

    def c(self):
        return _Config(self.device, self.max_slots, self.max_rows, self.kv_pages, self.max_context, self.state_units,
                       self.max_logit_rows, self.span_target)


@dataclass
class EngineRow:
    slot: int
    token: int
    position: int
    want_logits: bool
    verify: bool = False


@dataclass
class StepStats:
    rows: int
    launches: int
    gpu_seconds: float
    wall_seconds: float


def lib():
    """Load the C-ABI library. Fails loudly when it is missing: there is no other path."""
    global _LIB
    if _LIB is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: build it with `make -C splosh_b200/csrc` (or __graft_entry__.build())")
        L = C.CDLL(path)
        vp, i32, u64 = C.c_void_p, C.c_int32, C.c_uint64
        sig = {
            "spl_host_create": (i32, [C.POINTER(Geometry), C.POINTER(_Config), C.POINTER(vp)]),
            "spl_host_destroy": (None, [vp]),
            "spl_host_build_tables": (i32, [vp, C.POINTER(_Row), i32, C.POINTER(_Tables)]),
            "spl_host_finish_step": (None, [vp, C.POINTER(_Tables)]),
            "spl_host_reset_slot": (i32, [vp, i32]),
            "spl_host_discard_verify": (None, [vp, i32]),
            "spl_host_accept_verify": (i32, [vp, i32, i32, i32]),
            "spl_host_truncate": (None, [vp, i32, i32]),
            "spl_host_pages_held": (i32, [vp, i32]),
            "spl_host_free_page_count": (i32, [vp]),
            "spl_host_slot_unit": (i32, [vp, i32]),
            "spl_host_journal_pending": (i32, [vp, i32]),
            "spl_host_max_pages": (i32, [vp]),
            "spl_host_last_error": (C.c_char_p, [vp]),
            "spl_greedy_accept": (i32, [vp, vp, i32, C.POINTER(i32)]),
            "spl_host_pack_rows": (i32, [vp, vp, i32, vp, vp, vp, C.POINTER(i32), vp, C.POINTER(i32)]),
            "spl_engine_create": (i32, [C.POINTER(Geometry), C.POINTER(_Config), C.POINTER(vp)]),
            "spl_engine_destroy": (None, [vp]),
            "spl_last_error_string": (C.c_char_p, [vp]),
            "spl_weights_set_q4": (i32, [vp, i32, i32, i32, i32, vp, vp, vp]),
            "spl_weights_set_vector": (i32, [vp, i32, i32, vp, i32]),
            "spl_weights_synthesize_q4": (i32, [vp, u64]),
            "spl_weights_set_gguf": (i32, [vp, i32, i32, i32, i32, i32, vp]),
            "spl_tensor_create_q4": (i32, [vp, i32, i32, vp, vp, vp, C.POINTER(vp)]),
            "spl_tensor_create_vector": (i32, [vp, vp, i32, C.POINTER(vp)]),
            "spl_tensor_destroy": (None, [vp, vp]),
            "spl_pass_begin": (i32, [vp]),
            "spl_pass_gemm": (i32, [vp, vp, vp, i32, vp, vp]),
            "spl_pass_gemm_head": (i32, [vp, vp, i32, vp]),
            "spl_pass_norm": (i32, [vp, vp, vp, i32, i32, vp]),
            "spl_pass_embed": (i32, [vp, vp, i32, vp]),
            "spl_pass_mlp_in": (i32, [vp, vp, vp, vp, i32, vp, vp]),
            "spl_pass_wait": (i32, [vp]),
            "spl_weights_synthesize_gguf": (i32, [vp, u64, i32, i32]),
            "spl_weights_gguf_file_order": (i32, [vp, i32]),
            "spl_weights_load_gguf_file": (i32, [vp, C.c_char_p, C.c_char_p, C.c_size_t]),
            "spl_weights_load_splw_file": (i32, [vp, C.c_char_p, C.c_char_p, C.c_size_t]),
            "spl_splw_check": (i32, [C.c_char_p, C.POINTER(C.c_int32), C.c_char_p, C.c_size_t]),
            "spl_gguf_planes_unpack": (i32, [i32, vp, vp, vp, i32, i32, vp]),
            "spl_step": (i32, [vp, C.POINTER(_Row), i32, C.POINTER(_Stats)]),
            "spl_step_launch": (i32, [vp, C.POINTER(_Row), i32]),
            "spl_step_wait": (i32, [vp, C.POINTER(_Stats)]),
            "spl_step_tables": (i32, [vp, C.POINTER(_Tables), C.POINTER(_Stats)]),
            "spl_logits_row": (i32, [vp, i32, vp]),
            "spl_argmax": (i32, [vp, i32, vp]),
            "spl_slot_reset": (i32, [vp, i32]),
            "spl_verify_discard": (i32, [vp, i32]),
            "spl_verify_accept": (i32, [vp, i32, i32, i32]),
            "spl_slot_truncate": (i32, [vp, i32, i32]),
            "spl_pages_held": (i32, [vp, i32]),
            "spl_free_page_count": (i32, [vp]),
            "spl_memory": (i32, [vp, C.POINTER(_Memory)]),
            "spl_engine_host": (vp, [vp]),
            "spl_warmup": (i32, [vp]),
            "spl_debug_fill_kv": (i32, [vp, i32]),
            "spl_debug_fill_state": (i32, [vp, i32, u64]),
            "spl_debug_read": (i32, [vp, i32, i32, vp, C.c_size_t]),
            "spl_debug_taps": (i32, [vp, i32]),
            "spl_debug_kv_store": (i32, [vp, i32]),
            "spl_debug_gdn_chunk_min": (i32, [vp, i32]),
            "spl_debug_pair_blocks": (i32, [vp, i32]),
            "spl_debug_wait_budget": (i32, [vp, C.c_int64]),
            "spl_debug_drop_weight_stage": (i32, [vp, i32]),
            "spl_gemm_q4_static_status": (i32, [vp]),
            "spl_op_gemm_gguf": (i32, [i32, i32, vp, i32, i32, vp, i32, vp, vp]),
            "spl_state_bytes": (C.c_size_t, [vp]),
            "spl_state_export": (i32, [vp, i32, vp, C.c_size_t]),
            "spl_state_import": (i32, [vp, i32, vp, C.c_size_t]),
            "spl_kv_bytes": (C.c_size_t, [vp, i32]),
            "spl_kv_export": (i32, [vp, i32, i32, vp, C.c_size_t]),
            "spl_kv_import": (i32, [vp, i32, i32, vp, C.c_size_t]),
            "spl_plan_costs_reference": (None, [vp]),
            "spl_plan_costs_b200": (None, [vp]),
            "spl_plan_tier": (i32, [i32]),
            "spl_plan_cycle_ms": (C.c_double, [vp, i32]),
            "spl_plan_prefill_cap": (i32, [vp, i32, i32, C.c_double, C.c_double, C.c_double, i32, i32, i32]),
            "spl_plan_blocks": (i32, [vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]),
            "spl_topk": (i32, [vp, i32, i32, vp, vp]),
            "spl_sampler_uniform": (C.c_float, [vp]),
            "spl_sample_topk": (i32, [vp, vp, i32, C.c_float, C.c_float, vp]),
            "spl_sampler_distribution": (i32, [vp, i32, C.c_float, C.c_float, vp]),
            "spl_speculative_resolve": (i32, [i32, vp, vp, i32, vp, vp, i32, vp]),
            "spl_features_enable": (i32, [vp, vp, i32]),
            "spl_feature_width": (i32, [vp]),
            "spl_feature_row": (i32, [vp, i32, vp]),
            "spl_debug_profile": (i32, [vp, i32]),
            "spl_debug_profile_read": (i32, [vp, i32, C.POINTER(C.c_double), C.POINTER(C.c_int64), C.POINTER(C.c_double)]),
            "spl_op_gemm_q4": (i32, [i32, vp, vp, vp, i32, i32, vp, i32, vp, vp]),
            "spl_gemm_q4_static": (i32, [vp, i32, i32, vp, i32, vp, vp, vp]),
            "spl_draft_create": (i32, [vp, vp, vp]),
            "spl_draft_destroy": (None, [vp]),
            "spl_draft_set_tensor": (i32, [vp, C.c_char_p, vp, i32, i32]),
            "spl_draft_reset_slot": (i32, [vp, i32]),
            "spl_draft_truncate": (i32, [vp, i32, i32]),
            "spl_draft_context_length": (i32, [vp, i32, i32]),
            "spl_draft_push_context": (i32, [vp, vp, i32]),
            "spl_draft_propose": (i32, [vp, vp, i32, C.c_float, i32, vp, vp, vp, vp]),
            "spl_draft_quantize_q4": (i32, [vp, i32, i32, i32, vp, vp, vp]),
            "spl_draft_select": (i32, [i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, C.c_float, vp, vp, vp]),
            "spl_draft_debug_read": (i32, [vp, i32, i32, vp, C.c_uint64]),
            "spl_draft_load_safetensors": (i32, [vp, C.c_char_p, C.c_char_p, C.c_size_t]),
            "spl_draft_tensor_count": (i32, [vp]),
            "spl_draft_tensor_expected": (i32, [vp, i32, C.c_char_p, C.c_uint64, vp, vp]),
            "spl_draft_context_bytes": (C.c_uint64, [vp]),
            "spl_draft_export_context": (i32, [vp, i32, i32, vp, vp, vp]),
            "spl_draft_import_context": (i32, [vp, i32, i32, i32, vp, C.c_uint64]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _LIB = L
    return _LIB


EXPORTS = None  # filled by tests from include/splosh_cuda.h


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def _rows_array(rows):
    arr = (_Row * len(rows))()
    for i, r in enumerate(rows):
        arr[i].slot, arr[i].token, arr[i].position = r.slot, r.token, r.position
        arr[i].want_logits, arr[i].verify = int(bool(r.want_logits)), int(bool(r.verify))
    return arr


def _tables_dict(t, max_slots, max_pages):
    def arr(p, n):
        return np.ctypeslib.as_array(p, (n,)).copy() if n else np.zeros(0, np.uint32)
    return dict(rows=t.rows, step_pages=t.step_pages, live_rows=t.live_rows, spans=t.spans, pages_per_span=t.pages_per_span,
                tokens=arr(t.tokens, t.rows), row_slot=arr(t.row_slot, t.rows), row_pos=arr(t.row_pos, t.rows),
                runs=arr(t.runs, t.run_count * 3), run_info=arr(t.run_info, t.run_count * 2),
                row_read=arr(t.row_read, t.rows), row_write=arr(t.row_write, t.rows),
                gather_index=arr(t.gather_index, t.logit_rows), attn_blocks=arr(t.attn_blocks, t.attn_block_count * 2),
                page_table=arr(t.page_table, max_slots * max_pages).reshape(max_slots, max_pages))


class Host:
    """The host bookkeeping on its own (no GPU): page allocator, state units, table builder."""

    def __init__(self, geometry, config, handle=None):
        self.g, self.config = geometry, config
        self._own = handle is None
        if handle is None:
            h = C.c_void_p()
            cfg = config.c()
            status = lib().spl_host_create(C.byref(geometry), C.byref(cfg), C.byref(h))
            if status:
                raise EngineError(status, "invalid host configuration")
            handle = h
        self.handle = handle
        self.last = None

    def __del__(self):
        if getattr(self, "_own", False) and self.handle:
            lib().spl_host_destroy(self.handle); self.handle = None

    @property
    def max_pages(self):
        return lib().spl_host_max_pages(self.handle)

    def build(self, rows):
        t = _Tables()
        arr = _rows_array(rows)
        status = lib().spl_host_build_tables(self.handle, arr, len(rows), C.byref(t))
        if status:
            raise EngineError(status, lib().spl_host_last_error(self.handle).decode())
        self.last = t
        return _tables_dict(t, self.config.max_slots, self.max_pages)

    def finish_step(self):
        lib().spl_host_finish_step(self.handle, C.byref(self.last))

    def pack_rows(self, sessions, planner, block=8, max_verify_rows=64, speculate=True, prefill_rows_while_decoding=8, decode_weight=1.0):
        """BatchScheduler.buildRows: (rows, plan, waiting) for PackSession objects in the scheduler's order; plan entries are
        (kind, session index, count, complete) with kind 0 verify, 1 decode, 2 prefill."""
        n = len(sessions)
        arr = (_Session * max(n, 1))()
        keep = []
        for i, s in enumerate(sessions):
            bufs = [np.ascontiguousarray(x, np.int32) for x in (s.proposal, s.prompt, s.marks)]
            keep.append(bufs)
            arr[i].slot, arr[i].evaluated, arr[i].pending = s.slot, s.evaluated, -1 if s.pending is None else s.pending
            arr[i].proposal, arr[i].proposal_count = bufs[0].ctypes.data_as(C.POINTER(C.c_int32)), len(bufs[0])
            arr[i].prompt, arr[i].prompt_count, arr[i].fed = bufs[1].ctypes.data_as(C.POINTER(C.c_int32)), len(bufs[1]), s.fed
            arr[i].marks, arr[i].mark_count = bufs[2].ctypes.data_as(C.POINTER(C.c_int32)), len(bufs[2])
            arr[i].block_yield = s.block_yield
        cfg = _PackConfig(block, max_verify_rows, int(speculate), prefill_rows_while_decoding, decode_weight, C.addressof(planner.costs))
        rows = (_Row * self.config.max_rows)(); plan = (_Planned * max(n, 1))(); waiting = (C.c_int32 * max(n, 1))()
        plan_count, waiting_count = C.c_int32(), C.c_int32()
        count = lib().spl_host_pack_rows(self.handle, arr, n, C.byref(cfg), rows, plan, C.byref(plan_count), waiting, C.byref(waiting_count))
        if count < 0:
            raise EngineError(10, "spl_host_pack_rows: bad argument")
        out = [EngineRow(rows[i].slot, rows[i].token, rows[i].position, bool(rows[i].want_logits), bool(rows[i].verify)) for i in range(count)]
        return out, [(plan[i].kind, plan[i].session, plan[i].count, plan[i].complete) for i in range(plan_count.value)], list(waiting[:waiting_count.value])

    def reset_slot(self, slot):
        return lib().spl_host_reset_slot(self.handle, slot)

    def discard_verify(self, slot):
        lib().spl_host_discard_verify(self.handle, slot)

    def accept_verify(self, slot, rows, token_count):
        status = lib().spl_host_accept_verify(self.handle, slot, rows, token_count)
        if status:
            raise EngineError(status, lib().spl_host_last_error(self.handle).decode())

    def truncate(self, slot, token_count):
        lib().spl_host_truncate(self.handle, slot, token_count)

    def pages_held(self, slot):
        return lib().spl_host_pages_held(self.handle, slot)

    @property
    def free_page_count(self):
        return lib().spl_host_free_page_count(self.handle)

    def slot_unit(self, slot):
        return lib().spl_host_slot_unit(self.handle, slot)

    def journal_pending(self, slot):
        return lib().spl_host_journal_pending(self.handle, slot)


class PlanCosts(C.Structure):
    """spl_plan_costs: the width planner's cost table (BatchScheduler.swift:740-750)."""
    _fields_ = [("tier_ms", C.c_double * 5), ("beyond_ms_per_row", C.c_double), ("per_row_ms", C.c_double), ("fixed_ms", C.c_double),
                ("attention_first", C.c_double), ("attention_second", C.c_double), ("prefill_attention", C.c_double), ("tier_margin", C.c_double)]


class Planner:
    """prefillCap and planBlocks (BatchScheduler.swift:646-669, 751-789) over a cost table: the reference's or this
    library's measured one."""

    def __init__(self, costs="b200"):
        self.costs = PlanCosts()
        (lib().spl_plan_costs_reference if costs == "reference" else lib().spl_plan_costs_b200)(C.byref(self.costs))

    @staticmethod
    def tier(rows):
        return lib().spl_plan_tier(rows)

    def cycle_ms(self, rows):
        return lib().spl_plan_cycle_ms(C.byref(self.costs), rows)

    def prefill_cap(self, max_rows, decode_rows, decode_tokens, decode_attention_ms, backlog, first_fed, decode_weight=1.0, prefill_rows_while_decoding=8):
        return lib().spl_plan_prefill_cap(C.byref(self.costs), max_rows, decode_rows, decode_tokens, decode_attention_ms, decode_weight,
                                          backlog, first_fed, prefill_rows_while_decoding)

    def blocks(self, tail, block_yield, context_tokens, other_rows=0, block=8, max_rows=128, max_logit_rows=128, max_verify_rows=64, max_context=262144):
        t = np.ascontiguousarray(tail, np.float64); y = np.ascontiguousarray(block_yield, np.float64); c = np.ascontiguousarray(context_tokens, np.int32)
        out = np.zeros(len(t), np.int32)
        lib().spl_plan_blocks(C.byref(self.costs), len(t), _ptr(t), _ptr(y), _ptr(c), other_rows, block, max_rows, max_logit_rows, max_verify_rows,
                              max_context, _ptr(out))
        return [int(x) for x in out]


class Sampler:
    """Sampler (Sampler.swift:68-156) over the k largest logits that `Engine.topk` returns; the state is SplitMix64."""

    def __init__(self, temperature=1.0, top_p=0.95, top_k=20, seed=1):
        self.temperature, self.top_p, self.top_k = float(temperature), float(top_p), int(top_k)
        self.state = C.c_uint64(seed)

    def uniform01(self):
        return float(lib().spl_sampler_uniform(C.byref(self.state)))

    def sample(self, ids, values):
        ids = np.ascontiguousarray(ids, np.int32); values = np.ascontiguousarray(values, np.float32)
        return int(lib().spl_sample_topk(_ptr(ids), _ptr(values), len(ids), self.temperature, self.top_p, C.byref(self.state)))

    def distribution(self, ids, values):
        values = np.ascontiguousarray(values, np.float32)
        out = np.empty(len(values), np.float32)
        kept = lib().spl_sampler_distribution(_ptr(values), len(values), self.temperature, self.top_p, _ptr(out))
        return list(np.asarray(ids)[:kept]), out[:kept]

    def resolve(self, draft, candidates, draft_probabilities, target_ids, target_probabilities):
        """SpeculativeSampling.resolve (Sampler.swift:163-179): None when the draft is kept, else its replacement."""
        c = np.ascontiguousarray(candidates, np.int32); q = np.ascontiguousarray(draft_probabilities, np.float32)
        t = np.ascontiguousarray(target_ids, np.int32); pr = np.ascontiguousarray(target_probabilities, np.float32)
        out = lib().spl_speculative_resolve(int(draft), _ptr(c), _ptr(q), len(c), _ptr(t), _ptr(pr), len(t), C.byref(self.state))
        return None if out == -1 else int(out)


def greedy_accept(argmax_ids, drafts):
    """BatchScheduler.accept, greedy branch (BatchScheduler.swift:1583-1587)."""
    ids = np.ascontiguousarray(argmax_ids, np.int32); d = np.ascontiguousarray(drafts, np.int32)
    bonus = C.c_int32()
    agreed = lib().spl_greedy_accept(_ptr(ids), _ptr(d), len(d), C.byref(bonus))
    return agreed, bonus.value


class Engine:
    """Engine (Engine.swift:123): one per GPU, owned by one thread."""

    def __init__(self, geometry, config=None):
        self.g = geometry
        self.config = config or EngineConfig()
        h = C.c_void_p()
        cfg = self.config.c()
        status = lib().spl_engine_create(C.byref(geometry), C.byref(cfg), C.byref(h))
        self.handle = h
        if status:
            message = lib().spl_last_error_string(h).decode() if h else ""
            lib().spl_engine_destroy(h); self.handle = None
            raise EngineError(status, message)
        self.host = Host(geometry, self.config, handle=C.c_void_p(lib().spl_engine_host(self.handle)))
        self.last_logit_rows = 0

    def close(self):
        if getattr(self, "handle", None):
            lib().spl_engine_destroy(self.handle); self.handle = None

    def __del__(self):
        self.close()

    def _check(self, status):
        if status:
            raise EngineError(status, lib().spl_last_error_string(self.handle).decode())

    # ---- weights
    def set_q4(self, layer, kind, packed, scales, biases):
        packed = np.ascontiguousarray(packed, np.uint32); scales = np.ascontiguousarray(scales, np.uint16); biases = np.ascontiguousarray(biases, np.uint16)
        self._check(lib().spl_weights_set_q4(self.handle, layer, Q4_KINDS.index(kind), packed.shape[0], packed.shape[1] * 8,
                                              _ptr(packed), _ptr(scales), _ptr(biases)))

    def set_vector(self, layer, kind, bits):
        bits = np.ascontiguousarray(bits, np.uint16)
        self._check(lib().spl_weights_set_vector(self.handle, layer, VEC_KINDS.index(kind), _ptr(bits), bits.size))

    def synthesize_q4(self, seed):
        self._check(lib().spl_weights_synthesize_q4(self.handle, seed))

    # ---- the engine's primitives on device buffers (what the drafter builds its passes from); addresses are ints
    def tensor_q4(self, packed, scales, biases):
        packed = np.ascontiguousarray(packed, np.uint32); scales = np.ascontiguousarray(scales, np.uint16); biases = np.ascontiguousarray(biases, np.uint16)
        out = C.c_void_p()
        self._check(lib().spl_tensor_create_q4(self.handle, packed.shape[0], packed.shape[1] * 8, _ptr(packed), _ptr(scales), _ptr(biases), C.byref(out)))
        return out

    def tensor_vector(self, bits):
        bits = np.ascontiguousarray(bits, np.uint16)
        out = C.c_void_p()
        self._check(lib().spl_tensor_create_vector(self.handle, _ptr(bits), bits.size, C.byref(out)))
        return out

    def tensor_destroy(self, tensor):
        lib().spl_tensor_destroy(self.handle, tensor)

    def pass_begin(self):
        self._check(lib().spl_pass_begin(self.handle))

    def pass_gemm(self, tensor, device_in, rows, device_out, device_residual=None):
        self._check(lib().spl_pass_gemm(self.handle, tensor, C.c_void_p(device_in), rows, C.c_void_p(device_residual) if device_residual else None, C.c_void_p(device_out)))

    def pass_gemm_head(self, device_in, rows, device_out):
        self._check(lib().spl_pass_gemm_head(self.handle, C.c_void_p(device_in), rows, C.c_void_p(device_out)))

    def pass_norm(self, device_in, weight, rows, dim, device_out):
        self._check(lib().spl_pass_norm(self.handle, C.c_void_p(device_in), weight, rows, dim, C.c_void_p(device_out)))

    def pass_embed(self, device_tokens, rows, device_out):
        self._check(lib().spl_pass_embed(self.handle, C.c_void_p(device_tokens), rows, C.c_void_p(device_out)))

    def pass_mlp_in(self, gate, up, device_in, rows, device_out, device_scratch):
        self._check(lib().spl_pass_mlp_in(self.handle, gate, up, C.c_void_p(device_in), rows, C.c_void_p(device_out), C.c_void_p(device_scratch)))

    def pass_wait(self):
        self._check(lib().spl_pass_wait(self.handle))

    def set_gguf(self, layer, kind, gguf_kind, blocks):
        """One tensor as native GGUF K-quant super-blocks: blocks uint8 [rows, inner / 256, block bytes]; gguf_kind "Q4_K", "Q5_K" or "Q6_K"."""
        blocks = np.ascontiguousarray(blocks, np.uint8)
        self._check(lib().spl_weights_set_gguf(self.handle, layer, Q4_KINDS.index(kind), GGUF_TYPE[gguf_kind], blocks.shape[0], blocks.shape[1] * 256, _ptr(blocks)))

    def gguf_file_order(self, enabled=True):
        """The gated-delta out projections hold their columns in a GGUF file's order of the value heads."""
        self._check(lib().spl_weights_gguf_file_order(self.handle, int(enabled)))

    def load_gguf_file(self, path):
        """Every tensor of a llama.cpp GGUF file of this geometry (spl_weights_load_gguf_file)."""
        message = C.create_string_buffer(512)
        status = lib().spl_weights_load_gguf_file(self.handle, os.fsencode(path), message, len(message))
        if status:
            raise EngineError(status, message.value.decode() or "spl_weights_load_gguf_file failed")

    def load_splw_file(self, path):
        """Every tensor of an SPLW artifact of this geometry (spl_weights_load_splw_file)."""
        message = C.create_string_buffer(512)
        status = lib().spl_weights_load_splw_file(self.handle, os.fsencode(path), message, len(message))
        if status:
            raise EngineError(status, message.value.decode() or "spl_weights_load_splw_file failed")

    def synthesize_gguf(self, seed, block_kind="Q5_K", head_kind="Q6_K"):
        self._check(lib().spl_weights_synthesize_gguf(self.handle, seed, GGUF_TYPE[block_kind], GGUF_TYPE[head_kind]))

    def load_gguf_model(self, model):
        """Copy every tensor of an object with .gguf(layer, kind) -> (gguf kind, blocks) and .vec(layer, kind)."""
        for layer in range(self.g.layers):
            full = layer % 4 == 3
            for kind in (["q", "k", "v", "o"] if full else ["qkv", "z", "a", "b", "out"]) + ["gate", "up", "down"]:
                self.set_gguf(layer, kind, *model.gguf(layer, kind))
            for kind in ["input_norm", "post_norm"] + (["q_norm", "k_norm"] if full else ["conv", "a_log", "dt_bias", "gdn_norm"]):
                self.set_vector(layer, kind, model.vec(layer, kind))
        self.set_gguf(-1, "embed", *model.gguf(-1, "embed"))
        self.set_gguf(-1, "head", *model.gguf(-1, "head"))
        self.set_vector(-1, "final_norm", model.vec(-1, "final_norm"))

    def load_model(self, model):
        """Copy every tensor of an object with .q4(layer, kind) / .vec(layer, kind) (the synthetic model of the tests)."""
        for layer in range(self.g.layers):
            full = layer % 4 == 3
            for kind in (["q", "k", "v", "o"] if full else ["qkv", "z", "a", "b", "out"]) + ["gate", "up", "down"]:
                self.set_q4(layer, kind, *model.q4(layer, kind))
            for kind in ["input_norm", "post_norm"] + (["q_norm", "k_norm"] if full else ["conv", "a_log", "dt_bias", "gdn_norm"]):
                self.set_vector(layer, kind, model.vec(layer, kind))
        self.set_q4(-1, "embed", *model.q4(-1, "embed"))
        self.set_q4(-1, "head", *model.q4(-1, "head"))
        self.set_vector(-1, "final_norm", model.vec(-1, "final_norm"))

    # ---- the step
    def step(self, rows):
        stats = _Stats()
        arr = _rows_array(rows)
        self._check(lib().spl_step(self.handle, arr, len(rows), C.byref(stats)))
        self.last_logit_rows = sum(1 for r in rows if r.want_logits)
        return StepStats(stats.rows, stats.launches, stats.gpu_seconds, stats.wall_seconds)

    def step_launch(self, rows):
        """The first half of step: everything is enqueued when this returns; nothing else may be asked of the engine
        until step_wait."""
        self._flying_rows = _rows_array(rows)          # kept alive until the wait
        self._check(lib().spl_step_launch(self.handle, self._flying_rows, len(rows)))
        self._flying_logit_rows = sum(1 for r in rows if r.want_logits)

    def step_wait(self):
        stats = _Stats()
        self._check(lib().spl_step_wait(self.handle, C.byref(stats)))
        self.last_logit_rows = self._flying_logit_rows
        return StepStats(stats.rows, stats.launches, stats.gpu_seconds, stats.wall_seconds)

    def step_tables(self, tables: _Tables, logit_rows):
        stats = _Stats()
        self._check(lib().spl_step_tables(self.handle, C.byref(tables), C.byref(stats)))
        self.last_logit_rows = logit_rows
        return StepStats(stats.rows, stats.launches, stats.gpu_seconds, stats.wall_seconds)

    def logits(self, index):
        out = np.empty(self.g.vocab, np.float32)
        self._check(lib().spl_logits_row(self.handle, index, _ptr(out)))
        return out

    def all_logits(self):
        return np.stack([self.logits(i) for i in range(self.last_logit_rows)]) if self.last_logit_rows else np.zeros((0, self.g.vocab), np.float32)

    def argmax(self, vocab_limit=None):
        ids = np.zeros(max(self.last_logit_rows, 1), np.int32)
        self._check(lib().spl_argmax(self.handle, vocab_limit or self.g.vocab, _ptr(ids)))
        return ids[:self.last_logit_rows]

    # ---- slot lifecycle
    def reset_slot(self, slot):
        self._check(lib().spl_slot_reset(self.handle, slot))

    def discard_verify(self, slot):
        self._check(lib().spl_verify_discard(self.handle, slot))

    def accept_verify(self, slot, rows, token_count):
        self._check(lib().spl_verify_accept(self.handle, slot, rows, token_count))

    def truncate(self, slot, token_count):
        self._check(lib().spl_slot_truncate(self.handle, slot, token_count))

    def pages_held(self, slot):
        return lib().spl_pages_held(self.handle, slot)

    @property
    def free_page_count(self):
        return lib().spl_free_page_count(self.handle)

    @property
    def memory(self):
        m = _Memory()
        self._check(lib().spl_memory(self.handle, C.byref(m)))
        return {n: getattr(m, n) for n, _ in _Memory._fields_}

    # ---- debugging and benchmarking
    def debug_fill_kv(self, slot):
        self._check(lib().spl_debug_fill_kv(self.handle, slot))

    def debug_fill_state(self, slot, seed):
        self._check(lib().spl_debug_fill_state(self.handle, slot, seed))

    # ---- snapshots
    def export_state(self, slot):
        """Engine.exportState (Engine.swift:871-887): the slot's recurrent and conv state, journal folded in."""
        blob = np.empty(lib().spl_state_bytes(self.handle), np.uint8)
        self._check(lib().spl_state_export(self.handle, slot, _ptr(blob), blob.size))
        return blob

    def import_state(self, slot, blob):
        blob = np.ascontiguousarray(blob, np.uint8)
        self._check(lib().spl_state_import(self.handle, slot, _ptr(blob), blob.size))

    def export_kv(self, slot, token_count):
        """Engine.exportKV (Engine.swift:953-970): the pages covering the slot's first `token_count` tokens."""
        blob = np.empty(lib().spl_kv_bytes(self.handle, token_count), np.uint8)
        self._check(lib().spl_kv_export(self.handle, slot, token_count, _ptr(blob), blob.size))
        return blob

    def import_kv(self, slot, token_count, blob):
        blob = np.ascontiguousarray(blob, np.uint8)
        self._check(lib().spl_kv_import(self.handle, slot, token_count, _ptr(blob), blob.size))

    def topk(self, k=20, vocab_limit=None):
        """TopK.select (Sampler.swift:19-52) over every logit row of the last step: (ids, values), each [rows][k]."""
        n = max(self.last_logit_rows, 1)
        ids = np.zeros((n, k), np.int32); values = np.zeros((n, k), np.float32)
        self._check(lib().spl_topk(self.handle, vocab_limit or self.g.vocab, k, _ptr(ids), _ptr(values)))
        return ids[:self.last_logit_rows], values[:self.last_logit_rows]

    def enable_features(self, layers=None, enabled=True):
        """Engine.step(captureFeatures:) (Engine.swift:1316): keep the residual stream after the listed blocks
        (default Engine.featureLayers, Engine.swift:331) for `feature_row`."""
        if not enabled:
            self._check(lib().spl_features_enable(self.handle, None, 0))
        elif layers is None:
            self._check(lib().spl_features_enable(self.handle, None, 5))
        else:
            arr = np.ascontiguousarray(layers, np.int32)
            self._check(lib().spl_features_enable(self.handle, _ptr(arr), len(arr)))

    def feature_row(self, row):
        """Engine.featureRow (Engine.swift:1309-1313): taps x hidden floats of one row of the last step."""
        out = np.empty(lib().spl_feature_width(self.handle), np.float32)
        self._check(lib().spl_feature_row(self.handle, row, _ptr(out)))
        return out

    def debug_taps(self, enabled=True):
        self._check(lib().spl_debug_taps(self.handle, int(enabled)))

    def debug_wait_budget(self, nanoseconds):
        self._check(lib().spl_debug_wait_budget(self.handle, int(nanoseconds)))

    def debug_drop_weight_stage(self, stage):
        self._check(lib().spl_debug_drop_weight_stage(self.handle, int(stage)))

    def static_status(self):
        """spl_gemm_q4_static_status: raises EngineError('timeout') when a block of the last static GEMMs gave up a wait."""
        self._check(lib().spl_gemm_q4_static_status(self.handle))

    def debug_kv_store(self, enabled=True):
        self._check(lib().spl_debug_kv_store(self.handle, int(enabled)))

    def debug_gdn_chunk_min(self, rows):
        """Ordinary runs of at least `rows` rows (default 512) take the chunked gated-delta scan."""
        self._check(lib().spl_debug_gdn_chunk_min(self.handle, int(rows)))

    def debug_pair_blocks(self, enabled=True):
        """Prompt chunks' GEMMs on the pair form of the 128-row block (default) or on the one-tile block."""
        self._check(lib().spl_debug_pair_blocks(self.handle, int(enabled)))

    def debug_profile(self, enabled=True):
        self._check(lib().spl_debug_profile(self.handle, int(enabled)))

    def profile_read(self):
        out = {}
        for klass, name in enumerate(["gemm_q4", "elementwise", "gdn", "attention", "other"]):
            ms, n, b = C.c_double(), C.c_int64(), C.c_double()
            self._check(lib().spl_debug_profile_read(self.handle, klass, C.byref(ms), C.byref(n), C.byref(b)))
            out[name] = dict(ms=ms.value, launches=n.value, bytes=b.value)
        return out

    def debug_read(self, which, index, count, dtype=np.float32):
        names = ["state", "conv", "journal", "k_codes", "v_codes", "k_scale", "v_scale", "hidden", "tap", "proj", "core", "q", "attn_partials", "flags"]
        out = np.empty(count, dtype)
        self._check(lib().spl_debug_read(self.handle, names.index(which), index, _ptr(out), out.nbytes))
        return out


RESIDENT = ["in_proj", "out_proj", "gate_up", "down", "head"]


def debug_pair_blocks(enabled=True):
    """Steps of more than 64 rows on the pair form of the 128-row GEMM block (default) or on the one-tile block (process-wide)."""
    lib().spl_debug_pair_blocks(None, int(enabled))


def splw_check(path):
    """The container checks of an SPLW artifact, no engine needed (spl_splw_check): (format, tensor records)."""
    message = C.create_string_buffer(512)
    count = C.c_int32(0)
    status = lib().spl_splw_check(os.fsencode(path), C.byref(count), message, len(message))
    if status:
        raise EngineError(status, message.value.decode() or "spl_splw_check failed")
    return message.value.decode(), count.value


def gguf_planes_unpack(kind, plane0, plane1, meta, rows, inner):
    """The three planes of a GGUF weight back into native blocks (spl_gguf_planes_unpack): uint8 [rows][inner / 256][block bytes]."""
    import numpy as np
    type_id, block = {"Q4_K": (12, 144), "Q5_K": (13, 176), "Q6_K": (14, 210)}[kind]
    native = np.zeros((rows, inner // 256, block), np.uint8)
    p0, pm = np.ascontiguousarray(plane0, np.uint8), np.ascontiguousarray(meta, np.uint8)
    p1 = None if plane1 is None else np.ascontiguousarray(plane1, np.uint8)
    status = lib().spl_gguf_planes_unpack(type_id, _ptr(p0), None if p1 is None else _ptr(p1), _ptr(pm), rows, inner, _ptr(native))
    if status:
        raise EngineError(status, "spl_gguf_planes_unpack refused its arguments")
    return native


def gemm_q4_static(engine, layer, which, device_activations, rows, device_residual, device_out, stream=None):
    """The allocation-free GEMM on one of the engine's resident weights. The three buffer arguments are raw device
    addresses (ints); nothing is allocated, copied or waited for."""
    status = lib().spl_gemm_q4_static(engine.handle, layer, RESIDENT.index(which), C.c_void_p(device_activations), rows,
                                      C.c_void_p(device_residual) if device_residual else None, C.c_void_p(device_out),
                                      C.c_void_p(stream) if stream else None)
    if status:
        raise EngineError(status, lib().spl_last_error_string(engine.handle).decode())


GGUF_TYPE = {"Q4_K": 12, "Q5_K": 13, "Q6_K": 14}


def gemm_gguf(kind, blocks, activations, residual=None, device=0):
    """One GGUF K-quant GEMM on host arrays through the C ABI. blocks: uint8 [n, k / 256, block bytes] native super-blocks."""
    blocks = np.ascontiguousarray(blocks, np.uint8)
    a = np.ascontiguousarray(activations, np.float32)
    n, k = blocks.shape[0], blocks.shape[1] * 256
    out = np.zeros((a.shape[0], n), np.float32)
    res = None if residual is None else np.ascontiguousarray(residual, np.float32)
    status = lib().spl_op_gemm_gguf(device, GGUF_TYPE[kind], _ptr(blocks), n, k, _ptr(a), a.shape[0], None if res is None else _ptr(res), _ptr(out))
    if status != 0:
        raise EngineError(status, "spl_op_gemm_gguf")
    return out


def gemm_q4(packed, scales, biases, activations, residual=None, device=0):
    """One MLX affine-4 GEMM on host arrays through the C ABI (copies in, runs on the GPU, copies out)."""
    packed = np.ascontiguousarray(packed, np.uint32); scales = np.ascontiguousarray(scales, np.uint16); biases = np.ascontiguousarray(biases, np.uint16)
    a = np.ascontiguousarray(activations, np.float32)
    n, k = packed.shape[0], packed.shape[1] * 8
    out = np.empty((a.shape[0], n), np.float32)
    res = None if residual is None else np.ascontiguousarray(residual, np.float32)
    status = lib().spl_op_gemm_q4(device, _ptr(packed), _ptr(scales), _ptr(biases), n, k, _ptr(a), a.shape[0],
                                  None if res is None else _ptr(res), _ptr(out))
    if status:
        raise EngineError(status, "spl_op_gemm_q4 failed")
    return out
