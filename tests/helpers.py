"""Shared scaffolding of the parity tests: one synthetic model loaded into the CPU oracle and
into the CUDA engine, and a driver that feeds both the same rows."""
import numpy as np

import splosh_b200 as S
from oracle import oracle as O
from oracle import tables as T

OBSERVED = []


def observed(text):
    """Record a measured difference; conftest prints every line at the end of the run."""
    OBSERVED.append(text)
    print(text)


TABLE_FIELDS = ["tokens", "row_slot", "row_pos", "runs", "run_info", "row_read", "row_write", "gather_index", "attn_blocks"]
SCALARS = ["rows", "step_pages", "live_rows", "spans", "pages_per_span"]


def to_oracle_geometry(g):
    return O.Geometry.from_buffer_copy(bytes(g))


def assert_tables_equal(mine, ref):
    for name in SCALARS:
        assert int(mine[name]) == int(getattr(ref, name)), name
    for name in TABLE_FIELDS:
        assert np.array_equal(mine[name], getattr(ref, name)), name
    assert np.array_equal(mine["page_table"], ref.page_table), "page_table"


class Pair:
    """The CUDA engine and the CPU oracle side by side on the same seeded model."""

    def __init__(self, geometry, config, seed=0x5EED6D17, gpu=True, gguf=None):
        """gguf: None for the MLX affine-4 model, or (block kind, head kind), e.g. ("Q5_K", "Q6_K"), for the same model
        re-quantised to GGUF K-quants on both sides."""
        self.g, self.config = geometry, config
        og = to_oracle_geometry(geometry)
        self.model = O.Model(og, seed)
        if gguf:
            self.model.to_gguf(*gguf)
        self.ohost = T.Host(max_slots=config.max_slots, max_rows=config.max_rows, kv_pages=config.kv_pages,
                            max_context=config.max_context, state_units=config.state_units or None,
                            max_logit_rows=config.max_logit_rows or None, vocab=geometry.vocab, kv_heads=geometry.kv_heads,
                            span_target=config.span_target or 592, last_layer_full=geometry.layers % 4 == 0)
        self.oengine = O.Engine(self.model, config.max_slots, config.kv_pages, self.ohost.max_pages, self.ohost.state_units)
        self.engine = None
        if gpu:
            self.engine = S.Engine(geometry, config)
            if gguf:
                self.engine.load_gguf_model(self.model)
            else:
                self.engine.load_model(self.model)

    def step(self, rows, taps=False):
        """Run one step on both. Returns (gpu logits, oracle logits[, gpu taps, oracle taps])."""
        ot = self.ohost.build([T.Row(r.slot, r.token, r.position, r.want_logits, r.verify) for r in rows])
        if taps:
            ologits, otaps = self.oengine.step(ot, taps=True)
        else:
            ologits = self.oengine.step(ot)
        self.ohost.finish_step(ot)
        self.last_tables = ot
        if self.engine is None:
            return None, ologits
        if taps:
            self.engine.debug_taps(True)
        self.engine.step(rows)
        glogits = self.engine.all_logits()
        if taps:
            n = len(rows) * self.g.hidden
            gtaps = np.stack([self.engine.debug_read("tap", l, n).reshape(len(rows), self.g.hidden) for l in range(self.g.layers)])
            return glogits, ologits, gtaps, otaps
        return glogits, ologits

    def accept(self, slot, rows, token_count):
        self.ohost.accept_verify(slot, rows, token_count)
        if self.engine is not None:
            self.engine.accept_verify(slot, rows, token_count)

    def reset(self, slot):
        unit = self.ohost.reset_slot(slot)
        self.oengine.reset_slot(slot, unit)
        if self.engine is not None:
            self.engine.reset_slot(slot)


def top1_report(glogits, ologits, limit):
    """Arg-max agreement and, for every row, the oracle's top-1 margin."""
    ga = np.argmax(glogits[:, :limit], axis=1)
    oa = O.argmax(ologits, limit)
    srt = np.sort(ologits[:, :limit], axis=1)
    margin = srt[:, -1] - srt[:, -2]
    return ga, oa, margin


def tokens_for(seed, count, vocab):
    lib = O.lib()
    return [int(lib.orc_splitmix_at(seed, i) % vocab) for i in range(count)]
