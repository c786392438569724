"""CPU restatement of the reference's host-side step bookkeeping. TEST INFRASTRUCTURE ONLY.

Restates, in plain Python, what `Engine` keeps on the host between and before steps:
  * the paged-KV block allocator and the state-unit pool
    (Sources/SploshRuntime/Engine.swift:625-632, 810-868),
  * the per-step index tables and their validation (Engine.swift:1316-1398),
  * the span split of the attention scan (Engine.swift:2232-2239, with the span target as a
    parameter instead of the reference's Apple-GPU constants),
  * the row packer's ordering and the greedy accept rule
    (Sources/SploshRuntime/BatchScheduler.swift:1392-1440, 1579-1597).

The shipped library has its own C++ statement of the same logic; the tests compare the two
table for table, bit for bit.
"""
from dataclasses import dataclass, field
import numpy as np

PAGE_TOKENS = 256        # Engine.swift:124
JOURNAL_ROWS = 16        # Engine.swift:300
ATTN_BLOCK_ROWS = 8      # Engine.swift:523 (48 fused queries / 6 heads per KV head)


class InvalidRows(Exception):
    pass


class KVPoolExhausted(Exception):
    pass


class ContextExceeded(Exception):
    pass


@dataclass
class Row:                       # EngineRow, Engine.swift:50-62
    slot: int
    token: int
    position: int
    want_logits: bool
    verify: bool = False


@dataclass
class Tables:
    rows: int
    tokens: np.ndarray
    row_slot: np.ndarray
    row_pos: np.ndarray
    runs: np.ndarray             # (slot, start, length) per run
    run_info: np.ndarray         # (speculative, journal pending) per run
    row_read: np.ndarray
    row_write: np.ndarray
    gather_index: np.ndarray
    attn_blocks: np.ndarray      # (first row, count) per block
    page_table: np.ndarray       # [max_slots, max_pages]
    step_pages: int
    live_rows: int
    spans: int
    pages_per_span: int

    @property
    def run_count(self):
        return len(self.runs) // 3

    @property
    def logit_rows(self):
        return len(self.gather_index)

    @property
    def attn_block_count(self):
        return len(self.attn_blocks) // 2


class Host:
    """Allocator state plus the table builder, in the order of operations of Engine.step."""

    def __init__(self, max_slots=8, max_rows=64, kv_pages=256, max_context=32768, state_units=None,
                 max_logit_rows=None, vocab=1 << 30, kv_heads=4, span_target=592, last_layer_full=True):
        self.max_slots, self.max_rows, self.kv_pages, self.max_context = max_slots, max_rows, kv_pages, max_context
        self.state_units = state_units if state_units is not None else max_slots * (JOURNAL_ROWS + 1)
        self.max_logit_rows = max_logit_rows if max_logit_rows is not None else max_rows
        if self.state_units < max_slots:
            raise InvalidRows("stateUnits must be at least maxSlots")
        self.vocab, self.kv_heads, self.span_target, self.last_layer_full = vocab, kv_heads, span_target, last_layer_full
        self.max_pages = (max_context + PAGE_TOKENS - 1) // PAGE_TOKENS
        self.free_pages = list(reversed(range(kv_pages)))                 # Engine.swift:625
        self.slot_pages = [[] for _ in range(max_slots)]
        self.slot_unit = list(range(max_slots))
        self.free_units = list(reversed(range(max_slots, self.state_units)))
        self.pending_verify = [[] for _ in range(max_slots)]
        self.journal_pending = [0] * max_slots
        self.page_table = np.zeros((max_slots, self.max_pages), np.uint32)

    # ---- slot lifecycle (Engine.swift:810-868)
    def reset_slot(self, slot):
        self.free_pages.extend(self.slot_pages[slot])
        self.slot_pages[slot] = []
        self.discard_verify(slot)
        self.journal_pending[slot] = 0
        return self.slot_unit[slot]          # the unit whose conv history the caller zeroes

    def discard_verify(self, slot):
        self.free_units.extend(self.pending_verify[slot])
        self.pending_verify[slot] = []

    def accept_verify(self, slot, rows, token_count):
        units = self.pending_verify[slot]
        assert 1 <= rows <= len(units), "acceptVerify outside the verified run"
        self.free_units.append(self.slot_unit[slot])
        self.slot_unit[slot] = units[rows - 1]
        for index, unit in enumerate(units):
            if index != rows - 1:
                self.free_units.append(unit)
        self.pending_verify[slot] = []
        self.journal_pending[slot] = rows
        self.truncate(slot, token_count)

    def truncate(self, slot, token_count):
        keep = (token_count + PAGE_TOKENS - 1) // PAGE_TOKENS
        while len(self.slot_pages[slot]) > keep:
            self.free_pages.append(self.slot_pages[slot].pop())

    def ensure_page(self, slot, position):
        if position >= self.max_context:
            raise ContextExceeded(f"position {position} exceeds the context limit {self.max_context}")
        index = position // PAGE_TOKENS
        while len(self.slot_pages[slot]) <= index:
            if not self.free_pages:
                raise KVPoolExhausted(f"need {index + 1 - len(self.slot_pages[slot])} page(s), 0 free")
            page = self.free_pages.pop()
            self.page_table[slot, len(self.slot_pages[slot])] = page
            self.slot_pages[slot].append(page)

    # ---- the step's tables (Engine.swift:1316-1398)
    def build(self, rows):
        count = len(rows)
        if not (0 < count <= self.max_rows):
            raise InvalidRows(f"{count} rows; limit {self.max_rows}")
        for row in rows:
            if row.verify and 0 <= row.slot < self.max_slots:
                self.discard_verify(row.slot)
        step_pages = max(r.position for r in rows) // PAGE_TOKENS + 1
        blocks = []
        index = 0
        while index < count:
            length = 1
            while length < ATTN_BLOCK_ROWS and index + length < count and rows[index + length].slot == rows[index].slot:
                length += 1
            blocks += [index, length]
            index += length
        tokens = np.zeros(count, np.uint32); row_slot = np.zeros(count, np.uint32); row_pos = np.zeros(count, np.uint32)
        row_read = np.zeros(count, np.uint32); row_write = np.zeros(count, np.uint32)
        runs, info, gather = [], [], []
        seen = set()
        for index, row in enumerate(rows):
            if not (0 <= row.slot < self.max_slots and 0 <= row.token < self.vocab):
                raise InvalidRows(f"row {index} out of range")
            self.ensure_page(row.slot, row.position)
            tokens[index], row_slot[index], row_pos[index] = row.token, row.slot, row.position
            previous = self.pending_verify[row.slot][-1] if self.pending_verify[row.slot] else self.slot_unit[row.slot]
            row_read[index] = previous
            if row.verify:
                if not self.free_units:
                    raise InvalidRows("state unit pool exhausted")
                unit = self.free_units.pop()
                self.pending_verify[row.slot].append(unit)
                row_write[index] = unit
            else:
                if self.pending_verify[row.slot]:
                    raise InvalidRows(f"ordinary row after speculative rows in slot {row.slot}")
                row_write[index] = previous
            if index > 0 and rows[index - 1].slot == row.slot:
                if row.position != rows[index - 1].position + 1:
                    raise InvalidRows(f"slot {row.slot} positions are not consecutive")
                if row.verify != rows[index - 1].verify:
                    raise InvalidRows(f"slot {row.slot} mixes speculative and ordinary rows")
                runs[-1] += 1
                if row.verify and runs[-1] > JOURNAL_ROWS:
                    raise InvalidRows(f"more than {JOURNAL_ROWS} speculative rows in slot {row.slot}")
            else:
                if row.slot in seen:
                    raise InvalidRows(f"slot {row.slot} rows are not contiguous")
                seen.add(row.slot)
                runs += [row.slot, index, 1]
                info += [1 if row.verify else 0, self.journal_pending[row.slot]]
            if row.want_logits:
                if len(gather) >= self.max_logit_rows:
                    raise InvalidRows("too many logit rows")
                gather.append(index)
        # Rows the last block is computed for (Engine.swift:1419-1429).
        live = count
        if self.last_layer_full and count >= 8:
            wanted = max((i for i, r in enumerate(rows) if r.want_logits), default=-1) + 1
            live = 0 if wanted == 0 else min(count, max(wanted, 8))
        # Span split (Engine.swift:2236-2239): at most span_limit spans of whole pages.
        block_count = len(blocks) // 2
        span_limit = max(16, min(64, -(-self.span_target // (self.kv_heads * block_count))))
        pages_per_span = (step_pages + span_limit - 1) // span_limit
        spans = (step_pages + pages_per_span - 1) // pages_per_span
        return Tables(rows=count, tokens=tokens, row_slot=row_slot, row_pos=row_pos,
                      runs=np.array(runs, np.uint32), run_info=np.array(info, np.uint32),
                      row_read=row_read, row_write=row_write, gather_index=np.array(gather, np.uint32),
                      attn_blocks=np.array(blocks, np.uint32), page_table=self.page_table.copy(),
                      step_pages=step_pages, live_rows=live, spans=spans, pages_per_span=pages_per_span)

    def finish_step(self, tables):
        """Every slot in the step had its accepted journal entries replayed (Engine.swift:1537)."""
        for run in range(tables.run_count):
            self.journal_pending[int(tables.runs[run * 3])] = 0


# ---- the packer's row order and the greedy accept rule

@dataclass
class Session:
    """What the row packer reads of a session (BatchScheduler.swift:1323-1442)."""
    slot: int
    evaluated: int                       # tokens already in the slot (slotTokens[slot].count)
    pending: int = None                  # the token waiting to be evaluated; None while prefilling
    drafts: list = field(default_factory=list)    # proposed continuation (empty: plain decode)
    prompt: list = field(default_factory=list)    # tokens still to prefill start at `fed`
    fed: int = 0


def pack_rows(sessions, max_rows, max_logit_rows=None, prefill_cap=None):
    """Verify blocks (anchor + drafts, all wanting logits), then plain decoders, then prefill
    chunks shortest backlog first, a chunk asking for logits only on the prompt's last token
    (BatchScheduler.swift:1392-1440). Returns (rows, plan); plan entries are
    ("verify", session, n_drafts) | ("decode", session) | ("prefill", session, count, complete)."""
    max_logit_rows = max_rows if max_logit_rows is None else max_logit_rows
    rows, plan, logit_rows = [], [], 0
    decoders = [s for s in sessions if s.pending is not None]
    for s in [d for d in decoders if d.drafts]:
        for offset, token in enumerate([s.pending] + list(s.drafts)):
            rows.append(Row(s.slot, token, s.evaluated + offset, True, True))
        logit_rows += len(s.drafts) + 1
        plan.append(("verify", s, len(s.drafts)))
    for s in [d for d in decoders if not d.drafts]:
        rows.append(Row(s.slot, s.pending, s.evaluated, True))
        logit_rows += 1
        plan.append(("decode", s))
    prefillers = sorted((s for s in sessions if s.pending is None), key=lambda s: len(s.prompt) - s.fed)
    cap = max_rows if (not decoders or prefill_cap is None) else prefill_cap
    for s in prefillers:
        budget = cap - len(rows)
        if budget <= 0:
            break
        count = min(len(s.prompt) - s.fed, budget)
        complete = s.fed + count == len(s.prompt)
        if complete and logit_rows >= max_logit_rows:
            continue
        for offset in range(count):
            position = s.fed + offset
            rows.append(Row(s.slot, s.prompt[position], position, complete and offset == count - 1))
        if complete:
            logit_rows += 1
        plan.append(("prefill", s, count, complete))
    return rows, plan


def build_rows(host, sessions, planner_cap, block=8, max_verify_rows=64, speculate=True, attention_first=0.29, yields=None, marks=None):
    """BatchScheduler.buildRows in full (BatchScheduler.swift:1323-1442) over a Host's allocator state: the `fits` rule for
    speculating sessions (:1351-1353), KV-page reservation without eviction (:1336-1343), the prefill cap from
    `planner_cap(decode_rows, decode_tokens, decode_attention, backlog, first_fed)` (:1408-1409), chunks that end at a
    state mark (:1420-1422) or at the pages the slot already holds (:1423-1428).
    sessions: Session objects in the scheduler's order; yields[i]: a speculating session's expected block yield;
    marks[i]: positions where session i's prefill must stop. Returns (rows, plan, waiting) with plan entries
    (kind, session index, count, complete) and kind 0 verify, 1 decode, 2 prefill."""
    yields = yields or [0.0] * len(sessions); marks = marks or [[] for _ in sessions]
    rows, plan, waiting = [], [], []
    logit_rows, reserved = 0, 0
    decode_tokens, decode_attention = 0.0, 0.0

    def reserve(index, position):
        nonlocal reserved
        need = position // PAGE_TOKENS + 1 - len(host.slot_pages[sessions[index].slot])
        if need <= 0:
            return True
        if need > len(host.free_pages) - reserved:
            waiting.append(index)
            return False
        reserved += need
        return True

    decoders = [i for i, s in enumerate(sessions) if s.pending is not None][:host.max_slots]
    speculative, plain = [], []
    for i in decoders:
        s = sessions[i]
        ahead = len(speculative) + 1
        fits = (ahead * block <= max_verify_rows and len(rows) + ahead * block + len(plain) <= host.max_rows
                and logit_rows + ahead * block + len(plain) <= host.max_logit_rows)
        if speculate and s.evaluated + block < host.max_context:
            if fits and reserve(i, s.evaluated + 2 * block - 1):
                speculative.append(i)
        elif reserve(i, s.evaluated):
            plain.append(i)
    for i in speculative:
        decode_tokens += yields[i]
        decode_attention += attention_first * sessions[i].evaluated / 1000
    for i in speculative:
        s = sessions[i]
        for offset, token in enumerate([s.pending] + list(s.drafts)):
            rows.append(Row(s.slot, token, s.evaluated + offset, True, True))
        logit_rows += len(s.drafts) + 1
        plan.append((0, i, len(s.drafts), 0))
    for i in plain:
        s = sessions[i]
        rows.append(Row(s.slot, s.pending, s.evaluated, True))
        logit_rows += 1
        plan.append((1, i, 0, 0))
    prefillers = sorted((i for i, s in enumerate(sessions) if s.pending is None), key=lambda i: len(sessions[i].prompt) - sessions[i].fed)
    cap = host.max_rows
    if decoders:
        backlog = sum(len(sessions[i].prompt) - sessions[i].fed for i in prefillers)
        cap = planner_cap(len(rows), decode_tokens + len(plain), decode_attention, backlog, sessions[prefillers[0]].fed if prefillers else 0)
    for i in prefillers:
        s = sessions[i]
        budget = cap - len(rows)
        if budget <= 0:
            break
        count = min(len(s.prompt) - s.fed, budget)
        later = [m for m in marks[i] if m > s.fed]
        if later and min(later) < s.fed + count:
            count = min(later) - s.fed
        if not reserve(i, s.fed + count - 1):
            count = min(count, len(host.slot_pages[s.slot]) * PAGE_TOKENS - s.fed)
            if count <= 0:
                continue
            waiting.remove(i)
        complete = s.fed + count == len(s.prompt)
        if complete and logit_rows >= host.max_logit_rows:
            continue
        for offset in range(count):
            rows.append(Row(s.slot, s.prompt[s.fed + offset], s.fed + offset, complete and offset == count - 1))
        if complete:
            logit_rows += 1
        plan.append((2, i, count, 1 if complete else 0))
    return rows, plan, waiting


def greedy_accept(argmax_ids, drafts):
    """(agreed, bonus): the agreeing prefix of the drafts, then the target's own arg-max
    (BatchScheduler.swift:1583-1587). argmax_ids: the arg-max of the block's logit rows."""
    agreed = 0
    while agreed < len(drafts) and argmax_ids[agreed] == drafts[agreed]:
        agreed += 1
    return agreed, int(argmax_ids[agreed])
