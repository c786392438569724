"""The library's host bookkeeping (C ABI, spl_host_*) against the CPU oracle's restatement of
Engine.step's table build and allocator (Engine.swift:625-632, 810-868, 1316-1398): every table
bit for bit, on seeded scenarios and on the edge cases the reference validates."""
import numpy as np
import pytest

import splosh_b200 as S
from oracle import tables as T
from helpers import assert_tables_equal


def make(config, geometry=None):
    g = geometry or S.tiny_geometry()
    mine = S.Host(g, config)
    ref = T.Host(max_slots=config.max_slots, max_rows=config.max_rows, kv_pages=config.kv_pages, max_context=config.max_context,
                 state_units=config.state_units or None, max_logit_rows=config.max_logit_rows or None, vocab=g.vocab,
                 kv_heads=g.kv_heads, span_target=config.span_target or 592, last_layer_full=g.layers % 4 == 0)
    return mine, ref


def both(mine, ref, rows):
    a = mine.build(rows)
    b = ref.build([T.Row(r.slot, r.token, r.position, r.want_logits, r.verify) for r in rows])
    assert_tables_equal(a, b)
    mine.finish_step(); ref.finish_step(b)
    return a, b


def test_fresh_engine_hands_out_ascending_pages_and_reuses_lifo():
    mine, ref = make(S.EngineConfig(max_slots=3, max_rows=1024, kv_pages=12, max_context=2048))
    a, _ = both(mine, ref, [S.EngineRow(0, 1, p, False) for p in range(600)])
    assert a["page_table"][0, :3].tolist() == [0, 1, 2]
    both(mine, ref, [S.EngineRow(1, 1, p, False) for p in range(300)])
    mine.truncate(0, 256); ref.truncate(0, 256)          # frees pages 2 then 1
    a, _ = both(mine, ref, [S.EngineRow(2, 1, p, False) for p in range(300)])
    assert a["page_table"][2, :2].tolist() == [1, 2]     # last freed first
    assert mine.free_page_count == len(ref.free_pages)
    assert [mine.pages_held(s) for s in range(3)] == [len(p) for p in ref.slot_pages]


def test_packed_step_of_three_sessions_matches_the_first_benchmark_configuration():
    """A 512-row prefill chunk riding two 4-row verify blocks at 1K and 2K context (520 rows), in
    the packer's order (BatchScheduler.swift:1392-1440): verify blocks first, then the chunk."""
    mine, ref = make(S.EngineConfig(max_slots=4, max_rows=520, kv_pages=32, max_context=4096))
    sessions = [T.Session(slot=1, evaluated=1024, pending=11, drafts=[12, 13, 14]),
                T.Session(slot=2, evaluated=2048, pending=21, drafts=[22, 23, 24]),
                T.Session(slot=0, evaluated=0, prompt=list(range(100, 612)), fed=0)]
    rows, plan = T.pack_rows(sessions, max_rows=520)
    assert [p[0] for p in plan] == ["verify", "verify", "prefill"] and len(rows) == 520
    a, b = both(mine, ref, [S.EngineRow(r.slot, r.token, r.position, r.want_logits, r.verify) for r in rows])
    assert a["rows"] == 520 and len(a["gather_index"]) == 9 and a["live_rows"] == 520
    assert a["runs"].reshape(-1, 3).tolist() == [[1, 0, 4], [2, 4, 4], [0, 8, 512]]
    assert a["run_info"].reshape(-1, 2)[:, 0].tolist() == [1, 1, 0]


def test_speculative_units_and_journal_pending_follow_accept_and_discard():
    mine, ref = make(S.EngineConfig(max_slots=2, max_rows=64, kv_pages=8, max_context=1024))
    both(mine, ref, [S.EngineRow(0, 3, p, False) for p in range(10)])
    a, _ = both(mine, ref, [S.EngineRow(0, 3, 10 + i, True, True) for i in range(5)])
    assert a["row_read"].tolist() == [0, 2, 3, 4, 5] and a["row_write"].tolist() == [2, 3, 4, 5, 6]   # fresh units ascend from max_slots
    mine.accept_verify(0, 3, 13); ref.accept_verify(0, 3, 13)
    assert mine.slot_unit(0) == ref.slot_unit[0] == 4 and mine.journal_pending(0) == 3
    a, _ = both(mine, ref, [S.EngineRow(0, 3, 13 + i, True, True) for i in range(2)])
    assert a["run_info"].tolist() == [1, 3]
    assert mine.journal_pending(0) == 0                  # the step replayed the journal
    # An unaccepted run is dropped by the next speculative step of the slot (Engine.swift:1331).
    a, _ = both(mine, ref, [S.EngineRow(0, 3, 13 + i, True, True) for i in range(2)])
    mine.discard_verify(0); ref.discard_verify(0)
    both(mine, ref, [S.EngineRow(0, 3, 13, True)])


@pytest.mark.parametrize("seed", range(6))
def test_seeded_random_schedules(seed):
    rng = np.random.default_rng(seed)
    cfg = S.EngineConfig(max_slots=5, max_rows=96, kv_pages=40, max_context=2048, max_logit_rows=40)
    mine, ref = make(cfg)
    length = [0] * 5
    for step in range(30):
        rows, used = [], 0
        order = rng.permutation(5)
        for slot in order[:rng.integers(1, 6)]:
            kind = rng.integers(0, 3)
            if kind == 0 and length[slot] > 0:       # verify block
                n = int(rng.integers(1, 17))
                rows += [S.EngineRow(int(slot), int(rng.integers(0, 32000)), length[slot] + i, True, True) for i in range(n)]
            elif kind == 1 and length[slot] > 0:     # plain decode
                rows.append(S.EngineRow(int(slot), int(rng.integers(0, 32000)), length[slot], True))
            else:                                      # prefill chunk
                n = int(rng.integers(1, 40))
                rows += [S.EngineRow(int(slot), int(rng.integers(0, 32000)), length[slot] + i, i == n - 1) for i in range(n)]
        if len(rows) > cfg.max_rows or sum(r.want_logits for r in rows) > cfg.max_logit_rows:
            continue
        if any(r.position >= cfg.max_context - 64 for r in rows):
            for s in range(5):
                mine.reset_slot(s); ref.reset_slot(s); length[s] = 0
            continue
        a, b = both(mine, ref, rows)
        for run in a["runs"].reshape(-1, 3):
            slot, start, n = map(int, run)
            if rows[start].verify:
                keep = int(rng.integers(0, n + 1))
                if keep == 0:
                    mine.discard_verify(slot); ref.discard_verify(slot)
                else:
                    length[slot] += keep
                    mine.accept_verify(slot, keep, length[slot]); ref.accept_verify(slot, keep, length[slot])
            else:
                length[slot] += n
        assert mine.free_page_count == len(ref.free_pages)
        assert [mine.slot_unit(s) for s in range(5)] == ref.slot_unit


@pytest.mark.parametrize("rows,case", [
    ([], "invalidRows"),
    ([S.EngineRow(0, 1, p, False) for p in range(65)], "invalidRows"),                    # more rows than max_rows
    ([S.EngineRow(9, 1, 0, False)], "invalidRows"),                                       # slot out of range
    ([S.EngineRow(0, 32000, 0, False)], "invalidRows"),                                   # token out of range
    ([S.EngineRow(0, 1, 0, False), S.EngineRow(0, 1, 2, False)], "invalidRows"),          # positions not consecutive
    ([S.EngineRow(0, 1, 0, False), S.EngineRow(0, 1, 1, True, True)], "invalidRows"),     # mixes speculative and ordinary
    ([S.EngineRow(0, 1, 0, False), S.EngineRow(1, 1, 0, False), S.EngineRow(0, 1, 1, False)], "invalidRows"),   # not contiguous
    ([S.EngineRow(0, 1, i, True, True) for i in range(17)], "invalidRows"),               # more than 16 speculative rows
    ([S.EngineRow(0, 1, 600, False)], "contextExceeded"),
    ([S.EngineRow(0, 1, 500, False), S.EngineRow(1, 1, 500, False), S.EngineRow(2, 1, 500, False)], "kvPoolExhausted"),
])
def test_rejected_steps_name_the_reference_error_case(rows, case):
    """The checks of Engine.swift:1318-1385 and ensurePage (:848-861) with EngineError's cases."""
    cfg = S.EngineConfig(max_slots=3, max_rows=64, kv_pages=5, max_context=512)
    mine, ref = make(cfg)
    with pytest.raises(S.EngineError) as caught:
        mine.build(rows)
    assert caught.value.case == case
    expected = {"invalidRows": T.InvalidRows, "contextExceeded": T.ContextExceeded, "kvPoolExhausted": T.KVPoolExhausted}[case]
    with pytest.raises(expected):
        ref.build([T.Row(r.slot, r.token, r.position, r.want_logits, r.verify) for r in rows])


def test_last_block_is_trimmed_to_the_leading_rows_that_want_logits():
    """Engine.swift:1419-1429: with 8 or more rows the last block is computed only for the rows up to
    the last one wanting logits (at least 8)."""
    mine, ref = make(S.EngineConfig(max_slots=2, max_rows=64, kv_pages=8, max_context=1024))
    a, _ = both(mine, ref, [S.EngineRow(0, 1, 0, True)] + [S.EngineRow(1, 1, p, False) for p in range(40)])
    assert a["live_rows"] == 8
    a, _ = both(mine, ref, [S.EngineRow(1, 1, 40 + p, False) for p in range(20)])
    assert a["live_rows"] == 0
    a, _ = both(mine, ref, [S.EngineRow(1, 1, 60 + p, p == 4) for p in range(5)])
    assert a["live_rows"] == 5


def test_span_count_grows_for_narrow_steps():
    mine, ref = make(S.EngineConfig(max_slots=2, max_rows=64, kv_pages=200, max_context=45056), S.b27_geometry())
    a, _ = both(mine, ref, [S.EngineRow(0, 1, 40000, True)])
    assert a["step_pages"] == 157 and a["spans"] == 53 and a["pages_per_span"] == 3   # one block: up to 64 spans
    a, _ = both(mine, ref, [S.EngineRow(0, 1, 40001 + i, True) for i in range(8)] + [S.EngineRow(1, 1, i, False) for i in range(50)])
    assert a["spans"] == 18 and a["pages_per_span"] == 9      # eight blocks: limit ceil(592 / 32) = 19


def test_greedy_accept_rule():
    """BatchScheduler.swift:1583-1587: the agreeing prefix, then the target's own arg-max."""
    for ids, drafts in (([5, 6, 7, 8], [5, 6, 9]), ([5, 6, 7, 8], [5, 6, 7]), ([1, 2], [3]), ([4], [])):
        assert S.greedy_accept(ids, drafts) == T.greedy_accept(ids, drafts)
    assert S.greedy_accept([5, 6, 7, 8], [5, 6, 9]) == (2, 7)
