"""The row packer of the library (spl_host_pack_rows) against the restated BatchScheduler.buildRows
(Sources/SploshRuntime/BatchScheduler.swift:1323-1442; oracle/tables.py:build_rows), bit for bit on seeded session sets:
row order (verify blocks, decoders, prompt chunks shortest backlog first), the width prefillCap allows, KV-page
reservation against a pool that is sometimes too small, chunk ends on state marks, the logit-row limit.
No GPU: the packer is host arithmetic. The reference stores no packed step, so this is parity against the restatement."""
import numpy as np

import splosh_b200 as S
from oracle import planner as OP
from oracle import tables as T


def make(seed):
    rng = np.random.default_rng(seed)
    max_slots = int(rng.integers(2, 9))
    max_rows = int(rng.choice([32, 64, 96, 128]))
    kv_pages = int(rng.integers(4, 400))
    cfg = S.EngineConfig(max_slots=max_slots, max_rows=max_rows, kv_pages=kv_pages, max_context=int(rng.choice([4096, 65536])),
                         max_logit_rows=int(rng.choice([0, 24, 64])))
    g = S.tiny_geometry()
    mine = S.Host(g, cfg)
    ref = T.Host(max_slots=max_slots, max_rows=max_rows, kv_pages=kv_pages, max_context=cfg.max_context, max_logit_rows=cfg.max_logit_rows or None,
                 vocab=g.vocab, kv_heads=g.kv_heads)
    # Some slots already hold pages: a throwaway row at the end of their context on both hosts.
    held = {}
    for slot in range(max_slots):
        if rng.random() < 0.6:
            position = int(rng.integers(0, min(cfg.max_context - 64, 30000)))
            try:
                ref.build([T.Row(slot, 1, position, False)])
            except T.KVPoolExhausted:
                # Both allocators hand out pages until the pool is dry and then fail: the slot keeps what it got on both sides.
                try:
                    mine.build([S.EngineRow(slot, 1, position, False)])
                except S.EngineError:
                    pass
                continue
            mine.build([S.EngineRow(slot, 1, position, False)])
            held[slot] = position + 1
    sessions, yields, marks = [], [], []
    for slot in rng.permutation(max_slots)[:int(rng.integers(1, max_slots + 1))]:
        slot = int(slot)
        evaluated = held.get(slot, 0)
        kind = rng.integers(0, 3)
        if kind < 2 and evaluated > 0:
            drafts = tuple(int(x) for x in rng.integers(0, g.vocab, int(rng.choice([7, 15])))) if kind == 0 else ()
            sessions.append(S.PackSession(slot, evaluated, pending=int(rng.integers(0, g.vocab)), proposal=drafts, block_yield=float(rng.uniform(1, 6))))
            marks.append(())
        else:
            total = int(rng.integers(1, 3000))
            fed = int(rng.integers(0, total)) if evaluated == 0 else min(evaluated, total - 1)
            fed = min(fed, evaluated) if evaluated else 0
            m = tuple(sorted(int(x) for x in rng.integers(1, total + 1, int(rng.integers(0, 3)))))
            sessions.append(S.PackSession(slot, fed, prompt=tuple(int(x) for x in rng.integers(0, g.vocab, total)), fed=fed, marks=m))
            marks.append(m)
        yields.append(sessions[-1].block_yield)
    speculate = bool(rng.random() < 0.8)
    return cfg, mine, ref, sessions, yields, marks, speculate


def test_packed_rows_equal_the_restatement_on_seeded_session_sets():
    planner = S.Planner("reference")
    checked = 0
    for seed in range(400):
        cfg, mine, ref, sessions, yields, marks, speculate = make(seed)
        osessions = [T.Session(slot=s.slot, evaluated=s.evaluated, pending=s.pending, drafts=list(s.proposal), prompt=list(s.prompt), fed=s.fed) for s in sessions]
        cap = lambda rows, tokens, attention, backlog, first_fed: OP.prefill_cap(cfg.max_rows, rows, tokens, attention, backlog, first_fed)
        try:
            want_rows, want_plan, want_waiting = T.build_rows(ref, osessions, cap, speculate=speculate, yields=yields, marks=[list(m) for m in marks])
        except Exception:
            continue
        if len(want_rows) > cfg.max_rows:
            continue           # more rows than a step holds: the scheduler never offers such a set (its proposals are sized by planBlocks)
        rows, plan, waiting = mine.pack_rows(sessions, planner, speculate=speculate)
        assert [(r.slot, r.token, r.position, r.want_logits, r.verify) for r in rows] == \
               [(r.slot, r.token, r.position, bool(r.want_logits), bool(r.verify)) for r in want_rows], seed
        assert plan == want_plan and waiting == want_waiting, seed
        checked += 1
    assert checked > 300


def test_the_order_is_verify_blocks_then_decoders_then_the_shortest_backlog():
    g = S.tiny_geometry()
    cfg = S.EngineConfig(max_slots=4, max_rows=128, kv_pages=64, max_context=8192)
    host = S.Host(g, cfg)
    for slot, position in ((0, 999), (1, 499)):
        host.build([S.EngineRow(slot, 1, position, False)])
    sessions = [S.PackSession(2, 0, prompt=tuple(range(100, 400)), fed=0),
                S.PackSession(1, 500, pending=7),
                S.PackSession(3, 0, prompt=tuple(range(50)), fed=0, marks=(20,)),
                S.PackSession(0, 1000, pending=5, proposal=(11, 12, 13), block_yield=2.0)]
    rows, plan, waiting = host.pack_rows(sessions, S.Planner("reference"), speculate=True)
    # Session 1 could speculate (a draft source exists) and has no proposal: the packer still gives it a block of its anchor alone.
    kinds = [p[0] for p in plan]
    assert kinds[:2] == [0, 0] and plan[0][1] == 1 and plan[1][1] == 3
    assert [r.verify for r in rows[:5]] == [True] * 5
    prefill = [p for p in plan if p[0] == 2]
    assert prefill[0][1] == 2 and prefill[0][2] == 20 and prefill[0][3] == 0      # the 50-token prompt first, cut at its state mark
    assert waiting == []
