"""The width planner of the C ABI (spl_plan_prefill_cap, spl_plan_blocks, spl_plan_cycle_ms, spl_plan_tier) with the
reference's cost table against the CPU restatement of BatchScheduler.swift:646-669, 735-789 in oracle/planner.py, on
seeded random scheduler states; then the behaviour the reference's comments state. No GPU is involved."""
import numpy as np

import splosh_b200 as S
from oracle import planner as OP


def test_tiers_and_cycle_cost():
    ref = S.Planner("reference")
    for rows in list(range(1, 140)) + [160, 200]:
        assert S.Planner.tier(rows) == OP.tier(rows)
        assert ref.cycle_ms(rows) == OP.cycle_ms(rows)
    assert [S.Planner.tier(r) for r in (1, 16, 17, 32, 33, 64, 65, 96, 97, 128)] == [16, 16, 32, 32, 64, 64, 96, 96, 128, 128]


def test_prefill_cap_equals_the_restatement_on_random_states():
    rng = np.random.default_rng(3)
    ref = S.Planner("reference")
    for _ in range(3000):
        max_rows = int(rng.choice([64, 128]))
        decode_rows = int(rng.integers(0, max_rows))
        decode_tokens = float(rng.uniform(0, decode_rows + 1))
        attention = float(rng.uniform(0, 60))
        backlog = int(rng.choice([0, 3, 40, 500, 100000]))
        fed = int(rng.choice([0, 1000, 50000, 200000]))
        weight = float(rng.choice([1.0, 3.0]))
        assert ref.prefill_cap(max_rows, decode_rows, decode_tokens, attention, backlog, fed, weight) == \
            OP.prefill_cap(max_rows, decode_rows, decode_tokens, attention, backlog, fed, weight)


def test_plan_blocks_equals_the_restatement_on_random_states():
    rng = np.random.default_rng(5)
    ref = S.Planner("reference")
    for _ in range(3000):
        n = int(rng.integers(1, 9))
        tail = rng.uniform(0, 4, n); block_yield = rng.uniform(1, 8, n)
        context = rng.choice([500, 8000, 50000, 150000, 262140], n).astype(np.int32)
        other = int(rng.integers(0, 20))
        assert ref.blocks(tail, block_yield, context, other) == OP.plan_blocks(list(tail), list(block_yield), [int(c) for c in context], other)


def test_what_the_reference_says_about_its_plans():
    ref = S.Planner("reference")
    # "At 1 a waiting prompt always gets a full-width step, with the decoding sessions' rows riding in it."
    for decoders in (1, 2, 4, 8):
        assert ref.prefill_cap(128, decoders, float(decoders), 0.3 * decoders, 100000, 0, decode_weight=1.0) == 128
    # No backlog: the step is as wide as its decode rows.
    assert ref.prefill_cap(128, 5, 5.0, 1.0, 0, 0) == 5
    # One session at short context, blocks usually accepted whole: rows 9-16 are inside the tier it already pays for.
    assert ref.blocks([0.5 * 5], [6.0], [2000]) == [16]
    # At long context a second half is only drafted where blocks are usually accepted whole.
    assert ref.blocks([0.15 * 3], [3.5], [150000]) == [8]
    # Nothing is doubled past the verify-row budget.
    assert sum(ref.blocks([3.0] * 8, [6.0] * 8, [1000] * 8, max_verify_rows=64)) == 64


def test_the_b200_table_is_selectable_and_ordered():
    mine = S.Planner("b200")
    costs = [mine.cycle_ms(r) for r in (16, 32, 64, 96, 128)]
    assert all(a <= b for a, b in zip(costs, costs[1:])) and costs[-1] < S.Planner("reference").cycle_ms(16)
