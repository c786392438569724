"""TEST INFRASTRUCTURE ONLY — a CPU restatement of the reference's width planner, the checker of the library's
`spl_plan_*` entry points. Nothing shipped imports it.

Follows Sources/SploshRuntime/BatchScheduler.swift: tier and cycleMilliseconds (:740-745), attentionMilliseconds (:750),
prefillCap (:655-669), planBlocks (:763-789), with the reference's constants. Double precision, as the reference.

Parity unpinned: the reference's tests hold no stored plan; the restatement is checked against the source it follows
and against the behaviour its comments state (tests/test_planner_cpu.py)."""

TIER_MS = {16: 62.0, 32: 86.0, 64: 165.0, 96: 230.0, 128: 295.0}
ATTENTION_FIRST, ATTENTION_SECOND = 0.29, 0.22


def tier(rows):
    return 16 if rows <= 16 else ((rows + 31) // 32) * 32


def cycle_ms(rows):
    return TIER_MS.get(tier(rows), rows * 2.3) + 0.45 * rows + 10


def prefill_cap(max_rows, decode_rows, decode_tokens, decode_attention, backlog, first_fed, decode_weight=1.0, prefill_rows_while_decoding=8):
    if backlog <= 0:
        return decode_rows
    per_row = 0.022 * first_fed / 1000
    best_cap, best_rate = min(max_rows, tier(decode_rows + prefill_rows_while_decoding)), 0.0
    for width in (16, 32, 64, 96, 128):
        if not (width <= max_rows and width > decode_rows):
            continue
        prefill = min(backlog, width - decode_rows)
        ms = cycle_ms(decode_rows + prefill) + decode_attention + per_row * prefill
        rate = (decode_weight * decode_tokens + prefill) / ms
        if rate > best_rate:
            best_cap, best_rate = width, rate
    return best_cap


def plan_blocks(tail, block_yield, context_tokens, other_rows=0, block=8, max_rows=128, max_logit_rows=128, max_verify_rows=64, max_context=262144):
    n = len(tail)
    blocks = [block] * n
    base = n * block + other_rows
    thousands = lambda i: context_tokens[i] / 1000
    tail_cost = lambda i: 0.45 * block + ATTENTION_SECOND * thousands(i)
    candidates = sorted((i for i in range(n) if context_tokens[i] + 2 * block < max_context), key=lambda i: -(tail[i] / tail_cost(i)))
    tokens = sum(block_yield) + other_rows
    attention = sum(ATTENTION_FIRST * thousands(i) for i in range(n))
    best_count, best_rate = 0, tokens / (cycle_ms(base) + attention)
    for index, i in enumerate(candidates):
        rows = base + (index + 1) * block
        if not (rows <= max_rows and rows <= max_logit_rows and (n + index + 1) * block <= max_verify_rows):
            break
        tokens += tail[i]
        attention += ATTENTION_SECOND * thousands(i)
        rate = tokens / (cycle_ms(rows) + attention) * (1 if tier(rows) == tier(base) else 0.88)
        if rate > best_rate:
            best_count, best_rate = index + 1, rate
    for i in candidates[:best_count]:
        blocks[i] = 2 * block
    return blocks
