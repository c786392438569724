"""The host-side sampler of the C ABI (spl_sample_topk, spl_sampler_distribution, spl_speculative_resolve,
spl_sampler_uniform) against the CPU restatement of Sources/SploshRuntime/Sampler.swift in oracle/sampler.py:
the same seeds must give the same uniforms bit for bit and the same tokens. No GPU is involved: the entry
points take the k largest logits, which `spl_topk` produces on the device (tests/test_gpu_step.py)."""
import numpy as np

import splosh_b200 as S
from oracle import sampler as OS


def candidates(rng, k=20, vocab=32000, spread=3.0):
    logits = (rng.normal(0, spread, vocab)).astype(np.float32)
    ids, values = OS.topk_select(logits, vocab, k)
    return logits, ids, values


def test_uniforms_are_splitmix64_top_24_bits():
    mine, ref = S.Sampler(seed=0x5EED6D17), OS.Sampler(seed=0x5EED6D17)
    for _ in range(1000):
        assert np.float32(mine.uniform01()) == ref.uniform()
    assert mine.state.value == ref.state


def test_topk_select_orders_by_value_then_index_and_leaves_unfilled_slots():
    logits = np.array([1.0, 3.0, 3.0, -np.inf, 2.0, np.nan, 3.0], np.float32)
    ids, values = OS.topk_select(logits, 7, 6)
    assert ids == [1, 2, 6, 4, 0, 0] and list(values[:5]) == [3.0, 3.0, 3.0, 2.0, 1.0] and values[5] == -np.inf


def test_sample_sequence_equals_the_restated_sampler():
    rng = np.random.default_rng(7)
    for temperature, top_p, k in ((1.0, 0.95, 20), (0.7, 0.5, 20), (1.3, 1.0, 64), (0.0, 0.95, 20), (1.0, 0.95, 1)):
        mine, ref = S.Sampler(temperature, top_p, k, seed=42), OS.Sampler(temperature, top_p, k, seed=42)
        for _ in range(200):
            _, ids, values = candidates(rng, k)
            assert mine.sample(ids, values) == ref.sample(ids, values)
        assert mine.state.value == ref.state


def test_distribution_is_the_kept_nucleus_renormalised():
    rng = np.random.default_rng(11)
    for temperature, top_p in ((1.0, 0.95), (0.5, 0.3), (2.0, 1.0), (0.0, 0.9)):
        mine, ref = S.Sampler(temperature, top_p, 20), OS.Sampler(temperature, top_p, 20)
        for _ in range(50):
            _, ids, values = candidates(rng, 20, spread=1.5)
            mi, mp = mine.distribution(ids, values); ri, rp = ref.distribution(ids, values)
            assert list(mi) == list(ri) and np.allclose(mp, rp, rtol=2e-6, atol=0) and abs(float(mp.sum()) - 1) < 1e-5


def test_speculative_resolve_keeps_or_replaces_like_the_reference():
    rng = np.random.default_rng(13)
    mine, ref = S.Sampler(1.0, 0.95, 20, seed=99), OS.Sampler(1.0, 0.95, 20, seed=99)
    outcomes = set()
    for _ in range(300):
        _, tids, tvalues = candidates(rng, 20, spread=1.0)
        tids, tp = ref.distribution(tids, tvalues)
        # A draft distribution over an overlapping candidate set.
        cids = list(tids[: max(1, len(tids) // 2)]) + [int(x) for x in rng.integers(0, 32000, 4)]
        q = rng.random(len(cids)).astype(np.float32); q /= q.sum()
        draft = cids[int(rng.integers(0, len(cids)))]
        a = mine.resolve(draft, cids, q, tids, tp); b = ref.resolve(draft, cids, q, tids, tp)
        assert a == b
        outcomes.add(a is None)
    assert outcomes == {True, False} and mine.state.value == ref.state
