"""The drafter's host arithmetic (no device): DraftModel.quantize with its fitted ranges and CandidateSelector.select
(Sources/SploshRuntime/DraftModel.swift:479-531, 635-719), the library against the numpy restatement."""
import numpy as np

from oracle import draft as OD
from splosh_b200 import draft as SD


def test_quantiser_bit_for_bit_with_fitted_and_minmax_ranges():
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((48, 512)) * 0.02).astype(np.float32)
    w[0, :64] = 0.01            # a flat group: scale 1, bias the value
    w[1, 3] = 0.5               # an outlier: the fitted range clips it
    w[2, :64] = np.linspace(-1, 1, 64)
    bits = OD.bf16_bits(w)
    for fitted in (True, False):
        want, got = OD.quantize(bits, fitted), SD.quantize_q4(bits, fitted)
        for a, b in zip(want, got):
            assert np.array_equal(a, b)
    fitted, minmax = SD.quantize_q4(bits, True), SD.quantize_q4(bits, False)
    assert (fitted[1] != minmax[1]).any()          # the range rule changes some scales

    def error(q):
        codes = np.stack([(q[0] >> (4 * n)) & 15 for n in range(8)], axis=-1).reshape(48, 512).astype(np.float32)
        return ((OD.bits_float(bits) - (np.repeat(OD.bits_float(q[2]), 64, axis=1) + np.repeat(OD.bits_float(q[1]), 64, axis=1) * codes)) ** 2).sum()
    assert error(fitted) <= error(minmax)


def test_selector_greedy_and_sampled_paths():
    rng = np.random.default_rng(9)
    vocab, rank, hidden, k, drafted = 500, 32, 256, 8, 15
    projection = OD.bits_float(OD.bf16_bits((rng.standard_normal((rank, hidden)) * 0.05).astype(np.float32)))
    predecessor = OD.bf16_bits((rng.standard_normal((vocab, rank)) * 0.5).astype(np.float32))
    successor = OD.bf16_bits((rng.standard_normal((vocab, rank)) * 0.5).astype(np.float32))
    ids = np.stack([rng.choice(vocab, k, replace=False) for _ in range(drafted)]).astype(np.int32)
    values = np.sort(rng.standard_normal((drafted, k)).astype(np.float32) * 2, axis=1)[:, ::-1].copy()
    rows = rng.standard_normal((drafted, hidden)).astype(np.float32)
    tokens, none, state = SD.select(ids, values, rows, projection, predecessor, successor, anchor=17)
    want, _, _, margins = OD.select(ids, values, rows, projection, predecessor, successor, 17)
    assert margins.min() > 1e-4 and tokens.tolist() == want and none is None and state == 0
    tokens, probabilities, state = SD.select(ids, values, rows, projection, predecessor, successor, anchor=17, temperature=0.8, random_state=42)
    want, want_p, want_state, _ = OD.select(ids, values, rows, projection, predecessor, successor, 17, temperature=0.8, random_state=42)
    assert tokens.tolist() == want and state == want_state
    assert np.abs(probabilities - want_p).max() <= 1e-5 and np.allclose(probabilities.sum(axis=1), 1, atol=1e-5)
