"""Self-consistency of the CPU oracle's composed step: the properties the reference checks with
its in-engine self-tests (Sources/SploshCLI/GenerateCommand.swift:171-251 verify rows against
ordinary rows; :586-660 blocks re-verified after partial acceptance) hold for the oracle, and the
seeded synthetic model is reproducible."""
import numpy as np
import pytest

from helpers import Pair, tokens_for
import splosh_b200 as S
from splosh_b200 import synthetic


def small_geometry():
    g = S.tiny_geometry()
    return S.Geometry(4, 256, 512, 2048, 4, 2, 128, 32, 2, 4, 128, 1e-6, 1e7)


@pytest.fixture(scope="module")
def toks():
    return tokens_for(0xC0FFEE00, 4096, 2048)


def test_chunked_prefill_equals_token_by_token(toks):
    """A prompt fed as one chunk, as ragged chunks, or one row a step gives the same last-token logits
    (state carried in HBM between steps; conv history per unit)."""
    g = small_geometry()
    cfg = S.EngineConfig(max_slots=2, max_rows=64, kv_pages=8, max_context=1024)
    results = []
    for chunks in ([40], [7, 1, 16, 3, 13], [1] * 40):
        pair = Pair(g, cfg, gpu=False)
        fed = 0
        for n in chunks:
            _, logits = pair.step([S.EngineRow(0, toks[fed + i], fed + i, fed + i == 39) for i in range(n)])
            fed += n
        results.append(logits[0])
    for other in results[1:]:
        assert np.abs(other - results[0]).max() < 2e-2 * max(1.0, np.abs(results[0]).max())
        assert np.argmax(other) == np.argmax(results[0])


def test_verify_rows_equal_ordinary_rows_and_partial_acceptance_replays(toks):
    """Rows evaluated as a speculative block give the logits ordinary rows give; after accepting a
    prefix of the block the next step sees exactly the state an ordinary evaluation of that prefix
    leaves (journal replay + conv unit of the last kept row + KV truncation)."""
    g = small_geometry()
    cfg = S.EngineConfig(max_slots=2, max_rows=64, kv_pages=8, max_context=1024)
    plain = Pair(g, cfg, gpu=False); spec = Pair(g, cfg, gpu=False)
    prompt = 20
    for pair in (plain, spec):
        pair.step([S.EngineRow(0, toks[i], i, False) for i in range(prompt)])
    for keep in (1, 3, 8, 5):
        width = 8
        _, block = spec.step([S.EngineRow(0, toks[prompt + i], prompt + i, True, True) for i in range(width)])
        ordinary = []
        for i in range(keep):
            _, lg = plain.step([S.EngineRow(0, toks[prompt + i], prompt + i, True)])
            ordinary.append(lg[0])
        for i in range(keep):
            assert np.abs(block[i] - ordinary[i]).max() < 2e-2
            assert np.argmax(block[i]) == np.argmax(ordinary[i])
        spec.accept(0, keep, prompt + keep)
        prompt += keep
    # A rejected block leaves no trace.
    spec.step([S.EngineRow(0, toks[3000 + i], prompt + i, True, True) for i in range(6)])
    spec.ohost.discard_verify(0)
    _, a = spec.step([S.EngineRow(0, toks[prompt], prompt, True)])
    _, b = plain.step([S.EngineRow(0, toks[prompt], prompt, True)])
    assert np.abs(a - b).max() < 2e-2 and np.argmax(a) == np.argmax(b)


def test_deferred_norm_contract_is_the_plain_norm_up_to_rounding(toks):
    """The deferred form (operand bf16(h w), sums scaled by the row's rsqrt afterwards: Sources/Shaders/engine_na.metal:365-415,
    Sources/SploshRuntime/Engine.swift:1439-1451) and the plain RMSNorm (Sources/Shaders/engine.metal:159-178) differ only in
    where the bf16 rounding of the operand falls: same arg-max, logits within the step's tolerance."""
    import oracle.oracle as O
    g = small_geometry()
    cfg = S.EngineConfig(max_slots=2, max_rows=64, kv_pages=8, max_context=1024)
    rows = [S.EngineRow(0, toks[i], i, True) for i in range(24)]
    results = []
    try:
        for deferred in (True, False):
            O.set_norm_contract(deferred)
            pair = Pair(g, cfg, gpu=False)
            _, logits = pair.step(rows)
            results.append(logits)
    finally:
        O.set_norm_contract(True)
    a, b = results
    assert np.abs(a - b).max() > 0.0                      # the switch does something
    assert np.abs(a - b).max() < 2e-2 * max(1.0, np.abs(a).max())
    assert (np.argmax(a, axis=1) == np.argmax(b, axis=1)).mean() > 0.9


def test_sessions_do_not_interact(toks):
    """Rows of different slots share only the weights: a session's logits are the same alone or packed
    with others (what makes sharding by session exact)."""
    g = small_geometry()
    cfg = S.EngineConfig(max_slots=3, max_rows=64, kv_pages=12, max_context=1024)
    alone = Pair(g, cfg, gpu=False); packed = Pair(g, cfg, gpu=False)
    _, a = alone.step([S.EngineRow(1, toks[i], i, i == 11) for i in range(12)])
    rows = [S.EngineRow(0, toks[100 + i], i, i == 4) for i in range(5)] + [S.EngineRow(1, toks[i], i, i == 11) for i in range(12)] + \
           [S.EngineRow(2, toks[200 + i], i, False) for i in range(9)]
    _, b = packed.step(rows)
    assert np.array_equal(a[0], b[1])


def test_synthetic_vectors_match_between_package_and_oracle(oracle):
    g = S.tiny_geometry()
    model = oracle.Model(oracle.tiny_geometry())
    for layer, kind in [(0, "input_norm"), (0, "conv"), (1, "a_log"), (2, "dt_bias"), (0, "gdn_norm"), (3, "q_norm"), (3, "k_norm"),
                        (-1, "final_norm"), (3, "post_norm")]:
        assert np.array_equal(synthetic.vector(g, 0x5EED6D17, layer, kind), model.vec(layer, kind)), (layer, kind)


def test_synthetic_weights_have_the_stated_distribution(oracle):
    lib = oracle.lib()
    values = np.array([lib.orc_normal_at(12345, i, 0.02) for i in range(20000)])
    assert abs(values.mean()) < 5e-4 and abs(values.std() - 0.02) < 4e-4
    assert np.array_equal(synthetic.normal_at(12345, np.arange(2000), 0.02), values[:2000].astype(np.float32))
    u = np.array([lib.orc_uniform_at(777, i) for i in range(5000)])
    assert 0 <= u.min() and u.max() < 1 and abs(u.mean() - 0.5) < 0.02
    assert np.array_equal(synthetic.uniform_at(777, np.arange(5000)), u.astype(np.float32))


def test_gguf_weighted_oracle_stays_close_to_the_affine_model(toks):
    """The same synthetic model re-quantised to Q5_K blocks with a Q6_K embedding and head (the build's own encoder: parity is
    defined on the decoded blocks) gives logits close to the MLX affine-4 model's: the GGUF branch of the oracle's GEMM and its
    exact embedding decode are wired to the right tensors."""
    import oracle.oracle as O
    g = small_geometry()
    cfg = S.EngineConfig(max_slots=2, max_rows=64, kv_pages=8, max_context=1024)
    rows = [S.EngineRow(0, toks[i], i, True) for i in range(16)]
    O.set_norm_contract(False)
    try:
        _, plain = Pair(g, cfg, gpu=False).step(rows)
        _, gguf = Pair(g, cfg, gpu=False, gguf=("Q5_K", "Q6_K")).step(rows)
    finally:
        O.set_norm_contract(True)
    assert np.abs(plain - gguf).max() > 0.0
    # Re-quantising 4-bit weights moves every logit of a random model a little: the two stay strongly correlated.
    assert np.corrcoef(plain.ravel(), gguf.ravel())[0, 1] > 0.9
