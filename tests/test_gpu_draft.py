"""The DFlash 2 drafter (Sources/SploshRuntime/DraftModel.swift; Sources/Shaders/draft.metal) on the device against its
numpy restatement (oracle/draft.py): the context pass over the target's feature rows, the block pass (dynamic
convolutions, K/V ring, windowed non-causal attention, the engine's GEMMs) and the candidate selector.

Tolerance of the block pass: 2 % of the largest value. The restatement itself moves by 0.5 % of its largest logit when its
inputs move by 1e-6 (seeded check): every GEMM rounds its activations to bf16, the rings hold fp16, the MLP's product is
rounded to bf16, and a value that crosses a rounding boundary jumps by 2^-8 of itself. The pieces that have no such
boundary are held tighter: the rings to one fp16 step, the candidates and the selector's path exactly."""
import numpy as np
import pytest

import splosh_b200 as S
from helpers import observed
from oracle import draft as OD
from oracle import oracle as O
from safetensors_writer import write as write_safetensors

pytestmark = pytest.mark.gpu

CONFIG = S.DraftConfig(layers=2, heads=4, kv_heads=2, group_size=16, rank=32, window=24, ring_capacity=48, block_size=8, max_block=16,
                       candidates=8, mask_token=31999)
TAPS = [0, 2]


def checkpoint(g, c, seed=11):
    rng = np.random.default_rng(seed)
    H, I, D = g.hidden, g.inter, OD.HEAD_DIM
    groups = H // c.group_size
    t = {}

    def normal(shape, deviation, mean=0.0):
        return OD.bf16_bits((mean + deviation * rng.standard_normal(shape)).astype(np.float32))

    for layer in range(c.layers):
        p = f"layers.{layer}."
        t[p + "input_layernorm.weight"] = normal(H, 0.02, 1.0)
        t[p + "post_attention_layernorm.weight"] = normal(H, 0.02, 1.0)
        t[p + "self_attn.q_norm.weight"] = normal(D, 0.05, 1.0)
        t[p + "self_attn.k_norm.weight"] = normal(D, 0.05, 1.0)
        t[p + "attention_conv.base_kernel"] = normal((4, H), 0.3, 0.5)
        t[p + "mlp_conv.base_kernel"] = normal((4, H), 0.3, 0.5)
        t[p + "self_attn.q_proj.weight"] = normal((c.heads * D, H), 0.03)
        t[p + "self_attn.k_proj.weight"] = normal((c.kv_heads * D, H), 0.03)
        t[p + "self_attn.v_proj.weight"] = normal((c.kv_heads * D, H), 0.03)
        t[p + "self_attn.o_proj.weight"] = normal((H, c.heads * D), 0.03)
        t[p + "mlp.gate_proj.weight"] = normal((I, H), 0.03)
        t[p + "mlp.up_proj.weight"] = normal((I, H), 0.03)
        t[p + "mlp.down_proj.weight"] = normal((H, I), 0.03)
        t[p + "attention_conv.kernel_projection.weight"] = normal((4 * groups, H), 0.01)
        t[p + "mlp_conv.kernel_projection.weight"] = normal((4 * groups, H), 0.01)
    t["fc.weight"] = normal((H, H * len(TAPS)), 0.02)
    t["hidden_norm.weight"] = normal(H, 0.02, 1.0)
    t["norm.weight"] = normal(H, 0.02, 1.0)
    t["candidate_selector.hidden_projection.weight"] = normal((c.rank, H), 0.05)
    t["candidate_selector.predecessor_codebook"] = normal((g.vocab, c.rank), 0.5)
    t["candidate_selector.successor_codebook"] = normal((g.vocab, c.rank), 0.5)
    return t


@pytest.fixture(scope="module")
def setup():
    g = S.tiny_geometry()
    model = O.Model(O.tiny_geometry())
    engine = S.Engine(g, S.EngineConfig(max_slots=2, max_rows=64, kv_pages=8, max_context=1024))
    engine.load_model(model)
    engine.enable_features(TAPS)
    tensors = checkpoint(g, CONFIG)
    draft = S.DraftModel(engine, CONFIG)
    for name, bits in tensors.items():
        draft.set_tensor(name, bits)
    oracle = OD.Draft(model, CONFIG, tensors, TAPS)
    return g, engine, draft, oracle, tensors


def feed(engine, draft, oracle, slot, start, count, seed):
    """A prompt chunk through the target with feature taps, then its rows into both drafters' contexts."""
    rng = np.random.default_rng(seed)
    tokens = rng.integers(0, 31000, count)
    engine.step([S.EngineRow(slot, int(tokens[i]), start + i, i == count - 1) for i in range(count)])
    features = np.stack([engine.feature_row(i) for i in range(count)])
    draft.push_context([(slot, start + i, i) for i in range(count)])
    oracle.push_context(features, [slot] * count, [start + i for i in range(count)])


def numpy_topk(logits, limit, k):
    """TopK.select (Sampler.swift:19-52): value descending, the lower index first among equals."""
    order = np.lexsort((np.arange(limit), -logits[:limit].astype(np.float64)))[:k]
    return order.astype(np.int32), logits[order]


def test_context_rings_and_block_pass_against_the_restatement(setup):
    g, engine, draft, oracle, tensors = setup
    c = CONFIG
    for slot in range(2):
        engine.reset_slot(slot); draft.reset_slot(slot)
    feed(engine, draft, oracle, 0, 0, 30, 1)
    feed(engine, draft, oracle, 0, 30, 30, 2)          # positions 30..59: the ring of 48 wraps, the window of 24 cuts
    feed(engine, draft, oracle, 1, 0, 5, 3)
    assert draft.context_length(0, 60) == 23 and draft.context_length(0, 59) == 0 and draft.context_length(1, 5) == 5
    for layer in range(c.layers):
        ring_shape = (2, c.ring_capacity, c.kv_heads, OD.HEAD_DIM)
        k = draft.debug_read(2, ring_shape, np.float16, layer).astype(np.float32)
        v = draft.debug_read(3, ring_shape, np.float16, layer).astype(np.float32)
        want_k, want_v = oracle.k_ring[layer, :2].astype(np.float32), oracle.v_ring[layer, :2].astype(np.float32)
        observed(f"draft context ring, layer {layer}: max |K - restatement| {np.abs(k - want_k).max():.2e}, |V| {np.abs(v - want_v).max():.2e} "
                 f"(largest {np.abs(want_k).max():.2f}, {np.abs(want_v).max():.2f})")
        assert np.abs(k - want_k).max() <= 4e-3 * np.abs(want_k).max()
        assert np.abs(v - want_v).max() <= 4e-3 * np.abs(want_v).max()
    requests = [S.DraftRequest(0, 1234, 60, 16, True), S.DraftRequest(1, 77, 5, 8)]
    proposals = draft.propose(requests, vocab_limit=31000)
    want = oracle.propose(requests)
    picked = 15 + 7
    logits = draft.debug_read(0, (picked, g.vocab))
    selected = draft.debug_read(1, (picked, g.hidden))
    scale = np.abs(want["logits"]).max()
    observed(f"draft block pass (16-row isolated double block + 8-row block, 2 layers): max |logit - restatement| {np.abs(logits - want['logits']).max():.3e} "
             f"(largest logit {scale:.2f}); hidden rows {np.abs(selected - want['selected']).max():.3e} of {np.abs(want['selected']).max():.2f}")
    assert np.abs(selected - want["selected"]).max() <= 2e-2 * np.abs(want["selected"]).max()
    assert np.abs(logits - want["logits"]).max() <= 2e-2 * scale
    # The selector on the device pass's own logits and hidden rows: the library's path through the candidates is the restatement's.
    at = 0
    for request, proposal in zip(requests, proposals):
        n = request.block - 1
        ids = np.stack([numpy_topk(logits[at + i], 31000, c.candidates)[0] for i in range(n)])
        values = np.stack([numpy_topk(logits[at + i], 31000, c.candidates)[1] for i in range(n)])
        assert np.array_equal(np.array(proposal.candidates), ids)
        tokens, _, _, margins = OD.select(ids, values, selected[at:at + n], OD.bits_float(tensors["candidate_selector.hidden_projection.weight"]),
                                          tensors["candidate_selector.predecessor_codebook"], tensors["candidate_selector.successor_codebook"], request.anchor)
        assert margins.min() > 1e-4, "a near-tie in the seeded scene: reseed"
        assert proposal.tokens == tokens and proposal.probabilities is None
        at += n


def test_sampling_selector_and_a_block_without_context(setup):
    g, engine, draft, oracle, tensors = setup
    c = CONFIG
    draft.random_state = 0xC0FFEE
    # Slot 1 holds positions 0..4 (and the last test's block rows): a block that does not start at its context's end sees only itself.
    requests = [S.DraftRequest(1, 500, 9, 8)]
    assert draft.context_length(1, 9) == 0
    proposals = draft.propose(requests, temperature=0.7, vocab_limit=31000)
    oracle.end[1] = 5
    want = oracle.propose(requests)
    logits = draft.debug_read(0, (7, g.vocab))
    selected = draft.debug_read(1, (7, g.hidden))
    assert np.abs(logits - want["logits"]).max() <= 2e-2 * np.abs(want["logits"]).max()
    ids = np.stack([numpy_topk(logits[i], 31000, c.candidates)[0] for i in range(7)])
    values = np.stack([numpy_topk(logits[i], 31000, c.candidates)[1] for i in range(7)])
    tokens, probabilities, state, _ = OD.select(ids, values, selected, OD.bits_float(tensors["candidate_selector.hidden_projection.weight"]),
                                                tensors["candidate_selector.predecessor_codebook"], tensors["candidate_selector.successor_codebook"], 500,
                                                temperature=0.7, random_state=0xC0FFEE)
    assert draft.random_state == state
    assert proposals[0].tokens == tokens
    assert np.abs(np.array(proposals[0].probabilities) - probabilities).max() <= 1e-5
    observed(f"draft selector at temperature 0.7: seven draws equal to the restatement's, probabilities within {np.abs(np.array(proposals[0].probabilities) - probabilities).max():.1e}")


def test_context_bookkeeping_and_refusals(setup):
    g, engine, draft, oracle, tensors = setup
    draft.reset_slot(0)
    assert draft.context_length(0, 0) == 0
    feed(engine, draft, oracle, 0, 0, 12, 5)
    assert draft.context_length(0, 12) == 12
    draft.truncate(0, 7)
    assert draft.context_length(0, 7) == 7 and draft.context_length(0, 12) == 0
    with pytest.raises(S.EngineError):
        draft.propose([S.DraftRequest(0, 1, 7, 12)])                 # not a multiple of the block
    with pytest.raises(S.EngineError):
        draft.propose([S.DraftRequest(0, 1, 7, 24)])                 # beyond the longest block
    with pytest.raises(S.EngineError):
        draft.set_tensor("layers.0.self_attn.q_proj.weight", np.zeros((16, 256), np.uint16))        # wrong shape
    with pytest.raises(S.EngineError):
        draft.set_tensor("layers.9.mlp.up_proj.weight", np.zeros((16, 256), np.uint16))             # no such layer
    with pytest.raises(S.EngineError):
        S.DraftModel(engine, S.DraftConfig(layers=1, heads=3, kv_heads=2))


@pytest.mark.parametrize("heads, kv_heads", [(4, 2), (8, 1)])
def test_a_window_of_several_chunks_and_spans(heads, kv_heads):
    """A context longer than one chunk: the attention's spans run side by side and are merged; the window cuts the oldest
    positions and the ring has wrapped. Two query heads a kv head take the tensor-core form (a request's queries fit its 64);
    eight take the walk on the CUDA cores."""
    g = S.tiny_geometry()
    model = O.Model(O.tiny_geometry())
    engine = S.Engine(g, S.EngineConfig(max_slots=1, max_rows=64, kv_pages=4, max_context=1024))
    engine.load_model(model)
    engine.enable_features(TAPS)
    config = S.DraftConfig(layers=1, heads=heads, kv_heads=kv_heads, group_size=16, rank=32, window=300, ring_capacity=320, block_size=8, max_block=16,
                           candidates=8, mask_token=31999)
    tensors = checkpoint(g, config, seed=23)
    draft = S.DraftModel(engine, config)
    for name, bits in tensors.items():
        draft.set_tensor(name, bits)
    oracle = OD.Draft(model, config, tensors, TAPS)
    for chunk in range(6):
        feed(engine, draft, oracle, 0, 62 * chunk, 62, 40 + chunk)          # 372 positions: the ring of 320 has wrapped
    assert draft.context_length(0, 372) == 299
    requests = [S.DraftRequest(0, 4321, 372, 16, False)]
    draft.propose(requests, vocab_limit=31000)
    want = oracle.propose(requests)
    logits = draft.debug_read(0, (15, g.vocab))
    selected = draft.debug_read(1, (15, g.hidden))
    observed(f"draft block pass over a 300-position window ({heads} heads on {kv_heads} kv heads, 8 spans, wrapped ring): max |logit - restatement| {np.abs(logits - want['logits']).max():.3e} "
             f"(largest {np.abs(want['logits']).max():.2f}); hidden rows {np.abs(selected - want['selected']).max():.3e} of {np.abs(want['selected']).max():.2f}")
    assert np.abs(selected - want["selected"]).max() <= 2e-2 * np.abs(want["selected"]).max()
    assert np.abs(logits - want["logits"]).max() <= 2e-2 * np.abs(want["logits"]).max()
    draft.close(); engine.close()


def test_a_safetensors_checkpoint_and_a_context_snapshot(setup, tmp_path):
    """The checkpoint from a bf16 safetensors file steps like the one given tensor by tensor; a slot's context exported and
    imported into another slot drafts the same block; refused files say why in the reference's words."""
    g, engine, draft, oracle, tensors = setup
    shaped = dict(tensors)
    for layer in range(CONFIG.layers):
        for name in ("attention_conv.base_kernel", "mlp_conv.base_kernel"):
            shaped[f"layers.{layer}.{name}"] = tensors[f"layers.{layer}.{name}"].reshape(2, 2, g.hidden)
    assert dict(draft.expected_tensors()) == {n: tuple(np.shape(b)) for n, b in shaped.items()}
    path = tmp_path / "draft.safetensors"
    write_safetensors(path, shaped, metadata={"format": "pt"})
    loaded = S.DraftModel(engine, CONFIG)
    loaded.load_safetensors(path)
    for d in (draft, loaded):
        d.reset_slot(0); d.reset_slot(1)
    engine.reset_slot(0)
    rng = np.random.default_rng(77)
    toks = rng.integers(0, 31000, 20)
    engine.step([S.EngineRow(0, int(toks[i]), i, i == 19) for i in range(20)])
    for d in (draft, loaded):
        d.push_context([(0, i, i) for i in range(20)])
    request = [S.DraftRequest(0, 4242, 20, 8)]
    a = draft.propose(request, vocab_limit=31000)[0]
    logits_a = draft.debug_read(0, (7, g.vocab))
    b = loaded.propose(request, vocab_limit=31000)[0]
    assert np.array_equal(logits_a, loaded.debug_read(0, (7, g.vocab))) and a.tokens == b.tokens and a.candidates == b.candidates
    # the slot's context into slot 1 of the same drafter
    snapshot = draft.export_context(0, 20)
    assert snapshot is not None and snapshot[0] == 0 and snapshot[1] == 20 and draft.export_context(0, 25) is None
    draft.import_context(1, snapshot)
    assert draft.context_length(1, 20) == 20
    c = draft.propose([S.DraftRequest(1, 4242, 20, 8)], vocab_limit=31000)[0]
    assert np.array_equal(logits_a, draft.debug_read(0, (7, g.vocab))) and c.tokens == a.tokens
    draft.import_context(1, (0, 20, snapshot[2][:-2]))                 # a snapshot of another size resets the slot
    assert draft.context_length(1, 20) == 0
    # refusals
    fresh = S.DraftModel(engine, CONFIG)
    write_safetensors(path, shaped, drop=("norm.weight",))
    with pytest.raises(S.EngineError, match="missing tensor norm.weight"):
        fresh.load_safetensors(path)
    write_safetensors(path, shaped, lie={"fc.weight": "F16"})
    with pytest.raises(S.EngineError, match=r"fc.weight is F16 \[1024, 2048\]; expected BF16 \[1024, 2048\]"):
        fresh.load_safetensors(path)
    bad = dict(shaped); bad["hidden_norm.weight"] = shaped["hidden_norm.weight"][:512]
    write_safetensors(path, bad)
    with pytest.raises(S.EngineError, match=r"hidden_norm.weight is BF16 \[512\]; expected BF16 \[1024\]"):
        fresh.load_safetensors(path)
    with open(path, "wb") as f:
        f.write(b"\xff" * 64)
    with pytest.raises(S.EngineError, match="bad safetensors header"):
        fresh.load_safetensors(path)
    with pytest.raises(S.EngineError, match="cannot open"):
        fresh.load_safetensors(tmp_path / "nothing.safetensors")
    loaded.close(); fresh.close()
