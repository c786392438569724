"""Seeded synthetic model parts that are generated on the host: the small bf16 vectors.

The 4-bit projection weights are generated on the device (spl_weights_synthesize_q4). Both follow
one recipe: stream seed = base seed ^ fnv1a64(tensor name), value n of a stream from SplitMix64
(the generator of the reference's tests, Tests/SploshOracleTests/GdnCandidateTests.swift:118-134)
evaluated at index n. Norm weights are bf16(1 + N(0, 0.02)) and are applied directly, the
convention of the reference's engine (Sources/Shaders/engine.metal:147-149); conv1d, A_log and
dt_bias are uniform in the ranges of GdnCandidateTests.swift:141-145.
"""
import numpy as np

VEC_NAMES = {"input_norm": "input_layernorm", "post_norm": "post_attention_layernorm", "conv": "linear_attn.conv1d",
             "a_log": "linear_attn.A_log", "dt_bias": "linear_attn.dt_bias", "gdn_norm": "linear_attn.norm",
             "q_norm": "self_attn.q_norm", "k_norm": "self_attn.k_norm", "final_norm": "norm"}
_MASK = (1 << 64) - 1


def fnv1a64(text):
    h = 0xcbf29ce484222325
    for byte in text.encode():
        h = ((h ^ byte) * 0x100000001b3) & _MASK
    return h


def tensor_seed(base, layer, name):
    return base ^ fnv1a64(f"layers.{layer}.{name}" if layer >= 0 else name)


def splitmix_at(seed, n):
    """SplitMix64 outputs at indices n (array of uint64) of the stream starting at seed."""
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + (np.asarray(n, np.uint64) + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def uniform_at(seed, n):
    return (splitmix_at(seed, n) >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)


def normal_at(seed, n, deviation):
    """Centred sum of the four 16-bit fields of one draw (Irwin-Hall, n = 4) scaled to `deviation`."""
    z = splitmix_at(seed, n)
    total = ((z & np.uint64(0xFFFF)) + ((z >> np.uint64(16)) & np.uint64(0xFFFF)) + ((z >> np.uint64(32)) & np.uint64(0xFFFF))
             + (z >> np.uint64(48))).astype(np.int64) - 131070
    factor = np.float32(deviation) * (np.float32(1.0) / np.float32(37837.2265625))
    return total.astype(np.float32) * factor


def to_bf16(values):
    bits = np.ascontiguousarray(values, np.float32).view(np.uint32)
    return ((bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def vector(geometry, base_seed, layer, kind):
    """bf16 bits of one small tensor of the synthetic model."""
    g = geometry
    count = {"input_norm": g.hidden, "post_norm": g.hidden, "final_norm": g.hidden, "conv": g.channels * 4,
             "a_log": g.gdn_value_heads, "dt_bias": g.gdn_value_heads, "gdn_norm": g.gdn_head_dim,
             "q_norm": g.head_dim, "k_norm": g.head_dim}[kind]
    seed = tensor_seed(base_seed, layer, VEC_NAMES[kind])
    n = np.arange(count, dtype=np.uint64)
    ranges = {"conv": (-0.6, 0.6), "a_log": (-2.0, 1.0), "dt_bias": (-1.0, 1.0)}
    if kind in ranges:
        lo, hi = np.float32(ranges[kind][0]), np.float32(ranges[kind][1])
        values = lo + (hi - lo) * uniform_at(seed, n)
    else:
        values = np.float32(1.0) + normal_at(seed, n, 0.02)
    return to_bf16(values)


def load_vectors(engine, base_seed):
    """Set every bf16 vector of the synthetic model on an engine."""
    g = engine.g
    for layer in range(g.layers):
        full = layer % 4 == 3
        for kind in ["input_norm", "post_norm"] + (["q_norm", "k_norm"] if full else ["conv", "a_log", "dt_bias", "gdn_norm"]):
            engine.set_vector(layer, kind, vector(g, base_seed, layer, kind))
    engine.set_vector(-1, "final_norm", vector(g, base_seed, -1, "final_norm"))
