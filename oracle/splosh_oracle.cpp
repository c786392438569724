// splosh_oracle.cpp — CPU restatement of Splosh's packed ragged step.
//
// TEST INFRASTRUCTURE ONLY. This file is the checker the CUDA path is compared with; nothing in
// the shipped library may include, link or call it. It restates, in plain C++ with OpenMP, the
// arithmetic of the reference's step (Sources/SploshRuntime/Engine.swift:1316-1540) and of the
// Metal kernels that step dispatches, with geometry as a parameter instead of the reference's
// hard-coded 27B shape.
//
// Parity status: the per-format pieces (MLX affine-4 decode, Q4_K/Q5_K/Q6_K block decode, the
// gated-delta recurrence's hand cases, RoPE and SwiGLU) are pinned against the reference's own
// golden vectors and known-answer tests (see tests/test_oracle_pins.py). The WHOLE STEP is
// "parity unpinned": the reference holds no stored vector for a whole step and its own whole-step
// CPU path fails closed (Sources/SploshCLI/OracleCommand.swift:85-86), so the step composed here
// is defined by the sources cited at each function.
//
// Numerical contract (the accelerator path's rounding points, for every row count):
//   * GEMM activations are rounded to bf16 (RNE) (Sources/Shaders/engine_na.metal:42-57).
//     Weight contract 0 (default; the reference's accelerator q4 path and what the CUDA path
//     computes): per 64-group the dot of activations with the raw 4-bit codes, then
//     acc += dot * scale + sum * bias with the per-64 sums of the rounded activations
//     (engine_na.metal:91-103, Tests/SploshOracleTests/MlpFusedTests.swift:195-210).
//     Weight contract 1 (a study switch, not what ships): each weight is first rounded to bf16,
//     as the reference's GGUF tile kernels round a dequantised weight to 16 bits
//     (Sources/Shaders/gguf_formats.h:401-438). On the tiny model it moves logits by up to 0.07
//     and flips 6% of arg-maxes against contract 0, which is why the CUDA path keeps contract 0.
//   * residual stream, GEMM outputs, norms, conv, recurrence and softmax statistics are fp32.
//   * K/V are symmetric int8 with one fp32 scale per (token, kv head)
//     (engine_na.metal:2044-2094); queries are rounded to fp16 (engine_na.metal:1259); the
//     probability operand of P.V is bf16(p * vScale) (Sources/Shaders/candidates/attn_scan_r.metal:157).
//   * stored norm weights are applied directly (engine.metal:147-149,176).
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <string>
#include <algorithm>
#include <limits>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ------------------------------------------------------------------------------------------
// Scalars

inline float bf16_to_float(uint16_t bits) { uint32_t u = uint32_t(bits) << 16; float f; memcpy(&f, &u, 4); return f; }
// Round to nearest even, the rule of Sources/SploshRuntime/DraftModel.swift:721-724.
inline uint16_t float_to_bf16(float v) {
    uint32_t bits; memcpy(&bits, &v, 4);
    return uint16_t((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
}
inline float round_bf16(float v) { return bf16_to_float(float_to_bf16(v)); }
inline float round_f16(float v) { return float(_Float16(v)); }
// bf16(scale * code + bias) with one rounding: the sum is exact in double, goes to float by
// round-to-odd (which cannot create a tie), then to bf16 by nearest-even.
inline float bf16_fma_once(float code, float scale, float bias) {
    const double exact = double(code) * double(scale) + double(bias);
    float f = float(exact);
    if (double(f) != exact) {
        if (fabs(double(f)) > fabs(exact)) f = nextafterf(f, 0.0f);
        uint32_t bits; memcpy(&bits, &f, 4); bits |= 1u; memcpy(&f, &bits, 4);
    }
    return round_bf16(f);
}
int g_weight_contract = 0;
int g_norm_contract = 1;      // 1: a norm fed by a residual GEMM takes the deferred form (the shipped contract); 0: every norm plain
inline float silu(float x) { return x / (1.0f + expf(-x)); }
inline float sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }

// SplitMix64 as the reference's tests use it (Tests/SploshOracleTests/GdnCandidateTests.swift:118-134).
// The n-th output of a stream depends only on seed + n * gamma, so any element can be produced
// independently.
inline uint64_t splitmix_at(uint64_t seed, uint64_t n) {
    uint64_t z = seed + (n + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
inline float uniform_at(uint64_t seed, uint64_t n) { return float(splitmix_at(seed, n) >> 40) * (1.0f / 16777216.0f); }
// An approximately normal value from one draw: the centred sum of the draw's four 16-bit fields
// (Irwin-Hall, n = 4) scaled to the requested deviation. Integer up to the last multiply, so a
// device generator reproduces it bit for bit.
inline float normal_at(uint64_t seed, uint64_t n, float deviation) {
    const uint64_t z = splitmix_at(seed, n);
    const int32_t sum = int32_t(z & 0xFFFF) + int32_t((z >> 16) & 0xFFFF) + int32_t((z >> 32) & 0xFFFF) + int32_t(z >> 48);
    // Each field has variance (65536^2 - 1) / 12; four of them 37837.2^2.
    return float(sum - 131070) * (deviation * (1.0f / 37837.2265625f));
}
inline uint64_t fnv1a64(const char *s) {
    uint64_t h = 0xcbf29ce484222325ull;
    for (; *s; ++s) { h ^= uint8_t(*s); h *= 0x100000001b3ull; }
    return h;
}

struct Geometry {
    int32_t layers, hidden, inter, vocab;
    int32_t heads, kv_heads, head_dim, rotary_dim;
    int32_t gdn_key_heads, gdn_value_heads, gdn_head_dim;
    float eps, rope_theta;
    int channels() const { return (2 * gdn_key_heads + gdn_value_heads) * gdn_head_dim; }
    int value_dim() const { return gdn_value_heads * gdn_head_dim; }
    bool full(int layer) const { return layer % 4 == 3; }   // Sources/SploshModel/LayerGraph.swift:22
};

// MLX affine 4-bit, group 64 (Sources/SploshQuant/MlxAffine.swift:1-2,72-84).
struct Q4 {
    int rows = 0, inner = 0;
    std::vector<uint32_t> packed;    // [rows][inner / 8], eight low-first nibbles per word
    std::vector<uint16_t> scales;    // [rows][inner / 64] bf16
    std::vector<uint16_t> biases;
    // A GGUF-weighted model holds the tensor as native K-quant super-blocks instead ([rows][inner / 256], format = the
    // GGUF type number 12, 13 or 14); the MLX arrays above are then ignored.
    int gguf_format = 0;
    std::vector<uint8_t> gguf;
};

// The quantiser of Sources/SploshRuntime/DraftModel.swift:634-670 with the "minmax" range rule.
void quantize_group(const float *v, uint32_t *words, uint16_t *scale_bits, uint16_t *bias_bits) {
    float lo = INFINITY, hi = -INFINITY;
    for (int i = 0; i < 64; ++i) { lo = std::min(lo, v[i]); hi = std::max(hi, v[i]); }
    *scale_bits = float_to_bf16(hi > lo ? (hi - lo) / 15.0f : 1.0f);
    *bias_bits = float_to_bf16(lo);
    const float scale = bf16_to_float(*scale_bits), bias = bf16_to_float(*bias_bits);
    for (int w = 0; w < 8; ++w) {
        uint32_t bits = 0;
        for (int n = 0; n < 8; ++n) {
            const float code = std::min(15.0f, std::max(0.0f, roundf((v[w * 8 + n] - bias) / scale)));
            bits |= uint32_t(code) << (4 * n);
        }
        words[w] = bits;
    }
}

void synth_q4(Q4 &t, int rows, int inner, uint64_t seed, float deviation) {
    t.rows = rows; t.inner = inner;
    t.packed.resize(size_t(rows) * inner / 8);
    t.scales.resize(size_t(rows) * inner / 64);
    t.biases.resize(size_t(rows) * inner / 64);
    const int groups = inner / 64;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float v[64];
        for (int g = 0; g < groups; ++g) {
            const uint64_t first = uint64_t(r) * inner + uint64_t(g) * 64;
            for (int i = 0; i < 64; ++i) v[i] = normal_at(seed, first + i, deviation);
            const size_t slot = size_t(r) * groups + g;
            quantize_group(v, &t.packed[slot * 8], &t.scales[slot], &t.biases[slot]);
        }
    }
}

struct Layer {
    bool full = false;
    Q4 q4[12];                          // indexed by the ORC_Q4_* kinds below
    std::vector<uint16_t> vec[8];       // indexed by the ORC_VEC_* kinds below
};

enum { Q_QKV = 0, Q_Z, Q_A, Q_B, Q_OUT, Q_Q, Q_K, Q_V, Q_O, Q_GATE, Q_UP, Q_DOWN, Q_EMBED, Q_HEAD };
enum { V_IN_NORM = 0, V_POST_NORM, V_CONV, V_A_LOG, V_DT_BIAS, V_GDN_NORM, V_Q_NORM, V_K_NORM, V_FINAL_NORM };

struct Model {
    Geometry g;
    uint64_t seed;
    std::vector<Layer> layers;
    Q4 embed, head;
    std::vector<uint16_t> final_norm;
    // The gated-delta out projections hold their columns in a GGUF file's order of the value heads (file head i = engine head
    // ratio (i % key heads) + i / key heads, Sources/SploshModel/GgufNames.swift:73-84; the out projection stays in file order,
    // Sources/SploshModel/GgufConvert.swift:18-24): the blocks' outputs are arranged in that order before the projection.
    bool out_file_order = false;
};

uint64_t tensor_seed(uint64_t base, int layer, const char *name) {
    char full[128];
    if (layer >= 0) snprintf(full, sizeof full, "layers.%d.%s", layer, name); else snprintf(full, sizeof full, "%s", name);
    return base ^ fnv1a64(full);
}

void synth_vec(std::vector<uint16_t> &out, int count, uint64_t seed, int law, float a, float b) {
    out.resize(count);
    for (int i = 0; i < count; ++i) {
        // law 0: a + N(0, b); law 1: U(a, b)
        const float v = law == 0 ? a + normal_at(seed, i, b) : a + (b - a) * uniform_at(seed, i);
        out[i] = float_to_bf16(v);
    }
}

const char *q4_names[14] = {"linear_attn.in_proj_qkv", "linear_attn.in_proj_z", "linear_attn.in_proj_a", "linear_attn.in_proj_b",
                            "linear_attn.out_proj", "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                            "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj", "embed_tokens", "lm_head"};
const char *vec_names[9] = {"input_layernorm", "post_attention_layernorm", "linear_attn.conv1d", "linear_attn.A_log",
                            "linear_attn.dt_bias", "linear_attn.norm", "self_attn.q_norm", "self_attn.k_norm", "norm"};

void q4_shape(const Geometry &g, int kind, int *rows, int *inner) {
    const int H = g.hidden, VD = g.value_dim(), AD = g.heads * g.head_dim, KV = g.kv_heads * g.head_dim;
    switch (kind) {
    case Q_QKV: *rows = g.channels(); *inner = H; break;
    case Q_Z: *rows = VD; *inner = H; break;
    case Q_A: case Q_B: *rows = g.gdn_value_heads; *inner = H; break;
    case Q_OUT: *rows = H; *inner = VD; break;
    case Q_Q: *rows = 2 * AD; *inner = H; break;
    case Q_K: case Q_V: *rows = KV; *inner = H; break;
    case Q_O: *rows = H; *inner = AD; break;
    case Q_GATE: case Q_UP: *rows = g.inter; *inner = H; break;
    case Q_DOWN: *rows = H; *inner = g.inter; break;
    default: *rows = g.vocab; *inner = H; break;
    }
}

// ------------------------------------------------------------------------------------------
// Engine state

constexpr int kPageTokens = 256;      // Sources/SploshRuntime/Engine.swift:124
constexpr int kJournalRows = 16;      // Engine.swift:300
constexpr int kJournalWidth = 260;    // Sources/Shaders/engine.metal:639-641

struct Tables {                       // what Engine.step builds, Engine.swift:1322-1398
    uint32_t rows, run_count, logit_rows, attn_block_count, step_pages, live_rows, spans, pages_per_span;
    const uint32_t *tokens, *row_slot, *row_pos, *runs, *run_info, *row_read, *row_write, *gather_index;
    const uint32_t *attn_blocks, *page_table;
};

struct Engine {
    const Model *m;
    int max_slots, kv_pages, max_pages, state_units;
    std::vector<std::vector<int8_t>> k_codes, v_codes;    // per full layer [page][kvHead][256][headDim]
    std::vector<std::vector<float>> k_scale, v_scale;     // per full layer [page][kvHead][256]
    std::vector<std::vector<float>> state;                // per linear layer [slot][valueHead][value j][key i]
    std::vector<std::vector<float>> conv;                 // per linear layer [unit][channel][3], oldest first
    std::vector<std::vector<float>> journal;              // per linear layer [slot][16][valueHead][260]
};

struct Operand {                       // a GEMM's activation input: bf16-rounded values and per-64 sums
    int rows, inner;
    std::vector<float> values, sums;
    Operand(int r, int k) : rows(r), inner(k), values(size_t(r) * k), sums(size_t(r) * k / 64) {}
    void finish_row(int r) {
        for (int g = 0; g < inner / 64; ++g) {
            float s = 0;
            const float *v = &values[size_t(r) * inner + g * 64];
            for (int i = 0; i < 64; ++i) s += v[i];
            sums[size_t(r) * (inner / 64) + g] = s;
        }
    }
};

// out[r][n] = sum_k a[r][k] * w[n][k] (+ residual), under the weight contract in force.
extern "C" {
void orc_gguf_tile_weights(int format, const uint8_t *data, int blocks, float *out);
void orc_decode_q45k(const uint8_t *data, int blocks, int fifth_bit, float *out);
void orc_decode_q6k(const uint8_t *data, int blocks, float *out);
}

// The GGUF branch of the GEMM (Sources/SploshRuntime/Engine.swift:1666-1695, Sources/Shaders/engine_gguf.metal:82-273): the
// bf16-rounded activations against weights formed as the tile kernels form them (one fp32 operation, rounded to fp16).
void gemm_gguf_model(const Q4 &w, const Operand &a, int rows, float *out, int out_stride, const float *residual, const float *row_scale) {
    const int K = w.inner, per_row = K / 256, bytes = w.gguf_format == 14 ? 210 : w.gguf_format == 13 ? 176 : 144;
#pragma omp parallel
    {
        std::vector<float> weights(K);
#pragma omp for schedule(static)
        for (int n = 0; n < w.rows; ++n) {
            orc_gguf_tile_weights(w.gguf_format, w.gguf.data() + size_t(n) * per_row * bytes, per_row, weights.data());
            for (int r = 0; r < rows; ++r) {
                const float *x = &a.values[size_t(r) * K];
                double acc = 0;
                for (int i = 0; i < K; ++i) acc += double(x[i] * weights[i]);
                const size_t index = size_t(r) * out_stride + n;
                out[index] = residual ? float(acc + double(residual[index])) : row_scale ? float(acc) * row_scale[r] : float(acc);
            }
        }
    }
}

void gemm(const Q4 &w, const Operand &a, int rows, float *out, int out_stride, const float *residual, const float *row_scale = nullptr) {
    if (w.gguf_format) { gemm_gguf_model(w, a, rows, out, out_stride, residual, row_scale); return; }
    const int K = w.inner, groups = K / 64;
    const bool rounded = g_weight_contract == 1;
#pragma omp parallel
    {
        std::vector<float> codes(K);
#pragma omp for schedule(static)
        for (int n = 0; n < w.rows; ++n) {
            const uint32_t *pw = &w.packed[size_t(n) * K / 8];
            for (int i = 0; i < K / 8; ++i) {
                const uint32_t word = pw[i];
                for (int j = 0; j < 8; ++j) codes[i * 8 + j] = float((word >> (4 * j)) & 0xF);
            }
            if (rounded)
                for (int g = 0; g < groups; ++g) {
                    const float sc = bf16_to_float(w.scales[size_t(n) * groups + g]), bi = bf16_to_float(w.biases[size_t(n) * groups + g]);
                    for (int i = 0; i < 64; ++i) codes[g * 64 + i] = bf16_fma_once(codes[g * 64 + i], sc, bi);
                }
            for (int r = 0; r < rows; ++r) {
                const float *av = &a.values[size_t(r) * K];
                double acc = 0;
                for (int g = 0; g < groups; ++g) {
                    const float *x = av + g * 64, *c = &codes[g * 64];
                    if (rounded) {
                        // bf16 x bf16 products are exact in fp32; eight double lanes keep the sum exact enough.
                        double lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                        for (int k = 0; k < 64; k += 8)
                            for (int j = 0; j < 8; ++j) lane[j] += double(x[k + j] * c[k + j]);
                        acc += ((lane[0] + lane[1]) + (lane[2] + lane[3])) + ((lane[4] + lane[5]) + (lane[6] + lane[7]));
                    } else {
                        float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                        for (int k = 0; k < 64; k += 8)
                            for (int j = 0; j < 8; ++j) lane[j] += x[k + j] * c[k + j];
                        const float dot = ((lane[0] + lane[1]) + (lane[2] + lane[3])) + ((lane[4] + lane[5]) + (lane[6] + lane[7]));
                        acc += double(dot) * bf16_to_float(w.scales[size_t(n) * groups + g])
                             + double(a.sums[size_t(r) * groups + g]) * bf16_to_float(w.biases[size_t(n) * groups + g]);
                    }
                }
                const size_t index = size_t(r) * out_stride + n;
                // A deferred norm's per-row factor multiplies the finished sum (one fp32 multiply), as the consumers of the
                // reference's deferred path apply rowInv to the GEMM's output.
                out[index] = residual ? float(acc + double(residual[index])) : row_scale ? float(acc) * row_scale[r] : float(acc);
            }
        }
    }
}

// x * rsqrt(mean x^2 + eps) * w into a GEMM operand (engine.metal:159-178, 1609-1640).
void rmsnorm_operand(const float *x, int stride, const std::vector<uint16_t> &w, int rows, int dim, float eps, Operand &out) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const float *v = x + size_t(r) * stride;
        double ss = 0;
        for (int i = 0; i < dim; ++i) ss += double(v[i]) * v[i];
        const float inv = 1.0f / sqrtf(float(ss / dim) + eps);
        for (int i = 0; i < dim; ++i) out.values[size_t(r) * dim + i] = round_bf16(v[i] * inv * bf16_to_float(w[i]));
        out.finish_row(r);
    }
}

// The deferred form of the same norm (Sources/Shaders/engine_na.metal:365-415, Sources/SploshRuntime/Engine.swift:1439-1451):
// the residual GEMM that produced x emits bf16(x * w) with its per-64 sums and the squares of x; the GEMMs that read the
// operand multiply their sums by inv[r] = rsqrt(mean x^2 + eps). The rounding point moves from x * inv * w to x * w.
void rmsnorm_operand_deferred(const float *x, int stride, const std::vector<uint16_t> &w, int rows, int dim, float eps, Operand &out, std::vector<float> &inv) {
    inv.assign(rows, 1.0f);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const float *v = x + size_t(r) * stride;
        double ss = 0;
        for (int i = 0; i < dim; ++i) ss += double(v[i]) * v[i];
        inv[r] = 1.0f / sqrtf(float(ss / dim) + eps);
        for (int i = 0; i < dim; ++i) out.values[size_t(r) * dim + i] = round_bf16(v[i] * bf16_to_float(w[i]));
        out.finish_row(r);
    }
}

float rope(float x, float paired, int i, int rotary, uint32_t position, float theta) {
    // Sources/Shaders/engine_na.metal:1214-1219 (NeoX pairing over the first `rotary` dims).
    // The inverse frequency is formed in double and rounded to fp32 once (the reference forms it
    // with a single-precision pow per element); the angle is one fp32 multiply.
    const int half = rotary / 2, slot = i < half ? i : i - half;
    const float inv_freq = float(pow(double(theta), -2.0 * double(slot) / double(rotary)));
    const float angle = float(position) * inv_freq;
    return x * cosf(angle) + (i < half ? -paired : paired) * sinf(angle);
}

// Per-head RMSNorm then RoPE of one head vector (engine_na.metal:1236-1262, 2055-2081).
void norm_rope(const float *x, const std::vector<uint16_t> &w, int dim, int rotary, uint32_t position, float eps, float theta, float *out) {
    double ss = 0;
    for (int i = 0; i < dim; ++i) ss += double(x[i]) * x[i];
    const float inv = 1.0f / sqrtf(float(ss / dim) + eps);
    const int half = rotary / 2;
    for (int i = 0; i < dim; ++i) {
        float v = x[i] * inv * bf16_to_float(w[i]);
        if (i < rotary) {
            const int pi = i < half ? i + half : i - half;
            v = rope(v, x[pi] * inv * bf16_to_float(w[pi]), i, rotary, position, theta);
        }
        out[i] = v;
    }
}

// The rank-1 update written once so that replay from the journal reproduces it
// (engine.metal:654-659): S' = fma(S, decay, k * delta).
inline float gdn_update(float s, float decay, float k, float delta) {
    volatile float product = k * delta;     // rounded on its own, never contracted into the fma
    return fmaf(s, decay, product);
}

// One gated-delta layer over the step's runs: engine.metal:668-851 (sp_gdn_fast), with the CPU
// statement of the same semantics in Tests/SploshOracleTests/GdnCandidateTests.swift:403-537.
void gdn_layer(Engine &e, int linear_index, const Layer &L, const Tables &t, const float *mixed, const float *z,
               const float *a, const float *b, Operand &core) {
    const Geometry &g = e.m->g;
    const int d = g.gdn_head_dim, VH = g.gdn_value_heads, KH = g.gdn_key_heads, C = g.channels();
    const int rows = t.rows, per = VH / KH;
    std::vector<float> &state = e.state[linear_index], &conv = e.conv[linear_index], &journal = e.journal[linear_index];
    const std::vector<float> history = conv;      // rows read the history as it was before the step

    // Conv + SiLU for every channel of every row.
    std::vector<float> act(size_t(rows) * C);
    auto input = [&](uint32_t run, int tt, int channel) -> float {
        const uint32_t start = t.runs[run * 3 + 1];
        if (tt >= 0) return mixed[size_t(start + tt) * C + channel];
        return history[(size_t(t.row_read[start]) * C + channel) * 3 + 3 + tt];
    };
    for (uint32_t run = 0; run < t.run_count; ++run) {
        const int start = t.runs[run * 3 + 1], length = t.runs[run * 3 + 2];
#pragma omp parallel for schedule(static)
        for (int c = 0; c < C; ++c) {
            float w[4];
            for (int k = 0; k < 4; ++k) w[k] = bf16_to_float(L.vec[V_CONV][c * 4 + k]);
            for (int tt = 0; tt < length; ++tt) {
                float sum = 0;
                for (int tap = 0; tap < 4; ++tap) sum += w[tap] * input(run, tt - 3 + tap, c);
                act[size_t(start + tt) * C + c] = silu(sum);
            }
        }
    }
    // Decay, beta and the L2 norms.
    std::vector<float> decay(size_t(rows) * VH), beta(size_t(rows) * VH), inv_q(size_t(rows) * KH), inv_k(size_t(rows) * KH);
    for (int r = 0; r < rows; ++r) {
        for (int h = 0; h < VH; ++h) {
            const float x = a[size_t(r) * VH + h] + bf16_to_float(L.vec[V_DT_BIAS][h]);
            const float softplus = x > 20.0f ? x : logf(1.0f + expf(x));
            decay[size_t(r) * VH + h] = expf(-expf(bf16_to_float(L.vec[V_A_LOG][h])) * softplus);
            beta[size_t(r) * VH + h] = sigmoidf(b[size_t(r) * VH + h]);
        }
        for (int hk = 0; hk < KH; ++hk) {
            double qq = 0, kk = 0;
            const float *q = &act[size_t(r) * C + hk * d], *k = &act[size_t(r) * C + KH * d + hk * d];
            for (int i = 0; i < d; ++i) { qq += double(q[i]) * q[i]; kk += double(k[i]) * k[i]; }
            inv_q[size_t(r) * KH + hk] = (1.0f / sqrtf(float(qq) + 1e-6f)) * (1.0f / sqrtf(float(d)));
            inv_k[size_t(r) * KH + hk] = 1.0f / sqrtf(float(kk) + 1e-6f);
        }
    }
    // The recurrence, one (run, head) at a time.
    std::vector<float> raw(size_t(rows) * VH * d);
    const int pairs = int(t.run_count) * VH;
#pragma omp parallel for schedule(dynamic)
    for (int pair = 0; pair < pairs; ++pair) {
        const int run = pair / VH, h = pair % VH, hk = h / per;
        const uint32_t slot = t.runs[run * 3], start = t.runs[run * 3 + 1], length = t.runs[run * 3 + 2];
        const bool speculative = t.run_info[run * 2] != 0;
        const uint32_t pending = t.run_info[run * 2 + 1];
        float *stored = &state[(size_t(slot) * VH + h) * d * d];
        std::vector<float> s(stored, stored + size_t(d) * d);
        float *jhead = &journal[(size_t(slot) * kJournalRows * VH + h) * kJournalWidth];
        for (uint32_t en = 0; en < pending; ++en) {
            const float *entry = jhead + size_t(en) * VH * kJournalWidth;
            const float dk = entry[2 * d];
            for (int j = 0; j < d; ++j)
                for (int i = 0; i < d; ++i) s[j * d + i] = gdn_update(s[j * d + i], dk, entry[i], entry[d + j]);
        }
        if (speculative && pending != 0) memcpy(stored, s.data(), sizeof(float) * d * d);
        std::vector<float> delta(d);
        for (uint32_t tt = 0; tt < length; ++tt) {
            const uint32_t row = start + tt;
            const float *q = &act[size_t(row) * C + hk * d], *k = &act[size_t(row) * C + KH * d + hk * d];
            const float *v = &act[size_t(row) * C + 2 * KH * d + h * d];
            const float iq = inv_q[size_t(row) * KH + hk], ik = inv_k[size_t(row) * KH + hk];
            const float dk = decay[size_t(row) * VH + h], bt = beta[size_t(row) * VH + h];
            for (int j = 0; j < d; ++j) {
                double mem = 0;
                for (int i = 0; i < d; ++i) mem += double(s[j * d + i]) * k[i];
                delta[j] = (v[j] - float(mem) * dk * ik) * bt * ik;
            }
            for (int j = 0; j < d; ++j) {
                double o = 0;
                for (int i = 0; i < d; ++i) {
                    s[j * d + i] = gdn_update(s[j * d + i], dk, k[i], delta[j]);
                    o += double(s[j * d + i]) * q[i];
                }
                raw[(size_t(row) * VH + h) * d + j] = float(o) * iq;
            }
            if (speculative) {
                float *entry = jhead + size_t(tt) * VH * kJournalWidth;
                for (int i = 0; i < d; ++i) { entry[i] = k[i]; entry[d + i] = delta[i]; }
                entry[2 * d] = dk;
            } else if (tt + 1 == length) {
                memcpy(stored, s.data(), sizeof(float) * d * d);
            }
        }
    }
    // Gated RMSNorm into the out-projection's operand (engine.metal:812-833).
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        for (int h = 0; h < VH; ++h) {
            const float *o = &raw[(size_t(r) * VH + h) * d];
            double ss = 0;
            for (int j = 0; j < d; ++j) ss += double(o[j]) * o[j];
            const float inv = 1.0f / sqrtf(float(ss / d) + g.eps);
            for (int j = 0; j < d; ++j) {
                const float gate = z[(size_t(r) * VH + h) * d + j];
                const float result = bf16_to_float(L.vec[V_GDN_NORM][j]) * o[j] * inv * gate / (1.0f + expf(-gate));
                const int place = e.m->out_file_order ? KH * (h % per) + h / per : h;
                core.values[(size_t(r) * VH + place) * d + j] = round_bf16(result);
            }
        }
        core.finish_row(r);
    }
    // Conv history for every unit a row writes: the last three raw inputs up to that row
    // (engine.metal:838-849).
    for (uint32_t run = 0; run < t.run_count; ++run) {
        const int start = t.runs[run * 3 + 1], length = t.runs[run * 3 + 2];
        for (int tt = 0; tt < length; ++tt) {
            const int row = start + tt;
            if (tt + 1 != length && t.row_write[row + 1] == t.row_write[row]) continue;
            for (int c = 0; c < C; ++c)
                for (int back = 0; back < 3; ++back)
                    conv[(size_t(t.row_write[row]) * C + c) * 3 + 2 - back] = input(run, tt - back, c);
        }
    }
}

void attention_scan(Engine &e, int full_index, const Tables &t, int live, const float *q, const float *qproj, float *partials_out, Operand &core);

// One gated GQA layer: q prepare (engine_na.metal:1222-1266), int8 KV store (:2044-2094), the
// span scan (candidates/attn_scan_r.metal:46-202), the merge (engine.metal:2218-2255). The CPU
// statement of the scan and merge is Tests/SploshOracleTests/AttentionScanCandidateTests.swift:313-420.
void attention_layer(Engine &e, int full_index, const Layer &L, const Tables &t, int live, const float *qproj,
                     const float *kproj, const float *vproj, Operand &core) {
    const Geometry &g = e.m->g;
    const int hd = g.head_dim, heads = g.heads, kvh = g.kv_heads, rows = t.rows;
    std::vector<int8_t> &kc = e.k_codes[full_index], &vc = e.v_codes[full_index];
    std::vector<float> &ks = e.k_scale[full_index], &vs = e.v_scale[full_index];
    // Keys and values of every row of the step go in first, so rows of a block see each other.
    for (int r = 0; r < rows; ++r) {
        const uint32_t position = t.row_pos[r];
        const uint32_t page = t.page_table[size_t(t.row_slot[r]) * e.max_pages + position / kPageTokens];
        for (int h = 0; h < kvh; ++h) {
            std::vector<float> kv(hd);
            norm_rope(kproj + (size_t(r) * kvh + h) * hd, L.vec[V_K_NORM], hd, g.rotary_dim, position, g.eps, g.rope_theta, kv.data());
            const float *vv = vproj + (size_t(r) * kvh + h) * hd;
            float khi = 0, vhi = 0;
            for (int i = 0; i < hd; ++i) { khi = std::max(khi, fabsf(kv[i])); vhi = std::max(vhi, fabsf(vv[i])); }
            const float kS = khi > 0 ? khi / 127.0f : 1.0f, vS = vhi > 0 ? vhi / 127.0f : 1.0f;
            const size_t token = (size_t(page) * kvh + h) * kPageTokens + position % kPageTokens;
            for (int i = 0; i < hd; ++i) {
                kc[token * hd + i] = int8_t(std::min(127.0f, std::max(-127.0f, rintf(kv[i] / kS))));
                vc[token * hd + i] = int8_t(std::min(127.0f, std::max(-127.0f, rintf(vv[i] / vS))));
            }
            ks[token] = kS; vs[token] = vS;
        }
    }
    if (live <= 0) return;
    // Queries: norm, RoPE, fp16.
    std::vector<float> q(size_t(live) * heads * hd);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < live; ++r)
        for (int h = 0; h < heads; ++h) {
            float *out = &q[(size_t(r) * heads + h) * hd];
            norm_rope(qproj + (size_t(r) * heads + h) * 2 * hd, L.vec[V_Q_NORM], hd, g.rotary_dim, t.row_pos[r], g.eps, g.rope_theta, out);
            for (int i = 0; i < hd; ++i) out[i] = round_f16(out[i]);
        }
    attention_scan(e, full_index, t, live, q.data(), qproj, nullptr, core);
}

// The span scan and the merge on their own, over the pool as it stands: q [live][heads][head_dim] holds the prepared
// (fp16-representable) queries, qproj [rows][heads][2 head_dim] the projection whose second halves are the output gates.
// `partials_out`, when given, receives the span records [live][heads][spans][head_dim + 2].
void attention_scan(Engine &e, int full_index, const Tables &t, int live, const float *q, const float *qproj, float *partials_out, Operand &core) {
    const Geometry &g = e.m->g;
    const int hd = g.head_dim, heads = g.heads, kvh = g.kv_heads, perKV = heads / kvh;
    std::vector<int8_t> &kc = e.k_codes[full_index], &vc = e.v_codes[full_index];
    std::vector<float> &ks = e.k_scale[full_index], &vs = e.v_scale[full_index];
    const float scale = 1.0f / sqrtf(float(hd));
    const int spans = t.spans, pps = t.pages_per_span;
    const int record = hd + 2;
    std::vector<float> partials(size_t(live) * heads * spans * record, 0.0f);
    for (size_t i = 0; i < partials.size(); i += record) partials[i] = -INFINITY;
    // Blocks in row order; only those that hold computed rows.
    int blocks = 0;
    for (; blocks < int(t.attn_block_count); ++blocks) if (int(t.attn_blocks[blocks * 2]) >= live) break;
    const int jobs = blocks * kvh * spans;
#pragma omp parallel for schedule(dynamic)
    for (int job = 0; job < jobs; ++job) {
        const int block = job / (kvh * spans), kvHead = (job / spans) % kvh, span = job % spans;
        const uint32_t r0 = t.attn_blocks[block * 2], count = t.attn_blocks[block * 2 + 1];
        const uint32_t firstPos = t.row_pos[r0], maxVisible = firstPos + count;
        const int pages = int((maxVisible + kPageTokens - 1) / kPageTokens);
        const int firstPage = span * pps, lastPage = std::min(pages, firstPage + pps);
        const size_t tableBase = size_t(t.row_slot[r0]) * e.max_pages;
        std::vector<float> acc(hd), s(64), p(64);
        for (uint32_t rb = 0; rb < count; ++rb) {
            const uint32_t row = r0 + rb;
            if (int(row) >= live) continue;
            const uint32_t limit = firstPos + rb + 1;
            for (int hq = 0; hq < perKV; ++hq) {
                const int head = kvHead * perKV + hq;
                const float *qv = &q[(size_t(row) * heads + head) * hd];
                float reference = -INFINITY, total = 0;
                std::fill(acc.begin(), acc.end(), 0.0f);
                for (int pg = firstPage; pg < lastPage; ++pg) {
                    const size_t pageTokens = (size_t(t.page_table[tableBase + pg]) * kvh + kvHead) * kPageTokens;
                    for (int chunk = 0; chunk < kPageTokens / 64; ++chunk) {
                        const uint32_t t0 = pg * kPageTokens + chunk * 64;
                        if (t0 >= maxVisible) break;
                        const size_t tokenBase = pageTokens + chunk * 64;
                        float top = -INFINITY;
                        for (int c = 0; c < 64; ++c) {
                            if (t0 + c < limit) {
                                const int8_t *kk = &kc[(tokenBase + c) * hd];
                                float dot = 0;
                                for (int i = 0; i < hd; ++i) dot += qv[i] * float(kk[i]);
                                s[c] = dot * ks[tokenBase + c] * scale;
                                top = std::max(top, s[c]);
                            } else s[c] = -INFINITY;
                        }
                        // The reference of the exponentials moves only when passed by more than 30
                        // (attn_scan_r.metal:41,150).
                        const float next = top > reference + 30.0f ? top : reference;
                        float sum = 0;
                        for (int c = 0; c < 64; ++c) {
                            const bool seen = t0 + c < limit;
                            const float prob = seen ? expf(s[c] - next) : 0.0f;
                            sum += prob;
                            p[c] = seen ? round_bf16(prob * vs[tokenBase + c]) : 0.0f;
                        }
                        const float factor = (next == reference || reference == -INFINITY) ? 1.0f : expf(reference - next);
                        total = total * factor + sum;
                        reference = next;
                        for (int i = 0; i < hd; ++i) acc[i] *= factor;
                        for (int c = 0; c < 64; ++c) {
                            if (p[c] == 0.0f) continue;
                            const int8_t *vv = &vc[(tokenBase + c) * hd];
                            for (int i = 0; i < hd; ++i) acc[i] += p[c] * float(vv[i]);
                        }
                    }
                }
                float *partial = &partials[((size_t(row) * heads + head) * spans + span) * record];
                partial[0] = reference; partial[1] = total;
                memcpy(partial + 2, acc.data(), sizeof(float) * hd);
            }
        }
    }
    // Merge spans, gate, operand.
#pragma omp parallel for schedule(static)
    for (int r = 0; r < live; ++r) {
        for (int h = 0; h < heads; ++h) {
            const float *base = &partials[(size_t(r) * heads + h) * spans * record];
            float top = -INFINITY;
            for (int sp = 0; sp < spans; ++sp) top = std::max(top, base[sp * record]);
            for (int j = 0; j < hd; ++j) {
                float sum = 0, acc = 0;
                for (int sp = 0; sp < spans; ++sp) {
                    const float weight = expf(base[sp * record] - top);
                    if (weight > 0.0f) { sum += base[sp * record + 1] * weight; acc += base[sp * record + 2 + j] * weight; }
                }
                const float gate = qproj[(size_t(r) * heads + h) * 2 * hd + hd + j];
                core.values[(size_t(r) * heads + h) * hd + j] = round_bf16((acc / sum) * sigmoidf(gate));
            }
        }
        core.finish_row(r);
    }
    if (partials_out) memcpy(partials_out, partials.data(), partials.size() * sizeof(float));
}

}  // namespace

// ==========================================================================================
// C interface (ctypes)

extern "C" {

uint64_t orc_splitmix_at(uint64_t seed, uint64_t n) { return splitmix_at(seed, n); }
float orc_uniform_at(uint64_t seed, uint64_t n) { return uniform_at(seed, n); }
float orc_normal_at(uint64_t seed, uint64_t n, float deviation) { return normal_at(seed, n, deviation); }
uint64_t orc_fnv1a64(const char *s) { return fnv1a64(s); }
uint16_t orc_bf16(float v) { return float_to_bf16(v); }
float orc_f16_round(float v) { return round_f16(v); }
// 0: exact codes with per-group scale and bias (default); 1: weights rounded to bf16 once.
void orc_set_weight_contract(int contract) { g_weight_contract = contract; }
void orc_set_norm_contract(int contract) { g_norm_contract = contract; }
int orc_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// Quantise fp32 [rows][inner] to MLX affine-4 group 64 (DraftModel.swift:634-670, "minmax").
void orc_quantize_mlx4(const float *w, int rows, int inner, uint32_t *packed, uint16_t *scales, uint16_t *biases) {
    const int groups = inner / 64;
    for (int64_t r = 0; r < rows; ++r)
        for (int g = 0; g < groups; ++g) {
            const size_t slot = size_t(r) * groups + g;
            quantize_group(w + size_t(r) * inner + g * 64, packed + slot * 8, scales + slot, biases + slot);
        }
}

// value = scales[group] * nibble + biases[group] (MlxAffine.swift:72-84). `columns` need not be a
// multiple of 8 or 64: rows are ceil(columns / 8) words and ceil(columns / 64) groups.
void orc_dequant_mlx4(const uint32_t *packed, const float *scales, const float *biases, int rows, int columns, float *out) {
    const int words = (columns + 7) / 8, groups = (columns + 63) / 64;
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < columns; ++c) {
            const uint32_t nib = (packed[size_t(r) * words + c / 8] >> (4 * (c % 8))) & 0xF;
            out[size_t(r) * columns + c] = scales[size_t(r) * groups + c / 64] * float(nib) + biases[size_t(r) * groups + c / 64];
        }
}

static float half_at(const uint8_t *b, int at) { uint16_t bits; memcpy(&bits, b + at, 2); _Float16 h; memcpy(&h, &bits, 2); return float(h); }

// Q4_K (144 bytes) and Q5_K (176 bytes) super-blocks of 256 (Sources/SploshModel/GgufQuant.swift:191-211).
void orc_decode_q45k(const uint8_t *data, int blocks, int fifth_bit, float *out) {
    const int bytes = fifth_bit ? 176 : 144, codes = fifth_bit ? 48 : 16;
    for (int n = 0; n < blocks; ++n) {
        const uint8_t *b = data + size_t(n) * bytes;
        const float d = half_at(b, 0), dmin = half_at(b, 2);
        for (int j = 0; j < 8; ++j) {
            uint8_t scale, minimum;
            if (j < 4) { scale = b[4 + j] & 63; minimum = b[4 + j + 4] & 63; }
            else { scale = (b[4 + j + 4] & 0xF) | ((b[4 + j - 4] >> 6) << 4); minimum = (b[4 + j + 4] >> 4) | ((b[4 + j] >> 6) << 4); }
            const float scaled = d * float(scale), offset = dmin * float(minimum);
            for (int e = 0; e < 32; ++e) {
                const uint8_t byte = b[codes + 32 * (j / 2) + e];
                float code = float(j % 2 == 0 ? byte & 15 : byte >> 4);
                if (fifth_bit) code += 16.0f * float((b[16 + e] >> j) & 1);
                out[size_t(n) * 256 + 32 * j + e] = code * scaled - offset;
            }
        }
    }
}

// Q6_K (210 bytes) super-blocks of 256 (GgufQuant.swift:217-230).
void orc_decode_q6k(const uint8_t *data, int blocks, float *out) {
    for (int n = 0; n < blocks; ++n) {
        const uint8_t *b = data + size_t(n) * 210;
        const float d = half_at(b, 208);
        for (int j = 0; j < 8; ++j) {
            const int half = j / 4, quarter = j % 4;
            for (int e = 0; e < 32; ++e) {
                const int low = (b[64 * half + 32 * (quarter & 1) + e] >> (4 * (quarter >> 1))) & 15;
                const int high = (b[128 + 32 * half + e] >> (2 * quarter)) & 3;
                const float code = float(low | (high << 4)) - 32.0f;
                const float scale = float(int8_t(b[192 + 2 * j + e / 16]));
                out[size_t(n) * 256 + 32 * j + e] = d * scale * code;
            }
        }
    }
}

// The GGUF GEMM's weights as its tile kernels form them (Sources/Shaders/gguf_formats.h:390-438): one fp32
// multiply-add (Q4_K, Q5_K: fma(code, d * scale, -dmin * minimum)) or multiply (Q6_K: (code - 32) * (d * scale)),
// rounded once to fp16. format: 12 = Q4_K, 13 = Q5_K, 14 = Q6_K (the GGUF type numbers).
static float round_half(float v) { _Float16 h = _Float16(v); return float(h); }
void orc_gguf_tile_weights(int format, const uint8_t *data, int blocks, float *out) {
    for (int n = 0; n < blocks; ++n) {
        if (format == 14) {
            const uint8_t *b = data + size_t(n) * 210;
            const float d = half_at(b, 208);
            for (int j = 0; j < 8; ++j) {
                const int half = j / 4, quarter = j % 4;
                for (int e = 0; e < 32; ++e) {
                    const int low = (b[64 * half + 32 * (quarter & 1) + e] >> (4 * (quarter >> 1))) & 15;
                    const int high = (b[128 + 32 * half + e] >> (2 * quarter)) & 3;
                    const float code = float((low | (high << 4)) - 32);
                    const float s = d * float(int8_t(b[192 + 2 * j + e / 16]));
                    out[size_t(n) * 256 + 32 * j + e] = round_half(code * s);
                }
            }
        } else {
            const bool fifth = format == 13;
            const uint8_t *b = data + size_t(n) * (fifth ? 176 : 144);
            const int codes = fifth ? 48 : 16;
            const float d = half_at(b, 0), dmin = half_at(b, 2);
            for (int j = 0; j < 8; ++j) {
                uint8_t scale, minimum;
                if (j < 4) { scale = b[4 + j] & 63; minimum = b[4 + j + 4] & 63; }
                else { scale = (b[4 + j + 4] & 0xF) | ((b[4 + j - 4] >> 6) << 4); minimum = (b[4 + j + 4] >> 4) | ((b[4 + j] >> 6) << 4); }
                const float s = d * float(scale), m = -dmin * float(minimum);
                for (int e = 0; e < 32; ++e) {
                    const uint8_t byte = b[codes + 32 * (j / 2) + e];
                    int code = j % 2 == 0 ? byte & 15 : byte >> 4;
                    if (fifth) code += 16 * ((b[16 + e] >> j) & 1);
                    out[size_t(n) * 256 + 32 * j + e] = round_half(fmaf(float(code), s, m));
                }
            }
        }
    }
}

// GGUF GEMM (Sources/Shaders/engine_gguf.metal:82-273): out[r][n] = sum_k bf16(a[r][k]) * w16[n][k] (+ residual), fp32 sums;
// data: row-major native blocks [n][k / 256].
void orc_gemm_gguf(int format, const uint8_t *data, int n, int k, const float *a, int rows, const float *residual, float *out) {
    const int per_row = k / 256, bytes = format == 14 ? 210 : format == 13 ? 176 : 144;
    std::vector<float> rounded(size_t(rows) * k);
    for (size_t i = 0; i < rounded.size(); ++i) rounded[i] = round_bf16(a[i]);
#pragma omp parallel for schedule(static)
    for (int col = 0; col < n; ++col) {
        std::vector<float> w(k);
        orc_gguf_tile_weights(format, data + size_t(col) * per_row * bytes, per_row, w.data());
        for (int r = 0; r < rows; ++r) {
            float acc = 0.0f;
            const float *x = rounded.data() + size_t(r) * k;
            for (int i = 0; i < k; ++i) acc += x[i] * w[i];
            out[size_t(r) * n + col] = acc + (residual ? residual[size_t(r) * n + col] : 0.0f);
        }
    }
}

// One fp32 gated-delta update, state [head][key][value] and log-space decay: the per-op oracle of
// Sources/SploshOracle/GdnOracle.swift:44-64, kept to pin against Tests/SploshOracleTests/GdnOracleTests.swift.
void orc_gdn_decode(const float *query, const float *key, const float *value, const float *beta, const float *log_decay,
                    int heads, int key_dim, int value_dim, float *state, float *output) {
    for (int h = 0; h < heads; ++h) {
        float *s = state + size_t(h) * key_dim * value_dim;
        const float *q = query + h * key_dim, *k = key + h * key_dim, *v = value + h * value_dim;
        const float d = expf(log_decay[h]);
        for (int i = 0; i < key_dim * value_dim; ++i) s[i] *= d;
        std::vector<float> predicted(value_dim, 0.0f);
        for (int i = 0; i < key_dim; ++i) for (int j = 0; j < value_dim; ++j) predicted[j] += s[i * value_dim + j] * k[i];
        for (int j = 0; j < value_dim; ++j) {
            const float delta = beta[h] * (v[j] - predicted[j]);
            for (int i = 0; i < key_dim; ++i) s[i * value_dim + j] += k[i] * delta;
        }
        for (int j = 0; j < value_dim; ++j) {
            float o = 0;
            for (int i = 0; i < key_dim; ++i) o += s[i * value_dim + j] * q[i];
            output[h * value_dim + j] = o;
        }
    }
}

// The engine's form of the same update on one head: raw k with its inverse norm folded in, state
// [value j][key i] (engine.metal:774-786). Used to check the two statements against each other.
void orc_gdn_engine_update(const float *q, const float *k, const float *v, float beta, float decay, float inv_q, float inv_k,
                           int d, float *state, float *output) {
    std::vector<float> delta(d);
    for (int j = 0; j < d; ++j) {
        double mem = 0;
        for (int i = 0; i < d; ++i) mem += double(state[j * d + i]) * k[i];
        delta[j] = (v[j] - float(mem) * decay * inv_k) * beta * inv_k;
    }
    for (int j = 0; j < d; ++j) {
        double o = 0;
        for (int i = 0; i < d; ++i) { state[j * d + i] = gdn_update(state[j * d + i], decay, k[i], delta[j]); o += double(state[j * d + i]) * q[i]; }
        output[j] = float(o) * inv_q;
    }
}

// RoPE of one head at one position (Sources/SploshOracle/RopeOracle.swift:15-56 for text: all
// three position ids equal).
void orc_rope(const float *input, int head_dim, int rotary, float theta, uint32_t position, float *out) {
    const int half = rotary / 2;
    for (int i = 0; i < head_dim; ++i) {
        if (i < rotary) out[i] = rope(input[i], input[i < half ? i + half : i - half], i, rotary, position, theta);
        else out[i] = input[i];
    }
}

// bf16 in, bf16 out: silu(gate) * up (Sources/SploshOracle/SwigluOracle.swift:14-29).
void orc_swiglu_bf16(const uint16_t *gate, const uint16_t *up, int count, uint16_t *out) {
    for (int i = 0; i < count; ++i) out[i] = float_to_bf16(silu(bf16_to_float(gate[i])) * bf16_to_float(up[i]));
}

// First index of the maximum over [0, limit) (vDSP_maxvi, Sources/SploshRuntime/Sampler.swift:11-16,94-96).
int32_t orc_argmax(const float *logits, int limit) {
    int best = 0;
    for (int i = 1; i < limit; ++i) if (logits[i] > logits[best]) best = i;
    return best;
}

// ---- model

void *orc_model_create(const Geometry *g, uint64_t seed) {
    Model *m = new Model;
    m->g = *g; m->seed = seed;
    m->layers.resize(g->layers);
    for (int l = 0; l < g->layers; ++l) {
        Layer &L = m->layers[l];
        L.full = g->full(l);
        for (int kind = 0; kind < 12; ++kind) {
            const bool linear_kind = kind <= Q_OUT, full_kind = kind >= Q_Q && kind <= Q_O;
            if ((linear_kind && L.full) || (full_kind && !L.full)) continue;
            int rows, inner; q4_shape(*g, kind, &rows, &inner);
            synth_q4(L.q4[kind], rows, inner, tensor_seed(seed, l, q4_names[kind]), 0.02f);
        }
        synth_vec(L.vec[V_IN_NORM], g->hidden, tensor_seed(seed, l, vec_names[V_IN_NORM]), 0, 1.0f, 0.02f);
        synth_vec(L.vec[V_POST_NORM], g->hidden, tensor_seed(seed, l, vec_names[V_POST_NORM]), 0, 1.0f, 0.02f);
        if (L.full) {
            synth_vec(L.vec[V_Q_NORM], g->head_dim, tensor_seed(seed, l, vec_names[V_Q_NORM]), 0, 1.0f, 0.02f);
            synth_vec(L.vec[V_K_NORM], g->head_dim, tensor_seed(seed, l, vec_names[V_K_NORM]), 0, 1.0f, 0.02f);
        } else {
            // Ranges of Tests/SploshOracleTests/GdnCandidateTests.swift:141-145.
            synth_vec(L.vec[V_CONV], g->channels() * 4, tensor_seed(seed, l, vec_names[V_CONV]), 1, -0.6f, 0.6f);
            synth_vec(L.vec[V_A_LOG], g->gdn_value_heads, tensor_seed(seed, l, vec_names[V_A_LOG]), 1, -2.0f, 1.0f);
            synth_vec(L.vec[V_DT_BIAS], g->gdn_value_heads, tensor_seed(seed, l, vec_names[V_DT_BIAS]), 1, -1.0f, 1.0f);
            synth_vec(L.vec[V_GDN_NORM], g->gdn_head_dim, tensor_seed(seed, l, vec_names[V_GDN_NORM]), 0, 1.0f, 0.02f);
        }
    }
    synth_q4(m->embed, g->vocab, g->hidden, tensor_seed(seed, -1, q4_names[Q_EMBED]), 0.02f);
    synth_q4(m->head, g->vocab, g->hidden, tensor_seed(seed, -1, q4_names[Q_HEAD]), 0.02f);
    synth_vec(m->final_norm, g->hidden, tensor_seed(seed, -1, vec_names[V_FINAL_NORM]), 0, 1.0f, 0.02f);
    return m;
}
void orc_model_destroy(void *model) { delete static_cast<Model *>(model); }

// The stream seed of a tensor, for a generator elsewhere that must reproduce it.
uint64_t orc_tensor_seed(uint64_t base, int layer, int is_vec, int kind) {
    return tensor_seed(base, layer, is_vec ? vec_names[kind] : q4_names[kind]);
}

int orc_model_q4(void *model, int layer, int kind, int *rows, int *inner, const uint32_t **packed, const uint16_t **scales, const uint16_t **biases) {
    Model *m = static_cast<Model *>(model);
    const Q4 *t = kind == Q_EMBED ? &m->embed : kind == Q_HEAD ? &m->head : &m->layers[layer].q4[kind];
    if (t->rows == 0) return 1;
    *rows = t->rows; *inner = t->inner; *packed = t->packed.data(); *scales = t->scales.data(); *biases = t->biases.data();
    return 0;
}
// One tensor of the model as native GGUF blocks [rows][inner / 256] of `format` (12, 13, 14): the GEMMs and the embedding
// gather use them from then on. The tensor keeps its shape.
int orc_model_set_gguf(void *model, int layer, int kind, int format, const uint8_t *data) {
    Model *m = static_cast<Model *>(model);
    Q4 *t = kind == Q_EMBED ? &m->embed : kind == Q_HEAD ? &m->head : &m->layers[layer].q4[kind];
    if (t->rows == 0 || t->inner % 256 || (format != 12 && format != 13 && format != 14)) return 1;
    const size_t bytes = size_t(t->rows) * (t->inner / 256) * (format == 14 ? 210 : format == 13 ? 176 : 144);
    t->gguf.assign(data, data + bytes);
    t->gguf_format = format;
    return 0;
}
void orc_model_set_out_file_order(void *model, int enabled) { static_cast<Model *>(model)->out_file_order = enabled != 0; }
int orc_model_vec(void *model, int layer, int kind, const uint16_t **data, int *count) {
    Model *m = static_cast<Model *>(model);
    const std::vector<uint16_t> *v = kind == V_FINAL_NORM ? &m->final_norm : &m->layers[layer].vec[kind];
    if (v->empty()) return 1;
    *data = v->data(); *count = int(v->size());
    return 0;
}

// ---- engine

void *orc_engine_create(void *model, int max_slots, int kv_pages, int max_pages, int state_units) {
    Model *m = static_cast<Model *>(model);
    const Geometry &g = m->g;
    Engine *e = new Engine;
    e->m = m; e->max_slots = max_slots; e->kv_pages = kv_pages; e->max_pages = max_pages; e->state_units = state_units;
    const float nan = std::numeric_limits<float>::quiet_NaN();
    for (int l = 0; l < g.layers; ++l) {
        if (g.full(l)) {
            const size_t tokens = size_t(kv_pages) * g.kv_heads * kPageTokens;
            e->k_codes.emplace_back(tokens * g.head_dim, int8_t(-1));
            e->v_codes.emplace_back(tokens * g.head_dim, int8_t(-1));
            // A scale nobody stored is NaN, so a masked token that leaks shows
            // (Tests/SploshOracleTests/AttentionScanCandidateTests.swift:85-200).
            e->k_scale.emplace_back(tokens, nan);
            e->v_scale.emplace_back(tokens, nan);
        } else {
            const int d = g.gdn_head_dim;
            e->state.emplace_back(size_t(max_slots) * g.gdn_value_heads * d * d, 0.0f);
            e->conv.emplace_back(size_t(state_units) * g.channels() * 3, 0.0f);
            e->journal.emplace_back(size_t(max_slots) * kJournalRows * g.gdn_value_heads * kJournalWidth, 0.0f);
        }
    }
    return e;
}
void orc_engine_destroy(void *engine) { delete static_cast<Engine *>(engine); }

// Zero a slot's recurrent state and the conv history of its unit (Engine.swift:816-826).
void orc_engine_reset_slot(void *engine, int slot, int unit) {
    Engine *e = static_cast<Engine *>(engine);
    const Geometry &g = e->m->g;
    const size_t per_state = size_t(g.gdn_value_heads) * g.gdn_head_dim * g.gdn_head_dim, per_conv = size_t(g.channels()) * 3;
    for (size_t l = 0; l < e->state.size(); ++l) {
        std::fill_n(e->state[l].begin() + slot * per_state, per_state, 0.0f);
        std::fill_n(e->conv[l].begin() + unit * per_conv, per_conv, 0.0f);
    }
}

// Raw views for comparisons. which: 0 state, 1 conv, 2 journal (linear layer index); 3 k codes,
// 4 v codes, 5 k scale, 6 v scale (full layer index).
void *orc_engine_buffer(void *engine, int which, int index, size_t *bytes) {
    Engine *e = static_cast<Engine *>(engine);
    switch (which) {
    case 0: *bytes = e->state[index].size() * 4; return e->state[index].data();
    case 1: *bytes = e->conv[index].size() * 4; return e->conv[index].data();
    case 2: *bytes = e->journal[index].size() * 4; return e->journal[index].data();
    case 3: *bytes = e->k_codes[index].size(); return e->k_codes[index].data();
    case 4: *bytes = e->v_codes[index].size(); return e->v_codes[index].data();
    case 5: *bytes = e->k_scale[index].size() * 4; return e->k_scale[index].data();
    case 6: *bytes = e->v_scale[index].size() * 4; return e->v_scale[index].data();
    }
    *bytes = 0; return nullptr;
}

// The attention scan and merge of one layer over the engine's pool as it stands (test entry): q [live][heads][head_dim]
// prepared queries, qproj [rows][heads][2 head_dim]; writes partials [live][heads][spans][head_dim + 2] and the merged,
// gated, bf16-rounded output [live][heads * head_dim].
int orc_attention_scan(void *engine, int full_index, const Tables *tp, int live, const float *q, const float *qproj, float *partials_out, float *core_out) {
    Engine &e = *static_cast<Engine *>(engine);
    if (full_index < 0 || full_index >= int(e.k_codes.size()) || live <= 0) return 1;
    const Geometry &g = e.m->g;
    Operand core(int(tp->rows), g.heads * g.head_dim);
    attention_scan(e, full_index, *tp, live, q, qproj, partials_out, core);
    memcpy(core_out, core.values.data(), size_t(live) * g.heads * g.head_dim * sizeof(float));
    return 0;
}


// One step (Engine.swift:1400-1512). logits: [logit_rows][vocab]. hidden_taps, when not null:
// [layers][rows][hidden], the residual stream after each block. max_layers < 0 runs all blocks.
int orc_step(void *engine, const Tables *tp, float *logits, float *hidden_taps, int max_layers) {
    Engine &e = *static_cast<Engine *>(engine);
    const Model &m = *e.m;
    const Geometry &g = m.g;
    const Tables &t = *tp;
    const int R = t.rows, H = g.hidden;
    std::vector<float> h(size_t(R) * H);
    // Embedding (engine.metal:39-57).
    for (int r = 0; r < R; ++r) {
        const uint32_t token = t.tokens[r];
        if (m.embed.gguf_format) {
            // The embedding gather decodes its row exactly (Sources/Shaders/gguf_formats.h:463-501).
            const int per_row = H / 256, bytes = m.embed.gguf_format == 14 ? 210 : m.embed.gguf_format == 13 ? 176 : 144;
            const uint8_t *src = m.embed.gguf.data() + size_t(token) * per_row * bytes;
            if (m.embed.gguf_format == 14) orc_decode_q6k(src, per_row, &h[size_t(r) * H]);
            else orc_decode_q45k(src, per_row, m.embed.gguf_format == 13, &h[size_t(r) * H]);
            continue;
        }
        for (int c = 0; c < H; ++c) {
            const uint32_t nib = (m.embed.packed[size_t(token) * H / 8 + c / 8] >> (4 * (c % 8))) & 0xF;
            h[size_t(r) * H + c] = bf16_to_float(m.embed.scales[size_t(token) * H / 64 + c / 64]) * float(nib)
                                 + bf16_to_float(m.embed.biases[size_t(token) * H / 64 + c / 64]);
        }
    }
    int linear_index = 0, full_index = 0;
    const int layers = max_layers < 0 ? g.layers : std::min(max_layers, g.layers);
    for (int l = 0; l < layers; ++l) {
        const Layer &L = m.layers[l];
        // Rows the last block is computed for (Engine.swift:1419-1429); keys and values are stored for all.
        const int live = (l + 1 == g.layers) ? int(t.live_rows) : R;
        Operand xn(R, H);
        // The first block's input comes from the embedding: a plain norm. Every later input norm reads what the previous
        // block's down projection left, and takes the deferred form.
        std::vector<float> inv_in;
        const bool deferred_in = g_norm_contract == 1 && l > 0;
        if (deferred_in) rmsnorm_operand_deferred(h.data(), H, L.vec[V_IN_NORM], R, H, g.eps, xn, inv_in);
        else rmsnorm_operand(h.data(), H, L.vec[V_IN_NORM], R, H, g.eps, xn);
        const float *scale_in = deferred_in ? inv_in.data() : nullptr;
        if (!L.full) {
            const int C = g.channels(), VD = g.value_dim(), VH = g.gdn_value_heads;
            std::vector<float> mixed(size_t(R) * C), z(size_t(R) * VD), a(size_t(R) * VH), b(size_t(R) * VH);
            gemm(L.q4[Q_QKV], xn, R, mixed.data(), C, nullptr, scale_in);
            gemm(L.q4[Q_Z], xn, R, z.data(), VD, nullptr, scale_in);
            gemm(L.q4[Q_A], xn, R, a.data(), VH, nullptr, scale_in);
            gemm(L.q4[Q_B], xn, R, b.data(), VH, nullptr, scale_in);
            Operand core(R, VD);
            gdn_layer(e, linear_index, L, t, mixed.data(), z.data(), a.data(), b.data(), core);
            if (live > 0) gemm(L.q4[Q_OUT], core, live, h.data(), H, h.data());
            ++linear_index;
        } else {
            const int AD = g.heads * g.head_dim, KV = g.kv_heads * g.head_dim;
            std::vector<float> qp(size_t(R) * 2 * AD), kp(size_t(R) * KV), vp(size_t(R) * KV);
            if (live > 0) gemm(L.q4[Q_Q], xn, live, qp.data(), 2 * AD, nullptr, scale_in);
            gemm(L.q4[Q_K], xn, R, kp.data(), KV, nullptr, scale_in);
            gemm(L.q4[Q_V], xn, R, vp.data(), KV, nullptr, scale_in);
            Operand core(R, AD);
            attention_layer(e, full_index, L, t, live, qp.data(), kp.data(), vp.data(), core);
            if (live > 0) gemm(L.q4[Q_O], core, live, h.data(), H, h.data());
            ++full_index;
        }
        if (live > 0) {
            Operand pn(live, H);
            std::vector<float> inv_post;
            if (g_norm_contract == 1) rmsnorm_operand_deferred(h.data(), H, L.vec[V_POST_NORM], live, H, g.eps, pn, inv_post);
            else rmsnorm_operand(h.data(), H, L.vec[V_POST_NORM], live, H, g.eps, pn);
            const float *scale_post = g_norm_contract == 1 ? inv_post.data() : nullptr;
            std::vector<float> gate(size_t(live) * g.inter), up(size_t(live) * g.inter);
            gemm(L.q4[Q_GATE], pn, live, gate.data(), g.inter, nullptr, scale_post);
            gemm(L.q4[Q_UP], pn, live, up.data(), g.inter, nullptr, scale_post);
            Operand act(live, g.inter);      // engine.metal:200-219
#pragma omp parallel for schedule(static)
            for (int r = 0; r < live; ++r) {
                for (int i = 0; i < g.inter; ++i)
                    act.values[size_t(r) * g.inter + i] = round_bf16(silu(gate[size_t(r) * g.inter + i]) * up[size_t(r) * g.inter + i]);
                act.finish_row(r);
            }
            gemm(L.q4[Q_DOWN], act, live, h.data(), H, h.data());
        }
        if (hidden_taps) memcpy(hidden_taps + size_t(l) * R * H, h.data(), sizeof(float) * R * H);
    }
    if (t.logit_rows > 0 && logits && layers == g.layers) {
        std::vector<float> hs(size_t(t.logit_rows) * H);
        for (uint32_t i = 0; i < t.logit_rows; ++i) memcpy(&hs[size_t(i) * H], &h[size_t(t.gather_index[i]) * H], sizeof(float) * H);
        Operand hn(t.logit_rows, H);
        rmsnorm_operand(hs.data(), H, m.final_norm, t.logit_rows, H, g.eps, hn);
        gemm(m.head, hn, t.logit_rows, logits, g.vocab, nullptr);
    }
    return 0;
}

// A bare q4 GEMM on fp32 activations (rounded to bf16 here), for kernel-level comparisons.
void orc_gemm_q4(const uint32_t *packed, const uint16_t *scales, const uint16_t *biases, int n, int k,
                 const float *activations, int rows, const float *residual, float *out) {
    Q4 w; w.rows = n; w.inner = k;
    w.packed.assign(packed, packed + size_t(n) * k / 8);
    w.scales.assign(scales, scales + size_t(n) * k / 64);
    w.biases.assign(biases, biases + size_t(n) * k / 64);
    Operand a(rows, k);
    for (int r = 0; r < rows; ++r) {
        for (int i = 0; i < k; ++i) a.values[size_t(r) * k + i] = round_bf16(activations[size_t(r) * k + i]);
        a.finish_row(r);
    }
    gemm(w, a, rows, out, n, residual);
}

}  // extern "C"
