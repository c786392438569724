// spl_gdn.cuh — gated-delta-rule linear attention: causal conv1d + SiLU, and the per-token state
// update with journal replay, gated RMSNorm and the operand of the output projection.
//
// Stands in for encodeLinear's kernels (Sources/SploshRuntime/Engine.swift:2001-2077):
// sp_gdn_fast (Sources/Shaders/engine.metal:668-851) and the split path
// (Sources/Shaders/candidates/gdn_b.metal:205-349, engine.metal:987-1069).
//
// HBM layout (per gated-delta layer):
//   state    [slot][value head][value j][key i]  fp32      (the reference's, engine.metal:743-745)
//   conv     [unit][channel][3]                  fp32, oldest first; channels are q | k | v
//   journal  [slot][16 rows][value head][260]    fp32: k[128], delta[128], decay, 3 pad
#pragma once
#include "spl_common.cuh"
#include "spl_gemm_tc.cuh"

struct SplGdnParams {
    int rows, runs, channels, key_heads, value_heads, head_dim;
    int proj_ld, z_offset, a_offset, b_offset;     // columns of the fused input projection
    float eps;
    int chunk_min;     // > 0: ordinary runs of at least this many rows are left to the chunked kernels (spl_gdn_chunk.cuh)
    int out_file_order;     // the out projection's columns are in a GGUF file's order of the value heads (below)
};

// Where value head h's 128 outputs go among the out projection's inputs. A GGUF file orders the value heads differently from the
// engine: its head i is the engine's ratio * (i % key_heads) + i / key_heads, ratio = value heads per key head
// (Sources/SploshModel/GgufNames.swift:73-84). Rows of a weight are moved when such a file is loaded; the out projection has
// the heads as its columns, which cannot move without re-quantising, so it stays in file order and the blocks write their
// output in that order instead (Sources/SploshModel/GgufConvert.swift:18-24; the reference's `heads` kernels read it so).
__device__ __forceinline__ int spl_gdn_out_head(const SplGdnParams &p, int h) {
    const int ratio = p.value_heads / p.key_heads;
    return p.out_file_order ? p.key_heads * (h % ratio) + h / ratio : h;
}

// Conv (k = 4, depthwise, no bias) + SiLU over every channel of every run; then the conv history
// of every unit a row writes: the last three raw inputs up to and including that row
// (engine.metal:707-728, 838-849). Grid (ceil(channels / 256), runs, segments), 256 threads: a long run (a prompt chunk) is
// cut in segments of SPL_GDN_CONV_SEGMENT rows, each a block of its own (the filter has no recurrence: a row needs the
// three rows before it, which a later segment reads from the projection itself). The units are written by the run's first
// segment only, after it has read the history it starts from: a speculative run (at most 16 rows) is one segment, and an
// ordinary run writes one unit, the slot's current one, at its last row, which the first segment does from the run's last
// three inputs, so the block that reads a unit is the block that overwrites it.
#define SPL_GDN_CONV_SEGMENT 128
__global__ void __launch_bounds__(256)
spl_gdn_conv_kernel(const float *__restrict__ proj, const uint16_t *__restrict__ conv_weight, float *conv_state,
                    const uint32_t *__restrict__ runs, const uint32_t *__restrict__ row_read, const uint32_t *__restrict__ row_write,
                    float *act, SplGdnParams p) {
    spl_grid_begin();
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= p.channels) return;
    const uint32_t start = runs[blockIdx.y * 3 + 1], length = runs[blockIdx.y * 3 + 2];
    const uint32_t first = blockIdx.z * SPL_GDN_CONV_SEGMENT, last = min(length, first + SPL_GDN_CONV_SEGMENT);
    if (first >= length) return;
    float x3, x2, x1;
    if (first == 0) {
        const float *hist = conv_state + (size_t(row_read[start]) * p.channels + c) * 3;
        x3 = hist[0]; x2 = hist[1]; x1 = hist[2];
    } else {
        x3 = proj[size_t(start + first - 3) * p.proj_ld + c]; x2 = proj[size_t(start + first - 2) * p.proj_ld + c]; x1 = proj[size_t(start + first - 1) * p.proj_ld + c];
    }
    const float w0 = spl_bf16_to_float(conv_weight[c * 4]), w1 = spl_bf16_to_float(conv_weight[c * 4 + 1]);
    const float w2 = spl_bf16_to_float(conv_weight[c * 4 + 2]), w3 = spl_bf16_to_float(conv_weight[c * 4 + 3]);
    // Eight rows at a time: their inputs and the units they write are asked for together, then the rows are taken in order.
    for (uint32_t base = first; base < last; base += 8) {
        float xs[8];
        uint32_t unit[9];
#pragma unroll
        for (int u = 0; u < 8; ++u) xs[u] = base + u < last ? proj[size_t(start + base + u) * p.proj_ld + c] : 0.0f;
#pragma unroll
        for (int u = 0; u < 9; ++u) unit[u] = (first == 0 && base + u < length) ? row_write[start + base + u] : 0xFFFFFFFFu;      // past the run: "another unit"
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (base + u < last) {
                const uint32_t row = start + base + u;
                const float x0 = xs[u];
                const float y = ((w0 * x3 + w1 * x2) + w2 * x1) + w3 * x0;
                act[size_t(row) * p.channels + c] = spl_silu_exact(y);
                if (first == 0 && unit[u + 1] != unit[u]) {
                    float *dst = conv_state + (size_t(unit[u]) * p.channels + c) * 3;
                    dst[0] = x2; dst[1] = x1; dst[2] = x0;
                }
                x3 = x2; x2 = x1; x1 = x0;
            }
        }
    }
    // A run of more than one segment (ordinary rows, one unit): its last row's unit from the run's last three inputs.
    if (first == 0 && length > SPL_GDN_CONV_SEGMENT) {
        float *dst = conv_state + (size_t(row_write[start + length - 1]) * p.channels + c) * 3;
        dst[0] = proj[size_t(start + length - 3) * p.proj_ld + c]; dst[1] = proj[size_t(start + length - 2) * p.proj_ld + c]; dst[2] = proj[size_t(start + length - 1) * p.proj_ld + c];
    }
}

// The state update S' = S * decay + k * delta with the product rounded on its own, so that the
// replay of a journal entry reproduces the original update bit for bit (engine.metal:654-659).
__device__ __forceinline__ float2 spl_gdn_update2(float2 s, float2 decay, float2 k, float2 delta) {
    return spl_fma2(s, decay, spl_mul2(k, delta));
}

#define SPL_GDN_TC 8           // tokens per pass
#define SPL_GDN_D 128          // head dim (key and value)
#define SPL_GDN_THREADS 256
#define SPL_GDN_PART_LD (SPL_GDN_TC * SPL_GDN_D + 4)      // floats from one column group's partial sums to the next's: four banks on

// Dynamic shared memory of the recurrence kernel: q, k, v, o and the journal-form delta of a pass (5 x TC rows), the journal
// entries to replay (k and delta, SPL_JOURNAL_ROWS rows each), the eight column groups' partial products, and the two
// reduced products S0 k and S0 q (TC rows each).
constexpr size_t spl_gdn_recurrence_smem() {
    return sizeof(float) * (size_t(7 * SPL_GDN_TC + 2 * SPL_JOURNAL_ROWS) * SPL_GDN_D + 8 * SPL_GDN_PART_LD);
}

// One thread block per (value head, run): the head's whole 128 x 128 state in registers, a 4 x 16 tile a thread:
// thread (rg = tid / 8, cg = tid % 8) keeps rows j = 4 rg + r (r < 4) at columns i = 32 c + 4 cg + e (c < 4, e < 4).
// A token's k or q then costs a thread four 16-byte loads from shared memory for 64 state elements (a thread that
// held one row would load as much for 16 elements, and the kernel would be bound by shared-memory bandwidth).
// Per token (engine.metal:763-805), with k^ = k invK and q^ = q invQ:
//   mem = S k;  delta = (v - mem * decay * invK) * beta * invK;  S = S * decay + k (x) delta;  o = (S q) * invQ
// The tokens of a run are taken eight at a time (a pass), and inside a pass nothing waits for a state update: with
// S0 the state at the start of the pass, G(t) the product of the decays up to token t and d^(t) = delta(t) / invK(t),
//   decay(t) S(t-1) k^(t) = G(t) S0 k^(t) + sum over s < t of G(t)/G(s) (k^(s) . k^(t)) d^(s)
//   d^(t) = beta(t) (v(t) - G(t) S0 k^(t)) - sum over s < t of A(t, s) d^(s),   A(t, s) = beta(t) G(t)/G(s) k^(t) . k^(s)
//   o(t)  = G(t) S0 q^(t) + sum over s <= t of M(t, s) d^(s),                    M(t, s) = G(t)/G(s) q^(t) . k^(s)
// so the pass is: the two 8 x 8 matrices (64-element half dots, two threads a dot), the products S0 k and S0 q for all
// eight tokens at once (each thread its tile, partial sums over its 64 columns, the eight column groups added through
// shared memory), then one thread a value row walks the eight tokens (a chain of multiply-adds on 8 x 8 numbers).
// The token-serial form of the same pass was a chain of eight (product, reduce, update, product, reduce) rounds and
// took five times as long.
// The state moves on by the journal's own rule, S = S * decay + k (x) delta with the product rounded on its own
// (engine.metal:654-659), applied entry by entry: to the entries accepted from the previous speculative run
// (engine.metal:744-761), and to a pass's tokens when more of the run follows or an ordinary run writes its state.
// A speculative run leaves a journal entry per row instead of writing the state, so the state it would reach and the
// state a later replay reaches are the same numbers. Then the gated RMSNorm w * o * rsqrt(mean o^2 + eps) * silu(z)
// rounded to bf16, with its per-64 sums (engine.metal:812-833).
// Grid (value_heads, runs), 256 threads, two blocks to an SM.
__global__ void __launch_bounds__(SPL_GDN_THREADS, 2)
spl_gdn_recurrence_kernel(const float *__restrict__ act, const float *__restrict__ proj, const uint16_t *__restrict__ a_log,
                          const uint16_t *__restrict__ dt_bias, const uint16_t *__restrict__ norm_weight, float *state, float *journal,
                          const uint32_t *__restrict__ runs, const uint32_t *__restrict__ run_info, SplOperand core, SplGdnParams p) {
    constexpr int D = SPL_GDN_D, TC = SPL_GDN_TC, NT = SPL_GDN_THREADS, WARPS = NT / 32, PLD = SPL_GDN_PART_LD;
    static_assert(TC == WARPS, "the norm passes give a warp a token");
    extern __shared__ __align__(16) float gdn_smem[];
    float (*q_s)[D] = reinterpret_cast<float (*)[D]>(gdn_smem);
    float (*k_s)[D] = q_s + TC, (*v_s)[D] = k_s + TC, (*o_s)[D] = v_s + TC, (*d_s)[D] = o_s + TC;
    float (*pm)[D] = d_s + TC, (*rm)[D] = pm + TC;
    float (*jk_s)[D] = rm + TC, (*jd_s)[D] = jk_s + SPL_JOURNAL_ROWS;
    float *part = &jd_s[SPL_JOURNAL_ROWS][0];
    __shared__ float scal[TC][4], jdecay[SPL_JOURNAL_ROWS];        // invQ, invK, decay, beta per token; decay per replayed entry
    __shared__ float gam[TC], a_m[TC][TC], m_m[TC][TC];
    const int h = blockIdx.x, run = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rg = tid >> 3, cg = tid & 7;
    const uint32_t slot = runs[run * 3], start = runs[run * 3 + 1], length = runs[run * 3 + 2];
    const bool speculative = run_info[run * 2] != 0;
    const uint32_t pending = run_info[run * 2 + 1];
    if (!speculative && p.chunk_min > 0 && length >= uint32_t(p.chunk_min)) return;      // a long ordinary run: the chunked kernels take it
    const int VH = p.value_heads, KH = p.key_heads, hk = h / (VH / KH);
    float *jhead = journal + (size_t(slot) * SPL_JOURNAL_ROWS * VH + h) * SPL_JOURNAL_WIDTH;

    // Everything the block needs from memory is asked for before anything is waited for, and what no kernel of this step
    // has written (the state and the journal: the previous step's; the run tables: copied before the step's first kernel)
    // before the wait for the kernels in front: a block that has come onto an SM while the conv kernel runs has its state
    // on the way. The input projection's columns (gates, z) are two kernels back, the conv's output is one: after the wait.
    float2 S[4][4][2];          // [row r][column chunk c][pair]
    float4 *stored = reinterpret_cast<float4 *>(state + ((size_t(slot) * VH + h) * D + 4 * rg) * D) + cg;
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float4 v = stored[r * (D / 4) + 8 * c];
            S[r][c][0] = make_float2(v.x, v.y); S[r][c][1] = make_float2(v.z, v.w);
        }
    for (int idx = tid; idx < int(pending) * (2 * D / 4); idx += NT) {
        const int e = idx / (2 * D / 4), i4 = idx % (2 * D / 4);
        const float4 v = *reinterpret_cast<const float4 *>(jhead + size_t(e) * VH * SPL_JOURNAL_WIDTH + i4 * 4);
        float *dst = i4 < D / 4 ? &jk_s[e][i4 * 4] : &jd_s[e][i4 * 4 - D];
        *reinterpret_cast<float4 *>(dst) = v;
    }
    if (tid < int(pending)) jdecay[tid] = jhead[size_t(tid) * VH * SPL_JOURNAL_WIDTH + 2 * D];
    // The first pass's gate inputs and z, one warp a token.
    float gate_a0 = 0.0f, gate_b0 = 0.0f;
    float4 z0 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (uint32_t(warp) < length) {
        const size_t row = start + warp;
        if (lane == 0) { gate_a0 = proj[row * p.proj_ld + p.a_offset + h]; gate_b0 = proj[row * p.proj_ld + p.b_offset + h]; }
        z0 = *reinterpret_cast<const float4 *>(proj + row * p.proj_ld + p.z_offset + h * D + lane * 4);
    }
    spl_grid_begin();
    const float neg_a = -expf(spl_bf16_to_float(a_log[h])), bias = spl_bf16_to_float(dt_bias[h]);

    // One journal-form update of the thread's tile.
    auto apply = [&](const float *k_row, const float *delta_row, float decay) {
        const float4 d4 = *reinterpret_cast<const float4 *>(delta_row + 4 * rg);
        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
        const float2 c2 = make_float2(decay, decay);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float4 kv = *reinterpret_cast<const float4 *>(k_row + 32 * c + 4 * cg);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float2 d2 = make_float2(dl[r], dl[r]);
                S[r][c][0] = spl_gdn_update2(S[r][c][0], c2, make_float2(kv.x, kv.y), d2);
                S[r][c][1] = spl_gdn_update2(S[r][c][1], c2, make_float2(kv.z, kv.w), d2);
            }
        }
    };
    // The thread's partial sums of S x for the pass's tokens (x = k or q), into its column group's plane of `part`.
    auto product = [&](float (*x_s)[D], int count) {
#pragma unroll
        for (int tt = 0; tt < TC; ++tt) {
            if (tt < count) {
                float4 xv[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) xv[c] = *reinterpret_cast<const float4 *>(&x_s[tt][32 * c + 4 * cg]);
                float sum[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    float2 ma = make_float2(0.0f, 0.0f), mb = make_float2(0.0f, 0.0f);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        ma = spl_fma2(S[r][c][0], make_float2(xv[c].x, xv[c].y), ma);
                        mb = spl_fma2(S[r][c][1], make_float2(xv[c].z, xv[c].w), mb);
                    }
                    sum[r] = (ma.x + ma.y) + (mb.x + mb.y);
                }
                *reinterpret_cast<float4 *>(part + cg * PLD + tt * D + 4 * rg) = make_float4(sum[0], sum[1], sum[2], sum[3]);
            }
        }
    };
    // The eight column groups' partial sums added in a fixed order: four (token, row) pairs a thread.
    auto reduce = [&](float (*dst)[D], int count) {
#pragma unroll
        for (int n = 0; n < TC * D / NT; ++n) {
            const int idx = tid + NT * n, tt = idx / D, j = idx % D;
            if (tt < count) {
                float total = part[tt * D + j];
#pragma unroll
                for (int g = 1; g < 8; ++g) total += part[g * PLD + tt * D + j];
                dst[tt][j] = total;
            }
        }
    };

    // A run of no rows with entries to replay is a journal commit (Engine.commitJournal, Engine.swift:889-903): one pass, no tokens.
    for (uint32_t base = 0; base < length || (base == 0 && pending != 0); base += TC) {
        const int count = int(min(uint32_t(TC), length - base));
        if (base != 0) __syncthreads();
        // q, k, v of up to TC tokens; one warp a token for the norms and the gates.
        for (int idx = tid; idx < count * 3 * (D / 4); idx += NT) {
            const int tt = idx / (3 * (D / 4)), rest = idx % (3 * (D / 4)), kind = rest / (D / 4), i4 = rest % (D / 4);
            const int channel = kind == 0 ? hk * D : kind == 1 ? KH * D + hk * D : 2 * KH * D + h * D;
            const float4 v = *reinterpret_cast<const float4 *>(act + size_t(start + base + tt) * p.channels + channel + i4 * 4);
            float *dst = kind == 0 ? q_s[tt] : kind == 1 ? k_s[tt] : v_s[tt];
            *reinterpret_cast<float4 *>(dst + i4 * 4) = v;
        }
        float gate_a = gate_a0, gate_b = gate_b0;
        if (base != 0 && warp < count && lane == 0) {
            const size_t row = start + base + warp;
            gate_a = proj[row * p.proj_ld + p.a_offset + h]; gate_b = proj[row * p.proj_ld + p.b_offset + h];
        }
        __syncthreads();
        if (warp < count) {
            const float4 qv = *reinterpret_cast<const float4 *>(&q_s[warp][lane * 4]);
            const float4 kv = *reinterpret_cast<const float4 *>(&k_s[warp][lane * 4]);
            const float qq = spl_warp_sum(qv.x * qv.x + qv.y * qv.y + qv.z * qv.z + qv.w * qv.w);
            const float kk = spl_warp_sum(kv.x * kv.x + kv.y * kv.y + kv.z * kv.z + kv.w * kv.w);
            if (lane == 0) {
                scal[warp][0] = (1.0f / sqrtf(qq + 1e-6f)) * (1.0f / sqrtf(float(D)));
                scal[warp][1] = 1.0f / sqrtf(kk + 1e-6f);
                const float x = gate_a + bias;
                const float softplus = x > 20.0f ? x : logf(1.0f + expf(x));
                scal[warp][2] = expf(neg_a * softplus);
                scal[warp][3] = spl_sigmoid(gate_b);
            }
        }
        __syncthreads();      // the tokens' scalars are written
        if (count > 0) {
            // The two matrices: thread = (which, t, s, half of the 128 channels).
            const int which = tid >> 7, t = (tid >> 4) & 7, s = (tid >> 1) & 7, half = tid & 1;
            const bool wanted = t < count && (which ? s <= t : s < t);
            float dot = 0.0f;
            if (wanted) {
                const float *x = which ? q_s[t] : k_s[t], *y = k_s[s];
#pragma unroll 4
                for (int m = 0; m < D / 8; ++m) {
                    const float4 a = *reinterpret_cast<const float4 *>(x + 4 * (half + 2 * m)), b = *reinterpret_cast<const float4 *>(y + 4 * (half + 2 * m));
                    dot += (a.x * b.x + a.y * b.y) + (a.z * b.z + a.w * b.w);
                }
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            if (wanted && half == 0) {
                float ratio = 1.0f;
                for (int u = s + 1; u <= t; ++u) ratio *= scal[u][2];
                if (which) m_m[t][s] = ratio * dot * scal[t][0] * scal[s][1];
                else a_m[t][s] = scal[t][3] * ratio * dot * scal[t][1] * scal[s][1];
            }
            if (tid < count) {
                float g = 1.0f;
                for (int u = 0; u <= tid; ++u) g *= scal[u][2];
                gam[tid] = g;
            }
        }
        if (base == 0 && pending != 0) {
            // Replay the accepted entries; a speculative run then stores the state it starts from.
            for (uint32_t e = 0; e < pending; ++e) apply(jk_s[e], jd_s[e], jdecay[e]);
            if (speculative) {
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int c = 0; c < 4; ++c) stored[r * (D / 4) + 8 * c] = make_float4(S[r][c][0].x, S[r][c][0].y, S[r][c][1].x, S[r][c][1].y);
            }
        }
        if (count == 0) break;
        product(k_s, count);
        __syncthreads();
        reduce(pm, count);
        __syncthreads();      // the partial sums of S0 k have been read
        product(q_s, count);
        __syncthreads();
        reduce(rm, count);
        __syncthreads();
        if (tid < D) {
            const int j = tid;
            float dh[TC];
#pragma unroll
            for (int t = 0; t < TC; ++t) {
                if (t < count) {
                    float x = scal[t][3] * (v_s[t][j] - gam[t] * scal[t][1] * pm[t][j]);
#pragma unroll
                    for (int s = 0; s < t; ++s) x -= a_m[t][s] * dh[s];
                    dh[t] = x;
                    float o = gam[t] * scal[t][0] * rm[t][j];
#pragma unroll
                    for (int s = 0; s <= t; ++s) o += m_m[t][s] * dh[s];
                    o_s[t][j] = o;
                    d_s[t][j] = x * scal[t][1];
                }
            }
        }
        __syncthreads();
        if (speculative) {
            for (int idx = tid; idx < count * (2 * D / 4); idx += NT) {
                const int tt = idx / (2 * D / 4), i4 = idx % (2 * D / 4);
                float *entry = jhead + size_t(base + tt) * VH * SPL_JOURNAL_WIDTH;
                *reinterpret_cast<float4 *>(entry + 4 * i4) = i4 < D / 4 ? *reinterpret_cast<const float4 *>(&k_s[tt][4 * i4]) : *reinterpret_cast<const float4 *>(&d_s[tt][4 * i4 - D]);
            }
            if (tid < count) jhead[size_t(base + tid) * VH * SPL_JOURNAL_WIDTH + 2 * D] = scal[tid][2];
        }
        if (!speculative || base + TC < length)
            for (int tt = 0; tt < count; ++tt) apply(k_s[tt], d_s[tt], scal[tt][2]);
        // Gated RMSNorm and the bf16 operand, one warp a token.
        if (warp < count) {
            const int tt = warp;
            const size_t row = start + base + tt;
            const float4 z = base == 0 ? z0 : *reinterpret_cast<const float4 *>(proj + row * p.proj_ld + p.z_offset + h * D + lane * 4);
            const float4 ov = *reinterpret_cast<const float4 *>(&o_s[tt][lane * 4]);
            const float inv = 1.0f / sqrtf(spl_warp_sum(ov.x * ov.x + ov.y * ov.y + ov.z * ov.z + ov.w * ov.w) / float(D) + p.eps);
            const uint2 w = *reinterpret_cast<const uint2 *>(norm_weight + lane * 4);
            const float r0 = spl_bf16_to_float(uint16_t(w.x)) * ov.x * inv * spl_silu_exact(z.x);
            const float r1 = spl_bf16_to_float(uint16_t(w.x >> 16)) * ov.y * inv * spl_silu_exact(z.y);
            const float r2 = spl_bf16_to_float(uint16_t(w.y)) * ov.z * inv * spl_silu_exact(z.z);
            const float r3 = spl_bf16_to_float(uint16_t(w.y >> 16)) * ov.w * inv * spl_silu_exact(z.w);
            const uint16_t b0 = spl_float_to_bf16(r0), b1 = spl_float_to_bf16(r1), b2 = spl_float_to_bf16(r2), b3 = spl_float_to_bf16(r3);
            *reinterpret_cast<uint2 *>(core.values + core.at(int(row), spl_gdn_out_head(p, h) * D + lane * 4)) =
                spl_operand_pack4(spl_bf16_to_float(b0), spl_bf16_to_float(b1), spl_bf16_to_float(b2), spl_bf16_to_float(b3));
            // The following GEMM's per-64 sums: a 128-wide head is two quant groups, sixteen lanes each.
            float gsum = (spl_bf16_to_float(b0) + spl_bf16_to_float(b1)) + (spl_bf16_to_float(b2) + spl_bf16_to_float(b3));
#pragma unroll
            for (int o2 = 8; o2 > 0; o2 >>= 1) gsum += __shfl_xor_sync(0xffffffffu, gsum, o2);
            if ((lane & 15) == 0) core.put_sum(int(row), spl_gdn_out_head(p, h) * 2 + (lane >> 4), gsum);
        }
    }
    if (!speculative) {
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) stored[r * (D / 4) + 8 * c] = make_float4(S[r][c][0].x, S[r][c][0].y, S[r][c][1].x, S[r][c][1].y);
    }
}
