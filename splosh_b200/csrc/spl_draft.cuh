// spl_draft.cuh — the kernels of the DFlash 2 block-diffusion drafter that are its own (Sources/Shaders/draft.metal);
// everything linear in a draft pass runs on the engine's q4 GEMM, its norms and its embedding gather
// (Sources/SploshRuntime/DraftModel.swift:418-468).
#pragma once
#include "spl_common.cuh"

#define SPL_DRAFT_HEAD_DIM 128

// Full-width rotary embedding of element i of a 128-wide head at `position`: pairs (i, i + 64) (draft.metal:13-19).
__device__ __forceinline__ float spl_draft_rope(float x, float paired, int i, uint32_t position, float theta) {
    const int half = SPL_DRAFT_HEAD_DIM >> 1, slot = i < half ? i : i - half;
    const float angle = float(position) * powf(theta, -(2.0f * float(slot)) / float(SPL_DRAFT_HEAD_DIM));
    return x * cosf(angle) + (i < half ? -paired : paired) * sinf(angle);
}

// Grouped dynamic causal convolution (kernel size 2) over the rows of one block (draft.metal:21-57):
//   out[t][c] = sum over o in {0, 1} of (base[which][o][c] + dynamic[t][which][o][c / group_size]) * in[t - o][c]
// with in[t - o] zero before the block's first row (row_offset[t] is the row's index in its block); `accumulate` adds the
// result into out (the residual). Grid (ceil(hidden / 256), rows), 256 threads.
__global__ void __launch_bounds__(256)
spl_draft_conv_kernel(const float *__restrict__ in, const float *__restrict__ dynamic, const uint16_t *__restrict__ base, float *out,
                      int hidden, int group_size, int groups, int which, int accumulate, const uint32_t *__restrict__ row_offset) {
    spl_grid_begin();
    const int c = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
    if (c >= hidden) return;
    const int group = c / group_size;
    const uint32_t in_block = row_offset[t];
    float acc = 0.0f;
#pragma unroll
    for (int o = 0; o < 2; ++o) {
        if (in_block < uint32_t(o)) continue;
        const int tap = which * 2 + o;
        const float kernel = spl_bf16_to_float(base[size_t(tap) * hidden + c]) + dynamic[size_t(t) * (4 * groups) + tap * groups + group];
        acc += kernel * in[size_t(t - o) * hidden + c];
    }
    const size_t index = size_t(t) * hidden + c;
    out[index] = accumulate ? out[index] + acc : acc;
}

// Draft K and V into the per-slot context ring (draft.metal:59-100): K is RMSNorm (plain weight) then rotary, V verbatim;
// ring [slot][position % capacity][kv head][128] fp16. Grid (kv_heads, rows), 32 threads.
__global__ void __launch_bounds__(32)
spl_draft_kv_store_kernel(const float *__restrict__ kproj, const float *__restrict__ vproj, const uint16_t *__restrict__ norm_weight,
                          const uint32_t *__restrict__ row_slot, const uint32_t *__restrict__ row_pos, __half *kring, __half *vring,
                          int kv_heads, int capacity, float eps, float theta) {
    spl_grid_begin();
    constexpr int D = SPL_DRAFT_HEAD_DIM;
    const int head = blockIdx.x, row = blockIdx.y, lane = threadIdx.x;
    const size_t base = (size_t(row) * kv_heads + head) * D;
    float partial = 0.0f;
    for (int i = lane; i < D; i += 32) { const float x = kproj[base + i]; partial += x * x; }
    const float inv = 1.0f / sqrtf(spl_warp_sum(partial) / float(D) + eps);
    const uint32_t position = row_pos[row];
    const size_t dst = ((size_t(row_slot[row]) * capacity + position % uint32_t(capacity)) * kv_heads + head) * D;
    for (int i = lane; i < D; i += 32) {
        const int pi = i < D / 2 ? i + D / 2 : i - D / 2;
        const float x = kproj[base + i] * inv * spl_bf16_to_float(norm_weight[i]);
        const float paired = kproj[base + pi] * inv * spl_bf16_to_float(norm_weight[pi]);
        kring[dst + i] = __float2half_rn(spl_draft_rope(x, paired, i, position, theta));
        vring[dst + i] = __float2half_rn(vproj[base + i]);
    }
}

// Draft attention, non-causal within a sliding window (draft.metal:102-192): query row r sees every ring position in
// [row_lo[r], row_hi[r]) closer than `window`: the accumulated context plus the rows of its own block. The reference runs
// a 128-thread group per (head, row), thread j owning channel j, and walks the visible positions in chunks of 128 with a
// running maximum; this kernel is that walk (same chunking, same order of the sums) with the query heads of one kv head
// side by side in one block, so a chunk's keys and values are read once for all of them. Queries get their RMSNorm and
// rotary embedding here. G = heads / kv_heads (at most 8). The chunks are dealt to gridDim.z spans that run side by side and
// leave partial results for the merge kernel (the reference's sp_draft_attention_span, draft.metal:194-277: the walk of a
// full window is eighteen chunks in sequence otherwise). Grid (kv_heads, rows, spans), 128 threads.
template <int G>
__global__ void __launch_bounds__(128)
spl_draft_attention_kernel(const float *__restrict__ qproj, const uint16_t *__restrict__ norm_weight, const uint32_t *__restrict__ row_slot,
                           const uint32_t *__restrict__ row_pos, const uint32_t *__restrict__ row_lo, const uint32_t *__restrict__ row_hi,
                           const __half *__restrict__ kring, const __half *__restrict__ vring, float *partials, int heads, int kv_heads,
                           int capacity, int window, float scale, float eps, float theta) {
    constexpr int D = SPL_DRAFT_HEAD_DIM;
    __shared__ float query[G][D];
    __shared__ float scores[G][D];
    __shared__ float warp_max[G][4];
    spl_grid_begin();
    const int kv_head = blockIdx.x, row = blockIdx.y, j = threadIdx.x;
    const uint32_t position = row_pos[row];
    const int pj = j < D / 2 ? j + D / 2 : j - D / 2;
#pragma unroll
    for (int g = 0; g < G; ++g) scores[g][j] = qproj[(size_t(row) * heads + kv_head * G + g) * D + j];
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float ss = 0.0f;
        for (int i = 0; i < D; ++i) ss += scores[g][i] * scores[g][i];
        const float inv = 1.0f / sqrtf(ss / float(D) + eps);
        query[g][j] = spl_draft_rope(scores[g][j] * inv * spl_bf16_to_float(norm_weight[j]), scores[g][pj] * inv * spl_bf16_to_float(norm_weight[pj]), j, position, theta);
    }
    __syncthreads();

    const uint32_t first_visible = position + 1u > uint32_t(window) ? position + 1u - uint32_t(window) : 0u;
    const uint32_t lo = max(row_lo[row], first_visible), hi = row_hi[row];
    const uint32_t chunks = hi > lo ? (hi - lo + D - 1) / D : 0u;
    const uint32_t per_span = (chunks + gridDim.z - 1) / gridDim.z, chunk_begin = blockIdx.z * per_span, chunk_end = min(chunks, chunk_begin + per_span);
    const size_t ring_base = size_t(row_slot[row]) * capacity;
    float run_max[G], run_sum[G], acc[G];
#pragma unroll
    for (int g = 0; g < G; ++g) { run_max[g] = -INFINITY; run_sum[g] = 0.0f; acc[g] = 0.0f; }
    for (uint32_t chunk = chunk_begin; chunk < chunk_end; ++chunk) {
        const uint32_t first = lo + chunk * D;
        float score[G];
#pragma unroll
        for (int g = 0; g < G; ++g) score[g] = -INFINITY;
        if (first + j < hi) {
            const __half *k = kring + ((ring_base + (first + j) % uint32_t(capacity)) * kv_heads + kv_head) * D;
            float d[G];
#pragma unroll
            for (int g = 0; g < G; ++g) d[g] = 0.0f;
            for (int i = 0; i < D; i += 8) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(k + i);
                const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float2 kk = __half22float2(h2[u]);
#pragma unroll
                    for (int g = 0; g < G; ++g) { d[g] += query[g][i + 2 * u] * kk.x; d[g] += query[g][i + 2 * u + 1] * kk.y; }
                }
            }
#pragma unroll
            for (int g = 0; g < G; ++g) score[g] = d[g] * scale;
        }
        // The chunk's maximum: the four warps' maxima meet in shared memory (a maximum does not depend on the order).
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float m = spl_warp_max(score[g]);
            if ((j & 31) == 0) warp_max[g][j >> 5] = m;
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float chunk_max = fmaxf(fmaxf(warp_max[g][0], warp_max[g][1]), fmaxf(warp_max[g][2], warp_max[g][3]));
            const float new_max = fmaxf(run_max[g], chunk_max), rescale = expf(run_max[g] - new_max);
            acc[g] *= rescale; run_sum[g] *= rescale; run_max[g] = new_max;
            scores[g][j] = expf(score[g] - new_max);
        }
        __syncthreads();
        // Positions in order, as the reference adds them; a position past the row's range has probability zero and is not read.
        const uint32_t count = min(uint32_t(D), hi - first);
#pragma unroll 8
        for (uint32_t t = 0; t < count; ++t) {
            const float v = __half2float(vring[((ring_base + (first + t) % uint32_t(capacity)) * kv_heads + kv_head) * D + j]);
#pragma unroll
            for (int g = 0; g < G; ++g) { const float prob = scores[g][t]; run_sum[g] += prob; acc[g] += prob * v; }
        }
        __syncthreads();
    }
    // The span's share: [running maximum, running sum, 128 accumulated values] per (row, head, span) (draft.metal:194-199).
#pragma unroll
    for (int g = 0; g < G; ++g) {
        float *p = partials + ((size_t(row) * heads + kv_head * G + g) * gridDim.z + blockIdx.z) * (D + 2);
        if (j == 0) { p[0] = run_max[g]; p[1] = run_sum[g]; }
        p[2 + j] = acc[g];
    }
}

// The same attention on the tensor cores (the warp-level instruction, fp16 operands, fp32 sums): one block per (kv head,
// request, span). A request's rows x the kv head's G query heads are the M dimension (32 or 64 queries, 16 to a warp); the
// span's positions come through shared memory 64 at a time: S = Q K^T, the row-wise running maximum and sum, P (rounded to
// fp16) times V. Every (query, position) pair is masked by the row's own range [max(lo, position + 1 - window), hi). The
// result is the span's partial [maximum, sum, 128 values] per (row, head) for the merge kernel, as the other form leaves it.
// requests[2 r], [2 r + 1]: first row and row count of request r (count x G <= 64). Grid (kv_heads, requests, spans), 128 threads.
__device__ __forceinline__ void spl_draft_mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <int G>
__global__ void __launch_bounds__(128)
spl_draft_attention_mma_kernel(const float *__restrict__ qproj, const uint16_t *__restrict__ norm_weight, const uint32_t *__restrict__ requests,
                               const uint32_t *__restrict__ row_slot, const uint32_t *__restrict__ row_pos, const uint32_t *__restrict__ row_lo,
                               const uint32_t *__restrict__ row_hi, const __half *__restrict__ kring, const __half *__restrict__ vring, float *partials,
                               int heads, int kv_heads, int capacity, int window, float scale, float eps, float theta) {
    constexpr int D = SPL_DRAFT_HEAD_DIM, LD = D + 8, TK = 64;       // a row of 136 halves: the fragments' 32-bit loads meet no bank twice
    __shared__ __align__(16) __half ks[TK][LD];
    __shared__ __align__(16) __half qv[64][LD];                     // the queries first, then every chunk's values
    __shared__ uint32_t q_lo[64], q_hi[64];
    spl_grid_begin();
    const int kv_head = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t row0 = requests[2 * blockIdx.y], count = requests[2 * blockIdx.y + 1];
    const int queries = int(count) * G, mtiles = (queries + 15) / 16;
    // Queries: RMSNorm and rotary embedding, to fp16; a warp a query, a lane the elements lane, lane + 32 and their partners 64 on.
    for (int q = warp; q < 64; q += 4) {
        if (q < queries) {
            const uint32_t row = row0 + q / G;
            const float *src = qproj + (size_t(row) * heads + kv_head * G + q % G) * D;
            const float x0 = src[lane], x1 = src[lane + 32], y0 = src[lane + 64], y1 = src[lane + 96];
            const float inv = 1.0f / sqrtf(spl_warp_sum(x0 * x0 + x1 * x1 + y0 * y0 + y1 * y1) / float(D) + eps);
            const float w0 = spl_bf16_to_float(norm_weight[lane]), w1 = spl_bf16_to_float(norm_weight[lane + 32]);
            const float w2 = spl_bf16_to_float(norm_weight[lane + 64]), w3 = spl_bf16_to_float(norm_weight[lane + 96]);
            const float a0 = x0 * inv * w0, a1 = x1 * inv * w1, b0 = y0 * inv * w2, b1 = y1 * inv * w3;
            const uint32_t position = row_pos[row];
            qv[q][lane] = __float2half_rn(spl_draft_rope(a0, b0, lane, position, theta));
            qv[q][lane + 32] = __float2half_rn(spl_draft_rope(a1, b1, lane + 32, position, theta));
            qv[q][lane + 64] = __float2half_rn(spl_draft_rope(b0, a0, lane + 64, position, theta));
            qv[q][lane + 96] = __float2half_rn(spl_draft_rope(b1, a1, lane + 96, position, theta));
            if (lane == 0) {
                const uint32_t first_visible = position + 1u > uint32_t(window) ? position + 1u - uint32_t(window) : 0u;
                q_lo[q] = max(row_lo[row], first_visible); q_hi[q] = row_hi[row];
            }
        } else {
            qv[q][lane] = qv[q][lane + 32] = qv[q][lane + 64] = qv[q][lane + 96] = __float2half_rn(0.0f);
            if (lane == 0) { q_lo[q] = 0xFFFFFFFFu; q_hi[q] = 0u; }
        }
    }
    __syncthreads();
    const bool computing = warp < mtiles;
    const int m0 = warp * 16;
    uint32_t qa[8][4];                                              // the warp's sixteen queries as A fragments, eight steps of the 128 channels
    uint32_t lo_a = 0xFFFFFFFFu, hi_a = 0u, lo_b = 0xFFFFFFFFu, hi_b = 0u;
    if (computing) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            qa[kk][0] = *reinterpret_cast<const uint32_t *>(&qv[m0 + g][16 * kk + 2 * t]);
            qa[kk][1] = *reinterpret_cast<const uint32_t *>(&qv[m0 + g + 8][16 * kk + 2 * t]);
            qa[kk][2] = *reinterpret_cast<const uint32_t *>(&qv[m0 + g][16 * kk + 2 * t + 8]);
            qa[kk][3] = *reinterpret_cast<const uint32_t *>(&qv[m0 + g + 8][16 * kk + 2 * t + 8]);
        }
        lo_a = q_lo[m0 + g]; hi_a = q_hi[m0 + g]; lo_b = q_lo[m0 + g + 8]; hi_b = q_hi[m0 + g + 8];
    }
    // The request's whole range, dealt to the spans in runs of chunks.
    uint32_t lo_all = 0xFFFFFFFFu, hi_all = 0u;
    for (int q = 0; q < queries; q += G) { lo_all = min(lo_all, q_lo[q]); hi_all = max(hi_all, q_hi[q]); }
    const uint32_t chunks = hi_all > lo_all ? (hi_all - lo_all + TK - 1) / TK : 0u;
    const uint32_t per_span = (chunks + gridDim.z - 1) / gridDim.z, chunk_begin = blockIdx.z * per_span, chunk_end = min(chunks, chunk_begin + per_span);
    const size_t ring_base = size_t(row_slot[row0]) * capacity;
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
    float max_a = -INFINITY, max_b = -INFINITY, sum_a = 0.0f, sum_b = 0.0f;
    __syncthreads();                                                // the queries are in registers: their place takes the values
    for (uint32_t chunk = chunk_begin; chunk < chunk_end; ++chunk) {
        const uint32_t first = lo_all + chunk * TK;
        // 64 positions' keys and values, sixteen bytes a thread and turn; positions past the range are zero.
        for (int idx = threadIdx.x; idx < TK * (D / 8); idx += 128) {
            const int token = idx / (D / 8), piece = idx % (D / 8);
            uint4 kk = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
            if (first + token < hi_all) {
                const size_t at = ((ring_base + (first + token) % uint32_t(capacity)) * kv_heads + kv_head) * D + piece * 8;
                kk = *reinterpret_cast<const uint4 *>(kring + at); vv = *reinterpret_cast<const uint4 *>(vring + at);
            }
            *reinterpret_cast<uint4 *>(&ks[token][piece * 8]) = kk; *reinterpret_cast<uint4 *>(&qv[token][piece * 8]) = vv;
        }
        __syncthreads();
        if (computing) {
            float sc[8][4];
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.0f;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t b0 = *reinterpret_cast<const uint32_t *>(&ks[8 * n + g][16 * kk + 2 * t]);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t *>(&ks[8 * n + g][16 * kk + 2 * t + 8]);
                    spl_draft_mma_f16(sc[n], qa[kk], b0, b1);
                }
            }
            // Scale, mask by the rows' own ranges, the rows' maxima over the chunk (a row lives in a quad of lanes).
            float cm_a = -INFINITY, cm_b = -INFINITY;
#pragma unroll
            for (int n = 0; n < 8; ++n)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint32_t position = first + 8 * n + 2 * t + e;
                    sc[n][e] = (position >= lo_a && position < hi_a) ? sc[n][e] * scale : -INFINITY;
                    sc[n][2 + e] = (position >= lo_b && position < hi_b) ? sc[n][2 + e] * scale : -INFINITY;
                    cm_a = fmaxf(cm_a, sc[n][e]); cm_b = fmaxf(cm_b, sc[n][2 + e]);
                }
            cm_a = fmaxf(cm_a, __shfl_xor_sync(0xffffffffu, cm_a, 1)); cm_a = fmaxf(cm_a, __shfl_xor_sync(0xffffffffu, cm_a, 2));
            cm_b = fmaxf(cm_b, __shfl_xor_sync(0xffffffffu, cm_b, 1)); cm_b = fmaxf(cm_b, __shfl_xor_sync(0xffffffffu, cm_b, 2));
            const float new_a = fmaxf(max_a, cm_a), new_b = fmaxf(max_b, cm_b);
            const float rs_a = new_a == -INFINITY ? 1.0f : expf(max_a - new_a), rs_b = new_b == -INFINITY ? 1.0f : expf(max_b - new_b);
            max_a = new_a; max_b = new_b; sum_a *= rs_a; sum_b *= rs_b;
#pragma unroll
            for (int n = 0; n < 16; ++n) { o[n][0] *= rs_a; o[n][1] *= rs_a; o[n][2] *= rs_b; o[n][3] *= rs_b; }
            uint32_t pa[4][4];                                      // P as A fragments: four steps of sixteen positions
            float ps_a = 0.0f, ps_b = 0.0f;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const float p0 = new_a == -INFINITY ? 0.0f : expf(sc[n][0] - new_a), p1 = new_a == -INFINITY ? 0.0f : expf(sc[n][1] - new_a);
                const float p2 = new_b == -INFINITY ? 0.0f : expf(sc[n][2] - new_b), p3 = new_b == -INFINITY ? 0.0f : expf(sc[n][3] - new_b);
                const __half2 ha = __floats2half2_rn(p0, p1), hb = __floats2half2_rn(p2, p3);
                // the sums take the rounded probabilities, the ones the product uses
                ps_a += __low2float(ha) + __high2float(ha); ps_b += __low2float(hb) + __high2float(hb);
                pa[n >> 1][(n & 1) * 2] = *reinterpret_cast<const uint32_t *>(&ha);
                pa[n >> 1][(n & 1) * 2 + 1] = *reinterpret_cast<const uint32_t *>(&hb);
            }
            ps_a += __shfl_xor_sync(0xffffffffu, ps_a, 1); ps_a += __shfl_xor_sync(0xffffffffu, ps_a, 2);
            ps_b += __shfl_xor_sync(0xffffffffu, ps_b, 1); ps_b += __shfl_xor_sync(0xffffffffu, ps_b, 2);
            sum_a += ps_a; sum_b += ps_b;
            // O += P V: the values' fragments come transposed out of their rows (ldmatrix.trans), two channel tiles a load.
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int n2 = 0; n2 < 8; ++n2) {
                    uint32_t b0, b1, b2, b3;
                    const uint32_t address = uint32_t(__cvta_generic_to_shared(&qv[16 * j + (lane & 15)][16 * n2 + 8 * (lane >> 4)]));
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(address));
                    spl_draft_mma_f16(o[2 * n2], pa[j], b0, b1);
                    spl_draft_mma_f16(o[2 * n2 + 1], pa[j], b2, b3);
                }
        }
        __syncthreads();
    }
    if (computing) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int q = m0 + g + 8 * half;
            if (q < queries) {
                const uint32_t row = row0 + q / G;
                float *p = partials + ((size_t(row) * heads + kv_head * G + q % G) * gridDim.z + blockIdx.z) * (D + 2);
                if (t == 0) { p[0] = half ? max_b : max_a; p[1] = half ? sum_b : sum_a; }
#pragma unroll
                for (int n = 0; n < 16; ++n) { p[2 + 8 * n + 2 * t] = o[n][2 * half]; p[2 + 8 * n + 2 * t + 1] = o[n][2 * half + 1]; }
            }
        }
    }
}

// The spans of a (row, head) put together (sp_draft_attention_merge, draft.metal:279-300). Grid (heads, rows), 128 threads.
__global__ void __launch_bounds__(128)
spl_draft_attention_merge_kernel(const float *__restrict__ partials, float *out, int heads, int spans) {
    constexpr int D = SPL_DRAFT_HEAD_DIM;
    spl_grid_begin();
    const int head = blockIdx.x, row = blockIdx.y, j = threadIdx.x;
    const float *p = partials + (size_t(row) * heads + head) * spans * (D + 2);
    float top = -INFINITY;
    for (int s = 0; s < spans; ++s) top = fmaxf(top, p[s * (D + 2)]);
    float sum = 0.0f, acc = 0.0f;
    for (int s = 0; s < spans; ++s) {
        const float m = p[s * (D + 2)];
        if (m == -INFINITY) continue;               // a span without a visible position
        const float w = expf(m - top);
        sum += p[s * (D + 2) + 1] * w; acc += p[s * (D + 2) + 2 + j] * w;
    }
    out[(size_t(row) * heads + head) * D + j] = acc / sum;
}

// selected[p][:] = rows[gather[p]][:] (sp_gather_rows). Grid (ceil(hidden / 256), picked), 256 threads.
__global__ void __launch_bounds__(256)
spl_draft_gather_kernel(const float *__restrict__ rows, const uint32_t *__restrict__ gather, float *selected, int hidden) {
    spl_grid_begin();
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c < hidden) selected[size_t(blockIdx.y) * hidden + c] = rows[size_t(gather[blockIdx.y]) * hidden + c];
}

// features[i][:] = engine feature rows[engine_row[i]][:] (the context pass's memcpy of Engine.featureRow, DraftModel.swift:337-339).
__global__ void __launch_bounds__(256)
spl_draft_take_features_kernel(const float *__restrict__ features, const uint32_t *__restrict__ engine_row, float *out, int width) {
    spl_grid_begin();
    for (int c = blockIdx.x * 256 + threadIdx.x; c < width; c += gridDim.x * 256) out[size_t(blockIdx.y) * width + c] = features[size_t(engine_row[blockIdx.y]) * width + c];
}

// The selector's projection of the drafted positions' hidden states (CandidateSelector.select's matrix-vector product,
// DraftModel.swift:499-502): projected[p][r] = sum over h of projection[r][h] * selected[p][h]. Grid (picked, ceil(rank / 32)),
// 256 threads: a block takes 32 ranks of one position, a warp four of them.
__global__ void __launch_bounds__(256)
spl_draft_project_kernel(const float *__restrict__ projection, const float *__restrict__ selected, float *projected, int rank, int hidden) {
    spl_grid_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float *x = selected + size_t(blockIdx.x) * hidden;
    for (int r = blockIdx.y * 32 + warp; r < min(rank, int(blockIdx.y) * 32 + 32); r += 8) {
        const float *m = projection + size_t(r) * hidden;
        float sum = 0.0f;
        for (int h = lane; h < hidden; h += 32) sum += m[h] * x[h];
        sum = spl_warp_sum(sum);
        if (lane == 0) projected[size_t(blockIdx.x) * rank + r] = sum;
    }
}

// The best (value descending, index ascending) of a block of 256 threads' candidates; every thread gets it. index 0x7fffffff: none.
__device__ __forceinline__ void spl_draft_block_best(float &bv, int &bi, float *best_v, int *best_i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    __syncthreads();                 // the last round's readers are done with the arrays
    if ((threadIdx.x & 31) == 0) { best_v[threadIdx.x >> 5] = bv; best_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    bv = best_v[0]; bi = best_i[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) {
        const float ov = best_v[w]; const int oi = best_i[w];
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
}

// The k largest of [0, limit) per logit row, descending, the lower index first among equal values (TopK.select,
// Sampler.swift:19-52), in two kernels so that a row is many blocks' work: the k best of each of `segments` stretches of
// the row (k rounds of a block-wide selection, as the one-kernel form does over the whole row), then the k best of those.
// A stretch is at most 256 x 64 values: a thread keeps its 64 in registers, so the k rounds read the row once.
// Grid (rows, segments), 256 threads; candidates [rows][segments][k], index -1 where a stretch ran out (NaN and -inf never qualify).
#define SPL_DRAFT_TOPK_STRETCH (256 * 64)
__global__ void __launch_bounds__(256)
spl_draft_topk_segment_kernel(const float *__restrict__ logits, int ld, int limit, int k, int segments, float *cand_v, int32_t *cand_i) {
    __shared__ float best_v[8];
    __shared__ int best_i[8];
    spl_grid_begin();
    const int length = (limit + segments - 1) / segments, begin = blockIdx.y * length, end = min(limit, begin + length);
    const float *x = logits + size_t(blockIdx.x) * ld;
    float mine[64];
#pragma unroll
    for (int e = 0; e < 64; ++e) { const int i = begin + int(threadIdx.x) + 256 * e; mine[e] = i < end ? x[i] : -INFINITY; }
    float last_v = INFINITY; int last_i = -1;
    for (int round = 0; round < k; ++round) {
        float bv = -INFINITY; int bi = 0x7fffffff;
#pragma unroll
        for (int e = 0; e < 64; ++e) {
            const float v = mine[e];
            const int i = begin + int(threadIdx.x) + 256 * e;          // ascending in e: the first of equal values is the lowest index
            const bool after = v < last_v || (v == last_v && i > last_i);
            if (after && v > -INFINITY && v > bv) { bv = v; bi = i; }
        }
        spl_draft_block_best(bv, bi, best_v, best_i);
        const bool none = bi == 0x7fffffff;
        if (threadIdx.x == 0) {
            const size_t at = (size_t(blockIdx.x) * segments + blockIdx.y) * k + round;
            cand_v[at] = none ? -INFINITY : bv; cand_i[at] = none ? -1 : bi;
        }
        if (none) { last_v = -INFINITY; last_i = 0x7ffffffe; } else { last_v = bv; last_i = bi; }
    }
}
// Grid (rows), 256 threads; ids and values [rows][k]: fewer than k selectable values leave the reference's untouched slots, id 0 at -inf.
__global__ void __launch_bounds__(256)
spl_draft_topk_merge_kernel(const float *__restrict__ cand_v, const int32_t *__restrict__ cand_i, int count, int k, int32_t *ids, float *values) {
    __shared__ float best_v[8];
    __shared__ int best_i[8];
    spl_grid_begin();
    const float *cv = cand_v + size_t(blockIdx.x) * count;
    const int32_t *ci = cand_i + size_t(blockIdx.x) * count;
    float last_v = INFINITY; int last_i = -1;
    for (int round = 0; round < k; ++round) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int c = threadIdx.x; c < count; c += 256) {
            const float v = cv[c]; const int i = ci[c];
            const bool after = v < last_v || (v == last_v && i > last_i);
            if (i >= 0 && after && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
        }
        spl_draft_block_best(bv, bi, best_v, best_i);
        const bool none = bi == 0x7fffffff;
        if (threadIdx.x == 0) { ids[size_t(blockIdx.x) * k + round] = none ? 0 : bi; values[size_t(blockIdx.x) * k + round] = none ? -INFINITY : bv; }
        if (none) { last_v = -INFINITY; last_i = 0x7ffffffe; } else { last_v = bv; last_i = bi; }
    }
}
