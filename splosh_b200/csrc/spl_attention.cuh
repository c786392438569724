// spl_attention.cuh — gated GQA attention over the paged int8 KV cache with ragged rows.
//
// Stands in for encodeFull's kernels (Sources/SploshRuntime/Engine.swift:2167-2290):
// sp_attn_q_prepare_na and sp_attn_kv_store_i8 (Sources/Shaders/engine_na.metal:1222-1266,
// 2044-2094), the span scan sp_attn_scan_i8_r48c64s8 (Sources/Shaders/candidates/attn_scan_r.metal:46-202)
// and sp_attn_merge (Sources/Shaders/engine.metal:2218-2255).
//
// HBM layout (per attention layer; pages of 256 tokens shared by all slots):
//   k codes  [page][kv head][token 256][head_dim]  int8
//   v codes  [page][kv head][head_dim][token 256]  int8   (transposed: P.V reads 16 consecutive
//                                                          tokens of one channel as one 16-byte load)
//   k scale, v scale  [page][kv head][token 256]   fp32, value = scale * code
// A K or V vector is symmetric int8: scale = max|x| / 127 (1 when all zero),
// code = clamp(rint(x / scale), -127, 127) (engine_na.metal:2084-2093).
#pragma once
#include "spl_common.cuh"
#include "spl_gemm_tc.cuh"

struct SplAttnParams {
    int rows, live, heads, kv_heads, head_dim, rotary, max_pages;
    int proj_ld, k_offset, v_offset;      // columns of the fused q|k|v projection; q head h at h * 2 * head_dim
    int spans, pages_per_span;
    float eps, scale;
};

// Query rows: per-head RMSNorm, RoPE on the first `rotary` dims (NeoX pairing), fp16
// (engine_na.metal:1236-1262). Key/value rows: K the same norm + RoPE, V verbatim, both to int8
// with one scale per vector (engine_na.metal:2055-2093). inv_freq[i] = theta^(-2i / rotary) is
// computed once on the host in double precision.
// Grid (heads + kv_heads, rows), 128 threads.
__global__ void __launch_bounds__(128)
spl_attn_prepare_kernel(const float *__restrict__ proj, const uint16_t *__restrict__ q_norm, const uint16_t *__restrict__ k_norm,
                        const float *__restrict__ inv_freq, const uint32_t *__restrict__ row_slot, const uint32_t *__restrict__ row_pos,
                        const uint32_t *__restrict__ page_table, __half *q_out, int8_t *k_codes, float *k_scale, int8_t *v_codes,
                        float *v_scale, SplAttnParams p) {
    __shared__ float xs[256], red[4], red2[4];
    const int row = blockIdx.y, hd = p.head_dim, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool is_q = int(blockIdx.x) < p.heads;
    if (is_q && row >= p.live) return;
    const int head = is_q ? blockIdx.x : blockIdx.x - p.heads;
    const float *x = proj + size_t(row) * p.proj_ld + (is_q ? head * 2 * hd : p.k_offset + head * hd);
    const uint16_t *w = is_q ? q_norm : k_norm;
    float ss = 0.0f;
    for (int i = tid; i < hd; i += 128) { const float v = x[i]; ss += v * v; }
    ss = spl_warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    const float inv = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / float(hd) + p.eps);
    for (int i = tid; i < hd; i += 128) xs[i] = x[i] * inv * spl_bf16_to_float(w[i]);
    __syncthreads();
    const uint32_t position = row_pos[row];
    const int half = p.rotary / 2;
    float vals[2], vmax = 0.0f;
    for (int n = 0, i = tid; i < hd; i += 128, ++n) {
        float v = xs[i];
        if (i < p.rotary) {
            const int slot = i < half ? i : i - half;
            const float angle = float(position) * inv_freq[slot];
            const float paired = xs[i < half ? i + half : i - half];
            v = v * cosf(angle) + (i < half ? -paired : paired) * sinf(angle);
        }
        vals[n] = v; vmax = fmaxf(vmax, fabsf(v));
    }
    if (is_q) {
        for (int n = 0, i = tid; i < hd; i += 128, ++n) q_out[(size_t(row) * p.heads + head) * hd + i] = __float2half_rn(vals[n]);
        return;
    }
    // K and V to int8.
    const float *vx = proj + size_t(row) * p.proj_ld + p.v_offset + head * hd;
    float vv[2], vvmax = 0.0f;
    for (int n = 0, i = tid; i < hd; i += 128, ++n) { vv[n] = vx[i]; vvmax = fmaxf(vvmax, fabsf(vv[n])); }
    vmax = spl_warp_max(vmax); vvmax = spl_warp_max(vvmax);
    __syncthreads();
    if (lane == 0) { red[warp] = vmax; red2[warp] = vvmax; }
    __syncthreads();
    const float khi = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3])), vhi = fmaxf(fmaxf(red2[0], red2[1]), fmaxf(red2[2], red2[3]));
    const float ks = khi > 0.0f ? __fdiv_rn(khi, 127.0f) : 1.0f, vs = vhi > 0.0f ? __fdiv_rn(vhi, 127.0f) : 1.0f;
    const uint32_t page = page_table[size_t(row_slot[row]) * p.max_pages + position / SPL_PAGE_TOKENS];
    const size_t vec = size_t(page) * p.kv_heads + head;
    const uint32_t in_page = position % SPL_PAGE_TOKENS;
    for (int n = 0, i = tid; i < hd; i += 128, ++n) {
        k_codes[(vec * SPL_PAGE_TOKENS + in_page) * hd + i] = int8_t(fminf(127.0f, fmaxf(-127.0f, rintf(__fdiv_rn(vals[n], ks)))));
        v_codes[(vec * hd + i) * SPL_PAGE_TOKENS + in_page] = int8_t(fminf(127.0f, fmaxf(-127.0f, rintf(__fdiv_rn(vv[n], vs)))));
    }
    if (tid == 0) { k_scale[vec * SPL_PAGE_TOKENS + in_page] = ks; v_scale[vec * SPL_PAGE_TOKENS + in_page] = vs; }
}

// Four int8 in a word -> two half2 (exact): fp16 0x6400 | u is 1024 + u, with u = x + 128.
__device__ __forceinline__ void spl_s8x4_to_h2x2(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const uint32_t u = w ^ 0x80808080u;
    uint32_t a = __byte_perm(u, 0x64646464u, 0x4140), b = __byte_perm(u, 0x64646464u, 0x4342);
    const __half2 off = __floats2half2_rn(1152.0f, 1152.0f);
    __half2 ha = __hsub2(*reinterpret_cast<__half2 *>(&a), off), hb = __hsub2(*reinterpret_cast<__half2 *>(&b), off);
    lo = *reinterpret_cast<uint32_t *>(&ha); hi = *reinterpret_cast<uint32_t *>(&hb);
}

#define SPL_ATTN_C 64                 // tokens per chunk
#define SPL_ATTN_PS (SPL_ATTN_C + 4)  // row of the probability tile in shared memory (halves)
#define SPL_ATTN_PSCALE 4096.0f       // keeps small probabilities normal in fp16; removed at the end

// The span scan. One block per (kv head, span of pages, attention block of <= 8 rows). The
// block's queries (rows x the heads sharing the kv head) are M <= 16 MT rows of both products:
//   scores[M x 64 tokens] = Q[M x head_dim] K^T      fp16 x int8 (as fp16), fp32 accumulate
//   out[M x head_dim]    += P[M x 64] V               P = bf16(p * vScale) held as fp16 x 4096
// with an online softmax across chunks of 64 tokens: s = acc * kScale[token] * scale, visible when
// token < position + 1 of the query's row (attn_scan_r.metal:107-160). Each block leaves a partial
// [reference, sum p, out[head_dim]] per query and span; spl_attn_merge_kernel combines the spans.
// Warp w takes tokens 16w..16w+15 of a chunk in the score product and channels
// w * head_dim / 4 ... in the value product; probabilities cross warps through shared memory.
// The reduction (head) dimension and the token dimension are each fed to the tensor cores in a
// permuted order that lets a lane load 16 consecutive bytes of K (or of transposed V) and use
// them for four k16 steps; the query / probability fragments are read with the same permutation.
// Grid (kv_heads * spans, blocks), 128 threads.
template <int MT, int HD>
__global__ void __launch_bounds__(128)
spl_attn_scan_kernel(const __half *__restrict__ q, const uint32_t *__restrict__ blocks, const uint32_t *__restrict__ row_slot,
                     const uint32_t *__restrict__ row_pos, const uint32_t *__restrict__ page_table, const int8_t *__restrict__ k_codes,
                     const float *__restrict__ k_scale, const int8_t *__restrict__ v_codes, const float *__restrict__ v_scale,
                     float *partials, SplAttnParams p) {
    constexpr int M = 16 * MT, QS = HD + 4, NQ = HD / 64, NVW = HD / 32;   // NVW: n8 tiles of this warp's HD / 4 channels
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half *Qs = reinterpret_cast<__half *>(smem_raw);                        // [M][QS]
    __half *Ps = Qs + M * QS;                                                 // [M][SPL_ATTN_PS]
    float *smax = reinterpret_cast<float *>(Ps + M * SPL_ATTN_PS);            // [4][M]
    float *ssum = smax + 4 * M;                                               // [4][M]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g8 = lane >> 2, t = lane & 3;
    const int kv_head = blockIdx.x % p.kv_heads, span = blockIdx.x / p.kv_heads, block = blockIdx.y;
    const int per_kv = p.heads / p.kv_heads;
    const uint32_t r0 = blocks[block * 2], count = blocks[block * 2 + 1];
    const uint32_t first_pos = row_pos[r0], max_visible = first_pos + count;
    const int pages = int((max_visible + SPL_PAGE_TOKENS - 1) / SPL_PAGE_TOKENS);
    const int first_page = span * p.pages_per_span, last_page = min(pages, first_page + p.pages_per_span);
    const size_t table_base = size_t(row_slot[r0]) * p.max_pages;

    // Queries into shared memory, zero for padding rows.
    for (int idx = tid; idx < M * (HD / 4); idx += 128) {
        const int m = idx / (HD / 4), c4 = idx % (HD / 4);
        const int rb = m / per_kv, hq = m % per_kv;
        uint2 v = make_uint2(0, 0);
        if (rb < int(count) && int(r0) + rb < p.live)
            v = *reinterpret_cast<const uint2 *>(q + (size_t(r0 + rb) * p.heads + kv_head * per_kv + hq) * HD + c4 * 4);
        *reinterpret_cast<uint2 *>(Qs + m * QS + c4 * 4) = v;
    }
    // Per-thread view of its query rows: m = 16 mt + g8 + 8 hr.
    uint32_t limit[MT][2];
    float ref[MT][2], total[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            const int m = 16 * mt + g8 + 8 * hr, rb = m / per_kv;
            limit[mt][hr] = (rb < int(count) && int(r0) + rb < p.live) ? first_pos + rb + 1 : 0u;
            ref[mt][hr] = -INFINITY; total[mt][hr] = 0.0f;
        }
    float acc[MT][NVW][4] = {};               // value product: this warp's HD / 4 channels
    __syncthreads();

    for (int pg = first_page; pg < last_page; ++pg) {
        const size_t vec = size_t(page_table[table_base + pg]) * p.kv_heads + kv_head;
        for (int chunk = 0; chunk < SPL_PAGE_TOKENS / SPL_ATTN_C; ++chunk) {
            const uint32_t t0 = pg * SPL_PAGE_TOKENS + chunk * SPL_ATTN_C;
            if (t0 >= max_visible) break;
            const size_t token_base = vec * SPL_PAGE_TOKENS + chunk * SPL_ATTN_C;
            // ---- scores for this warp's 16 tokens
            float s[MT][2][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int jn = 0; jn < 2; ++jn)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[mt][jn][e] = 0.0f;
#pragma unroll
            for (int ci = 0; ci < NQ; ++ci) {
                uint4 kc[2];
#pragma unroll
                for (int jn = 0; jn < 2; ++jn)
                    kc[jn] = __ldg(reinterpret_cast<const uint4 *>(k_codes + (token_base + 16 * warp + 8 * jn + g8) * HD + (t + 4 * ci) * 16));
#pragma unroll
                for (int sx = 0; sx < 4; ++sx) {
                    uint32_t b[2][2];
#pragma unroll
                    for (int jn = 0; jn < 2; ++jn) {
                        const uint32_t w = sx == 0 ? kc[jn].x : sx == 1 ? kc[jn].y : sx == 2 ? kc[jn].z : kc[jn].w;
                        spl_s8x4_to_h2x2(w, b[jn][0], b[jn][1]);
                    }
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const __half *qa = Qs + (16 * mt + g8) * QS + (t + 4 * ci) * 16 + 4 * sx;
                        const uint2 lo = *reinterpret_cast<const uint2 *>(qa), hi = *reinterpret_cast<const uint2 *>(qa + 8 * QS);
                        const uint32_t a[4] = {lo.x, hi.x, lo.y, hi.y};
                        spl_mma_f16(s[mt][0], a, b[0][0], b[0][1]);
                        spl_mma_f16(s[mt][1], a, b[1][0], b[1][1]);
                    }
                }
            }
            // ---- softmax bookkeeping. Element (jn, e): token 16 warp + 8 jn + 2 t + (e & 1), row hr = e >> 1.
            float ksc[2][2], vsc[2][2];
#pragma unroll
            for (int jn = 0; jn < 2; ++jn) {
                const float2 k2 = __ldg(reinterpret_cast<const float2 *>(k_scale + token_base + 16 * warp + 8 * jn + 2 * t));
                const float2 v2 = __ldg(reinterpret_cast<const float2 *>(v_scale + token_base + 16 * warp + 8 * jn + 2 * t));
                ksc[jn][0] = k2.x; ksc[jn][1] = k2.y; vsc[jn][0] = v2.x; vsc[jn][1] = v2.y;
            }
            const uint32_t tok = t0 + 16 * warp + 2 * t;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int hr = 0; hr < 2; ++hr) {
                    float top = -INFINITY;
#pragma unroll
                    for (int jn = 0; jn < 2; ++jn)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const bool seen = tok + 8 * jn + e < limit[mt][hr];
                            const float v = seen ? s[mt][jn][2 * hr + e] * ksc[jn][e] * p.scale : -INFINITY;
                            s[mt][jn][2 * hr + e] = v;
                            top = fmaxf(top, v);
                        }
                    top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 1));
                    top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 2));
                    if (t == 0) smax[warp * M + 16 * mt + g8 + 8 * hr] = top;
                }
            __syncthreads();
            float factor[MT][2];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int hr = 0; hr < 2; ++hr) {
                    const int m = 16 * mt + g8 + 8 * hr;
                    const float top = fmaxf(fmaxf(smax[m], smax[M + m]), fmaxf(smax[2 * M + m], smax[3 * M + m]));
                    const float next = fmaxf(ref[mt][hr], top);
                    float sum = 0.0f;
#pragma unroll
                    for (int jn = 0; jn < 2; ++jn) {
                        float pw[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float v = s[mt][jn][2 * hr + e];
                            const bool seen = v != -INFINITY;
                            const float prob = seen ? expf(v - next) : 0.0f;
                            sum += prob;
                            pw[e] = seen ? spl_round_bf16(prob * vsc[jn][e]) * SPL_ATTN_PSCALE : 0.0f;
                        }
                        *reinterpret_cast<__half2 *>(Ps + m * SPL_ATTN_PS + 16 * warp + 8 * jn + 2 * t) = __floats2half2_rn(pw[0], pw[1]);
                    }
                    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                    if (t == 0) ssum[warp * M + m] = sum;
                    factor[mt][hr] = (ref[mt][hr] == -INFINITY || next == ref[mt][hr]) ? 1.0f : expf(ref[mt][hr] - next);
                    ref[mt][hr] = next;
                }
            __syncthreads();
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int hr = 0; hr < 2; ++hr) {
                    const int m = 16 * mt + g8 + 8 * hr;
                    total[mt][hr] = total[mt][hr] * factor[mt][hr] + (((ssum[m] + ssum[M + m]) + ssum[2 * M + m]) + ssum[3 * M + m]);
#pragma unroll
                    for (int nj = 0; nj < NVW; ++nj) { acc[mt][nj][2 * hr] *= factor[mt][hr]; acc[mt][nj][2 * hr + 1] *= factor[mt][hr]; }
                }
            // ---- value product for this warp's channels
#pragma unroll
            for (int nj = 0; nj < NVW; ++nj) {
                const int d = warp * (HD / 4) + 8 * nj + g8;
                const uint4 vc = __ldg(reinterpret_cast<const uint4 *>(v_codes + (vec * HD + d) * SPL_PAGE_TOKENS + chunk * SPL_ATTN_C + t * 16));
#pragma unroll
                for (int sx = 0; sx < 4; ++sx) {
                    const uint32_t w = sx == 0 ? vc.x : sx == 1 ? vc.y : sx == 2 ? vc.z : vc.w;
                    uint32_t b0, b1;
                    spl_s8x4_to_h2x2(w, b0, b1);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const __half *pa = Ps + (16 * mt + g8) * SPL_ATTN_PS + t * 16 + 4 * sx;
                        const uint2 lo = *reinterpret_cast<const uint2 *>(pa), hi = *reinterpret_cast<const uint2 *>(pa + 8 * SPL_ATTN_PS);
                        const uint32_t a[4] = {lo.x, hi.x, lo.y, hi.y};
                        spl_mma_f16(acc[mt][nj], a, b0, b1);
                    }
                }
            }
            // The next chunk's probabilities must not overwrite the tile while a warp still reads it;
            // the barrier after its score product covers smax, this one covers Ps and ssum.
            __syncthreads();
        }
    }

    // Partials. acc element e of (mt, nj): row hr = e >> 1, channel warp * HD/4 + 8 nj + 2 t + (e & 1).
    const int record = HD + 2;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            const int m = 16 * mt + g8 + 8 * hr, rb = m / per_kv, hq = m % per_kv;
            if (rb >= int(count) || int(r0) + rb >= p.live) continue;
            float *partial = partials + ((size_t(r0 + rb) * p.heads + kv_head * per_kv + hq) * p.spans + span) * record;
            if (warp == 0 && t == 0) { partial[0] = ref[mt][hr]; partial[1] = total[mt][hr]; }
#pragma unroll
            for (int nj = 0; nj < NVW; ++nj) {
                float2 v = make_float2(acc[mt][nj][2 * hr] * (1.0f / SPL_ATTN_PSCALE), acc[mt][nj][2 * hr + 1] * (1.0f / SPL_ATTN_PSCALE));
                *reinterpret_cast<float2 *>(partial + 2 + warp * (HD / 4) + 8 * nj + 2 * t) = v;
            }
        }
}

// Merge span partials by log-sum-exp, apply the sigmoid output gate, round to the bf16 operand of
// the output projection and emit its per-64 sums (engine.metal:2218-2255). Grid (heads, live rows), head_dim threads.
__global__ void spl_attn_merge_kernel(const float *__restrict__ partials, const float *__restrict__ proj, SplOperand core, SplAttnParams p) {
    __shared__ float warp_sums[8];
    const int head = blockIdx.x, row = blockIdx.y, j = threadIdx.x, hd = p.head_dim, record = hd + 2;
    const float *base = partials + (size_t(row) * p.heads + head) * p.spans * record;
    float top = -INFINITY;
    for (int s = 0; s < p.spans; ++s) top = fmaxf(top, base[s * record]);
    float sum = 0.0f, acc = 0.0f;
    for (int s = 0; s < p.spans; ++s) {
        const float weight = expf(base[s * record] - top);
        if (weight > 0.0f) { sum += base[s * record + 1] * weight; acc += base[s * record + 2 + j] * weight; }
    }
    const float gate = proj[size_t(row) * p.proj_ld + head * 2 * hd + hd + j];
    const uint16_t bits = spl_float_to_bf16((acc / sum) * spl_sigmoid(gate));
    reinterpret_cast<__half *>(core.values)[core.at(row, head * hd + j)] = __float2half_rn(spl_bf16_to_float(bits));
    const float wsum = spl_warp_sum(spl_bf16_to_float(bits));
    if ((j & 31) == 0) warp_sums[j >> 5] = wsum;
    __syncthreads();
    if ((j & 63) == 0) core.put_sum(row, (head * hd + j) / 64, warp_sums[j >> 5] + warp_sums[(j >> 5) + 1]);
}
