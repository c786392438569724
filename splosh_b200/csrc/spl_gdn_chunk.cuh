// spl_gdn_chunk.cuh — the gated delta rule over long runs (prompt chunks) in chunks of 64 tokens.
//
// The reference has no chunk-parallel form: its production recurrence walks a run token by token
// (Sources/Shaders/candidates/gdn_b.metal:282-316; Sources/SploshModel/GdnLayer.swift:73-88 loops runToken). This file
// computes the same recurrence (the per-token form is spl_gdn_recurrence_kernel, Sources/Shaders/engine.metal:763-805)
// for runs of ordinary rows of at least SPL_GDN_CHUNK_MIN tokens, with the work of a chunk arranged as small matrix
// products so that a 2,048-row prompt chunk is not 2,048 dependent steps. Results agree with the per-token kernel up
// to the order of fp32 additions (the reference allows 5e-4 relative between its kernels and its CPU reference,
// Tests/SploshOracleTests/GdnCandidateTests.swift:41-47).
//
// With k^ = k * invK, q^ = q * invQ (the L2 norms), a = decay and b = beta of a token, the recurrence is
//     S_t = a_t S_{t-1} (I - b_t k^_t k^_t^T) + b_t v_t k^_t^T,     o_t = S_t q^_t          (S is [value][key])
// Write u_t = b_t (v_t - a_t S_{t-1} k^_t), so S_t = a_t S_{t-1} + u_t k^_t^T. Inside a chunk that starts from S_0, with
// g_t the product of the decays up to t:
//     u_t = b_t v_t - b_t g_t S_0 k^_t - sum_{s<t} A[t][s] u_s,   A[t][s] = b_t (g_t / g_s) (k^_t . k^_s)
// a unit lower triangular system: U = T (diag(b) V) - (T diag(b g) K^) S_0^T with T = (I + A)^-1. Then
//     o_t = g_t S_0 q^_t + sum_{s<=t} P[t][s] u_s,   P[t][s] = (g_t / g_s) (q^_t . k^_s)
//     S_C = g_C S_0 + sum_s (g_C / g_s) u_s k^_s^T
// Everything that does not depend on S_0 (T, W = T diag(b g) K^, Uv = T diag(b) V, P, g q^, (g_C / g) k^) is computed for
// all chunks in parallel by spl_gdn_chunk_prepare_kernel; spl_gdn_chunk_scan_kernel then walks a run's chunks in
// order, a block per (value head, slice of the value dimension): a row of S only ever meets its own column of U, so
// the slices are independent. spl_gdn_chunk_finish_kernel applies the gated RMSNorm (engine.metal:812-833) to whole
// heads and writes the output projection's operand.
#pragma once
#include "spl_gdn.cuh"

#define SPL_GDN_CHUNK 64           // tokens per chunk
#define SPL_GDN_CHUNK_MIN 512      // ordinary runs at least this long take the chunked path by default: below about five chunks the
                                   // per-token kernel is the faster one (a chunk costs it 83 us; the three kernels here 150 us + 50 us a chunk)
#define SPL_GDN_SLICES 8           // slices of the value dimension in the scan (16 values each)
#define SPL_GDN_SLICE (SPL_GDN_D / SPL_GDN_SLICES)
#define SPL_GDN_LD (SPL_GDN_D + 4)   // floats between rows of D in shared memory
#define SPL_GDN_PLD (SPL_GDN_CHUNK + 4)   // and between rows of a chunk x chunk matrix
// Floats of the per-(chunk, value head) record the prepare kernel leaves for the scan.
#define SPL_GDN_REC_W 0                                             // [64][128]  T diag(b g) K^
#define SPL_GDN_REC_UV (SPL_GDN_REC_W + 64 * 128)                   // [64][128]  T diag(b) V
#define SPL_GDN_REC_QG (SPL_GDN_REC_UV + 64 * 128)                  // [64][128]  g_t q^_t
#define SPL_GDN_REC_KD (SPL_GDN_REC_QG + 64 * 128)                  // [64][128]  (g_C / g_s) k^_s
#define SPL_GDN_REC_P (SPL_GDN_REC_KD + 64 * 128)                   // [64][64]   P, zero above the diagonal
#define SPL_GDN_REC_GC (SPL_GDN_REC_P + 64 * 64)                    // [4]        g_C and padding
#define SPL_GDN_REC_FLOATS (SPL_GDN_REC_GC + 4)

struct SplGdnChunkTables {
    const uint32_t *runs;       // [chunked runs][4]: slot, first row, length, journal entries to replay first
    const uint32_t *chunks;     // [chunks][4]: chunked run, first row, tokens (<= 64), index of the chunk in its run
    int run_count, chunk_count;
};

// The matrix products of the prepare and scan kernels run on the tensor cores' warp-level instruction (m16n8k8, tf32
// operands, fp32 accumulators): they are fp32 products of small matrices in a chain (a chunk's depend on the state the one
// before left; T on A), which the block-wide tcgen05 pipeline with its barriers does not suit, and on the CUDA cores they were bound by the shared-memory
// reads of their operands (a thread's four outputs took five 16-byte loads a step). Every operand is split in two tf32
// numbers, x = hi + lo with hi the upper 19 bits of x and lo those of x - hi, and a product is three instructions, lo x hi + hi x lo +
// hi x hi (lo x lo is below 2^-22 of the term): fp32 accuracy to within the rounding of the sums.
__device__ __forceinline__ void spl_split_tf32(float x, uint32_t &hi, uint32_t &lo) {
    // The instruction reads the upper 19 bits of an operand register: hi is x with the rest cleared, lo the exact remainder
    // (of which the instruction again reads the upper 19 bits: what it drops is below 2^-21 of x).
    hi = __float_as_uint(x) & 0xFFFFE000u;
    lo = __float_as_uint(x - __uint_as_float(hi));
}
// c += a b for a 16 x 8 (row-major) and b 8 x 8 (column-major) in the instruction's register layout: with g = lane / 4 and
// t = lane % 4, a = {(g, t), (g + 8, t), (g, t + 4), (g + 8, t + 4)}, b = {(k = t, n = g), (k = t + 4, n = g)},
// c = {(g, 2t), (g, 2t + 1), (g + 8, 2t), (g + 8, 2t + 1)}.
__device__ __forceinline__ void spl_mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void spl_mma_3xtf32(float (&c)[4], const float (&a)[4], const float (&b)[2]) {
    uint32_t ah[4], al[4], bh[2], bl[2];
#pragma unroll
    for (int i = 0; i < 4; ++i) spl_split_tf32(a[i], ah[i], al[i]);
#pragma unroll
    for (int i = 0; i < 2; ++i) spl_split_tf32(b[i], bh[i], bl[i]);
    spl_mma_tf32(c, al, bh); spl_mma_tf32(c, ah, bl); spl_mma_tf32(c, ah, bh);
}

#define SPL_GDN_KLD (SPL_GDN_D + 8)     // floats between rows of a D-wide matrix read as a product's k x n operand, whose lanes go four rows by eight columns
#define SPL_GDN_TLD (SPL_GDN_CHUNK + 4)   // floats between rows of T

// Grid (value heads, chunks), 256 threads. Everything of a chunk that does not depend on the state it starts from.
__global__ void __launch_bounds__(256)
spl_gdn_chunk_prepare_kernel(const float *__restrict__ act, const float *__restrict__ proj, const uint16_t *__restrict__ a_log,
                             const uint16_t *__restrict__ dt_bias, SplGdnChunkTables tables, float *records, SplGdnParams p) {
    spl_grid_begin();
    constexpr int D = SPL_GDN_D, C = SPL_GDN_CHUNK, LD = SPL_GDN_LD, KLD = SPL_GDN_KLD, TLD = SPL_GDN_TLD;      // shared rows are padded: rows read side by side fall in different banks
    extern __shared__ __align__(16) float spl_gdn_chunk_smem[];
    float *kh = spl_gdn_chunk_smem;            // [C][LD] k^
    float *x = kh + C * LD;                     // [C][LD] q^, then (rows KLD apart: the k x n operand of a product) b g k^, then b v
    float *am = x + C * KLD;                    // [C][TLD] A
    float *tm = am + C * TLD;                   // [C][TLD] T
    float *g = tm + C * TLD;                    // [C] log of the running decay product
    float *beta = g + C;                        // [C]
    float *scal = beta + C;                     // [C][2] invQ, invK
    float *eg = scal + 2 * C, *ed = eg + C;    // [C] each: g_t and g_C / g_t as numbers (g holds logarithms)
    const int h = blockIdx.x, chunk = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t first = tables.chunks[chunk * 4 + 1], count = tables.chunks[chunk * 4 + 2];
    const int VH = p.value_heads, KH = p.key_heads, hk = h / (VH / KH);
    float *rec = records + (size_t(chunk) * VH + h) * SPL_GDN_REC_FLOATS;
    const float neg_a = -expf(spl_bf16_to_float(a_log[h])), bias = spl_bf16_to_float(dt_bias[h]);

    // k and q of the chunk's tokens (zero rows past its end), their norms, the gates.
    for (int idx = tid; idx < C * (D / 4); idx += 256) {
        const int tt = idx / (D / 4), i4 = idx % (D / 4);
        float4 kv = make_float4(0, 0, 0, 0), qv = kv;
        if (tt < int(count)) {
            const float *row = act + size_t(first + tt) * p.channels;
            qv = *reinterpret_cast<const float4 *>(row + hk * D + i4 * 4);
            kv = *reinterpret_cast<const float4 *>(row + KH * D + hk * D + i4 * 4);
        }
        *reinterpret_cast<float4 *>(kh + tt * LD + i4 * 4) = kv;
        *reinterpret_cast<float4 *>(x + tt * LD + i4 * 4) = qv;
    }
    __syncthreads();
    for (int tt = warp; tt < C; tt += 8) {
        const float4 qv = *reinterpret_cast<const float4 *>(x + tt * LD + lane * 4), kv = *reinterpret_cast<const float4 *>(kh + tt * LD + lane * 4);
        const float qq = spl_warp_sum(qv.x * qv.x + qv.y * qv.y + qv.z * qv.z + qv.w * qv.w);
        const float kk = spl_warp_sum(kv.x * kv.x + kv.y * kv.y + kv.z * kv.z + kv.w * kv.w);
        if (lane == 0) {
            scal[tt * 2] = (1.0f / sqrtf(qq + 1e-6f)) * (1.0f / sqrtf(float(D)));
            scal[tt * 2 + 1] = 1.0f / sqrtf(kk + 1e-6f);
            float log_decay = 0.0f, b = 0.0f;
            if (tt < int(count)) {
                const size_t row = first + tt;
                const float xa = proj[row * p.proj_ld + p.a_offset + h] + bias;
                const float softplus = xa > 20.0f ? xa : logf(1.0f + expf(xa));
                log_decay = neg_a * softplus;                  // decay = exp(log_decay)
                b = spl_sigmoid(proj[row * p.proj_ld + p.b_offset + h]);
            }
            g[tt] = log_decay; beta[tt] = b;
        }
    }
    __syncthreads();
    if (tid == 0) { float run = 0.0f; for (int tt = 0; tt < C; ++tt) { run += g[tt]; g[tt] = run; } }
    for (int idx = tid; idx < C * D; idx += 256) { const int tt = idx / D, at = tt * LD + idx % D; kh[at] *= scal[tt * 2 + 1]; x[at] *= scal[tt * 2]; }
    __syncthreads();
    const float g_end = g[C - 1];      // rows past the chunk's end have log decay 0, so this is the last token's
    if (tid < C) { eg[tid] = expf(g[tid]); ed[tid] = expf(g_end - g[tid]); }
    __syncthreads();
    // A[t][s] = b_t (g_t / g_s) (k^_t . k^_s) below the diagonal; P[t][s] = (g_t / g_s) (q^_t . k^_s) on and below it (to the record).
    // Tiles of 16 tokens t by 8 tokens s on and below the diagonal (twenty of 32), both products of a tile together: they
    // share the k^_s operand.
    {
        const int gq = lane >> 2, tq = lane & 3;
        for (int tile = warp; tile < 20; tile += 8) {
            const int mt = tile < 2 ? 0 : tile < 6 ? 1 : tile < 12 ? 2 : 3, nt = tile - (mt == 0 ? 0 : mt == 1 ? 2 : mt == 2 ? 6 : 12);
            const int m0 = 16 * mt, n0 = 8 * nt;
            float ka[4] = {0.0f, 0.0f, 0.0f, 0.0f}, qa[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
            for (int k0 = 0; k0 < D; k0 += 8) {
                const float b[2] = {kh[(n0 + gq) * LD + k0 + tq], kh[(n0 + gq) * LD + k0 + tq + 4]};
                const float ak[4] = {kh[(m0 + gq) * LD + k0 + tq], kh[(m0 + gq + 8) * LD + k0 + tq], kh[(m0 + gq) * LD + k0 + tq + 4], kh[(m0 + gq + 8) * LD + k0 + tq + 4]};
                const float aq[4] = {x[(m0 + gq) * LD + k0 + tq], x[(m0 + gq + 8) * LD + k0 + tq], x[(m0 + gq) * LD + k0 + tq + 4], x[(m0 + gq + 8) * LD + k0 + tq + 4]};
                spl_mma_3xtf32(ka, ak, b);
                spl_mma_3xtf32(qa, aq, b);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int t = m0 + gq + 8 * (e >> 1), s = n0 + 2 * tq + (e & 1);
                const float ratio = s <= t ? expf(g[t] - g[s]) : 0.0f;
                am[t * TLD + s] = s < t ? beta[t] * ratio * ka[e] : 0.0f;
                rec[SPL_GDN_REC_P + t * C + s] = s <= t ? ratio * qa[e] : 0.0f;
            }
        }
        // The tiles above the diagonal are zero.
        for (int idx = tid; idx < C * C; idx += 256) {
            const int t = idx / C, s = idx % C;
            if ((s >> 3) > 2 * (t >> 4) + 1) { am[t * TLD + s] = 0.0f; rec[SPL_GDN_REC_P + idx] = 0.0f; }
        }
    }
    // g_t q^_t and (g_C / g_s) k^_s to the record while q^ is still in shared memory.
    for (int idx = tid; idx < C * D; idx += 256) {
        const int tt = idx / D, at = tt * LD + idx % D;
        rec[SPL_GDN_REC_QG + idx] = x[at] * eg[tt];
        rec[SPL_GDN_REC_KD + idx] = kh[at] * ed[tt];
    }
    if (tid == 0) rec[SPL_GDN_REC_GC] = expf(g_end);
    __syncthreads();
    // T = (I + A)^-1 in blocks of sixteen tokens. The four diagonal blocks by forward substitution, side by side, four
    // threads a column: T[t][c] = [t == c] - sum_{c <= s < t} A[t][s] T[s][c], the sum in four interleaved parts added in one
    // fixed order (a column's threads sit in one warp). Then the blocks below the diagonal, a sub-diagonal at a time:
    // T(i, j) = -T(i, i) sum_{j <= k < i} A(i, k) T(k, j), two small products a warp (a block's eight columns each).
    {
        const int blk = tid >> 6, c = (tid & 63) >> 2, part = tid & 3, base = 16 * blk;
        for (int t = 0; t < 16; ++t) {
            float acc = 0.0f;
            for (int sx = c + part; sx < t; sx += 4) acc -= am[(base + t) * TLD + base + sx] * tm[(base + sx) * TLD + base + c];
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (part == 0) tm[(base + t) * TLD + base + c] = t > c ? acc : t == c ? 1.0f : 0.0f;
            __syncwarp();
        }
        // The blocks above the diagonal are zero.
        for (int idx = tid; idx < C * C; idx += 256) { const int t = idx / C, sx = idx % C; if ((sx >> 4) > (t >> 4)) tm[t * TLD + sx] = 0.0f; }
    }
    __syncthreads();
    {
        const int gq = lane >> 2, tq = lane & 3;
        float *scratch = x + warp * 16 * 12;          // [16][12] a warp: the inner sum, handed from the first product's result layout to the second's operand layout (x is free here)
        for (int d = 1; d < 4; ++d) {
            if (warp < 2 * (4 - d)) {
                const int i = d + (warp >> 1), j = i - d, n0 = 16 * j + 8 * (warp & 1);
                float inner[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                for (int k0 = 16 * j; k0 < 16 * i; k0 += 8) {
                    const float a[4] = {am[(16 * i + gq) * TLD + k0 + tq], am[(16 * i + gq + 8) * TLD + k0 + tq], am[(16 * i + gq) * TLD + k0 + tq + 4], am[(16 * i + gq + 8) * TLD + k0 + tq + 4]};
                    const float b[2] = {tm[(k0 + tq) * TLD + n0 + gq], tm[(k0 + tq + 4) * TLD + n0 + gq]};
                    spl_mma_3xtf32(inner, a, b);
                }
                scratch[gq * 12 + 2 * tq] = inner[0]; scratch[gq * 12 + 2 * tq + 1] = inner[1];
                scratch[(gq + 8) * 12 + 2 * tq] = inner[2]; scratch[(gq + 8) * 12 + 2 * tq + 1] = inner[3];
                __syncwarp();
                float out[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int k0 = 0; k0 < 16; k0 += 8) {
                    const float a[4] = {tm[(16 * i + gq) * TLD + 16 * i + k0 + tq], tm[(16 * i + gq + 8) * TLD + 16 * i + k0 + tq], tm[(16 * i + gq) * TLD + 16 * i + k0 + tq + 4], tm[(16 * i + gq + 8) * TLD + 16 * i + k0 + tq + 4]};
                    const float b[2] = {scratch[(k0 + tq) * 12 + gq], scratch[(k0 + tq + 4) * 12 + gq]};
                    spl_mma_3xtf32(out, a, b);
                }
                tm[(16 * i + gq) * TLD + n0 + 2 * tq] = -out[0]; tm[(16 * i + gq) * TLD + n0 + 2 * tq + 1] = -out[1];
                tm[(16 * i + gq + 8) * TLD + n0 + 2 * tq] = -out[2]; tm[(16 * i + gq + 8) * TLD + n0 + 2 * tq + 1] = -out[3];
            }
            __syncthreads();
        }
    }
    // W = T diag(b g) K^ and Uv = T diag(b) V: x <- b g k^, product, then x <- b v, product.
    for (int pass = 0; pass < 2; ++pass) {
        for (int idx = tid; idx < C * (D / 4); idx += 256) {
            const int tt = idx / (D / 4), i4 = idx % (D / 4);
            float4 v = make_float4(0, 0, 0, 0);
            if (pass == 0) {
                const float f = beta[tt] * eg[tt];
                const float4 k4 = *reinterpret_cast<const float4 *>(kh + tt * LD + i4 * 4);
                v = make_float4(k4.x * f, k4.y * f, k4.z * f, k4.w * f);
            } else if (tt < int(count)) {
                const float f = beta[tt];
                const float4 v4 = *reinterpret_cast<const float4 *>(act + size_t(first + tt) * p.channels + 2 * KH * D + h * D + i4 * 4);
                v = make_float4(v4.x * f, v4.y * f, v4.z * f, v4.w * f);
            }
            *reinterpret_cast<float4 *>(x + tt * KLD + i4 * 4) = v;
        }
        __syncthreads();
        // out[t][i] = sum_{s<=t} T[t][s] x[s][i]: warp w has tokens 16 (w / 2) ... + 15 and columns 64 (w % 2) ... + 63, eight tiles
        // of eight columns that share the T operand; T is lower triangular, so the sum stops at the warp's last token.
        {
            const int gq = lane >> 2, tq = lane & 3, m0 = 16 * (warp >> 1), c0 = 64 * (warp & 1);
            float acc[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[nt][e] = 0.0f;
            for (int k0 = 0; k0 < m0 + 16; k0 += 8) {
                const float a[4] = {tm[(m0 + gq) * TLD + k0 + tq], tm[(m0 + gq + 8) * TLD + k0 + tq], tm[(m0 + gq) * TLD + k0 + tq + 4], tm[(m0 + gq + 8) * TLD + k0 + tq + 4]};
                uint32_t ah[4], al[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) spl_split_tf32(a[e], ah[e], al[e]);
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
                    uint32_t bh[2], bl[2];
                    spl_split_tf32(x[(k0 + tq) * KLD + c0 + 8 * nt + gq], bh[0], bl[0]);
                    spl_split_tf32(x[(k0 + tq + 4) * KLD + c0 + 8 * nt + gq], bh[1], bl[1]);
                    spl_mma_tf32(acc[nt], al, bh); spl_mma_tf32(acc[nt], ah, bl); spl_mma_tf32(acc[nt], ah, bh);
                }
            }
            float *out = rec + (pass == 0 ? SPL_GDN_REC_W : SPL_GDN_REC_UV);
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                *reinterpret_cast<float2 *>(out + (m0 + gq) * D + c0 + 8 * nt + 2 * tq) = make_float2(acc[nt][0], acc[nt][1]);
                *reinterpret_cast<float2 *>(out + (m0 + gq + 8) * D + c0 + 8 * nt + 2 * tq) = make_float2(acc[nt][2], acc[nt][3]);
            }
        }
        __syncthreads();
    }
}
__host__ __device__ constexpr size_t spl_gdn_chunk_prepare_smem() {
    return sizeof(float) * (SPL_GDN_CHUNK * SPL_GDN_LD + SPL_GDN_CHUNK * SPL_GDN_KLD + 2 * SPL_GDN_CHUNK * SPL_GDN_TLD + 6 * SPL_GDN_CHUNK);
}

#define SPL_GDN_ULD 24                  // floats between rows of U (sixteen values a row): the same pattern over its rows

// Grid (value heads, chunked runs, SPL_GDN_SLICES), 256 threads. The run's chunks in order over one slice of the value
// dimension: the slice of S in shared memory, U and O of the chunk formed from the prepared record. Eight warps: for the
// 64 x 16 products (U, O) warp w has tokens 16 (w / 2) ... + 15 and values 8 (w % 2) ... + 7 of the slice; for the state's
// 16 x 128 update it has columns 16 w ... + 15.
__global__ void __launch_bounds__(256)
spl_gdn_chunk_scan_kernel(const float *__restrict__ records, SplGdnChunkTables tables, float *state, const float *__restrict__ journal,
                          float *o_raw, SplGdnParams p) {
    spl_grid_begin();
    constexpr int D = SPL_GDN_D, C = SPL_GDN_CHUNK, SL = SPL_GDN_SLICE, LD = SPL_GDN_LD, PLD = SPL_GDN_PLD, KLD = SPL_GDN_KLD, ULD = SPL_GDN_ULD, SLD = D + 4;
    extern __shared__ __align__(16) float spl_gdn_scan_smem[];
    // One buffer holds W, then g q^ (rows LD apart), then Kd (rows KLD apart) in turn: three blocks share an SM, and the 384
    // blocks of a 48-head run are resident at once.
    float *w_s = spl_gdn_scan_smem;           // [C][KLD] W, then g q^, then Kd
    float *p_s = w_s + C * KLD;                // [C][PLD] P
    float *s_s = p_s + C * PLD;                // [SL][SLD] the slice of the state (rows padded)
    float *u_s = s_s + SL * SLD;               // [C][ULD] U
    const int h = blockIdx.x, run = blockIdx.y, slice = blockIdx.z, tid = threadIdx.x;
    const int VH = p.value_heads;
    const uint32_t slot = tables.runs[run * 4], length = tables.runs[run * 4 + 2], pending = tables.runs[run * 4 + 3];
    float *stored = state + ((size_t(slot) * VH + h) * D + slice * SL) * D;
    for (int idx = tid; idx < SL * (D / 4); idx += 256) {
        const int j = idx / (D / 4), i4 = idx % (D / 4);
        *reinterpret_cast<float4 *>(s_s + j * SLD + i4 * 4) = *reinterpret_cast<const float4 *>(stored + j * D + i4 * 4);
    }
    __syncthreads();
    // Journal entries accepted from the run before are replayed first, with the update's one expression (engine.metal:654-659).
    if (pending) {
        const float *jhead = journal + (size_t(slot) * SPL_JOURNAL_ROWS * VH + h) * SPL_JOURNAL_WIDTH;
        for (uint32_t e = 0; e < pending; ++e) {
            const float *entry = jhead + size_t(e) * VH * SPL_JOURNAL_WIDTH;
            const float decay = entry[2 * D];
            for (int idx = tid; idx < SL * D; idx += 256) {
                const int j = idx / D, i = idx % D;
                s_s[j * SLD + i] = __fmaf_rn(s_s[j * SLD + i], decay, __fmul_rn(entry[i], entry[D + slice * SL + j]));
            }
            __syncthreads();
        }
    }
    // The first chunk of the run in the chunk table: chunks of a run are consecutive there.
    int chunk = 0;
    for (; chunk < tables.chunk_count; ++chunk) if (tables.chunks[chunk * 4] == uint32_t(run)) break;
    const int chunks = int((length + C - 1) / C);
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int m0 = 16 * (warp >> 1), n0 = 8 * (warp & 1);          // the warp's tokens and values of the slice in the 64 x 16 products
    for (int n = 0; n < chunks; ++n, ++chunk) {
        const float *rec = records + (size_t(chunk) * VH + h) * SPL_GDN_REC_FLOATS;
        const uint32_t first = tables.chunks[chunk * 4 + 1], count = tables.chunks[chunk * 4 + 2];
        for (int idx = tid; idx < C * (D / 4); idx += 256)
            *reinterpret_cast<float4 *>(w_s + (idx / (D / 4)) * LD + (idx % (D / 4)) * 4) = reinterpret_cast<const float4 *>(rec + SPL_GDN_REC_W)[idx];
        for (int idx = tid; idx < C * (C / 4); idx += 256)
            *reinterpret_cast<float4 *>(p_s + (idx / (C / 4)) * PLD + (idx % (C / 4)) * 4) = reinterpret_cast<const float4 *>(rec + SPL_GDN_REC_P)[idx];
        const float g_end = rec[SPL_GDN_REC_GC];
        // Uv of the thread's four outputs (tokens m0 + g and + 8, values n0 + 2t and + 1), asked for before the product.
        const float2 uv0 = *reinterpret_cast<const float2 *>(rec + SPL_GDN_REC_UV + (m0 + g) * D + slice * SL + n0 + 2 * t);
        const float2 uv1 = *reinterpret_cast<const float2 *>(rec + SPL_GDN_REC_UV + (m0 + g + 8) * D + slice * SL + n0 + 2 * t);
        __syncthreads();
        // x[token][value] = sum_i X[token][i] S[value][i] for X = W or g q^ in w_s.
        auto against_state = [&](float (&acc)[4]) {
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] = 0.0f;
#pragma unroll 4
            for (int k0 = 0; k0 < D; k0 += 8) {
                const float a[4] = {w_s[(m0 + g) * LD + k0 + t], w_s[(m0 + g + 8) * LD + k0 + t], w_s[(m0 + g) * LD + k0 + t + 4], w_s[(m0 + g + 8) * LD + k0 + t + 4]};
                const float b[2] = {s_s[(n0 + g) * SLD + k0 + t], s_s[(n0 + g) * SLD + k0 + t + 4]};
                spl_mma_3xtf32(acc, a, b);
            }
        };
        // U[t][j] = Uv[t][j] - sum_i W[t][i] S[j][i]
        float acc[4];
        against_state(acc);
        *reinterpret_cast<float2 *>(u_s + (m0 + g) * ULD + n0 + 2 * t) = make_float2(uv0.x - acc[0], uv0.y - acc[1]);
        *reinterpret_cast<float2 *>(u_s + (m0 + g + 8) * ULD + n0 + 2 * t) = make_float2(uv1.x - acc[2], uv1.y - acc[3]);
        __syncthreads();
        for (int idx = tid; idx < C * (D / 4); idx += 256)
            *reinterpret_cast<float4 *>(w_s + (idx / (D / 4)) * LD + (idx % (D / 4)) * 4) = reinterpret_cast<const float4 *>(rec + SPL_GDN_REC_QG)[idx];
        __syncthreads();
        // O[t][j] = sum_i (g q^)[t][i] S[j][i] + sum_{s<=t} P[t][s] U[s][j]   (P is zero above the diagonal: its tiles there are left out)
        float o[4];
        against_state(o);
        for (int k0 = 0; k0 < m0 + 16; k0 += 8) {
            const float a[4] = {p_s[(m0 + g) * PLD + k0 + t], p_s[(m0 + g + 8) * PLD + k0 + t], p_s[(m0 + g) * PLD + k0 + t + 4], p_s[(m0 + g + 8) * PLD + k0 + t + 4]};
            const float b[2] = {u_s[(k0 + t) * ULD + n0 + g], u_s[(k0 + t + 4) * ULD + n0 + g]};
            spl_mma_3xtf32(o, a, b);
        }
        if (m0 + g < int(count))
            *reinterpret_cast<float2 *>(o_raw + size_t(first + m0 + g) * (size_t(VH) * D) + h * D + slice * SL + n0 + 2 * t) = make_float2(o[0], o[1]);
        if (m0 + g + 8 < int(count))
            *reinterpret_cast<float2 *>(o_raw + size_t(first + m0 + g + 8) * (size_t(VH) * D) + h * D + slice * SL + n0 + 2 * t) = make_float2(o[2], o[3]);
        __syncthreads();          // every thread has finished with g q^
        for (int idx = tid; idx < C * (D / 4); idx += 256)
            *reinterpret_cast<float4 *>(w_s + (idx / (D / 4)) * KLD + (idx % (D / 4)) * 4) = reinterpret_cast<const float4 *>(rec + SPL_GDN_REC_KD)[idx];
        __syncthreads();
        // S[j][i] = g_C S[j][i] + sum_s U[s][j] Kd[s][i]: the warp's sixteen columns, two tiles of eight.
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int c0 = 16 * warp + 8 * half;
            const float2 lo = *reinterpret_cast<const float2 *>(s_s + g * SLD + c0 + 2 * t), hi = *reinterpret_cast<const float2 *>(s_s + (g + 8) * SLD + c0 + 2 * t);
            float sacc[4] = {g_end * lo.x, g_end * lo.y, g_end * hi.x, g_end * hi.y};
#pragma unroll 4
            for (int k0 = 0; k0 < C; k0 += 8) {
                const float a[4] = {u_s[(k0 + t) * ULD + g], u_s[(k0 + t) * ULD + g + 8], u_s[(k0 + t + 4) * ULD + g], u_s[(k0 + t + 4) * ULD + g + 8]};
                const float b[2] = {w_s[(k0 + t) * KLD + c0 + g], w_s[(k0 + t + 4) * KLD + c0 + g]};
                spl_mma_3xtf32(sacc, a, b);
            }
            *reinterpret_cast<float2 *>(s_s + g * SLD + c0 + 2 * t) = make_float2(sacc[0], sacc[1]);
            *reinterpret_cast<float2 *>(s_s + (g + 8) * SLD + c0 + 2 * t) = make_float2(sacc[2], sacc[3]);
        }
        __syncthreads();
    }
    for (int idx = tid; idx < SL * (D / 4); idx += 256) {
        const int j = idx / (D / 4), i4 = idx % (D / 4);
        *reinterpret_cast<float4 *>(stored + j * D + i4 * 4) = *reinterpret_cast<const float4 *>(s_s + j * SLD + i4 * 4);
    }
}
__host__ __device__ constexpr size_t spl_gdn_chunk_scan_smem() {
    return sizeof(float) * (SPL_GDN_CHUNK * SPL_GDN_KLD + SPL_GDN_CHUNK * SPL_GDN_PLD + SPL_GDN_SLICE * (SPL_GDN_D + 4) + SPL_GDN_CHUNK * SPL_GDN_ULD);
}

// Gated RMSNorm of whole heads and the bf16 operand of the output projection with its per-64 sums
// (engine.metal:812-833), for the rows of the chunked runs. Grid (value heads, chunks), 256 threads: a warp a token.
__global__ void __launch_bounds__(256)
spl_gdn_chunk_finish_kernel(const float *__restrict__ o_raw, const float *__restrict__ proj, const uint16_t *__restrict__ norm_weight,
                            SplGdnChunkTables tables, SplOperand core, SplGdnParams p) {
    spl_grid_begin();
    constexpr int D = SPL_GDN_D;
    const int h = blockIdx.x, chunk = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t first = tables.chunks[chunk * 4 + 1], count = tables.chunks[chunk * 4 + 2];
    const uint2 w = *reinterpret_cast<const uint2 *>(norm_weight + lane * 4);
    for (uint32_t tt = warp; tt < count; tt += 8) {
        const size_t row = first + tt;
        const float4 z = *reinterpret_cast<const float4 *>(proj + row * p.proj_ld + p.z_offset + h * D + lane * 4);
        const float4 ov = *reinterpret_cast<const float4 *>(o_raw + row * (size_t(p.value_heads) * D) + h * D + lane * 4);
        const float inv = 1.0f / sqrtf(spl_warp_sum(ov.x * ov.x + ov.y * ov.y + ov.z * ov.z + ov.w * ov.w) / float(D) + p.eps);
        const float r0 = spl_bf16_to_float(uint16_t(w.x)) * ov.x * inv * spl_silu_exact(z.x);
        const float r1 = spl_bf16_to_float(uint16_t(w.x >> 16)) * ov.y * inv * spl_silu_exact(z.y);
        const float r2 = spl_bf16_to_float(uint16_t(w.y)) * ov.z * inv * spl_silu_exact(z.z);
        const float r3 = spl_bf16_to_float(uint16_t(w.y >> 16)) * ov.w * inv * spl_silu_exact(z.w);
        const uint16_t b0 = spl_float_to_bf16(r0), b1 = spl_float_to_bf16(r1), b2 = spl_float_to_bf16(r2), b3 = spl_float_to_bf16(r3);
        *reinterpret_cast<uint2 *>(core.values + core.at(int(row), spl_gdn_out_head(p, h) * D + lane * 4)) =
            spl_operand_pack4(spl_bf16_to_float(b0), spl_bf16_to_float(b1), spl_bf16_to_float(b2), spl_bf16_to_float(b3));
        float gsum = (spl_bf16_to_float(b0) + spl_bf16_to_float(b1)) + (spl_bf16_to_float(b2) + spl_bf16_to_float(b3));
#pragma unroll
        for (int o2 = 8; o2 > 0; o2 >>= 1) gsum += __shfl_xor_sync(0xffffffffu, gsum, o2);
        if ((lane & 15) == 0) core.put_sum(int(row), spl_gdn_out_head(p, h) * 2 + (lane >> 4), gsum);
    }
}
