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

// Grid (value heads, chunks), 256 threads. Everything of a chunk that does not depend on the state it starts from.
__global__ void __launch_bounds__(256)
spl_gdn_chunk_prepare_kernel(const float *__restrict__ act, const float *__restrict__ proj, const uint16_t *__restrict__ a_log,
                             const uint16_t *__restrict__ dt_bias, SplGdnChunkTables tables, float *records, SplGdnParams p) {
    spl_grid_begin();
    constexpr int D = SPL_GDN_D, C = SPL_GDN_CHUNK, LD = SPL_GDN_LD;      // shared rows of D floats are LD apart: rows read side by side fall in different banks
    extern __shared__ __align__(16) float spl_gdn_chunk_smem[];
    float *kh = spl_gdn_chunk_smem;            // [C][LD] k^
    float *x = kh + C * LD;                     // [C][LD] q^, then b g k^, then b v
    float *am = x + C * LD;                     // [C][C] A, then P
    float *tm = am + C * C;                     // [C][C + 1] T (rows padded against bank conflicts)
    float *g = tm + C * (C + 1);                // [C] log of the running decay product
    float *beta = g + C;                        // [C]
    float *scal = beta + C;                     // [C][2] invQ, invK
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
    // A[t][s] = b_t (g_t / g_s) (k^_t . k^_s) below the diagonal; P[t][s] = (g_t / g_s) (q^_t . k^_s) on and below it (to the record).
    for (int idx = tid; idx < C * C; idx += 256) {
        const int t = idx / C, s = idx % C;
        float ka = 0.0f, qa = 0.0f;
        if (s <= t) {
            const float4 *kt = reinterpret_cast<const float4 *>(kh + t * LD), *ks = reinterpret_cast<const float4 *>(kh + s * LD), *qt = reinterpret_cast<const float4 *>(x + t * LD);
#pragma unroll 8
            for (int i = 0; i < D / 4; ++i) {
                const float4 a4 = kt[i], b4 = ks[i], c4 = qt[i];
                ka += a4.x * b4.x + a4.y * b4.y + a4.z * b4.z + a4.w * b4.w;
                qa += c4.x * b4.x + c4.y * b4.y + c4.z * b4.z + c4.w * b4.w;
            }
        }
        const float ratio = s <= t ? expf(g[t] - g[s]) : 0.0f;
        am[idx] = s < t ? beta[t] * ratio * ka : 0.0f;
        rec[SPL_GDN_REC_P + idx] = s <= t ? ratio * qa : 0.0f;
    }
    // g_t q^_t and (g_C / g_s) k^_s to the record while q^ is still in shared memory.
    for (int idx = tid; idx < C * D; idx += 256) {
        const int tt = idx / D, at = tt * LD + idx % D;
        rec[SPL_GDN_REC_QG + idx] = x[at] * expf(g[tt]);
        rec[SPL_GDN_REC_KD + idx] = kh[at] * expf(g_end - g[tt]);
    }
    if (tid == 0) rec[SPL_GDN_REC_GC] = expf(g_end);
    __syncthreads();
    // T = (I + A)^-1 by forward substitution, four threads a column: T[t][c] = [t == c] - sum_{s<t} A[t][s] T[s][c], the sum
    // in four interleaved parts added in one fixed order. A column's threads sit in one warp.
    {
        const int c = tid >> 2, part = tid & 3;
        for (int t = 0; t < C; ++t) {
            float acc = 0.0f;
            for (int s = c + part; s < t; s += 4) acc -= am[t * C + s] * tm[s * (C + 1) + c];      // T is lower triangular: T[s][c] = 0 for s < c
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (part == 0) tm[t * (C + 1) + c] = t > c ? acc : t == c ? 1.0f : 0.0f;
            __syncwarp();
        }
    }
    __syncthreads();
    // W = T diag(b g) K^ and Uv = T diag(b) V: x <- b g k^, product, then x <- b v, product.
    for (int pass = 0; pass < 2; ++pass) {
        for (int idx = tid; idx < C * (D / 4); idx += 256) {
            const int tt = idx / (D / 4), i4 = idx % (D / 4);
            float4 v = make_float4(0, 0, 0, 0);
            if (pass == 0) {
                const float f = beta[tt] * expf(g[tt]);
                const float4 k4 = *reinterpret_cast<const float4 *>(kh + tt * LD + i4 * 4);
                v = make_float4(k4.x * f, k4.y * f, k4.z * f, k4.w * f);
            } else if (tt < int(count)) {
                const float f = beta[tt];
                const float4 v4 = *reinterpret_cast<const float4 *>(act + size_t(first + tt) * p.channels + 2 * KH * D + h * D + i4 * 4);
                v = make_float4(v4.x * f, v4.y * f, v4.z * f, v4.w * f);
            }
            *reinterpret_cast<float4 *>(x + tt * LD + i4 * 4) = v;
        }
        __syncthreads();
        // out[t][i] = sum_{s<=t} T[t][s] x[s][i]: a thread four rows t and four columns i (rows t, t + 16, t + 32, t + 48: even work).
        {
            const int ig = tid & 31, tg = tid >> 5;       // columns 4 ig .. + 3; rows tg, tg + 8, ... (8 of them, in two rounds of four)
            for (int round = 0; round < 2; ++round) {
                float4 acc[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) acc[r] = make_float4(0, 0, 0, 0);
                const int t_max = tg + 8 * (4 * round + 3);
                for (int s = 0; s <= t_max; ++s) {
                    const float4 xv = *reinterpret_cast<const float4 *>(x + s * LD + ig * 4);
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const int t = tg + 8 * (4 * round + r);
                        const float w = s <= t ? tm[t * (C + 1) + s] : 0.0f;
                        acc[r].x += w * xv.x; acc[r].y += w * xv.y; acc[r].z += w * xv.z; acc[r].w += w * xv.w;
                    }
                }
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int t = tg + 8 * (4 * round + r);
                    *reinterpret_cast<float4 *>(rec + (pass == 0 ? SPL_GDN_REC_W : SPL_GDN_REC_UV) + t * D + ig * 4) = acc[r];
                }
            }
        }
        __syncthreads();
    }
}
__host__ __device__ constexpr size_t spl_gdn_chunk_prepare_smem() {
    return sizeof(float) * (2 * SPL_GDN_CHUNK * SPL_GDN_LD + SPL_GDN_CHUNK * SPL_GDN_CHUNK + SPL_GDN_CHUNK * (SPL_GDN_CHUNK + 1) + 4 * SPL_GDN_CHUNK);
}

// Grid (value heads, chunked runs, SPL_GDN_SLICES), 256 threads. The run's chunks in order over one slice of the value
// dimension: the slice of S in shared memory, U and O of the chunk formed from the prepared record.
__global__ void __launch_bounds__(256)
spl_gdn_chunk_scan_kernel(const float *__restrict__ records, SplGdnChunkTables tables, float *state, const float *__restrict__ journal,
                          float *o_raw, SplGdnParams p) {
    spl_grid_begin();
    constexpr int D = SPL_GDN_D, C = SPL_GDN_CHUNK, SL = SPL_GDN_SLICE, LD = SPL_GDN_LD, PLD = SPL_GDN_PLD;
    extern __shared__ __align__(16) float spl_gdn_scan_smem[];
    // One [C][LD] buffer holds W, then g q^, then Kd in turn: with 64 KB a block three blocks share an SM, and the 384
    // blocks of a 48-head run are resident at once (with a buffer each for W and g q^ it was two to an SM and a second
    // wave of 88 blocks doubled the kernel's time).
    float *w_s = spl_gdn_scan_smem;           // [C][LD] W, then g q^, then Kd
    float *p_s = w_s + C * LD;                 // [C][PLD] P
    float *s_s = p_s + C * PLD;                // [SL][D + 4] the slice of the state (rows padded)
    float *u_s = s_s + SL * (D + 4);           // [C][SL] U
    const int h = blockIdx.x, run = blockIdx.y, slice = blockIdx.z, tid = threadIdx.x;
    const int VH = p.value_heads;
    const uint32_t slot = tables.runs[run * 4], length = tables.runs[run * 4 + 2], pending = tables.runs[run * 4 + 3];
    float *stored = state + ((size_t(slot) * VH + h) * D + slice * SL) * D;
    for (int idx = tid; idx < SL * (D / 4); idx += 256) {
        const int j = idx / (D / 4), i4 = idx % (D / 4);
        *reinterpret_cast<float4 *>(s_s + j * (D + 4) + i4 * 4) = *reinterpret_cast<const float4 *>(stored + j * D + i4 * 4);
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
                s_s[j * (D + 4) + i] = __fmaf_rn(s_s[j * (D + 4) + i], decay, __fmul_rn(entry[i], entry[D + slice * SL + j]));
            }
            __syncthreads();
        }
    }
    // The first chunk of the run in the chunk table: chunks of a run are consecutive there.
    int chunk = 0;
    for (; chunk < tables.chunk_count; ++chunk) if (tables.chunks[chunk * 4] == uint32_t(run)) break;
    const int chunks = int((length + C - 1) / C);
    const int tq = tid >> 2, jq = tid & 3;          // U and O: token tq, values jq, jq + 4, jq + 8, jq + 12 of the slice (the four lanes of a token read
                                                    // neighbouring rows of S, which the rows' padding puts in different banks)
    for (int n = 0; n < chunks; ++n, ++chunk) {
        const float *rec = records + (size_t(chunk) * VH + h) * SPL_GDN_REC_FLOATS;
        const uint32_t first = tables.chunks[chunk * 4 + 1], count = tables.chunks[chunk * 4 + 2];
        for (int idx = tid; idx < C * (D / 4); idx += 256)
            *reinterpret_cast<float4 *>(w_s + (idx / (D / 4)) * LD + (idx % (D / 4)) * 4) = reinterpret_cast<const float4 *>(rec + SPL_GDN_REC_W)[idx];
        for (int idx = tid; idx < C * (C / 4); idx += 256)
            *reinterpret_cast<float4 *>(p_s + (idx / (C / 4)) * PLD + (idx % (C / 4)) * 4) = reinterpret_cast<const float4 *>(rec + SPL_GDN_REC_P)[idx];
        const float g_end = rec[SPL_GDN_REC_GC];
        __syncthreads();
        // U[t][j] = Uv[t][j] - sum_i W[t][i] S[j][i];  O0[t][j] = sum_i (g q^)[t][i] S[j][i]
        float u[4], o[4];
        {
#pragma unroll
            for (int r = 0; r < 4; ++r) u[r] = rec[SPL_GDN_REC_UV + tq * D + slice * SL + jq + 4 * r];
#pragma unroll
            for (int r = 0; r < 4; ++r) o[r] = 0.0f;
            for (int i = 0; i < D; i += 4) {
                const float4 wv = *reinterpret_cast<const float4 *>(w_s + tq * LD + i);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float4 sv = *reinterpret_cast<const float4 *>(s_s + (jq + 4 * r) * (D + 4) + i);
                    u[r] -= wv.x * sv.x + wv.y * sv.y + wv.z * sv.z + wv.w * sv.w;
                }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) u_s[tq * SL + jq + 4 * r] = u[r];
        }
        __syncthreads();
        for (int idx = tid; idx < C * (D / 4); idx += 256)
            *reinterpret_cast<float4 *>(w_s + (idx / (D / 4)) * LD + (idx % (D / 4)) * 4) = reinterpret_cast<const float4 *>(rec + SPL_GDN_REC_QG)[idx];
        __syncthreads();
        for (int i = 0; i < D; i += 4) {
            const float4 qv = *reinterpret_cast<const float4 *>(w_s + tq * LD + i);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float4 sv = *reinterpret_cast<const float4 *>(s_s + (jq + 4 * r) * (D + 4) + i);
                o[r] += qv.x * sv.x + qv.y * sv.y + qv.z * sv.z + qv.w * sv.w;
            }
        }
        // O[t][j] = O0 + sum_{s<=t} P[t][s] U[s][j]; meanwhile the record's Kd replaces W in shared memory.
        for (int s = 0; s <= tq; ++s) {
            const float w = p_s[tq * PLD + s];
#pragma unroll
            for (int r = 0; r < 4; ++r) o[r] += w * u_s[s * SL + jq + 4 * r];
        }
        if (tq < int(count))
#pragma unroll
            for (int r = 0; r < 4; ++r) o_raw[size_t(first + tq) * (size_t(VH) * D) + h * D + slice * SL + jq + 4 * r] = o[r];
        __syncthreads();          // every thread has finished with g q^
        for (int idx = tid; idx < C * (D / 4); idx += 256)
            *reinterpret_cast<float4 *>(w_s + (idx / (D / 4)) * LD + (idx % (D / 4)) * 4) = reinterpret_cast<const float4 *>(rec + SPL_GDN_REC_KD)[idx];
        __syncthreads();
        // S[j][i] = g_C S[j][i] + sum_s U[s][j] Kd[s][i]: a thread one value row j and eight columns i.
        {
            const int j = tid >> 4, i0 = (tid & 15) * 4;      // columns i0 .. + 3 and 64 + i0 .. + 3: sixteen lanes read 16-byte pieces side by side
            float4 lo = *reinterpret_cast<const float4 *>(s_s + j * (D + 4) + i0), hi = *reinterpret_cast<const float4 *>(s_s + j * (D + 4) + 64 + i0);
            float acc[8] = {g_end * lo.x, g_end * lo.y, g_end * lo.z, g_end * lo.w, g_end * hi.x, g_end * hi.y, g_end * hi.z, g_end * hi.w};
            for (int s = 0; s < C; ++s) {
                const float us = u_s[s * SL + j];
                const float4 k0 = *reinterpret_cast<const float4 *>(w_s + s * LD + i0), k1 = *reinterpret_cast<const float4 *>(w_s + s * LD + 64 + i0);
                acc[0] += us * k0.x; acc[1] += us * k0.y; acc[2] += us * k0.z; acc[3] += us * k0.w;
                acc[4] += us * k1.x; acc[5] += us * k1.y; acc[6] += us * k1.z; acc[7] += us * k1.w;
            }
            *reinterpret_cast<float4 *>(s_s + j * (D + 4) + i0) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            *reinterpret_cast<float4 *>(s_s + j * (D + 4) + 64 + i0) = make_float4(acc[4], acc[5], acc[6], acc[7]);
        }
        __syncthreads();
    }
    for (int idx = tid; idx < SL * (D / 4); idx += 256) {
        const int j = idx / (D / 4), i4 = idx % (D / 4);
        *reinterpret_cast<float4 *>(stored + j * D + i4 * 4) = *reinterpret_cast<const float4 *>(s_s + j * (D + 4) + i4 * 4);
    }
}
__host__ __device__ constexpr size_t spl_gdn_chunk_scan_smem() {
    return sizeof(float) * (SPL_GDN_CHUNK * SPL_GDN_LD + SPL_GDN_CHUNK * SPL_GDN_PLD + SPL_GDN_SLICE * (SPL_GDN_D + 4) + SPL_GDN_CHUNK * SPL_GDN_SLICE);
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
