// spl_attention.cuh — gated GQA attention over the paged int8 KV cache with ragged rows.
//
// Stands in for encodeFull's kernels (Sources/SploshRuntime/Engine.swift:2167-2290):
// sp_attn_q_prepare_na and sp_attn_kv_store_i8 (Sources/Shaders/engine_na.metal:1222-1266,
// 2044-2094), the span scan sp_attn_scan_i8_r48c64s8 (Sources/Shaders/candidates/attn_scan_r.metal:46-202)
// and sp_attn_merge (Sources/Shaders/engine.metal:2218-2255).
//
// HBM layout (per attention layer; pages of 256 tokens shared by all slots). A page of one kv head is two
// chunks of 128 tokens; a chunk of K, of V and of each scale array is contiguous, so one bulk copy brings it
// to shared memory, and inside a chunk the 16-byte pieces are ordered so that the thread that converts a
// token's K (or a channel's V) reads consecutive pieces with its neighbours (no bank conflicts):
//   k codes  [page][kv head][chunk 2][channel block head_dim/16][token 128][16 channels]   int8
//   v codes  [page][kv head][chunk 2][token block 8][channel head_dim][16 tokens]          int8
//   k scale, v scale  [page][kv head][token 256]   fp32, value = scale * code
// A K or V vector is symmetric int8: scale = max|x| / 127 (1 when all zero),
// code = clamp(rint(x / scale), -127, 127) (engine_na.metal:2084-2093), stored as the byte code + 128.
#pragma once
#include "spl_common.cuh"
#include "spl_gemm_tc.cuh"

// Index of channel `d` of token `in_page` in the code arrays; vec = page * kv_heads + kv_head.
__host__ __device__ __forceinline__ size_t spl_k_code_index(size_t vec, uint32_t in_page, int d, int hd) {
    return vec * (SPL_PAGE_TOKENS * size_t(hd)) + size_t(in_page >> 7) * (128 * size_t(hd)) + size_t(d >> 4) * 2048 + (in_page & 127) * 16 + (d & 15);
}
__host__ __device__ __forceinline__ size_t spl_v_code_index(size_t vec, uint32_t in_page, int d, int hd) {
    return vec * (SPL_PAGE_TOKENS * size_t(hd)) + size_t(in_page >> 7) * (128 * size_t(hd)) + size_t((in_page & 127) >> 4) * (16 * size_t(hd)) + size_t(d) * 16 + (in_page & 15);
}

// A code is stored as code + 128 in a byte (offset binary): the scan turns four bytes into fp16 with two byte
// permutes and two subtractions, without a sign fix.
__host__ __device__ __forceinline__ int8_t spl_code_byte(float code) { return int8_t(uint8_t(int(code) + 128)); }
__host__ __device__ __forceinline__ int8_t spl_code_value(int8_t byte) { return int8_t(int(uint8_t(byte)) - 128); }

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
    spl_grid_begin();
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
        k_codes[spl_k_code_index(vec, in_page, i, hd)] = spl_code_byte(fminf(127.0f, fmaxf(-127.0f, rintf(__fdiv_rn(vals[n], ks)))));
        v_codes[spl_v_code_index(vec, in_page, i, hd)] = spl_code_byte(fminf(127.0f, fmaxf(-127.0f, rintf(__fdiv_rn(vv[n], vs)))));
    }
    if (tid == 0) { k_scale[vec * SPL_PAGE_TOKENS + in_page] = ks; v_scale[vec * SPL_PAGE_TOKENS + in_page] = vs; }
}

// ---- the span scan on the tensor cores ----------------------------------------------------------
// One block per (kv head, span of pages, attention block of <= 8 rows). The block's queries (rows x the
// PER_KV heads that share the kv head) are the N = NQ columns of both products, which run TRANSPOSED so that
// the int8 cache is the tensor cores' A operand, converted to fp16 on its way into tensor memory and never
// written back to shared memory:
//   S^T[128 tokens x NQ]   = K[128 x head_dim] Q^T          A = K (tensor memory, lane = token), B = Q (shared)
//   O^T[head_dim x NQ]    += V^T[head_dim x 128] P^T        A = V^T (tensor memory, lane = channel), B = P (shared)
// with the online softmax of attn_scan_r.metal:107-160 between them: s = acc * kScale[token] * scale, visible
// when token < position + 1 of the query's row, P = bf16(p * vScale[token]) (held as fp16 x 4096, exact for
// normal values). A softmax thread owns one token of the chunk, so a query's maximum over the chunk is a
// warp reduction (redux) plus a four-way exchange; sums stay per thread until the end of the span.
// When a maximum moves, the softmax warps rescale O^T in tensor memory before the next value product.
//
// Warps: 0-3, 16-19 (and 20-23 with three groups) softmax (a share of the queries each), rescale and the partial's output,
// 4-7 K -> tensor memory, 8-11 V -> tensor memory, 12 and 15 copies (bulk copies of whole 128-token chunks into rings),
// 13 and 14 tensor-core issue of the score and the value product. Every wait is bounded.
// Tensor memory (512 columns): S two buffers of NQ columns at 0, O two halves of NQ columns at 96, K operand a ring
// of three 64-column slots (128 channels each) at 192, V operand two 64-column halves at 384.
#define SPL_ATTN_CH 128               // tokens per chunk
#define SPL_ATTN_HEADROOM 6.0f        // a score may exceed its query's reference by this much (log2) before the reference is raised
#define SPL_ATTN_PSCALE 64.0f         // 4096 / 2^headroom: keeps small probabilities normal in fp16 and large ones finite; removed at the end
struct SplTrue { static constexpr bool value = true; };
struct SplFalse { static constexpr bool value = false; };
// Softmax warp groups: a group has a share of the queries (the columns of S^T) and four warps, one per quarter of the chunk's
// tokens (a warp reaches the tensor-memory lanes of its index mod 4). The softmax warps are the block's critical path (busy
// nine tenths of a chunk's time with two groups), so a 48-column block has three groups of 16 columns.
__host__ __device__ constexpr int spl_attn_groups(int nq) { return nq % 48 == 0 ? 3 : 2; }
__host__ __device__ constexpr int spl_attn_threads(int nq) { return 384 + 128 * spl_attn_groups(nq); }

__host__ __device__ constexpr int spl_attn_nq(int per_kv) { return (8 * per_kv + 15) / 16 * 16; }
// Shared-memory rings of 128-token chunks. K is converted as soon as it lands, so two stages do; V waits for the
// probabilities of its chunk, so it has three and the copies still run two chunks ahead; scales are small.
__host__ __device__ constexpr int spl_attn_k_stages(int hd) { return hd >= 256 ? 2 : 3; }
__host__ __device__ constexpr int spl_attn_v_stages(int hd) { return hd >= 256 ? 3 : 4; }
#define SPL_ATTN_S_STAGES 4
__host__ __device__ constexpr size_t spl_attn_smem_bytes(int hd, int nq) {
    return 1024 + size_t(spl_attn_k_stages(hd) + spl_attn_v_stages(hd)) * SPL_ATTN_CH * hd + SPL_ATTN_S_STAGES * 1024 + size_t(hd / 64) * nq * 128 /* Q */ + size_t(2) * 2 * nq * 128 /* P */
           + size_t(2) * 4 * nq * 4 /* chunk maxima */ + size_t(4) * nq * 8 /* per-warp reference and factor */ + size_t(4) * nq * 4 /* sums */ + 512 /* barriers */;
}

__device__ __forceinline__ void spl_tc_st32(uint32_t taddr, const uint32_t *r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                   "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
                   "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
                   "r"(r[30]), "r"(r[31]) : "memory");
}
// Eight columns of this warp's 32 lanes; the load and its wait are one statement (see spl_tc_ld16).
__device__ __forceinline__ void spl_tc_ld8(uint32_t (&r)[8], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 "tcgen05.wait::ld.sync.aligned;\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr));
}
__device__ __forceinline__ void spl_tc_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void spl_fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ float spl_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float spl_redux_max(float v) {
    float m;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;\n" : "=f"(m) : "f"(v));
    return m;
}
// Sixteen stored codes (a 16-byte piece, each byte u = code + 128) -> eight registers of fp16 pairs (exact): fp16 0x6400 | u is 1024 + u.
__device__ __forceinline__ void spl_s8x16_to_h2x8(const uint4 &piece, uint32_t *out) {
    const __half2 off = __floats2half2_rn(1152.0f, 1152.0f);
    const uint32_t w4[4] = {piece.x, piece.y, piece.z, piece.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t u = w4[i];
        uint32_t a = __byte_perm(u, 0x64646464u, 0x4140), b = __byte_perm(u, 0x64646464u, 0x4342);
        const __half2 ha = __hsub2(*reinterpret_cast<__half2 *>(&a), off), hb = __hsub2(*reinterpret_cast<__half2 *>(&b), off);
        out[2 * i] = *reinterpret_cast<const uint32_t *>(&ha); out[2 * i + 1] = *reinterpret_cast<const uint32_t *>(&hb);
    }
}
// Byte offset of element (row, k) in a K-major operand tile of 128-byte rows with the 128-byte swizzle; k < 64.
__device__ __forceinline__ uint32_t spl_sw128_offset(int row, int k) {
    return uint32_t((row >> 3) * 1024 + (row & 7) * 128 + ((((k >> 3) ^ (row & 7)) & 7) << 4) + (k & 7) * 2);
}

template <int HD, int PER_KV>
__global__ void __launch_bounds__(spl_attn_threads(spl_attn_nq(PER_KV)), 1)
spl_attn_scan_kernel(const __half *__restrict__ q, const uint32_t *__restrict__ blocks, const uint32_t *__restrict__ row_slot,
                     const uint32_t *__restrict__ row_pos, const uint32_t *__restrict__ page_table, const int8_t *__restrict__ k_codes,
                     const float *__restrict__ k_scale, const int8_t *__restrict__ v_codes, const float *__restrict__ v_scale,
                     float *partials, SplAttnParams p, int *error_flag) {
    spl_grid_begin();
    constexpr int NQ = spl_attn_nq(PER_KV), GROUPS = spl_attn_groups(NQ), NH = NQ / GROUPS, SW = 4 * GROUPS, NTHREADS = spl_attn_threads(NQ), CH = SPL_ATTN_CH, NKS = spl_attn_k_stages(HD), NVS = spl_attn_v_stages(HD), NSS = SPL_ATTN_S_STAGES;
    constexpr int HALVES = HD / 128, QGROUPS = HD / 64, CHUNK_BYTES = CH * HD, QTILE = NQ * 128, PTILE = 2 * NQ * 128;
    constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
    static_assert(NH % 8 == 0 && NQ <= 48, "softmax groups of NQ / GROUPS queries, eight at a time; tensor memory holds two S and two O of NQ columns below column 192");
    extern __shared__ unsigned char spl_attn_smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(spl_attn_smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char *q_tile = smem;                                   // [QGROUPS][NQ rows x 128 B]   B operand of the score product
    unsigned char *p_tile = q_tile + QGROUPS * QTILE;               // [2][2 token groups][NQ x 128 B] B operand of the value product
    unsigned char *k_ring = p_tile + 2 * PTILE;                     // [NKS][K chunk]
    unsigned char *v_ring = k_ring + size_t(NKS) * CHUNK_BYTES;     // [NVS][V chunk]
    unsigned char *s_ring = v_ring + size_t(NVS) * CHUNK_BYTES;     // [NSS][k scales 512 B | v scales 512 B]
    float *xmax = reinterpret_cast<float *>(s_ring + NSS * 1024);          // [2][4 token quarters][NQ]
    float *ref_next = xmax + 2 * 4 * NQ, *ref_factor = ref_next + 4 * NQ;  // [4][NQ] each: running reference (log2 domain) and the chunk's rescale factor, a copy per softmax warp
    float *xsum = ref_factor + 4 * NQ;                                     // [4][NQ]
    uint64_t *bars = reinterpret_cast<uint64_t *>(xsum + 4 * NQ);
    uint64_t *full_k = bars, *empty_k = full_k + NKS, *full_v = empty_k + NKS, *empty_v = full_v + NVS, *full_sc = empty_v + NVS, *empty_sc = full_sc + NSS,
             *ka_full = empty_sc + NSS, *ka_free = ka_full + 3, *va_full = ka_free + 3,
             *va_free = va_full + 2, *s_full = va_free + 2, *s_free = s_full + 2, *p_full = s_free + 2, *p_free = p_full + 2, *o_done = p_free + 2, *x_full = o_done + 2, *y_full = x_full + 2 * GROUPS, *sum_full = y_full + 2 * GROUPS;      // x_full, y_full: [group][chunk parity]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sum_full + 1);
    int *xflag = reinterpret_cast<int *>(tmem_slot + 1);          // [group][2] last chunk (+1) of each parity whose scores called for a raise

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kv_head = blockIdx.x % p.kv_heads, span = blockIdx.x / p.kv_heads, block = blockIdx.y;
    const uint32_t r0 = blocks[block * 2], count = blocks[block * 2 + 1];
    const uint32_t first_pos = row_pos[r0], max_visible = first_pos + count;
    const int valid_rows = min(int(count), p.live - int(r0));                   // rows of the block that are computed
    const int pages = int((max_visible + SPL_PAGE_TOKENS - 1) / SPL_PAGE_TOKENS);
    const int first_page = span * p.pages_per_span, last_page = min(pages, first_page + p.pages_per_span);
    const uint32_t token_begin = uint32_t(first_page) * SPL_PAGE_TOKENS;
    const uint32_t token_end = last_page > first_page ? min(uint32_t(last_page) * SPL_PAGE_TOKENS, max_visible) : token_begin;
    const int chunks = int((token_end - token_begin + CH - 1) / CH);
    const size_t table_base = size_t(row_slot[r0]) * p.max_pages;

    if (tid == 0) {
        for (int i = 0; i < NKS; ++i) { spl_mbar_init(&full_k[i], 1); spl_mbar_init(&empty_k[i], 4); }        // the K warps
        for (int i = 0; i < NVS; ++i) { spl_mbar_init(&full_v[i], 1); spl_mbar_init(&empty_v[i], 4); }        // the V warps
        for (int i = 0; i < NSS; ++i) { spl_mbar_init(&full_sc[i], 1); spl_mbar_init(&empty_sc[i], SW); }      // the softmax warps
        for (int i = 0; i < 3; ++i) { spl_mbar_init(&ka_full[i], 4); spl_mbar_init(&ka_free[i], 1); }
        for (int i = 0; i < 2; ++i) {
            spl_mbar_init(&va_full[i], 4); spl_mbar_init(&va_free[i], 1);
            spl_mbar_init(&s_full[i], 1); spl_mbar_init(&s_free[i], SW); spl_mbar_init(&p_full[i], SW); spl_mbar_init(&p_free[i], 1);
            spl_mbar_init(&o_done[i], 1);
            // A group's references are its own columns': its four warps agree among themselves whether to raise them.
            for (int grp = 0; grp < GROUPS; ++grp) { spl_mbar_init(&x_full[grp * 2 + i], 4); spl_mbar_init(&y_full[grp * 2 + i], 4); xflag[grp * 2 + i] = 0; }
        }
        spl_mbar_init(sum_full, SW);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 13) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(spl_smem_addr(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    // Queries into the swizzled operand tile, zero for padding rows: 16-byte pieces of eight channels.
    for (int idx = tid; idx < NQ * (HD / 8); idx += NTHREADS) {
        const int m = idx / (HD / 8), piece = idx % (HD / 8);
        const int rb = m / PER_KV, hq = m % PER_KV, g = piece >> 3, k8 = piece & 7;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (rb < valid_rows)
            v = *reinterpret_cast<const uint4 *>(q + (size_t(r0 + rb) * p.heads + kv_head * PER_KV + hq) * HD + piece * 8);
        *reinterpret_cast<uint4 *>(q_tile + g * QTILE + spl_sw128_offset(m, k8 * 8)) = v;
    }
    spl_fence_proxy_async();
    spl_tc_fence_before();
    __syncthreads();
    spl_tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_s = tmem, tmem_o = tmem + 96, tmem_ka = tmem + 192, tmem_va = tmem + 384;
    bool ok = true;
    // Debug trace (builds with -DSPL_TRACE only): cycles per chunk that one thread of each role of block (0, 0) spends in
    // its waits and its work.
#ifdef SPL_TRACE
    const bool trace = blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && error_flag[1] == 0x7ACE && (error_flag[2] & 0x200);
    long long tt[8] = {0, 0, 0, 0, 0, 0, 0, 0}, t_mark = 0;
#define SPL_A0() do { if (trace) t_mark = clock64(); } while (0)
#define SPL_A1(k) do { if (trace) { const long long now__ = clock64(); tt[k] += now__ - t_mark; t_mark = now__; } } while (0)
#define SPL_AOUT(base, n) do { if (trace && chunks > 0) for (int k__ = 0; k__ < n; ++k__) error_flag[base + k__] = int(tt[k__] / chunks); } while (0)
#define SPL_ACHUNKS() do { if (trace) error_flag[55] = chunks; } while (0)
#else
#define SPL_A0() do { } while (0)
#define SPL_A1(k) do { } while (0)
#define SPL_AOUT(base, n) do { } while (0)
#define SPL_ACHUNKS() do { } while (0)
#endif

    if (warp == 12 || warp == 15) {
        // ---- copies: a chunk = 128 tokens of one kv head = K, V and their scales, each contiguous in the pool. Warp 12 brings
        // K and the scales, warp 15 brings V, so that a full V ring does not hold back the K that the score product needs next.
        if (lane == 0) {
            for (int i = 0; i < chunks && ok; ++i) {
                const uint32_t token0 = token_begin + uint32_t(i) * CH;
                const size_t vec = size_t(page_table[table_base + token0 / SPL_PAGE_TOKENS]) * p.kv_heads + kv_head;
                const int sub = int(token0 % SPL_PAGE_TOKENS) / CH;
                SPL_A0();
                if (warp == 12) {
                    const int st = i % NKS, ss = i % NSS;
                    ok = spl_mbar_wait(&empty_k[st], ((i / NKS) & 1) ^ 1) && spl_mbar_wait(&empty_sc[ss], ((i / NSS) & 1) ^ 1);
                    SPL_A1(0);
                    if (!ok) break;
                    spl_mbar_expect_tx(&full_k[st], CHUNK_BYTES);
                    spl_bulk_g2s(k_ring + size_t(st) * CHUNK_BYTES, k_codes + vec * (SPL_PAGE_TOKENS * HD) + size_t(sub) * CHUNK_BYTES, CHUNK_BYTES, &full_k[st]);
                    spl_mbar_expect_tx(&full_sc[ss], 1024);
                    spl_bulk_g2s(s_ring + ss * 1024, k_scale + vec * SPL_PAGE_TOKENS + sub * CH, 512, &full_sc[ss]);
                    spl_bulk_g2s(s_ring + ss * 1024 + 512, v_scale + vec * SPL_PAGE_TOKENS + sub * CH, 512, &full_sc[ss]);
                } else {
                    const int st = i % NVS;
                    ok = spl_mbar_wait(&empty_v[st], ((i / NVS) & 1) ^ 1);
                    SPL_A1(0);
                    if (!ok) break;
                    spl_mbar_expect_tx(&full_v[st], CHUNK_BYTES);
                    spl_bulk_g2s(v_ring + size_t(st) * CHUNK_BYTES, v_codes + vec * (SPL_PAGE_TOKENS * HD) + size_t(sub) * CHUNK_BYTES, CHUNK_BYTES, &full_v[st]);
                }
                SPL_A1(1);
            }
            if (warp == 12) SPL_AOUT(32, 2);
        }
    } else if (warp == 13) {
        // ---- tensor-core issue, score product: S^T[buffer] = K (tensor memory) x Q (shared memory), sixteen channels per instruction.
        // The whole warp runs the loop and its waits and one elected lane issues (spl_elect_one); the two products have
        // a warp each, so that one's waits run under the other's instructions.
        constexpr uint32_t idesc = spl_tc_idesc(NQ);
        const uint64_t q_desc = spl_tc_desc_sw128(spl_smem_addr(q_tile));
        for (int i = 0; i < chunks && ok; ++i) {
            const int buf = i & 1;
            SPL_A0();
            ok = spl_mbar_wait_warp(&s_free[buf], ((i >> 1) & 1) ^ 1);
            SPL_A1(0);
            if (!ok) break;
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
                const int piece = i * HALVES + h, slot = piece % 3;
                ok = spl_mbar_wait_warp(&ka_full[slot], (piece / 3) & 1);
                SPL_A1(1);
                if (!ok) break;
                spl_tc_fence_after();
                if (spl_elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const int step = h * 8 + ks;
                        if (step == 0) spl_tc_mma_ts(tmem_s + buf * NQ, tmem_ka + slot * 64 + ks * 8, q_desc + uint64_t(((step >> 2) * QTILE + (step & 3) * 32) >> 4), idesc, 0u);
                        else spl_tc_mma_ts_acc(tmem_s + buf * NQ, tmem_ka + slot * 64 + ks * 8, q_desc + uint64_t(((step >> 2) * QTILE + (step & 3) * 32) >> 4), idesc);
                    }
                    spl_tc_commit(&ka_free[slot]);
                    if (h == HALVES - 1) spl_tc_commit(&s_full[buf]);
                }
                __syncwarp();
                SPL_A1(2);
            }
        }
        if (lane == 0) SPL_AOUT(34, 3);
    } else if (warp == 14) {
        // ---- tensor-core issue, value product: O^T[half] += V^T (tensor memory) x P (shared memory), sixteen tokens per instruction.
        constexpr uint32_t idesc = spl_tc_idesc(NQ);
        const uint64_t p_desc = spl_tc_desc_sw128(spl_smem_addr(p_tile));
        for (int i = 0; i < chunks && ok; ++i) {
            const int pb = i & 1;
            SPL_A0();
            ok = spl_mbar_wait_warp(&p_full[pb], (i >> 1) & 1);
            SPL_A1(0);
            if (!ok) break;
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
                ok = spl_mbar_wait_warp(&va_full[h], i & 1);
                SPL_A1(1);
                if (!ok) break;
                spl_tc_fence_after();
                if (spl_elect_one()) {
                    spl_tc_mma_ts(tmem_o + h * NQ, tmem_va + h * 64, p_desc + uint64_t((pb * PTILE) >> 4), idesc, i > 0 ? 1u : 0u);
#pragma unroll
                    for (int ks = 1; ks < 8; ++ks)
                        spl_tc_mma_ts_acc(tmem_o + h * NQ, tmem_va + h * 64 + ks * 8, p_desc + uint64_t((pb * PTILE + (ks >> 2) * QTILE + (ks & 3) * 32) >> 4), idesc);
                    spl_tc_commit(&va_free[h]);
                    if (h == HALVES - 1) { spl_tc_commit(&p_free[pb]); spl_tc_commit(&o_done[pb]); }
                }
                __syncwarp();
                SPL_A1(2);
            }
        }
        if (lane == 0) SPL_AOUT(37, 3);
    } else if (warp >= 4 && warp < 8) {
        // ---- K: thread = token. Its head_dim int8 -> fp16 pairs -> tensor memory, 128 channels (a 64-column slot of the ring) at a time.
        const int token = (warp & 3) * 32 + lane;
        const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
        for (int i = 0; i < chunks && ok; ++i) {
            const int st = i % NKS;
            SPL_A0();
            ok = spl_mbar_wait(&full_k[st], (i / NKS) & 1);
            SPL_A1(0);
            if (!ok) break;
            const unsigned char *src = k_ring + size_t(st) * CHUNK_BYTES + token * 16;
#pragma unroll 1
            for (int h = 0; h < HALVES; ++h) {
                const int piece = i * HALVES + h, slot = piece % 3;
                SPL_A1(1);
                ok = spl_mbar_wait(&ka_free[slot], ((piece / 3) & 1) ^ 1);
                SPL_A1(2);
                if (!ok) break;
                spl_tc_fence_after();
#pragma unroll 1
                for (int b = 0; b < 2; ++b) {
                    uint32_t a[32];
#pragma unroll
                    for (int pc = 0; pc < 4; ++pc)
                        spl_s8x16_to_h2x8(*reinterpret_cast<const uint4 *>(src + (h * 8 + 4 * b + pc) * (CH * 16)), a + pc * 8);
                    spl_tc_st32(tmem_ka + lane_base + slot * 64 + 32 * b, a);
                }
                if (h == HALVES - 1) { __syncwarp(); if (lane == 0) spl_mbar_arrive(&empty_k[st]); }
                spl_tc_st_wait();
                spl_tc_fence_before();
                __syncwarp();
                if (lane == 0) spl_mbar_arrive(&ka_full[slot]);
                SPL_A1(3);
            }
        }
        if (warp == 4) SPL_AOUT(40, 4);
    } else if (warp >= 8 && warp < 12) {
        // ---- V: thread = channel of a half. Its 128 tokens int8 -> fp16 pairs -> tensor memory.
        const int channel = (warp & 3) * 32 + lane;
        const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
        for (int i = 0; i < chunks && ok; ++i) {
            const int st = i % NVS;
            SPL_A0();
            ok = spl_mbar_wait(&full_v[st], (i / NVS) & 1);
            SPL_A1(0);
            if (!ok) break;
            const unsigned char *src = v_ring + size_t(st) * CHUNK_BYTES;
#pragma unroll 1
            for (int h = 0; h < HALVES; ++h) {
                SPL_A1(1);
                ok = spl_mbar_wait(&va_free[h], (i & 1) ^ 1);
                SPL_A1(2);
                if (!ok) break;
                spl_tc_fence_after();
#pragma unroll 1
                for (int b = 0; b < 2; ++b) {
                    uint32_t a[32];
#pragma unroll
                    for (int tb = 0; tb < 4; ++tb)
                        spl_s8x16_to_h2x8(*reinterpret_cast<const uint4 *>(src + (4 * b + tb) * (HD * 16) + (h * 128 + channel) * 16), a + tb * 8);
                    spl_tc_st32(tmem_va + lane_base + h * 64 + 32 * b, a);
                }
                if (h == HALVES - 1) { __syncwarp(); if (lane == 0) spl_mbar_arrive(&empty_v[st]); }
                spl_tc_st_wait();
                spl_tc_fence_before();
                __syncwarp();
                if (lane == 0) spl_mbar_arrive(&va_full[h]);
                SPL_A1(3);
            }
        }
        if (warp == 8) SPL_AOUT(44, 4);
    } else if (warp < 4 || warp >= 16) {
        // ---- softmax: thread = token of the chunk (scores), = channel of a half (rescale and output); the warp group
        // (warps 0-3, 16-19, 20-23) has its share of the queries.
        const int w4 = warp & 3, token = w4 * 32 + lane, sg = warp < 4 ? 0 : (warp - 12) >> 2, cb = sg * NH;       // cb: first query column of the group
        const uint32_t lane_base = uint32_t(w4 * 32) << 16;
        float *my_next = ref_next + w4 * NQ + cb, *my_factor = ref_factor + w4 * NQ + cb;      // this warp's copy: no cross-warp hazards
        float sum[NH];              // sum of p per query over this thread's tokens; reduced over lanes and warps at the end of the span
#pragma unroll
        for (int n = 0; n < NH; ++n) sum[n] = 0.0f;
        if (lane < NH) { my_next[lane] = -INFINITY; my_factor[lane] = 1.0f; }
        __syncwarp();
        // The thread's byte offsets inside an operand row for each of the eight swizzle phases of a row.
        uint32_t phase_offset[8];
        int raises[2] = {0, 0};            // completed exchanges of maxima, per chunk parity
#pragma unroll
        for (int j = 0; j < 8; ++j) phase_offset[j] = uint32_t((token >> 6) * QTILE) + spl_sw128_offset(j, token & 63);
        for (int i = 0; i < chunks && ok; ++i) {
            const int ss = i % NSS, buf = i & 1, par = i & 1;
            SPL_A0();
            ok = spl_mbar_wait(&full_sc[ss], (i / NSS) & 1);
            SPL_A1(0);
            if (!ok) break;
            const float *scales = reinterpret_cast<const float *>(s_ring + ss * 1024);
            const uint32_t token_index = token_begin + uint32_t(i) * CH + token;
            // Tokens past the last visible one were never written: their scales are whatever the pool held.
            const bool written = token_index < max_visible;
            const float ksl = written ? scales[token] * p.scale * LOG2E : 0.0f, vsc = written ? scales[CH + token] * SPL_ATTN_PSCALE : 0.0f;
            __syncwarp();
            if (lane == 0) spl_mbar_arrive(&empty_sc[ss]);
            // A token is visible to rows rb >= first_seen; a chunk wholly below the first row's position needs no mask
            // (padding queries are zero there and their columns are never written out).
            const bool whole = token_begin + uint32_t(i + 1) * CH <= first_pos + 1;
            const int first_seen = max(0, int(token_index) - int(first_pos));
            ok = spl_mbar_wait(&s_full[buf], (i >> 1) & 1);
            SPL_A1(1);
            if (!ok) break;
            spl_tc_fence_after();
            const uint32_t s_addr = tmem_s + lane_base + buf * NQ + cb, p_base = spl_smem_addr(p_tile + buf * PTILE);
            auto chunk_body = [&](auto masked_tag) -> bool {
                constexpr bool MASKED = decltype(masked_tag)::value;
                // Pass 1: does any score of the chunk exceed its query's reference by more than the head-room?
                float over = -INFINITY;
#pragma unroll
                for (int c0 = 0; c0 < NH; c0 += 8) {
                    uint32_t v[8];
                    float nx[8];
#pragma unroll
                    for (int r4 = 0; r4 < 2; ++r4) *reinterpret_cast<float4 *>(nx + 4 * r4) = *reinterpret_cast<const float4 *>(my_next + c0 + 4 * r4);
                    spl_tc_ld8(v, s_addr + c0);
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        float t = fmaf(__uint_as_float(v[r]), ksl, -nx[r]);
                        if (MASKED) { const int rb = (cb + c0 + r) / PER_KV; t = (rb >= first_seen && rb < valid_rows) ? t : -INFINITY; }
                        over = fmaxf(over, t);
                    }
                }
                const bool any_over = __any_sync(0xffffffffu, over > SPL_ATTN_HEADROOM);
                SPL_A1(2);
                if (lane == 0) {
                    if (any_over) atomicMax(xflag + sg * 2 + par, i + 1);
                    spl_mbar_arrive(&x_full[sg * 2 + par]);
                }
                if (!spl_mbar_wait(&x_full[sg * 2 + par], (i >> 1) & 1)) return false;
                const bool raise = *reinterpret_cast<volatile int *>(xflag + sg * 2 + par) == i + 1;
                SPL_A1(3);
                // The probability tile of two chunks ago has been read (and with it that chunk's value product has finished,
                // so a wait on the previous chunk's completion cannot see a stale phase).
                if (!spl_mbar_wait(&p_free[buf], ((i >> 1) & 1) ^ 1)) return false;
                SPL_A1(4);
                if (raise) {
                    // Some score is far above its reference (always so in a span's first chunk): raise every reference to its
                    // query's maximum so far, and rescale the sums and O^T by exp2(old - new).
#pragma unroll 1
                    for (int c0 = 0; c0 < NH; c0 += 8) {
                        uint32_t v[8];
                        spl_tc_ld8(v, s_addr + c0);
#pragma unroll
                        for (int r = 0; r < 8; ++r) {
                            const int n = cb + c0 + r;
                            float sc = __uint_as_float(v[r]) * ksl;
                            if (MASKED) { const int rb = n / PER_KV; sc = (rb >= first_seen && rb < valid_rows) ? sc : -INFINITY; }
                            const float top = spl_redux_max(sc);
                            if (lane == r) xmax[(par * 4 + w4) * NQ + n] = top;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) spl_mbar_arrive(&y_full[sg * 2 + par]);
                    if (!spl_mbar_wait(&y_full[sg * 2 + par], raises[par] & 1)) return false;
                    ++raises[par];
                    if (lane < NH) {
                        const int n = cb + lane;
                        const float top = fmaxf(fmaxf(xmax[(par * 4 + 0) * NQ + n], xmax[(par * 4 + 1) * NQ + n]),
                                                fmaxf(xmax[(par * 4 + 2) * NQ + n], xmax[(par * 4 + 3) * NQ + n]));
                        const float old = my_next[lane], next = fmaxf(old, top);
                        my_next[lane] = next; my_factor[lane] = (old == -INFINITY || next == old) ? 1.0f : spl_ex2(old - next);
                    }
                    __syncwarp();
                    float f[NH];
#pragma unroll
                    for (int r4 = 0; r4 < NH / 4; ++r4) *reinterpret_cast<float4 *>(f + 4 * r4) = *reinterpret_cast<const float4 *>(my_factor + 4 * r4);
#pragma unroll
                    for (int n = 0; n < NH; ++n) sum[n] *= f[n];
                    if (i > 0) {
                        if (!spl_mbar_wait(&o_done[(i - 1) & 1], ((i - 1) >> 1) & 1)) return false;
                        spl_tc_fence_after();
#pragma unroll
                        for (int c0 = 0; c0 < NH; c0 += 8)
#pragma unroll
                            for (int h = 0; h < HALVES; ++h) {
                                uint32_t v[8];
                                spl_tc_ld8(v, tmem_o + lane_base + h * NQ + cb + c0);
#pragma unroll
                                for (int r = 0; r < 8; ++r) v[r] = __float_as_uint(__uint_as_float(v[r]) * f[c0 + r]);
                                spl_tc_st8(tmem_o + lane_base + h * NQ + cb + c0, v);
                            }
                        spl_tc_st_wait();
                        spl_tc_fence_before();
                    }
                }
                SPL_A1(5);
                // Pass 2: probabilities into the operand tile of the value product, two queries at a time:
                // P = bf16(p * vScale), held as fp16 of SPL_ATTN_PSCALE * P (both roundings of a pair are single instructions).
#pragma unroll
                for (int c0 = 0; c0 < NH; c0 += 8) {
                    uint32_t v[8];
                    float nx[8];
#pragma unroll
                    for (int r4 = 0; r4 < 2; ++r4) *reinterpret_cast<float4 *>(nx + 4 * r4) = *reinterpret_cast<const float4 *>(my_next + c0 + 4 * r4);
                    spl_tc_ld8(v, s_addr + c0);
#pragma unroll
                    for (int r = 0; r < 8; r += 2) {
                        float pr[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            pr[e] = spl_ex2(fmaf(__uint_as_float(v[r + e]), ksl, -nx[r + e]));
                            if (MASKED) { const int rb = (cb + c0 + r + e) / PER_KV; pr[e] = (rb >= first_seen && rb < valid_rows) ? pr[e] : 0.0f; }
                            sum[c0 + r + e] += pr[e];
                        }
                        uint32_t packed_bf16, packed_f16;
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;\n" : "=r"(packed_bf16) : "f"(pr[1] * vsc), "f"(pr[0] * vsc));
                        asm("cvt.rn.f16x2.f32 %0, %1, %2;\n" : "=r"(packed_f16) : "f"(__uint_as_float(packed_bf16 & 0xFFFF0000u)), "f"(__uint_as_float(packed_bf16 << 16)));
                        const int n0 = cb + c0 + r, n1 = n0 + 1;
                        // No memory clobber: the stores need no order against this thread's loads, and the fences that
                        // follow the pass order them against everything later.
                        asm volatile("{\n .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %2;\n st.shared.b16 [%0], lo;\n st.shared.b16 [%1], hi;\n}\n"
                                     ::"r"(p_base + uint32_t((n0 >> 3) * 1024) + phase_offset[r & 7]),          // cb and c0 are multiples of 8
                                       "r"(p_base + uint32_t((n1 >> 3) * 1024) + phase_offset[(r + 1) & 7]), "r"(packed_f16));
                    }
                }
                return true;
            };
            ok = whole ? chunk_body(SplFalse{}) : chunk_body(SplTrue{});
            if (!ok) break;
            spl_tc_fence_before();
            spl_fence_proxy_async();
            __syncwarp();
            if (lane == 0) { spl_mbar_arrive(&s_free[buf]); spl_mbar_arrive(&p_full[buf]); }
            SPL_A1(6);
        }
        if (warp == 0) { SPL_AOUT(48, 7); SPL_ACHUNKS(); }
        // ---- the span's partial: [reference, sum p, out[head_dim]] per query (row, head).
        if (ok && chunks > 0) ok = spl_mbar_wait(&o_done[(chunks - 1) & 1], ((chunks - 1) >> 1) & 1);
        if (ok) {
            spl_tc_fence_after();
#pragma unroll
            for (int n = 0; n < NH; ++n) {
                const float total = spl_warp_sum(sum[n]);
                if (lane == n) xsum[w4 * NQ + cb + n] = total;
            }
            __syncwarp();
            if (lane == 0) spl_mbar_arrive(sum_full);
            ok = spl_mbar_wait(sum_full, 0);
        }
        if (ok) {
            const int record = HD + 2;
            if (w4 == 0 && lane < NH && (cb + lane) / PER_KV < valid_rows && cb + lane < 8 * PER_KV) {
                const int n = cb + lane, rb = n / PER_KV, hq = n % PER_KV;
                float *partial = partials + ((size_t(r0 + rb) * p.heads + kv_head * PER_KV + hq) * p.spans + span) * record;
                partial[0] = chunks > 0 ? my_next[lane] * LN2 : -INFINITY;
                partial[1] = ((xsum[n] + xsum[NQ + n]) + xsum[2 * NQ + n]) + xsum[3 * NQ + n];
            }
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
#pragma unroll
                for (int c0 = 0; c0 < NH; c0 += 8) {
                    uint32_t v[8];
                    if (chunks > 0) spl_tc_ld8(v, tmem_o + lane_base + h * NQ + cb + c0);
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        const int n = cb + c0 + r, rb = n / PER_KV, hq = n % PER_KV;
                        if (rb < valid_rows && n < 8 * PER_KV) {
                            float *partial = partials + ((size_t(r0 + rb) * p.heads + kv_head * PER_KV + hq) * p.spans + span) * record;
                            partial[2 + h * 128 + token] = chunks > 0 ? __uint_as_float(v[r]) * (1.0f / SPL_ATTN_PSCALE) : 0.0f;
                        }
                    }
                }
        }
    }
    if (!ok) atomicExch(error_flag, 100 + warp);
    spl_tc_fence_before();
    __syncthreads();
    if (warp == 13) {
        spl_tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512) : "memory");
    }
}

// Merge span partials by log-sum-exp, apply the sigmoid output gate, round to the bf16 operand of
// the output projection and emit its per-64 sums (engine.metal:2218-2255). Grid (heads, live rows), head_dim threads.
__global__ void spl_attn_merge_kernel(const float *__restrict__ partials, const float *__restrict__ proj, SplOperand core, SplAttnParams p) {
    spl_grid_begin();
    __shared__ float warp_sums[8];
    const int head = blockIdx.x, row = blockIdx.y, j = threadIdx.x, hd = p.head_dim, record = hd + 2;
    const float *base = partials + (size_t(row) * p.heads + head) * p.spans * record;
    // The spans' weights and the sum of the weighted totals once for the block (the first warp, a lane a span; at most 64
    // spans; both numbers of a span are asked for together: one trip to memory), then every thread walks its channel with
    // the loads of eight spans in flight and the additions in span order.
    __shared__ float weights[64];
    __shared__ float total;
    if (j < 32) {
        float ref[2], tot[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int s = j + 32 * u;
            ref[u] = s < p.spans ? base[s * record] : -INFINITY;
            tot[u] = s < p.spans ? base[s * record + 1] : 0.0f;
        }
        const float top = spl_warp_max(fmaxf(ref[0], ref[1]));
        float part = 0.0f;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int s = j + 32 * u;
            const float weight = s < p.spans ? expf(ref[u] - top) : 0.0f;
            if (s < p.spans) weights[s] = weight;
            if (weight > 0.0f) part += tot[u] * weight;
        }
        part = spl_warp_sum(part);
        if (j == 0) total = part;
    }
    __syncthreads();
    const float sum = total;
    float acc = 0.0f;
    int s = 0;
    for (; s + 8 <= p.spans; s += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = base[(s + u) * record + 2 + j];
#pragma unroll
        for (int u = 0; u < 8; ++u) if (weights[s + u] > 0.0f) acc += v[u] * weights[s + u];
    }
    for (; s + 4 <= p.spans; s += 4) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = base[(s + u) * record + 2 + j];
#pragma unroll
        for (int u = 0; u < 4; ++u) if (weights[s + u] > 0.0f) acc += v[u] * weights[s + u];
    }
    for (; s < p.spans; ++s) if (weights[s] > 0.0f) acc += base[s * record + 2 + j] * weights[s];
    const float gate = proj[size_t(row) * p.proj_ld + head * 2 * hd + hd + j];
    const uint16_t bits = spl_float_to_bf16((acc / sum) * spl_sigmoid(gate));
    reinterpret_cast<__half *>(core.values)[core.at(row, head * hd + j)] = __float2half_rn(spl_bf16_to_float(bits));
    const float wsum = spl_warp_sum(spl_bf16_to_float(bits));
    if ((j & 31) == 0) warp_sums[j >> 5] = wsum;
    __syncthreads();
    if ((j & 63) == 0) core.put_sum(row, (head * hd + j) / 64, warp_sums[j >> 5] + warp_sums[(j >> 5) + 1]);
}
