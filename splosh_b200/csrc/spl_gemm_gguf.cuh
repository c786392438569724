// spl_gemm_gguf.cuh — GGUF K-quant (Q4_K, Q5_K, Q6_K) dequant-GEMM on the 5th-generation tensor cores.
//
// Stands in for the GGUF branch of Engine.gemm and its tile kernels (Sources/SploshRuntime/Engine.swift:1666-1695;
// Sources/Shaders/engine_gguf.metal:82-273; weight formation Sources/Shaders/gguf_formats.h:160-249, 390-438):
//
//   out[r][n] = sum_k a[r][k] * w16[n][k] (+ residual[r][n])
//
// with a the bf16-rounded activations and w16 the weight rounded ONCE to fp16 from one fp32 operation:
// fma(code, d * scale, -dmin * minimum) for Q4_K / Q5_K, (code - 32) * (d * scale) for Q6_K.
//
// The kernel is spl_gemm_q4_tc_kernel's pipeline (spl_gemm_tc.cuh) with another dequant stage and no bias term: a
// super-block of 256 is one shared-memory stage (four 64-groups), the dequant warps (thread = output column) form the
// fp16 weights and store them into tensor memory as the A operand, the activations (held as fp16) are the B operand.
//
// Device layout of a weight (private to this library): for each tile of 128 output columns and each super-block,
// the columns' blocks cut in 16-byte pieces, [piece][column][16 bytes] (a column's thread reads its piece beside its
// neighbours': no bank conflicts). Q4_K keeps the native bytes: header (d, dmin, 12 scale bytes), then 8 pieces of 4-bit
// codes. Q5_K and Q6_K are widened to ONE BYTE A CODE when they are repacked (the fifth bit, or the two high bits, merged
// into the nibble then, once, and not by every block of every step): header pieces first (Q5_K: d, dmin, scale bytes;
// Q6_K: 16 scales, then d), then 16 pieces of codes in contraction order. The dequant stage was bound by its integer
// instructions, not by memory: the wider layout reads 272 (288) bytes a block where the native one has 176 (210), and
// forms a weight from a byte permute, a subtraction and a multiply-add.
#pragma once
#include "spl_gemm_tc.cuh"

#define SPL_GGUF_Q4K 12      // the GGUF type numbers
#define SPL_GGUF_Q5K 13
#define SPL_GGUF_Q6K 14
__host__ __device__ constexpr int spl_gguf_block_bytes(int format) { return format == SPL_GGUF_Q6K ? 210 : format == SPL_GGUF_Q5K ? 176 : 144; }
__host__ __device__ constexpr int spl_gguf_pieces(int format) { return format == SPL_GGUF_Q6K ? 18 : format == SPL_GGUF_Q5K ? 17 : 9; }

struct SplGgufDev {
    int n = 0, ld = 0, tiles = 0, k = 0, format = 0;
    unsigned char *blocks = nullptr;        // [tiles][k / 256][pieces][128][16]
    size_t bytes() const { return size_t(n) * (k / 256) * spl_gguf_block_bytes(format); }
    size_t device_bytes() const { return size_t(tiles) * (k / 256) * spl_gguf_pieces(format) * 2048; }
};

// Native row-major blocks [rows][k / 256][block bytes] -> the tile layout, as columns [n0, n0 + rows) of a (fused) tensor.
// One thread a (row, super-block, piece).
__global__ void spl_repack_gguf_kernel(const unsigned char *__restrict__ native, int rows, int supers, int format, unsigned char *tiles, int n0) {
    const int pieces = spl_gguf_pieces(format), bytes = spl_gguf_block_bytes(format);
    const size_t total = size_t(rows) * supers * pieces;
    for (size_t idx = blockIdx.x * size_t(blockDim.x) + threadIdx.x; idx < total; idx += size_t(gridDim.x) * blockDim.x) {
        const int piece = int(idx % pieces), sb = int((idx / pieces) % supers), row = int(idx / (size_t(pieces) * supers));
        const unsigned char *src = native + (size_t(row) * supers + sb) * bytes;
        unsigned char out[16];
        if (format == SPL_GGUF_Q6K) {
            // native: ql[128] qh[64] scales[16] d[2]  ->  scales, (d, 0...), then a byte a code: piece 2 + 4 g + 2 part + q4
            // holds elements 64 g + 32 part + 16 q4 .. + 15 (low nibble from ql, two high bits from qh)
            if (piece < 2) {
                for (int i = 0; i < 16; ++i) out[i] = piece == 0 ? src[192 + i] : i < 2 ? src[208 + i] : 0;
            } else {
                const int c = piece - 2, g = c >> 2, part = (c >> 1) & 1, q4 = c & 1, half128 = g >> 1, hi = g & 1;
                for (int i = 0; i < 16; ++i) {
                    const int low = src[64 * half128 + 32 * part + 16 * q4 + i], high = src[128 + 32 * half128 + 16 * q4 + i];
                    out[i] = uint8_t(((low >> (4 * hi)) & 15) | (((high >> (4 * hi + 2 * part)) & 3) << 4));
                }
            }
        } else if (format == SPL_GGUF_Q5K) {
            // native: d dmin scales[12] qh[32] qs[128]  ->  header, then a byte a code: piece 1 + 4 g + 2 part + q4 holds
            // elements 16 q4 .. + 15 of sub-block 2 g + part (nibble from qs, fifth bit from qh)
            if (piece == 0) {
                for (int i = 0; i < 16; ++i) out[i] = src[i];
            } else {
                const int c = piece - 1, g = c >> 2, part = (c >> 1) & 1, q4 = c & 1;
                for (int i = 0; i < 16; ++i) {
                    const int l = 16 * q4 + i;
                    out[i] = uint8_t(((src[48 + 32 * g + l] >> (4 * part)) & 15) | (((src[16 + l] >> (2 * g + part)) & 1) << 4));
                }
            }
        } else {
            for (int i = 0; i < 16; ++i) out[i] = src[16 * piece + i];
        }
        const int tile = (n0 + row) >> 7, col = (n0 + row) & 127;
        unsigned char *dst = tiles + ((size_t(tile) * supers + sb) * pieces + piece) * 2048 + col * 16;
        for (int i = 0; i < 16; ++i) dst[i] = out[i];
    }
}

// Stages of weight blocks in flight: three, or two where the widened blocks beside 64 rows of activations would not fit
// (as many as fit, five at 16 rows, were measured: no change, the kernel does not wait for memory).
__host__ __device__ constexpr int spl_gguf_cstages(int rn, int format) { return (rn >= 64 && format != SPL_GGUF_Q4K) ? 2 : 3; }
#define SPL_GG_THREADS 480       // warps 0-3, 8-11 and 4-7: three dequant sets; 12 copies; 13-14 tensor-core issue
__host__ __device__ constexpr size_t spl_gguf_smem_bytes(int rn, int format) {
    return 1024 + size_t(spl_gguf_cstages(rn, format)) * spl_gguf_pieces(format) * 2048 + size_t(4) * SPL_TC_SUPER * rn * 128 + 1024;
}
__device__ __forceinline__ float spl_half_bits_to_float(uint32_t bits) { return __half2float(__ushort_as_half(uint16_t(bits))); }
// Two fp32 values -> one register of two fp16, each rounded to nearest even.
__device__ __forceinline__ uint32_t spl_pack_half2(float lo, float hi) {
    uint32_t out;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;\n" : "=r"(out) : "f"(hi), "f"(lo));
    return out;
}

// Bytes `B` and `B + 1` of `word` less `bias`, as two floats, exactly: ONE byte permute places both bytes under the fp16
// exponent of 2^10 (where a byte is the number 1024 + byte), and the mixed-precision addition (an fp16 term plus an fp32
// term, in fp32) takes 1024 + bias away. The logic pipe bounds this kernel, and this is one of its instructions for two
// codes. Measured, GEMM a 16-row step: every code through the integer-to-float conversion (a quarter-rate pipe) 11.0 ms;
// a permute a code under the fp32 exponent of 2^23 and a subtraction 10.3 ms on the native layout, 8.4 ms on this one.
template <int B>
__device__ __forceinline__ float2 spl_bytes_to_float2(uint32_t word, float bias) {
    const uint32_t pair = __byte_perm(word, 0x64006400u, 0x7050 | B | ((B + 1) << 8));
    float2 x;
    asm("{\n .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %2;\n add.rn.f32.f16 %0, lo, %3;\n add.rn.f32.f16 %1, hi, %3;\n}\n"
        : "=f"(x.x), "=f"(x.y) : "r"(pair), "f"(-1024.0f - bias));
    return x;
}

// One 64-group of one column into 32 registers of fp16 pairs (k = 2c, 2c + 1 in register c). `stage` is the super-block's
// stage [piece][128][16], `g` the group (0..3).
template <int FMT>
__device__ __forceinline__ void spl_gguf_dequant64(const unsigned char *stage, int col, int g, uint32_t *a) {
    if (FMT == SPL_GGUF_Q6K) {
        const uint4 sc = *reinterpret_cast<const uint4 *>(stage + col * 16);
        const float d = spl_half_bits_to_float(*reinterpret_cast<const uint32_t *>(stage + 2048 + col * 16) & 0xFFFFu);
        const int half128 = g >> 1, hi = g & 1;
        const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
        // scale bytes 8 half128 + {0, 1} (+ 4 hi) for k < 32 and + 2 for k >= 32
#pragma unroll
        for (int part = 0; part < 2; ++part) {            // k in [32 part, 32 part + 32)
            const int sbase = 8 * half128 + 4 * hi + 2 * part;
            float s[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) s[e] = d * float(int8_t((scw[(sbase + e) >> 2] >> (8 * ((sbase + e) & 3))) & 0xFFu));
#pragma unroll
            for (int q4 = 0; q4 < 2; ++q4) {              // sixteen codes a piece
                const uint4 q = *reinterpret_cast<const uint4 *>(stage + (2 + 4 * g + 2 * part + q4) * 2048 + col * 16);
                const uint32_t cw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint32_t code = cw[w];
                    const float2 s2 = make_float2(s[q4], s[q4]);
                    const float2 v01 = spl_mul2(spl_bytes_to_float2<0>(code, 32.0f), s2), v23 = spl_mul2(spl_bytes_to_float2<2>(code, 32.0f), s2);
                    a[16 * part + 8 * q4 + 2 * w] = spl_pack_half2(v01.x, v01.y);
                    a[16 * part + 8 * q4 + 2 * w + 1] = spl_pack_half2(v23.x, v23.y);
                }
            }
        }
    } else {
        const uint4 header = *reinterpret_cast<const uint4 *>(stage + col * 16);
        const float d = spl_half_bits_to_float(header.x & 0xFFFFu), dmin = spl_half_bits_to_float(header.x >> 16);
        // scale bytes: header bytes 4..15 = words y, z, w (get_scale_min_k4 of the format; gguf_formats.h:160-178)
        float s[2], m[2];
#pragma unroll
        for (int part = 0; part < 2; ++part) {
            const int j = 2 * g + part;
            uint32_t scale, minimum;
            if (j < 4) { scale = (header.y >> (8 * j)) & 63u; minimum = (header.z >> (8 * j)) & 63u; }
            else {
                const uint32_t shift = 8u * (j - 4), nib = header.w >> shift;
                scale = (nib & 0xFu) | ((((header.y >> shift) >> 6) & 3u) << 4);
                minimum = ((nib >> 4) & 0xFu) | ((((header.z >> shift) >> 6) & 3u) << 4);
            }
            s[part] = d * float(scale); m[part] = -dmin * float(minimum);
        }
        if (FMT == SPL_GGUF_Q5K) {
#pragma unroll
            for (int part = 0; part < 2; ++part)
#pragma unroll
                for (int q4 = 0; q4 < 2; ++q4) {          // sixteen codes a piece: elements l = 16 q4 .. + 15 of sub-block 2 g + part
                    const uint4 q = *reinterpret_cast<const uint4 *>(stage + (1 + 4 * g + 2 * part + q4) * 2048 + col * 16);
                    const uint32_t cw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const uint32_t code = cw[w];
                        const float2 s2 = make_float2(s[part], s[part]), m2 = make_float2(m[part], m[part]);
                        const float2 v01 = spl_fma2(spl_bytes_to_float2<0>(code, 0.0f), s2, m2), v23 = spl_fma2(spl_bytes_to_float2<2>(code, 0.0f), s2, m2);
                        a[16 * part + 8 * q4 + 2 * w] = spl_pack_half2(v01.x, v01.y);
                        a[16 * part + 8 * q4 + 2 * w + 1] = spl_pack_half2(v23.x, v23.y);
                    }
                }
        } else {
#pragma unroll
            for (int q4 = 0; q4 < 2; ++q4) {              // sixteen bytes of codes: elements l = 16 q4 .. + 15 of both sub-blocks
                const uint4 qs = *reinterpret_cast<const uint4 *>(stage + (1 + 2 * g + q4) * 2048 + col * 16);
                const uint32_t cw[4] = {qs.x, qs.y, qs.z, qs.w};
#pragma unroll
                for (int w = 0; w < 4; ++w)
#pragma unroll
                    for (int part = 0; part < 2; ++part) {
                        const uint32_t code = (cw[w] >> (4 * part)) & 0x0F0F0F0Fu;
                        const float2 s2 = make_float2(s[part], s[part]), m2 = make_float2(m[part], m[part]);
                        const float2 v01 = spl_fma2(spl_bytes_to_float2<0>(code, 0.0f), s2, m2), v23 = spl_fma2(spl_bytes_to_float2<2>(code, 0.0f), s2, m2);
                        a[16 * part + 8 * q4 + 2 * w] = spl_pack_half2(v01.x, v01.y);
                        a[16 * part + 8 * q4 + 2 * w + 1] = spl_pack_half2(v23.x, v23.y);
                    }
            }
        }
    }
}

// Grid (tiles, splits, row blocks in use), as spl_gemm_q4_tc_kernel; `supers` super-blocks of 256 in the contraction,
// `supers_per_split` of them a split.
template <int RN, int FMT>
__global__ void __launch_bounds__(SPL_GG_THREADS, 1)
spl_gemm_gguf_tc_kernel(const unsigned char *__restrict__ blocks, const __nv_bfloat16 *__restrict__ act, float *out, int out_ld,
                        const float *residual, float *partials, int rows, int op_blocks, int supers_total, int supers_per_split, int *error_flag) {
    constexpr int BST = 4, CST = spl_gguf_cstages(RN, FMT), ASUP = 2, AST = 4 * ASUP, PIECES = spl_gguf_pieces(FMT);
    constexpr int BTILE = SPL_TC_SUPER * RN * 128, WSTAGE = PIECES * 2048;
    extern __shared__ unsigned char spl_gg_smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(spl_gg_smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char *b_ring = smem;                                   // [BST][4][RN * 128] activations
    unsigned char *w_ring = b_ring + size_t(BST) * BTILE;           // [CST][pieces][128][16] blocks
    uint64_t *bars = reinterpret_cast<uint64_t *>(w_ring + size_t(CST) * WSTAGE);
    uint64_t *full_c = bars, *empty_c = full_c + CST, *full_b = empty_c + CST, *empty_b = full_b + BST, *full_a = empty_b + BST, *finished = full_a + AST / 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(finished + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y, rb = blockIdx.z, row_blocks = op_blocks;
    const int rows_padded = op_blocks * RN, groups = supers_total * SPL_TC_SUPER;
    const int s_first = split * supers_per_split, supers = min(supers_per_split, supers_total - s_first);
    const int units = supers * 2;

    if (threadIdx.x == 0) {
        for (int i = 0; i < CST; ++i) { spl_mbar_init(&full_c[i], 1); spl_mbar_init(&empty_c[i], 8); }
        for (int i = 0; i < BST; ++i) { spl_mbar_init(&full_b[i], 1); spl_mbar_init(&empty_b[i], 2); }
        for (int i = 0; i < AST / 2; ++i) spl_mbar_init(&full_a[i], 4);
        spl_mbar_init(finished, 2);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 13) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(spl_smem_addr(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    spl_tc_fence_before();
    __syncthreads();
    spl_tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    constexpr int NACC = RN <= 32 ? 4 : 2;
    const uint32_t tmem_d = tmem, tmem_a = tmem + 128;
    bool ok = true;
    (void)groups;

    if (!(warp == 12 && lane == 0)) spl_grid_begin();
    if (warp == 12) {
        if (lane == 0) {
            const unsigned char *wsrc = blocks + (size_t(tile) * supers_total + s_first) * WSTAGE;
            const unsigned char *bsrc = reinterpret_cast<const unsigned char *>(act) + ((size_t(s_first) * SPL_TC_SUPER * row_blocks + rb) * RN) * 128;
            const int ahead = min(CST, supers);
            for (int j = 0; j < ahead; ++j) {          // weights are nobody's output: asked for before the wait on the predecessor
                spl_mbar_expect_tx(&full_c[j], WSTAGE);
                spl_bulk_g2s(w_ring + size_t(j) * WSTAGE, wsrc + size_t(j) * WSTAGE, WSTAGE, &full_c[j]);
            }
            spl_grid_begin();
            for (int j = 0; j < supers && ok; ++j) {
                const int sc = j % CST, sbq = j % BST;
                if (j >= ahead) {
                    ok = spl_mbar_wait(&empty_c[sc], ((j / CST) & 1) ^ 1);
                    if (!ok) break;
                    spl_mbar_expect_tx(&full_c[sc], WSTAGE);
                    spl_bulk_g2s(w_ring + size_t(sc) * WSTAGE, wsrc + size_t(j) * WSTAGE, WSTAGE, &full_c[sc]);
                }
                ok = spl_mbar_wait(&empty_b[sbq], ((j / BST) & 1) ^ 1);
                if (!ok) break;
                spl_mbar_expect_tx(&full_b[sbq], uint32_t(BTILE));
                if (row_blocks == 1) {
                    spl_bulk_g2s(b_ring + size_t(sbq) * BTILE, bsrc + size_t(j) * BTILE, BTILE, &full_b[sbq]);
                } else {
                    for (int u = 0; u < SPL_TC_SUPER; ++u) {
                        const size_t g = size_t(j) * SPL_TC_SUPER + u;
                        spl_bulk_g2s(b_ring + size_t(sbq) * BTILE + u * RN * 128, bsrc + g * row_blocks * RN * 128, RN * 128, &full_b[sbq]);
                    }
                }
            }
        }
    } else if (warp >= 13) {
        // The whole warp runs the loop and its waits; one elected lane issues (spl_elect_one). Warp 13 issues the first
        // two k16 steps of every group and warp 14 the last two, each into accumulators of its own.
        const int m = warp - 13;
        constexpr uint32_t idesc = spl_tc_idesc(RN);
        const uint64_t b_desc0 = spl_tc_desc_sw128(spl_smem_addr(b_ring));
        for (int j = 0; j < supers && ok; ++j) {
            const int sbq = j % BST;
            const uint64_t b_desc = b_desc0 + uint64_t((sbq * BTILE) >> 4);
            const uint32_t a_base = tmem_a + (j % ASUP) * (SPL_TC_SUPER * 32);
            ok = spl_mbar_wait_warp(&full_b[sbq], (j / BST) & 1);
            if (!ok) break;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int un = 2 * j + half;
                ok = spl_mbar_wait_warp(&full_a[un % (AST / 2)], (un / (AST / 2)) & 1);
                if (!ok) break;
                spl_tc_fence_after();
                if (spl_elect_one()) {
#pragma unroll
                    for (int v = 0; v < 2; ++v) {
                        const int u = 2 * half + v;
#pragma unroll
                        for (int l = 0; l < 2; ++l) {
                            const int ks = 2 * m + l, acc = NACC == 4 ? ks : m;
                            const uint32_t d = tmem_d + acc * RN, a = a_base + u * 32 + ks * 8;
                            const uint64_t b = b_desc + uint64_t((u * RN * 128 + ks * 32) >> 4);
                            if (NACC == 2 && l > 0) spl_tc_mma_ts_acc(d, a, b, idesc);
                            else if (j > 0 || u > 0) spl_tc_mma_ts_acc(d, a, b, idesc);
                            else spl_tc_mma_ts(d, a, b, idesc, 0u);
                        }
                    }
                    if (half == 1) spl_tc_commit(&empty_b[sbq]);
                }
                __syncwarp();
            }
        }
        if (ok && spl_elect_one()) spl_tc_commit(finished);
        __syncwarp();
    } else {
        const int quarter = warp & 3, col = quarter * 32 + lane, set = warp < 4 ? 0 : warp >= 8 ? 1 : 2;
        const uint32_t lane_base = uint32_t(quarter * 32) << 16;
        for (int un = set; un < units && ok; un += 3) {
            const int j = un >> 1, half = un & 1, sc = j % CST;
            ok = spl_mbar_wait(&full_c[sc], (j / CST) & 1);
            if (!ok) break;
            uint32_t a[2][32];
#pragma unroll
            for (int v = 0; v < 2; ++v) spl_gguf_dequant64<FMT>(w_ring + size_t(sc) * WSTAGE, col, 2 * half + v, a[v]);
            __syncwarp();
            if (lane == 0) spl_mbar_arrive(&empty_c[sc]);
            // The A slots were last used ASUP stages ago; that stage's completion is the one its activation stage is freed by.
            if (j >= ASUP) ok = spl_mbar_wait(&empty_b[(j - ASUP) % BST], ((j - ASUP) / BST) & 1);
            if (!ok) break;
            spl_tc_fence_after();
#pragma unroll
            for (int v = 0; v < 2; ++v) {
                const int sa = (j % ASUP) * SPL_TC_SUPER + 2 * half + v;
                spl_tc_st16(tmem_a + lane_base + sa * 32, *reinterpret_cast<uint32_t (*)[16]>(&a[v][0]));
                spl_tc_st16(tmem_a + lane_base + sa * 32 + 16, *reinterpret_cast<uint32_t (*)[16]>(&a[v][16]));
            }
            spl_tc_st_wait();
            spl_tc_fence_before();
            __syncwarp();
            if (lane == 0) spl_mbar_arrive(&full_a[un % (AST / 2)]);
        }
        if (ok) ok = spl_mbar_wait(finished, 0);
        if (ok) {
            spl_tc_fence_after();
            const int n = tile * 128 + col;
            const bool is_split = gridDim.y > 1;
            float *dst = is_split ? partials + size_t(split) * rows_padded * out_ld : out;
#pragma unroll
            for (int cb = 0; cb < RN / 16; ++cb) {
                if (cb % 3 != set) continue;
                const int c0 = cb * 16;
                float total[16];
#pragma unroll
                for (int acc = 0; acc < NACC; ++acc) {
                    uint32_t v[16];
                    spl_tc_ld16(v, tmem_d + lane_base + acc * RN + c0);
#pragma unroll
                    for (int r = 0; r < 16; ++r) total[r] = acc == 0 ? __uint_as_float(v[r]) : total[r] + __uint_as_float(v[r]);
                }
                if (n < out_ld) {
#pragma unroll
                    for (int r = 0; r < 16; ++r) {
                        const int row = rb * RN + c0 + r;
                        if (row < rows) {
                            const size_t index = size_t(row) * out_ld + n;
                            dst[index] = (!is_split && residual) ? total[r] + residual[index] : total[r];
                        }
                    }
                }
            }
        }
    }
    if (!ok) atomicExch(error_flag, 1 + warp);
    spl_tc_fence_before();
    __syncthreads();
    if (warp == 13) {
        spl_tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512) : "memory");
    }
}

// ---- a GGUF-weighted model's other pieces -----------------------------------------------------
// One weight of a native block, exactly (fp32; Sources/SploshQuant/GgufQuant.swift:191-230, the form the reference's
// embedding gather uses, Sources/Shaders/gguf_formats.h:463-501): block `b` of `format`, element i of its 256.
__device__ __forceinline__ float spl_gguf_decode_one(const unsigned char *b, int format, int i) {
    if (format == SPL_GGUF_Q6K) {
        // ql[128] qh[64] scales[16] d: halves of 128, in each four runs of 32 sharing ql / qh bytes
        const int half = i >> 7, r = i & 127, run = r >> 5, l = r & 31;
        const unsigned char lo = b[64 * half + l + ((run & 1) ? 32 : 0)];
        const int nib = (run < 2) ? (lo & 0xF) : (lo >> 4);
        const int high = (b[128 + 32 * half + l] >> (2 * run)) & 3;
        const int q = (nib | (high << 4)) - 32;
        const float d = __half2float(__ushort_as_half(uint16_t(b[208] | (b[209] << 8))));
        const int scale = int(reinterpret_cast<const signed char *>(b)[192 + 8 * half + 2 * run + (l >> 4)]);
        return __fmul_rn(__fmul_rn(d, float(scale)), float(q));
    }
    const float d = __half2float(__ushort_as_half(uint16_t(b[0] | (b[1] << 8)))), dmin = __half2float(__ushort_as_half(uint16_t(b[2] | (b[3] << 8))));
    const unsigned char *sc = b + 4;
    const int j = i >> 5;      // sub-block of 32
    int scale, minimum;
    if (j < 4) { scale = sc[j] & 63; minimum = sc[j + 4] & 63; }
    else { scale = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4); minimum = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
    const int pair = i >> 6, l = i & 31, upper = (i >> 5) & 1;
    int q;
    if (format == SPL_GGUF_Q5K) {
        const unsigned char ql = b[48 + 32 * pair + l];
        q = (upper ? (ql >> 4) : (ql & 0xF)) | (((b[16 + l] >> j) & 1) << 4);
    } else {
        const unsigned char ql = b[16 + 32 * pair + l];
        q = upper ? (ql >> 4) : (ql & 0xF);
    }
    return __fsub_rn(__fmul_rn(__fmul_rn(d, float(scale)), float(q)), __fmul_rn(dmin, float(minimum)));      // every product rounded on its own, as the host decoders do
}

// Embedding rows of a native GGUF table [vocab][hidden / 256] blocks: out[r][:] = row token[r], decoded exactly. Grid (rows).
__global__ void spl_embed_gguf_kernel(const unsigned char *__restrict__ table, int format, const uint32_t *__restrict__ tokens, float *out, int hidden) {
    spl_grid_begin();
    const int row = blockIdx.x, bytes = spl_gguf_block_bytes(format);
    const unsigned char *src = table + size_t(tokens[row]) * (hidden / 256) * bytes;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) out[size_t(row) * hidden + c] = spl_gguf_decode_one(src + size_t(c >> 8) * bytes, format, c & 255);
}

// act = bf16(silu(gate) * up) of an unfused gate|up output [rows][2 inter] (gate columns first) as the down projection's
// operand with its per-64 sums (Sources/Shaders/engine.metal:200-219). Grid (inter / 64, rows), 32 threads.
__global__ void spl_swiglu_kernel(const float *__restrict__ gate_up, int ld, int inter, SplOperand out) {
    spl_grid_begin();
    const int group = blockIdx.x, row = blockIdx.y, lane = threadIdx.x, n = group * 64 + 2 * lane;
    const float2 g = *reinterpret_cast<const float2 *>(gate_up + size_t(row) * ld + n), u = *reinterpret_cast<const float2 *>(gate_up + size_t(row) * ld + inter + n);
    const float v0 = spl_bf16_to_float(spl_float_to_bf16(spl_silu_exact(g.x) * u.x)), v1 = spl_bf16_to_float(spl_float_to_bf16(spl_silu_exact(g.y) * u.y));
    *reinterpret_cast<__half2 *>(reinterpret_cast<__half *>(out.values) + out.at(row, n)) = __halves2half2(__float2half_rn(v0), __float2half_rn(v1));
    float sum = v0 + v1;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane == 0) out.put_sum(row, group, sum);
}

// Seeded synthetic blocks for timing: every byte pseudo-random, then the fp16 fields set so that weights have a
// deviation of about 0.02 (d and dmin small positive numbers). One thread a block.
__global__ void spl_synth_gguf_kernel(unsigned char *native, size_t blocks, int format, uint64_t seed) {
    const int bytes = spl_gguf_block_bytes(format);
    for (size_t idx = blockIdx.x * size_t(blockDim.x) + threadIdx.x; idx < blocks; idx += size_t(gridDim.x) * blockDim.x) {
        unsigned char *b = native + idx * bytes;
        for (int i = 0; i < bytes; i += 2) {
            const uint64_t z = spl_splitmix_at(seed, idx * 128 + (i >> 1));
            b[i] = uint8_t(z); if (i + 1 < bytes) b[i + 1] = uint8_t(z >> 8);
        }
        const float u = float(spl_splitmix_at(seed ^ 0x5151, idx) >> 40) * (1.0f / 16777216.0f);
        if (format == SPL_GGUF_Q6K) {
            const uint16_t d = __half_as_ushort(__float2half_rn(2.0e-5f * (0.5f + u)));     // x scale (|s| < 128) x code (|q| <= 32)
            b[208] = uint8_t(d); b[209] = uint8_t(d >> 8);
        } else {
            const float top = format == SPL_GGUF_Q5K ? 31.0f : 15.0f;
            const uint16_t d = __half_as_ushort(__float2half_rn(0.07f / (32.0f * top) * (0.5f + u))), m = __half_as_ushort(__float2half_rn(0.035f / 32.0f * (0.5f + u)));
            b[0] = uint8_t(d); b[1] = uint8_t(d >> 8); b[2] = uint8_t(m); b[3] = uint8_t(m >> 8);
        }
    }
}
