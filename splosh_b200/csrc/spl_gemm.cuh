// spl_gemm.cuh — MLX affine-4 (group 64) dequant-GEMM for narrow steps, the weight repack and the
// seeded weight generator.
//
// Stands in for Engine.gemm and the q4 kernels it selects (Sources/SploshRuntime/Engine.swift:1651-1806;
// Sources/Shaders/engine.metal:79-124, 1833-1985; Sources/Shaders/engine_na.metal:862-1011).
//
//   out[r][n] = sum over 64-groups g of ( dot(a[r][g], code[n][g]) * scale[n][g] + sum(a[r][g]) * bias[n][g] )  (+ residual[r][n])
//
// with a the bf16-rounded activations and sum(a) the per-64 sums of the rounded values: the
// reference's accelerator contract (engine_na.metal:42-57, 91-103). The dot runs on the tensor
// cores over exact operands (bf16 activations, 4-bit codes as bf16) with fp32 accumulation.
//
// Device layout of a weight (private to this library). Output columns are taken 16 at a time
// ("n16 block" nb), the contraction 64 at a time (quant group g). For each (nb, g):
//   codes: 32 lanes x 4 words. Lane l = 4 * g8 + t holds, in word ks (k0 = 64 g + 16 ks), the eight
//          codes of the m16n8k16 A fragment: rows nb*16 + g8 and + 8, columns k0 + 2t, 2t+1, 2t+8,
//          2t+9, as nibbles [a0 a2 a4 a6 a1 a3 a5 a7] so that (word >> 4j) & 0x000F000F is register j.
//   sb:    16 words, one per output column: scale in the low half, bias in the high half (bf16).
// A warp therefore reads 512 contiguous bytes of codes per (nb, g), 16 bytes a lane, and every
// byte of the weight exactly once per pass.
#pragma once
#include "spl_common.cuh"

struct SplQ4Dev {
    int n = 0;         // logical output columns
    int n16 = 0;       // 16-column blocks (n rounded up)
    int k = 0;         // contraction length, a multiple of 256
    uint4 *codes = nullptr;       // [n16][k/64][32] uint4
    uint32_t *sb = nullptr;       // [n16][k/64][16]
    size_t bytes() const { return size_t(n16) * (k / 64) * (512 + 64); }
};

// ---- repack: MLX row-major -> fragment layout, rows [n0, n0 + rows) of a fused tensor -------
__global__ void spl_repack_q4_kernel(const uint32_t *__restrict__ packed, const uint16_t *__restrict__ scales,
                                     const uint16_t *__restrict__ biases, int rows, int k, uint32_t *codes, uint32_t *sb,
                                     int nb_first, int nb_count) {
    const int groups = k / 64;
    const size_t total = size_t(nb_count) * groups * 128;
    for (size_t idx = blockIdx.x * size_t(blockDim.x) + threadIdx.x; idx < total; idx += size_t(gridDim.x) * blockDim.x) {
        const int ks = idx & 3, lane = (idx >> 2) & 31;
        const size_t ng = idx >> 7;
        const int g = int(ng % groups), nbl = int(ng / groups);
        const int g8 = lane >> 2, t = lane & 3;
        const int k0 = g * 64 + ks * 16;
        uint32_t word = 0;
#pragma unroll
        for (int a = 0; a < 8; ++a) {
            const int row = nbl * 16 + g8 + ((a >> 1) & 1) * 8;
            const int col = k0 + 2 * t + (a & 1) + ((a >> 2) & 1) * 8;
            uint32_t code = 0;
            if (row < rows) code = (packed[size_t(row) * (k / 8) + col / 8] >> (4 * (col % 8))) & 0xFu;
            const int pos = (a >> 1) + 4 * (a & 1);
            word |= code << (4 * pos);
        }
        codes[(size_t(nb_first + nbl) * groups + g) * 128 + lane * 4 + ks] = word;
        if (ks == 0 && lane < 16) {
            const int row = nbl * 16 + lane;
            uint32_t v = 0;
            if (row < rows) v = uint32_t(scales[size_t(row) * groups + g]) | (uint32_t(biases[size_t(row) * groups + g]) << 16);
            sb[(size_t(nb_first + nbl) * groups + g) * 16 + lane] = v;
        }
    }
}

// ---- seeded generator: value n of a tensor's stream, quantised group by group ---------------
// Value = (sum of the four 16-bit fields of SplitMix64 output n, less 131070) * factor; then the
// MLX rule: scale = bf16((max - min) / 15) (1 when flat), bias = bf16(min),
// code = clamp(round_half_away((v - bias) / scale), 0, 15)  (DraftModel.swift:634-670, "minmax").
// Every operation is a single IEEE operation so that a host generator reproduces it exactly.
__global__ void spl_synth_q4_kernel(uint64_t seed, float factor, int rows, int k, uint32_t *packed, uint16_t *scales, uint16_t *biases) {
    const int groups = k / 64;
    const size_t total = size_t(rows) * groups;
    for (size_t slot = blockIdx.x * size_t(blockDim.x) + threadIdx.x; slot < total; slot += size_t(gridDim.x) * blockDim.x) {
        const size_t first = slot * 64;       // row * k + g * 64
        float lo = INFINITY, hi = -INFINITY;
        for (int i = 0; i < 64; ++i) {
            const uint64_t z = spl_splitmix_at(seed, first + i);
            const int sum = int(z & 0xFFFF) + int((z >> 16) & 0xFFFF) + int((z >> 32) & 0xFFFF) + int(z >> 48);
            const float v = __fmul_rn(float(sum - 131070), factor);
            lo = fminf(lo, v); hi = fmaxf(hi, v);
        }
        const uint16_t sbits = spl_float_to_bf16(hi > lo ? __fdiv_rn(__fsub_rn(hi, lo), 15.0f) : 1.0f);
        const uint16_t bbits = spl_float_to_bf16(lo);
        const float scale = spl_bf16_to_float(sbits), bias = spl_bf16_to_float(bbits);
        scales[slot] = sbits; biases[slot] = bbits;
        for (int w = 0; w < 8; ++w) {
            uint32_t bits = 0;
            for (int nib = 0; nib < 8; ++nib) {
                const uint64_t z = spl_splitmix_at(seed, first + w * 8 + nib);
                const int sum = int(z & 0xFFFF) + int((z >> 16) & 0xFFFF) + int((z >> 32) & 0xFFFF) + int(z >> 48);
                const float v = __fmul_rn(float(sum - 131070), factor);
                const float code = fminf(15.0f, fmaxf(0.0f, roundf(__fdiv_rn(__fsub_rn(v, bias), scale))));
                bits |= uint32_t(code) << (4 * nib);
            }
            packed[slot * 8 + w] = bits;
        }
    }
}

// ---- the GEMM -------------------------------------------------------------------------------
#define SPL_GEMM_KC 256                     // contraction per staged activation chunk
#define SPL_GEMM_LDS (SPL_GEMM_KC + 8)      // padded row of the chunk in shared memory (bf16)
#define SPL_GEMM_WARPS 8

// Eight 4-bit codes of a word -> four bf16x2 registers of exact values: 0x4300 | c is 128 + c.
__device__ __forceinline__ void spl_codes4(uint32_t w, uint32_t (&a)[4]) {
    const __nv_bfloat162 bias128 = __floats2bfloat162_rn(128.0f, 128.0f);
    uint32_t q0 = (w & 0x000F000Fu) | 0x43004300u;
    uint32_t q1 = ((w >> 4) & 0x000F000Fu) | 0x43004300u;
    uint32_t q2 = ((w >> 8) & 0x000F000Fu) | 0x43004300u;
    uint32_t q3 = ((w >> 12) & 0x000F000Fu) | 0x43004300u;
    __nv_bfloat162 c0 = __hsub2(*reinterpret_cast<__nv_bfloat162 *>(&q0), bias128);
    __nv_bfloat162 c1 = __hsub2(*reinterpret_cast<__nv_bfloat162 *>(&q1), bias128);
    __nv_bfloat162 c2 = __hsub2(*reinterpret_cast<__nv_bfloat162 *>(&q2), bias128);
    __nv_bfloat162 c3 = __hsub2(*reinterpret_cast<__nv_bfloat162 *>(&q3), bias128);
    a[0] = *reinterpret_cast<uint32_t *>(&c0); a[1] = *reinterpret_cast<uint32_t *>(&c1);
    a[2] = *reinterpret_cast<uint32_t *>(&c2); a[3] = *reinterpret_cast<uint32_t *>(&c3);
}

// Grid (ceil(n16 / (WARPS * NBW)), splits). A block walks its share of the contraction in chunks
// of 256 (four quant groups); all warps share the staged activation chunk and its per-64 sums,
// each warp owns NBW n16 blocks. Per group the tensor cores form dot(a, codes) exactly as the
// reference's accelerator path does, and the epilogue adds dot * scale + sum(a) * bias.
// With splits > 1 each block writes its partial sums to `partials[split][row][n]` and
// spl_gemm_reduce_kernel adds them in split order, so the result does not depend on timing.
template <int RT, int NBW>
__global__ void __launch_bounds__(SPL_GEMM_WARPS * 32)
spl_gemm_q4_kernel(const uint4 *__restrict__ codes, const uint32_t *__restrict__ sb, const __nv_bfloat16 *__restrict__ act,
                   const float *__restrict__ act_sums, int act_ld, float *out, int out_ld, const float *residual, float *partials,
                   int rows, int n16, int groups, int chunks_per_split) {
    extern __shared__ __align__(16) unsigned char spl_gemm_smem[];
    constexpr int TILE = RT * 8 * SPL_GEMM_LDS;
    __nv_bfloat16 *tile0 = reinterpret_cast<__nv_bfloat16 *>(spl_gemm_smem);       // [2][RT * 8][SPL_GEMM_LDS]
    float *sums0 = reinterpret_cast<float *>(tile0 + 2 * TILE);                    // [2][RT * 8][4]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g8 = lane >> 2, t = lane & 3;
    const int nb0 = (blockIdx.x * SPL_GEMM_WARPS + warp) * NBW;
    const int chunk_first = blockIdx.y * chunks_per_split;
    const int total_chunks = groups / 4;
    const int chunk_count = min(chunks_per_split, total_chunks - chunk_first);

    float acc[NBW][RT][4];
#pragma unroll
    for (int i = 0; i < NBW; ++i)
#pragma unroll
        for (int r = 0; r < RT; ++r)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][r][e] = 0.0f;

    auto stage = [&](int chunk, int buffer) {
        // RT * 8 rows of 256 bf16: 32 threads a row, 16 bytes a thread; then the chunk's sums.
        const int k0 = chunk * SPL_GEMM_KC;
#pragma unroll
        for (int pass = 0; pass < RT; ++pass) {
            const int row = pass * 8 + (threadIdx.x >> 5), col = (threadIdx.x & 31) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < rows) v = *reinterpret_cast<const uint4 *>(act + size_t(row) * act_ld + k0 + col);
            *reinterpret_cast<uint4 *>(tile0 + buffer * TILE + row * SPL_GEMM_LDS + col) = v;
        }
        if (threadIdx.x < RT * 8) {
            const int row = threadIdx.x;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < rows) v = *reinterpret_cast<const float4 *>(act_sums + size_t(row) * (act_ld / 64) + chunk * 4);
            *reinterpret_cast<float4 *>(sums0 + (buffer * RT * 8 + row) * 4) = v;
        }
    };

    uint4 cw[NBW][4];
    auto fetch = [&](int chunk) {
#pragma unroll
        for (int i = 0; i < NBW; ++i) {
            const int nb = nb0 + i;
#pragma unroll
            for (int g = 0; g < 4; ++g)
                cw[i][g] = nb < n16 ? __ldg(codes + (size_t(nb) * groups + chunk * 4 + g) * 32 + lane) : make_uint4(0, 0, 0, 0);
        }
    };

    if (chunk_count > 0) { stage(chunk_first, 0); fetch(chunk_first); }
    __syncthreads();
    for (int c = 0; c < chunk_count; ++c) {
        const int chunk = chunk_first + c, buffer = c & 1;
        uint4 cur[NBW][4];
#pragma unroll
        for (int i = 0; i < NBW; ++i)
#pragma unroll
            for (int g = 0; g < 4; ++g) cur[i][g] = cw[i][g];
        if (c + 1 < chunk_count) { fetch(chunk + 1); stage(chunk + 1, buffer ^ 1); }
        const __nv_bfloat16 *ts = tile0 + buffer * TILE;
        const float *ss = sums0 + buffer * RT * 8 * 4;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float sA[NBW], bA[NBW], sB[NBW], bB[NBW];
            uint32_t a[NBW][4][4];
#pragma unroll
            for (int i = 0; i < NBW; ++i) {
                const int nb = nb0 + i;
                uint32_t x0 = 0, x1 = 0;
                if (nb < n16) {
                    const uint32_t *p = sb + (size_t(nb) * groups + chunk * 4 + g) * 16;
                    x0 = __ldg(p + g8); x1 = __ldg(p + g8 + 8);
                }
                sA[i] = __uint_as_float(x0 << 16); bA[i] = __uint_as_float(x0 & 0xFFFF0000u);
                sB[i] = __uint_as_float(x1 << 16); bB[i] = __uint_as_float(x1 & 0xFFFF0000u);
                spl_codes4(cur[i][g].x, a[i][0]); spl_codes4(cur[i][g].y, a[i][1]);
                spl_codes4(cur[i][g].z, a[i][2]); spl_codes4(cur[i][g].w, a[i][3]);
            }
#pragma unroll
            for (int r = 0; r < RT; ++r) {
                uint32_t b[4][2];
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const __nv_bfloat16 *p = ts + (r * 8 + g8) * SPL_GEMM_LDS + g * 64 + ks * 16 + 2 * t;
                    b[ks][0] = *reinterpret_cast<const uint32_t *>(p);
                    b[ks][1] = *reinterpret_cast<const uint32_t *>(p + 8);
                }
                const float sum0 = ss[(r * 8 + 2 * t) * 4 + g], sum1 = ss[(r * 8 + 2 * t + 1) * 4 + g];
#pragma unroll
                for (int i = 0; i < NBW; ++i) {
                    float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) spl_mma_bf16(part, a[i][ks], b[ks][0], b[ks][1]);
                    acc[i][r][0] += part[0] * sA[i] + sum0 * bA[i];
                    acc[i][r][1] += part[1] * sA[i] + sum1 * bA[i];
                    acc[i][r][2] += part[2] * sB[i] + sum0 * bB[i];
                    acc[i][r][3] += part[3] * sB[i] + sum1 * bB[i];
                }
            }
        }
        __syncthreads();
    }

    const bool split = gridDim.y > 1;
    float *dst = split ? partials + size_t(blockIdx.y) * (RT * 8) * out_ld : out;
#pragma unroll
    for (int i = 0; i < NBW; ++i) {
        const int nb = nb0 + i;
        if (nb >= n16) continue;
#pragma unroll
        for (int r = 0; r < RT; ++r) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = r * 8 + 2 * t + (e & 1), col = nb * 16 + g8 + (e >> 1) * 8;
                if (row >= rows) continue;
                const size_t index = size_t(row) * out_ld + col;
                float v = acc[i][r][e];
                if (!split && residual) v += residual[index];
                dst[index] = v;
            }
        }
    }
}

// out[r][n] = sum over splits, in split order, of partials[s][r][n] (+ residual[r][n]).
__global__ void spl_gemm_reduce_kernel(const float *__restrict__ partials, int splits, int rows_padded, int rows, int ld,
                                       const float *residual, float *out) {
    const size_t total = size_t(rows) * ld / 4;
    for (size_t idx = blockIdx.x * size_t(blockDim.x) + threadIdx.x; idx < total; idx += size_t(gridDim.x) * blockDim.x) {
        float4 sum = reinterpret_cast<const float4 *>(partials)[idx];
        for (int s = 1; s < splits; ++s) {
            const float4 p = reinterpret_cast<const float4 *>(partials + size_t(s) * rows_padded * ld)[idx];
            sum.x += p.x; sum.y += p.y; sum.z += p.z; sum.w += p.w;
        }
        if (residual) {
            const float4 r = reinterpret_cast<const float4 *>(residual)[idx];
            sum.x += r.x; sum.y += r.y; sum.z += r.z; sum.w += r.w;
        }
        reinterpret_cast<float4 *>(out)[idx] = sum;
    }
}
