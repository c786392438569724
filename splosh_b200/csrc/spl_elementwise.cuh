// spl_elementwise.cuh — embedding, RMSNorm, SiLU gate, row gather and arg-max.
#pragma once
#include "spl_common.cuh"
#include "spl_gemm_tc.cuh"

// Embedding: gather a q4 row per token and dequantise it, h = scale * nibble + bias in fp32
// (Sources/Shaders/engine.metal:39-57). The embedding keeps the MLX row-major layout.
// Grid (rows), any block size.
__global__ void spl_embed_q4_kernel(const uint32_t *__restrict__ packed, const uint16_t *__restrict__ scales,
                                    const uint16_t *__restrict__ biases, const uint32_t *__restrict__ tokens, float *out, int hidden) {
    spl_grid_begin();
    const int row = blockIdx.x;
    const uint32_t token = tokens[row];
    const int words = hidden / 8, groups = hidden / 64;
    for (int w = threadIdx.x; w < words; w += blockDim.x) {
        const uint32_t word = packed[size_t(token) * words + w];
        const float s = spl_bf16_to_float(scales[size_t(token) * groups + (w >> 3)]);
        const float b = spl_bf16_to_float(biases[size_t(token) * groups + (w >> 3)]);
        float v[8];
#pragma unroll
        for (int nib = 0; nib < 8; ++nib) v[nib] = __fmaf_rn(s, float((word >> (4 * nib)) & 0xFu), b);
        float4 *dst = reinterpret_cast<float4 *>(out + size_t(row) * hidden + w * 8);
        dst[0] = make_float4(v[0], v[1], v[2], v[3]);
        dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// RMSNorm into a GEMM operand (layout: SplOperand in spl_gemm_tc.cuh): bf16(x * rsqrt(mean x^2 + eps) * w) and the
// per-64 sums of the rounded values, the stored weight applied directly (engine.metal:159-178, 1609-1640; operand
// rounding engine_na.metal:42-57). When `index` is not
// null row r of the output reads input row index[r] (the logit-row gather, engine.metal:273-281).
// Grid (rows), a multiple of 32 threads up to 1,024.
__global__ void __launch_bounds__(1024)
spl_rmsnorm_kernel(const float *input, int in_ld, const uint16_t *__restrict__ weight, const uint32_t *__restrict__ index,
                   SplOperand out, int dim, float eps) {
    spl_grid_begin();
    __shared__ float part[32];
    const int stride = blockDim.x * 4, warps = blockDim.x >> 5;
    const int row = blockIdx.x;
    const float *x = input + size_t(index ? index[row] : row) * in_ld;
    float ss = 0.0f;
    for (int i = threadIdx.x * 4; i < dim; i += stride) {
        const float4 v = *reinterpret_cast<const float4 *>(x + i);
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = spl_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.0f;
    for (int i = 0; i < warps; ++i) total += part[i];
    const float inv = 1.0f / sqrtf(total / float(dim) + eps);
    for (int base = 0; base < dim; base += stride) {
        const int i = base + threadIdx.x * 4;
        float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
        if (i < dim) {
            const float4 v = *reinterpret_cast<const float4 *>(x + i);
            const uint2 w = *reinterpret_cast<const uint2 *>(weight + i);
            const uint16_t b0 = spl_float_to_bf16(v.x * inv * spl_bf16_to_float(uint16_t(w.x)));
            const uint16_t b1 = spl_float_to_bf16(v.y * inv * spl_bf16_to_float(uint16_t(w.x >> 16)));
            const uint16_t b2 = spl_float_to_bf16(v.z * inv * spl_bf16_to_float(uint16_t(w.y)));
            const uint16_t b3 = spl_float_to_bf16(v.w * inv * spl_bf16_to_float(uint16_t(w.y >> 16)));
            r0 = spl_bf16_to_float(b0); r1 = spl_bf16_to_float(b1); r2 = spl_bf16_to_float(b2); r3 = spl_bf16_to_float(b3);
            *reinterpret_cast<uint2 *>(out.values + out.at(row, i)) = spl_operand_pack4(r0, r1, r2, r3);
        }
        // Per-64 sums of the rounded values: sixteen consecutive threads hold one group.
        float gsum = (r0 + r1) + (r2 + r3);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) gsum += __shfl_xor_sync(0xffffffffu, gsum, o);
        if (i < dim && (threadIdx.x & 15) == 0) out.put_sum(row, i / 64, gsum);
    }
}

// Arg-max over [0, limit) per logit row, first index on ties (vDSP_maxvi, Sampler.swift:11-16;
// the vocabulary limit Sampler.swift:94-96). Grid (rows), 1024 threads.
__global__ void __launch_bounds__(1024)
spl_argmax_kernel(const float *__restrict__ logits, int ld, int limit, int32_t *ids) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const float *x = logits + size_t(blockIdx.x) * ld;
    float bv = -INFINITY; int bi = 0x7fffffff;
    // Sixteen-byte loads, four of them in flight a thread (rows start on 16-byte boundaries: the vocabulary is a multiple
    // of 16); ascending i per thread, so strict > keeps the first.
    const int quads = limit / 4;
    int q = threadIdx.x;
    for (; q + 3 * int(blockDim.x) < quads; q += 4 * blockDim.x) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = reinterpret_cast<const float4 *>(x)[q + u * blockDim.x];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = 4 * (q + u * int(blockDim.x));
            if (v[u].x > bv) { bv = v[u].x; bi = i; }
            if (v[u].y > bv) { bv = v[u].y; bi = i + 1; }
            if (v[u].z > bv) { bv = v[u].z; bi = i + 2; }
            if (v[u].w > bv) { bv = v[u].w; bi = i + 3; }
        }
    }
    for (; q < quads; q += blockDim.x) {
        const float4 v = reinterpret_cast<const float4 *>(x)[q];
        const int i = 4 * q;
        if (v.x > bv) { bv = v.x; bi = i; }
        if (v.y > bv) { bv = v.y; bi = i + 1; }
        if (v.z > bv) { bv = v.z; bi = i + 2; }
        if (v.w > bv) { bv = v.w; bi = i + 3; }
    }
    for (int i = 4 * quads + threadIdx.x; i < limit; i += blockDim.x) {
        const float v = x[i];
        if (v > bv) { bv = v; bi = i; }
    }
    if (bi == 0x7fffffff) { bv = -INFINITY; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { best_v[threadIdx.x >> 5] = bv; best_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        bv = best_v[threadIdx.x]; bi = best_i[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        // A row of NaNs or -inf never beats the initial value: index 0, as a scan from 0 would give.
        if (threadIdx.x == 0) ids[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

// The k largest of [0, limit) per logit row in descending order, the lower index first among equal values
// (TopK.select, Sampler.swift:19-52). k rounds of a block-wide selection: round r takes the best element that comes
// strictly after the previous pick in the order (value descending, index ascending); the row stays in L2 between rounds.
// Grid (rows), 1024 threads; ids and values [rows][k].
__global__ void __launch_bounds__(1024)
spl_topk_kernel(const float *__restrict__ logits, int ld, int limit, int k, int32_t *ids, float *values) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    __shared__ float pick_v;
    __shared__ int pick_i;
    const float *x = logits + size_t(blockIdx.x) * ld;
    float last_v = INFINITY; int last_i = -1;
    for (int round = 0; round < k; ++round) {
        float bv = -INFINITY; int bi = 0x7fffffff;
        for (int i = threadIdx.x; i < limit; i += blockDim.x) {
            const float v = x[i];
            const bool after = v < last_v || (v == last_v && i > last_i);          // not taken in an earlier round (NaNs never qualify)
            if (after && v > -INFINITY && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if ((threadIdx.x & 31) == 0) { best_v[threadIdx.x >> 5] = bv; best_i[threadIdx.x >> 5] = bi; }
        __syncthreads();
        if (threadIdx.x < 32) {
            bv = best_v[threadIdx.x]; bi = best_i[threadIdx.x];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (threadIdx.x == 0) {
                // Fewer than k selectable values (a short row, NaNs, -inf): the reference's untouched slots, id 0 at -inf.
                const bool none = bi == 0x7fffffff;
                pick_v = none ? -INFINITY : bv; pick_i = none ? -1 : bi;
                ids[size_t(blockIdx.x) * k + round] = none ? 0 : bi; values[size_t(blockIdx.x) * k + round] = pick_v;
            }
        }
        __syncthreads();
        if (pick_i < 0) { last_v = -INFINITY; last_i = 0x7ffffffe; } else { last_v = pick_v; last_i = pick_i; }
        __syncthreads();
    }
}

// Fill helpers for synthetic contexts.
__global__ void spl_fill_codes_kernel(uint64_t *words, size_t count, uint64_t seed) {
    for (size_t idx = blockIdx.x * size_t(blockDim.x) + threadIdx.x; idx < count; idx += size_t(gridDim.x) * blockDim.x)
        words[idx] = spl_splitmix_at(seed, idx);
}
__global__ void spl_fill_float_kernel(float *data, size_t count, float value) {
    for (size_t idx = blockIdx.x * size_t(blockDim.x) + threadIdx.x; idx < count; idx += size_t(gridDim.x) * blockDim.x) data[idx] = value;
}
__global__ void spl_fill_uniform_kernel(float *data, size_t count, uint64_t seed, float lo, float hi) {
    for (size_t idx = blockIdx.x * size_t(blockDim.x) + threadIdx.x; idx < count; idx += size_t(gridDim.x) * blockDim.x)
        data[idx] = lo + (hi - lo) * (float(spl_splitmix_at(seed, idx) >> 40) * (1.0f / 16777216.0f));
}
