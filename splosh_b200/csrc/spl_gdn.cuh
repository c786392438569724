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
};

// Conv (k = 4, depthwise, no bias) + SiLU over every channel of every run; then the conv history
// of every unit a row writes: the last three raw inputs up to and including that row
// (engine.metal:707-728, 838-849). Grid (ceil(channels / 256), runs), 256 threads.
__global__ void __launch_bounds__(256)
spl_gdn_conv_kernel(const float *__restrict__ proj, const uint16_t *__restrict__ conv_weight, float *conv_state,
                    const uint32_t *__restrict__ runs, const uint32_t *__restrict__ row_read, const uint32_t *__restrict__ row_write,
                    float *act, SplGdnParams p) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= p.channels) return;
    const uint32_t start = runs[blockIdx.y * 3 + 1], length = runs[blockIdx.y * 3 + 2];
    const float *hist = conv_state + (size_t(row_read[start]) * p.channels + c) * 3;
    float x3 = hist[0], x2 = hist[1], x1 = hist[2];
    const float w0 = spl_bf16_to_float(conv_weight[c * 4]), w1 = spl_bf16_to_float(conv_weight[c * 4 + 1]);
    const float w2 = spl_bf16_to_float(conv_weight[c * 4 + 2]), w3 = spl_bf16_to_float(conv_weight[c * 4 + 3]);
    for (uint32_t t = 0; t < length; ++t) {
        const uint32_t row = start + t;
        const float x0 = proj[size_t(row) * p.proj_ld + c];
        const float y = ((w0 * x3 + w1 * x2) + w2 * x1) + w3 * x0;
        act[size_t(row) * p.channels + c] = spl_silu_exact(y);
        if (t + 1 == length || row_write[row + 1] != row_write[row]) {
            float *dst = conv_state + (size_t(row_write[row]) * p.channels + c) * 3;
            dst[0] = x2; dst[1] = x1; dst[2] = x0;
        }
        x3 = x2; x2 = x1; x1 = x0;
    }
}

// The state update S' = S * decay + k * delta with the product rounded on its own, so that the
// replay of a journal entry reproduces the original update bit for bit (engine.metal:654-659).
__device__ __forceinline__ float spl_gdn_update(float s, float decay, float k, float delta) {
    return __fmaf_rn(s, decay, __fmul_rn(k, delta));
}

#define SPL_GDN_TC 16          // tokens prepared per pass
#define SPL_GDN_D 128          // head dim (key and value)

// One thread block per (value head, run). Thread (j = tid / 2, half = tid % 2) keeps 64 elements
// of state row j in registers: i = 8 m + 4 half + e. Per token (engine.metal:763-805):
//   mem = S k;  delta = (v - mem * decay * invK) * beta * invK;  S = S * decay + k (x) delta;
//   o = (S q) * invQ
// then the gated RMSNorm w * o * rsqrt(mean o^2 + eps) * silu(z) rounded to bf16, with its per-64
// sums (engine.metal:812-833). A speculative run leaves a journal entry per row instead of writing
// the state; entries accepted from the previous run are replayed first (engine.metal:744-761).
// Grid (value_heads, runs), 256 threads.
__global__ void __launch_bounds__(256)
spl_gdn_recurrence_kernel(const float *__restrict__ act, const float *__restrict__ proj, const uint16_t *__restrict__ a_log,
                          const uint16_t *__restrict__ dt_bias, const uint16_t *__restrict__ norm_weight, float *state, float *journal,
                          const uint32_t *__restrict__ runs, const uint32_t *__restrict__ run_info, SplOperand core, SplGdnParams p) {
    constexpr int D = SPL_GDN_D, TC = SPL_GDN_TC;
    __shared__ __align__(16) float q_s[TC][D], k_s[TC][D], v_s[TC][D], o_s[TC][D];
    __shared__ float scal[TC][4];        // invQ, invK, decay, beta
    const int h = blockIdx.x, run = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int j = tid >> 1, half = tid & 1;
    const uint32_t slot = runs[run * 3], start = runs[run * 3 + 1], length = runs[run * 3 + 2];
    const bool speculative = run_info[run * 2] != 0;
    const uint32_t pending = run_info[run * 2 + 1];
    const int VH = p.value_heads, KH = p.key_heads, hk = h / (VH / KH);

    float4 S[16];
    float4 *stored = reinterpret_cast<float4 *>(state + ((size_t(slot) * VH + h) * D + j) * D) + half;
#pragma unroll
    for (int m = 0; m < 16; ++m) S[m] = stored[2 * m];

    float *jhead = journal + (size_t(slot) * SPL_JOURNAL_ROWS * VH + h) * SPL_JOURNAL_WIDTH;
    // Replay accepted entries. The entry's k goes through shared memory.
    for (uint32_t e = 0; e < pending; ++e) {
        const float *entry = jhead + size_t(e) * VH * SPL_JOURNAL_WIDTH;
        __syncthreads();
        if (tid < D) k_s[0][tid] = entry[tid];
        __syncthreads();
        const float delta = entry[D + j], decay = entry[2 * D];
#pragma unroll
        for (int m = 0; m < 16; ++m) {
            const float4 kv = *reinterpret_cast<const float4 *>(&k_s[0][8 * m + 4 * half]);
            S[m].x = spl_gdn_update(S[m].x, decay, kv.x, delta); S[m].y = spl_gdn_update(S[m].y, decay, kv.y, delta);
            S[m].z = spl_gdn_update(S[m].z, decay, kv.z, delta); S[m].w = spl_gdn_update(S[m].w, decay, kv.w, delta);
        }
    }
    if (speculative && pending != 0) {
#pragma unroll
        for (int m = 0; m < 16; ++m) stored[2 * m] = S[m];
    }

    const float neg_a = -expf(spl_bf16_to_float(a_log[h])), bias = spl_bf16_to_float(dt_bias[h]);
    for (uint32_t base = 0; base < length; base += TC) {
        const int count = min(uint32_t(TC), length - base);
        __syncthreads();
        // q, k, v of up to TC tokens; one warp a token for the norms.
        for (int idx = tid; idx < count * 3 * (D / 4); idx += 256) {
            const int tt = idx / (3 * (D / 4)), rest = idx % (3 * (D / 4)), kind = rest / (D / 4), i4 = rest % (D / 4);
            const int channel = kind == 0 ? hk * D : kind == 1 ? KH * D + hk * D : 2 * KH * D + h * D;
            const float4 v = *reinterpret_cast<const float4 *>(act + size_t(start + base + tt) * p.channels + channel + i4 * 4);
            float *dst = kind == 0 ? q_s[tt] : kind == 1 ? k_s[tt] : v_s[tt];
            *reinterpret_cast<float4 *>(dst + i4 * 4) = v;
        }
        __syncthreads();
        for (int tt = warp; tt < count; tt += 8) {
            const float4 qv = *reinterpret_cast<const float4 *>(&q_s[tt][lane * 4]);
            const float4 kv = *reinterpret_cast<const float4 *>(&k_s[tt][lane * 4]);
            const float qq = spl_warp_sum(qv.x * qv.x + qv.y * qv.y + qv.z * qv.z + qv.w * qv.w);
            const float kk = spl_warp_sum(kv.x * kv.x + kv.y * kv.y + kv.z * kv.z + kv.w * kv.w);
            if (lane == 0) {
                const size_t row = start + base + tt;
                scal[tt][0] = (1.0f / sqrtf(qq + 1e-6f)) * (1.0f / sqrtf(float(D)));
                scal[tt][1] = 1.0f / sqrtf(kk + 1e-6f);
                const float x = proj[row * p.proj_ld + p.a_offset + h] + bias;
                const float softplus = x > 20.0f ? x : logf(1.0f + expf(x));
                scal[tt][2] = expf(neg_a * softplus);
                scal[tt][3] = spl_sigmoid(proj[row * p.proj_ld + p.b_offset + h]);
            }
        }
        __syncthreads();
        for (int tt = 0; tt < count; ++tt) {
            const float inv_q = scal[tt][0], inv_k = scal[tt][1], decay = scal[tt][2], beta = scal[tt][3];
            float mem = 0.0f;
#pragma unroll
            for (int m = 0; m < 16; ++m) {
                const float4 kv = *reinterpret_cast<const float4 *>(&k_s[tt][8 * m + 4 * half]);
                mem += S[m].x * kv.x + S[m].y * kv.y + S[m].z * kv.z + S[m].w * kv.w;
            }
            mem += __shfl_xor_sync(0xffffffffu, mem, 1);
            const float delta = (v_s[tt][j] - mem * decay * inv_k) * beta * inv_k;
            float o = 0.0f;
#pragma unroll
            for (int m = 0; m < 16; ++m) {
                const float4 kv = *reinterpret_cast<const float4 *>(&k_s[tt][8 * m + 4 * half]);
                const float4 qv = *reinterpret_cast<const float4 *>(&q_s[tt][8 * m + 4 * half]);
                S[m].x = spl_gdn_update(S[m].x, decay, kv.x, delta); S[m].y = spl_gdn_update(S[m].y, decay, kv.y, delta);
                S[m].z = spl_gdn_update(S[m].z, decay, kv.z, delta); S[m].w = spl_gdn_update(S[m].w, decay, kv.w, delta);
                o += S[m].x * qv.x + S[m].y * qv.y + S[m].z * qv.z + S[m].w * qv.w;
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            if (half == 0) o_s[tt][j] = o * inv_q;
            if (speculative) {
                float *entry = jhead + size_t(base + tt) * VH * SPL_JOURNAL_WIDTH;
                if (tid < D) entry[tid] = k_s[tt][tid];
                if (half == 0) entry[D + j] = delta;
                if (tid == 0) entry[2 * D] = decay;
            }
        }
        __syncthreads();
        // Gated RMSNorm and the bf16 operand, one warp a token.
        for (int tt = warp; tt < count; tt += 8) {
            const size_t row = start + base + tt;
            const float4 ov = *reinterpret_cast<const float4 *>(&o_s[tt][lane * 4]);
            const float inv = 1.0f / sqrtf(spl_warp_sum(ov.x * ov.x + ov.y * ov.y + ov.z * ov.z + ov.w * ov.w) / float(D) + p.eps);
            const float4 z = *reinterpret_cast<const float4 *>(proj + row * p.proj_ld + p.z_offset + h * D + lane * 4);
            const uint2 w = *reinterpret_cast<const uint2 *>(norm_weight + lane * 4);
            const float r0 = spl_bf16_to_float(uint16_t(w.x)) * ov.x * inv * spl_silu_exact(z.x);
            const float r1 = spl_bf16_to_float(uint16_t(w.x >> 16)) * ov.y * inv * spl_silu_exact(z.y);
            const float r2 = spl_bf16_to_float(uint16_t(w.y)) * ov.z * inv * spl_silu_exact(z.z);
            const float r3 = spl_bf16_to_float(uint16_t(w.y >> 16)) * ov.w * inv * spl_silu_exact(z.w);
            const uint16_t b0 = spl_float_to_bf16(r0), b1 = spl_float_to_bf16(r1), b2 = spl_float_to_bf16(r2), b3 = spl_float_to_bf16(r3);
            *reinterpret_cast<uint2 *>(core.values + core.at(int(row), h * D + lane * 4)) =
                spl_operand_pack4(spl_bf16_to_float(b0), spl_bf16_to_float(b1), spl_bf16_to_float(b2), spl_bf16_to_float(b3));
            // The following GEMM's per-64 sums: a 128-wide head is two quant groups, sixteen lanes each.
            float gsum = (spl_bf16_to_float(b0) + spl_bf16_to_float(b1)) + (spl_bf16_to_float(b2) + spl_bf16_to_float(b3));
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) gsum += __shfl_xor_sync(0xffffffffu, gsum, o);
            if ((lane & 15) == 0) core.put_sum(int(row), h * 2 + (lane >> 4), gsum);
        }
    }
    if (!speculative) {
#pragma unroll
        for (int m = 0; m < 16; ++m) stored[2 * m] = S[m];
    }
}
