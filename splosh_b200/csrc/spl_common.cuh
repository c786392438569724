// spl_common.cuh — small device helpers shared by the kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SPL_PAGE_TOKENS 256
#define SPL_JOURNAL_ROWS 16
#define SPL_JOURNAL_WIDTH 260

__device__ __forceinline__ float spl_bf16_to_float(uint16_t bits) { return __uint_as_float(uint32_t(bits) << 16); }
// Round to nearest even (the rule of the reference's quantiser, DraftModel.swift:721-724).
__device__ __forceinline__ uint16_t spl_float_to_bf16(float v) {
    const uint32_t bits = __float_as_uint(v);
    return uint16_t((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
}
__device__ __forceinline__ float spl_silu_exact(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float spl_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

__device__ __forceinline__ float spl_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float spl_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Packed pairs of fp32 (Blackwell's two-wide fp32 instructions): each half is an IEEE single operation, so the
// results are bit for bit those of the scalar code.
__device__ __forceinline__ float2 spl_fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(reinterpret_cast<unsigned long long &>(d))
        : "l"(reinterpret_cast<unsigned long long &>(a)), "l"(reinterpret_cast<unsigned long long &>(b)), "l"(reinterpret_cast<unsigned long long &>(c)));
    return d;
}
__device__ __forceinline__ float2 spl_add2(float2 a, float2 b) {
    float2 d;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(reinterpret_cast<unsigned long long &>(d))
        : "l"(reinterpret_cast<unsigned long long &>(a)), "l"(reinterpret_cast<unsigned long long &>(b)));
    return d;
}
__device__ __forceinline__ float2 spl_mul2(float2 a, float2 b) {
    float2 d;
    asm("mul.rn.f32x2 %0, %1, %2;\n" : "=l"(reinterpret_cast<unsigned long long &>(d))
        : "l"(reinterpret_cast<unsigned long long &>(a)), "l"(reinterpret_cast<unsigned long long &>(b)));
    return d;
}

// Programmatic dependent launch. A step's kernels are launched with programmatic stream serialisation: a kernel may be
// scheduled while its predecessor still runs, so each one waits here (for the predecessor to have completed and its
// writes to be visible) before it touches anything a predecessor wrote, and then lets its own successor be scheduled.
// Without the launch attribute both instructions do nothing.
__device__ __forceinline__ void spl_grid_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void spl_grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void spl_grid_begin() { spl_grid_wait(); spl_grid_launch_dependents(); }

// SplitMix64 at an index: output n of the stream that starts at `seed`.
__host__ __device__ __forceinline__ uint64_t spl_splitmix_at(uint64_t seed, uint64_t n) {
    uint64_t z = seed + (n + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
