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
__device__ __forceinline__ float spl_round_bf16(float v) { return spl_bf16_to_float(spl_float_to_bf16(v)); }
__device__ __forceinline__ float spl_silu(float x) { return __fdividef(x, 1.0f + expf(-x)); }
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

__device__ __forceinline__ void spl_cp_async16(void *smem, const void *gmem) {
    const uint32_t s = uint32_t(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void spl_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void spl_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void spl_ldmatrix_x4(uint32_t (&r)[4], const void *smem) {
    const uint32_t s = uint32_t(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
// D(16x8, f32) = A(16x16, bf16, row) * B(16x8, bf16, col) + C, with D and C separate registers.
__device__ __forceinline__ void spl_mma_bf16_dc(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, const float (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// Packed pairs of fp32 (Blackwell's two-wide fp32 instructions): each half is an IEEE single operation, so the
// results are bit for bit those of the scalar code.
__device__ __forceinline__ float2 spl_fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(reinterpret_cast<unsigned long long &>(d))
        : "l"(reinterpret_cast<unsigned long long &>(a)), "l"(reinterpret_cast<unsigned long long &>(b)), "l"(reinterpret_cast<unsigned long long &>(c)));
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

// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void spl_mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void spl_mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
