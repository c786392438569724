// spl_gemm_tc.cuh — MLX affine-4 (group 64) dequant-GEMM on the 5th-generation tensor cores.
//
// Stands in for Engine.gemm and the q4 kernels it selects (Sources/SploshRuntime/Engine.swift:1651-1806;
// Sources/Shaders/engine_na.metal:188-428, 862-1011). The numerical contract is the reference's
// accelerator path (engine_na.metal:42-57, 91-103):
//
//   out[r][n] = sum over 64-groups g of ( dot(a[r][g], code[n][g]) * scale[n][g] + sum(a[r][g]) * bias[n][g] ) (+ residual[r][n])
//
// with a the bf16-rounded activations and sum(a) the fp32 per-64 sums of the rounded values.
//
// Shape of the computation. The product is taken transposed, D[n][r] = w[n][k] * a[r][k]^T, so
// that 128 output columns are the M dimension of one tcgen05.mma and the step's rows (16..64 per
// tile) are its N dimension. Per quant group (K = 64, four k16 instructions):
//   * TMA bulk copies bring four groups at a time into shared memory, from two warps that run independently: one
//     copies the weights (16 KiB of codes and 2 KiB of scale/bias words, a ring handed back as soon as the codes are
//     in registers), the other the activations' slice (held until the tensor core has finished with it) and the
//     tiles of split means, each of which serves sixteen groups;
//   * dequant warps (one thread per output column, four sets of four warps taking units of two groups in turn)
//     turn the codes into exact fp16 values scale * (code - 8), sixteen registers at a time, and write them into
//     tensor memory as the A operand (tcgen05.st): weights never pass through shared memory expanded and are
//     never re-read. A pair of weights costs one shift, one logic operation and one fused multiply-add;
//   * the activations' producer already wrote them (bf16-rounded, held as fp16) in the
//     128-byte-swizzled K-major image the tensor core reads as the B operand;
//   * two warps issue the tcgen05.mma, a unit each in turn (eight k16 instructions and a ninth for the unit's
//     share of the bias term), into an accumulator each; the accumulators stay in tensor memory for the whole
//     contraction. The warps run their loops and waits whole, with one elected lane issuing;
//   * the bias term, (bias + 8 scale) * sum(a) per group, comes from exact fp16 pairs of (64 bias, 512 scale)
//     in tensor memory and the group means split in two fp16 numbers;
//   * at the end every dequant warp reads its share of the accumulators (tcgen05.ld) and writes the output.
// Everything is ordered by mbarriers. Every wait is bounded: a wait that runs out sets an error
// word and the block unwinds, still releasing its tensor memory.
//
// Device layout of a weight (private to this library): for each tile of 128 output columns and each
// group, 4,096 bytes of codes [half h][column n][16 bytes] holding k = 64 g + 32 h + 0..31, each
// 32-bit word's nibbles in the order [k0 k2 k4 k6 k1 k3 k5 k7] so that (word >> 4j) & 0x000F000F is
// the pair of codes (k_2j, k_2j+1); and 128 words (scale | bias << 16) per (tile, group).
#pragma once
#include "spl_common.cuh"

struct SplQ4Dev {
    int n = 0;            // logical output columns
    int ld = 0;           // columns rounded up to 16: the width of an output row
    int tiles = 0;        // 128-column tiles
    int k = 0;            // contraction length, a multiple of 64
    int interleave = 0;   // > 0 for a fused gate|up tensor of 2 x interleave columns: tile t holds elements [64 t, 64 t + 64), in runs of 32 columns = sixteen gate columns then the sixteen up columns of the same elements
    uint32_t *codes = nullptr;      // [tiles][k/64][2][128][4] words
    uint32_t *sb = nullptr;         // [tiles][k/64][128] words
    size_t bytes() const { return size_t(ld) * (k / 64) * 36; }   // algorithmic: 32 B of codes + 4 B of scale and bias per (column, group)
    size_t device_bytes() const { return size_t(tiles) * (k / 64) * (4096 + 512); }
};

// ---- operand (B side) layout ------------------------------------------------------------------
// A GEMM's activation operand is the bf16-rounded activations held as fp16 (the tensor-core instruction wants
// both operands in one 16-bit format, and the weights need fp16's 11 bits). A bf16 value of magnitude
// 2^-14 .. 65504 is exact in fp16; a smaller one moves by at most 2^-25, below the fp32 accumulator's own
// rounding for activations of order one. The per-64 sums are taken from the bf16 values themselves.
// The operand is cut in 64-wide groups and in row blocks of RN rows (RN = 16, 32 or 64, fixed per step). Block (g, rb) is RN * 128 bytes: row r at (r / 8) * 1024 + (r % 8) * 128,
// its eight 16-byte units XOR-swizzled by r % 8: the canonical K-major SWIZZLE_128B image. The
// per-64 sums sit beside it as tiles of the same shape, sixteen groups to a tile (SplOperand::put_sum).
// Four bf16-rounded values (as floats) -> four fp16 in two words.
__device__ __forceinline__ uint2 spl_operand_pack4(float r0, float r1, float r2, float r3) {
    const __half2 lo = __floats2half2_rn(r0, r1), hi = __floats2half2_rn(r2, r3);
    return make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
}

// Floats (4-byte cells) of the split-means array of an operand of `rows_padded` rows and contraction k.
__host__ __device__ constexpr size_t spl_operand_sums_floats(size_t rows_padded, size_t k) { return ((k / 64 + 15) / 16) * rows_padded * 32; }

struct SplOperand {
    __nv_bfloat16 *values;      // 16-bit cells (fp16 bits of the bf16-rounded values)
    float *sums;               // tiles of split means, see put_sum
    int rn, blocks;            // rows per block (16, 32, 64 or 128: a power of two), row blocks
    __device__ __forceinline__ size_t at(int row, int k) const {
        const int g = k >> 6, kk = k & 63, rb = row >> (31 - __clz(rn)), r = row & (rn - 1);
        return (size_t(g) * blocks + rb) * (size_t(rn) * 64) + size_t(r >> 3) * 512 + (r & 7) * 64 + (((kk >> 3) ^ (r & 7)) << 3) + (kk & 7);
    }
    // The group's sum as the B operand of the GEMM's second term: (hi, lo, hi, lo) with hi + lo = sum / 64 in two fp16
    // numbers, at contraction index 4 (g % 16) of row `row` of tile (g / 16, row block), the tiles laid out as `at` lays out
    // the values. (`sums` is that array; the name is kept from the fp32 sums it replaces.)
    __device__ __forceinline__ void put_sum(int row, int g, float sum) const {
        const float mean = sum * 0.015625f;
        const __half hi = __float2half_rn(mean), lo = __float2half_rn(mean - __half2float(hi));
        const __half2 pair = __halves2half2(hi, lo);
        const uint32_t bits = *reinterpret_cast<const uint32_t *>(&pair);
        const int rb = row >> (31 - __clz(rn)), r = row & (rn - 1), kk = 4 * (g & 15);
        __half *tile = reinterpret_cast<__half *>(sums) + (size_t(g >> 4) * blocks + rb) * (size_t(rn) * 64);
        *reinterpret_cast<uint2 *>(tile + size_t(r >> 3) * 512 + (r & 7) * 64 + (((kk >> 3) ^ (r & 7)) << 3) + (kk & 7)) = make_uint2(bits, bits);
    }
};

// ---- repack: MLX row-major -> tile layout, rows [n0, n0 + rows) of a fused tensor ------------
__global__ void spl_repack_q4_kernel(const uint32_t *__restrict__ packed, const uint16_t *__restrict__ scales,
                                     const uint16_t *__restrict__ biases, int rows, int k, uint32_t *codes, uint32_t *sb, int n0, int *out_of_range, int interleave) {
    const int groups = k / 64, words = k / 8;
    const size_t total = size_t(rows) * words;
    for (size_t idx = blockIdx.x * size_t(blockDim.x) + threadIdx.x; idx < total; idx += size_t(gridDim.x) * blockDim.x) {
        const int row = int(idx / words), w = int(idx % words);
        const uint32_t src = packed[idx];
        // nibbles [0 1 2 3 4 5 6 7] -> [0 2 4 6 1 3 5 7]
        uint32_t dst = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            dst |= ((src >> (8 * j)) & 0xFu) << (4 * j);
            dst |= ((src >> (8 * j + 4)) & 0xFu) << (4 * j + 16);
        }
        int n = n0 + row;
        if (interleave > 0) { const int c = n < interleave ? n : n - interleave; n = (c >> 6) * 128 + ((c & 63) >> 4) * 32 + (n < interleave ? 0 : 16) + (c & 15); }
        const int tile = n >> 7, col = n & 127, g = w >> 3, h = (w >> 2) & 1, j = w & 3;
        codes[(((size_t(tile) * groups + g) * 2 + h) * 128 + col) * 4 + j] = dst;
        if ((w & 7) == 0) {
            const uint16_t sbits = scales[size_t(row) * groups + g];
            sb[(size_t(tile) * groups + g) * 128 + col] = uint32_t(sbits) | (uint32_t(biases[size_t(row) * groups + g]) << 16);
            // The GEMM holds scale * (code - 8) in fp16 and forms it also from scale / 16: the scale must be zero, or at least
            // 2^-13 (scale / 16 keeps its eight bits); it also holds 512 scale and 64 bias in fp16.
            const float sc = fabsf(spl_bf16_to_float(sbits));
            const float bi = fabsf(spl_bf16_to_float(biases[size_t(row) * groups + g]));
            if (!((sc == 0.0f || (sc >= 1.220703125e-04f && sc <= 127.0f)) && bi <= 1023.0f)) atomicExch(out_of_range, 1);
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

// ---- PTX wrappers -----------------------------------------------------------------------------
// Every wait inside a kernel is bounded in time: a wait that outlasts the budget returns false, the kernel sets its error
// word and unwinds. The budget is a device variable so that a test can shorten it (spl_debug_wait_budget).
#define SPL_WAIT_HINT_NS 2000u        // suspend-time hint of one poll (100 to 10,000 ns measured: no difference)
__device__ unsigned long long spl_wait_budget_ns = 250ull * 1000 * 1000;

__device__ __forceinline__ uint32_t spl_smem_addr(const void *p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ unsigned long long spl_global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    return t;
}
__device__ __forceinline__ void spl_mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(spl_smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void spl_mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(spl_smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void spl_mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(spl_smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool spl_mbar_try(uint32_t addr, uint32_t parity) {
    uint32_t done;
    // The hint lets the hardware keep the thread suspended (off the issue slots its neighbours need) for up to that many
    // nanoseconds per poll; completion of the phase wakes it at once.
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done) : "r"(addr), "r"(parity), "r"(SPL_WAIT_HINT_NS) : "memory");
    return done != 0;
}
// Bounded wait on a phase parity. Returns false when the time budget ran out, or when `abort` (a word of the block's
// shared memory that any role sets when its own wait ran out) is set: one lost arrival then unwinds the whole block
// within one budget instead of one budget per waiting role.
__device__ __forceinline__ bool spl_mbar_wait(uint64_t *bar, uint32_t parity, const volatile int *abort = nullptr) {
    const uint32_t addr = spl_smem_addr(bar);
    // The ordinary case ends within these polls (each may suspend for the hint's time); the clock is read only after them.
    // (The poll loops must stay loops: unrolled, every wait in a kernel becomes dozens of copies of itself and the
    // kernels' hot loops no longer fit the instruction cache.)
    // The clock sits far from the SMs: a thread that reads it is gone for a microsecond, which a hand-over between roles
    // cannot afford, so it is not looked at until a wait has outlasted any ordinary one by far.
#pragma unroll 1
    for (int spin = 0; spin < (1 << 14); ++spin)
        if (spl_mbar_try(addr, parity)) return true;
    const unsigned long long t0 = spl_global_timer(), budget = spl_wait_budget_ns;
    for (;;) {
#pragma unroll 1
        for (int spin = 0; spin < 32; ++spin)
            if (spl_mbar_try(addr, parity)) return true;
        if (abort && *abort) return false;
        if (spl_global_timer() - t0 > budget) return false;
    }
}
__device__ __forceinline__ void spl_bulk_g2s(void *smem, const void *gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(spl_smem_addr(smem)), "l"(gmem), "r"(bytes), "r"(spl_smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void spl_tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void spl_tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void spl_tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(spl_smem_addr(bar)) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor]; one thread issues.
__device__ __forceinline__ void spl_tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the accumulate flag fixed at one (no predicate to compute in the issuing loop).
__device__ __forceinline__ void spl_tc_mma_ts_acc(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
    asm volatile("{\n .reg .pred p;\n setp.eq.u32 p, 1, 1;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc) : "memory");
}
// One lane of a converged warp. The tensor-core instructions of a kernel are issued from loops that the WHOLE warp runs
// (waits included), with only the instruction itself under this predicate: with warp-uniform control flow the
// descriptors stay in uniform registers and one warp issues a k16 instruction every 32 cycles (the tensor pipe's own
// rate at N = 64); the same loop under `if (lane == 0)` measured 51-57 cycles an instruction at best and 140-150 with a
// few run-time conditions between the instructions.
__device__ __forceinline__ bool spl_elect_one() {
    uint32_t pred;
    asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
    return pred != 0;
}
// A bounded wait by every lane of a converged warp, with one answer for the warp (a lane that gave up alone would leave
// the warp's later warp-wide instructions waiting for it).
__device__ __forceinline__ bool spl_mbar_wait_warp(uint64_t *bar, uint32_t parity, const volatile int *abort = nullptr) {
    return __all_sync(0xffffffffu, spl_mbar_wait(bar, parity, abort));
}
// K-major, 128-byte swizzle, rows of 128 bytes, eight-row groups 1,024 bytes apart.
__device__ __forceinline__ uint64_t spl_tc_desc_sw128(uint32_t smem_byte_addr) {
    uint64_t d = 0;
    d |= uint64_t((smem_byte_addr & 0x3FFFFu) >> 4);        // start address
    d |= uint64_t(1) << 16;                                 // leading byte offset (unused with this swizzle)
    d |= uint64_t(1024 >> 4) << 32;                         // stride byte offset
    d |= uint64_t(1) << 46;                                 // descriptor version of sm_100
    d |= uint64_t(2) << 61;                                 // SWIZZLE_128B
    return d;
}
// kind::f16 instruction descriptor: fp32 accumulate, A and B fp16 (format 0), both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t spl_tc_idesc(int n) {
    return (1u << 4) | (0u << 7) | (0u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(128 >> 4) << 24);
}

__device__ __forceinline__ void spl_tc_ld16(uint32_t (&r)[16], uint32_t taddr) {
    // The load and its wait are one statement: the registers are defined only after the wait, and a separate
    // wait statement would not stop the compiler from scheduling their readers before it.
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                 "tcgen05.wait::ld.sync.aligned;\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]) : "r"(taddr));
}
__device__ __forceinline__ void spl_tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void spl_tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
                   "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void spl_tc_st4(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(taddr), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}
// The first wait of a launch that ran out leaves its place in the error words: [1] which wait (the codes are listed where
// the engine turns them into text), [2] the stage or unit it was at, [3] the block.
__device__ __forceinline__ void spl_note_wait(int *error_flag, int code, int where) {
    if (atomicCAS(error_flag + 1, 0, code) == 0) { error_flag[2] = where; error_flag[3] = int(blockIdx.x) | (int(blockIdx.z) << 16); }
}
// Barriers among some of a block's threads, with the barrier's number in the instruction itself so that the compiler
// counts it: number 1 for all dequant threads of the q4 GEMM, 2 + set for the 128 threads of one dequant set.
template <int ID, int COUNT> __device__ __forceinline__ void spl_named_barrier() { asm volatile("bar.sync %0, %1;\n" ::"n"(ID), "n"(COUNT) : "memory"); }
__device__ __forceinline__ void spl_set_barrier(int set) {
    if (set == 0) spl_named_barrier<2, 128>();
    else if (set == 1) spl_named_barrier<3, 128>();
    else if (set == 2) spl_named_barrier<4, 128>();
    else spl_named_barrier<5, 128>();
}

// ---- the kernel -------------------------------------------------------------------------------
// How the contract is kept with everything on the tensor cores. With c the 4-bit code,
//   scale * c + bias = scale * (c - 8) + (bias + 8 * scale).
// First term. scale is bf16 (8 significant bits) and |c - 8| <= 8, so scale * (c - 8) has at most 11 significant
// bits: it is EXACT in fp16 (for scales in the range checked when a weight is loaded). The tensor cores multiply
// these exact weights by the bf16-rounded activations (held as fp16) and accumulate every group in fp32.
// Second term, (bias + 8 scale) * sum(a) per group: one more k16 instruction per four groups. Its A operand holds,
// per group, the pairs (64 bias, 64 bias) and (512 scale, 512 scale) (exact in fp16 for |bias| <= 1023 and
// scale <= 127, checked at load); its B operand holds, per row and group, (hi, lo, hi, lo) with hi + lo the
// group's mean sum(a) / 64 split in two fp16 numbers by the operand's producer (SplOperand::put_sum). The four
// products add up to (bias + 8 scale) * sum(a) to within 2^-22 of the term, beside the fp32 accumulator's own 2^-24.
// The result is the reference's sum of per-group terms up to the order of fp32 additions.
//
// How the work is cut. Every tile's contraction is cut in `splits` equal runs of stages (a stage = four groups, two in
// the wide block): one block per (tile, split, row block). With one split a block owns its tile and writes the output
// itself, fused forms included. With more, every block leaves its partial sums in a slot of its own and a second
// kernel (spl_gemm_fixup_kernel) adds a tile's slots in the order of the contraction, so the sum's order is fixed, and
// does what follows the sum: residual, output, the next deferred norm's operand. The GEMM block's output stage is
// then stores only. That matters: a block reaches it while the other blocks still stream weights at the memory's full
// rate, and a load issued then waits behind megabytes of queued copies (a few microseconds a round trip); an earlier
// form that met in the kernel (tickets, the last arriver adding the slots) paid six such trips a tile.
#define SPL_TC_SUPER 4           // groups per shared-memory stage of the GGUF kernel and of the narrow q4 blocks: one bulk copy brings 256 of the contraction
#define SPL_TC_AUNITS 5          // A operand slots in tensor memory, a unit (two groups, 64 columns) each, with 8 columns each for the second term
#define SPL_TC_SETS 4            // dequant sets of four warps (a warp writes the tensor-memory lanes of its index mod 4); they take the units in turn
#define SPL_TC_DEQUANT (SPL_TC_SETS * 128)
#define SPL_TC_THREADS (SPL_TC_DEQUANT + 128)       // the sets; then a warp that copies weights, a tensor-core issue warp, a warp that copies activations, the other issue warp
// The pair form of the 128-row block (prefill chunks of two row blocks and more): a block works on two tiles of the weight
// against one stream of activations, a tile per issuing warp and accumulator. At the tensor pipe's full rate a 128 x 128 block
// needs 64 bytes of activations a cycle from L2 (an instruction of K = 16 reads 4 KB of them and lasts 64 cycles), 148 SMs
// three times what L2 delivers; with two tiles the same bytes feed twice the instructions. Tensor memory: two accumulators of
// 128 columns, three operand slots of 64 with their 8 second-term columns (472 of 512). Shared memory: three stages of
// activations (two groups: 32 KB), four of codes (two groups of each tile: 18 KB), the two tiles of split means.
#define SPL_TC_PAIR_BSTAGES 3
#define SPL_TC_PAIR_CSTAGES 4
#define SPL_TC_PAIR_AUNITS 3

// The shape of a block by its row count RN (the N of its tcgen05.mma). Narrow blocks (16, 32, 64 rows: decode and verify
// steps) take stages of four groups and two issuing warps with an accumulator each. The wide block (128 rows: prefill
// chunks, one instruction is 128 x 128 x 16) takes stages of two groups, so that four stages of activations still fit
// in shared memory, and one issuing warp with one accumulator: an instruction then keeps the tensor pipe 64 cycles and
// one warp issues at that rate.
__host__ __device__ constexpr int spl_tc_super(int rn) { return rn >= 128 ? 2 : 4; }          // groups per stage
__host__ __device__ constexpr int spl_tc_issuers(int rn) { return rn >= 128 ? 1 : 2; }        // issuing warps = units per stage
// Stages of activations: held until the tensor core has finished with them. Stages of codes with their scale/bias
// words: handed back as soon as they are in registers.
__host__ __device__ constexpr int spl_tc_bstages(int rn) { return rn >= 64 ? 4 : 6; }
__host__ __device__ constexpr int spl_tc_cstages(int rn) { return rn >= 64 ? 4 : 6; }
__host__ __device__ constexpr size_t spl_tc_bstage_bytes(int rn) { return size_t(spl_tc_super(rn)) * size_t(rn) * 128; }
#define SPL_TC_CONTROL_BYTES 4096       // barriers, row factors, the output stage's exchange cells
__host__ __device__ constexpr size_t spl_tc_smem_bytes(int rn) {
    return 1024 /* alignment slack */ + size_t(spl_tc_cstages(rn)) * spl_tc_super(rn) * (4096 + 512) + size_t(spl_tc_bstages(rn)) * spl_tc_bstage_bytes(rn)
           + size_t(2) * rn * 128 /* tiles of split means */ + SPL_TC_CONTROL_BYTES;
}
__host__ __device__ constexpr size_t spl_tc_pair_smem_bytes() {
    return 1024 + size_t(SPL_TC_PAIR_CSTAGES) * SPL_TC_SUPER * (4096 + 512) + size_t(SPL_TC_PAIR_BSTAGES) * 2 * 128 * 128 + size_t(2) * 128 * 128 + SPL_TC_CONTROL_BYTES;
}
// Floats of the slot array a launch may write: none when every tile is one piece, else a slot of rn x 128 a block.
__host__ __device__ constexpr size_t spl_tc_slot_floats(int pieces, int splits, int row_blocks, int rn) {
    return splits <= 1 ? 0 : size_t(pieces) * row_blocks * rn * 128;
}

struct SplGemmArgs {
    const uint32_t *codes, *sb;            // the weight (SplQ4Dev)
    const __nv_bfloat16 *act;              // the operand (SplOperand layout) and its tiles of split means
    const float *act_sums;
    float *out;                            // [rows][out_ld]
    const float *residual;                 // null, or [rows][out_ld] added to the output (may be `out`)
    float *slots;                          // partial sums of cut tiles: [row block][piece = tile x splits + split][RN][128]
    int *error_flag;
    int out_ld, rows, op_blocks, tiles, stages_per_tile, interleave, fuse;
    int pieces, row_blocks;                // the grid: pieces x row blocks, the row block the fast index
    int drop_stage;                        // -1, or (a test of the timeout path) the stage of every block's weights that is never copied
    int splits;                            // every tile is cut in this many pieces (pieces = tiles x splits)
    SplOperand act_out;                    // fuse: the SiLU-gated activation, written as the next GEMM's operand
    // The operand came from a deferred norm: out = sum * rsqrt(mean of the row's squares + eps). [row][in_groups] squares.
    const float *in_squares; int in_groups; float in_dim, eps;
    // The output feeds a deferred norm: also write bf16(out * emit_weight) as an operand, with its sums and the squares of out.
    const uint16_t *emit_weight; SplOperand emit_out; float *emit_squares;
};

// Grid (pieces x row blocks). Block x works on piece x / row_blocks of the weight for row block x % row_blocks: the
// blocks that run at the same time are then the row blocks of a few pieces, and a piece comes from HBM once and
// from L2 for the other row blocks. See "How the work is cut" above.
#define SPL_TC_PLAIN 0
#define SPL_TC_EMIT 1
#define SPL_TC_FUSE 2


// What a dequant thread needs in the output stage (spl_tc_output_stage): its place in the block and the block's
// place in the launch, the accumulators, and the block's shared control words.
struct SplTcOutput {
    uint32_t tmem_d, lane_base;
    int rb, c, tile, set, quarter, col, lane;
    uint64_t *finished;
    int *abort_word;
    float *row_factor, *cells;
};

// The output stage of a block, run by all 512 dequant threads (its barriers are theirs). Kept out of line: inlined
// into the conversion loop it cost that loop its registers. The sixteen rows a thread holds stay in registers
// (every loop over them is unrolled). Returns the thread's `ok`.
template <int RN, int MODE>
__device__ __noinline__ bool spl_tc_output_stage(const SplGemmArgs &args, const SplTcOutput &o, bool ok) {
    // The arguments by value: read through the reference, every store of this function could have changed them as far as the
    // compiler knows, and each re-read is a trip to the parameter space.
    SplGemmArgs a;
    a.out = args.out; a.residual = args.residual; a.slots = args.slots; a.error_flag = args.error_flag;
    a.out_ld = args.out_ld; a.rows = args.rows; a.tiles = args.tiles; a.interleave = args.interleave; a.splits = args.splits; a.pieces = args.pieces;
    a.act_out.values = args.act_out.values; a.act_out.sums = args.act_out.sums; a.act_out.rn = args.act_out.rn; a.act_out.blocks = args.act_out.blocks;
    a.in_squares = args.in_squares;
    a.emit_weight = args.emit_weight; a.emit_squares = args.emit_squares;
    a.emit_out.values = args.emit_out.values; a.emit_out.sums = args.emit_out.sums; a.emit_out.rn = args.emit_out.rn; a.emit_out.blocks = args.emit_out.blocks;
    constexpr int NW = spl_tc_issuers(RN);
    const uint32_t tmem_d = o.tmem_d, lane_base = o.lane_base;
    const int rb = o.rb, tile = o.tile, set = o.set, quarter = o.quarter, col = o.col, lane = o.lane;
    int *abort_word = o.abort_word;
    const volatile int *abort = abort_word;
    const float *row_factor = o.row_factor;
    float *cells = o.cells;
    if (ok && !spl_mbar_wait_warp(o.finished, 0, abort)) { ok = false; if (!*abort && lane == 0) spl_note_wait(a.error_flag, 40, 0); *abort_word = 1; }
    if (ok) spl_tc_fence_after();
    float *my_slot = a.slots + (size_t(rb) * a.pieces + o.c) * (RN * 128);
    // A set takes the sixteen-row chunks set, set + 4, ...
#pragma unroll 1
    for (int c0 = set * 16; c0 < RN; c0 += SPL_TC_SETS * 16) {
        float total[16];
#pragma unroll
        for (int r = 0; r < 16; ++r) total[r] = 0.0f;
        if (ok) {
            uint32_t v0[16];
            spl_tc_ld16(v0, tmem_d + lane_base + c0);
#pragma unroll
            for (int r = 0; r < 16; ++r) total[r] = __uint_as_float(v0[r]);
            if (NW == 2) {
                uint32_t v1[16];
                spl_tc_ld16(v1, tmem_d + lane_base + RN + c0);
#pragma unroll
                for (int r = 0; r < 16; ++r) total[r] += __uint_as_float(v1[r]);
            }
        }
        // The rows' factors of a deferred norm: a cut tile's partial sums are scaled one by one, so their sum is.
        if (a.in_squares)
#pragma unroll
            for (int r = 0; r < 16; ++r) total[r] *= row_factor[c0 + r];
        if (a.splits > 1) {
            if (ok)
#pragma unroll
                for (int r = 0; r < 16; ++r) my_slot[(c0 + r) * 128 + col] = total[r];
            continue;
        }
        if (MODE == SPL_TC_FUSE) {
            // A fused gate|up tensor: in each run of 32 columns of a tile the first sixteen are gate columns and the
            // next sixteen the up columns of the same elements, so a lane and the lane sixteen further hold a pair.
            // They exchange halves of their rows; each then forms act = bf16(silu(gate) * up) for eight rows
            // (Sources/Shaders/engine.metal:200-219) and writes it straight into the next GEMM's operand with its per-64 sums.
            // The operand's row blocks are this kernel's (rn = RN) and the eight rows are one eight-row group of the
            // swizzled tile: one base address, no divisions.
            const int element = tile * 64 + quarter * 16 + (lane & 15), r_first = lane < 16 ? 0 : 8, kk = element & 63;
            const bool keep = ok && element < a.interleave;
            __half *base = reinterpret_cast<__half *>(a.act_out.values) + (size_t(element >> 6) * a.act_out.blocks + rb) * (size_t(RN) * 64)
                           + size_t((c0 + r_first) >> 3) * 512 + (kk & 7);
            float v[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float mine = lane < 16 ? total[r] : total[r + 8];
                const float other = __shfl_xor_sync(0xffffffffu, lane < 16 ? total[r + 8] : total[r], 16);
                const float gate = lane < 16 ? mine : other, up = lane < 16 ? other : mine;
                const bool valid = keep && rb * RN + c0 + r_first + r < a.rows;
                v[r] = valid ? spl_bf16_to_float(spl_float_to_bf16(spl_silu_exact(gate) * up)) : 0.0f;
            }
#pragma unroll
            for (int r = 0; r < 8; ++r)
                if (keep && rb * RN + c0 + r_first + r < a.rows) base[r * 64 + ((((kk >> 3) ^ r) & 7) << 3)] = __float2half_rn(v[r]);
            // The sums in one fixed order: a butterfly over the sixteen elements a half warp holds, then the four quarters.
#pragma unroll
            for (int off = 8; off > 0; off >>= 1)
#pragma unroll
                for (int r = 0; r < 8; ++r) v[r] += __shfl_xor_sync(0xffffffffu, v[r], off);
            if ((lane & 15) == 0)
#pragma unroll
                for (int r = 0; r < 8; ++r) cells[((set * 4 + quarter) * 16 + r_first + r) * 2] = v[r];
            spl_set_barrier(set);
            if (quarter == 0 && lane < 16) {
                const int row = rb * RN + c0 + lane;
                const float *cell = cells + (set * 4 * 16 + lane) * 2;
                if (ok && row < a.rows) a.act_out.put_sum(row, tile, ((cell[0] + cell[32]) + cell[64]) + cell[96]);
            }
            spl_set_barrier(set);
        } else {
            const int n = tile * 128 + col;
            int n_out = n;
            if (a.interleave > 0) { const int e = tile * 64 + (col >> 5) * 16 + (col & 15); n_out = ((col & 16) ? a.interleave : 0) + e; }
            const bool inside = ok && (a.interleave > 0 ? (tile * 64 + (col >> 5) * 16 + (col & 15)) < a.interleave : n < a.out_ld);
            const bool emit = MODE == SPL_TC_EMIT;
            // Every load first (one trip to memory for all of them), then the stores.
            float x[16];
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                const int row = rb * RN + c0 + r;
                x[r] = (inside && a.residual && row < a.rows) ? a.residual[size_t(row) * a.out_ld + n_out] : 0.0f;
            }
            const float w = (emit && inside) ? spl_bf16_to_float(a.emit_weight[n]) : 0.0f;
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                const bool valid = inside && rb * RN + c0 + r < a.rows;
                x[r] = valid ? total[r] + x[r] : 0.0f;
                if (valid) a.out[size_t(rb * RN + c0 + r) * a.out_ld + n_out] = x[r];
            }
            if (emit) {
                // The output feeds a deferred norm (Sources/Shaders/engine_na.metal:365-415): bf16(x * w) as the next operand
                // (two eight-row groups of the swizzled tile of row block rb), its per-64 sums, and the squares of x per 64 columns.
                const int kk = n & 63;
                __half *base = reinterpret_cast<__half *>(a.emit_out.values) + (size_t(n >> 6) * a.emit_out.blocks + rb) * (size_t(RN) * 64) + size_t(c0 >> 3) * 512 + (kk & 7);
                float v[16];
#pragma unroll
                for (int r = 0; r < 16; ++r) {
                    v[r] = spl_bf16_to_float(spl_float_to_bf16(x[r] * w));
                    if (inside && rb * RN + c0 + r < a.rows) base[(r >> 3) * 512 + (r & 7) * 64 + ((((kk >> 3) ^ r) & 7) << 3)] = __float2half_rn(v[r]);
                    x[r] *= x[r];
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1)
#pragma unroll
                    for (int r = 0; r < 16; ++r) { v[r] += __shfl_xor_sync(0xffffffffu, v[r], off); x[r] += __shfl_xor_sync(0xffffffffu, x[r], off); }
#pragma unroll
                for (int r = 0; r < 16; ++r)
                    if (lane == r) { cells[((set * 4 + quarter) * 16 + r) * 2] = v[r]; cells[((set * 4 + quarter) * 16 + r) * 2 + 1] = x[r]; }
                spl_set_barrier(set);
                if (quarter < 2 && lane < 16) {            // warp 0 of the set: the tile's first 64 columns; warp 1: its last
                    const int row = rb * RN + c0 + lane, group = tile * 2 + quarter;
                    const float *cell = cells + ((set * 4 + 2 * quarter) * 16 + lane) * 2;
                    if (ok && row < a.rows && group * 64 < a.out_ld) {
                        a.emit_out.put_sum(row, group, cell[0] + cell[32]);
                        a.emit_squares[size_t(row) * (a.out_ld / 64) + group] = cell[1] + cell[33];
                    }
                }
                spl_set_barrier(set);
            }
        }
    }
    return ok;
}

// MODE: what the output stage does besides the sum (one kernel each, so that a block's once-only code stays small):
// 0 plain output (+ residual), 1 also the next deferred norm's operand and squares, 2 the SiLU gate of a fused gate|up tensor.
template <int RN, int MODE>
__global__ void __launch_bounds__(SPL_TC_THREADS, 1)
spl_gemm_q4_tc_kernel(const __grid_constant__ SplGemmArgs a) {
    constexpr int BST = spl_tc_bstages(RN), CST = spl_tc_cstages(RN), AUN = SPL_TC_AUNITS, SUPER = spl_tc_super(RN), UPS = SUPER / 2, NW = spl_tc_issuers(RN);
    static_assert(UPS == NW, "every issuing warp takes one unit of every stage");
    constexpr int BTILE = SUPER * RN * 128, WSTAGE = SUPER * 4096, QSTAGE = SUPER * 128, TTILE = RN * 128;
    extern __shared__ unsigned char spl_tc_smem_raw[];
    // The swizzled activation tiles must sit on 1,024-byte boundaries.
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(spl_tc_smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char *b_ring = smem;                                                       // [BST][SUPER][RN * 128] activations
    unsigned char *t_ring = b_ring + size_t(BST) * BTILE;                               // [2][RN * 128] split means of sixteen groups
    unsigned char *w_ring = t_ring + 2 * TTILE;                                         // [CST][SUPER][4096] codes
    uint32_t *q_ring = reinterpret_cast<uint32_t *>(w_ring + size_t(CST) * WSTAGE);     // [CST][SUPER][128] scale | bias << 16
    uint64_t *bars = reinterpret_cast<uint64_t *>(q_ring + CST * QSTAGE);
    uint64_t *full_c = bars, *empty_c = full_c + CST, *full_b = empty_c + CST, *done = full_b + BST;      // done[un % 16]: the instructions that read unit un have completed
    uint64_t *full_a = done + 16, *full_t = full_a + 2 * AUN, *empty_t = full_t + 2, *finished = empty_t + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(finished + 1);
    int *abort_word = reinterpret_cast<int *>(tmem_slot + 1);
    float *row_factor = reinterpret_cast<float *>(bars) + 256;                          // [128] at byte 1,024 of the control area
    float *cells = row_factor + 128;                                                    // [SETS][4 warps][16 rows][2] the output stage's exchange

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int W_COPY = SPL_TC_SETS * 4, W_MMA0 = W_COPY + 1, W_COPYB = W_COPY + 2, W_MMA1 = W_COPY + 3;
    const int rb = int(blockIdx.x) % a.row_blocks, c = int(blockIdx.x) / a.row_blocks, row_blocks = a.op_blocks, S = a.stages_per_tile;
    // This block's piece: an equal share of the stages of its tile (the host keeps splits <= S, so no piece is empty).
    // Stages are counted along the weight array: stage w is stage w % S of tile w / S.
    const int tile = c / a.splits, split = c % a.splits;
    const int w0 = tile * S + S * split / a.splits, w1 = tile * S + S * (split + 1) / a.splits, stages = w1 - w0;
    // Every block of a GEMM reads the same activation lines. Blocks therefore walk their piece from different starting
    // points (the order of a sum of groups does not matter beyond fp32 rounding, and it is a fixed function of the
    // piece), so that at any moment they ask L2 for different lines: step i of the block is stage place(i) of its piece.
    const int rot = stages > 1 ? int((uint32_t(c) * 2654435761u >> 12) % uint32_t(stages)) : 0;
    auto place = [&](int i) { const int p = i + rot; return p >= stages ? p - stages : p; };
    const volatile int *abort = abort_word;

    // The thread that copies weights sets up its own barriers and asks for the first stages at once: they are nobody's
    // output (no wait for the predecessor in the stream), and they travel while the block is still being set up.
    const int ahead = min(CST, stages);
    int issued_c = 0, issued_b = 0, issued_t = 0;       // stages and tiles of split means this thread has asked for (copy roles)
    const int drop = a.drop_stage;
    const unsigned char *wsrc = reinterpret_cast<const unsigned char *>(a.codes) + size_t(w0) * WSTAGE;
    const uint32_t *qsrc = a.sb + size_t(w0) * QSTAGE;
    if (warp == W_COPY && lane == 0) {
        for (int i = 0; i < CST; ++i) spl_mbar_init(&full_c[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        issued_c = ahead;
        for (int i = 0; i < ahead; ++i) {
            if (i == drop) continue;
            spl_mbar_expect_tx(&full_c[i], WSTAGE + QSTAGE * 4);
            spl_bulk_g2s(w_ring + size_t(i) * WSTAGE, wsrc + size_t(place(i)) * WSTAGE, WSTAGE, &full_c[i]);
            spl_bulk_g2s(q_ring + i * QSTAGE, qsrc + size_t(place(i)) * QSTAGE, QSTAGE * 4, &full_c[i]);
        }
    }
    if (warp == 0) {
        // One barrier a lane: the arrival count of barrier i (in the order of the pointers above, after full_c).
        const int total = int(finished + 1 - bars);
        for (int b = lane + CST; b < total; b += 32) {
            uint64_t *bar = bars + b;
            const uint32_t count = bar < full_b ? uint32_t(4 * UPS)   // empty_c: the sets (four warps each) that take the stage's units
                                 : bar < done ? 1u                // full_b: the copy's bytes
                                 : bar < full_a ? 1u              // done: the commit of the issuing warp that took the unit
                                 : bar < full_t ? 4u              // full_a (one per unit modulo 2 AUN): the four warps of a set
                                 : bar < empty_t ? 1u             // full_t
                                 : uint32_t(NW);                  // empty_t and finished: the issuing warps
            spl_mbar_init(bar, count);
        }
        if (lane == 0) *abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == W_MMA0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(spl_smem_addr(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    spl_tc_fence_before();
    __syncthreads();
    spl_tc_fence_after();
    const uint32_t tmem = *tmem_slot;                 // lane 0, first allocated column
    // The accumulators, one per issuing warp (instructions of different warps are not ordered against each other), in
    // columns [0, 128); the A ring, 64 columns a unit; the second-term operand, 8 columns a unit.
    const uint32_t tmem_d = tmem, tmem_a = tmem + 128, tmem_aq = tmem + 128 + AUN * 64;
    bool ok = true;
    spl_grid_begin();
    if (warp == W_COPY) {
        // ---- copies of weights: codes and their scale/bias words, one ring, one contiguous piece of the arrays.
        if (lane == 0) {
            for (int i = ahead; i < stages; ++i) {
                const int sc = i % CST;
                const bool got_c = spl_mbar_wait(&empty_c[sc], ((i / CST) & 1) ^ 1, abort);
                if (!got_c) { ok = false; if (!*abort) spl_note_wait(a.error_flag, 10, i); break; }
                issued_c = i + 1;
                if (i == drop) continue;
                spl_mbar_expect_tx(&full_c[sc], WSTAGE + QSTAGE * 4);
                spl_bulk_g2s(w_ring + size_t(sc) * WSTAGE, wsrc + size_t(place(i)) * WSTAGE, WSTAGE, &full_c[sc]);
                spl_bulk_g2s(q_ring + sc * QSTAGE, qsrc + size_t(place(i)) * QSTAGE, QSTAGE * 4, &full_c[sc]);
            }
        }
    } else if (warp == W_COPYB) {
        // ---- copies of activations and of the tiles of split means.
        if (lane == 0) {
            const unsigned char *bsrc = reinterpret_cast<const unsigned char *>(a.act) + size_t(rb) * RN * 128;
            const unsigned char *tsrc = reinterpret_cast<const unsigned char *>(a.act_sums);
            int mean_tile = -1, mean_loads = 0;
            for (int i = 0; i < stages; ++i) {
                const int j = (w0 + place(i)) % S, sbq = i % BST;  // the stage's place in the contraction
                const int want = (j * SUPER) >> 4;                 // the tile of split means that holds its groups (sixteen groups to a tile)
                if (want != mean_tile) {
                    const int slot = mean_loads & 1;
                    if (!spl_mbar_wait(&empty_t[slot], ((mean_loads >> 1) & 1) ^ 1, abort)) { ok = false; if (!*abort) spl_note_wait(a.error_flag, 20, i); break; }
                    spl_mbar_expect_tx(&full_t[slot], TTILE);
                    spl_bulk_g2s(t_ring + slot * TTILE, tsrc + (size_t(want) * row_blocks + rb) * TTILE, TTILE, &full_t[slot]);
                    mean_tile = want; ++mean_loads; issued_t = mean_loads;
                }
                if (i >= BST) {            // the stage's last tenant: its units have to have completed
                    bool freed = true;
                    for (int h = 0; h < UPS; ++h) { const int u = UPS * (i - BST) + h; freed = freed && spl_mbar_wait(&done[u & 15], (u >> 4) & 1, abort); }
                    if (!freed) { ok = false; if (!*abort) spl_note_wait(a.error_flag, 21, i); break; }
                }
                issued_b = i + 1;
                spl_mbar_expect_tx(&full_b[sbq], BTILE);
                if (row_blocks == 1) {
                    spl_bulk_g2s(b_ring + size_t(sbq) * BTILE, bsrc + size_t(j) * BTILE, BTILE, &full_b[sbq]);
                } else {
                    for (int u = 0; u < SUPER; ++u) {
                        const size_t g = size_t(j) * SUPER + u;
                        spl_bulk_g2s(b_ring + size_t(sbq) * BTILE + u * RN * 128, bsrc + g * row_blocks * RN * 128, RN * 128, &full_b[sbq]);
                    }
                }
            }
        }
    } else if (warp == W_MMA0 || warp == W_MMA1) {
        // ---- tensor-core issue: D[128 x RN] += A[128 x 64] (fp16, tensor memory) * B[RN x 64]^T (fp16, shared memory).
        // The whole warp runs the loop and its waits; one elected lane issues (spl_elect_one). An elected lane is held
        // while the tensor pipe works through its instructions, and a wait on a barrier costs its latency even when the
        // phase is complete, so in the narrow blocks two warps take the units in turn (one the first unit of every stage,
        // the other the second), each into an accumulator of its own: one warp's waits run under the other's
        // instructions. A unit is eight k16 instructions at fixed offsets from the unit's bases and a ninth for its share
        // of the second term (the unit's 8 values of that contraction; the other 8 columns of its operand slot are zero).
        const int m = warp == W_MMA0 ? 0 : 1;
        if (m < NW) {
        constexpr uint32_t idesc = spl_tc_idesc(RN);
        int mean_tile = -1, mean_loads = 0, mean_slot = 0;
        const uint64_t b_desc0 = spl_tc_desc_sw128(spl_smem_addr(b_ring)), t_desc0 = spl_tc_desc_sw128(spl_smem_addr(t_ring));
        const uint32_t d_mine = tmem_d + m * RN;
        // A unit's operand slot is un % AUN, but its "converted" barrier is un % (2 AUN): the slots alternate between the two
        // issuing warps (AUN is odd), so with one barrier a slot a warp that runs ahead of the other would meet the barrier
        // two uses behind and take the previous tenant's completion for its own unit's. Barrier un % (2 AUN) belongs to one warp.
        int slot = m, fa = m;                              // un % AUN, un % (2 AUN)
        uint32_t a_parity = 0;                             // (un / (2 AUN)) & 1
        for (int i = 0; i < stages; ++i) {
            const int un = UPS * i + m, j = (w0 + place(i)) % S, sbq = i % BST;
            const int gu = j * UPS + m;                    // the unit's place in the contraction: 8 units to a tile of means, 2 to a k16 of the second term
            const bool first = i == 0, last = i + 1 == stages;
            const uint64_t b_desc = b_desc0 + uint64_t((sbq * BTILE + m * 2 * RN * 128) >> 4);
            const uint32_t a_base = tmem_a + slot * 64;
            const int want = gu >> 3;
            if (want != mean_tile) {
                if (mean_tile >= 0 && spl_elect_one()) spl_tc_commit(&empty_t[mean_slot]);      // every instruction of this warp that read the old tile has been issued
                __syncwarp();
                mean_slot = mean_loads & 1;
                if (!spl_mbar_wait_warp(&full_t[mean_slot], (mean_loads >> 1) & 1, abort)) { ok = false; if (!*abort && lane == 0) spl_note_wait(a.error_flag, 30 + m, i); break; }
                mean_tile = want; ++mean_loads;
            }
            if (!spl_mbar_wait_warp(&full_b[sbq], (i / BST) & 1, abort)) { ok = false; if (!*abort && lane == 0) spl_note_wait(a.error_flag, 34 + m, i); break; }
            if (!spl_mbar_wait_warp(&full_a[fa], a_parity, abort)) { ok = false; if (!*abort && lane == 0) spl_note_wait(a.error_flag, 36 + m, i); break; }
            spl_tc_fence_after();
            const uint64_t t_desc = t_desc0 + uint64_t((mean_slot * TTILE + ((gu >> 1) & 3) * 32) >> 4);
            if (!first) {                                        // the common case: nothing to decide between the instructions
                if (spl_elect_one()) {
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        spl_tc_mma_ts_acc(d_mine, a_base + q * 8, b_desc + uint64_t(((q >> 2) * RN * 128 + (q & 3) * 32) >> 4), idesc);
                    spl_tc_mma_ts_acc(d_mine, tmem_aq + slot * 8, t_desc, idesc);
                    spl_tc_commit(&done[un & 15]);            // the unit's A slot is free, and with the stage's other unit its activations
                    if (last) spl_tc_commit(finished);
                }
            } else if (spl_elect_one()) {                        // the first unit of this warp overwrites its accumulator
                for (int q = 0; q < 8; ++q)
                    spl_tc_mma_ts(d_mine, a_base + q * 8, b_desc + uint64_t(((q >> 2) * RN * 128 + (q & 3) * 32) >> 4), idesc, q ? 1u : 0u);
                spl_tc_mma_ts_acc(d_mine, tmem_aq + slot * 8, t_desc, idesc);
                spl_tc_commit(&done[un & 15]);
                if (last) spl_tc_commit(finished);
            }
            __syncwarp();
            slot += UPS; if (slot >= AUN) slot -= AUN;
            fa += UPS; if (fa >= 2 * AUN) { fa -= 2 * AUN; a_parity ^= 1u; }
        }
        }
    } else {
        // ---- dequant: thread = output column; codes -> scale * (code - 8), exact in fp16 -> tensor memory. The sets
        // of four warps take the units of two groups in turn; a set's warps write the lanes of their
        // warp index mod 4. A unit also carries its two groups' pairs of the second-term operand.
        // Every one of these 512 threads runs the output stage and its barriers whatever its waits returned
        // (a failed thread skips the work, never a barrier), and `ok` is the same in all lanes of a warp.
        const int quarter = warp & 3, col = quarter * 32 + lane, set = warp >> 2;
        const uint32_t lane_base = uint32_t(quarter * 32) << 16;
        // The rows' factors of a deferred norm, a warp a row (rows warp, warp + 16, ...): [row][in_groups] sums of squares.
        // They are read here, while the first weights are still on their way: a load issued in the output stage would wait
        // behind the whole device's queued copies.
        constexpr int FROWS = (RN + 15) / 16;
        float part[FROWS];
#pragma unroll
        for (int n = 0; n < FROWS; ++n) part[n] = 0.0f;
        if (a.in_squares)
            for (int g0 = lane; g0 < a.in_groups; g0 += 128) {       // 128 of a row at a time, all asked for before any is added
                float v[FROWS][4];
#pragma unroll
                for (int n = 0; n < FROWS; ++n)
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int r = warp + 16 * n, row = rb * RN + r, g = g0 + 32 * u;
                        v[n][u] = (r < RN && row < a.rows && g < a.in_groups) ? a.in_squares[size_t(row) * a.in_groups + g] : 0.0f;
                    }
#pragma unroll
                for (int n = 0; n < FROWS; ++n) part[n] += (v[n][0] + v[n][1]) + (v[n][2] + v[n][3]);
            }
        SplTcOutput out;
        out.tmem_d = tmem_d; out.lane_base = lane_base; out.rb = rb; out.c = c; out.tile = tile;
        out.set = set; out.quarter = quarter; out.col = col; out.lane = lane; out.finished = finished;
        out.abort_word = abort_word; out.row_factor = row_factor; out.cells = cells;
        // The conversion loop of the units that are this set's, then the output stage. j is the stage's place in its tile's contraction.
        {
            const int un_end = UPS * stages;
#pragma unroll 1
            for (int un = set; ok && un < un_end; un += SPL_TC_SETS) {
            const int i = un / UPS, h = un % UPS, sc = i % CST;
            const int j = w0 + place(i) - tile * S;
            if (!spl_mbar_wait_warp(&full_c[sc], (i / CST) & 1, abort)) { ok = false; if (!*abort && lane == 0) spl_note_wait(a.error_flag, 41, un); break; }
            // The unit's codes and scale/bias words are read before anything is converted, so the codes can be handed back at once.
            uint4 lo[2], hi[2];
            uint32_t sbw[2];
#pragma unroll
            for (int v = 0; v < 2; ++v) {
                const int u = 2 * h + v;
                lo[v] = *reinterpret_cast<const uint4 *>(w_ring + size_t(sc) * WSTAGE + u * 4096 + col * 16);
                hi[v] = *reinterpret_cast<const uint4 *>(w_ring + size_t(sc) * WSTAGE + u * 4096 + 2048 + col * 16);
                sbw[v] = q_ring[sc * QSTAGE + u * 128 + col];
            }
            __syncwarp();
            if (lane == 0) spl_mbar_arrive(&empty_c[sc]);
            // The unit's slot was last used by unit un - AUN, which has to have completed.
            const int slot = un % AUN;
            if (un >= AUN && !spl_mbar_wait_warp(&done[(un - AUN) & 15], ((un - AUN) >> 4) & 1, abort)) { ok = false; if (!*abort && lane == 0) spl_note_wait(a.error_flag, 42, un); break; }
            spl_tc_fence_after();
            // A nibble moved to mantissa bits 6-9 under the exponent of 16 (0x4C00) is the fp16 number 16 + c, and
            // fma(16 + c, s, -24 s) = s * (c - 8) with one rounding of a result that fp16 holds exactly; -24 s is exact in
            // fp16 too (3 * 8 significant bits). One shift and one logic operation place the nibbles of both halves of a
            // word, one fused multiply-add converts the pair. Sixteen registers (32 weights) are converted and stored at a time.
            uint32_t aq[4];
#pragma unroll
            for (int v = 0; v < 2; ++v) {
                const float sf = __uint_as_float(sbw[v] << 16), bf = __uint_as_float(sbw[v] & 0xFFFF0000u);
                const __half2 s2h = __float2half2_rn(sf), m24h = __float2half2_rn(sf * -24.0f);
                const uint32_t s2 = *reinterpret_cast<const uint32_t *>(&s2h), m24 = *reinterpret_cast<const uint32_t *>(&m24h);
                const __half2 q1 = __float2half2_rn(bf * 64.0f), q2 = __float2half2_rn(sf * 512.0f);
                aq[2 * v] = *reinterpret_cast<const uint32_t *>(&q1); aq[2 * v + 1] = *reinterpret_cast<const uint32_t *>(&q2);
#pragma unroll
                for (int part = 0; part < 2; ++part) {
                    const uint4 src = part == 0 ? lo[v] : hi[v];
                    const uint32_t w4[4] = {src.x, src.y, src.z, src.w};
                    uint32_t regs[16];
#pragma unroll
                    for (int w = 0; w < 4; ++w)
                        asm volatile("{\n .reg .b32 xa, xb, xc, xd;\n"      // volatile: converted sixteen registers at a time, in step with the stores, not all up front
                            " shl.b32 xa, %4, 6;\n shl.b32 xb, %4, 2;\n shr.b32 xc, %4, 2;\n shr.b32 xd, %4, 6;\n"
                            " lop3.b32 xa, xa, 0x03C003C0, 0x4C004C00, 0xEA;\n"
                            " lop3.b32 xb, xb, 0x03C003C0, 0x4C004C00, 0xEA;\n"
                            " lop3.b32 xc, xc, 0x03C003C0, 0x4C004C00, 0xEA;\n"
                            " lop3.b32 xd, xd, 0x03C003C0, 0x4C004C00, 0xEA;\n"
                            " fma.rn.f16x2 %0, xa, %5, %6;\n fma.rn.f16x2 %1, xb, %5, %6;\n"
                            " fma.rn.f16x2 %2, xc, %5, %6;\n fma.rn.f16x2 %3, xd, %5, %6;\n}\n"
                            : "=r"(regs[4 * w]), "=r"(regs[4 * w + 1]), "=r"(regs[4 * w + 2]), "=r"(regs[4 * w + 3])
                            : "r"(w4[w]), "r"(s2), "r"(m24));
                    spl_tc_st16(tmem_a + lane_base + slot * 64 + v * 32 + part * 16, regs);
                }
            }
            // The unit's share of the second-term operand sits at its place among the sixteen values of its k16 instruction
            // (two units to an instruction, by the unit's place in the contraction); the rest is zero.
            if (((j * UPS + h) & 1) == 0) { spl_tc_st4(tmem_aq + lane_base + slot * 8, aq[0], aq[1], aq[2], aq[3]); spl_tc_st4(tmem_aq + lane_base + slot * 8 + 4, 0u, 0u, 0u, 0u); }
            else { spl_tc_st4(tmem_aq + lane_base + slot * 8, 0u, 0u, 0u, 0u); spl_tc_st4(tmem_aq + lane_base + slot * 8 + 4, aq[0], aq[1], aq[2], aq[3]); }
            spl_tc_st_wait();
            spl_tc_fence_before();
            __syncwarp();
            if (lane == 0) spl_mbar_arrive(&full_a[un % (2 * AUN)]);
            }
            if (!ok) *abort_word = 1;
            // Whatever happened, every dequant thread runs the output stage: its barriers are counted in threads.
            if (a.in_squares) {
                // The squares in one fixed order: a lane's groups, then a butterfly.
#pragma unroll
                for (int n = 0; n < FROWS; ++n) {
                    float ss = part[n];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    if (lane == 0 && warp + 16 * n < RN) row_factor[warp + 16 * n] = 1.0f / sqrtf(ss / a.in_dim + a.eps);
                }
                spl_named_barrier<1, 512>();
            }
            ok = spl_tc_output_stage<RN, MODE>(a, out, ok);
        }
    }
    if (!ok) { *abort_word = 1; atomicExch(a.error_flag, 1 + warp); }
    spl_tc_fence_before();
    __syncthreads();
    if (warp == W_MMA0) {
        spl_tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512) : "memory");
    }
    // A block that gave up may have copies in flight that nobody waited for: the copying threads wait (bounded) for the
    // last one they asked for in every ring slot before the block's shared memory is handed on.
    if (*abort_word && lane == 0) {
        if (warp == W_COPY)
            for (int sc = 0; sc < CST && sc < issued_c; ++sc) { const int i = sc + (issued_c - 1 - sc) / CST * CST; spl_mbar_wait(&full_c[sc], (i / CST) & 1); }
        if (warp == W_COPYB) {
            for (int sb = 0; sb < BST && sb < issued_b; ++sb) { const int i = sb + (issued_b - 1 - sb) / BST * BST; spl_mbar_wait(&full_b[sb], (i / BST) & 1); }
            for (int st = 0; st < 2 && st < issued_t; ++st) { const int n = st + (issued_t - 1 - st) / 2 * 2; spl_mbar_wait(&full_t[st], (n >> 1) & 1); }
        }
    }
}

// ---- the narrow block (16, 32, 64 rows: decode and verify steps) -------------------------------
// Grid (tiles, splits, row blocks), one tile's share of the contraction a block: groups [split x groups_per_split, ...)
// (a multiple of four). With one split the block writes the output (or, `fuse`, the SiLU-gated operand of the next
// GEMM); with more it leaves its partial sums in partials[split][row][column] for spl_gemm_fixup_rows_kernel. Its
// output stage is stores only: a block reaches it while the others still stream weights at the memory's full rate,
// and a load issued then waits behind megabytes of queued copies.
template <int RN, bool PAIR = false>
__global__ void __launch_bounds__(SPL_TC_THREADS, 1)
spl_gemm_q4_narrow_kernel(const uint32_t *__restrict__ codes, const uint32_t *__restrict__ sb, const __nv_bfloat16 *__restrict__ act,
                      const float *__restrict__ act_sums, float *out, int out_ld, const float *residual, float *partials,
                      int rows, int op_blocks, int groups, int groups_per_split, int *error_flag, int interleave, SplOperand act_out, int fuse,
                      const float *__restrict__ in_squares, int in_groups, float in_dim, float eps, int drop) {
    static_assert(!PAIR || RN == 128, "the pair form is the 128-row block");
    constexpr int GPS = PAIR ? 2 : SPL_TC_SUPER;       // groups of the contraction a stage covers (the pair form: two, for each of its two tiles)
    constexpr int BST = PAIR ? SPL_TC_PAIR_BSTAGES : spl_tc_bstages(RN), CST = PAIR ? SPL_TC_PAIR_CSTAGES : spl_tc_cstages(RN), AUN = PAIR ? SPL_TC_PAIR_AUNITS : SPL_TC_AUNITS;
    constexpr int BTILE = GPS * RN * 128, WSTAGE = SPL_TC_SUPER * 4096, QSTAGE = SPL_TC_SUPER * 128, TTILE = RN * 128;
    extern __shared__ unsigned char spl_tc_smem_raw[];
    // The swizzled activation tiles must sit on 1,024-byte boundaries.
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(spl_tc_smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char *b_ring = smem;                                                       // [BST][SUPER][RN * 128] activations
    unsigned char *t_ring = b_ring + size_t(BST) * BTILE;                               // [2][RN * 128] split means of sixteen groups
    unsigned char *w_ring = t_ring + 2 * TTILE;                                         // [CST][SUPER][4096] codes
    uint32_t *q_ring = reinterpret_cast<uint32_t *>(w_ring + size_t(CST) * WSTAGE);     // [CST][SUPER][128] scale | bias << 16
    uint64_t *bars = reinterpret_cast<uint64_t *>(q_ring + CST * QSTAGE);
    uint64_t *full_c = bars, *empty_c = full_c + CST, *full_b = empty_c + CST, *done = full_b + BST;      // done[un % 16]: the instructions that read unit un have completed
    uint64_t *full_a = done + 16, *full_t = full_a + 2 * AUN, *empty_t = full_t + 2, *finished = empty_t + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(finished + 1);
    int *abort_word = reinterpret_cast<int *>(tmem_slot + 1);        // set by the first role whose wait ran out: the others stop waiting
    const volatile int *abort = abort_word;
    float *row_factor = reinterpret_cast<float *>(bars) + 256;          // [RN] at byte 1,024 of the control area

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int W_COPY = SPL_TC_SETS * 4, W_MMA0 = W_COPY + 1, W_COPYB = W_COPY + 2, W_MMA1 = W_COPY + 3;
    // The pair form's grid has pair and row block in one dimension, the row block the fast index (the splits in the second): the blocks that run together are then the row
    // blocks of a few pairs, and a pair's weights come from HBM once and from L2 for the other row blocks.
    const int run_blocks = PAIR ? (rows + RN - 1) / RN : 1;
    const int tile = PAIR ? int(blockIdx.x) / run_blocks : int(blockIdx.x), split = int(blockIdx.y), rb = PAIR ? int(blockIdx.x) % run_blocks : int(blockIdx.z);
    const int row_blocks = op_blocks;   // the operand's row blocks (>= the grid's)
    const int tiles_all = (out_ld + 127) / 128;
    const int tile0 = PAIR ? 2 * tile : tile, tile1 = PAIR ? min(2 * tile + 1, tiles_all - 1) : tile;      // an odd tensor's last pair does its one tile twice
    const bool has1 = !PAIR || 2 * tile + 1 < tiles_all;
    const int rows_padded = op_blocks * RN;
    const int g_first = split * groups_per_split;
    const int g_count = min(groups_per_split, groups - g_first);
    const int supers = (g_count + GPS - 1) / GPS;
    const int units = PAIR ? 2 * supers : (g_count + 1) / 2;            // a unit = two groups of one tile = one hand-over from a dequant set
    // Every block of a GEMM reads the same activation lines. Blocks therefore walk the contraction from
    // different starting points (the order of a sum of groups does not matter beyond fp32 rounding, and it
    // is a fixed function of the tile), so that at any moment they ask L2 for different lines.
    const int rot = (g_count % GPS == 0 && supers > 1) ? int((uint32_t(tile) * 2654435761u >> 12) % uint32_t(supers)) : 0;

    // The thread that copies weights sets up its own barriers and asks for the first stages at once: they are nobody's
    // output (no wait for the predecessor in the stream), and they travel while the block is still being set up.
    const int ahead = min(CST, supers);
    int issued_c = 0, issued_b = 0, issued_t = 0;       // stages and tiles of split means this thread has asked for (copy roles)
    // Stage j of the block's share of the contraction into slot sc of the code ring: its codes and scale/bias words. The pair
    // form brings two groups of each of its two tiles (tile 0's at the slot's start, tile 1's after them).
    auto copy_codes = [&](int sc, int j, int n) {
        if (PAIR) {
            spl_mbar_expect_tx(&full_c[sc], 2u * uint32_t(n) * (4096 + 512));
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const size_t first = size_t(m ? tile1 : tile0) * groups + g_first + size_t(j) * GPS;
                spl_bulk_g2s(w_ring + size_t(sc) * WSTAGE + m * (GPS * 4096), reinterpret_cast<const unsigned char *>(codes) + first * 4096, uint32_t(n) * 4096, &full_c[sc]);
                spl_bulk_g2s(q_ring + sc * QSTAGE + m * (GPS * 128), sb + first * 128, uint32_t(n) * 512, &full_c[sc]);
            }
        } else {
            const size_t first = size_t(tile) * groups + g_first + size_t(j) * GPS;
            spl_mbar_expect_tx(&full_c[sc], uint32_t(n) * (4096 + 512));
            spl_bulk_g2s(w_ring + size_t(sc) * WSTAGE, reinterpret_cast<const unsigned char *>(codes) + first * 4096, uint32_t(n) * 4096, &full_c[sc]);
            spl_bulk_g2s(q_ring + sc * QSTAGE, sb + first * 128, uint32_t(n) * 512, &full_c[sc]);
        }
    };
    if (warp == W_COPY && lane == 0) {
        for (int i = 0; i < CST; ++i) spl_mbar_init(&full_c[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        issued_c = ahead;
        for (int j0 = 0; j0 < ahead; ++j0) {
            const int j = j0 + rot < supers ? j0 + rot : j0 + rot - supers;
            const int n = min(GPS, g_count - j0 * GPS);
            if (j0 == drop) continue;
            copy_codes(j0, j, n);
        }
    }
    if (warp == 0) {
        // One barrier a lane: the arrival count of barrier i (in the order of the pointers above, after full_c).
        const int i = lane + CST;
        const int total = int(finished + 1 - bars);
        for (int b = i; b < total; b += 32) {
            uint64_t *bar = bars + b;
            const uint32_t count = bar < full_b ? 8u              // empty_c: the two sets (four warps each) that take the stage's units
                                 : bar < done ? 1u                // full_b: the copy's bytes
                                 : bar < full_a ? 1u              // done: the commit of the issuing warp that took the unit
                                 : bar < full_t ? 4u              // full_a (one per unit modulo 2 AUN): the four warps of a set
                                 : bar < empty_t ? 1u             // full_t
                                 : 2u;                            // empty_t and finished: the two issuing warps
            spl_mbar_init(bar, count);
        }
        if (lane == 0) *abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == W_MMA0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(spl_smem_addr(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    spl_tc_fence_before();
    __syncthreads();
    spl_tc_fence_after();
    const uint32_t tmem = *tmem_slot;                 // lane 0, first allocated column
    // Two accumulators, one per issuing warp (instructions of different warps are not ordered against each other);
    // the A ring, 64 columns a unit; the second-term operand, 8 columns a unit.
    const uint32_t tmem_d = tmem, tmem_a = tmem + (PAIR ? 2 * RN : 128), tmem_aq = tmem_a + AUN * 64;
    bool ok = true;

    if (!(warp == W_COPY && lane == 0)) spl_grid_begin();     // the thread that copies weights first asks for some (below)
    if (warp == W_COPY) {
        // ---- copies of weights: codes and their scale/bias words, one ring.
        if (lane == 0) {
            spl_grid_begin();
            for (int j0 = ahead; j0 < supers && ok; ++j0) {
                const int j = j0 + rot < supers ? j0 + rot : j0 + rot - supers;      // the stage's source; j0 is its place in the pipeline
                const int n = min(GPS, g_count - j0 * GPS);         // with a rotation every stage is full
                const int sc = j0 % CST;
                ok = spl_mbar_wait(&empty_c[sc], ((j0 / CST) & 1) ^ 1, abort);
                if (!ok) { if (!*abort) spl_note_wait(error_flag, 10, j0); break; }
                issued_c = j0 + 1;
                if (j0 == drop) continue;
                copy_codes(sc, j, n);
            }
        }
    } else if (warp == W_COPYB) {
        // ---- copies of activations and of the tiles of split means.
        if (lane == 0) {
            const unsigned char *bsrc = reinterpret_cast<const unsigned char *>(act) + ((size_t(g_first) * row_blocks + rb) * RN) * 128;
            const unsigned char *tsrc = reinterpret_cast<const unsigned char *>(act_sums);
            int mean_tile = -1, mean_loads = 0;
            for (int j0 = 0; j0 < supers && ok; ++j0) {
                const int j = j0 + rot < supers ? j0 + rot : j0 + rot - supers;
                const int n = min(GPS, g_count - j0 * GPS);
                const int sbq = j0 % BST;
                // The tile of split means that holds this stage's groups (sixteen groups to a tile).
                const int want = (g_first + j * GPS) >> 4;
                if (want != mean_tile) {
                    const int slot = mean_loads & 1;
                    ok = spl_mbar_wait(&empty_t[slot], ((mean_loads >> 1) & 1) ^ 1, abort);
                    if (!ok) { if (!*abort) spl_note_wait(error_flag, 20, j0); break; }
                    spl_mbar_expect_tx(&full_t[slot], TTILE);
                    spl_bulk_g2s(t_ring + slot * TTILE, tsrc + (size_t(want) * row_blocks + rb) * TTILE, TTILE, &full_t[slot]);
                    mean_tile = want; ++mean_loads; issued_t = mean_loads;
                }
                if (j0 >= BST) {            // the stage's last tenant: both of its units have to have completed
                    const int u0 = 2 * (j0 - BST);
                    ok = spl_mbar_wait(&done[u0 & 15], (u0 >> 4) & 1, abort) && spl_mbar_wait(&done[(u0 + 1) & 15], ((u0 + 1) >> 4) & 1, abort);
                }
                if (!ok) { if (!*abort) spl_note_wait(error_flag, 21, j0); break; }
                issued_b = j0 + 1;
                spl_mbar_expect_tx(&full_b[sbq], uint32_t(n) * RN * 128);
                if (row_blocks == 1) {
                    spl_bulk_g2s(b_ring + size_t(sbq) * BTILE, bsrc + size_t(j) * BTILE, uint32_t(n) * RN * 128, &full_b[sbq]);
                } else {
                    for (int u = 0; u < n; ++u) {
                        const size_t g = size_t(j) * GPS + u;
                        spl_bulk_g2s(b_ring + size_t(sbq) * BTILE + u * RN * 128, bsrc + g * row_blocks * RN * 128, RN * 128, &full_b[sbq]);
                    }
                }
            }
        }
    } else if (warp == W_MMA0 || warp == W_MMA1) {
        // ---- tensor-core issue: D[128 x RN] += A[128 x 64] (fp16, tensor memory) * B[RN x 64]^T (fp16, shared memory).
        // The whole warp runs the loop and its waits; one elected lane issues (spl_elect_one). An elected lane is held
        // while the tensor pipe works through its instructions, and a wait on a barrier costs its latency even when the
        // phase is complete, so two warps take the units in turn (one the first unit of every stage, the other the
        // second), each into an accumulator of its own: one warp's waits run under the other's instructions. A unit is
        // eight k16 instructions at fixed offsets from the unit's bases and a ninth for its share of the second term
        // (the unit's 8 values of that contraction; the other 8 columns of its operand slot are zero).
        const int m = warp == W_MMA0 ? 0 : 1;
        constexpr uint32_t idesc = spl_tc_idesc(RN);
        int mean_tile = -1, mean_loads = 0, mean_slot = 0;
        const uint64_t b_desc0 = spl_tc_desc_sw128(spl_smem_addr(b_ring)), t_desc0 = spl_tc_desc_sw128(spl_smem_addr(t_ring));
        const uint32_t d_mine = tmem_d + m * RN;
        // A unit's operand slot is un % AUN, but its "converted" barrier is un % (2 AUN): the slots alternate between the two
        // issuing warps (AUN is odd), so with one barrier a slot a warp that runs ahead of the other would meet the barrier
        // two uses behind and take the previous tenant's completion for its own unit's. Barrier un % (2 AUN) belongs to one warp.
        int slot = m, fa = m;                              // un % AUN, un % (2 AUN)
        uint32_t a_parity = 0;                             // (un / (2 AUN)) & 1
        for (int un = m; un < units && ok; un += 2) {
            const int j0 = un >> 1, sbq = j0 % BST, n = min(GPS, g_count - j0 * GPS) - (PAIR ? 0 : 2 * m);     // groups of this unit: 1 or 2
            const uint64_t b_desc = b_desc0 + uint64_t((sbq * BTILE + (PAIR ? 0 : m * 2 * RN * 128)) >> 4);      // the pair's two tiles meet the same activations
            const uint32_t a_base = tmem_a + slot * 64;
            // The stage's share of the second term: its 16 values of the contraction are a quarter of a 128-byte row of the tile.
            const int j = j0 + rot < supers ? j0 + rot : j0 + rot - supers;
            const int quarter = (g_first + j * GPS) >> 2, want = quarter >> 2;
            if (want != mean_tile) {
                if (mean_tile >= 0 && spl_elect_one()) spl_tc_commit(&empty_t[mean_slot]);      // every instruction of this warp that read the old tile has been issued
                __syncwarp();
                mean_slot = mean_loads & 1;
                ok = spl_mbar_wait_warp(&full_t[mean_slot], (mean_loads >> 1) & 1, abort);
                if (!ok) { if (!*abort && lane == 0) spl_note_wait(error_flag, 30 + m, un); break; }
                mean_tile = want; ++mean_loads;
            }
            ok = spl_mbar_wait_warp(&full_b[sbq], (j0 / BST) & 1, abort);
            if (!ok) { if (!*abort && lane == 0) spl_note_wait(error_flag, 34 + m, un); break; }
            ok = spl_mbar_wait_warp(&full_a[fa], a_parity, abort);
            if (!ok) { if (!*abort && lane == 0) spl_note_wait(error_flag, 36 + m, un); break; }
            spl_tc_fence_after();
            const uint64_t t_desc = t_desc0 + uint64_t((mean_slot * TTILE + (quarter & 3) * 32) >> 4);
            if (n >= 2 && un >= 2) {                             // the common case: nothing to decide between the instructions
                if (spl_elect_one()) {
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        spl_tc_mma_ts_acc(d_mine, a_base + q * 8, b_desc + uint64_t(((q >> 2) * RN * 128 + (q & 3) * 32) >> 4), idesc);
                    spl_tc_mma_ts_acc(d_mine, tmem_aq + slot * 8, t_desc, idesc);
                    spl_tc_commit(&done[un & 15]);            // the unit's A slot is free, and with the stage's other unit its activations
                }
            } else if (spl_elect_one()) {                        // the warp's first unit (it overwrites the accumulator) and a unit of one group
                for (int q = 0; q < 8; ++q)
                    if ((q >> 2) < n)
                        spl_tc_mma_ts(d_mine, a_base + q * 8, b_desc + uint64_t(((q >> 2) * RN * 128 + (q & 3) * 32) >> 4), idesc, (un >= 2 || q) ? 1u : 0u);
                spl_tc_mma_ts_acc(d_mine, tmem_aq + slot * 8, t_desc, idesc);
                spl_tc_commit(&done[un & 15]);
            }
            __syncwarp();
            slot += 2; if (slot >= AUN) slot -= AUN;
            fa += 2; if (fa >= 2 * AUN) { fa -= 2 * AUN; a_parity ^= 1u; }
        }
        if (ok && spl_elect_one()) spl_tc_commit(finished);
        __syncwarp();
    } else {
        // ---- dequant: thread = output column; codes -> scale * (code - 8), exact in fp16 -> tensor memory. The sets
        // of four warps take the units of two groups in turn; a set's warps write the lanes of their
        // warp index mod 4. A unit also carries its two groups' pairs of the second-term operand.
        const int quarter = warp & 3, col = quarter * 32 + lane, set = warp >> 2;
        const uint32_t lane_base = uint32_t(quarter * 32) << 16;
        // The rows' factors of a deferred norm (the operand came from one: out = sum * rsqrt(mean of the row's squares + eps)),
        // a warp a row (rows warp, warp + 16, ...): [row][in_groups] sums of squares. They are read here, while the first
        // weights are still on their way (a load issued in the output stage would wait behind the whole device's queued
        // copies), 128 of a row at a time and all asked for before any is added: one trip to memory, not one a load.
        constexpr int FROWS = (RN + 15) / 16;
        float part[FROWS];
#pragma unroll
        for (int f = 0; f < FROWS; ++f) part[f] = 0.0f;
        if (in_squares)
            for (int g0 = lane; g0 < in_groups; g0 += 128) {
                float v[FROWS][4];
#pragma unroll
                for (int f = 0; f < FROWS; ++f)
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int r = warp + 16 * f, row = rb * RN + r, g = g0 + 32 * u;
                        v[f][u] = (r < RN && row < rows && g < in_groups) ? in_squares[size_t(row) * in_groups + g] : 0.0f;
                    }
#pragma unroll
                for (int f = 0; f < FROWS; ++f) part[f] += (v[f][0] + v[f][1]) + (v[f][2] + v[f][3]);
            }
        for (int un = set; un < units && ok; un += SPL_TC_SETS) {
            const int j = un >> 1, half = un & 1, sc = j % CST;
            ok = spl_mbar_wait(&full_c[sc], (j / CST) & 1, abort);
            if (!ok) { if (!*abort && lane == 0) spl_note_wait(error_flag, 41, un); break; }
            const int n = PAIR ? 2 * half + min(GPS, g_count - j * GPS) : min(SPL_TC_SUPER, g_count - j * SPL_TC_SUPER);      // code groups of the stage up to this unit's last; the unit has those from 2 * half (the pair form: tile `half`'s two)
            // The unit's codes and scale/bias words are read before anything is converted, so the codes can be handed back at once.
            uint4 lo[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)}, hi[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
            uint32_t sbw[2] = {0u, 0u};
#pragma unroll
            for (int v = 0; v < 2; ++v) {
                const int u = 2 * half + v;
                if (u < n) {
                    lo[v] = *reinterpret_cast<const uint4 *>(w_ring + size_t(sc) * WSTAGE + u * 4096 + col * 16);
                    hi[v] = *reinterpret_cast<const uint4 *>(w_ring + size_t(sc) * WSTAGE + u * 4096 + 2048 + col * 16);
                    sbw[v] = q_ring[sc * QSTAGE + u * 128 + col];
                }
            }
            __syncwarp();
            if (lane == 0) spl_mbar_arrive(&empty_c[sc]);
            // The unit's slot was last used by unit un - AUN, which has to have completed.
            const int slot = un % AUN;
            if (un >= AUN) ok = spl_mbar_wait(&done[(un - AUN) & 15], ((un - AUN) >> 4) & 1, abort);
            if (!ok) { if (!*abort && lane == 0) spl_note_wait(error_flag, 42, un); break; }
            spl_tc_fence_after();
            // A nibble moved to mantissa bits 6-9 under the exponent of 16 (0x4C00) is the fp16 number 16 + c, and
            // fma(16 + c, s, -24 s) = s * (c - 8) with one rounding of a result that fp16 holds exactly; -24 s is exact in
            // fp16 too (3 * 8 significant bits). One shift and one logic operation place the nibbles of both halves of a
            // word, one fused multiply-add converts the pair. Sixteen registers (32 weights) are converted and stored at a time.
            uint32_t aq[4];
#pragma unroll
            for (int v = 0; v < 2; ++v) {
                const float sf = __uint_as_float(sbw[v] << 16), bf = __uint_as_float(sbw[v] & 0xFFFF0000u);
                const __half2 s2h = __float2half2_rn(sf), m24h = __float2half2_rn(sf * -24.0f);
                const uint32_t s2 = *reinterpret_cast<const uint32_t *>(&s2h), m24 = *reinterpret_cast<const uint32_t *>(&m24h);
                const __half2 q1 = __float2half2_rn(bf * 64.0f), q2 = __float2half2_rn(sf * 512.0f);      // zero for a group past the end
                aq[2 * v] = *reinterpret_cast<const uint32_t *>(&q1); aq[2 * v + 1] = *reinterpret_cast<const uint32_t *>(&q2);
                if (2 * half + v < n) {
#pragma unroll
                    for (int part = 0; part < 2; ++part) {
                        const uint4 src = part == 0 ? lo[v] : hi[v];
                        const uint32_t w4[4] = {src.x, src.y, src.z, src.w};
                        uint32_t a[16];
#pragma unroll
                        for (int w = 0; w < 4; ++w)
                            asm("{\n .reg .b32 xa, xb, xc, xd;\n"
                                " shl.b32 xa, %4, 6;\n shl.b32 xb, %4, 2;\n shr.b32 xc, %4, 2;\n shr.b32 xd, %4, 6;\n"
                                " lop3.b32 xa, xa, 0x03C003C0, 0x4C004C00, 0xEA;\n"
                                " lop3.b32 xb, xb, 0x03C003C0, 0x4C004C00, 0xEA;\n"
                                " lop3.b32 xc, xc, 0x03C003C0, 0x4C004C00, 0xEA;\n"
                                " lop3.b32 xd, xd, 0x03C003C0, 0x4C004C00, 0xEA;\n"
                                " fma.rn.f16x2 %0, xa, %5, %6;\n fma.rn.f16x2 %1, xb, %5, %6;\n"
                                " fma.rn.f16x2 %2, xc, %5, %6;\n fma.rn.f16x2 %3, xd, %5, %6;\n}\n"
                                : "=r"(a[4 * w]), "=r"(a[4 * w + 1]), "=r"(a[4 * w + 2]), "=r"(a[4 * w + 3])
                                : "r"(w4[w]), "r"(s2), "r"(m24));
                        spl_tc_st16(tmem_a + lane_base + slot * 64 + v * 32 + part * 16, a);
                    }
                }
            }
            // The unit's share of the second-term operand sits at its place among the stage's sixteen values; the rest is zero.
            // (The pair form's stage is two groups of the contraction: they are the first or the second half of their four.)
            int place = half;
            if (PAIR) { const int jsrc = j + rot < supers ? j + rot : j + rot - supers; place = ((g_first + jsrc * GPS) >> 1) & 1; }
            if (place == 0) { spl_tc_st4(tmem_aq + lane_base + slot * 8, aq[0], aq[1], aq[2], aq[3]); spl_tc_st4(tmem_aq + lane_base + slot * 8 + 4, 0u, 0u, 0u, 0u); }
            else { spl_tc_st4(tmem_aq + lane_base + slot * 8, 0u, 0u, 0u, 0u); spl_tc_st4(tmem_aq + lane_base + slot * 8 + 4, aq[0], aq[1], aq[2], aq[3]); }
            spl_tc_st_wait();
            spl_tc_fence_before();
            __syncwarp();
            if (lane == 0) spl_mbar_arrive(&full_a[un % (2 * AUN)]);
        }
        if (!ok) *abort_word = 1;
        // Every dequant thread comes to the barriers below, whatever happened to it before: they cannot be left waiting.
        if (in_squares) {
            // The squares in one fixed order: a lane's groups, then a butterfly.
#pragma unroll
            for (int f = 0; f < FROWS; ++f) {
                float ss = part[f];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0 && warp + 16 * f < RN) row_factor[warp + 16 * f] = 1.0f / sqrtf(ss / in_dim + eps);
            }
            spl_named_barrier<1, SPL_TC_SETS * 128>();
        }
        if (ok && !spl_mbar_wait(finished, 0, abort)) { ok = false; if (!*abort && lane == 0) spl_note_wait(error_flag, 40, 0); }
        // A fused gate|up tensor (interleave > 0) holds, in tile t, the gate columns [64 t, 64 t + 64) and then the up columns of
        // the same range. Without `fuse` the output goes to the columns of the plain layout; with it the block writes
        // act = bf16(silu(gate) * up) and its per-64 sums (engine.metal:200-219) straight into the next GEMM's operand:
        // the accumulators pass through shared memory (the activation ring is idle by now) so that a thread holds the
        // gate and the up value of the same element.
        float *stage = reinterpret_cast<float *>(b_ring);       // [RN][128] fp32
        // The pair form holds two tiles' sums, one per issuing warp's accumulator: the output stage runs once for each.
#pragma unroll 1
        for (int om = 0; om < (PAIR ? 2 : 1); ++om) {
        const int otile = PAIR ? (om ? tile1 : tile0) : tile;
        if (PAIR && om == 1 && !has1) break;
        if (ok) {
            spl_tc_fence_after();
            const int n = otile * 128 + col;
            const int n_out = interleave > 0 ? (((col & 16) ? interleave : 0) + otile * 64 + (col >> 5) * 16 + (col & 15)) : n;
            const bool is_split = partials != nullptr;          // the second kernel finishes: residual, output, the next operand
            float *dst = is_split ? partials + size_t(split) * rows_padded * out_ld : out;
            // (one copy of the body: code that runs once a block is paid for in instruction fetches)
#pragma unroll 1
            for (int cb = set; cb < RN / 16; cb += SPL_TC_SETS) {
                const int c0 = cb * 16;
                float total[16];
#pragma unroll
                for (int a = 0; a < (!PAIR && units > 1 ? 2 : 1); ++a) {
                    uint32_t v[16];
                    spl_tc_ld16(v, tmem_d + lane_base + (PAIR ? om : a) * RN + c0);
#pragma unroll
                    for (int r = 0; r < 16; ++r) total[r] = a == 0 ? __uint_as_float(v[r]) : total[r] + __uint_as_float(v[r]);
                }
                // A cut tile's partial sums are scaled one by one, so their sum is.
                if (in_squares)
#pragma unroll
                    for (int r = 0; r < 16; ++r) total[r] *= row_factor[c0 + r];
                if (fuse) {
#pragma unroll
                    for (int r = 0; r < 16; ++r) stage[(c0 + r) * 128 + col] = total[r];
                } else if (n < out_ld) {
                    float res[16];
#pragma unroll
                    for (int r = 0; r < 16; ++r) {
                        const int row = rb * RN + c0 + r;
                        res[r] = (!is_split && residual && row < rows) ? residual[size_t(row) * out_ld + n_out] : 0.0f;
                    }
#pragma unroll
                    for (int r = 0; r < 16; ++r) {
                        const int row = rb * RN + c0 + r;
                        if (row < rows) dst[size_t(row) * out_ld + n_out] = total[r] + res[r];
                    }
                }
            }
        }
        if (fuse) {
            // Every dequant thread comes here, whatever happened to it before: the barrier cannot be left waiting.
            spl_named_barrier<1, SPL_TC_SETS * 128>();
            const int t = threadIdx.x, c8 = (t & 7) * 8;
            for (int rr = t >> 3; rr < RN; rr += SPL_TC_SETS * 16) {
                const int row = rb * RN + rr;
                float r[8];
                {
                    const int gc = (c8 >> 4) * 32 + (c8 & 15);        // the gate columns of elements c8 ... c8 + 7; their up columns are sixteen further
                    const float4 g0 = *reinterpret_cast<const float4 *>(stage + rr * 128 + gc), g1 = *reinterpret_cast<const float4 *>(stage + rr * 128 + gc + 4);
                    const float4 u0 = *reinterpret_cast<const float4 *>(stage + rr * 128 + 16 + gc), u1 = *reinterpret_cast<const float4 *>(stage + rr * 128 + 16 + gc + 4);
                    const float gs[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, us[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) r[i] = (ok && row < rows) ? spl_bf16_to_float(spl_float_to_bf16(spl_silu_exact(gs[i]) * us[i])) : 0.0f;
                }
                // The sums in one fixed order: fours, then a butterfly over the sixteen fours of a group (8, 4, 2, 1 apart);
                // a thread here holds two neighbouring fours, so the last level is its own addition.
                float sa = (r[0] + r[1]) + (r[2] + r[3]), sb2 = (r[4] + r[5]) + (r[6] + r[7]);
#pragma unroll
                for (int o = 4; o > 0; o >>= 1) { sa += __shfl_xor_sync(0xffffffffu, sa, o); sb2 += __shfl_xor_sync(0xffffffffu, sb2, o); }
                if (ok && row < rows) {
                    const uint2 lo8 = spl_operand_pack4(r[0], r[1], r[2], r[3]), hi8 = spl_operand_pack4(r[4], r[5], r[6], r[7]);
                    *reinterpret_cast<uint4 *>(act_out.values + act_out.at(row, otile * 64 + c8)) = make_uint4(lo8.x, lo8.y, hi8.x, hi8.y);
                    if ((t & 7) == 0) act_out.put_sum(row, otile, sa + sb2);
                }
            }
            if (PAIR) spl_named_barrier<1, SPL_TC_SETS * 128>();      // the staged sums have been read: the other tile's may follow
        }
        }
    }
    if (!ok) { *abort_word = 1; atomicExch(error_flag, 1 + warp); }
    spl_tc_fence_before();
    __syncthreads();
    if (warp == W_MMA0) {
        spl_tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512) : "memory");
    }
    // A block that gave up may have copies in flight that nobody waited for: the copying threads wait (bounded) for the
    // last one they asked for in every ring slot before the block's shared memory is handed on.
    if (*abort_word && lane == 0) {
        if (warp == W_COPY)
            for (int sc = 0; sc < CST && sc < issued_c; ++sc) { const int i = sc + (issued_c - 1 - sc) / CST * CST; if (i != drop) spl_mbar_wait(&full_c[sc], (i / CST) & 1); }
        if (warp == W_COPYB) {
            for (int sq = 0; sq < BST && sq < issued_b; ++sq) { const int i = sq + (issued_b - 1 - sq) / BST * BST; spl_mbar_wait(&full_b[sq], (i / BST) & 1); }
            for (int st = 0; st < 2 && st < issued_t; ++st) { const int n = st + (issued_t - 1 - st) / 2 * 2; spl_mbar_wait(&full_t[st], (n >> 1) & 1); }
        }
    }
}

// What follows the sum of a cut GEMM (splits > 1): a warp per (row, 64 columns of a tile) adds the tile's slots in the
// order of the contraction, adds the residual and writes the output. With `emit_weight` the output feeds a deferred norm
// (Sources/Shaders/engine_na.metal:365-415): bf16(x * w) goes to the next operand with its per-64 sum, and the squares of
// x per 64 columns beside it. Both sums are butterflies over the warp: one fixed order.
__global__ void __launch_bounds__(256) spl_gemm_fixup_kernel(const float *__restrict__ slots, int splits, int pieces, int rn, int rows, int tiles, int out_ld, int interleave,
                                                             const float *residual, float *out, const uint16_t *__restrict__ emit_weight, SplOperand emit_out, float *emit_squares) {
    spl_grid_begin();
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const long long total = (long long)rows * tiles * 2;
    for (long long item = (long long)blockIdx.x * warps + (threadIdx.x >> 5); item < total; item += (long long)gridDim.x * warps) {
        const int half = int(item & 1), tile = int((item >> 1) % tiles), row = int((item >> 1) / tiles);
        const int rb = row / rn, rr = row % rn, col = half * 64 + 2 * lane;
        const float *src = slots + ((size_t(rb) * pieces + size_t(tile) * splits) * rn + rr) * 128 + col;
        float2 sum = __ldcg(reinterpret_cast<const float2 *>(src));
        for (int sp = 1; sp < splits; ++sp) {
            const float2 part = __ldcg(reinterpret_cast<const float2 *>(src + size_t(sp) * rn * 128));
            sum.x += part.x; sum.y += part.y;
        }
        const int n = tile * 128 + col;
        int n_out = n;
        bool inside = n < out_ld;
        if (interleave > 0) { const int e = tile * 64 + (col >> 5) * 16 + (col & 15); n_out = ((col & 16) ? interleave : 0) + e; inside = e < interleave; }
        float2 x = make_float2(0.0f, 0.0f);
        if (inside) {
            if (residual) { const float2 res = *reinterpret_cast<const float2 *>(residual + size_t(row) * out_ld + n_out); sum.x += res.x; sum.y += res.y; }
            *reinterpret_cast<float2 *>(out + size_t(row) * out_ld + n_out) = sum;
            x = sum;
        }
        if (emit_weight) {
            float v0 = 0.0f, v1 = 0.0f;
            if (inside) {
                const uint32_t w2 = *reinterpret_cast<const uint32_t *>(emit_weight + n);
                v0 = spl_bf16_to_float(spl_float_to_bf16(x.x * spl_bf16_to_float(uint16_t(w2 & 0xFFFFu))));
                v1 = spl_bf16_to_float(spl_float_to_bf16(x.y * spl_bf16_to_float(uint16_t(w2 >> 16))));
                *reinterpret_cast<__half2 *>(reinterpret_cast<__half *>(emit_out.values) + emit_out.at(row, n)) = __halves2half2(__float2half_rn(v0), __float2half_rn(v1));
            }
            float vs = v0 + v1, sq = x.x * x.x + x.y * x.y;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) { vs += __shfl_xor_sync(0xffffffffu, vs, off); sq += __shfl_xor_sync(0xffffffffu, sq, off); }
            const int group = tile * 2 + half;
            if (lane == 0 && group * 64 < out_ld) { emit_out.put_sum(row, group, vs); emit_squares[size_t(row) * (out_ld / 64) + group] = sq; }
        }
    }
}

// The same for the narrow block's partial sums, partials[split][row][column] in the output's own columns: a warp per
// (row, 64 columns).
__global__ void __launch_bounds__(256) spl_gemm_fixup_rows_kernel(const float *__restrict__ partials, int splits, int rows_padded, int rows, int ld,
                                                                  const float *residual, float *out, const uint16_t *__restrict__ emit_weight, SplOperand emit_out, float *emit_squares) {
    spl_grid_begin();
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5, groups = (ld + 63) / 64;
    const long long total = (long long)rows * groups;
    for (long long item = (long long)blockIdx.x * warps + (threadIdx.x >> 5); item < total; item += (long long)gridDim.x * warps) {
        const int row = int(item / groups), group = int(item % groups), n = group * 64 + 2 * lane;
        const bool inside = n < ld;
        float2 x = make_float2(0.0f, 0.0f);
        uint32_t w2 = 0u;
        if (inside) {
            // Everything is asked for before anything is added (the sums stay in split order): one trip to L2, not one a split.
            const float *src = partials + size_t(row) * ld + n;
            float2 res = make_float2(0.0f, 0.0f);
            if (residual) res = *reinterpret_cast<const float2 *>(residual + size_t(row) * ld + n);
            if (emit_weight) w2 = *reinterpret_cast<const uint32_t *>(emit_weight + n);
            for (int sp0 = 0; sp0 < splits; sp0 += 4) {
                float2 part[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    part[u] = sp0 + u < splits ? __ldcg(reinterpret_cast<const float2 *>(src + size_t(sp0 + u) * rows_padded * ld)) : make_float2(0.0f, 0.0f);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (sp0 + u == 0) x = part[u];
                    else if (sp0 + u < splits) { x.x += part[u].x; x.y += part[u].y; }
                }
            }
            if (residual) { x.x += res.x; x.y += res.y; }
            *reinterpret_cast<float2 *>(out + size_t(row) * ld + n) = x;
        }
        if (emit_weight) {
            float v0 = 0.0f, v1 = 0.0f;
            if (inside) {
                v0 = spl_bf16_to_float(spl_float_to_bf16(x.x * spl_bf16_to_float(uint16_t(w2 & 0xFFFFu))));
                v1 = spl_bf16_to_float(spl_float_to_bf16(x.y * spl_bf16_to_float(uint16_t(w2 >> 16))));
                *reinterpret_cast<__half2 *>(reinterpret_cast<__half *>(emit_out.values) + emit_out.at(row, n)) = __halves2half2(__float2half_rn(v0), __float2half_rn(v1));
            }
            float vs = v0 + v1, sq = x.x * x.x + x.y * x.y;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) { vs += __shfl_xor_sync(0xffffffffu, vs, off); sq += __shfl_xor_sync(0xffffffffu, sq, off); }
            if (lane == 0) { emit_out.put_sum(row, group, vs); emit_squares[size_t(row) * groups + group] = sq; }
        }
    }
}

// out[r][n] = sum over splits, in split order, of partials[s][r][n] (+ residual[r][n]): the reduction pass of the
// GGUF kernel's split contraction.
__global__ void spl_gemm_reduce_kernel(const float *__restrict__ partials, int splits, int rows_padded, int rows, int ld,
                                       const float *residual, float *out) {
    spl_grid_begin();
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
