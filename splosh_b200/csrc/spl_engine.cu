// spl_engine.cu — the engine behind the C ABI: device memory, weight upload, and one packed
// ragged step as a sequence of kernel launches on one stream.
//
// Stands in for Engine.init and Engine.step (Sources/SploshRuntime/Engine.swift:355-686, 1316-1540)
// and for encodeLinear / encodeFull (:2001-2077, :2167-2290). The reference separates dependent
// dispatches of one command encoder with barriers ("stages"); here stream order does that.
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "spl_attention.cuh"
#include "spl_gemm_gguf.cuh"
#include "spl_elementwise.cuh"
#include "spl_gdn.cuh"
#include "spl_gdn_chunk.cuh"
#include "spl_gemm_tc.cuh"
#include "spl_host.h"

namespace {

struct LayerWeights {
    bool full = false;
    SplQ4Dev in_proj, out_proj, gate_up, down;     // in_proj: qkv|z|a|b (gated-delta) or q|k|v (attention)
    SplGgufDev g_in_proj, g_out_proj, g_gate_up, g_down;      // the same tensors of a GGUF-weighted model (gate|up: gate columns, then up columns)
    uint16_t *vec[SPL_VEC_KINDS] = {};
};

enum { KLASS_GEMM = 0, KLASS_ELEMENTWISE, KLASS_GDN, KLASS_ATTENTION, KLASS_OTHER, KLASS_COUNT };

struct ProfileSlot { cudaEvent_t begin, end; int klass; double bytes; };

}  // namespace

struct spl_engine {
    spl_geometry g;
    spl_config c;
    spl_host *host = nullptr;
    int device = 0;
    cudaStream_t stream = nullptr;
    std::string error;
    // A step between spl_step_launch and spl_step_wait: its tables (the host object's arrays) and its start on the wall clock.
    bool in_flight = false;
    spl_tables flying{};
    int flying_rows = 0, flying_logit_rows = 0;
    std::chrono::steady_clock::time_point wall0;

    std::vector<LayerWeights> layers;
    SplQ4Dev head;
    SplGgufDev g_head;                  // a GGUF-weighted model's head, and its embedding table as native blocks [vocab][hidden / 256]
    unsigned char *g_embed = nullptr; int g_embed_format = 0;
    uint32_t *embed_packed = nullptr; uint16_t *embed_scales = nullptr, *embed_biases = nullptr;
    uint16_t *final_norm = nullptr;
    float *inv_freq = nullptr;
    size_t weight_bytes = 0;

    // Per-session state.
    std::vector<int8_t *> k_codes, v_codes;
    std::vector<float *> k_scale, v_scale, state, conv, journal;
    size_t kv_page_bytes = 0, kv_pool_bytes = 0, state_layer_bytes = 0, conv_unit_bytes = 0, journal_bytes = 0;

    // Activations and scratch.
    float *h = nullptr, *proj = nullptr, *gate_up = nullptr, *gdn_act = nullptr, *partials = nullptr, *attn_partials = nullptr, *logits = nullptr;
    float *taps = nullptr;
    __nv_bfloat16 *xn = nullptr, *core = nullptr, *act = nullptr, *hsn = nullptr;      // GEMM operands (tile layout)
    float *xn_sums = nullptr, *core_sums = nullptr, *act_sums = nullptr, *hsn_sums = nullptr;
    float *gdn_records = nullptr, *gdn_o_raw = nullptr;      // the chunked gated-delta path: per (chunk, value head) records; raw outputs [row][value dim]
    int gdn_chunks_max = 0;
    uint32_t *d_chunk_runs = nullptr, *d_chunks = nullptr;
    float *xn_squares = nullptr;       // [row][hidden / 64] squares of the residual stream, left by the GEMM that feeds a deferred norm
    float *slots = nullptr;            // partial sums of the GEMM tiles that several blocks share
    size_t slot_floats = 0;
    bool gdn_out_file_order = false;      // spl_weights_gguf_file_order
    int gdn_chunk_min = SPL_GDN_CHUNK_MIN;      // ordinary runs at least this long take the chunked gated-delta scan (spl_debug_gdn_chunk_min)
    int sms = 148;
    int rows_padded = 0, logit_rows_padded = 0;
    int *tc_error = nullptr;
    // Drafter feature taps (Engine.swift:330-331, 1488-1497): the residual stream after the listed blocks, [row][tap][hidden].
    float *features = nullptr;
    std::vector<int> feature_layers;
    int32_t *topk_ids = nullptr; float *topk_values = nullptr;      // allocated by the first spl_topk
    __half *q = nullptr;
    int32_t *argmax_ids = nullptr;
    int proj_ld = 0, gate_up_ld = 0, core_ld = 0, logits_ld = 0;
    size_t partial_floats = 0, attn_partial_floats = 0, scratch_bytes = 0;

    // Step tables: one pinned blob copied in one transfer.
    uint32_t *tables_host = nullptr, *tables_dev = nullptr;
    size_t tables_words = 0;
    uint32_t *d_tokens, *d_row_slot, *d_row_pos, *d_row_read, *d_row_write, *d_runs, *d_run_info, *d_gather, *d_blocks, *d_page_table;
    spl_tables last = {};
    int last_rows = 0, last_logit_rows = 0;

    bool taps_enabled = false, profile = false;
    bool kv_store = true;            // false: test switch, the step's rows leave the KV pool as it is (spl_debug_kv_store)
    std::vector<ProfileSlot> profile_slots;
    size_t profile_used = 0;
    double klass_ms[KLASS_COUNT] = {}, klass_bytes[KLASS_COUNT] = {};
    int64_t klass_launches[KLASS_COUNT] = {};
    int launches = 0;
    cudaEvent_t ev_begin = nullptr, ev_end = nullptr;

    spl_status fail(spl_status code, const std::string &text) { error = text; return code; }
};

namespace {

#define SPL_CUDA(call)                                                                                  \
    do {                                                                                                \
        cudaError_t err__ = (call);                                                                     \
        if (err__ != cudaSuccess) {                                                                     \
            return e->fail(err__ == cudaErrorMemoryAllocation ? SPL_ERR_ALLOCATION_FAILED : SPL_ERR_DEVICE, \
                           std::string(#call) + ": " + cudaGetErrorString(err__));                      \
        }                                                                                               \
    } while (0)

// Between spl_step_launch and spl_step_wait the step's tables, slots, logits and weights belong to the GPU.
#define SPL_NOT_IN_FLIGHT(e)                                                                                        \
    do { if ((e)->in_flight) return (e)->fail(SPL_ERR_INVALID_ARGUMENT, "a step is in flight: call spl_step_wait first"); } while (0)

template <typename T>
spl_status device_alloc(spl_engine *e, T **ptr, size_t count, size_t *account = nullptr) {
    SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(ptr), std::max<size_t>(count, 1) * sizeof(T)));
    if (account) *account += count * sizeof(T);
    return SPL_OK;
}

int round16(int v) { return (v + 15) / 16 * 16; }

struct Shapes {
    int C, VD, VH, AD, KV;
    int gdn_z, gdn_a, gdn_b, gdn_n;        // column offsets in the fused gated-delta input projection
    int att_k, att_v, att_n;               // column offsets in the fused attention input projection
    explicit Shapes(const spl_geometry &g) {
        C = (2 * g.gdn_key_heads + g.gdn_value_heads) * g.gdn_head_dim; VD = g.gdn_value_heads * g.gdn_head_dim; VH = g.gdn_value_heads;
        AD = g.heads * g.head_dim; KV = g.kv_heads * g.head_dim;
        gdn_z = C; gdn_a = C + VD; gdn_b = gdn_a + round16(VH); gdn_n = gdn_b + round16(VH);
        att_k = 2 * AD; att_v = att_k + KV; att_n = att_v + KV;
    }
};

spl_status alloc_q4(spl_engine *e, SplQ4Dev &w, int n, int k) {
    w.n = n; w.ld = round16(n); w.tiles = (n + 127) / 128; w.k = k;
    const size_t units = size_t(w.tiles) * (k / 64);
    SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&w.codes), units * 4096));
    SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&w.sb), units * 512));
    SPL_CUDA(cudaMemsetAsync(w.codes, 0, units * 4096, e->stream));
    SPL_CUDA(cudaMemsetAsync(w.sb, 0, units * 512, e->stream));
    e->weight_bytes += units * 4608;
    return SPL_OK;
}

void profile_begin(spl_engine *e, int klass, double bytes) {
    ++e->launches;
    if (!e->profile) return;
    if (e->profile_used == e->profile_slots.size()) {
        ProfileSlot s; cudaEventCreate(&s.begin); cudaEventCreate(&s.end); s.klass = klass; s.bytes = 0;
        e->profile_slots.push_back(s);
    }
    ProfileSlot &s = e->profile_slots[e->profile_used];
    s.klass = klass; s.bytes = bytes;
    cudaEventRecord(s.begin, e->stream);
}
void profile_end(spl_engine *e) {
    if (!e->profile) return;
    cudaEventRecord(e->profile_slots[e->profile_used].end, e->stream);
    ++e->profile_used;
}
void profile_collect(spl_engine *e) {
    if (!e->profile) return;
    for (size_t i = 0; i < e->profile_used; ++i) {
        float ms = 0;
        cudaEventElapsedTime(&ms, e->profile_slots[i].begin, e->profile_slots[i].end);
        e->klass_ms[e->profile_slots[i].klass] += ms;
        e->klass_bytes[e->profile_slots[i].klass] += e->profile_slots[i].bytes;
        e->klass_launches[e->profile_slots[i].klass] += 1;
    }
    e->profile_used = 0;
}

// Launch of one of a step's kernels with programmatic stream serialisation: the kernel may be scheduled while its
// predecessor in the stream still runs; each kernel itself waits for that predecessor (spl_grid_wait) before it reads
// or writes anything a predecessor touched.
template <typename... KArgs, typename... Args>
void launch_step(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

// ---- GEMM launch ------------------------------------------------------------------------------
// Rows per operand block for a step of `rows` rows.
int operand_rn(int rows) { return rows <= 16 ? 16 : rows <= 32 ? 32 : rows <= 64 ? 64 : 128; }

// Splits of the contraction for a GGUF GEMM of `blocks` (tile, row block) pairs and `groups` quant
// groups: the count that minimises waves x groups per block on `sms` single-block SMs, with a
// fixed cost per block (pipeline fill) and a reduction pass counted in.
int choose_splits(int blocks, int groups, int sms, size_t partial_capacity, size_t partial_per_split) {
    int best = 1; double best_cost = 1e30;
    for (int s = 1; s <= groups / 8 && s <= 32; ++s) {
        const int gps = ((groups + s - 1) / s + 3) / 4 * 4, eff = (groups + gps - 1) / gps;      // a split starts on a multiple of four groups
        if (eff != s) continue;
        if (s > 1 && size_t(s) * partial_per_split > partial_capacity) break;
        const int waves = (blocks * s + sms - 1) / sms;
        const double cost = double(waves) * (gps + 20.0) + (s > 1 ? 4.0 : 0.0);     // a block costs about twenty groups of time besides its groups (measured: fill, first loads, output)
        if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
    }
    return best;
}

struct GemmOperand { const __nv_bfloat16 *values; const float *sums; int rn, blocks; };
// What a GEMM does besides the product. `fuse_act`: a fused gate|up tensor writes the SiLU-gated activation as the next
// operand. `in_squares`: the operand came from a deferred norm, the sums are scaled by the rows' factors. `emit_weight`:
// the output feeds a deferred norm, whose operand and squares the GEMM leaves as well.
struct GemmExtras {
    const SplOperand *fuse_act = nullptr;
    const float *in_squares = nullptr; int in_dim = 0; float eps = 0.0f;
    const uint16_t *emit_weight = nullptr; const SplOperand *emit_out = nullptr; float *emit_squares = nullptr;
};
// Where the blocks of a cut tile leave their partial sums, the launch's error words, the device's SM count.
struct GemmScratch { float *slots; size_t slot_floats; int *error_flag; int sms; spl_engine *timed = nullptr; };    // timed: the engine whose profile times the second kernel as elementwise work

// The kernels that need more than the default shared memory, opted in on the current device (the attribute is per device).
template <int RN> void configure_gemm() {
    cudaFuncSetAttribute(spl_gemm_q4_tc_kernel<RN, SPL_TC_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(spl_tc_smem_bytes(RN)));
    cudaFuncSetAttribute(spl_gemm_q4_tc_kernel<RN, SPL_TC_EMIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(spl_tc_smem_bytes(RN)));
    cudaFuncSetAttribute(spl_gemm_q4_tc_kernel<RN, SPL_TC_FUSE>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(spl_tc_smem_bytes(RN)));
    if constexpr (RN < 128) cudaFuncSetAttribute(spl_gemm_q4_narrow_kernel<RN>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(spl_tc_smem_bytes(RN)));
    if constexpr (RN == 128) cudaFuncSetAttribute(spl_gemm_q4_narrow_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(spl_tc_pair_smem_bytes()));
}
template <int RN, int FMT> void configure_gguf() { cudaFuncSetAttribute(spl_gemm_gguf_tc_kernel<RN, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(spl_gguf_smem_bytes(RN, FMT))); }
template <int HD, int PER_KV> void configure_scan() { cudaFuncSetAttribute(spl_attn_scan_kernel<HD, PER_KV>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(spl_attn_smem_bytes(HD, spl_attn_nq(PER_KV)))); }
// Once per device and process, with that device current. `sms` (may be null) receives its SM count.
bool configure_device(int device, int *sms) {
    static bool done[64] = {};
    static int count[64] = {};
    if (device < 0 || device >= 64) return false;
    if (!done[device]) {
        configure_gemm<16>(); configure_gemm<32>(); configure_gemm<64>(); configure_gemm<128>();
        configure_gguf<16, SPL_GGUF_Q4K>(); configure_gguf<32, SPL_GGUF_Q4K>(); configure_gguf<64, SPL_GGUF_Q4K>();
        configure_gguf<16, SPL_GGUF_Q5K>(); configure_gguf<32, SPL_GGUF_Q5K>(); configure_gguf<64, SPL_GGUF_Q5K>();
        configure_gguf<16, SPL_GGUF_Q6K>(); configure_gguf<32, SPL_GGUF_Q6K>(); configure_gguf<64, SPL_GGUF_Q6K>();
        configure_scan<256, 6>(); configure_scan<128, 4>();
        cudaFuncSetAttribute(spl_gdn_recurrence_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(spl_gdn_recurrence_smem()));
        cudaFuncSetAttribute(spl_gdn_chunk_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(spl_gdn_chunk_prepare_smem()));
        cudaFuncSetAttribute(spl_gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(spl_gdn_chunk_scan_smem()));
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return false;
        count[device] = prop.multiProcessorCount;
        if (cudaGetLastError() != cudaSuccess) return false;
        done[device] = true;
    }
    if (sms) *sms = count[device];
    return true;
}

// How a GEMM's weight is cut in pieces, one block a piece and row block: every tile in `splits` pieces, the count that
// minimises waves x stages per block with a fixed cost per block, and the second kernel of a cut GEMM, counted in.
// `whole`: the block's output stage needs the whole sum (the fused SiLU gate), so tiles are not cut.
// Test switch (spl_debug_drop_weight_stage): the q4 GEMM's weight-copy role leaves out this stage of every block's piece, so
// the roles that wait for it run out of time. -1: off.
static int g_drop_weight_stage = -1;
// Test switch (spl_debug_pair_blocks): 0 keeps prompt chunks on the one-tile 128-row block.
static int g_pair_blocks = 1;

struct GemmCut { int pieces, splits; };
GemmCut gemm_cut(const SplQ4Dev &w, int sms, int rn, int row_blocks, bool whole) {
    const int stages = w.k / (64 * spl_tc_super(rn));
    int best = 1; double best_cost = 1e30;
    for (int s = 1; s <= stages && s <= 16 && !(whole && s > 1); ++s) {
        const int per = (stages + s - 1) / s;
        if (s > 1 && per < 2) break;
        const int waves = (w.tiles * s * row_blocks + sms - 1) / sms;
        const double cost = double(waves) * (per * spl_tc_super(rn) + 20.0) + (s > 1 ? 12.0 : 0.0);      // in groups of time: a block's fill and output cost about twenty, the second kernel twelve
        if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
    }
    return {w.tiles * best, best};
}

// The pair form of the 128-row block (two tiles of the weight a block): into how many runs of whole stages every pair's
// contraction is cut, by the same count of waves x work a block with a fixed cost per block; 0 when the form does not apply
// (the switch is off, or the contraction is not whole stages of 256).
int pair_splits(const SplQ4Dev &w, int sms, int row_blocks, bool whole) {
    if (!g_pair_blocks || w.k % 256 != 0) return 0;
    const int pairs = (w.tiles + 1) / 2, stages = w.k / 256;
    int best = 1; double best_cost = 1e30;
    for (int s = 1; s <= stages && s <= 16 && !(whole && s > 1); ++s) {
        const int per = (stages + s - 1) / s;
        if (s > 1 && per < 2) break;
        const int waves = (pairs * s * row_blocks + sms - 1) / sms;
        const double cost = double(waves) * (per * 8 + 20.0) + (s > 1 ? 12.0 : 0.0);      // a stage of 256 is eight groups of work for two tiles
        if (cost < best_cost - 1e-9) { best_cost = cost; best = s; }
    }
    const int per = (stages + best - 1) / best;
    return (stages + per - 1) / per;
}

// Floats of scratch a GEMM on `w` may leave for its second kernel: the wide block's slots, or the narrow block's
// partials[split][row][column] (cut tiles, and every tile when the output feeds a deferred norm: `emit`).
size_t gemm_slot_floats(const SplQ4Dev &w, int sms, int rn, int row_blocks, bool emit, bool whole) {
    const GemmCut cut = gemm_cut(w, sms, rn, row_blocks, whole);
    if (rn >= 128) {
        // The pair form leaves cut contractions, and an output that feeds a deferred norm, to the second kernel.
        const int ps = pair_splits(w, sms, row_blocks, whole);
        const size_t pair = (ps > 1 || (ps == 1 && emit)) ? size_t(ps) * row_blocks * rn * w.ld : 0;
        return std::max(spl_tc_slot_floats(cut.pieces, cut.splits, row_blocks, rn), pair);
    }
    const int stages = w.k / 256, per = (stages + cut.splits - 1) / cut.splits, splits = (stages + per - 1) / per;
    return (splits > 1 || emit) ? size_t(splits) * row_blocks * rn * w.ld : 0;
}

template <int RN>
bool launch_gemm_tc(cudaStream_t stream, const SplQ4Dev &w, const GemmOperand &op, float *out, const float *residual, int rows,
                    const GemmScratch &scratch, const GemmExtras &x, int *launches) {
    const int row_blocks = (rows + RN - 1) / RN;
    const GemmCut cut = gemm_cut(w, scratch.sms, RN, row_blocks, x.fuse_act != nullptr);
    if (RN >= 128 && spl_tc_slot_floats(cut.pieces, cut.splits, row_blocks, RN) > scratch.slot_floats) return false;
    SplGemmArgs a = {};
    a.codes = w.codes; a.sb = w.sb; a.act = op.values; a.act_sums = op.sums; a.out = out; a.residual = residual;
    a.slots = scratch.slots; a.error_flag = scratch.error_flag;
    a.out_ld = w.ld; a.rows = rows; a.op_blocks = op.blocks; a.tiles = w.tiles; a.stages_per_tile = w.k / (64 * spl_tc_super(RN)); a.interleave = w.interleave;
    a.pieces = cut.pieces; a.row_blocks = row_blocks; a.splits = cut.splits;
    a.drop_stage = g_drop_weight_stage;
    a.fuse = x.fuse_act ? 1 : 0;
    a.act_out = x.fuse_act ? *x.fuse_act : SplOperand{nullptr, nullptr, RN, 1};
    a.in_squares = x.in_squares; a.in_groups = x.in_dim / 64; a.in_dim = float(x.in_dim); a.eps = x.eps;
    const SplOperand emit_out = x.emit_out ? *x.emit_out : SplOperand{nullptr, nullptr, RN, 1};
    a.emit_weight = x.emit_weight; a.emit_out = emit_out; a.emit_squares = x.emit_squares;
    const dim3 grid(cut.pieces * row_blocks), block(SPL_TC_THREADS);
    if constexpr (RN < 128) {
        // The narrow block: a tile's contraction in `splits` runs of whole stages. A cut GEMM, and one whose output feeds a
        // deferred norm, leave partial sums for the second kernel.
        const int stages = w.k / 256, per = (stages + cut.splits - 1) / cut.splits, splits = (stages + per - 1) / per;
        const bool second = splits > 1 || x.emit_weight != nullptr;
        const size_t rows_padded = size_t(op.blocks) * RN;
        if (second && size_t(splits) * rows_padded * w.ld > scratch.slot_floats) return false;
        launch_step(spl_gemm_q4_narrow_kernel<RN>, dim3(w.tiles, splits, row_blocks), block, spl_tc_smem_bytes(RN), stream, (const uint32_t *)w.codes, (const uint32_t *)w.sb, op.values, op.sums,
                    out, w.ld, second ? (const float *)nullptr : residual, second ? scratch.slots : (float *)nullptr, rows, op.blocks, w.k / 64, per * 4, scratch.error_flag, w.interleave,
                    a.act_out, a.fuse, x.in_squares, x.in_dim / 64, float(x.in_dim), x.eps, g_drop_weight_stage);
        if (launches) ++*launches;
        if (second) {
            if (scratch.timed) { profile_end(scratch.timed); profile_begin(scratch.timed, KLASS_ELEMENTWISE, 0); }
            else if (launches) ++*launches;
            const long long warps = (long long)rows * ((w.ld + 63) / 64);
            launch_step(spl_gemm_fixup_rows_kernel, dim3(int(std::min<long long>((warps + 7) / 8, 8LL * scratch.sms))), dim3(256), 0, stream, (const float *)scratch.slots, splits, int(rows_padded), rows, w.ld,
                        residual, out, x.emit_weight, emit_out, x.emit_squares);
        }
        return true;
    }
    if constexpr (RN == 128) {
        // The pair form, two tiles of the weight a block against one stream of activations.
        const int splits = pair_splits(w, scratch.sms, row_blocks, x.fuse_act != nullptr);
        if (splits > 0) {
            const int stages = w.k / 256, per = (stages + splits - 1) / splits;
            const bool second = splits > 1 || x.emit_weight != nullptr;
            const size_t rows_padded = size_t(op.blocks) * RN;
            if (second && size_t(splits) * rows_padded * w.ld > scratch.slot_floats) return false;
            launch_step(spl_gemm_q4_narrow_kernel<128, true>, dim3(((w.tiles + 1) / 2) * row_blocks, splits), block, spl_tc_pair_smem_bytes(), stream, (const uint32_t *)w.codes, (const uint32_t *)w.sb, op.values, op.sums,
                        out, w.ld, second ? (const float *)nullptr : residual, second ? scratch.slots : (float *)nullptr, rows, op.blocks, w.k / 64, per * 4, scratch.error_flag, w.interleave,
                        a.act_out, a.fuse, x.in_squares, x.in_dim / 64, float(x.in_dim), x.eps, g_drop_weight_stage);
            if (launches) ++*launches;
            if (second) {
                if (scratch.timed) { profile_end(scratch.timed); profile_begin(scratch.timed, KLASS_ELEMENTWISE, 0); }
                else if (launches) ++*launches;
                const long long warps = (long long)rows * ((w.ld + 63) / 64);
                launch_step(spl_gemm_fixup_rows_kernel, dim3(int(std::min<long long>((warps + 7) / 8, 8LL * scratch.sms))), dim3(256), 0, stream, (const float *)scratch.slots, splits, int(rows_padded), rows, w.ld,
                            residual, out, x.emit_weight, emit_out, x.emit_squares);
            }
            return true;
        }
    }
    if (x.fuse_act) launch_step(spl_gemm_q4_tc_kernel<RN, SPL_TC_FUSE>, grid, block, spl_tc_smem_bytes(RN), stream, a);
    else if (x.emit_weight && cut.splits == 1) launch_step(spl_gemm_q4_tc_kernel<RN, SPL_TC_EMIT>, grid, block, spl_tc_smem_bytes(RN), stream, a);
    else launch_step(spl_gemm_q4_tc_kernel<RN, SPL_TC_PLAIN>, grid, block, spl_tc_smem_bytes(RN), stream, a);
    if (launches) ++*launches;
    if (cut.splits > 1) {
        // The second kernel of a cut GEMM: the slots' sum in the order of the contraction, the residual, the output, the emitted operand.
        if (scratch.timed) { profile_end(scratch.timed); profile_begin(scratch.timed, KLASS_ELEMENTWISE, 0); }
        else if (launches) ++*launches;
        const long long warps = (long long)rows * w.tiles * 2;
        const int blocks = int(std::min<long long>((warps + 7) / 8, 8LL * scratch.sms));
        launch_step(spl_gemm_fixup_kernel, dim3(blocks), dim3(256), 0, stream, (const float *)scratch.slots, cut.splits, cut.pieces, RN, rows, w.tiles, w.ld, w.interleave,
                    residual, out, x.emit_weight, emit_out, x.emit_squares);
    }
    return true;
}

// out[r][:] = GEMM(w, operand[r][:]) (+ residual) for the first `rows` rows of the operand. False when the scratch is too small.
bool launch_gemm_rows(cudaStream_t stream, const SplQ4Dev &w, const GemmOperand &op, float *out, const float *residual, int rows,
                      const GemmScratch &scratch, const GemmExtras &x, int *launches) {
    if (op.rn == 16) return launch_gemm_tc<16>(stream, w, op, out, residual, rows, scratch, x, launches);
    if (op.rn == 32) return launch_gemm_tc<32>(stream, w, op, out, residual, rows, scratch, x, launches);
    if (op.rn == 64) return launch_gemm_tc<64>(stream, w, op, out, residual, rows, scratch, x, launches);
    return launch_gemm_tc<128>(stream, w, op, out, residual, rows, scratch, x, launches);
}

template <int RN, int FMT>
void launch_gemm_gguf_tc(cudaStream_t stream, const SplGgufDev &w, const GemmOperand &op, float *out, const float *residual, int rows,
                         float *partials, size_t partial_floats, int *error_flag) {
    const int supers = w.k / 256;
    const int row_blocks = (rows + RN - 1) / RN, rows_padded = op.blocks * RN;
    // The q4 rule in units of four groups: a split is a whole number of super-blocks.
    const int splits4 = choose_splits(w.tiles * row_blocks, supers * 4, 148, partial_floats, size_t(rows_padded) * w.ld);
    const int sps = (supers + splits4 - 1) / splits4, splits = (supers + sps - 1) / sps;
    const size_t smem = spl_gguf_smem_bytes(RN, FMT);
    launch_step(spl_gemm_gguf_tc_kernel<RN, FMT>, dim3(w.tiles, splits, row_blocks), dim3(SPL_GG_THREADS), smem, stream,
                w.blocks, op.values, out, w.ld, residual, partials, rows, op.blocks, supers, sps, error_flag);
    if (splits > 1) {
        const size_t total = size_t(rows) * w.ld / 4;
        launch_step(spl_gemm_reduce_kernel, dim3(int(std::min<size_t>((total + 255) / 256, 2048))), dim3(256), 0, stream, partials, splits, rows_padded, rows, w.ld, residual, out);
    }
}
template <int FMT>
void launch_gemm_gguf_rows(cudaStream_t stream, const SplGgufDev &w, const GemmOperand &op, float *out, const float *residual, int rows,
                           float *partials, size_t partial_floats, int *error_flag) {
    if (op.rn == 16) launch_gemm_gguf_tc<16, FMT>(stream, w, op, out, residual, rows, partials, partial_floats, error_flag);
    else if (op.rn == 32) launch_gemm_gguf_tc<32, FMT>(stream, w, op, out, residual, rows, partials, partial_floats, error_flag);
    else launch_gemm_gguf_tc<64, FMT>(stream, w, op, out, residual, rows, partials, partial_floats, error_flag);
}
void launch_gemm_gguf(cudaStream_t stream, const SplGgufDev &w, const GemmOperand &op, float *out, const float *residual, int rows,
                      float *partials, size_t partial_floats, int *error_flag) {
    if (w.format == SPL_GGUF_Q6K) launch_gemm_gguf_rows<SPL_GGUF_Q6K>(stream, w, op, out, residual, rows, partials, partial_floats, error_flag);
    else if (w.format == SPL_GGUF_Q5K) launch_gemm_gguf_rows<SPL_GGUF_Q5K>(stream, w, op, out, residual, rows, partials, partial_floats, error_flag);
    else launch_gemm_gguf_rows<SPL_GGUF_Q4K>(stream, w, op, out, residual, rows, partials, partial_floats, error_flag);
}

bool launch_gemm(spl_engine *e, const SplQ4Dev &w, const GemmOperand &op, float *out, const float *residual, int rows, const GemmExtras &x = GemmExtras()) {
    profile_begin(e, KLASS_GEMM, double(w.bytes()) * ((rows + op.rn - 1) / op.rn));
    --e->launches;      // profile_begin counted one; the launcher counts the kernels it really starts
    const GemmScratch scratch{e->slots, e->slot_floats, e->tc_error, e->sms, e};
    const bool fits = launch_gemm_rows(e->stream, w, op, out, residual, rows, scratch, x, &e->launches);
    profile_end(e);
    return fits;
}

template <int HD, int PER_KV>
void launch_scan_tc(spl_engine *e, dim3 grid, const SplAttnParams &p, int layer) {
    const size_t smem = spl_attn_smem_bytes(HD, spl_attn_nq(PER_KV));
    launch_step(spl_attn_scan_kernel<HD, PER_KV>, dim3(grid), dim3(spl_attn_threads(spl_attn_nq(PER_KV))), smem, e->stream, e->q, e->d_blocks, e->d_row_slot, e->d_row_pos, e->d_page_table,
        e->k_codes[layer], e->k_scale[layer], e->v_codes[layer], e->v_scale[layer], e->attn_partials, p, e->tc_error);
}
// The scan is built for the head shapes in use: head_dim 256 with six query heads per kv head, and head_dim 128 with four.
bool scan_supported(const spl_geometry &g) {
    const int per_kv = g.kv_heads > 0 ? g.heads / g.kv_heads : 0;
    return (g.head_dim == 256 && per_kv == 6) || (g.head_dim == 128 && per_kv == 4);
}
void launch_scan(spl_engine *e, dim3 grid, const SplAttnParams &p, int layer) {
    if (e->g.head_dim == 256) launch_scan_tc<256, 6>(e, grid, p, layer);
    else launch_scan_tc<128, 4>(e, grid, p, layer);
}

spl_status check_launch(spl_engine *e, const char *what) {
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return e->fail(SPL_ERR_DEVICE, std::string(what) + ": " + cudaGetErrorString(err));
    return SPL_OK;
}

// Everything of a step up to its last launch; finish_step waits for it.
spl_status enqueue_step(spl_engine *e, const spl_tables *t) {
    e->wall0 = std::chrono::steady_clock::now();
    const spl_geometry &g = e->g;
    const Shapes sh(g);
    const int R = int(t->rows);
    if (R <= 0 || R > e->c.max_rows) return e->fail(SPL_ERR_INVALID_ROWS, "invalid step rows: row count outside the engine's limit");
    if (int(t->logit_rows) > e->host->config.max_logit_rows) return e->fail(SPL_ERR_INVALID_ROWS, "invalid step rows: too many logit rows");
    const bool gguf = e->g_head.blocks != nullptr;      // a GGUF-weighted model: every GEMM tensor and the embedding came through spl_weights_set_gguf
    if (gguf) {
        bool all = e->g_embed != nullptr;
        for (const LayerWeights &L : e->layers) all = all && L.g_in_proj.blocks && L.g_out_proj.blocks && L.g_gate_up.blocks && L.g_down.blocks;
        if (!all) return e->fail(SPL_ERR_INVALID_ARGUMENT, "a GGUF-weighted engine needs every tensor as GGUF blocks");
    }
    for (size_t l = 0; l < e->layers.size(); ++l) {
        const LayerWeights &L = e->layers[l];
        if ((!gguf && !L.in_proj.codes) || !L.vec[SPL_VEC_INPUT_NORM]) return e->fail(SPL_ERR_INVALID_ARGUMENT, "weights of a block are not set");
    }
    if ((!gguf && (!e->head.codes || !e->embed_packed)) || !e->final_norm) return e->fail(SPL_ERR_INVALID_ARGUMENT, "model-level weights are not set");
    SPL_CUDA(cudaSetDevice(e->device));
    // Tables: pack into the pinned blob, one copy.
    uint32_t *hb = e->tables_host;
    size_t off = 0;
    auto put = [&](const uint32_t *src, size_t n, uint32_t **dev) { *dev = e->tables_dev + off; if (n) memcpy(hb + off, src, n * 4); off += (n + 3) / 4 * 4; };
    put(t->tokens, R, &e->d_tokens); put(t->row_slot, R, &e->d_row_slot); put(t->row_pos, R, &e->d_row_pos);
    put(t->row_read, R, &e->d_row_read); put(t->row_write, R, &e->d_row_write);
    put(t->runs, size_t(t->run_count) * 3, &e->d_runs); put(t->run_info, size_t(t->run_count) * 2, &e->d_run_info);
    put(t->gather_index, t->logit_rows, &e->d_gather); put(t->attn_blocks, size_t(t->attn_block_count) * 2, &e->d_blocks);
    put(t->page_table, size_t(e->c.max_slots) * e->host->max_pages, &e->d_page_table);
    // Long ordinary runs take the chunked gated-delta kernels: their list, and the list of their 64-token chunks.
    std::vector<uint32_t> chunk_runs, chunks;
    for (uint32_t r = 0; r < t->run_count; ++r) {
        const uint32_t length = t->runs[r * 3 + 2];
        if (t->run_info[r * 2] != 0 || int(length) < e->gdn_chunk_min || e->state.empty()) continue;
        const uint32_t index = uint32_t(chunk_runs.size() / 4);
        chunk_runs.insert(chunk_runs.end(), {t->runs[r * 3], t->runs[r * 3 + 1], length, t->run_info[r * 2 + 1]});
        for (uint32_t first = 0, n = 0; first < length; first += SPL_GDN_CHUNK, ++n)
            chunks.insert(chunks.end(), {index, t->runs[r * 3 + 1] + first, std::min<uint32_t>(SPL_GDN_CHUNK, length - first), n});
    }
    const int chunked_runs = int(chunk_runs.size() / 4), chunk_count = int(chunks.size() / 4);
    if (chunk_count > e->gdn_chunks_max) return e->fail(SPL_ERR_INVALID_ROWS, "invalid step rows: more chunks than the engine's gated-delta scratch holds");
    put(chunk_runs.data(), chunk_runs.size(), &e->d_chunk_runs); put(chunks.data(), chunks.size(), &e->d_chunks);
    if (off > e->tables_words) return e->fail(SPL_ERR_INVALID_ROWS, "invalid step rows: tables exceed the engine's buffers");
    e->launches = 0;
    SPL_CUDA(cudaEventRecord(e->ev_begin, e->stream));
    SPL_CUDA(cudaMemcpyAsync(e->tables_dev, hb, off * 4, cudaMemcpyHostToDevice, e->stream));

    const int H = g.hidden;
    // GEMM operands of this step: row blocks of rn rows, in the tile layout the tensor cores read.
    const int rn = gguf ? std::min(operand_rn(R), 64) : operand_rn(R), blocks = (R + rn - 1) / rn;      // the GGUF kernel's blocks hold up to 64 rows
    const SplOperand xn{e->xn, e->xn_sums, rn, blocks}, core{e->core, e->core_sums, rn, blocks}, act{e->act, e->act_sums, rn, blocks};
    const GemmOperand gxn{e->xn, e->xn_sums, rn, blocks}, gcore{e->core, e->core_sums, rn, blocks}, gact{e->act, e->act_sums, rn, blocks};
    profile_begin(e, KLASS_ELEMENTWISE, 0);
    if (gguf) launch_step(spl_embed_gguf_kernel, dim3(R), dim3(256), 0, e->stream, (const unsigned char *)e->g_embed, e->g_embed_format, (const uint32_t *)e->d_tokens, e->h, H);
    else launch_step(spl_embed_q4_kernel, dim3(R), dim3(128), 0, e->stream, e->embed_packed, e->embed_scales, e->embed_biases, e->d_tokens, e->h, H);
    profile_end(e);
    // A GGUF-weighted model: the GGUF GEMM (spl_gemm_gguf.cuh) has no fused forms, so its blocks run plain norms and an
    // unfused SiLU gate (the results are the deferred forms' up to the operand's rounding point).
    auto ggemm = [&](const SplGgufDev &w, const GemmOperand &op, float *out, const float *residual, int rows) {
        profile_begin(e, KLASS_GEMM, double(w.bytes()) * ((rows + op.rn - 1) / op.rn));
        launch_gemm_gguf(e->stream, w, op, out, residual, rows, e->partials, e->partial_floats, e->tc_error);
        profile_end(e);
    };

    // The attention partials of the widest scan of the step have to fit (checked before anything is launched, so a
    // refused step leaves no slot half-advanced).
    if (!e->k_codes.empty() && size_t(R) * g.heads * t->spans * (g.head_dim + 2) > e->attn_partial_floats)
        return e->fail(SPL_ERR_INVALID_ROWS, "invalid step rows: attention partials exceed the engine's buffers");
    // A plain RMSNorm into an operand: the first block's input (the embedding's output) and the final norm.
    auto norm = [&](int rows, const uint16_t *weight, const uint32_t *gather, const SplOperand &dst) {
        launch_step(spl_rmsnorm_kernel, dim3(rows), dim3(256), 0, e->stream, e->h, H, weight, gather, dst, H, g.eps);
    };
    // Every other norm is deferred (Sources/SploshRuntime/Engine.swift:1439-1451): the GEMM that adds into the residual
    // stream leaves bf16(h * w) as the next operand with the squares of h, and the GEMM that reads it scales its sums.
    GemmExtras scaled; scaled.in_squares = e->xn_squares; scaled.in_dim = H; scaled.eps = g.eps;
    bool fits = true;
    int linear_index = 0, full_index = 0;
    // The conv kernel cuts long runs in segments of rows, a block each: as many as the step's longest run has.
    int conv_segments = 1;
    for (uint32_t r = 0; r < t->run_count; ++r) conv_segments = std::max(conv_segments, int((t->runs[r * 3 + 2] + SPL_GDN_CONV_SEGMENT - 1) / SPL_GDN_CONV_SEGMENT));
    for (int l = 0; l < g.layers; ++l) {
        const LayerWeights &L = e->layers[l];
        const int live = (l + 1 == g.layers) ? int(t->live_rows) : R;
        int feature_tap = -1;
        for (size_t f = 0; f < e->feature_layers.size(); ++f) if (e->feature_layers[f] == l) feature_tap = int(f);
        if (l == 0 || gguf) {
            profile_begin(e, KLASS_ELEMENTWISE, 0);
            norm(R, L.vec[SPL_VEC_INPUT_NORM], nullptr, xn);
            profile_end(e);
        }
        if (gguf) ggemm(L.g_in_proj, gxn, e->proj, nullptr, R);
        else fits &= launch_gemm(e, L.in_proj, gxn, e->proj, nullptr, R, l == 0 ? GemmExtras() : scaled);
        if (!L.full) {
            SplGdnParams p;
            p.rows = R; p.runs = int(t->run_count); p.channels = sh.C; p.key_heads = g.gdn_key_heads; p.value_heads = g.gdn_value_heads;
            p.head_dim = g.gdn_head_dim; p.proj_ld = L.in_proj.ld; p.z_offset = sh.gdn_z; p.a_offset = sh.gdn_a; p.b_offset = sh.gdn_b; p.eps = g.eps; p.chunk_min = chunked_runs > 0 ? e->gdn_chunk_min : 0; p.out_file_order = e->gdn_out_file_order ? 1 : 0;
            profile_begin(e, KLASS_GDN, 0);
            launch_step(spl_gdn_conv_kernel, dim3(dim3((sh.C + 255) / 256, t->run_count, conv_segments)), dim3(256), 0, e->stream, 
                e->proj, L.vec[SPL_VEC_CONV], e->conv[linear_index], e->d_runs, e->d_row_read, e->d_row_write, e->gdn_act, p);
            profile_end(e);
            profile_begin(e, KLASS_GDN, 0);
            launch_step(spl_gdn_recurrence_kernel, dim3(dim3(g.gdn_value_heads, t->run_count)), dim3(SPL_GDN_THREADS), spl_gdn_recurrence_smem(), e->stream, 
                e->gdn_act, e->proj, L.vec[SPL_VEC_A_LOG], L.vec[SPL_VEC_DT_BIAS], L.vec[SPL_VEC_GDN_NORM], e->state[linear_index],
                e->journal[linear_index], e->d_runs, e->d_run_info, core, p);
            profile_end(e);
            if (chunked_runs > 0) {
                const SplGdnChunkTables ct{e->d_chunk_runs, e->d_chunks, chunked_runs, chunk_count};
                profile_begin(e, KLASS_GDN, 0);
                launch_step(spl_gdn_chunk_prepare_kernel, dim3(g.gdn_value_heads, chunk_count), dim3(256), spl_gdn_chunk_prepare_smem(), e->stream,
                    e->gdn_act, e->proj, L.vec[SPL_VEC_A_LOG], L.vec[SPL_VEC_DT_BIAS], ct, e->gdn_records, p);
                profile_end(e);
                profile_begin(e, KLASS_GDN, 0);
                launch_step(spl_gdn_chunk_scan_kernel, dim3(g.gdn_value_heads, chunked_runs, SPL_GDN_SLICES), dim3(256), spl_gdn_chunk_scan_smem(), e->stream,
                    e->gdn_records, ct, e->state[linear_index], e->journal[linear_index], e->gdn_o_raw, p);
                profile_end(e);
                profile_begin(e, KLASS_GDN, 0);
                launch_step(spl_gdn_chunk_finish_kernel, dim3(g.gdn_value_heads, chunk_count), dim3(256), 0, e->stream,
                    e->gdn_o_raw, e->proj, L.vec[SPL_VEC_GDN_NORM], ct, core, p);
                profile_end(e);
            }
            ++linear_index;
        } else {
            SplAttnParams p;
            p.rows = R; p.live = live; p.heads = g.heads; p.kv_heads = g.kv_heads; p.head_dim = g.head_dim; p.rotary = g.rotary_dim;
            p.max_pages = e->host->max_pages; p.proj_ld = L.in_proj.ld; p.k_offset = sh.att_k; p.v_offset = sh.att_v;
            p.spans = int(t->spans); p.pages_per_span = int(t->pages_per_span); p.eps = g.eps; p.scale = 1.0f / sqrtf(float(g.head_dim));
            profile_begin(e, KLASS_ATTENTION, 0);
            launch_step(spl_attn_prepare_kernel, dim3(dim3(g.heads + (e->kv_store ? g.kv_heads : 0), R)), dim3(128), 0, e->stream, 
                e->proj, L.vec[SPL_VEC_Q_NORM], L.vec[SPL_VEC_K_NORM], e->inv_freq, e->d_row_slot, e->d_row_pos, e->d_page_table, e->q,
                e->k_codes[full_index], e->k_scale[full_index], e->v_codes[full_index], e->v_scale[full_index], p);
            profile_end(e);
            if (live > 0) {
                // Blocks are in row order: those that begin below `live` hold the computed rows.
                int blocks = 0;
                for (; blocks < int(t->attn_block_count); ++blocks)
                    if (int(t->attn_blocks[blocks * 2]) >= live) break;
                profile_begin(e, KLASS_ATTENTION, 0);
                launch_scan(e, dim3(g.kv_heads * t->spans, blocks), p, full_index);
                profile_end(e);
                profile_begin(e, KLASS_ATTENTION, 0);
                launch_step(spl_attn_merge_kernel, dim3(dim3(g.heads, live)), dim3(g.head_dim), 0, e->stream, e->attn_partials, e->proj, core, p);
                profile_end(e);
            }
            ++full_index;
        }
        if (live > 0 && gguf) {
            ggemm(L.g_out_proj, gcore, e->h, e->h, live);
            profile_begin(e, KLASS_ELEMENTWISE, 0);
            norm(live, L.vec[SPL_VEC_POST_NORM], nullptr, xn);
            profile_end(e);
            ggemm(L.g_gate_up, gxn, e->gate_up, nullptr, live);
            profile_begin(e, KLASS_ELEMENTWISE, 0);
            launch_step(spl_swiglu_kernel, dim3(g.inter / 64, live), dim3(32), 0, e->stream, (const float *)e->gate_up, e->gate_up_ld, g.inter, act);
            profile_end(e);
            ggemm(L.g_down, gact, e->h, e->h, live);
        } else if (live > 0) {
            // The mixer's output projection adds into the residual stream and leaves the post norm's operand.
            GemmExtras mixer; mixer.emit_weight = L.vec[SPL_VEC_POST_NORM]; mixer.emit_out = &xn; mixer.emit_squares = e->xn_squares;
            fits &= launch_gemm(e, L.out_proj, gcore, e->h, e->h, live, mixer);
            // gate|up and the SiLU gate in one kernel: the GEMM's blocks write act = bf16(silu(gate) * up) and its sums.
            GemmExtras mlp = scaled; mlp.fuse_act = &act;
            fits &= launch_gemm(e, L.gate_up, gxn, e->gate_up, nullptr, live, mlp);
            // The down projection leaves the next block's input norm operand (the final norm gathers rows: it stays a kernel).
            GemmExtras down;
            if (l + 1 < g.layers) { down.emit_weight = e->layers[l + 1].vec[SPL_VEC_INPUT_NORM]; down.emit_out = &xn; down.emit_squares = e->xn_squares; }
            fits &= launch_gemm(e, L.down, gact, e->h, e->h, live, down);
        }
        if (e->taps_enabled) SPL_CUDA(cudaMemcpyAsync(e->taps + size_t(l) * e->c.max_rows * H, e->h, size_t(R) * H * 4, cudaMemcpyDeviceToDevice, e->stream));
        if (feature_tap >= 0) {
            const size_t width = e->feature_layers.size() * size_t(H);
            SPL_CUDA(cudaMemcpy2DAsync(e->features + size_t(feature_tap) * H, width * 4, e->h, size_t(H) * 4, size_t(H) * 4, live,
                                       cudaMemcpyDeviceToDevice, e->stream));
        }
    }
    if (t->logit_rows > 0) {
        profile_begin(e, KLASS_OTHER, 0);
        const int lrn = gguf ? std::min(operand_rn(int(t->logit_rows)), 64) : operand_rn(int(t->logit_rows)), lblocks = (int(t->logit_rows) + lrn - 1) / lrn;
        norm(int(t->logit_rows), e->final_norm, e->d_gather, SplOperand{e->hsn, e->hsn_sums, lrn, lblocks});
        profile_end(e);
        if (gguf) ggemm(e->g_head, GemmOperand{e->hsn, e->hsn_sums, lrn, lblocks}, e->logits, nullptr, int(t->logit_rows));
        else fits &= launch_gemm(e, e->head, GemmOperand{e->hsn, e->hsn_sums, lrn, lblocks}, e->logits, nullptr, int(t->logit_rows));
    }
    if (!fits) return e->fail(SPL_ERR_INVALID_ROWS, "invalid step rows: the GEMM scratch is smaller than the step needs");
    SPL_CUDA(cudaEventRecord(e->ev_end, e->stream));
    e->flying_rows = R; e->flying_logit_rows = int(t->logit_rows);
    return check_launch(e, "step launch");
}

spl_status finish_step(spl_engine *e, spl_step_stats *stats) {
    const int R = e->flying_rows;
    SPL_CUDA(cudaSetDevice(e->device));
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    {
        int flag[4] = {0, 0, 0, 0};
        SPL_CUDA(cudaMemcpy(flag, e->tc_error, sizeof flag, cudaMemcpyDeviceToHost));
        if (flag[0]) {
            cudaMemset(e->tc_error, 0, sizeof flag);
            if (flag[0] >= 100) return e->fail(SPL_ERR_TIMEOUT, "an attention scan block gave up waiting (warp " + std::to_string(flag[0] - 100) + ")");
            // The wait that ran out first: 10 weight copy for a free stage; 20, 21 activation copy for a free tile of means, a free
            // stage; 30-37 tensor-core issue (two warps) for a tile of means, activations, converted weights;
            // 40-42 conversion for the accumulators' completion, a weight stage, a free operand slot.
            return e->fail(SPL_ERR_TIMEOUT, "a GEMM block gave up waiting (warp " + std::to_string(flag[0] - 1) + "; first wait " + std::to_string(flag[1]) +
                                            " at " + std::to_string(flag[2]) + ", block " + std::to_string(flag[3] & 0xFFFF) + ")");
        }
    }
    profile_collect(e);
    e->last_rows = R; e->last_logit_rows = e->flying_logit_rows;
    if (stats) {
        float ms = 0;
        cudaEventElapsedTime(&ms, e->ev_begin, e->ev_end);
        stats->rows = R; stats->launches = e->launches; stats->gpu_seconds = ms / 1000.0;
        stats->wall_seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - e->wall0).count();
    }
    return SPL_OK;
}

spl_status run_step(spl_engine *e, const spl_tables *t, spl_step_stats *stats) {
    if (e->in_flight) return e->fail(SPL_ERR_INVALID_ARGUMENT, "a step is in flight: call spl_step_wait first");
    const spl_status queued = enqueue_step(e, t);
    return queued == SPL_OK ? finish_step(e, stats) : queued;
}

spl_status upload_q4_into(spl_engine *e, SplQ4Dev &w, int n0, int rows, int inner, const uint32_t *packed, const uint16_t *scales,
                          const uint16_t *biases, bool device_source) {
    const size_t words = size_t(rows) * inner / 8, groups = size_t(rows) * inner / 64;
    const uint32_t *dp = packed; const uint16_t *ds = scales, *db = biases;
    uint32_t *sp = nullptr; uint16_t *ss = nullptr, *sbias = nullptr;
    if (!device_source) {
        SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&sp), words * 4));
        SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&ss), groups * 2));
        SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&sbias), groups * 2));
        SPL_CUDA(cudaMemcpyAsync(sp, packed, words * 4, cudaMemcpyHostToDevice, e->stream));
        SPL_CUDA(cudaMemcpyAsync(ss, scales, groups * 2, cudaMemcpyHostToDevice, e->stream));
        SPL_CUDA(cudaMemcpyAsync(sbias, biases, groups * 2, cudaMemcpyHostToDevice, e->stream));
        dp = sp; ds = ss; db = sbias;
    }
    int *bad = nullptr;
    SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&bad), sizeof(int)));
    SPL_CUDA(cudaMemsetAsync(bad, 0, sizeof(int), e->stream));
    spl_repack_q4_kernel<<<int(std::min<size_t>((words + 255) / 256, 16384)), 256, 0, e->stream>>>(dp, ds, db, rows, inner, w.codes, w.sb, n0, bad, w.interleave);
    spl_status launched = check_launch(e, "repack");
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    int flag = 0;
    cudaMemcpy(&flag, bad, sizeof flag, cudaMemcpyDeviceToHost);
    cudaFree(bad);
    if (sp) { cudaFree(sp); cudaFree(ss); cudaFree(sbias); }
    if (launched == SPL_OK && flag) launched = e->fail(SPL_ERR_INVALID_ARGUMENT, "a quantisation scale is outside [2^-13, 127] or a bias beyond 1023 in magnitude: the weight would not be exact in fp16");
    return launched;
}

// Where a tensor kind lands: which fused device tensor and at which 16-column block.
struct Placement { SplQ4Dev *dst; int n0; int rows; int inner; };   // n0: first column of the tensor inside the fused one

spl_status place(spl_engine *e, int layer, int kind, Placement *out) {
    const spl_geometry &g = e->g;
    const Shapes sh(g);
    if (layer < 0) {
        if (kind == SPL_Q4_HEAD) { *out = {&e->head, 0, g.vocab, g.hidden}; return SPL_OK; }
        return e->fail(SPL_ERR_INVALID_ARGUMENT, "model-level q4 kind must be embed or head");
    }
    if (layer >= g.layers) return e->fail(SPL_ERR_INVALID_ARGUMENT, "layer out of range");
    LayerWeights &L = e->layers[layer];
    switch (kind) {
    case SPL_Q4_QKV: if (L.full) break; *out = {&L.in_proj, 0, sh.C, g.hidden}; return SPL_OK;
    case SPL_Q4_Z: if (L.full) break; *out = {&L.in_proj, sh.gdn_z, sh.VD, g.hidden}; return SPL_OK;
    case SPL_Q4_A: if (L.full) break; *out = {&L.in_proj, sh.gdn_a, sh.VH, g.hidden}; return SPL_OK;
    case SPL_Q4_B: if (L.full) break; *out = {&L.in_proj, sh.gdn_b, sh.VH, g.hidden}; return SPL_OK;
    case SPL_Q4_OUT: if (L.full) break; *out = {&L.out_proj, 0, g.hidden, sh.VD}; return SPL_OK;
    case SPL_Q4_Q: if (!L.full) break; *out = {&L.in_proj, 0, 2 * sh.AD, g.hidden}; return SPL_OK;
    case SPL_Q4_K: if (!L.full) break; *out = {&L.in_proj, sh.att_k, sh.KV, g.hidden}; return SPL_OK;
    case SPL_Q4_V: if (!L.full) break; *out = {&L.in_proj, sh.att_v, sh.KV, g.hidden}; return SPL_OK;
    case SPL_Q4_O: if (!L.full) break; *out = {&L.out_proj, 0, g.hidden, sh.AD}; return SPL_OK;
    case SPL_Q4_GATE: *out = {&L.gate_up, 0, g.inter, g.hidden}; return SPL_OK;
    case SPL_Q4_UP: *out = {&L.gate_up, g.inter, g.inter, g.hidden}; return SPL_OK;
    case SPL_Q4_DOWN: *out = {&L.down, 0, g.hidden, g.inter}; return SPL_OK;
    }
    return e->fail(SPL_ERR_INVALID_ARGUMENT, "q4 kind does not belong to this layer's mixer");
}

int vec_count(const spl_geometry &g, int kind) {
    const Shapes sh(g);
    switch (kind) {
    case SPL_VEC_INPUT_NORM: case SPL_VEC_POST_NORM: case SPL_VEC_FINAL_NORM: return g.hidden;
    case SPL_VEC_CONV: return sh.C * 4;
    case SPL_VEC_A_LOG: case SPL_VEC_DT_BIAS: return sh.VH;
    case SPL_VEC_GDN_NORM: return g.gdn_head_dim;
    case SPL_VEC_Q_NORM: case SPL_VEC_K_NORM: return g.head_dim;
    }
    return -1;
}

spl_status create(const spl_geometry *gp, const spl_config *cp, spl_engine *e) {
    const spl_geometry &g = e->g = *gp;
    e->c = *cp;
    const Shapes sh(g);
    if (g.layers <= 0 || g.hidden % 256 || g.inter % 256 || sh.VD % 256 || sh.AD % 256 || g.gdn_head_dim != 128 ||
        (g.head_dim != 128 && g.head_dim != 256) || g.heads % g.kv_heads || g.gdn_value_heads % g.gdn_key_heads || g.vocab % 16 ||
        g.inter % 16 || sh.C % 16 || g.rotary_dim > g.head_dim || g.rotary_dim % 2 || !scan_supported(g))
        return e->fail(SPL_ERR_INVALID_ARGUMENT, "unsupported geometry");
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) return e->fail(SPL_ERR_UNSUPPORTED_DEVICE, "unsupported device: no CUDA device");
    if (cp->device < 0 || cp->device >= count) return e->fail(SPL_ERR_UNSUPPORTED_DEVICE, "unsupported device: ordinal out of range");
    cudaDeviceProp prop;
    SPL_CUDA(cudaGetDeviceProperties(&prop, cp->device));
    if (prop.major != 10) return e->fail(SPL_ERR_UNSUPPORTED_DEVICE, "unsupported device: kernels are built for sm_100a only");
    e->device = cp->device;
    SPL_CUDA(cudaSetDevice(e->device));
    if (!configure_device(e->device, &e->sms)) return e->fail(SPL_ERR_UNSUPPORTED_DEVICE, "unsupported device: the kernels' shared-memory opt-in failed");
    spl_status hs = spl_host_create(gp, cp, &e->host);
    if (hs != SPL_OK) return e->fail(hs, "invalid engine configuration");
    e->c = e->host->config;
    SPL_CUDA(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
    SPL_CUDA(cudaEventCreate(&e->ev_begin));
    SPL_CUDA(cudaEventCreate(&e->ev_end));
    const int R = e->c.max_rows, H = g.hidden;

    e->layers.resize(g.layers);
    for (int l = 0; l < g.layers; ++l) {
        LayerWeights &L = e->layers[l];
        L.full = l % 4 == 3;
        spl_status s;
        if ((s = alloc_q4(e, L.in_proj, L.full ? sh.att_n : sh.gdn_n, H)) != SPL_OK) return s;
        if ((s = alloc_q4(e, L.out_proj, H, L.full ? sh.AD : sh.VD)) != SPL_OK) return s;
        if ((s = alloc_q4(e, L.gate_up, 2 * g.inter, H)) != SPL_OK) return s;
        L.gate_up.interleave = g.inter;
        if ((s = alloc_q4(e, L.down, H, g.inter)) != SPL_OK) return s;
    }
    spl_status s;
    if ((s = alloc_q4(e, e->head, g.vocab, H)) != SPL_OK) return s;
    if ((s = device_alloc(e, &e->embed_packed, size_t(g.vocab) * H / 8, &e->weight_bytes)) != SPL_OK) return s;
    if ((s = device_alloc(e, &e->embed_scales, size_t(g.vocab) * H / 64, &e->weight_bytes)) != SPL_OK) return s;
    if ((s = device_alloc(e, &e->embed_biases, size_t(g.vocab) * H / 64, &e->weight_bytes)) != SPL_OK) return s;
    {
        std::vector<float> freq(std::max(1, g.rotary_dim / 2));
        for (int i = 0; i < g.rotary_dim / 2; ++i) freq[i] = float(std::pow(double(g.rope_theta), -2.0 * double(i) / double(g.rotary_dim)));
        if ((s = device_alloc(e, &e->inv_freq, freq.size())) != SPL_OK) return s;
        SPL_CUDA(cudaMemcpy(e->inv_freq, freq.data(), freq.size() * 4, cudaMemcpyHostToDevice));
    }
    // Session state.
    const size_t page_vecs = size_t(g.kv_heads) * SPL_PAGE_TOKENS;
    e->kv_page_bytes = (page_vecs * g.head_dim + page_vecs * 4) * 2;
    e->state_layer_bytes = size_t(g.gdn_value_heads) * 128 * 128 * 4;
    e->conv_unit_bytes = size_t(sh.C) * 3 * 4;
    e->journal_bytes = size_t(e->c.max_slots) * SPL_JOURNAL_ROWS * g.gdn_value_heads * SPL_JOURNAL_WIDTH * 4;
    for (int l = 0; l < g.layers; ++l) {
        if (l % 4 == 3) {
            int8_t *kc, *vc; float *ks, *vs;
            const size_t codes = size_t(e->c.kv_pages) * page_vecs * g.head_dim, scales = size_t(e->c.kv_pages) * page_vecs;
            if ((s = device_alloc(e, &kc, codes, &e->kv_pool_bytes)) != SPL_OK) return s;
            if ((s = device_alloc(e, &vc, codes, &e->kv_pool_bytes)) != SPL_OK) return s;
            if ((s = device_alloc(e, &ks, scales, &e->kv_pool_bytes)) != SPL_OK) return s;
            if ((s = device_alloc(e, &vs, scales, &e->kv_pool_bytes)) != SPL_OK) return s;
            // A scale that was never stored reads as NaN, so a masked token that leaks shows.
            SPL_CUDA(cudaMemsetAsync(kc, 0xFF, codes, e->stream)); SPL_CUDA(cudaMemsetAsync(vc, 0xFF, codes, e->stream));
            SPL_CUDA(cudaMemsetAsync(ks, 0xFF, scales * 4, e->stream)); SPL_CUDA(cudaMemsetAsync(vs, 0xFF, scales * 4, e->stream));
            e->k_codes.push_back(kc); e->v_codes.push_back(vc); e->k_scale.push_back(ks); e->v_scale.push_back(vs);
        } else {
            float *st, *cv, *jr;
            if ((s = device_alloc(e, &st, size_t(e->c.max_slots) * e->state_layer_bytes / 4)) != SPL_OK) return s;
            if ((s = device_alloc(e, &cv, size_t(e->c.state_units) * e->conv_unit_bytes / 4)) != SPL_OK) return s;
            if ((s = device_alloc(e, &jr, e->journal_bytes / 4)) != SPL_OK) return s;
            SPL_CUDA(cudaMemsetAsync(st, 0, size_t(e->c.max_slots) * e->state_layer_bytes, e->stream));
            SPL_CUDA(cudaMemsetAsync(cv, 0, size_t(e->c.state_units) * e->conv_unit_bytes, e->stream));
            SPL_CUDA(cudaMemsetAsync(jr, 0, e->journal_bytes, e->stream));
            e->state.push_back(st); e->conv.push_back(cv); e->journal.push_back(jr);
        }
    }
    // Activations.
    e->proj_ld = std::max(sh.gdn_n, sh.att_n); e->gate_up_ld = 2 * g.inter; e->core_ld = std::max(sh.VD, sh.AD); e->logits_ld = g.vocab;
    const int LR = e->c.max_logit_rows;
    if ((s = device_alloc(e, &e->h, size_t(R) * H, &e->scratch_bytes)) != SPL_OK) return s;
    e->rows_padded = (R + 127) / 128 * 128; e->logit_rows_padded = (e->c.max_logit_rows + 127) / 128 * 128;
    const int RP = e->rows_padded, LP = e->logit_rows_padded;
    if ((s = device_alloc(e, &e->xn, size_t(RP) * H, &e->scratch_bytes)) != SPL_OK) return s;
    if ((s = device_alloc(e, &e->xn_sums, spl_operand_sums_floats(RP, H), &e->scratch_bytes)) != SPL_OK) return s;
    if ((s = device_alloc(e, &e->core_sums, spl_operand_sums_floats(RP, e->core_ld), &e->scratch_bytes)) != SPL_OK) return s;
    if ((s = device_alloc(e, &e->act_sums, spl_operand_sums_floats(RP, g.inter), &e->scratch_bytes)) != SPL_OK) return s;
    if ((s = device_alloc(e, &e->hsn_sums, spl_operand_sums_floats(LP, H), &e->scratch_bytes)) != SPL_OK) return s;
    if ((s = device_alloc(e, &e->tc_error, 64)) != SPL_OK) return s;
    SPL_CUDA(cudaMemsetAsync(e->tc_error, 0, 64 * sizeof(int), e->stream));
    SPL_CUDA(cudaMemsetAsync(e->xn, 0, size_t(RP) * H * 2, e->stream));
    SPL_CUDA(cudaMemsetAsync(e->xn_sums, 0, spl_operand_sums_floats(RP, H) * 4, e->stream));
    SPL_CUDA(cudaMemsetAsync(e->core_sums, 0, spl_operand_sums_floats(RP, e->core_ld) * 4, e->stream));
    SPL_CUDA(cudaMemsetAsync(e->act_sums, 0, spl_operand_sums_floats(RP, g.inter) * 4, e->stream));
    SPL_CUDA(cudaMemsetAsync(e->hsn_sums, 0, spl_operand_sums_floats(LP, H) * 4, e->stream));
    if ((s = device_alloc(e, &e->proj, size_t(R) * e->proj_ld, &e->scratch_bytes)) != SPL_OK) return s;
    if ((s = device_alloc(e, &e->gdn_act, size_t(R) * sh.C, &e->scratch_bytes)) != SPL_OK) return s;
    if ((s = device_alloc(e, &e->core, size_t(RP) * e->core_ld, &e->scratch_bytes)) != SPL_OK) return s;
    SPL_CUDA(cudaMemsetAsync(e->core, 0, size_t(RP) * e->core_ld * 2, e->stream));
    if ((s = device_alloc(e, &e->gate_up, size_t(R) * e->gate_up_ld, &e->scratch_bytes)) != SPL_OK) return s;
    if ((s = device_alloc(e, &e->act, size_t(RP) * g.inter, &e->scratch_bytes)) != SPL_OK) return s;
    SPL_CUDA(cudaMemsetAsync(e->act, 0, size_t(RP) * g.inter * 2, e->stream));
    if ((s = device_alloc(e, &e->q, size_t(R) * sh.AD, &e->scratch_bytes)) != SPL_OK) return s;
    if ((s = device_alloc(e, &e->hsn, size_t(LP) * H, &e->scratch_bytes)) != SPL_OK) return s;
    SPL_CUDA(cudaMemsetAsync(e->hsn, 0, size_t(LP) * H * 2, e->stream));
    if ((s = device_alloc(e, &e->logits, size_t(LR) * e->logits_ld, &e->scratch_bytes)) != SPL_OK) return s;
    if ((s = device_alloc(e, &e->argmax_ids, size_t(LR), &e->scratch_bytes)) != SPL_OK) return s;
    e->partial_floats = size_t(16) * RP * std::max(H, 4096);      // split-K partial sums of the GGUF kernel
    if ((s = device_alloc(e, &e->partials, e->partial_floats, &e->scratch_bytes)) != SPL_OK) return s;
    // Where the blocks of a cut tile of the q4 GEMM leave their partial sums: a slot of rn x 128 sums a block.
    const int row_blocks = std::max(RP, LP) / 128;      // more than 64 rows go in blocks of 128
    // The most slot space any of the engine's tensors takes, at any row count.
    e->slot_floats = 0;
    {
        struct Use { const SplQ4Dev *w; bool emit, whole; };
        std::vector<Use> all{{&e->head, false, false}};
        for (const LayerWeights &L : e->layers) { all.push_back({&L.in_proj, false, false}); all.push_back({&L.out_proj, true, false}); all.push_back({&L.gate_up, false, true}); all.push_back({&L.down, true, false}); }
        for (const Use &u : all)
            for (int rn : {16, 32, 64, 128})
                for (int rbs = 1; rbs <= (rn == 128 ? row_blocks : 1); ++rbs)
                    e->slot_floats = std::max(e->slot_floats, gemm_slot_floats(*u.w, e->sms, rn, rbs, u.emit, u.whole));
    }
    if ((s = device_alloc(e, &e->slots, e->slot_floats, &e->scratch_bytes)) != SPL_OK) return s;
    if (R >= SPL_GDN_CHUNK && !e->state.empty()) {
        e->gdn_chunks_max = R / SPL_GDN_CHUNK + e->c.max_slots;
        if ((s = device_alloc(e, &e->gdn_records, size_t(e->gdn_chunks_max) * g.gdn_value_heads * SPL_GDN_REC_FLOATS, &e->scratch_bytes)) != SPL_OK) return s;
        if ((s = device_alloc(e, &e->gdn_o_raw, size_t(R) * sh.VD, &e->scratch_bytes)) != SPL_OK) return s;
    }
    if ((s = device_alloc(e, &e->xn_squares, size_t(RP) * (H / 64), &e->scratch_bytes)) != SPL_OK) return s;
    SPL_CUDA(cudaMemsetAsync(e->xn_squares, 0, size_t(RP) * (H / 64) * 4, e->stream));
    e->attn_partial_floats = size_t(std::max(16 * R, 64 * std::min(R, 128))) * g.heads * (g.head_dim + 2);
    if ((s = device_alloc(e, &e->attn_partials, e->attn_partial_floats, &e->scratch_bytes)) != SPL_OK) return s;
    e->tables_words = size_t(R) * 5 + size_t(e->c.max_slots) * 5 + size_t(LR) + size_t(R) * 2 + size_t(e->c.max_slots) * e->host->max_pages + 64
                      + size_t(e->c.max_slots) * 4 + (size_t(R) / SPL_GDN_CHUNK + e->c.max_slots) * 4 + 16;
    SPL_CUDA(cudaMallocHost(reinterpret_cast<void **>(&e->tables_host), e->tables_words * 4));
    if ((s = device_alloc(e, &e->tables_dev, e->tables_words)) != SPL_OK) return s;
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    return SPL_OK;
}

}  // namespace

extern "C" {

spl_status spl_engine_create(const spl_geometry *geometry, const spl_config *config, spl_engine **out) {
    if (!geometry || !config || !out) return SPL_ERR_INVALID_ARGUMENT;
    spl_engine *e = new spl_engine;
    const spl_status s = create(geometry, config, e);
    *out = e;               // returned even on failure so the caller can read the error string
    return s;
}

void spl_engine_destroy(spl_engine *e) {
    if (!e) return;
    if (e->stream) cudaStreamSynchronize(e->stream);
    auto release_q4 = [](SplQ4Dev &w) { cudaFree(w.codes); cudaFree(w.sb); };
    for (LayerWeights &L : e->layers) {
        release_q4(L.in_proj); release_q4(L.out_proj); release_q4(L.gate_up); release_q4(L.down);
        for (uint16_t *v : L.vec) cudaFree(v);
    }
    release_q4(e->head);
    cudaFree(e->embed_packed); cudaFree(e->embed_scales); cudaFree(e->embed_biases); cudaFree(e->final_norm); cudaFree(e->inv_freq);
    cudaFree(e->g_embed); cudaFree(e->g_head.blocks);
    for (LayerWeights &L : e->layers) { cudaFree(L.g_in_proj.blocks); cudaFree(L.g_out_proj.blocks); cudaFree(L.g_gate_up.blocks); cudaFree(L.g_down.blocks); }
    for (auto p : e->k_codes) cudaFree(p); for (auto p : e->v_codes) cudaFree(p);
    for (auto p : e->k_scale) cudaFree(p); for (auto p : e->v_scale) cudaFree(p);
    for (auto p : e->state) cudaFree(p); for (auto p : e->conv) cudaFree(p); for (auto p : e->journal) cudaFree(p);
    cudaFree(e->h); cudaFree(e->xn); cudaFree(e->proj); cudaFree(e->gdn_act); cudaFree(e->core); cudaFree(e->gate_up); cudaFree(e->act);
    cudaFree(e->q); cudaFree(e->hsn); cudaFree(e->logits); cudaFree(e->argmax_ids); cudaFree(e->partials); cudaFree(e->attn_partials);
    cudaFree(e->taps); cudaFree(e->features); cudaFree(e->topk_ids); cudaFree(e->topk_values); cudaFree(e->tables_dev); cudaFree(e->gdn_records); cudaFree(e->gdn_o_raw); cudaFree(e->slots); cudaFree(e->xn_squares); cudaFree(e->xn_sums); cudaFree(e->core_sums); cudaFree(e->act_sums); cudaFree(e->hsn_sums); cudaFree(e->tc_error);
    if (e->tables_host) cudaFreeHost(e->tables_host);
    for (ProfileSlot &s : e->profile_slots) { cudaEventDestroy(s.begin); cudaEventDestroy(s.end); }
    if (e->ev_begin) cudaEventDestroy(e->ev_begin);
    if (e->ev_end) cudaEventDestroy(e->ev_end);
    if (e->stream) cudaStreamDestroy(e->stream);
    spl_host_destroy(e->host);
    delete e;
}

const char *spl_last_error_string(const spl_engine *e) {
    if (!e) return "no engine";
    if (e->error.empty() && e->host) return e->host->error.c_str();
    return e->error.c_str();
}

spl_status spl_weights_set_q4(spl_engine *e, int32_t layer, int32_t kind, int32_t rows, int32_t inner,
                              const uint32_t *packed, const uint16_t *scales, const uint16_t *biases) {
    if (!e || !packed || !scales || !biases) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    if (layer < 0 && kind == SPL_Q4_EMBED) {
        if (rows != e->g.vocab || inner != e->g.hidden) return e->fail(SPL_ERR_INVALID_ARGUMENT, "embedding shape does not match the geometry");
        SPL_CUDA(cudaMemcpy(e->embed_packed, packed, size_t(rows) * inner / 2, cudaMemcpyHostToDevice));
        SPL_CUDA(cudaMemcpy(e->embed_scales, scales, size_t(rows) * inner / 32, cudaMemcpyHostToDevice));
        SPL_CUDA(cudaMemcpy(e->embed_biases, biases, size_t(rows) * inner / 32, cudaMemcpyHostToDevice));
        return SPL_OK;
    }
    Placement pl;
    const spl_status s = place(e, layer, kind, &pl);
    if (s != SPL_OK) return s;
    if (rows != pl.rows || inner != pl.inner) return e->fail(SPL_ERR_INVALID_ARGUMENT, "tensor shape does not match the geometry");
    return upload_q4_into(e, *pl.dst, pl.n0, rows, inner, packed, scales, biases, false);
}

spl_status spl_weights_set_vector(spl_engine *e, int32_t layer, int32_t kind, const uint16_t *bf16, int32_t count) {
    if (!e || !bf16 || kind < 0 || kind >= SPL_VEC_KINDS) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    if (count != vec_count(e->g, kind)) return e->fail(SPL_ERR_INVALID_ARGUMENT, "vector length does not match the geometry");
    SPL_CUDA(cudaSetDevice(e->device));
    uint16_t **slot = nullptr;
    if (kind == SPL_VEC_FINAL_NORM) slot = &e->final_norm;
    else {
        if (layer < 0 || layer >= e->g.layers) return e->fail(SPL_ERR_INVALID_ARGUMENT, "layer out of range");
        slot = &e->layers[layer].vec[kind];
    }
    if (!*slot) SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(slot), size_t(count) * 2));
    SPL_CUDA(cudaMemcpy(*slot, bf16, size_t(count) * 2, cudaMemcpyHostToDevice));
    return SPL_OK;
}

// The GGUF twin of a q4 device tensor of the engine.
static SplGgufDev *gguf_twin(spl_engine *e, const SplQ4Dev *q) {
    if (q == &e->head) return &e->g_head;
    for (LayerWeights &L : e->layers) {
        if (q == &L.in_proj) return &L.g_in_proj;
        if (q == &L.out_proj) return &L.g_out_proj;
        if (q == &L.gate_up) return &L.g_gate_up;
        if (q == &L.down) return &L.g_down;
    }
    return nullptr;
}

// Native blocks [rows][inner / 256] of `format` become columns [n0, n0 + rows) of the GGUF twin of `q`; the twin is
// allocated (and the q4 tensor it replaces freed) the first time.
static spl_status upload_gguf_into(spl_engine *e, SplQ4Dev &q, int n0, int rows, int inner, int format, const unsigned char *native, bool device_source) {
    SplGgufDev *w = gguf_twin(e, &q);
    if (!w) return e->fail(SPL_ERR_INVALID_ARGUMENT, "no such tensor");
    if (inner % 256) return e->fail(SPL_ERR_INVALID_ARGUMENT, "a GGUF tensor's inner dimension must be a multiple of 256");
    if (!w->blocks) {
        w->n = q.n; w->ld = q.ld; w->tiles = q.tiles; w->k = q.k; w->format = format;
        SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&w->blocks), w->device_bytes()));
        SPL_CUDA(cudaMemsetAsync(w->blocks, 0, w->device_bytes(), e->stream));      // columns nobody sets are zero blocks: weights 0
        e->weight_bytes += w->device_bytes();
        if (q.codes) { e->weight_bytes -= q.device_bytes(); cudaFree(q.codes); cudaFree(q.sb); q.codes = nullptr; q.sb = nullptr; }
    } else if (w->format != format) {
        return e->fail(SPL_ERR_INVALID_ARGUMENT, "tensors fused into one device tensor (qkv, z, a, b; q, k, v; gate, up) must share a GGUF type");
    }
    const size_t bytes = size_t(rows) * (inner / 256) * spl_gguf_block_bytes(format);
    unsigned char *staged = nullptr;
    if (!device_source) {
        SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&staged), bytes));
        SPL_CUDA(cudaMemcpyAsync(staged, native, bytes, cudaMemcpyHostToDevice, e->stream));
        native = staged;
    }
    const size_t items = size_t(rows) * (inner / 256) * spl_gguf_pieces(format);
    spl_repack_gguf_kernel<<<int(std::min<size_t>((items + 255) / 256, 16384)), 256, 0, e->stream>>>(native, rows, inner / 256, format, w->blocks, n0);
    const spl_status launched = check_launch(e, "gguf repack");
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    cudaFree(staged);
    return launched;
}

spl_status spl_engine_geometry(const spl_engine *e, spl_geometry *out) {
    if (!e || !out) return SPL_ERR_INVALID_ARGUMENT;
    *out = e->g;
    return SPL_OK;
}

spl_status spl_weights_gguf_file_order(spl_engine *e, int32_t enabled) {
    if (!e) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    e->gdn_out_file_order = enabled != 0;
    return SPL_OK;
}

static bool gguf_type_ok(int type) { return type == SPL_GGUF_Q4K || type == SPL_GGUF_Q5K || type == SPL_GGUF_Q6K; }

spl_status spl_weights_set_gguf(spl_engine *e, int32_t layer, int32_t kind, int32_t type, int32_t rows, int32_t inner, const uint8_t *blocks) {
    if (!e || !blocks) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    if (!gguf_type_ok(type)) return e->fail(SPL_ERR_INVALID_ARGUMENT, "GGUF type must be 12 (Q4_K), 13 (Q5_K) or 14 (Q6_K)");
    SPL_CUDA(cudaSetDevice(e->device));
    if (layer < 0 && kind == SPL_Q4_EMBED) {
        if (rows != e->g.vocab || inner != e->g.hidden || inner % 256) return e->fail(SPL_ERR_INVALID_ARGUMENT, "embedding shape does not match the geometry");
        const size_t bytes = size_t(rows) * (inner / 256) * spl_gguf_block_bytes(type);
        cudaFree(e->g_embed); e->g_embed = nullptr;
        SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&e->g_embed), bytes));
        SPL_CUDA(cudaMemcpy(e->g_embed, blocks, bytes, cudaMemcpyHostToDevice));
        e->g_embed_format = type;
        return SPL_OK;
    }
    Placement pl;
    const spl_status s = place(e, layer, kind, &pl);
    if (s != SPL_OK) return s;
    if (rows != pl.rows || inner != pl.inner) return e->fail(SPL_ERR_INVALID_ARGUMENT, "tensor shape does not match the geometry");
    return upload_gguf_into(e, *pl.dst, pl.n0, rows, inner, type, blocks, false);
}

// Seeded synthetic GGUF weights for timing (no host copy of a 27B model exists here): every block tensor as
// `block_type`, the embedding and the head as `head_type`.
spl_status spl_weights_synthesize_gguf(spl_engine *e, uint64_t seed, int32_t block_type, int32_t head_type) {
    if (!e) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    if (!gguf_type_ok(block_type) || !gguf_type_ok(head_type)) return e->fail(SPL_ERR_INVALID_ARGUMENT, "GGUF type must be 12 (Q4_K), 13 (Q5_K) or 14 (Q6_K)");
    SPL_CUDA(cudaSetDevice(e->device));
    const spl_geometry &g = e->g;
    if (g.hidden % 256 || g.inter % 256) return e->fail(SPL_ERR_INVALID_ARGUMENT, "GGUF tensors need inner dimensions that are multiples of 256");
    const size_t most = size_t(std::max(g.vocab, std::max(2 * g.heads * g.head_dim, g.inter))) * (std::max(g.hidden, g.inter) / 256) * 210;
    unsigned char *staged = nullptr;
    SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&staged), most));
    spl_status result = SPL_OK;
    auto fill = [&](unsigned char *dst, int rows, int inner, int type, uint64_t stream_seed) {
        const size_t blocks = size_t(rows) * (inner / 256);
        spl_synth_gguf_kernel<<<int(std::min<size_t>((blocks + 127) / 128, 65535)), 128, 0, e->stream>>>(dst, blocks, type, stream_seed);
    };
    for (int layer = -1; layer < g.layers && result == SPL_OK; ++layer)
        for (int kind = 0; kind < SPL_Q4_KINDS && result == SPL_OK; ++kind) {
            if (layer < 0) {
                if (kind == SPL_Q4_EMBED) {
                    const size_t bytes = size_t(g.vocab) * (g.hidden / 256) * spl_gguf_block_bytes(head_type);
                    cudaFree(e->g_embed); e->g_embed = nullptr;
                    if (cudaMalloc(reinterpret_cast<void **>(&e->g_embed), bytes) != cudaSuccess) { result = e->fail(SPL_ERR_ALLOCATION_FAILED, "embedding table"); break; }
                    fill(e->g_embed, g.vocab, g.hidden, head_type, seed ^ 0xE3BEDull);
                    e->g_embed_format = head_type;
                } else if (kind == SPL_Q4_HEAD) {
                    fill(staged, g.vocab, g.hidden, head_type, seed ^ 0x4EADull);
                    result = upload_gguf_into(e, e->head, 0, g.vocab, g.hidden, head_type, staged, true);
                }
                continue;
            }
            if (kind >= SPL_Q4_EMBED) continue;
            const bool full_layer = e->layers[layer].full;
            if ((kind <= SPL_Q4_OUT && full_layer) || (kind >= SPL_Q4_Q && kind <= SPL_Q4_O && !full_layer)) continue;
            Placement pl;
            if ((result = place(e, layer, kind, &pl)) != SPL_OK) break;
            fill(staged, pl.rows, pl.inner, block_type, seed ^ (uint64_t(layer) * 64 + kind + 1) * 0x9E3779B97F4A7C15ull);
            result = upload_gguf_into(e, *pl.dst, pl.n0, pl.rows, pl.inner, block_type, staged, true);
        }
    cudaStreamSynchronize(e->stream);
    cudaFree(staged);
    return result;
}

static uint64_t fnv1a64(const char *s) {
    uint64_t h = 0xcbf29ce484222325ull;
    for (; *s; ++s) { h ^= uint8_t(*s); h *= 0x100000001b3ull; }
    return h;
}

spl_status spl_weights_synthesize_q4(spl_engine *e, uint64_t seed) {
    if (!e) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    static const char *names[SPL_Q4_KINDS] = {"linear_attn.in_proj_qkv", "linear_attn.in_proj_z", "linear_attn.in_proj_a", "linear_attn.in_proj_b",
                                              "linear_attn.out_proj", "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                                              "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj", "embed_tokens", "lm_head"};
    const float factor = 0.02f * (1.0f / 37837.2265625f);
    // Staging for the largest tensor in MLX layout.
    const size_t max_weights = size_t(std::max(e->g.vocab, std::max(2 * e->g.heads * e->g.head_dim, e->g.inter))) * std::max(e->g.hidden, e->g.inter);
    uint32_t *sp; uint16_t *ss, *sbias;
    SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&sp), max_weights / 2));
    SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&ss), max_weights / 32));
    SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&sbias), max_weights / 32));
    spl_status result = SPL_OK;
    for (int layer = -1; layer < e->g.layers && result == SPL_OK; ++layer) {
        for (int kind = 0; kind < SPL_Q4_KINDS && result == SPL_OK; ++kind) {
            char full[128];
            Placement pl;
            if (layer < 0) {
                if (kind != SPL_Q4_EMBED && kind != SPL_Q4_HEAD) continue;
                snprintf(full, sizeof full, "%s", names[kind]);
                pl = {kind == SPL_Q4_HEAD ? &e->head : nullptr, 0, e->g.vocab, e->g.hidden};
            } else {
                if (kind >= SPL_Q4_EMBED) continue;
                const bool full_layer = e->layers[layer].full;
                if ((kind <= SPL_Q4_OUT && full_layer) || (kind >= SPL_Q4_Q && kind <= SPL_Q4_O && !full_layer)) continue;
                snprintf(full, sizeof full, "layers.%d.%s", layer, names[kind]);
                if ((result = place(e, layer, kind, &pl)) != SPL_OK) break;
            }
            const size_t slots = size_t(pl.rows) * pl.inner / 64;
            uint32_t *dp = sp; uint16_t *ds = ss, *db = sbias;
            if (!pl.dst) { dp = e->embed_packed; ds = e->embed_scales; db = e->embed_biases; }
            spl_synth_q4_kernel<<<int(std::min<size_t>((slots + 127) / 128, 65535)), 128, 0, e->stream>>>(seed ^ fnv1a64(full), factor, pl.rows, pl.inner, dp, ds, db);
            if ((result = check_launch(e, "synthesize")) != SPL_OK) break;
            if (pl.dst) result = upload_q4_into(e, *pl.dst, pl.n0, pl.rows, pl.inner, sp, ss, sbias, true);
        }
    }
    cudaStreamSynchronize(e->stream);
    cudaFree(sp); cudaFree(ss); cudaFree(sbias);
    return result;
}

// Tables built outside the library are checked for range before anything is launched: the kernels index with them.
static spl_status check_tables(spl_engine *e, const spl_tables *t) {
    const int max_pages = e->host->max_pages;
    auto bad = [&](const char *what) { return e->fail(SPL_ERR_INVALID_ROWS, std::string("invalid step rows: ") + what); };
    if (t->rows == 0 || int(t->rows) > e->c.max_rows) return bad("row count outside the engine's limit");
    if (!t->tokens || !t->row_slot || !t->row_pos || !t->runs || !t->run_info || !t->row_read || !t->row_write || !t->attn_blocks || !t->page_table ||
        (t->logit_rows && !t->gather_index)) return bad("a table is missing");
    if (t->live_rows > t->rows || t->spans == 0 || t->spans > 64 || t->pages_per_span == 0 || t->run_count == 0 || t->run_count > t->rows ||
        t->attn_block_count == 0 || t->attn_block_count > t->rows) return bad("a count is out of range");
    for (uint32_t r = 0; r < t->rows; ++r) {
        if (int(t->tokens[r]) >= e->g.vocab || int(t->row_slot[r]) >= e->c.max_slots || int(t->row_pos[r]) >= e->c.max_context ||
            int(t->row_read[r]) >= e->c.state_units || int(t->row_write[r]) >= e->c.state_units) return bad("a row's token, slot, position or state unit is out of range");
        if (int(t->page_table[size_t(t->row_slot[r]) * max_pages + t->row_pos[r] / SPL_PAGE_TOKENS]) >= e->c.kv_pages) return bad("a page id is out of range");
    }
    uint32_t covered = 0;
    for (uint32_t r = 0; r < t->run_count; ++r) {
        if (int(t->runs[r * 3]) >= e->c.max_slots || t->runs[r * 3 + 1] != covered || t->runs[r * 3 + 2] == 0 || t->run_info[r * 2 + 1] > SPL_JOURNAL_ROWS ||
            (t->run_info[r * 2] && t->runs[r * 3 + 2] > SPL_JOURNAL_ROWS)) return bad("a run is out of range");
        covered += t->runs[r * 3 + 2];
    }
    if (covered != t->rows) return bad("the runs do not cover the rows");
    covered = 0;
    for (uint32_t b = 0; b < t->attn_block_count; ++b) {
        if (t->attn_blocks[b * 2] != covered || t->attn_blocks[b * 2 + 1] == 0 || t->attn_blocks[b * 2 + 1] > 8) return bad("an attention block is out of range");
        covered += t->attn_blocks[b * 2 + 1];
    }
    if (covered != t->rows) return bad("the attention blocks do not cover the rows");
    for (uint32_t i = 0; i < t->logit_rows; ++i) if (t->gather_index[i] >= t->rows) return bad("a logit row is out of range");
    // Every page a slot's rows can see has to be a valid id (the scan walks the table up to the last visible position).
    for (uint32_t b = 0; b < t->attn_block_count; ++b) {
        const uint32_t r0 = t->attn_blocks[b * 2], last = t->row_pos[r0] + t->attn_blocks[b * 2 + 1] - 1;
        if (int(last) >= e->c.max_context) return bad("an attention block runs past the context limit");
        for (uint32_t pg = 0; pg <= last / SPL_PAGE_TOKENS; ++pg)
            if (int(t->page_table[size_t(t->row_slot[r0]) * max_pages + pg]) >= e->c.kv_pages) return bad("a page id is out of range");
    }
    return SPL_OK;
}

spl_status spl_step_tables(spl_engine *e, const spl_tables *tables, spl_step_stats *stats) {
    if (!e || !tables) return SPL_ERR_INVALID_ARGUMENT;
    e->error.clear();
    SPL_NOT_IN_FLIGHT(e);
    const spl_status checked = check_tables(e, tables);
    if (checked != SPL_OK) return checked;
    return run_step(e, tables, stats);
}

spl_status spl_step(spl_engine *e, const spl_row *rows, int32_t count, spl_step_stats *stats) {
    if (!e || !rows) return SPL_ERR_INVALID_ARGUMENT;
    e->error.clear();
    spl_tables t;
    const spl_status built = spl_host_build_tables(e->host, rows, count, &t);
    if (built != SPL_OK) return e->fail(built, e->host->error);
    const spl_status ran = run_step(e, &t, stats);
    if (ran == SPL_OK) spl_host_finish_step(e->host, &t);
    return ran;
}

// The asynchronous pair (Engine.step split in two: the host may pack the next step's rows, or sample from the last
// step's logits on another engine, while this one runs). Between the two calls the engine accepts no other call that
// touches slots, logits or weights; spl_step_wait returns the step's status and statistics.
spl_status spl_step_launch(spl_engine *e, const spl_row *rows, int32_t count) {
    if (!e || !rows) return SPL_ERR_INVALID_ARGUMENT;
    if (e->in_flight) return e->fail(SPL_ERR_INVALID_ARGUMENT, "a step is in flight: call spl_step_wait first");
    e->error.clear();
    const spl_status built = spl_host_build_tables(e->host, rows, count, &e->flying);
    if (built != SPL_OK) return e->fail(built, e->host->error);
    const spl_status queued = enqueue_step(e, &e->flying);
    if (queued == SPL_OK) e->in_flight = true;
    return queued;
}

spl_status spl_step_wait(spl_engine *e, spl_step_stats *stats) {
    if (!e) return SPL_ERR_INVALID_ARGUMENT;
    if (!e->in_flight) return e->fail(SPL_ERR_INVALID_ARGUMENT, "no step is in flight");
    e->in_flight = false;
    const spl_status ran = finish_step(e, stats);
    if (ran == SPL_OK) spl_host_finish_step(e->host, &e->flying);
    return ran;
}

spl_status spl_logits_row(spl_engine *e, int32_t index, float *dst) {
    if (!e || !dst || index < 0 || index >= e->last_logit_rows) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    SPL_CUDA(cudaMemcpyAsync(dst, e->logits + size_t(index) * e->logits_ld, size_t(e->g.vocab) * 4, cudaMemcpyDeviceToHost, e->stream));
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    return SPL_OK;
}

spl_status spl_argmax(spl_engine *e, int32_t vocab_limit, int32_t *ids) {
    if (!e || !ids || vocab_limit <= 0 || vocab_limit > e->g.vocab) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    if (e->last_logit_rows == 0) return SPL_OK;
    SPL_CUDA(cudaSetDevice(e->device));
    spl_argmax_kernel<<<e->last_logit_rows, 1024, 0, e->stream>>>(e->logits, e->logits_ld, vocab_limit, e->argmax_ids);
    const spl_status launched = check_launch(e, "argmax");
    if (launched != SPL_OK) return launched;
    SPL_CUDA(cudaMemcpyAsync(ids, e->argmax_ids, size_t(e->last_logit_rows) * 4, cudaMemcpyDeviceToHost, e->stream));
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    return SPL_OK;
}

spl_status spl_topk(spl_engine *e, int32_t vocab_limit, int32_t k, int32_t *ids, float *values) {
    if (!e || !ids || !values || vocab_limit <= 0 || vocab_limit > e->g.vocab || k < 1 || k > 64 || k > vocab_limit) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    if (e->last_logit_rows == 0) return SPL_OK;
    SPL_CUDA(cudaSetDevice(e->device));
    const size_t cells = size_t(e->host->config.max_logit_rows) * 64;
    if (!e->topk_ids) {
        SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&e->topk_ids), cells * 4));
        SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&e->topk_values), cells * 4));
    }
    spl_topk_kernel<<<e->last_logit_rows, 1024, 0, e->stream>>>(e->logits, e->logits_ld, vocab_limit, k, e->topk_ids, e->topk_values);
    const spl_status launched = check_launch(e, "top-k");
    if (launched != SPL_OK) return launched;
    SPL_CUDA(cudaMemcpyAsync(ids, e->topk_ids, size_t(e->last_logit_rows) * k * 4, cudaMemcpyDeviceToHost, e->stream));
    SPL_CUDA(cudaMemcpyAsync(values, e->topk_values, size_t(e->last_logit_rows) * k * 4, cudaMemcpyDeviceToHost, e->stream));
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    return SPL_OK;
}

spl_status spl_slot_reset(spl_engine *e, int32_t slot) {
    if (!e || slot < 0 || slot >= e->c.max_slots) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    const int unit = spl_host_reset_slot(e->host, slot);
    for (size_t l = 0; l < e->state.size(); ++l) {
        SPL_CUDA(cudaMemsetAsync(reinterpret_cast<char *>(e->state[l]) + size_t(slot) * e->state_layer_bytes, 0, e->state_layer_bytes, e->stream));
        SPL_CUDA(cudaMemsetAsync(reinterpret_cast<char *>(e->conv[l]) + size_t(unit) * e->conv_unit_bytes, 0, e->conv_unit_bytes, e->stream));
    }
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    return SPL_OK;
}
spl_status spl_verify_discard(spl_engine *e, int32_t slot) {
    if (!e || slot < 0 || slot >= e->c.max_slots) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    spl_host_discard_verify(e->host, slot); return SPL_OK;
}
spl_status spl_verify_accept(spl_engine *e, int32_t slot, int32_t rows, int32_t token_count) {
    if (!e || slot < 0 || slot >= e->c.max_slots) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    const spl_status s = spl_host_accept_verify(e->host, slot, rows, token_count);
    if (s != SPL_OK) e->error = e->host->error;
    return s;
}
spl_status spl_slot_truncate(spl_engine *e, int32_t slot, int32_t token_count) {
    if (!e || slot < 0 || slot >= e->c.max_slots) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    spl_host_truncate(e->host, slot, token_count); return SPL_OK;
}
int32_t spl_pages_held(const spl_engine *e, int32_t slot) { return spl_host_pages_held(e->host, slot); }
int32_t spl_free_page_count(const spl_engine *e) { return spl_host_free_page_count(e->host); }
spl_host *spl_engine_host(spl_engine *e) { return e ? e->host : nullptr; }
// Engine.warmUp (Engine.swift:1191-1197): a full-width step and a one-row step on slot 0, which is left empty.
spl_status spl_warmup(spl_engine *e) {
    if (!e) return SPL_ERR_INVALID_ARGUMENT;
    if (e->in_flight) return e->fail(SPL_ERR_INVALID_ARGUMENT, "a step is in flight: call spl_step_wait first");
    const int width = std::min(e->c.max_rows, std::min(e->c.max_context - 1, e->c.kv_pages * SPL_PAGE_TOKENS - 1));
    if (width < 1) return SPL_OK;
    spl_status s = spl_slot_reset(e, 0);
    std::vector<spl_row> rows(width);
    for (int i = 0; i < width; ++i) { rows[i] = {}; rows[i].slot = 0; rows[i].token = 0; rows[i].position = i; rows[i].want_logits = i == width - 1; }
    if (s == SPL_OK) s = spl_step(e, rows.data(), width, nullptr);
    spl_row one = {}; one.slot = 0; one.token = 0; one.position = width; one.want_logits = 1;
    if (s == SPL_OK) s = spl_step(e, &one, 1, nullptr);
    const spl_status cleared = spl_slot_reset(e, 0);
    return s == SPL_OK ? cleared : s;
}

spl_status spl_memory(const spl_engine *ce, spl_memory_info *out) {
    spl_engine *e = const_cast<spl_engine *>(ce);
    if (!e || !out) return SPL_ERR_INVALID_ARGUMENT;
    const int linear = int(e->state.size());
    out->weight_bytes = int64_t(e->weight_bytes); out->kv_pool_bytes = int64_t(e->kv_pool_bytes);
    out->kv_bytes_per_page = int64_t(e->kv_page_bytes * e->k_codes.size());
    out->kv_pages_total = e->c.kv_pages; out->kv_pages_used = e->c.kv_pages - spl_host_free_page_count(e->host);
    out->state_bytes_per_slot = int64_t((e->state_layer_bytes + e->conv_unit_bytes) * linear);
    out->state_units_used = e->c.state_units - int64_t(e->host->free_units.size());
    out->state_bytes_total = int64_t(e->state_layer_bytes) * linear * e->c.max_slots + int64_t(e->conv_unit_bytes) * linear * out->state_units_used;
    out->scratch_bytes = int64_t(e->scratch_bytes);
    size_t free_b = 0, total_b = 0;
    SPL_CUDA(cudaSetDevice(e->device));
    SPL_CUDA(cudaMemGetInfo(&free_b, &total_b));
    out->device_total_bytes = int64_t(total_b); out->device_free_bytes = int64_t(free_b);
    return SPL_OK;
}

spl_status spl_debug_fill_kv(spl_engine *e, int32_t slot) {
    if (!e || slot < 0 || slot >= e->c.max_slots) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    const size_t page_vecs = size_t(e->g.kv_heads) * SPL_PAGE_TOKENS, page_codes = page_vecs * e->g.head_dim;
    for (size_t l = 0; l < e->k_codes.size(); ++l)
        for (uint32_t page : e->host->slot_pages[slot]) {
            const uint64_t seed = 0x9E3779B97F4A7C15ull ^ (uint64_t(l) << 32) ^ page;
            spl_fill_codes_kernel<<<64, 256, 0, e->stream>>>(reinterpret_cast<uint64_t *>(e->k_codes[l] + page * page_codes), page_codes / 8, seed);
            spl_fill_codes_kernel<<<64, 256, 0, e->stream>>>(reinterpret_cast<uint64_t *>(e->v_codes[l] + page * page_codes), page_codes / 8, seed + 1);
            spl_fill_float_kernel<<<4, 256, 0, e->stream>>>(e->k_scale[l] + page * page_vecs, page_vecs, 0.01f);
            spl_fill_float_kernel<<<4, 256, 0, e->stream>>>(e->v_scale[l] + page * page_vecs, page_vecs, 0.01f);
        }
    const spl_status launched = check_launch(e, "fill kv");
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    return launched;
}

spl_status spl_debug_fill_state(spl_engine *e, int32_t slot, uint64_t seed) {
    if (!e || slot < 0 || slot >= e->c.max_slots) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    const size_t count = e->state_layer_bytes / 4;
    for (size_t l = 0; l < e->state.size(); ++l)
        spl_fill_uniform_kernel<<<256, 256, 0, e->stream>>>(e->state[l] + size_t(slot) * count, count, seed + l * 1315423911ull + uint64_t(slot), -0.5f, 0.5f);
    const spl_status launched = check_launch(e, "fill state");
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    return launched;
}

spl_status spl_debug_taps(spl_engine *e, int32_t enabled) {
    if (!e) return SPL_ERR_INVALID_ARGUMENT;
    SPL_CUDA(cudaSetDevice(e->device));
    if (enabled && !e->taps) SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&e->taps), size_t(e->g.layers) * e->c.max_rows * e->g.hidden * 4));
    e->taps_enabled = enabled != 0;
    return SPL_OK;
}

spl_status spl_debug_wait_budget(spl_engine *e, int64_t nanoseconds) {
    if (!e || nanoseconds <= 0) return SPL_ERR_INVALID_ARGUMENT;
    SPL_CUDA(cudaSetDevice(e->device));
    const unsigned long long value = static_cast<unsigned long long>(nanoseconds);
    SPL_CUDA(cudaMemcpyToSymbol(spl_wait_budget_ns, &value, sizeof value));
    return SPL_OK;
}

spl_status spl_debug_drop_weight_stage(spl_engine *e, int32_t stage) {
    if (!e) return SPL_ERR_INVALID_ARGUMENT;
    g_drop_weight_stage = stage;
    return SPL_OK;
}

spl_status spl_debug_pair_blocks(spl_engine *, int32_t enabled) {
    g_pair_blocks = enabled ? 1 : 0;
    return SPL_OK;
}

spl_status spl_debug_gdn_chunk_min(spl_engine *e, int32_t rows) {
    if (!e || rows < SPL_GDN_CHUNK) return SPL_ERR_INVALID_ARGUMENT;
    e->gdn_chunk_min = rows;
    return SPL_OK;
}

spl_status spl_debug_kv_store(spl_engine *e, int32_t enabled) {
    if (!e) return SPL_ERR_INVALID_ARGUMENT;
    e->kv_store = enabled != 0;
    return SPL_OK;
}

spl_status spl_features_enable(spl_engine *e, const int32_t *layers, int32_t count) {
    if (!e || count < 0 || count > 16) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    static const int32_t reference_layers[5] = {5, 19, 33, 47, 61};
    if (count > 0 && !layers) { layers = reference_layers; count = 5; }
    std::vector<int> wanted;
    for (int i = 0; i < count; ++i) {
        if (layers[i] < 0) return e->fail(SPL_ERR_INVALID_ARGUMENT, "feature layer below zero");
        if (layers[i] < e->g.layers) wanted.push_back(layers[i]);      // taps of blocks this geometry does not have are left out
    }
    SPL_CUDA(cudaSetDevice(e->device));
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    if (e->features) { cudaFree(e->features); e->features = nullptr; }
    e->feature_layers = wanted;
    if (!wanted.empty()) {
        const size_t bytes = size_t(e->c.max_rows) * wanted.size() * e->g.hidden * 4;
        SPL_CUDA(cudaMalloc(reinterpret_cast<void **>(&e->features), bytes));
        SPL_CUDA(cudaMemsetAsync(e->features, 0, bytes, e->stream));
    }
    return SPL_OK;
}

int32_t spl_feature_width(const spl_engine *e) { return e ? int32_t(e->feature_layers.size()) * e->g.hidden : 0; }

spl_status spl_feature_row(spl_engine *e, int32_t row, float *dst) {
    if (!e || !dst) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    if (!e->features) return e->fail(SPL_ERR_INVALID_ARGUMENT, "feature taps are not enabled");
    if (row < 0 || row >= e->last_rows) return e->fail(SPL_ERR_INVALID_ROWS, "invalid step rows: no such row in the last step");
    SPL_CUDA(cudaSetDevice(e->device));
    const size_t width = e->feature_layers.size() * size_t(e->g.hidden);
    SPL_CUDA(cudaMemcpy(dst, e->features + size_t(row) * width, width * 4, cudaMemcpyDeviceToHost));
    return SPL_OK;
}

spl_status spl_debug_profile(spl_engine *e, int32_t enabled) {
    if (!e) return SPL_ERR_INVALID_ARGUMENT;
    e->profile = enabled != 0;
    for (int k = 0; k < KLASS_COUNT; ++k) { e->klass_ms[k] = 0; e->klass_bytes[k] = 0; e->klass_launches[k] = 0; }
    return SPL_OK;
}
spl_status spl_debug_profile_read(spl_engine *e, int32_t klass, double *milliseconds, int64_t *launches, double *bytes) {
    if (!e || klass < 0 || klass >= KLASS_COUNT) return SPL_ERR_INVALID_ARGUMENT;
    if (milliseconds) *milliseconds = e->klass_ms[klass];
    if (launches) *launches = e->klass_launches[klass];
    if (bytes) *bytes = e->klass_bytes[klass];
    return SPL_OK;
}

spl_status spl_debug_read(spl_engine *e, int32_t which, int32_t index, void *dst, size_t bytes) {
    if (!e || !dst) return SPL_ERR_INVALID_ARGUMENT;
    SPL_CUDA(cudaSetDevice(e->device));
    const void *src = nullptr; size_t have = 0;
    const size_t page_vecs = size_t(e->g.kv_heads) * SPL_PAGE_TOKENS, codes = size_t(e->c.kv_pages) * page_vecs * e->g.head_dim;
    auto pick = [&](const std::vector<float *> &v, size_t n) { if (index >= 0 && index < int(v.size())) { src = v[index]; have = n; } };
    switch (which) {
    case 0: pick(e->state, size_t(e->c.max_slots) * e->state_layer_bytes); break;
    case 1: pick(e->conv, size_t(e->c.state_units) * e->conv_unit_bytes); break;
    case 2: pick(e->journal, e->journal_bytes); break;
    case 3: if (index >= 0 && index < int(e->k_codes.size())) { src = e->k_codes[index]; have = codes; } break;
    case 4: if (index >= 0 && index < int(e->v_codes.size())) { src = e->v_codes[index]; have = codes; } break;
    case 5: pick(e->k_scale, size_t(e->c.kv_pages) * page_vecs * 4); break;
    case 6: pick(e->v_scale, size_t(e->c.kv_pages) * page_vecs * 4); break;
    case 7: src = e->h; have = size_t(e->last_rows) * e->g.hidden * 4; break;
    case 9: src = e->proj; have = size_t(e->last_rows) * e->proj_ld * 4; break;
    case 10: src = e->core; have = size_t(e->rows_padded) * e->core_ld * 2; break;
    case 11: src = e->q; have = size_t(e->last_rows) * e->g.heads * e->g.head_dim * 2; break;
    case 12: src = e->attn_partials; have = e->attn_partial_floats * 4; break;
    case 13: src = e->tc_error; have = 64 * sizeof(int); break;
    case 8: if (e->taps && index >= 0 && index < e->g.layers) { src = e->taps + size_t(index) * e->c.max_rows * e->g.hidden; have = size_t(e->last_rows) * e->g.hidden * 4; } break;
    }
    if (!src || bytes > have) return e->fail(SPL_ERR_INVALID_ARGUMENT, "debug read outside the buffer");
    if (which == 3 || which == 4) {
        // The code arrays are read out as signed codes in the plain order [page][kv head][token][channel], whatever the pool's own order and byte form are.
        const int hd = e->g.head_dim;
        std::vector<int8_t> raw(have);
        SPL_CUDA(cudaMemcpy(raw.data(), src, have, cudaMemcpyDeviceToHost));
        int8_t *out = static_cast<int8_t *>(dst);
        for (size_t i = 0; i < bytes; ++i) {
            const size_t vec = i / (size_t(SPL_PAGE_TOKENS) * hd), rest = i % (size_t(SPL_PAGE_TOKENS) * hd);
            const uint32_t token = uint32_t(rest / hd); const int d = int(rest % hd);
            out[i] = spl_code_value(raw[which == 3 ? spl_k_code_index(vec, token, d, hd) : spl_v_code_index(vec, token, d, hd)]);
        }
        return SPL_OK;
    }
    SPL_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
    return SPL_OK;
}

}  // extern "C"

// ---- slot snapshots (Engine.swift:870-1042) -----------------------------------------------------
// Two opaque, versioned blobs. State: the slot's recurrent state of every gated-delta block with the journal folded
// in, and the conv history of its current unit. KV: the pages that cover the slot's first `token_count` tokens,
// every attention block, in the pool's own byte order. A blob is valid for engines of the same geometry only.
namespace {
struct SnapshotHeader { uint32_t magic, version; uint64_t identity; uint32_t blocks, tokens; uint64_t payload; };
constexpr uint32_t kStateMagic = 0x53504C53u, kKvMagic = 0x4B504C53u, kSnapshotVersion = 2u;      // "SLPS", "SLPK"

uint64_t snapshot_identity(const spl_engine *e) {
    const spl_geometry &g = e->g;
    const int fields[] = {g.layers, g.hidden, g.heads, g.kv_heads, g.head_dim, g.rotary_dim, g.gdn_key_heads, g.gdn_value_heads, g.gdn_head_dim, SPL_PAGE_TOKENS};
    uint64_t h = 1469598103934665603ull;
    for (int f : fields) for (int b = 0; b < 4; ++b) { h ^= uint64_t((f >> (8 * b)) & 0xFF); h *= 1099511628211ull; }
    return h;
}
size_t state_payload(const spl_engine *e) { return e->state.size() * (e->state_layer_bytes + e->conv_unit_bytes); }
size_t kv_page_payload(const spl_engine *e) {       // one page of one attention block: K codes, V codes, K scales, V scales
    const size_t vecs = size_t(e->g.kv_heads) * SPL_PAGE_TOKENS;
    return 2 * vecs * e->g.head_dim + 2 * vecs * 4;
}
// Engine.commitJournal (Engine.swift:889-903): fold the slot's accepted journal entries into its stored state. The
// recurrence kernel does it when given a run of no rows.
spl_status commit_journal(spl_engine *e, int slot) {
    const uint32_t pending = e->host->journal_pending[slot];
    if (pending == 0) return SPL_OK;
    const uint32_t table[5] = {uint32_t(slot), 0u, 0u, /* run_info: */ 0u, pending};
    memcpy(e->tables_host, table, sizeof table);
    SPL_CUDA(cudaMemcpyAsync(e->tables_dev, e->tables_host, sizeof table, cudaMemcpyHostToDevice, e->stream));
    const Shapes sh(e->g);
    SplGdnParams p;
    p.rows = 0; p.runs = 1; p.channels = sh.C; p.key_heads = e->g.gdn_key_heads; p.value_heads = e->g.gdn_value_heads; p.head_dim = e->g.gdn_head_dim;
    p.proj_ld = e->proj_ld; p.z_offset = sh.gdn_z; p.a_offset = sh.gdn_a; p.b_offset = sh.gdn_b; p.eps = e->g.eps; p.chunk_min = 0;
    const int rn = 16;
    const SplOperand core{e->core, e->core_sums, rn, 1};
    int linear = 0;
    for (size_t l = 0; l < e->layers.size(); ++l) {
        if (e->layers[l].full) continue;
        spl_gdn_recurrence_kernel<<<dim3(e->g.gdn_value_heads, 1), SPL_GDN_THREADS, spl_gdn_recurrence_smem(), e->stream>>>(
            e->gdn_act, e->proj, e->layers[l].vec[SPL_VEC_A_LOG], e->layers[l].vec[SPL_VEC_DT_BIAS], e->layers[l].vec[SPL_VEC_GDN_NORM],
            e->state[linear], e->journal[linear], e->tables_dev, e->tables_dev + 3, core, p);
        ++linear;
    }
    const spl_status launched = check_launch(e, "journal commit");
    if (launched != SPL_OK) return launched;
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    e->host->journal_pending[slot] = 0;
    return SPL_OK;
}
}  // namespace

extern "C" {

size_t spl_state_bytes(const spl_engine *e) { return e ? sizeof(SnapshotHeader) + state_payload(e) : 0; }

spl_status spl_state_export(spl_engine *e, int32_t slot, void *dst, size_t capacity) {
    if (!e || !dst || slot < 0 || slot >= e->c.max_slots) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    if (capacity < spl_state_bytes(e)) return e->fail(SPL_ERR_INVALID_ARGUMENT, "state export: the buffer is smaller than spl_state_bytes");
    SPL_CUDA(cudaSetDevice(e->device));
    const spl_status committed = commit_journal(e, slot);
    if (committed != SPL_OK) return committed;
    SnapshotHeader header = {kStateMagic, kSnapshotVersion, snapshot_identity(e), uint32_t(e->state.size()), 0u, uint64_t(state_payload(e))};
    memcpy(dst, &header, sizeof header);
    unsigned char *out = static_cast<unsigned char *>(dst) + sizeof header;
    const uint32_t unit = e->host->slot_unit[slot];
    for (size_t l = 0; l < e->state.size(); ++l) {
        SPL_CUDA(cudaMemcpyAsync(out, reinterpret_cast<const char *>(e->state[l]) + size_t(slot) * e->state_layer_bytes, e->state_layer_bytes, cudaMemcpyDeviceToHost, e->stream));
        out += e->state_layer_bytes;
        SPL_CUDA(cudaMemcpyAsync(out, reinterpret_cast<const char *>(e->conv[l]) + size_t(unit) * e->conv_unit_bytes, e->conv_unit_bytes, cudaMemcpyDeviceToHost, e->stream));
        out += e->conv_unit_bytes;
    }
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    return SPL_OK;
}

spl_status spl_state_import(spl_engine *e, int32_t slot, const void *src, size_t bytes) {
    if (!e || !src || slot < 0 || slot >= e->c.max_slots) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SnapshotHeader header;
    if (bytes < sizeof header) return e->fail(SPL_ERR_SNAPSHOT_MISMATCH, "snapshot mismatch: truncated state blob");
    memcpy(&header, src, sizeof header);
    if (header.magic != kStateMagic || header.version != kSnapshotVersion || header.identity != snapshot_identity(e) ||
        header.payload != state_payload(e) || bytes < sizeof header + header.payload)
        return e->fail(SPL_ERR_SNAPSHOT_MISMATCH, "snapshot mismatch: the state blob is not one of this engine's geometry and layout");
    SPL_CUDA(cudaSetDevice(e->device));
    spl_host_discard_verify(e->host, slot);
    e->host->journal_pending[slot] = 0;
    const unsigned char *in = static_cast<const unsigned char *>(src) + sizeof header;
    const uint32_t unit = e->host->slot_unit[slot];
    for (size_t l = 0; l < e->state.size(); ++l) {
        SPL_CUDA(cudaMemcpyAsync(reinterpret_cast<char *>(e->state[l]) + size_t(slot) * e->state_layer_bytes, in, e->state_layer_bytes, cudaMemcpyHostToDevice, e->stream));
        in += e->state_layer_bytes;
        SPL_CUDA(cudaMemcpyAsync(reinterpret_cast<char *>(e->conv[l]) + size_t(unit) * e->conv_unit_bytes, in, e->conv_unit_bytes, cudaMemcpyHostToDevice, e->stream));
        in += e->conv_unit_bytes;
    }
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    return SPL_OK;
}

size_t spl_kv_bytes(const spl_engine *e, int32_t token_count) {
    if (!e || token_count < 0) return 0;
    const size_t pages = size_t(token_count + SPL_PAGE_TOKENS - 1) / SPL_PAGE_TOKENS;
    return sizeof(SnapshotHeader) + pages * e->k_codes.size() * kv_page_payload(e);
}

spl_status spl_kv_export(spl_engine *e, int32_t slot, int32_t token_count, void *dst, size_t capacity) {
    if (!e || !dst || slot < 0 || slot >= e->c.max_slots || token_count < 0) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    const size_t pages = size_t(token_count + SPL_PAGE_TOKENS - 1) / SPL_PAGE_TOKENS;
    if (pages > e->host->slot_pages[slot].size()) return e->fail(SPL_ERR_INVALID_ARGUMENT, "kv export: the slot holds fewer tokens than asked for");
    if (capacity < spl_kv_bytes(e, token_count)) return e->fail(SPL_ERR_INVALID_ARGUMENT, "kv export: the buffer is smaller than spl_kv_bytes");
    SPL_CUDA(cudaSetDevice(e->device));
    SnapshotHeader header = {kKvMagic, kSnapshotVersion, snapshot_identity(e), uint32_t(e->k_codes.size()), uint32_t(token_count),
                             uint64_t(pages * e->k_codes.size() * kv_page_payload(e))};
    memcpy(dst, &header, sizeof header);
    unsigned char *out = static_cast<unsigned char *>(dst) + sizeof header;
    const size_t vecs = size_t(e->g.kv_heads) * SPL_PAGE_TOKENS, codes = vecs * e->g.head_dim;
    for (size_t l = 0; l < e->k_codes.size(); ++l)
        for (size_t pg = 0; pg < pages; ++pg) {
            const size_t page = e->host->slot_pages[slot][pg];
            SPL_CUDA(cudaMemcpyAsync(out, e->k_codes[l] + page * codes, codes, cudaMemcpyDeviceToHost, e->stream)); out += codes;
            SPL_CUDA(cudaMemcpyAsync(out, e->v_codes[l] + page * codes, codes, cudaMemcpyDeviceToHost, e->stream)); out += codes;
            SPL_CUDA(cudaMemcpyAsync(out, e->k_scale[l] + page * vecs, vecs * 4, cudaMemcpyDeviceToHost, e->stream)); out += vecs * 4;
            SPL_CUDA(cudaMemcpyAsync(out, e->v_scale[l] + page * vecs, vecs * 4, cudaMemcpyDeviceToHost, e->stream)); out += vecs * 4;
        }
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    return SPL_OK;
}

spl_status spl_kv_import(spl_engine *e, int32_t slot, int32_t token_count, const void *src, size_t bytes) {
    if (!e || !src || slot < 0 || slot >= e->c.max_slots || token_count < 0) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SnapshotHeader header;
    if (bytes < sizeof header) return e->fail(SPL_ERR_SNAPSHOT_MISMATCH, "snapshot mismatch: truncated KV blob");
    memcpy(&header, src, sizeof header);
    const size_t pages = size_t(token_count + SPL_PAGE_TOKENS - 1) / SPL_PAGE_TOKENS;
    const size_t stored_pages = size_t(header.tokens + SPL_PAGE_TOKENS - 1) / SPL_PAGE_TOKENS;
    if (header.magic != kKvMagic || header.version != kSnapshotVersion || header.identity != snapshot_identity(e) || header.blocks != e->k_codes.size() ||
        uint32_t(token_count) > header.tokens || header.payload != stored_pages * e->k_codes.size() * kv_page_payload(e) || bytes < sizeof header + header.payload)
        return e->fail(SPL_ERR_SNAPSHOT_MISMATCH, "snapshot mismatch: the KV blob is not one of this engine's geometry and layout, or holds fewer tokens");
    SPL_CUDA(cudaSetDevice(e->device));
    // The slot keeps exactly the pages of the imported prefix (Engine.kvPrefix, Engine.swift:974-991: a prefix of a stored KV is valid as it is).
    spl_host_truncate(e->host, slot, 0);
    if (token_count > 0) {
        const spl_status paged = e->host->ensure_page(slot, token_count - 1);
        if (paged != SPL_OK) return e->fail(paged, e->host->error);
    }
    const unsigned char *in = static_cast<const unsigned char *>(src) + sizeof header;
    const size_t vecs = size_t(e->g.kv_heads) * SPL_PAGE_TOKENS, codes = vecs * e->g.head_dim;
    for (size_t l = 0; l < e->k_codes.size(); ++l)
        for (size_t pg = 0; pg < stored_pages; ++pg) {
            if (pg < pages) {
                const size_t page = e->host->slot_pages[slot][pg];
                SPL_CUDA(cudaMemcpyAsync(e->k_codes[l] + page * codes, in, codes, cudaMemcpyHostToDevice, e->stream));
                SPL_CUDA(cudaMemcpyAsync(e->v_codes[l] + page * codes, in + codes, codes, cudaMemcpyHostToDevice, e->stream));
                SPL_CUDA(cudaMemcpyAsync(e->k_scale[l] + page * vecs, in + 2 * codes, vecs * 4, cudaMemcpyHostToDevice, e->stream));
                SPL_CUDA(cudaMemcpyAsync(e->v_scale[l] + page * vecs, in + 2 * codes + vecs * 4, vecs * 4, cudaMemcpyHostToDevice, e->stream));
            }
            in += kv_page_payload(e);
        }
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    return SPL_OK;
}

}  // extern "C"

// ---- A GEMM that allocates nothing ---------------------------------------------------------
//
// For callers that may not allocate device memory: a host that handed the whole GPU to its own
// pool at start-up, or a serving loop that bans allocator calls on its hot path because
// cudaMalloc and cudaFree synchronise the whole device. The scratch the ordinary path takes from the engine's buffers (the bf16 operand with its
// per-64 sums, and the slots where the blocks of a cut tile leave their partial sums) lives here in
// one file-scope device array, so every GPU that loads the library holds SPL_STATIC_BYTES (about 12.3 MiB) until the
// process exits.
#define SPL_STATIC_ROWS 64
#define SPL_STATIC_INNER 17408
#define SPL_STATIC_OPERAND_BYTES (SPL_STATIC_ROWS * SPL_STATIC_INNER * 2)
#define SPL_STATIC_SUMS_BYTES (SPL_STATIC_ROWS * ((SPL_STATIC_INNER / 64 + 15) / 16) * 128)      // tiles of split means
#define SPL_STATIC_CONTROL_BYTES 256       // the error words
#define SPL_STATIC_SLOTS 320               // room for partial sums, in units of 64 x 128 floats: splits x 64 rows x the tensor's columns must fit (else the call is refused)
#define SPL_STATIC_SLOT_BYTES (SPL_STATIC_SLOTS * 64 * 128 * 4)
#define SPL_STATIC_BYTES (SPL_STATIC_OPERAND_BYTES + SPL_STATIC_SUMS_BYTES + SPL_STATIC_CONTROL_BYTES + SPL_STATIC_SLOT_BYTES)
static __device__ __align__(256) unsigned char spl_static_scratch[SPL_STATIC_BYTES];
// The array's address on each device, asked for once per device. The symbol itself is only a
// host-side handle: a kernel must be given what cudaGetSymbolAddress returns.
static void *spl_static_address[64] = {};

// fp32 rows -> the bf16 GEMM operand and its per-64 sums (Sources/Shaders/engine_na.metal:42-57;
// layout: SplOperand). Groups past the contraction in the last tile of split means are written as zero, so nothing an
// earlier call left there is ever multiplied. Grid (rows), 256 threads.
__global__ void __launch_bounds__(256)
spl_operand_kernel(const float *__restrict__ input, SplOperand out, int inner) {
    // A pass queues this kernel behind the one that wrote `input`, and behind the GEMM that still reads the operand this
    // one overwrites: it may not run ahead of either.
    spl_grid_begin();
    const int row = blockIdx.x;
    for (int base = 0; base < inner; base += 1024) {
        const int i = base + threadIdx.x * 4;
        float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;
        if (i < inner) {
            const float4 v = *reinterpret_cast<const float4 *>(input + size_t(row) * inner + i);
            const uint16_t b0 = spl_float_to_bf16(v.x), b1 = spl_float_to_bf16(v.y), b2 = spl_float_to_bf16(v.z), b3 = spl_float_to_bf16(v.w);
            r0 = spl_bf16_to_float(b0); r1 = spl_bf16_to_float(b1); r2 = spl_bf16_to_float(b2); r3 = spl_bf16_to_float(b3);
            *reinterpret_cast<uint2 *>(out.values + out.at(row, i)) = spl_operand_pack4(r0, r1, r2, r3);
        }
        float gsum = (r0 + r1) + (r2 + r3);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) gsum += __shfl_xor_sync(0xffffffffu, gsum, o);
        if (i < inner && (threadIdx.x & 15) == 0) out.put_sum(row, i / 64, gsum);
    }
    const int groups = inner / 64;
    for (int g = groups + int(threadIdx.x); g < (groups + 15) / 16 * 16; g += blockDim.x) out.put_sum(row, g, 0.0f);
}

static spl_status static_base(spl_engine *e, unsigned char **base) {
    SPL_CUDA(cudaSetDevice(e->device));
    if (e->device >= 64) return e->fail(SPL_ERR_UNSUPPORTED_DEVICE, "spl_gemm_q4_static: device ordinal beyond 63");
    if (!spl_static_address[e->device]) {
        // First call on this device: resolve the array's device address (this device is current).
        void *address = nullptr;
        SPL_CUDA(cudaGetSymbolAddress(&address, spl_static_scratch));
        spl_static_address[e->device] = address;
    }
    *base = static_cast<unsigned char *>(spl_static_address[e->device]);
    return SPL_OK;
}

extern "C" spl_status spl_gemm_q4_static(spl_engine *e, int32_t layer, int32_t which, const float *device_activations, int32_t rows,
                                         const float *device_residual, float *device_out, void *stream_handle) {
    if (!e || !device_activations || !device_out) return SPL_ERR_INVALID_ARGUMENT;
    const SplQ4Dev *w = nullptr;
    if (layer < 0) { if (which == SPL_RESIDENT_HEAD) w = &e->head; }
    else if (layer < e->g.layers) {
        const LayerWeights &L = e->layers[layer];
        w = which == SPL_RESIDENT_IN_PROJ ? &L.in_proj : which == SPL_RESIDENT_OUT_PROJ ? &L.out_proj : which == SPL_RESIDENT_GATE_UP ? &L.gate_up
          : which == SPL_RESIDENT_DOWN ? &L.down : nullptr;
    }
    if (!w || !w->codes) return e->fail(SPL_ERR_INVALID_ARGUMENT, "no such resident tensor");
    if (rows < 1 || rows > SPL_STATIC_ROWS)
        return e->fail(SPL_ERR_INVALID_ROWS, "spl_gemm_q4_static: rows must be 1..64 (the static scratch holds a 64-row operand)");
    if (w->k > SPL_STATIC_INNER)
        return e->fail(SPL_ERR_INVALID_ARGUMENT, "spl_gemm_q4_static: contraction longer than 17408 does not fit the static scratch");
    unsigned char *base = nullptr;
    const spl_status found = static_base(e, &base);
    if (found != SPL_OK) return found;
    __nv_bfloat16 *operand = reinterpret_cast<__nv_bfloat16 *>(base);
    float *sums = reinterpret_cast<float *>(base + SPL_STATIC_OPERAND_BYTES);
    int *control = reinterpret_cast<int *>(base + SPL_STATIC_OPERAND_BYTES + SPL_STATIC_SUMS_BYTES);
    float *slots = reinterpret_cast<float *>(base + SPL_STATIC_OPERAND_BYTES + SPL_STATIC_SUMS_BYTES + SPL_STATIC_CONTROL_BYTES);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
    const int rn = operand_rn(rows);
    // The array keeps what the last call left. The error words have to start at zero; the
    // operand and sums of the rows in use are rewritten here, the block's other rows feed outputs
    // that are never stored, and every slot the second kernel reads is written by this call.
    SPL_CUDA(cudaMemsetAsync(control, 0, SPL_STATIC_CONTROL_BYTES, stream));
    spl_operand_kernel<<<rows, 256, 0, stream>>>(device_activations, SplOperand{operand, sums, rn, 1}, w->k);
    const GemmScratch scratch{slots, SPL_STATIC_SLOT_BYTES / 4, control, e->sms};
    if (!launch_gemm_rows(stream, *w, GemmOperand{operand, sums, rn, 1}, device_out, device_residual, rows, scratch, GemmExtras(), nullptr))
        return e->fail(SPL_ERR_INVALID_ARGUMENT, "spl_gemm_q4_static: the tensor does not fit the static scratch");
    return check_launch(e, "spl_gemm_q4_static");
}

// Whether a block of the last spl_gemm_q4_static calls on this engine's device gave up a wait (its output is then
// incomplete). Call it after the stream those calls were queued on has been synchronised; it allocates nothing.
extern "C" spl_status spl_gemm_q4_static_status(spl_engine *e) {
    if (!e) return SPL_ERR_INVALID_ARGUMENT;
    unsigned char *base = nullptr;
    const spl_status found = static_base(e, &base);
    if (found != SPL_OK) return found;
    int flag = 0;
    SPL_CUDA(cudaMemcpy(&flag, base + SPL_STATIC_OPERAND_BYTES + SPL_STATIC_SUMS_BYTES, sizeof flag, cudaMemcpyDeviceToHost));
    if (flag) return e->fail(SPL_ERR_TIMEOUT, "spl_gemm_q4_static: a GEMM block gave up waiting (warp " + std::to_string(flag - 1) + "); the output is incomplete");
    return SPL_OK;
}

extern "C" {

// One GEMM on host buffers: the whole path a caller without an engine sees.
spl_status spl_op_gemm_q4(int32_t device, const uint32_t *packed, const uint16_t *scales, const uint16_t *biases,
                          int32_t n, int32_t k, const float *activations, int32_t rows, const float *residual, float *out) {
    if (!packed || !scales || !biases || !activations || !out || n <= 0 || k <= 0 || k % 256 || rows <= 0) return SPL_ERR_INVALID_ARGUMENT;   // inner dimensions are multiples of 256 in every geometry this library accepts
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return SPL_ERR_UNSUPPORTED_DEVICE;
    spl_engine local;                     // only stream, scratch and error text are used
    spl_engine *e = &local;
    e->device = device;
    SPL_CUDA(cudaSetDevice(device));
    if (!configure_device(device, &e->sms)) return SPL_ERR_UNSUPPORTED_DEVICE;
    SPL_CUDA(cudaStreamCreate(&e->stream));
    SplQ4Dev w;
    spl_status s = alloc_q4(e, w, n, k);
    const int ld = w.ld;
    const int rn = operand_rn(rows), blocks = (rows + rn - 1) / rn;
    float *d_act32 = nullptr, *d_out = nullptr, *d_sums = nullptr; __nv_bfloat16 *d_act = nullptr; int *d_flag = nullptr;
    e->slot_floats = gemm_slot_floats(w, e->sms, rn, blocks, false, false);
    if (s == SPL_OK) s = device_alloc(e, &d_act32, size_t(rows) * k);
    if (s == SPL_OK) s = device_alloc(e, &d_act, size_t(blocks) * rn * k);
    if (s == SPL_OK) s = device_alloc(e, &d_sums, spl_operand_sums_floats(size_t(blocks) * rn, k));
    if (s == SPL_OK) s = device_alloc(e, &d_out, size_t(rows) * ld);
    if (s == SPL_OK) s = device_alloc(e, &d_flag, 64);
    if (s == SPL_OK) s = device_alloc(e, &e->slots, e->slot_floats);
    if (s == SPL_OK) s = upload_q4_into(e, w, 0, n, k, packed, scales, biases, false);
    if (s == SPL_OK) {
        cudaMemsetAsync(d_act, 0, size_t(blocks) * rn * k * 2, e->stream);
        cudaMemsetAsync(d_sums, 0, spl_operand_sums_floats(size_t(blocks) * rn, k) * 4, e->stream);
        cudaMemsetAsync(d_flag, 0, 64 * sizeof(int), e->stream);
        cudaMemcpyAsync(d_act32, activations, size_t(rows) * k * 4, cudaMemcpyHostToDevice, e->stream);
        spl_operand_kernel<<<rows, 256, 0, e->stream>>>(d_act32, SplOperand{d_act, d_sums, rn, blocks}, k);
        if (residual) cudaMemcpy2DAsync(d_out, size_t(ld) * 4, residual, size_t(n) * 4, size_t(n) * 4, rows, cudaMemcpyHostToDevice, e->stream);
        const GemmScratch scratch{e->slots, e->slot_floats, d_flag, e->sms};
        if (!launch_gemm_rows(e->stream, w, GemmOperand{d_act, d_sums, rn, blocks}, d_out, residual ? d_out : nullptr, rows, scratch, GemmExtras(), nullptr)) s = SPL_ERR_INVALID_ARGUMENT;
        if (s == SPL_OK) s = check_launch(e, "gemm");
        if (cudaStreamSynchronize(e->stream) != cudaSuccess) s = SPL_ERR_DEVICE;
        int flag = 0;
        if (s == SPL_OK) { cudaMemcpy(&flag, d_flag, sizeof flag, cudaMemcpyDeviceToHost); if (flag) s = SPL_ERR_TIMEOUT; }
        if (s == SPL_OK) cudaMemcpy2D(out, size_t(n) * 4, d_out, size_t(ld) * 4, size_t(n) * 4, rows, cudaMemcpyDeviceToHost);
    }
    cudaFree(d_sums); cudaFree(d_flag);
    cudaFree(w.codes); cudaFree(w.sb); cudaFree(d_act32); cudaFree(d_act); cudaFree(d_out); cudaFree(e->gdn_records); cudaFree(e->gdn_o_raw); cudaFree(e->slots);
    cudaStreamDestroy(e->stream);
    e->stream = nullptr; e->slots = nullptr;
    return s;
}

// Engine.gemm's GGUF branch for one K-quant tensor on host buffers (tests, micro-benchmarks): native super-blocks
// [n][k / 256][block bytes] of GGUF type `format` (12 Q4_K, 13 Q5_K, 14 Q6_K).
spl_status spl_op_gemm_gguf(int32_t device, int32_t format, const uint8_t *blocks, int32_t n, int32_t k, const float *activations, int32_t rows,
                            const float *residual, float *out) {
    if (!blocks || !activations || !out || n <= 0 || k <= 0 || k % 256 || rows <= 0 ||
        (format != SPL_GGUF_Q4K && format != SPL_GGUF_Q5K && format != SPL_GGUF_Q6K)) return SPL_ERR_INVALID_ARGUMENT;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return SPL_ERR_UNSUPPORTED_DEVICE;
    spl_engine local;
    spl_engine *e = &local;
    e->device = device;
    SPL_CUDA(cudaSetDevice(device));
    if (!configure_device(device, &e->sms)) return SPL_ERR_UNSUPPORTED_DEVICE;
    SPL_CUDA(cudaStreamCreate(&e->stream));
    SplGgufDev w;
    w.n = n; w.ld = round16(n); w.tiles = (n + 127) / 128; w.k = k; w.format = format;
    const int ld = w.ld, rn = std::min(operand_rn(rows), 64), row_blocks = (rows + rn - 1) / rn;      // the GGUF kernel's blocks hold up to 64 rows
    float *d_act32 = nullptr, *d_out = nullptr, *d_sums = nullptr; __nv_bfloat16 *d_act = nullptr; int *d_flag = nullptr; unsigned char *d_native = nullptr;
    e->partial_floats = size_t(16) * row_blocks * rn * ld;
    spl_status s = SPL_OK;
    if (cudaMalloc(reinterpret_cast<void **>(&w.blocks), w.device_bytes()) != cudaSuccess || cudaMalloc(reinterpret_cast<void **>(&d_native), w.bytes()) != cudaSuccess)
        s = SPL_ERR_ALLOCATION_FAILED;
    if (s == SPL_OK) s = device_alloc(e, &d_act32, size_t(rows) * k);
    if (s == SPL_OK) s = device_alloc(e, &d_act, size_t(row_blocks) * rn * k);
    if (s == SPL_OK) s = device_alloc(e, &d_sums, spl_operand_sums_floats(size_t(row_blocks) * rn, k));
    if (s == SPL_OK) s = device_alloc(e, &d_out, size_t(rows) * ld);
    if (s == SPL_OK) s = device_alloc(e, &d_flag, 64);
    if (s == SPL_OK) s = device_alloc(e, &e->partials, e->partial_floats);
    if (s == SPL_OK) {
        cudaMemsetAsync(w.blocks, 0, w.device_bytes(), e->stream);           // columns past n are zero blocks: weights 0
        cudaMemcpyAsync(d_native, blocks, w.bytes(), cudaMemcpyHostToDevice, e->stream);
        const size_t items = size_t(n) * (k / 256) * spl_gguf_pieces(format);
        spl_repack_gguf_kernel<<<int(std::min<size_t>((items + 255) / 256, 16384)), 256, 0, e->stream>>>(d_native, n, k / 256, format, w.blocks, 0);
        cudaMemsetAsync(d_act, 0, size_t(row_blocks) * rn * k * 2, e->stream);
        cudaMemsetAsync(d_sums, 0, spl_operand_sums_floats(size_t(row_blocks) * rn, k) * 4, e->stream);
        cudaMemsetAsync(d_flag, 0, 64 * sizeof(int), e->stream);
        cudaMemcpyAsync(d_act32, activations, size_t(rows) * k * 4, cudaMemcpyHostToDevice, e->stream);
        spl_operand_kernel<<<rows, 256, 0, e->stream>>>(d_act32, SplOperand{d_act, d_sums, rn, row_blocks}, k);
        if (residual) cudaMemcpy2DAsync(d_out, size_t(ld) * 4, residual, size_t(n) * 4, size_t(n) * 4, rows, cudaMemcpyHostToDevice, e->stream);
        launch_gemm_gguf(e->stream, w, GemmOperand{d_act, d_sums, rn, row_blocks}, d_out, residual ? d_out : nullptr, rows, e->partials, e->partial_floats, d_flag);
        s = check_launch(e, "gguf gemm");
        if (cudaStreamSynchronize(e->stream) != cudaSuccess) s = SPL_ERR_DEVICE;
        int flag = 0;
        if (s == SPL_OK) { cudaMemcpy(&flag, d_flag, sizeof flag, cudaMemcpyDeviceToHost); if (flag) s = SPL_ERR_TIMEOUT; }
        if (s == SPL_OK) cudaMemcpy2D(out, size_t(n) * 4, d_out, size_t(ld) * 4, size_t(n) * 4, rows, cudaMemcpyDeviceToHost);
    }
    cudaFree(d_sums); cudaFree(d_flag); cudaFree(d_native);
    cudaFree(w.blocks); cudaFree(d_act32); cudaFree(d_act); cudaFree(d_out); cudaFree(e->partials);
    cudaStreamDestroy(e->stream);
    e->stream = nullptr; e->partials = nullptr;
    return s;
}


// ---- The engine's primitives on device buffers: what the drafter builds its passes from -------
// (Sources/SploshRuntime/DraftModel.swift:344-357, 418-468; Engine.gemm / norm / mlpIn / embed, Engine.swift:1561-1625,
// 1905-1998.) Every call queues on the engine's stream and returns; spl_pass_wait finishes the pass.

struct spl_tensor {
    SplQ4Dev q;                 // a q4 tensor in the GEMM's device layout, or
    uint16_t *vec = nullptr;    // a bf16 vector
    int count = 0;
};

// fp32 rows -> x * rsqrt(mean x^2 + eps) * w as fp32 rows (Sources/Shaders/engine.metal:159-178). Grid (rows), 256 threads.
static __global__ void __launch_bounds__(256) spl_norm_rows_kernel(const float *__restrict__ in, const uint16_t *__restrict__ weight, float *out, int dim, float eps) {
    __shared__ float parts[8];
    spl_grid_begin();
    const float *x = in + size_t(blockIdx.x) * dim;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < dim; i += 256) ss += x[i] * x[i];
    ss = spl_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) parts[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < 8; ++w) total += parts[w];
    const float inv = 1.0f / sqrtf(total / float(dim) + eps);
    for (int i = threadIdx.x; i < dim; i += 256) out[size_t(blockIdx.x) * dim + i] = x[i] * inv * spl_bf16_to_float(weight[i]);
}
// gate <- bf16(silu(gate) * up), elementwise (Sources/Shaders/engine.metal:200-219).
static __global__ void spl_silu_mul_kernel(float *gate, const float *__restrict__ up, size_t count) {
    spl_grid_begin();
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < count; i += size_t(gridDim.x) * blockDim.x)
        gate[i] = spl_bf16_to_float(spl_float_to_bf16(spl_silu_exact(gate[i]) * up[i]));
}

spl_status spl_tensor_create_q4(spl_engine *e, int32_t rows, int32_t inner, const uint32_t *packed, const uint16_t *scales, const uint16_t *biases, spl_tensor **out) {
    if (!e || !packed || !scales || !biases || !out || rows <= 0 || inner <= 0 || inner % 256) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    if (inner > e->g.inter) return e->fail(SPL_ERR_INVALID_ARGUMENT, "a tensor's inner dimension may not exceed the engine's MLP width (its operand scratch is sized for that)");
    spl_tensor *t = new spl_tensor;
    spl_status s = alloc_q4(e, t->q, rows, inner);
    if (s == SPL_OK) s = upload_q4_into(e, t->q, 0, rows, inner, packed, scales, biases, false);
    // The GEMM's scratch for partial sums has to hold this tensor's at any row count.
    size_t need = 0;
    const int row_blocks = std::max(1, e->c.max_rows / 128);
    for (int rn : {16, 32, 64, 128})
        for (int rbs = 1; rbs <= (rn == 128 ? row_blocks : 1); ++rbs) need = std::max(need, gemm_slot_floats(t->q, e->sms, rn, rbs, false, false));
    if (s == SPL_OK && need > e->slot_floats) {
        cudaFree(e->slots); e->slots = nullptr;
        if (cudaMalloc(reinterpret_cast<void **>(&e->slots), need * 4) != cudaSuccess) s = e->fail(SPL_ERR_ALLOCATION_FAILED, "GEMM scratch");
        else e->slot_floats = need;
    }
    if (s != SPL_OK) { cudaFree(t->q.codes); cudaFree(t->q.sb); delete t; return s; }
    *out = t;
    return SPL_OK;
}
spl_status spl_tensor_create_vector(spl_engine *e, const uint16_t *bf16, int32_t count, spl_tensor **out) {
    if (!e || !bf16 || !out || count <= 0) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    spl_tensor *t = new spl_tensor;
    if (cudaMalloc(reinterpret_cast<void **>(&t->vec), size_t(count) * 2) != cudaSuccess) { delete t; return e->fail(SPL_ERR_ALLOCATION_FAILED, "vector"); }
    cudaMemcpy(t->vec, bf16, size_t(count) * 2, cudaMemcpyHostToDevice);
    t->count = count;
    *out = t;
    return SPL_OK;
}
void spl_tensor_destroy(spl_engine *e, spl_tensor *t) {
    if (!e || !t) return;
    cudaSetDevice(e->device);
    cudaStreamSynchronize(e->stream);
    cudaFree(t->q.codes); cudaFree(t->q.sb); cudaFree(t->vec);
    delete t;
}

spl_status spl_pass_begin(spl_engine *e) {
    if (!e) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    return SPL_OK;
}

// device_out[r][:] = GEMM(w, device_in[r][:]) (+ device_residual), rows of w.k floats in, w.n floats out (Engine.gemm).
static spl_status pass_gemm(spl_engine *e, const SplQ4Dev &w, const float *device_in, int rows, const float *device_residual, float *device_out) {
    if (!device_in || !device_out || rows <= 0 || rows > e->c.max_rows) return e->fail(SPL_ERR_INVALID_ROWS, "invalid step rows: row count outside the engine's limit");
    if (w.ld != w.n) return e->fail(SPL_ERR_INVALID_ARGUMENT, "the tensor's row count must be a multiple of 16");
    const int rn = operand_rn(rows), blocks = (rows + rn - 1) / rn;
    const SplOperand operand{e->act, e->act_sums, rn, blocks};
    launch_step(spl_operand_kernel, dim3(rows), dim3(256), 0, e->stream, device_in, operand, w.k);
    const GemmScratch scratch{e->slots, e->slot_floats, e->tc_error, e->sms};
    if (!launch_gemm_rows(e->stream, w, GemmOperand{e->act, e->act_sums, rn, blocks}, device_out, device_residual, rows, scratch, GemmExtras(), nullptr))
        return e->fail(SPL_ERR_INVALID_ROWS, "invalid step rows: the GEMM scratch is smaller than the call needs");
    return check_launch(e, "spl_pass_gemm");
}
spl_status spl_pass_gemm(spl_engine *e, const spl_tensor *weight, const float *device_in, int32_t rows, const float *device_residual, float *device_out) {
    if (!e || !weight || !weight->q.codes) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    return pass_gemm(e, weight->q, device_in, rows, device_residual, device_out);
}
// The target's lm_head on the caller's rows (DraftModel.swift:462-466 reuses it): [rows][hidden] -> [rows][vocab].
spl_status spl_pass_gemm_head(spl_engine *e, const float *device_in, int32_t rows, float *device_out) {
    if (!e) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    if (!e->head.codes) return e->fail(SPL_ERR_INVALID_ARGUMENT, "the head is not an MLX affine-4 tensor of this engine");
    return pass_gemm(e, e->head, device_in, rows, nullptr, device_out);
}
spl_status spl_pass_norm(spl_engine *e, const float *device_in, const spl_tensor *weight, int32_t rows, int32_t dim, float *device_out) {
    if (!e || !device_in || !device_out || !weight || !weight->vec || rows <= 0 || dim <= 0 || weight->count != dim) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    launch_step(spl_norm_rows_kernel, dim3(rows), dim3(256), 0, e->stream, device_in, (const uint16_t *)weight->vec, device_out, int(dim), e->g.eps);
    return check_launch(e, "spl_pass_norm");
}
spl_status spl_pass_embed(spl_engine *e, const uint32_t *device_tokens, int32_t rows, float *device_out) {
    if (!e || !device_tokens || !device_out || rows <= 0) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    if (e->g_embed) launch_step(spl_embed_gguf_kernel, dim3(rows), dim3(256), 0, e->stream, (const unsigned char *)e->g_embed, e->g_embed_format, device_tokens, device_out, e->g.hidden);
    else launch_step(spl_embed_q4_kernel, dim3(rows), dim3(128), 0, e->stream, e->embed_packed, e->embed_scales, e->embed_biases, (uint32_t *)device_tokens, device_out, e->g.hidden);
    return check_launch(e, "spl_pass_embed");
}
// Engine.mlpIn (Engine.swift:1905-1967): device_out = bf16(silu(gate x) * (up x)) as fp32 rows; device_scratch holds up x.
spl_status spl_pass_mlp_in(spl_engine *e, const spl_tensor *gate, const spl_tensor *up, const float *device_in, int32_t rows, float *device_out, float *device_scratch) {
    if (!e || !gate || !up || !gate->q.codes || !up->q.codes || !device_scratch || gate->q.n != up->q.n || gate->q.k != up->q.k) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    spl_status s = pass_gemm(e, gate->q, device_in, rows, nullptr, device_out);
    if (s == SPL_OK) s = pass_gemm(e, up->q, device_in, rows, nullptr, device_scratch);
    if (s != SPL_OK) return s;
    const size_t count = size_t(rows) * gate->q.n;
    launch_step(spl_silu_mul_kernel, dim3(int(std::min<size_t>((count + 255) / 256, 4096))), dim3(256), 0, e->stream, device_out, (const float *)device_scratch, count);
    return check_launch(e, "spl_pass_mlp_in");
}
// The pass's end (CommandGraph.commitAndWait): waits for everything queued, reports a kernel that gave up a wait.
spl_status spl_pass_wait(spl_engine *e) {
    if (!e) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    int flag[4] = {0, 0, 0, 0};
    SPL_CUDA(cudaMemcpy(flag, e->tc_error, sizeof flag, cudaMemcpyDeviceToHost));
    if (flag[0]) {
        cudaMemset(e->tc_error, 0, sizeof flag);
        return e->fail(SPL_ERR_TIMEOUT, "a GEMM block of the pass gave up waiting (warp " + std::to_string(flag[0] - 1) + "; first wait " + std::to_string(flag[1]) + ")");
    }
    return SPL_OK;
}

}  // extern "C"

#include "spl_draft_impl.cuh"
