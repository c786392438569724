// spl_draft_impl.cuh — the DFlash 2 block-diffusion drafter over the engine's primitives (Sources/SploshRuntime/DraftModel.swift).
// Included at the end of spl_engine.cu: it uses the engine's stream, scratch and feature rows directly.
//
// A draft pass proposes a whole block of tokens at once: the block is [anchor, mask x (block - 1)], and a few non-causal
// layers attend over the block plus a sliding window of context derived from the target's hidden states at its tap
// layers (DraftModel.swift:1-13). A selector then traces one path through the top candidates of every position
// (:479-531). The checkpoint is bf16; its linear layers are quantised here to the target's MLX affine-4 form (:635-727).
#pragma once
#include "spl_draft.cuh"
#include <thread>

#define SPL_DRAFT_ATTENTION_SPANS 8       // the reference walks eight; a span here is a block of four query heads

// ---- host arithmetic shared with the tests (no device needed) ---------------------------------
static inline float draft_bf16_float(uint16_t bits) { uint32_t u = uint32_t(bits) << 16; float f; memcpy(&f, &u, 4); return f; }
static inline uint16_t draft_float_bf16(float v) {            // DraftModel.bf16 (:721-724)
    uint32_t bits; memcpy(&bits, &v, 4);
    return uint16_t((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
}
// Swift's rounded() rounds to nearest with ties away from zero.
static inline float draft_code_of(float value, float bias, float scale) { return std::min(15.0f, std::max(0.0f, std::round((value - bias) / scale))); }

// DraftModel.fitRange (:682-719): a few clipped ranges, scale and bias refitted to the codes each gives by least squares,
// the candidate with the least squared error (after bf16 rounding) kept.
static void draft_fit_range(const float *x, float lowest, float highest, uint16_t &scale_bits, uint16_t &bias_bits) {
    auto error = [&](uint16_t sb, uint16_t bb) -> float {
        const float scale = draft_bf16_float(sb), bias = draft_bf16_float(bb);
        if (!(scale > 0.0f) || !std::isfinite(scale) || !std::isfinite(bias)) return INFINITY;
        float sum = 0.0f;
        for (int i = 0; i < 64; ++i) {
            const float code = draft_code_of(x[i], bias, scale), difference = x[i] - (bias + scale * code);
            sum += difference * difference;
        }
        return sum;
    };
    uint16_t best_s = scale_bits, best_b = bias_bits;
    float best_error = error(best_s, best_b);
    const float range = highest - lowest, count = 64.0f, cuts[3] = {0.0f, 0.04f, 0.08f};
    for (float low : cuts)
        for (float high : cuts) {
            float scale = (range * (1.0f - low - high)) / 15.0f, bias = lowest + low * range;
            for (int pass = 0; pass < 2; ++pass) {
                float sum_code = 0.0f, sum_value = 0.0f, sum_code2 = 0.0f, sum_code_value = 0.0f;
                for (int i = 0; i < 64; ++i) {
                    const float code = draft_code_of(x[i], bias, scale);
                    sum_code += code; sum_value += x[i]; sum_code2 += code * code; sum_code_value += code * x[i];
                }
                const float determinant = count * sum_code2 - sum_code * sum_code;
                if (!(determinant > 0.0f)) break;
                const float refitted = (count * sum_code_value - sum_code * sum_value) / determinant;
                if (!(refitted > 0.0f)) break;
                scale = refitted;
                bias = (sum_value - refitted * sum_code) / count;
            }
            const uint16_t cs = draft_float_bf16(scale), cb = draft_float_bf16(bias);
            const float candidate_error = error(cs, cb);
            if (candidate_error < best_error) { best_s = cs; best_b = cb; best_error = candidate_error; }
        }
    scale_bits = best_s; bias_bits = best_b;
}

static void draft_quantize_rows(const uint16_t *source, int row0, int row1, int inner, bool fitted, uint32_t *packed, uint16_t *scales, uint16_t *biases) {
    const int groups = inner / 64, words = inner / 8;
    float values[64];
    for (int row = row0; row < row1; ++row)
        for (int group = 0; group < groups; ++group) {
            const uint16_t *input = source + size_t(row) * inner + group * 64;
            float lowest = INFINITY, highest = -INFINITY;
            for (int i = 0; i < 64; ++i) { values[i] = draft_bf16_float(input[i]); lowest = std::min(lowest, values[i]); highest = std::max(highest, values[i]); }
            uint16_t scale_bits = draft_float_bf16(highest > lowest ? (highest - lowest) / 15.0f : 1.0f), bias_bits = draft_float_bf16(lowest);
            if (fitted && highest > lowest) draft_fit_range(values, lowest, highest, scale_bits, bias_bits);
            const float scale = draft_bf16_float(scale_bits), bias = draft_bf16_float(bias_bits);
            const size_t slot = size_t(row) * groups + group;
            scales[slot] = scale_bits; biases[slot] = bias_bits;
            for (int word = 0; word < 8; ++word) {
                uint32_t bits = 0;
                for (int nibble = 0; nibble < 8; ++nibble) bits |= uint32_t(draft_code_of(values[word * 8 + nibble], bias, scale)) << (nibble * 4);
                packed[size_t(row) * words + group * 8 + word] = bits;
            }
        }
}

struct DraftLayer {
    spl_tensor *input_norm = nullptr, *post_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr, *attention_base = nullptr, *mlp_base = nullptr;
    spl_tensor *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr, *gate = nullptr, *up = nullptr, *down = nullptr, *attention_kernel = nullptr, *mlp_kernel = nullptr;
    __half *k_ring = nullptr, *v_ring = nullptr;
    float *c_k = nullptr, *c_v = nullptr;
};

struct spl_draft {
    spl_engine *e = nullptr;
    spl_draft_config c{};
    int hidden = 0, inter = 0, vocab = 0, groups = 0, attention = 0, kv = 0, feature_width = 0, context_rows = 0, block_rows = 0;
    std::vector<DraftLayer> layers;
    spl_tensor *fc = nullptr, *hidden_norm = nullptr, *final_norm = nullptr;
    std::vector<float> hidden_projection;                  // [rank][hidden]
    std::vector<uint16_t> predecessor, successor;          // [vocab][rank] bf16
    std::vector<int> context_first, context_end;
    // the context pass
    float *c_features = nullptr, *c_hidden = nullptr, *c_normed = nullptr;
    uint32_t *c_meta = nullptr;                            // engine row, slot, position: three runs of context_rows
    __nv_bfloat16 *wide_act = nullptr; float *wide_sums = nullptr;      // the fc GEMM's operand: its inner dimension is the taps' width, wider than the engine's scratch
    // the block pass
    uint32_t *b_meta = nullptr;                            // tokens, slot, position, lo, hi, gather, offset: seven runs of the rows; then (first row, rows) per request
    float *dh = nullptr, *x = nullptr, *xc = nullptr, *t = nullptr, *dyn = nullptr, *qp = nullptr, *kp = nullptr, *vp = nullptr, *ao = nullptr,
          *gate = nullptr, *up = nullptr, *dn = nullptr, *selected = nullptr, *logits = nullptr, *top_values = nullptr;
    int32_t *top_ids = nullptr;
    float *attention_partials = nullptr;                          // [rows][heads][spans][2 + 128]
    float *cand_values = nullptr; int32_t *cand_ids = nullptr;     // the candidates of the row's stretches [picked][segments][candidates]
    float *projection_dev = nullptr, *projected = nullptr;      // the selector's matrix [rank][hidden] and its products with the drafted rows [picked][rank]
    int last_picked = 0, topk_segments = 16;                     // stretches a row of logits is cut in: each at most SPL_DRAFT_TOPK_STRETCH values
    std::string error;
};

static spl_status draft_fail(spl_draft *d, spl_status s, const std::string &why) { d->error = why; return d->e->fail(s, "draft model: " + why); }

template <typename T> static bool draft_alloc(T **p, size_t count) {
    if (cudaMalloc(reinterpret_cast<void **>(p), std::max<size_t>(count, 4) * sizeof(T)) != cudaSuccess) return false;
    return cudaMemset(*p, 0, std::max<size_t>(count, 4) * sizeof(T)) == cudaSuccess;
}

// A q4 tensor of any inner dimension (the engine's own operand scratch limits spl_tensor_create_q4 to its MLP width).
static spl_status draft_linear(spl_draft *d, const uint16_t *bf16, int rows, int inner, spl_tensor **out) {
    spl_engine *e = d->e;
    if (inner % 256 || rows % 16) return draft_fail(d, SPL_ERR_INVALID_ARGUMENT, "a linear tensor wants rows in sixteens and an inner dimension in 256s");
    std::vector<uint32_t> packed(size_t(rows) * inner / 8);
    std::vector<uint16_t> scales(size_t(rows) * inner / 64), biases(size_t(rows) * inner / 64);
    const int workers = std::max(1, std::min<int>(int(std::thread::hardware_concurrency()), rows / 16));
    std::vector<std::thread> pool;
    for (int w = 0; w < workers; ++w) {
        const int r0 = int(int64_t(rows) * w / workers), r1 = int(int64_t(rows) * (w + 1) / workers);
        pool.emplace_back(draft_quantize_rows, bf16, r0, r1, inner, d->c.minmax_ranges == 0, packed.data(), scales.data(), biases.data());
    }
    for (auto &t : pool) t.join();
    if (inner <= e->g.inter) return spl_tensor_create_q4(e, rows, inner, packed.data(), scales.data(), biases.data(), out);
    spl_tensor *t = new spl_tensor;
    spl_status s = alloc_q4(e, t->q, rows, inner);
    if (s == SPL_OK) s = upload_q4_into(e, t->q, 0, rows, inner, packed.data(), scales.data(), biases.data(), false);
    size_t need = 0;
    for (int rn : {16, 32, 64, 128}) need = std::max(need, gemm_slot_floats(t->q, e->sms, rn, std::max(1, e->c.max_rows / 128), false, false));
    if (s == SPL_OK && need > e->slot_floats) {
        cudaFree(e->slots); e->slots = nullptr;
        if (cudaMalloc(reinterpret_cast<void **>(&e->slots), need * 4) != cudaSuccess) s = e->fail(SPL_ERR_ALLOCATION_FAILED, "GEMM scratch");
        else e->slot_floats = need;
    }
    if (s != SPL_OK) { cudaFree(t->q.codes); cudaFree(t->q.sb); delete t; return s; }
    *out = t;
    return SPL_OK;
}

// Engine.gemm on an operand scratch of the drafter's own (the context pass's fc).
static spl_status draft_gemm_wide(spl_draft *d, const SplQ4Dev &w, const float *in, int rows, float *out) {
    spl_engine *e = d->e;
    const int rn = operand_rn(rows), blocks = (rows + rn - 1) / rn;
    const SplOperand operand{d->wide_act, d->wide_sums, rn, blocks};
    launch_step(spl_operand_kernel, dim3(rows), dim3(256), 0, e->stream, in, operand, w.k);
    const GemmScratch scratch{e->slots, e->slot_floats, e->tc_error, e->sms};
    if (!launch_gemm_rows(e->stream, w, GemmOperand{d->wide_act, d->wide_sums, rn, blocks}, out, nullptr, rows, scratch, GemmExtras(), nullptr))
        return draft_fail(d, SPL_ERR_INVALID_ROWS, "the GEMM scratch is smaller than the context pass needs");
    return check_launch(e, "draft fc");
}

template <int G>
static void draft_attention_launch(spl_draft *d, const DraftLayer &L, int rows, int requests, const uint32_t *request_rows, const uint32_t *slots, const uint32_t *positions,
                                   const uint32_t *lo, const uint32_t *hi) {
    spl_engine *e = d->e;
    const float scale = 1.0f / sqrtf(float(SPL_DRAFT_HEAD_DIM));
    if (d->c.max_block * G <= 64)
        // a request's rows x G query heads fit the tensor-core form's 64 queries a block
        launch_step(spl_draft_attention_mma_kernel<G>, dim3(d->c.kv_heads, requests, SPL_DRAFT_ATTENTION_SPANS), dim3(128), 0, e->stream, (const float *)d->qp,
                    (const uint16_t *)L.q_norm->vec, request_rows, slots, positions, lo, hi, (const __half *)L.k_ring, (const __half *)L.v_ring, d->attention_partials,
                    int(d->c.heads), int(d->c.kv_heads), int(d->c.ring_capacity), int(d->c.window), scale, e->g.eps, e->g.rope_theta);
    else
        launch_step(spl_draft_attention_kernel<G>, dim3(d->c.kv_heads, rows, SPL_DRAFT_ATTENTION_SPANS), dim3(128), 0, e->stream, (const float *)d->qp, (const uint16_t *)L.q_norm->vec, slots,
                    positions, lo, hi, (const __half *)L.k_ring, (const __half *)L.v_ring, d->attention_partials, int(d->c.heads), int(d->c.kv_heads), int(d->c.ring_capacity),
                    int(d->c.window), scale, e->g.eps, e->g.rope_theta);
    launch_step(spl_draft_attention_merge_kernel, dim3(d->c.heads, rows), dim3(128), 0, e->stream, (const float *)d->attention_partials, d->ao, int(d->c.heads), SPL_DRAFT_ATTENTION_SPANS);
}

extern "C" {

spl_status spl_draft_quantize_q4(const uint16_t *bf16, int32_t rows, int32_t inner, int32_t fitted, uint32_t *packed, uint16_t *scales, uint16_t *biases) {
    if (!bf16 || !packed || !scales || !biases || rows <= 0 || inner <= 0 || inner % 64) return SPL_ERR_INVALID_ARGUMENT;
    draft_quantize_rows(bf16, 0, rows, inner, fitted != 0, packed, scales, biases);
    return SPL_OK;
}

// The path through the candidates given every position's projected hidden state [drafted][rank] (DraftModel.swift:503-529).
static spl_status draft_select_projected(int drafted, int k, int rank, int anchor, const int32_t *ids, const float *values, const float *projected_rows,
                                         const uint16_t *predecessor, const uint16_t *successor, float temperature, uint64_t *random_state, int32_t *tokens,
                                         float *probabilities) {
    std::vector<float> gated(rank), scores(k), q(k);
    int predecessor_token = anchor;
    for (int position = 0; position < drafted; ++position) {
        const float *projected = projected_rows + size_t(position) * rank;
        const uint16_t *before = predecessor + size_t(predecessor_token) * rank;
        for (int r = 0; r < rank; ++r) gated[r] = draft_bf16_float(before[r]) * projected[r];
        for (int c = 0; c < k; ++c) {
            const uint16_t *after = successor + size_t(ids[position * k + c]) * rank;
            float pairwise = 0.0f;
            for (int r = 0; r < rank; ++r) pairwise += gated[r] * draft_bf16_float(after[r]);
            scores[c] = values[position * k + c] + pairwise;
        }
        int choice = 0;
        if (temperature > 0.0f) {
            float top = scores[0];
            for (int c = 1; c < k; ++c) top = std::max(top, scores[c]);
            float total = 0.0f;
            for (int c = 0; c < k; ++c) { q[c] = expf((scores[c] - top) / temperature); total += q[c]; }
            for (int c = 0; c < k; ++c) q[c] /= total;
            *random_state += 0x9E3779B97F4A7C15ull;                 // SplitMix.uniform (:731-739)
            uint64_t z = *random_state;
            z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull; z ^= z >> 31;
            float draw = float(z >> 40) / 16777216.0f;
            choice = k - 1;
            for (int c = 0; c < k; ++c) { draw -= q[c]; if (draw <= 0.0f) { choice = c; break; } }
            for (int c = 0; c < k; ++c) probabilities[position * k + c] = q[c];
        } else {
            for (int c = 1; c < k; ++c) if (scores[c] > scores[choice]) choice = c;
        }
        predecessor_token = ids[position * k + choice];
        tokens[position] = predecessor_token;
    }
    return SPL_OK;
}

spl_status spl_draft_select(int32_t drafted, int32_t k, int32_t rank, int32_t hidden, int32_t anchor, const int32_t *ids, const float *values,
                            const float *hidden_rows, const float *hidden_projection, const uint16_t *predecessor, const uint16_t *successor,
                            float temperature, uint64_t *random_state, int32_t *tokens, float *probabilities) {
    if (drafted < 0 || k < 1 || rank < 1 || hidden < 1 || !ids || !values || !hidden_rows || !hidden_projection || !predecessor || !successor || !tokens ||
        (temperature > 0.0f && (!random_state || !probabilities))) return SPL_ERR_INVALID_ARGUMENT;
    std::vector<float> projected(size_t(std::max(drafted, 1)) * rank);
    for (int position = 0; position < drafted; ++position)
        for (int r = 0; r < rank; ++r) {
            const float *m = hidden_projection + size_t(r) * hidden, *hs = hidden_rows + size_t(position) * hidden;
            float sum = 0.0f;
            for (int h = 0; h < hidden; ++h) sum += m[h] * hs[h];
            projected[size_t(position) * rank + r] = sum;
        }
    return draft_select_projected(drafted, k, rank, anchor, ids, values, projected.data(), predecessor, successor, temperature, random_state, tokens, probabilities);
}

void spl_draft_destroy(spl_draft *d) {
    if (!d) return;
    spl_engine *e = d->e;
    cudaSetDevice(e->device);
    cudaStreamSynchronize(e->stream);
    for (DraftLayer &L : d->layers) {
        for (spl_tensor *t : {L.input_norm, L.post_norm, L.q_norm, L.k_norm, L.attention_base, L.mlp_base, L.q, L.k, L.v, L.o, L.gate, L.up, L.down, L.attention_kernel, L.mlp_kernel})
            spl_tensor_destroy(e, t);
        cudaFree(L.k_ring); cudaFree(L.v_ring); cudaFree(L.c_k); cudaFree(L.c_v);
    }
    for (spl_tensor *t : {d->fc, d->hidden_norm, d->final_norm}) spl_tensor_destroy(e, t);
    for (void *p : {(void *)d->c_features, (void *)d->c_hidden, (void *)d->c_normed, (void *)d->c_meta, (void *)d->wide_act, (void *)d->wide_sums, (void *)d->b_meta, (void *)d->dh,
                    (void *)d->x, (void *)d->xc, (void *)d->t, (void *)d->dyn, (void *)d->qp, (void *)d->kp, (void *)d->vp, (void *)d->ao, (void *)d->gate, (void *)d->up, (void *)d->dn,
                    (void *)d->selected, (void *)d->logits, (void *)d->top_values, (void *)d->top_ids, (void *)d->projection_dev, (void *)d->projected, (void *)d->cand_values, (void *)d->cand_ids, (void *)d->attention_partials}) cudaFree(p);
    delete d;
}

spl_status spl_draft_create(spl_engine *e, const spl_draft_config *config, spl_draft **out) {
    if (!e || !config || !out) return SPL_ERR_INVALID_ARGUMENT;
    SPL_NOT_IN_FLIGHT(e);
    const spl_draft_config &c = *config;
    const int G = c.kv_heads > 0 ? c.heads / c.kv_heads : 0;
    if (c.layers < 1 || c.heads < 1 || c.kv_heads < 1 || c.heads % c.kv_heads || (G != 1 && G != 2 && G != 4 && G != 8) || c.group_size < 1 || e->g.hidden % c.group_size ||
        c.rank < 1 || c.window < 1 || c.block_size < 1 || c.max_block < c.block_size || c.max_block % c.block_size || c.ring_capacity < c.window + c.max_block ||
        c.candidates < 1 || c.candidates > 64 || c.mask_token < 0 || c.mask_token >= e->g.vocab)
        return e->fail(SPL_ERR_INVALID_ARGUMENT, "draft model: invalid configuration");
    if (e->feature_layers.empty()) return e->fail(SPL_ERR_INVALID_ARGUMENT, "draft model: the engine's feature taps are not enabled");
    if (e->c.max_slots * c.max_block > e->c.max_rows) return e->fail(SPL_ERR_INVALID_ARGUMENT, "draft model: a block of every slot must fit the engine's row limit");
    SPL_CUDA(cudaSetDevice(e->device));
    spl_draft *d = new spl_draft;
    d->e = e; d->c = c;
    d->hidden = e->g.hidden; d->inter = e->g.inter; d->vocab = e->g.vocab; d->groups = e->g.hidden / c.group_size;
    d->attention = c.heads * SPL_DRAFT_HEAD_DIM; d->kv = c.kv_heads * SPL_DRAFT_HEAD_DIM;
    d->feature_width = int(e->feature_layers.size()) * e->g.hidden;
    d->context_rows = e->c.max_rows; d->block_rows = e->c.max_slots * c.max_block;
    d->topk_segments = std::max(16, (e->g.vocab + SPL_DRAFT_TOPK_STRETCH - 1) / SPL_DRAFT_TOPK_STRETCH);
    d->layers.resize(c.layers);
    d->context_first.assign(e->c.max_slots, 0); d->context_end.assign(e->c.max_slots, 0);
    const size_t CR = d->context_rows, BR = d->block_rows, H = d->hidden, RP = size_t((e->c.max_rows + 127) / 128) * 128;
    const size_t wide = std::max<size_t>(d->feature_width, 256);
    bool ok = draft_alloc(&d->c_features, CR * d->feature_width) && draft_alloc(&d->c_hidden, CR * H) && draft_alloc(&d->c_normed, CR * H) && draft_alloc(&d->c_meta, CR * 3) &&
              draft_alloc(&d->wide_act, RP * wide) && draft_alloc(&d->wide_sums, spl_operand_sums_floats(RP, wide)) &&
              draft_alloc(&d->b_meta, BR * 9) && draft_alloc(&d->dh, BR * H) && draft_alloc(&d->x, BR * H) && draft_alloc(&d->xc, BR * H) && draft_alloc(&d->t, BR * H) &&
              draft_alloc(&d->dyn, BR * 4 * d->groups) && draft_alloc(&d->qp, BR * d->attention) && draft_alloc(&d->kp, BR * d->kv) && draft_alloc(&d->vp, BR * d->kv) &&
              draft_alloc(&d->ao, BR * d->attention) && draft_alloc(&d->gate, BR * d->inter) && draft_alloc(&d->up, BR * d->inter) && draft_alloc(&d->dn, BR * H) &&
              draft_alloc(&d->selected, BR * H) && draft_alloc(&d->logits, BR * size_t(d->vocab)) && draft_alloc(&d->top_values, BR * 64) && draft_alloc(&d->top_ids, BR * 64) &&
              draft_alloc(&d->projection_dev, size_t(c.rank) * H) && draft_alloc(&d->projected, BR * c.rank) &&
              draft_alloc(&d->attention_partials, BR * c.heads * SPL_DRAFT_ATTENTION_SPANS * (SPL_DRAFT_HEAD_DIM + 2)) && draft_alloc(&d->cand_values, BR * d->topk_segments * 64) && draft_alloc(&d->cand_ids, BR * d->topk_segments * 64);
    for (DraftLayer &L : d->layers)
        ok = ok && draft_alloc(&L.k_ring, size_t(e->c.max_slots) * c.ring_capacity * d->kv) && draft_alloc(&L.v_ring, size_t(e->c.max_slots) * c.ring_capacity * d->kv) &&
             draft_alloc(&L.c_k, CR * d->kv) && draft_alloc(&L.c_v, CR * d->kv);
    if (!ok) { spl_draft_destroy(d); return e->fail(SPL_ERR_ALLOCATION_FAILED, "draft model: buffers"); }
    *out = d;
    return SPL_OK;
}

// One tensor of the checkpoint by its safetensors name (DraftModel.swift:172-203), as bf16 [rows][inner] (vectors: rows = 1).
spl_status spl_draft_set_tensor(spl_draft *d, const char *name, const uint16_t *bf16, int32_t rows, int32_t inner) {
    if (!d || !name || !bf16 || rows <= 0 || inner <= 0) return SPL_ERR_INVALID_ARGUMENT;
    spl_engine *e = d->e;
    SPL_NOT_IN_FLIGHT(e);
    SPL_CUDA(cudaSetDevice(e->device));
    const std::string n(name);
    const int H = d->hidden, D = SPL_DRAFT_HEAD_DIM;
    auto shape = [&](int want_rows, int want_inner) -> bool { return rows == want_rows && inner == want_inner; };
    auto wrong = [&]() { return draft_fail(d, SPL_ERR_INVALID_ARGUMENT, "shape mismatch: " + n); };
    auto vector_into = [&](spl_tensor **slot, int count) -> spl_status {
        if (size_t(rows) * inner != size_t(count)) return wrong();
        if (*slot) { spl_tensor_destroy(e, *slot); *slot = nullptr; }
        return spl_tensor_create_vector(e, bf16, count, slot);
    };
    auto linear_into = [&](spl_tensor **slot, int want_rows, int want_inner) -> spl_status {
        if (!shape(want_rows, want_inner)) return wrong();
        if (*slot) { spl_tensor_destroy(e, *slot); *slot = nullptr; }
        return draft_linear(d, bf16, rows, inner, slot);
    };
    if (n == "fc.weight") return linear_into(&d->fc, H, d->feature_width);
    if (n == "hidden_norm.weight") return vector_into(&d->hidden_norm, H);
    if (n == "norm.weight") return vector_into(&d->final_norm, H);
    if (n == "candidate_selector.hidden_projection.weight") {
        if (!shape(d->c.rank, H)) return wrong();
        d->hidden_projection.resize(size_t(rows) * inner);
        for (size_t i = 0; i < d->hidden_projection.size(); ++i) d->hidden_projection[i] = draft_bf16_float(bf16[i]);
        SPL_CUDA(cudaMemcpy(d->projection_dev, d->hidden_projection.data(), d->hidden_projection.size() * 4, cudaMemcpyHostToDevice));
        return SPL_OK;
    }
    if (n == "candidate_selector.predecessor_codebook" || n == "candidate_selector.successor_codebook") {
        if (!shape(d->vocab, d->c.rank)) return wrong();
        (n == "candidate_selector.predecessor_codebook" ? d->predecessor : d->successor).assign(bf16, bf16 + size_t(rows) * inner);
        return SPL_OK;
    }
    if (n.rfind("layers.", 0) == 0) {
        const size_t dot = n.find('.', 7);
        if (dot == std::string::npos) return draft_fail(d, SPL_ERR_INVALID_ARGUMENT, "unknown tensor: " + n);
        const int index = atoi(n.substr(7, dot - 7).c_str());
        if (index < 0 || index >= d->c.layers) return draft_fail(d, SPL_ERR_INVALID_ARGUMENT, "no such layer: " + n);
        DraftLayer &L = d->layers[index];
        const std::string rest = n.substr(dot + 1);
        if (rest == "input_layernorm.weight") return vector_into(&L.input_norm, H);
        if (rest == "post_attention_layernorm.weight") return vector_into(&L.post_norm, H);
        if (rest == "self_attn.q_norm.weight") return vector_into(&L.q_norm, D);
        if (rest == "self_attn.k_norm.weight") return vector_into(&L.k_norm, D);
        if (rest == "attention_conv.base_kernel") return vector_into(&L.attention_base, 4 * H);
        if (rest == "mlp_conv.base_kernel") return vector_into(&L.mlp_base, 4 * H);
        if (rest == "self_attn.q_proj.weight") return linear_into(&L.q, d->attention, H);
        if (rest == "self_attn.k_proj.weight") return linear_into(&L.k, d->kv, H);
        if (rest == "self_attn.v_proj.weight") return linear_into(&L.v, d->kv, H);
        if (rest == "self_attn.o_proj.weight") return linear_into(&L.o, H, d->attention);
        if (rest == "mlp.gate_proj.weight") return linear_into(&L.gate, d->inter, H);
        if (rest == "mlp.up_proj.weight") return linear_into(&L.up, d->inter, H);
        if (rest == "mlp.down_proj.weight") return linear_into(&L.down, H, d->inter);
        if (rest == "attention_conv.kernel_projection.weight") return linear_into(&L.attention_kernel, 4 * d->groups, H);
        if (rest == "mlp_conv.kernel_projection.weight") return linear_into(&L.mlp_kernel, 4 * d->groups, H);
    }
    return draft_fail(d, SPL_ERR_INVALID_ARGUMENT, "unknown tensor: " + n);
}

static spl_status draft_complete(spl_draft *d) {
    bool all = d->fc && d->hidden_norm && d->final_norm && !d->hidden_projection.empty() && !d->predecessor.empty() && !d->successor.empty();
    for (const DraftLayer &L : d->layers)
        all = all && L.input_norm && L.post_norm && L.q_norm && L.k_norm && L.attention_base && L.mlp_base && L.q && L.k && L.v && L.o && L.gate && L.up && L.down &&
              L.attention_kernel && L.mlp_kernel;
    return all ? SPL_OK : draft_fail(d, SPL_ERR_INVALID_ARGUMENT, "missing tensors");
}

spl_status spl_draft_reset_slot(spl_draft *d, int32_t slot);
// The checkpoint's tensors in the order the reference asks for them (DraftModel.swift:172-203), with their shapes.
static void draft_expected(const spl_draft *d, std::vector<std::string> *names, std::vector<std::vector<int64_t>> *shapes) {
    const int64_t H = d->hidden, D = SPL_DRAFT_HEAD_DIM;
    auto add = [&](const std::string &n, std::vector<int64_t> shape) { names->push_back(n); shapes->push_back(std::move(shape)); };
    for (int index = 0; index < d->c.layers; ++index) {
        const std::string p = "layers." + std::to_string(index) + ".";
        add(p + "input_layernorm.weight", {H}); add(p + "post_attention_layernorm.weight", {H});
        add(p + "self_attn.q_norm.weight", {D}); add(p + "self_attn.k_norm.weight", {D});
        add(p + "attention_conv.base_kernel", {2, 2, H}); add(p + "mlp_conv.base_kernel", {2, 2, H});
        add(p + "self_attn.q_proj.weight", {d->attention, H}); add(p + "self_attn.k_proj.weight", {d->kv, H}); add(p + "self_attn.v_proj.weight", {d->kv, H});
        add(p + "self_attn.o_proj.weight", {H, d->attention});
        add(p + "mlp.gate_proj.weight", {d->inter, H}); add(p + "mlp.up_proj.weight", {d->inter, H}); add(p + "mlp.down_proj.weight", {H, d->inter});
        add(p + "attention_conv.kernel_projection.weight", {4 * d->groups, H}); add(p + "mlp_conv.kernel_projection.weight", {4 * d->groups, H});
    }
    add("fc.weight", {H, d->feature_width}); add("hidden_norm.weight", {H}); add("norm.weight", {H});
    add("candidate_selector.hidden_projection.weight", {d->c.rank, H});
    add("candidate_selector.predecessor_codebook", {d->vocab, d->c.rank}); add("candidate_selector.successor_codebook", {d->vocab, d->c.rank});
}
int32_t spl_draft_tensor_count(const spl_draft *d) {
    if (!d) return 0;
    std::vector<std::string> names; std::vector<std::vector<int64_t>> shapes;
    draft_expected(d, &names, &shapes);
    return int32_t(names.size());
}
// Tensor `index` of the checkpoint: its name and its shape (up to four dimensions, *dimensions of them).
spl_status spl_draft_tensor_expected(const spl_draft *d, int32_t index, char *name, uint64_t name_bytes, int64_t *shape, int32_t *dimensions) {
    if (!d || !name || !name_bytes || !shape || !dimensions) return SPL_ERR_INVALID_ARGUMENT;
    std::vector<std::string> names; std::vector<std::vector<int64_t>> shapes;
    draft_expected(d, &names, &shapes);
    if (index < 0 || index >= int(names.size()) || names[index].size() + 1 > name_bytes) return SPL_ERR_INVALID_ARGUMENT;
    memcpy(name, names[index].c_str(), names[index].size() + 1);
    *dimensions = int32_t(shapes[index].size());
    for (size_t i = 0; i < shapes[index].size(); ++i) shape[i] = shapes[index][i];
    return SPL_OK;
}

// ---- context snapshots (DraftModel.exportContext / importContext, :285-311) ----
// The slot's rings as they stand for a prefix of `token_count` tokens: [first, end) and the rings' bytes, layer by layer, K then V.
uint64_t spl_draft_context_bytes(const spl_draft *d) { return d ? uint64_t(d->c.layers) * 2 * d->c.ring_capacity * d->kv * 2 : 0; }
// *first < 0 on return: nothing useful is held for that prefix (the reference's nil); `rings` is then untouched.
spl_status spl_draft_export_context(spl_draft *d, int32_t slot, int32_t token_count, int32_t *first, int32_t *end, void *rings) {
    if (!d || slot < 0 || slot >= int(d->context_end.size()) || !first || !end || !rings) return SPL_ERR_INVALID_ARGUMENT;
    spl_engine *e = d->e;
    SPL_NOT_IN_FLIGHT(e);
    *first = -1; *end = 0;
    if (d->context_end[slot] < token_count) return SPL_OK;
    // Positions evaluated after the prefix overwrote ring entries one capacity back.
    const int begin = std::max(d->context_first[slot], d->context_end[slot] + d->c.max_block - d->c.ring_capacity);
    if (begin >= token_count) return SPL_OK;
    SPL_CUDA(cudaSetDevice(e->device));
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    const size_t per_slot = size_t(d->c.ring_capacity) * d->kv * 2;
    uint8_t *out = static_cast<uint8_t *>(rings);
    for (DraftLayer &L : d->layers) {
        SPL_CUDA(cudaMemcpy(out, reinterpret_cast<const uint8_t *>(L.k_ring) + slot * per_slot, per_slot, cudaMemcpyDeviceToHost)); out += per_slot;
        SPL_CUDA(cudaMemcpy(out, reinterpret_cast<const uint8_t *>(L.v_ring) + slot * per_slot, per_slot, cudaMemcpyDeviceToHost)); out += per_slot;
    }
    *first = begin; *end = token_count;
    return SPL_OK;
}
// A snapshot of another size resets the slot, as the reference does.
spl_status spl_draft_import_context(spl_draft *d, int32_t slot, int32_t first, int32_t end, const void *rings, uint64_t bytes) {
    if (!d || slot < 0 || slot >= int(d->context_end.size()) || !rings || first < 0 || end < first) return SPL_ERR_INVALID_ARGUMENT;
    spl_engine *e = d->e;
    SPL_NOT_IN_FLIGHT(e);
    if (bytes != spl_draft_context_bytes(d)) return spl_draft_reset_slot(d, slot);
    SPL_CUDA(cudaSetDevice(e->device));
    SPL_CUDA(cudaStreamSynchronize(e->stream));
    const size_t per_slot = size_t(d->c.ring_capacity) * d->kv * 2;
    const uint8_t *in = static_cast<const uint8_t *>(rings);
    for (DraftLayer &L : d->layers) {
        SPL_CUDA(cudaMemcpy(reinterpret_cast<uint8_t *>(L.k_ring) + slot * per_slot, in, per_slot, cudaMemcpyHostToDevice)); in += per_slot;
        SPL_CUDA(cudaMemcpy(reinterpret_cast<uint8_t *>(L.v_ring) + slot * per_slot, in, per_slot, cudaMemcpyHostToDevice)); in += per_slot;
    }
    d->context_first[slot] = first; d->context_end[slot] = end;
    return SPL_OK;
}

// ---- context (DraftModel.swift:277-359) ----
spl_status spl_draft_reset_slot(spl_draft *d, int32_t slot) {
    if (!d || slot < 0 || slot >= int(d->context_end.size())) return SPL_ERR_INVALID_ARGUMENT;
    d->context_first[slot] = 0; d->context_end[slot] = 0;
    return SPL_OK;
}
spl_status spl_draft_truncate(spl_draft *d, int32_t slot, int32_t token_count) {
    if (!d || slot < 0 || slot >= int(d->context_end.size()) || token_count < 0) return SPL_ERR_INVALID_ARGUMENT;
    if (token_count >= d->context_end[slot]) return SPL_OK;
    // Later positions may have overwritten ring entries older than one capacity back.
    d->context_first[slot] = std::max(d->context_first[slot], d->context_end[slot] + d->c.max_block - d->c.ring_capacity);
    d->context_end[slot] = token_count;
    if (d->context_first[slot] >= d->context_end[slot]) d->context_first[slot] = token_count;
    return SPL_OK;
}
int32_t spl_draft_context_length(const spl_draft *d, int32_t slot, int32_t start) {
    if (!d || slot < 0 || slot >= int(d->context_end.size())) return 0;
    return d->context_end[slot] == start ? start - std::max(d->context_first[slot], start - d->c.window + 1) : 0;
}

static void draft_kv_store(spl_draft *d, const DraftLayer &L, const float *k, const float *v, const uint32_t *slots, const uint32_t *positions, int rows) {
    spl_engine *e = d->e;
    launch_step(spl_draft_kv_store_kernel, dim3(d->c.kv_heads, rows), dim3(32), 0, e->stream, k, v, (const uint16_t *)L.k_norm->vec, slots, positions, L.k_ring, L.v_ring,
                int(d->c.kv_heads), int(d->c.ring_capacity), e->g.eps, e->g.rope_theta);
}

// Fold target hidden states into the draft's context, straight after an engine step with feature taps: the step rows to keep
// and their positions (DraftModel.pushContext).
spl_status spl_draft_push_context(spl_draft *d, const spl_draft_context_entry *entries, int32_t count) {
    if (!d || (count > 0 && !entries) || count < 0) return SPL_ERR_INVALID_ARGUMENT;
    spl_engine *e = d->e;
    SPL_NOT_IN_FLIGHT(e);
    if (count == 0) return SPL_OK;
    spl_status s = draft_complete(d);
    if (s != SPL_OK) return s;
    if (count > d->context_rows) return draft_fail(d, SPL_ERR_INVALID_ROWS, "too many context rows");
    if (!e->features) return draft_fail(d, SPL_ERR_INVALID_ARGUMENT, "the engine's feature taps are not enabled");
    std::vector<uint32_t> meta(size_t(count) * 3);
    for (int i = 0; i < count; ++i) {
        const spl_draft_context_entry &en = entries[i];
        if (en.slot < 0 || en.slot >= e->c.max_slots || en.position < 0 || en.engine_row < 0 || en.engine_row >= e->last_rows)
            return draft_fail(d, SPL_ERR_INVALID_ROWS, "a context entry names no slot, position or row of the last step");
        meta[i] = uint32_t(en.engine_row); meta[count + i] = uint32_t(en.slot); meta[2 * size_t(count) + i] = uint32_t(en.position);
    }
    for (int i = 0; i < count; ++i) {
        const spl_draft_context_entry &en = entries[i];
        if (en.position != d->context_end[en.slot]) d->context_first[en.slot] = en.position;
        d->context_end[en.slot] = en.position + 1;
    }
    SPL_CUDA(cudaSetDevice(e->device));
    SPL_CUDA(cudaMemcpyAsync(d->c_meta, meta.data(), meta.size() * 4, cudaMemcpyHostToDevice, e->stream));
    const uint32_t *rows_dev = d->c_meta, *slots_dev = d->c_meta + count, *pos_dev = d->c_meta + 2 * size_t(count);
    launch_step(spl_draft_take_features_kernel, dim3(std::min((d->feature_width + 255) / 256, 64), count), dim3(256), 0, e->stream, (const float *)e->features, rows_dev,
                d->c_features, d->feature_width);
    s = draft_gemm_wide(d, d->fc->q, d->c_features, count, d->c_hidden);
    if (s == SPL_OK) s = spl_pass_norm(e, d->c_hidden, d->hidden_norm, count, d->hidden, d->c_normed);
    for (DraftLayer &L : d->layers) {
        if (s == SPL_OK) s = spl_pass_gemm(e, L.k, d->c_normed, count, nullptr, L.c_k);
        if (s == SPL_OK) s = spl_pass_gemm(e, L.v, d->c_normed, count, nullptr, L.c_v);
    }
    if (s != SPL_OK) return s;
    for (DraftLayer &L : d->layers) draft_kv_store(d, L, L.c_k, L.c_v, slots_dev, pos_dev, count);
    s = check_launch(e, "draft context");
    return s == SPL_OK ? spl_pass_wait(e) : s;
}

// Draft `block - 1` tokens for each request (DraftModel.propose). Outputs, request after request, a request's drafted
// positions in order: tokens [drafted], candidates [drafted][candidates], probabilities [drafted][candidates] (temperature > 0).
spl_status spl_draft_propose(spl_draft *d, const spl_draft_request *requests, int32_t count, float temperature, int32_t vocab_limit, uint64_t *random_state,
                             int32_t *tokens, int32_t *candidates, float *probabilities) {
    if (!d || (count > 0 && !requests) || count < 0 || !tokens || !candidates) return SPL_ERR_INVALID_ARGUMENT;
    spl_engine *e = d->e;
    SPL_NOT_IN_FLIGHT(e);
    if (count == 0) return SPL_OK;
    spl_status s = draft_complete(d);
    if (s != SPL_OK) return s;
    const spl_draft_config &c = d->c;
    int rows = 0;
    for (int i = 0; i < count; ++i) {
        const spl_draft_request &r = requests[i];
        if (r.block < c.block_size || r.block > c.max_block || r.block % c.block_size)
            return draft_fail(d, SPL_ERR_INVALID_ARGUMENT, "draft block must be a multiple of " + std::to_string(c.block_size) + " up to " + std::to_string(c.max_block));
        if (r.slot < 0 || r.slot >= e->c.max_slots || r.anchor < 0 || r.anchor >= d->vocab || r.start < 0) return draft_fail(d, SPL_ERR_INVALID_ARGUMENT, "a request names no slot, token or position");
        rows += r.block;
    }
    if (rows > d->block_rows || count > e->c.max_slots) return draft_fail(d, SPL_ERR_INVALID_ROWS, "too many draft requests");
    if (vocab_limit <= 0 || vocab_limit > d->vocab || c.candidates > vocab_limit) return draft_fail(d, SPL_ERR_INVALID_ARGUMENT, "vocabulary limit");
    if (temperature > 0.0f && (!random_state || !probabilities)) return SPL_ERR_INVALID_ARGUMENT;
    const size_t R = size_t(rows);
    std::vector<uint32_t> meta(R * 9);
    uint32_t *m_tokens = meta.data(), *m_slot = m_tokens + R, *m_pos = m_slot + R, *m_lo = m_pos + R, *m_hi = m_lo + R, *m_gather = m_hi + R, *m_offset = m_gather + R,
             *m_requests = m_offset + R;
    std::vector<int> first_picked;
    int row = 0, picked = 0;
    for (int i = 0; i < count; ++i) {
        const spl_draft_request &r = requests[i];
        // Without contiguous context up to the anchor, the block attends only to itself.
        const int first = d->context_end[r.slot] == r.start ? d->context_first[r.slot] : r.start;
        first_picked.push_back(picked);
        m_requests[2 * i] = uint32_t(row); m_requests[2 * i + 1] = uint32_t(r.block);
        for (int offset = 0; offset < r.block; ++offset) {
            m_tokens[row] = uint32_t(offset == 0 ? r.anchor : c.mask_token);
            m_slot[row] = uint32_t(r.slot); m_pos[row] = uint32_t(r.start + offset); m_lo[row] = uint32_t(first);
            m_hi[row] = uint32_t(r.start + (r.isolate_prefix && offset < c.block_size ? c.block_size : r.block));
            m_offset[row] = uint32_t(offset);
            if (offset > 0) m_gather[picked++] = uint32_t(row);
            ++row;
        }
    }
    SPL_CUDA(cudaSetDevice(e->device));
    SPL_CUDA(cudaMemcpyAsync(d->b_meta, meta.data(), meta.size() * 4, cudaMemcpyHostToDevice, e->stream));
    const uint32_t *b_tokens = d->b_meta, *b_slot = b_tokens + R, *b_pos = b_slot + R, *b_lo = b_pos + R, *b_hi = b_lo + R, *b_gather = b_hi + R, *b_offset = b_gather + R, *b_requests = b_offset + R;
    const int H = d->hidden, G = c.heads / c.kv_heads;
    auto conv = [&](const float *in, const spl_tensor *base, float *out, int which, int accumulate) {
        launch_step(spl_draft_conv_kernel, dim3((H + 255) / 256, rows), dim3(256), 0, e->stream, in, (const float *)d->dyn, (const uint16_t *)base->vec, out, H, int(c.group_size),
                    d->groups, which, accumulate, b_offset);
    };
    s = spl_pass_embed(e, b_tokens, rows, d->dh);
    for (DraftLayer &L : d->layers) {
        if (s != SPL_OK) break;
        s = spl_pass_norm(e, d->dh, L.input_norm, rows, H, d->x);
        if (s == SPL_OK) s = spl_pass_gemm(e, L.attention_kernel, d->x, rows, nullptr, d->dyn);
        if (s != SPL_OK) break;
        conv(d->x, L.attention_base, d->xc, 0, 0);
        s = spl_pass_gemm(e, L.q, d->xc, rows, nullptr, d->qp);
        if (s == SPL_OK) s = spl_pass_gemm(e, L.k, d->xc, rows, nullptr, d->kp);
        if (s == SPL_OK) s = spl_pass_gemm(e, L.v, d->xc, rows, nullptr, d->vp);
        if (s != SPL_OK) break;
        draft_kv_store(d, L, d->kp, d->vp, b_slot, b_pos, rows);
        if (G == 1) draft_attention_launch<1>(d, L, rows, count, b_requests, b_slot, b_pos, b_lo, b_hi);
        else if (G == 2) draft_attention_launch<2>(d, L, rows, count, b_requests, b_slot, b_pos, b_lo, b_hi);
        else if (G == 4) draft_attention_launch<4>(d, L, rows, count, b_requests, b_slot, b_pos, b_lo, b_hi);
        else draft_attention_launch<8>(d, L, rows, count, b_requests, b_slot, b_pos, b_lo, b_hi);
        s = spl_pass_gemm(e, L.o, d->ao, rows, nullptr, d->t);
        if (s != SPL_OK) break;
        conv(d->t, L.attention_base, d->dh, 1, 1);
        s = spl_pass_norm(e, d->dh, L.post_norm, rows, H, d->x);
        if (s == SPL_OK) s = spl_pass_gemm(e, L.mlp_kernel, d->x, rows, nullptr, d->dyn);
        if (s != SPL_OK) break;
        conv(d->x, L.mlp_base, d->xc, 0, 0);
        s = spl_pass_mlp_in(e, L.gate, L.up, d->xc, rows, d->gate, d->up);
        if (s == SPL_OK) s = spl_pass_gemm(e, L.down, d->gate, rows, nullptr, d->t);
        if (s != SPL_OK) break;
        conv(d->t, L.mlp_base, d->dh, 1, 1);
    }
    if (s == SPL_OK) s = spl_pass_norm(e, d->dh, d->final_norm, rows, H, d->dn);
    if (s != SPL_OK) return s;
    launch_step(spl_draft_gather_kernel, dim3((H + 255) / 256, picked), dim3(256), 0, e->stream, (const float *)d->dn, b_gather, d->selected, H);
    s = spl_pass_gemm_head(e, d->selected, picked, d->logits);
    if (s != SPL_OK) return s;
    // The candidates of every drafted position: TopK.select over the first `vocab_limit` logits (Sampler.swift:19-52), on the device.
    launch_step(spl_draft_project_kernel, dim3(picked, (c.rank + 31) / 32), dim3(256), 0, e->stream, (const float *)d->projection_dev, (const float *)d->selected, d->projected, int(c.rank), H);
    launch_step(spl_draft_topk_segment_kernel, dim3(picked, d->topk_segments), dim3(256), 0, e->stream, (const float *)d->logits, d->vocab, int(vocab_limit), int(c.candidates),
                d->topk_segments, d->cand_values, d->cand_ids);
    launch_step(spl_draft_topk_merge_kernel, dim3(picked), dim3(256), 0, e->stream, (const float *)d->cand_values, (const int32_t *)d->cand_ids, d->topk_segments * int(c.candidates),
                int(c.candidates), d->top_ids, d->top_values);
    s = check_launch(e, "draft block");
    if (s == SPL_OK) s = spl_pass_wait(e);
    if (s != SPL_OK) return s;
    d->last_picked = picked;
    const int k = c.candidates;
    std::vector<float> values(size_t(picked) * k), projected(size_t(picked) * c.rank);
    SPL_CUDA(cudaMemcpy(candidates, d->top_ids, size_t(picked) * k * 4, cudaMemcpyDeviceToHost));
    SPL_CUDA(cudaMemcpy(values.data(), d->top_values, values.size() * 4, cudaMemcpyDeviceToHost));
    SPL_CUDA(cudaMemcpy(projected.data(), d->projected, projected.size() * 4, cudaMemcpyDeviceToHost));
    for (int i = 0; i < count; ++i) {
        const int first = first_picked[i], drafted = requests[i].block - 1;
        s = draft_select_projected(drafted, k, c.rank, requests[i].anchor, candidates + size_t(first) * k, values.data() + size_t(first) * k, projected.data() + size_t(first) * c.rank,
                                   d->predecessor.data(), d->successor.data(), temperature, random_state, tokens + first, probabilities ? probabilities + size_t(first) * k : nullptr);
        if (s != SPL_OK) return s;
    }
    return SPL_OK;
}

// The last block pass's buffers for tests: 0 logits [picked][vocab], 1 the selected hidden rows [picked][hidden], 2 layer `index`'s
// K ring, 3 its V ring (fp16), 4 the block's residual stream after the last layer [rows][hidden]; 5-11 the last layer's x, xc, dyn, q, attention output, t, gate.
spl_status spl_draft_debug_read(spl_draft *d, int32_t what, int32_t index, void *dst, uint64_t bytes) {
    if (!d || !dst) return SPL_ERR_INVALID_ARGUMENT;
    spl_engine *e = d->e;
    SPL_CUDA(cudaSetDevice(e->device));
    const void *src = nullptr; size_t have = 0;
    const size_t ring = size_t(e->c.max_slots) * d->c.ring_capacity * d->kv * 2;
    switch (what) {
    case 0: src = d->logits; have = size_t(d->last_picked) * d->vocab * 4; break;
    case 1: src = d->selected; have = size_t(d->last_picked) * d->hidden * 4; break;
    case 2: if (index < 0 || index >= d->c.layers) return SPL_ERR_INVALID_ARGUMENT; src = d->layers[index].k_ring; have = ring; break;
    case 3: if (index < 0 || index >= d->c.layers) return SPL_ERR_INVALID_ARGUMENT; src = d->layers[index].v_ring; have = ring; break;
    case 4: src = d->dh; have = size_t(d->block_rows) * d->hidden * 4; break;
    case 5: src = d->x; have = size_t(d->block_rows) * d->hidden * 4; break;
    case 6: src = d->xc; have = size_t(d->block_rows) * d->hidden * 4; break;
    case 7: src = d->dyn; have = size_t(d->block_rows) * 4 * d->groups * 4; break;
    case 8: src = d->qp; have = size_t(d->block_rows) * d->attention * 4; break;
    case 9: src = d->ao; have = size_t(d->block_rows) * d->attention * 4; break;
    case 10: src = d->t; have = size_t(d->block_rows) * d->hidden * 4; break;
    case 11: src = d->gate; have = size_t(d->block_rows) * d->inter * 4; break;
    default: return SPL_ERR_INVALID_ARGUMENT;
    }
    if (bytes > have) return SPL_ERR_INVALID_ARGUMENT;
    SPL_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
    return SPL_OK;
}

}  // extern "C"
