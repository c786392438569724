/* splosh_cuda.h — C ABI of SploshCUDA, the B200 (sm_100a) implementation of Splosh's packed
 * ragged step.
 *
 * The reference has no C ABI: its Swift `Engine` class calls Metal directly. Each entry point
 * below names the Swift interface it stands in for (paths are relative to the reference's
 * repository root), so that a Swift `Engine` facade can forward to it one call for one call.
 *
 * Threading: like the reference's engine ("The engine is not thread-safe; the scheduler owns it
 * and serialises steps", Sources/SploshRuntime/Engine.swift:12) one thread owns an engine.
 * One engine drives one GPU; N GPUs are N engines.
 *
 * All pointers in signatures are HOST pointers unless a name says `device`. Nothing here takes
 * or returns a framework type. There is no CPU fallback: every compute entry point fails with
 * SPL_ERR_UNSUPPORTED_DEVICE when no sm_100 device is present.
 */
#ifndef SPLOSH_CUDA_H
#define SPLOSH_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* EngineError (Engine.swift:88-108) plus the two device conditions Metal reported through
 * CommandGraphError.executionFailed (Sources/SploshCore/CommandGraph.swift:150-152). */
typedef enum spl_status {
    SPL_OK = 0,
    SPL_ERR_KV_POOL_EXHAUSTED = 1,
    SPL_ERR_CONTEXT_EXCEEDED = 2,
    SPL_ERR_UNSUPPORTED_DEVICE = 3,
    SPL_ERR_ALLOCATION_FAILED = 4,
    SPL_ERR_INVALID_ROWS = 5,
    SPL_ERR_SNAPSHOT_MISMATCH = 6,
    SPL_ERR_INVALID_KERNEL_CHOICE = 7,
    SPL_ERR_DEVICE = 8,
    SPL_ERR_TIMEOUT = 9,
    SPL_ERR_INVALID_ARGUMENT = 10
} spl_status;

/* ModelGeometry (Sources/SploshModel/ModelWeights.swift:66-88), a parameter here. Layer i is a
 * gated-attention layer when i % 4 == 3, otherwise a gated-delta layer
 * (Sources/SploshModel/LayerGraph.swift:22). */
typedef struct spl_geometry {
    int32_t layers, hidden, inter, vocab;
    int32_t heads, kv_heads, head_dim, rotary_dim;
    int32_t gdn_key_heads, gdn_value_heads, gdn_head_dim;
    float eps, rope_theta;
} spl_geometry;

/* EngineConfig (Engine.swift:19-48). Zero in state_units / max_logit_rows / span_target takes the
 * default (max_slots * 17, max_rows, 592). */
typedef struct spl_config {
    int32_t device;
    int32_t max_slots, max_rows, kv_pages, max_context;
    int32_t state_units, max_logit_rows;
    int32_t span_target;        /* thread blocks the attention scan aims for; sets the span count */
} spl_config;

/* EngineRow (Engine.swift:50-62). */
typedef struct spl_row {
    int32_t slot, token, position;
    uint8_t want_logits, verify;
    uint8_t reserved[2];
} spl_row;

/* The per-step index tables Engine.step builds on the host (Engine.swift:1322-1398). Arrays are
 * owned by whoever built them and must stay valid for the call they are passed to. */
typedef struct spl_tables {
    uint32_t rows, run_count, logit_rows, attn_block_count, step_pages, live_rows, spans, pages_per_span;
    const uint32_t *tokens, *row_slot, *row_pos;      /* [rows] */
    const uint32_t *runs;                             /* [run_count][3]: slot, first row, length */
    const uint32_t *run_info;                         /* [run_count][2]: speculative, journal pending */
    const uint32_t *row_read, *row_write;             /* [rows]: conv-history unit read / written */
    const uint32_t *gather_index;                     /* [logit_rows] */
    const uint32_t *attn_blocks;                      /* [attn_block_count][2]: first row, count <= 8 */
    const uint32_t *page_table;                       /* [max_slots][max_pages] */
} spl_tables;

/* EngineStepStats (Engine.swift:64-69). */
typedef struct spl_step_stats {
    int32_t rows, launches;
    double gpu_seconds, wall_seconds;
} spl_step_stats;

/* EngineMemory (Engine.swift:71-86). */
typedef struct spl_memory_info {
    int64_t weight_bytes, kv_pool_bytes, kv_bytes_per_page, kv_pages_total, kv_pages_used;
    int64_t state_bytes_per_slot, state_bytes_total, state_units_used, scratch_bytes;
    int64_t device_total_bytes, device_free_bytes;
} spl_memory_info;

/* Tensor kinds of one block (BlockWeights / MixerWeights, ModelWeights.swift:30-63). Layer -1
 * addresses the model-level tensors (embed, head, final norm). */
enum { SPL_Q4_QKV = 0, SPL_Q4_Z, SPL_Q4_A, SPL_Q4_B, SPL_Q4_OUT, SPL_Q4_Q, SPL_Q4_K, SPL_Q4_V, SPL_Q4_O,
       SPL_Q4_GATE, SPL_Q4_UP, SPL_Q4_DOWN, SPL_Q4_EMBED, SPL_Q4_HEAD, SPL_Q4_KINDS };
enum { SPL_VEC_INPUT_NORM = 0, SPL_VEC_POST_NORM, SPL_VEC_CONV, SPL_VEC_A_LOG, SPL_VEC_DT_BIAS, SPL_VEC_GDN_NORM,
       SPL_VEC_Q_NORM, SPL_VEC_K_NORM, SPL_VEC_FINAL_NORM, SPL_VEC_KINDS };

/* ---- Host-side bookkeeping: no GPU needed -------------------------------------------------
 * The page allocator, state-unit pool and table builder that live inside the reference's Engine
 * (Engine.swift:625-632, 810-868, 1316-1398). A Swift host that keeps its own may skip these and
 * hand its tables to spl_step_tables. */
typedef struct spl_host spl_host;
spl_status spl_host_create(const spl_geometry *geometry, const spl_config *config, spl_host **out);
void spl_host_destroy(spl_host *host);
/* Engine.step's validation and table build (Engine.swift:1316-1398). `out` points into the host
 * object and is valid until the next build on it. */
spl_status spl_host_build_tables(spl_host *host, const spl_row *rows, int32_t count, spl_tables *out);
/* The end of Engine.step (Engine.swift:1537): the step's slots have replayed their journals. */
void spl_host_finish_step(spl_host *host, const spl_tables *tables);
/* Engine.resetSlot's host half (Engine.swift:816-826); returns the state unit to be zeroed. */
int32_t spl_host_reset_slot(spl_host *host, int32_t slot);
void spl_host_discard_verify(spl_host *host, int32_t slot);                                   /* Engine.swift:829-832 */
spl_status spl_host_accept_verify(spl_host *host, int32_t slot, int32_t rows, int32_t token_count); /* Engine.swift:836-846 */
void spl_host_truncate(spl_host *host, int32_t slot, int32_t token_count);                    /* Engine.swift:865-868 */
int32_t spl_host_pages_held(const spl_host *host, int32_t slot);                              /* Engine.swift:807 */
int32_t spl_host_free_page_count(const spl_host *host);                                       /* Engine.swift:808 */
int32_t spl_host_slot_unit(const spl_host *host, int32_t slot);
int32_t spl_host_journal_pending(const spl_host *host, int32_t slot);
int32_t spl_host_max_pages(const spl_host *host);
const char *spl_host_last_error(const spl_host *host);
/* BatchScheduler.accept, greedy branch (Sources/SploshRuntime/BatchScheduler.swift:1583-1587):
 * the agreeing prefix of `drafts` against the block's arg-max ids, and the bonus token. */
int32_t spl_greedy_accept(const int32_t *argmax_ids, const int32_t *drafts, int32_t draft_count, int32_t *bonus);
/* ---- Width planner (Sources/SploshRuntime/BatchScheduler.swift:646-669, 735-789) ---------------
 * How many rows a mixed step may hold (prefillCap) and which speculating sessions get a double block
 * (planBlocks). The arithmetic is the reference's; its cost table (tierMilliseconds :740, cycleMilliseconds
 * :743-745, attentionMilliseconds :750, 0.022 :659, 0.88 :779) is an argument: spl_plan_costs_reference fills
 * in the reference's (M5) figures, spl_plan_costs_b200 this library's measured ones. */
typedef struct spl_plan_costs {
    double tier_ms[5];          /* a decode step of up to 16, 32, 64, 96, 128 rows */
    double beyond_ms_per_row;   /* per row past the last tier */
    double per_row_ms, fixed_ms;/* the rest of a cycle: per row, and fixed */
    double attention_first, attention_second;   /* ms per thousand context tokens: a block's first and second eight rows */
    double prefill_attention;   /* ms per prefill row and thousand tokens of its prompt's context */
    double tier_margin;         /* a plan that crosses a tier keeps this fraction of its rate */
} spl_plan_costs;
void spl_plan_costs_reference(spl_plan_costs *costs);
void spl_plan_costs_b200(spl_plan_costs *costs);
int32_t spl_plan_tier(int32_t rows);
double spl_plan_cycle_ms(const spl_plan_costs *costs, int32_t rows);
int32_t spl_plan_prefill_cap(const spl_plan_costs *costs, int32_t max_rows, int32_t decode_rows, double decode_tokens, double decode_attention_ms,
                             double decode_weight, int32_t backlog, int32_t first_fed, int32_t prefill_rows_while_decoding);
int32_t spl_plan_blocks(const spl_plan_costs *costs, int32_t sessions, const double *tail, const double *block_yield, const int32_t *context_tokens,
                        int32_t other_rows, int32_t block, int32_t max_rows, int32_t max_logit_rows, int32_t max_verify_rows, int32_t max_context,
                        int32_t *blocks_out);
/* ---- Row packer (BatchScheduler.buildRows, Sources/SploshRuntime/BatchScheduler.swift:1323-1442) -----------
 * Which rows the next step holds and in which order: verify blocks of the speculating sessions (anchor + proposal, every
 * row wanting logits), then one row for each plainly decoding session, then prompt chunks shortest backlog first under
 * the width prefillCap allows; KV pages are reserved against the host's free pages as rows are taken (:1336-1343), a
 * chunk ends where the session's state is to be kept (:1420-1422) and shrinks to the pages its slot already holds when
 * the pool cannot give more (:1423-1428). What stays with the caller: where proposals come from (the draft model, the
 * lookup index) and which idle slot to evict when memory is short (sessions that sat out are listed in `waiting`). */
typedef struct spl_session {
    int32_t slot, evaluated;            /* tokens already in the slot (slotTokens[slot].count) */
    int32_t pending;                    /* the token waiting to be evaluated; -1 while the prompt is being fed */
    const int32_t *proposal;            /* drafted continuation of a speculating session (BatchScheduler.swift:1395) */
    int32_t proposal_count;
    const int32_t *prompt;              /* request.promptTokens */
    int32_t prompt_count, fed;
    const int32_t *marks;               /* positions where a prefill step must end (stateMarks, diskMarks, turnMark) */
    int32_t mark_count;
    double block_yield;                 /* expected tokens of its verify block (SpeculationState.BlockStats.blockYield) */
} spl_session;
typedef struct spl_pack_config {
    int32_t block;                      /* DraftModel.blockSize */
    int32_t max_verify_rows;            /* BatchScheduler.maxVerifyRows */
    int32_t speculate;                  /* a draft source exists (draft != nil) */
    int32_t prefill_rows_while_decoding;
    double decode_weight;
    const spl_plan_costs *costs;        /* the cost table prefillCap reads */
} spl_pack_config;
enum { SPL_PLAN_VERIFY = 0, SPL_PLAN_DECODE = 1, SPL_PLAN_PREFILL = 2 };
typedef struct spl_planned { int32_t kind, session, count, complete; } spl_planned;   /* count: proposal tokens, or prefill rows */
/* Returns the number of rows written to `rows` (capacity: the engine's max_rows), or -1 on a bad argument. `plan`
 * (capacity: sessions) receives what each packed session does, `waiting` (capacity: sessions) the indices of sessions
 * that sat the step out for want of KV pages. Sessions are given in the scheduler's order (active). */
int32_t spl_host_pack_rows(const spl_host *host, const spl_session *sessions, int32_t session_count, const spl_pack_config *config,
                           spl_row *rows, spl_planned *plan, int32_t *plan_count, int32_t *waiting, int32_t *waiting_count);
/* Sampler (Sources/SploshRuntime/Sampler.swift:68-156), the part after the k largest logits are known
 * (spl_topk gives them): `state` is the sampler's SplitMix64 state, advanced by every draw.
 *   spl_sampler_uniform     Sampler.uniform01 (:79-90)
 *   spl_sample_topk         Sampler.sample (:128-156): temperature softmax over the k values, the smallest
 *                           prefix reaching top_p, one draw; temperature <= 0 returns ids[0]
 *   spl_sampler_distribution Sampler.distribution (:100-116): writes the kept candidates' renormalised
 *                           probabilities, returns how many are kept
 *   spl_speculative_resolve SpeculativeSampling.resolve (:163-179): -1 when the draft is kept, else its replacement */
float spl_sampler_uniform(uint64_t *state);
int32_t spl_sample_topk(const int32_t *ids, const float *values, int32_t k, float temperature, float top_p, uint64_t *state);
int32_t spl_sampler_distribution(const float *values, int32_t k, float temperature, float top_p, float *probabilities);
int32_t spl_speculative_resolve(int32_t draft, const int32_t *candidates, const float *draft_probabilities, int32_t candidate_count,
                                const int32_t *target_ids, const float *target_probabilities, int32_t target_count, uint64_t *state);

/* ---- Engine ------------------------------------------------------------------------------- */
typedef struct spl_engine spl_engine;
/* Engine.init(device:weights:config:) (Engine.swift:355). Weights are set afterwards. */
spl_status spl_engine_create(const spl_geometry *geometry, const spl_config *config, spl_engine **out);
void spl_engine_destroy(spl_engine *engine);
const char *spl_last_error_string(const spl_engine *engine);
/* Q4Handle (Sources/SploshCore/Allocator.swift:34-88): MLX affine-4, group 64, row-major packed
 * u32 [rows][inner/8] with bf16 scales and biases [rows][inner/64]. The caller keeps ownership of
 * the host arrays; the engine copies them into its own device layout before returning.
 * The tensor cores hold scale * (code - 8), 512 * scale and 64 * bias exactly in fp16: a tensor with a
 * non-zero scale outside [2^-13, 127] or a bias beyond 1023 in magnitude is refused
 * (SPL_ERR_INVALID_ARGUMENT), not approximated. */
spl_status spl_weights_set_q4(spl_engine *engine, int32_t layer, int32_t kind, int32_t rows, int32_t inner,
                              const uint32_t *packed, const uint16_t *scales, const uint16_t *biases);
/* TensorHandle for the bf16 vectors (norm weights, conv1d, A_log, dt_bias). */
spl_status spl_weights_set_vector(spl_engine *engine, int32_t layer, int32_t kind, const uint16_t *bf16, int32_t count);
/* Benchmarking: fill every q4 tensor on the device from the seeded streams the synthetic-model
 * recipe defines (value n of tensor `name` = centred sum of the four 16-bit fields of
 * SplitMix64(seed ^ fnv1a64(name), n), scaled to deviation 0.02, then quantised group by group). */
spl_status spl_weights_synthesize_q4(spl_engine *engine, uint64_t seed);
/* A GGUF-weighted model (the GGUF branch of Engine.gemm, Sources/SploshRuntime/Engine.swift:1666-1695; tensors as
 * Sources/SploshModel/GgufConvert.swift:1-33 leaves them): one tensor as native K-quant super-blocks
 * [rows][inner / 256][144, 176 or 210 bytes], `type` the GGUF type number 12 (Q4_K), 13 (Q5_K) or 14 (Q6_K), `kind`
 * and `layer` as for spl_weights_set_q4 (SPL_Q4_EMBED and SPL_Q4_HEAD with layer -1). The engine copies. Tensors that
 * share a device tensor (qkv, z, a, b; q, k, v; gate, up) must share a type. Once the head is GGUF the engine steps as
 * a GGUF-weighted model and wants every GEMM tensor and the embedding as GGUF: its GEMMs form weights as the
 * reference's tile kernels do (one fp32 operation, rounded to fp16, Sources/Shaders/gguf_formats.h:390-438), the
 * embedding gather decodes exactly (:463-501), norms are plain RMSNorms and the SiLU gate a kernel of its own.
 * Device memory: Q4_K byte for byte; Q5_K and Q6_K tensors are kept at one byte a code (272 and 288 bytes a
 * super-block), so the GEMMs form a weight without extracting its bits anew every step. */
spl_status spl_weights_set_gguf(spl_engine *engine, int32_t layer, int32_t kind, int32_t type, int32_t rows, int32_t inner, const uint8_t *blocks);
/* A GGUF file orders the value heads of a gated-delta block differently from the engine (file head i = engine head
 * 3 (i % 16) + i / 16 for 48 value and 16 key heads, Sources/SploshModel/GgufNames.swift:73-84). Tensors that hold the heads
 * as rows are re-ordered when they are loaded; the out projection holds them as columns, which cannot move without
 * re-quantising, so it is given in the file's order (Sources/SploshModel/GgufConvert.swift:18-24) and, with this switch on,
 * the gated-delta blocks write their outputs in that order, as the reference's `heads` kernels read them
 * (Sources/Shaders/engine_gguf.metal). Off by default. */
spl_status spl_weights_gguf_file_order(spl_engine *engine, int32_t enabled);
/* A llama.cpp GGUF file (versions 2 and 3) of a model of the engine's geometry into the engine: the reference's reader and
 * converter of such a file (Sources/SploshModel/GgufFile.swift, GgufNames.swift:13-44, GgufConvert.swift:15-32) with the
 * engine as its destination. Packed weights Q4_K / Q5_K / Q6_K, dense tensors F32 / F16 / BF16 (rounded to bf16, nearest
 * even); value heads re-ordered where they are rows, channels or elements, the out projection left in file order with
 * spl_weights_gguf_file_order switched on; ssm_a (-exp(A_log)) turned into A_log; an MTP block left out; a file without
 * output.weight ties the head to the embedding. `message` (may be null) receives what was wrong with the file. */
spl_status spl_weights_load_gguf_file(spl_engine *engine, const char *path, char *message, size_t message_bytes);
/* An SPLW artifact, the reference's own weight container (Sources/SploshModel/WeightFile.swift:88-141, Converter.swift:46-82),
 * of a model of the engine's geometry into the engine: the tensors of ModelWeights.resolve (Sources/SploshModel/ModelWeights.swift:181-248)
 * under "language_model.", each checked against the geometry. Formats "mlxAffine4" (row-major triplets) and
 * "mlxAffine4.tiled128" (Sources/SploshModel/Retile.swift: eligible triplets in tiles of 128 rows, put back in rows on the
 * way), and the GGUF-derived "gguf.tiled128" (Sources/SploshModel/GgufConvert.swift:1-33: every 2-D weight as three planes,
 * put back into native Q4_K / Q5_K / Q6_K blocks; the out projections in file order, so spl_weights_gguf_file_order is
 * switched on); 8-bit packs are refused with a message. `message` (may be null)
 * receives what was wrong with the file, in the reference's words where it has them. */
spl_status spl_weights_load_splw_file(spl_engine *engine, const char *path, char *message, size_t message_bytes);
/* GgufPlanes.unpack (Sources/SploshModel/GgufPlanes.swift:150-190): the three planes of a Q4_K (12), Q5_K (13) or Q6_K (14)
 * weight, each in tiles of 128 rows (planes of rows rounded up to 128), back into native blocks [rows][inner / 256][144, 176
 * or 210 bytes]. `plane1` may be null for Q4_K. Host code. */
spl_status spl_gguf_planes_unpack(int32_t type, const uint8_t *plane0, const uint8_t *plane1, const uint8_t *meta, int32_t rows, int32_t inner, uint8_t *native);
/* The container's own checks without an engine or a GPU (framing, header, quantization, alignment, every record's bounds,
 * order, alignment and padding, no unaccounted bytes): SPL_OK with the header's format in `message` and the record count in
 * `tensors` (may be null), or SPL_ERR_INVALID_ARGUMENT with the reason. */
spl_status spl_splw_check(const char *path, int32_t *tensors, char *message, size_t message_bytes);
spl_status spl_engine_geometry(const spl_engine *engine, spl_geometry *out);
/* Benchmarking: pseudo-random GGUF blocks for every tensor (`block_type`) and for the embedding and head
 * (`head_type`), generated on the device. */
spl_status spl_weights_synthesize_gguf(spl_engine *engine, uint64_t seed, int32_t block_type, int32_t head_type);
/* Engine.step(_:) (Engine.swift:1316): validate, build tables with the engine's own host state,
 * run the pass, wait. */
spl_status spl_step(spl_engine *engine, const spl_row *rows, int32_t count, spl_step_stats *stats);
/* The same pass from tables the caller built (the north star's split: packer and allocator stay
 * with the host language). */
spl_status spl_step_tables(spl_engine *engine, const spl_tables *tables, spl_step_stats *stats);

/* Engine.step in two halves (Sources/SploshRuntime/Engine.swift:1316 commits its command graph and waits for it in
 * one call; a host that wants to pack the next step's rows or sample while the GPU runs uses the halves). spl_step_launch
 * validates and packs the rows, copies the tables and enqueues every kernel of the step, then returns;
 * spl_step_wait waits for them and returns the step's status and statistics, after which logits, arg-max and the
 * slot calls see the step. Exactly one spl_step_wait per successful spl_step_launch; no other call on the engine
 * in between (SPL_ERR_INVALID_ARGUMENT otherwise). spl_step is the two in a row. */
spl_status spl_step_launch(spl_engine *engine, const spl_row *rows, int32_t count);
spl_status spl_step_wait(spl_engine *engine, spl_step_stats *stats);
/* Engine.logits(_:) (Engine.swift:1202-1205): row i of the last step's logits, vocab floats. */
spl_status spl_logits_row(spl_engine *engine, int32_t index, float *dst);
/* Sampler.argmax over [0, vocab_limit) for every logit row of the last step, on the device
 * (Sources/SploshRuntime/Sampler.swift:11-16, 94-96): the first index of the maximum. */
spl_status spl_argmax(spl_engine *engine, int32_t vocab_limit, int32_t *ids);
/* TopK.select (Sampler.swift:19-52) for every logit row of the last step: the k <= 64 largest of [0, vocab_limit) in
 * descending order, the lower index first among equal values; ids and values [logit rows][k] on the host. Rows with
 * fewer than k values above -inf end in (0, -inf) entries, as the reference's untouched slots do. */
spl_status spl_topk(spl_engine *engine, int32_t vocab_limit, int32_t k, int32_t *ids, float *values);
spl_status spl_slot_reset(spl_engine *engine, int32_t slot);                                  /* Engine.resetSlot */
spl_status spl_verify_discard(spl_engine *engine, int32_t slot);                              /* Engine.discardVerify */
spl_status spl_verify_accept(spl_engine *engine, int32_t slot, int32_t rows, int32_t token_count); /* Engine.acceptVerify */
spl_status spl_slot_truncate(spl_engine *engine, int32_t slot, int32_t token_count);          /* Engine.truncate */
int32_t spl_pages_held(const spl_engine *engine, int32_t slot);                               /* Engine.pagesHeld(by:) */
int32_t spl_free_page_count(const spl_engine *engine);                                        /* Engine.freePageCount */
spl_status spl_memory(const spl_engine *engine, spl_memory_info *out);                        /* Engine.memory */
spl_host *spl_engine_host(spl_engine *engine);
/* Engine.warmUp (Engine.swift:1191-1197): a full-width step and a one-row step on slot 0, so that the first real request
 * does not pay for module loading and first touches; slot 0 is left empty. */
spl_status spl_warmup(spl_engine *engine);
/* Engine.debugFillKV (Engine.swift:1218-1236): pseudo-random codes and scale 0.01 in every page
 * the slot holds; and a U(-0.5, 0.5) recurrent state as the reference's tests draw it
 * (Tests/SploshOracleTests/GdnCandidateTests.swift:146). */
spl_status spl_debug_fill_kv(spl_engine *engine, int32_t slot);
spl_status spl_debug_fill_state(spl_engine *engine, int32_t slot, uint64_t seed);
/* Raw device buffers for tests. which: 0 state, 1 conv history, 2 journal (index = gated-delta
 * layer ordinal); 3 k codes, 4 v codes, 5 k scale, 6 v scale (index = attention layer ordinal);
 * 7 residual stream after the last step [rows][hidden]; 8 residual stream after block `index`
 * (needs spl_debug_taps(engine, 1) before the step); 9 the last block's fused input projection
 * [rows][ld] fp32; 10 its mixer output [rows][ld] bf16; 11 its queries [rows][heads][head_dim] fp16;
 * 12 its attention partials [rows][heads][spans][head_dim + 2] fp32. Layouts: state [slot][value head][value j][key i];
 * conv [unit][channel][3] oldest first; journal [slot][16][value head][260];
 * codes [page][kv head][256][head_dim] (V codes are stored [page][kv head][head_dim][256]). */
spl_status spl_debug_read(spl_engine *engine, int32_t which, int32_t index, void *dst, size_t bytes);
spl_status spl_debug_taps(spl_engine *engine, int32_t enabled);
/* Test switch: with `enabled` 0 the following steps do not store their rows' keys and values, so the attention scan
 * reads the pool exactly as a test wrote it, the rows' own positions included (the scenes of
 * Tests/SploshOracleTests/AttentionScanCandidateTests.swift:85-200 place large keys there). 1 restores the store. */
/* Tests: ordinary runs of at least `rows` rows (>= 64; default 512) take the chunked gated-delta scan instead of the
 * per-token kernel. */
spl_status spl_debug_gdn_chunk_min(spl_engine *engine, int32_t rows);
/* Tests and measurements: with `enabled` 0 the GEMMs of steps of more than 64 rows run on the 128-row block that works on
 * one tile of the weight, instead of the pair form that works on two against one stream of activations (process-wide,
 * `engine` may be null; default 1). */
spl_status spl_debug_pair_blocks(spl_engine *engine, int32_t enabled);
spl_status spl_debug_kv_store(spl_engine *engine, int32_t enabled);
/* Every wait inside a kernel (a role of a block waiting for another role of the same block) gives up after a time
 * budget, 250 ms unless changed here, and the step then returns SPL_ERR_TIMEOUT with the engine still usable.
 * spl_debug_drop_weight_stage is the test of that path: the q4 GEMM's weight-copy role leaves out stage `stage` of
 * every block's piece (a stage nothing delivers), -1 switches it off. Both settings hold for every engine on the
 * engine's device until changed. */
spl_status spl_debug_wait_budget(spl_engine *engine, int64_t nanoseconds);
spl_status spl_debug_drop_weight_stage(spl_engine *engine, int32_t stage);

/* ---- Slot snapshots ------------------------------------------------------------------------
 * exportState / importState (Engine.swift:871-939) and exportKV / kvPrefix / importSlot's KV part (:953-1042), as two
 * opaque, versioned blobs on host memory. The state blob is the slot's recurrent state of every gated-delta block,
 * accepted journal entries folded in first (Engine.commitJournal, :889-903), with the conv history of its current
 * unit. The KV blob is the pages covering the slot's first `token_count` tokens in every attention block; KV is
 * append-only, so it is valid for any prefix of what the slot has evaluated, and importing fewer tokens than a blob
 * holds takes the prefix (kvPrefix). A blob of another geometry or layout is refused with SPL_ERR_SNAPSHOT_MISMATCH
 * (EngineError.snapshotMismatch). Import leaves the slot holding exactly the imported pages and no pending journal. */
size_t spl_state_bytes(const spl_engine *engine);
spl_status spl_state_export(spl_engine *engine, int32_t slot, void *dst, size_t capacity);
spl_status spl_state_import(spl_engine *engine, int32_t slot, const void *src, size_t bytes);
size_t spl_kv_bytes(const spl_engine *engine, int32_t token_count);
spl_status spl_kv_export(spl_engine *engine, int32_t slot, int32_t token_count, void *dst, size_t capacity);
spl_status spl_kv_import(spl_engine *engine, int32_t slot, int32_t token_count, const void *src, size_t bytes);

/* ---- Drafter feature taps ------------------------------------------------------------------
 * step(_:captureFeatures:) and featureRow(_:) (Engine.swift:1316, 1309-1313; taps at
 * Engine.featureLayers = [5, 19, 33, 47, 61], Engine.swift:331, copied by sp_copy_rows :1488-1497):
 * while enabled, every step leaves the residual stream after each listed block as
 * [row][tap][hidden] fp32. `layers` null with count > 0 selects the reference's list; blocks the
 * geometry does not have are left out; count 0 disables. The last block is computed for the rows
 * that want logits only, so a tap on it holds those rows (the reference keeps every row there). */
spl_status spl_features_enable(spl_engine *engine, const int32_t *layers, int32_t count);
/* Floats of one row: taps in use x hidden. */
int32_t spl_feature_width(const spl_engine *engine);
/* Engine.featureRow: the taps of row `row` of the last step, copied to the host. */
spl_status spl_feature_row(spl_engine *engine, int32_t row, float *dst);
/* Per-kernel-class device time of the last step when enabled (events around every launch; slow). */
spl_status spl_debug_profile(spl_engine *engine, int32_t enabled);
/* class: 0 q4 gemm, 1 norms and elementwise, 2 gated-delta, 3 attention, 4 head/argmax/other.
 * Returns accumulated milliseconds and launches since the last reset (reset = enabling). */
spl_status spl_debug_profile_read(spl_engine *engine, int32_t klass, double *milliseconds, int64_t *launches, double *bytes);

/* ---- The engine's primitives on device buffers ------------------------------------------------
 * DraftModel builds its own passes out of Engine.gemm / norm / mlpIn / embed on buffers it owns and reuses the target's
 * lm_head (Sources/SploshRuntime/DraftModel.swift:344-357, 418-468; Engine.swift:1561-1625, 1905-1998). Here: tensors of
 * the caller's own (spl_tensor_create_*), calls that queue work on the engine's stream over DEVICE pointers the caller
 * owns (fp32 rows, row-major), and spl_pass_wait as the pass's commitAndWait. Rows per call: at most the engine's
 * max_rows; a tensor's inner dimension: a multiple of 256, at most the engine's MLP width. Not between spl_step_launch
 * and spl_step_wait. The calls use the engine's operand scratch, so one pass at a time per engine. */
typedef struct spl_tensor spl_tensor;
spl_status spl_tensor_create_q4(spl_engine *engine, int32_t rows, int32_t inner, const uint32_t *packed, const uint16_t *scales,
                                const uint16_t *biases, spl_tensor **out);                  /* rows a multiple of 16 */
spl_status spl_tensor_create_vector(spl_engine *engine, const uint16_t *bf16, int32_t count, spl_tensor **out);
void spl_tensor_destroy(spl_engine *engine, spl_tensor *tensor);
spl_status spl_pass_begin(spl_engine *engine);
/* Engine.gemm: out[r][:] = w x in[r][:] (+ residual[r][:]); in [rows][inner], out and residual [rows][w rows]. */
spl_status spl_pass_gemm(spl_engine *engine, const spl_tensor *weight, const float *device_in, int32_t rows, const float *device_residual, float *device_out);
/* The target's lm_head: in [rows][hidden] -> out [rows][vocab]. */
spl_status spl_pass_gemm_head(spl_engine *engine, const float *device_in, int32_t rows, float *device_out);
/* Engine.norm: out = in * rsqrt(mean in^2 + eps) * weight, fp32 rows of `dim`. */
spl_status spl_pass_norm(spl_engine *engine, const float *device_in, const spl_tensor *weight, int32_t rows, int32_t dim, float *device_out);
/* Engine.embed: rows of the target's embedding table for `device_tokens` (uint32 on the device). */
spl_status spl_pass_embed(spl_engine *engine, const uint32_t *device_tokens, int32_t rows, float *device_out);
/* Engine.mlpIn: out = bf16(silu(gate x in) * (up x in)) as fp32 rows; scratch [rows][gate rows] holds up x in. */
spl_status spl_pass_mlp_in(spl_engine *engine, const spl_tensor *gate, const spl_tensor *up, const float *device_in, int32_t rows, float *device_out, float *device_scratch);
spl_status spl_pass_wait(spl_engine *engine);

/* ---- The DFlash 2 block-diffusion drafter (Sources/SploshRuntime/DraftModel.swift) -----------------
 * A draft pass proposes a whole block at once: [anchor, mask x (block - 1)] through a few non-causal layers that attend
 * over the block and a sliding window of context made from the target's hidden states at its tap layers
 * (spl_features_enable), then a selector traces one path through the top candidates of every position. Built from the
 * primitives above plus the drafter's own kernels (Sources/Shaders/draft.metal: dynamic convolution, K/V ring store,
 * windowed attention). Heads are 128 wide. The checkpoint's linear layers are quantised to MLX affine-4 on the way in
 * (DraftModel.quantize, :635-727; `minmax_ranges` non-zero restores MLX's range rule, SPLOSH_DRAFT_QUANT=minmax there). */
typedef struct spl_draft spl_draft;
typedef struct spl_draft_config {
    int32_t layers, heads, kv_heads;          /* 5, 32, 8 in the reference's checkpoint */
    int32_t group_size;                       /* channels per dynamic-convolution group: 16 (hidden / 16 groups) */
    int32_t rank;                             /* the selector's codebook width: 256 */
    int32_t window, ring_capacity;            /* 2048; ring positions per slot: 2304 (>= window + max_block) */
    int32_t block_size, max_block;            /* 8; 16 */
    int32_t candidates;                       /* 16 */
    int32_t mask_token;                       /* 248070 */
    int32_t minmax_ranges;
} spl_draft_config;
typedef struct spl_draft_request { int32_t slot, anchor, start, block, isolate_prefix; } spl_draft_request;      /* DraftRequest (:29-42) */
typedef struct spl_draft_context_entry { int32_t slot, position, engine_row; } spl_draft_context_entry;
/* Needs the engine's feature taps enabled and max_slots * max_block <= max_rows. */
spl_status spl_draft_create(spl_engine *engine, const spl_draft_config *config, spl_draft **out);
void spl_draft_destroy(spl_draft *draft);
/* One tensor of the checkpoint by its safetensors name (DraftModel.swift:172-203: "layers.N.self_attn.q_proj.weight",
 * "fc.weight", "norm.weight", "candidate_selector.predecessor_codebook", ...), bf16 [rows][inner]. The draft copies. */
spl_status spl_draft_set_tensor(spl_draft *draft, const char *name, const uint16_t *bf16, int32_t rows, int32_t inner);
spl_status spl_draft_reset_slot(spl_draft *draft, int32_t slot);
spl_status spl_draft_truncate(spl_draft *draft, int32_t slot, int32_t token_count);
int32_t spl_draft_context_length(const spl_draft *draft, int32_t slot, int32_t start);
/* DraftModel.pushContext: straight after an engine step, the step rows to fold into the context and their positions. */
spl_status spl_draft_push_context(spl_draft *draft, const spl_draft_context_entry *entries, int32_t count);
/* DraftModel.propose. Outputs request after request, a request's block - 1 drafted positions in order: tokens [drafted],
 * candidates [drafted][candidates], probabilities [drafted][candidates] (temperature > 0; may be null otherwise).
 * `random_state` is the selector's SplitMix64 state, advanced by every draw. */
spl_status spl_draft_propose(spl_draft *draft, const spl_draft_request *requests, int32_t count, float temperature, int32_t vocab_limit,
                             uint64_t *random_state, int32_t *tokens, int32_t *candidates, float *probabilities);
/* Host arithmetic, no device: DraftModel.quantize on row-major bf16 [rows][inner] (inner a multiple of 64), and
 * CandidateSelector.select (:479-531) for one request: ids and values [drafted][k] are the top candidates of every
 * position, hidden_rows [drafted][hidden] the draft's final hidden states, codebooks bf16 [vocab][rank]. */
spl_status spl_draft_quantize_q4(const uint16_t *bf16, int32_t rows, int32_t inner, int32_t fitted, uint32_t *packed, uint16_t *scales, uint16_t *biases);
spl_status spl_draft_select(int32_t drafted, int32_t k, int32_t rank, int32_t hidden, int32_t anchor, const int32_t *ids, const float *values,
                            const float *hidden_rows, const float *hidden_projection, const uint16_t *predecessor, const uint16_t *successor,
                            float temperature, uint64_t *random_state, int32_t *tokens, float *probabilities);
/* The checkpoint as the reference reads it: a bf16 safetensors file (MappedFile / SafetensorsHeader, DraftModel.swift:742-794).
 * The file is mapped read-only for the call; refusals say why in `message` ("missing tensor <name>", "<name> is F16 [..];
 * expected BF16 [..]", "bad safetensors header", ...). spl_draft_tensor_count / _expected list what the drafter asks for. */
spl_status spl_draft_load_safetensors(spl_draft *draft, const char *path, char *message, size_t message_bytes);
int32_t spl_draft_tensor_count(const spl_draft *draft);
spl_status spl_draft_tensor_expected(const spl_draft *draft, int32_t index, char *name, uint64_t name_bytes, int64_t *shape, int32_t *dimensions);
/* DraftModel.exportContext / importContext (:285-311): a slot's K and V rings (spl_draft_context_bytes of them, layer by
 * layer, K then V, fp16) and the range [first, end) of positions valid in them for a prefix of `token_count` tokens.
 * *first < 0 after an export: nothing useful is held (the reference's nil). A snapshot of another size resets the slot. */
uint64_t spl_draft_context_bytes(const spl_draft *draft);
spl_status spl_draft_export_context(spl_draft *draft, int32_t slot, int32_t token_count, int32_t *first, int32_t *end, void *rings);
spl_status spl_draft_import_context(spl_draft *draft, int32_t slot, int32_t first, int32_t end, const void *rings, uint64_t bytes);
/* For tests: the last block pass's buffers. 0 logits [picked][vocab], 1 selected hidden rows [picked][hidden], 2 / 3 layer
 * `index`'s K / V ring (fp16), 4 the block's residual stream after the last layer. */
spl_status spl_draft_debug_read(spl_draft *draft, int32_t what, int32_t index, void *dst, uint64_t bytes);

/* ---- A GEMM for callers that must not allocate ---------------------------------------------
 * No counterpart in the reference (Metal hands out buffers freely; nothing there is barred from
 * allocating). Some CUDA hosts are: one that gave the whole GPU to its own pool at start-up and has
 * nothing left for cudaMalloc to hand out, or a serving loop that bans allocator calls on its hot
 * path because cudaMalloc and cudaFree synchronise the whole device.
 * This entry point runs out[r][:] = GEMM(weights, activations[r][:]) (+ residual) on one of the
 * engine's resident weights and calls no cudaMalloc, cudaFree or other allocating routine: the
 * GEMM operand, its per-64 sums, the partial sums of a cut contraction and the calls' error words live in a
 * static device array of about 12.3 MiB that every GPU loading the library holds until exit.
 *   - all three buffers are DEVICE pointers: activations fp32 [rows][inner], residual (may be
 *     null, may alias out) and out fp32 [rows][ld], ld = the tensor's columns rounded up to 16;
 *   - rows must be 1..64 and the tensor's inner dimension at most 17408, else SPL_ERR_INVALID_ROWS
 *     / SPL_ERR_INVALID_ARGUMENT with the reason in spl_last_error_string;
 *   - the first call on a device looks up the array's address (cudaGetSymbolAddress); make that
 *     call before any stream capture begins;
 *   - work is queued on `stream` (a cudaStream_t, null for the default stream) and not waited for;
 *   - every call on a device shares the one array: two calls whose kernels can overlap on the GPU
 *     (different streams, no dependency between them) race on it. */
enum { SPL_RESIDENT_IN_PROJ = 0, SPL_RESIDENT_OUT_PROJ, SPL_RESIDENT_GATE_UP, SPL_RESIDENT_DOWN, SPL_RESIDENT_HEAD };
spl_status spl_gemm_q4_static(spl_engine *engine, int32_t layer, int32_t which, const float *device_activations, int32_t rows,
                              const float *device_residual, float *device_out, void *stream);
/* The static array also holds the error word of those calls. After the caller has synchronised the stream they were
 * queued on, this returns SPL_ERR_TIMEOUT when a block of one of them gave up a wait (its output is then incomplete),
 * SPL_OK otherwise. It allocates nothing. No counterpart in the reference. */
spl_status spl_gemm_q4_static_status(spl_engine *engine);

/* ---- Single operators on host buffers (tests, micro-benchmarks) --------------------------- */
/* Engine.gemm (Engine.swift:1651-1806) for one MLX affine-4 tensor: out[r][n] = sum_k
 * bf16(a[r][k]) * w[n][k] (+ residual[r][n]). Allocates, copies in, runs, copies out. */
spl_status spl_op_gemm_q4(int32_t device, const uint32_t *packed, const uint16_t *scales, const uint16_t *biases,
                          int32_t n, int32_t k, const float *activations, int32_t rows, const float *residual, float *out);

/* Engine.gemm's GGUF branch (Engine.swift:1666-1695; kernels Sources/Shaders/engine_gguf.metal:82-273) for one K-quant
 * tensor: blocks = native GGUF super-blocks of 256, row-major [n][k / 256][144 | 176 | 210 bytes], format = the GGUF
 * type number (12 Q4_K, 13 Q5_K, 14 Q6_K). out[r][n] = sum_k bf16(a[r][k]) * w16[n][k] (+ residual[r][n]) with each
 * weight rounded once to fp16 from fma(code, d * scale, -dmin * minimum) (Q4_K, Q5_K) or (code - 32) * (d * scale)
 * (Q6_K), as the reference's tile kernels form it (Sources/Shaders/gguf_formats.h:390-438). */
spl_status spl_op_gemm_gguf(int32_t device, int32_t format, const uint8_t *blocks, int32_t n, int32_t k, const float *activations,
                            int32_t rows, const float *residual, float *out);

#ifdef __cplusplus
}
#endif
#endif
