// spl_host.cpp — the host-side bookkeeping of a step: paged-KV block allocator, state-unit pool,
// row validation and the per-step index tables. Plain C++; nothing here touches the GPU.
//
// In the reference this lives inside Engine (Sources/SploshRuntime/Engine.swift:625-632 free lists,
// :810-868 slot lifecycle, :1316-1398 the table build at the top of step()). Page ids come off the
// end of a free list that starts reversed, so a fresh engine hands out ascending ids and freed
// pages are reused last-in first-out; slot i starts on state unit i and speculative rows take
// fresh units from max_slots upward.
#include "spl_host.h"
#include <cmath>
#include <algorithm>

#include <algorithm>
#include <cstdio>
#include <set>

static constexpr int kPageTokens = 256;
static constexpr int kJournalRows = 16;
static constexpr int kAttnBlockRows = 8;

spl_host::spl_host(const spl_geometry &g, const spl_config &c) : geometry(g), config(c) {
    if (config.state_units <= 0) config.state_units = config.max_slots * (kJournalRows + 1);
    if (config.max_logit_rows <= 0) config.max_logit_rows = config.max_rows;
    if (config.span_target <= 0) config.span_target = 592;
    max_pages = (config.max_context + kPageTokens - 1) / kPageTokens;
    for (int p = config.kv_pages - 1; p >= 0; --p) free_pages.push_back(uint32_t(p));
    slot_pages.assign(config.max_slots, {});
    slot_unit.resize(config.max_slots);
    for (int s = 0; s < config.max_slots; ++s) slot_unit[s] = uint32_t(s);
    for (int u = config.state_units - 1; u >= config.max_slots; --u) free_units.push_back(uint32_t(u));
    pending_verify.assign(config.max_slots, {});
    journal_pending.assign(config.max_slots, 0);
    page_table.assign(size_t(config.max_slots) * max_pages, 0);
}

int32_t spl_host::reset_slot(int slot) {
    free_pages.insert(free_pages.end(), slot_pages[slot].begin(), slot_pages[slot].end());
    slot_pages[slot].clear();
    discard_verify(slot);
    journal_pending[slot] = 0;
    return int32_t(slot_unit[slot]);
}

void spl_host::discard_verify(int slot) {
    free_units.insert(free_units.end(), pending_verify[slot].begin(), pending_verify[slot].end());
    pending_verify[slot].clear();
}

spl_status spl_host::accept_verify(int slot, int rows, int token_count) {
    std::vector<uint32_t> &units = pending_verify[slot];
    if (rows < 1 || rows > int(units.size())) return fail(SPL_ERR_INVALID_ARGUMENT, "acceptVerify outside the verified run");
    free_units.push_back(slot_unit[slot]);
    slot_unit[slot] = units[rows - 1];
    for (int i = 0; i < int(units.size()); ++i) if (i != rows - 1) free_units.push_back(units[i]);
    units.clear();
    journal_pending[slot] = uint32_t(rows);
    truncate(slot, token_count);
    return SPL_OK;
}

void spl_host::truncate(int slot, int token_count) {
    const size_t keep = size_t((token_count + kPageTokens - 1) / kPageTokens);
    while (slot_pages[slot].size() > keep) { free_pages.push_back(slot_pages[slot].back()); slot_pages[slot].pop_back(); }
}

spl_status spl_host::ensure_page(int slot, int position) {
    if (position >= config.max_context) {
        char text[96]; snprintf(text, sizeof text, "position %d exceeds the context limit %d", position, config.max_context);
        return fail(SPL_ERR_CONTEXT_EXCEEDED, text);
    }
    const size_t index = size_t(position / kPageTokens);
    while (slot_pages[slot].size() <= index) {
        if (free_pages.empty()) {
            char text[96]; snprintf(text, sizeof text, "KV pool exhausted: need %d page(s), 0 free", int(index + 1 - slot_pages[slot].size()));
            return fail(SPL_ERR_KV_POOL_EXHAUSTED, text);
        }
        const uint32_t page = free_pages.back(); free_pages.pop_back();
        page_table[size_t(slot) * max_pages + slot_pages[slot].size()] = page;
        slot_pages[slot].push_back(page);
    }
    return SPL_OK;
}

spl_status spl_host::fail(spl_status code, const std::string &text) { error = text; return code; }

spl_status spl_host::build(const spl_row *rows, int count, spl_tables *out) {
    if (count <= 0 || count > config.max_rows) {
        char text[64]; snprintf(text, sizeof text, "invalid step rows: %d rows; limit %d", count, config.max_rows);
        return fail(SPL_ERR_INVALID_ROWS, text);
    }
    for (int i = 0; i < count; ++i)
        if (rows[i].verify && rows[i].slot >= 0 && rows[i].slot < config.max_slots) discard_verify(rows[i].slot);
    int max_position = 0;
    for (int i = 0; i < count; ++i) max_position = std::max(max_position, rows[i].position);
    const uint32_t step_pages = uint32_t(max_position / kPageTokens + 1);
    // Attention blocks: up to eight consecutive rows of one slot.
    attn_blocks.clear();
    for (int index = 0; index < count;) {
        int length = 1;
        while (length < kAttnBlockRows && index + length < count && rows[index + length].slot == rows[index].slot) ++length;
        attn_blocks.push_back(uint32_t(index)); attn_blocks.push_back(uint32_t(length));
        index += length;
    }
    tokens.assign(count, 0); row_slot.assign(count, 0); row_pos.assign(count, 0);
    row_read.assign(count, 0); row_write.assign(count, 0);
    runs.clear(); run_info.clear(); gather_index.clear();
    std::set<int> seen;
    char text[128];
    for (int index = 0; index < count; ++index) {
        const spl_row &row = rows[index];
        if (row.slot < 0 || row.slot >= config.max_slots || row.token < 0 || row.token >= geometry.vocab) {
            snprintf(text, sizeof text, "invalid step rows: row %d out of range", index);
            return fail(SPL_ERR_INVALID_ROWS, text);
        }
        if (row.position < 0) return fail(SPL_ERR_INVALID_ROWS, "invalid step rows: negative position");
        const spl_status paged = ensure_page(row.slot, row.position);
        if (paged != SPL_OK) return paged;
        tokens[index] = uint32_t(row.token); row_slot[index] = uint32_t(row.slot); row_pos[index] = uint32_t(row.position);
        // State units: in place for ordinary rows, a fresh unit per speculative row.
        const uint32_t previous = pending_verify[row.slot].empty() ? slot_unit[row.slot] : pending_verify[row.slot].back();
        row_read[index] = previous;
        if (row.verify) {
            if (free_units.empty()) return fail(SPL_ERR_INVALID_ROWS, "invalid step rows: state unit pool exhausted");
            const uint32_t unit = free_units.back(); free_units.pop_back();
            pending_verify[row.slot].push_back(unit);
            row_write[index] = unit;
        } else {
            if (!pending_verify[row.slot].empty()) {
                snprintf(text, sizeof text, "invalid step rows: ordinary row after speculative rows in slot %d", row.slot);
                return fail(SPL_ERR_INVALID_ROWS, text);
            }
            row_write[index] = previous;
        }
        if (index > 0 && rows[index - 1].slot == row.slot) {
            if (row.position != rows[index - 1].position + 1) {
                snprintf(text, sizeof text, "invalid step rows: slot %d positions are not consecutive", row.slot);
                return fail(SPL_ERR_INVALID_ROWS, text);
            }
            if (bool(row.verify) != bool(rows[index - 1].verify)) {
                snprintf(text, sizeof text, "invalid step rows: slot %d mixes speculative and ordinary rows", row.slot);
                return fail(SPL_ERR_INVALID_ROWS, text);
            }
            runs[runs.size() - 1] += 1;
            if (row.verify && runs.back() > uint32_t(kJournalRows)) {
                snprintf(text, sizeof text, "invalid step rows: more than %d speculative rows in slot %d", kJournalRows, row.slot);
                return fail(SPL_ERR_INVALID_ROWS, text);
            }
        } else {
            if (!seen.insert(row.slot).second) {
                snprintf(text, sizeof text, "invalid step rows: slot %d rows are not contiguous", row.slot);
                return fail(SPL_ERR_INVALID_ROWS, text);
            }
            runs.push_back(uint32_t(row.slot)); runs.push_back(uint32_t(index)); runs.push_back(1);
            run_info.push_back(row.verify ? 1u : 0u); run_info.push_back(journal_pending[row.slot]);
        }
        if (row.want_logits) {
            if (int(gather_index.size()) >= config.max_logit_rows) return fail(SPL_ERR_INVALID_ROWS, "invalid step rows: too many logit rows");
            gather_index.push_back(uint32_t(index));
        }
    }
    // Rows the model's last block is computed for: a leading run that holds every row wanting
    // logits (Engine.swift:1419-1429). Keys and values are still stored for all rows.
    uint32_t live = uint32_t(count);
    if (geometry.layers % 4 == 0 && count >= 8) {
        int wanted = 0;
        for (int i = 0; i < count; ++i) if (rows[i].want_logits) wanted = i + 1;
        live = wanted == 0 ? 0u : uint32_t(std::min(count, std::max(wanted, 8)));
    }
    // Span split of the attention scan (Engine.swift:2236-2239): whole pages per span, at most
    // span_limit spans; the limit grows for narrow steps so the scan still fills the GPU.
    const int blocks = int(attn_blocks.size() / 2);
    const int wanted_spans = (config.span_target + geometry.kv_heads * blocks - 1) / (geometry.kv_heads * blocks);
    const uint32_t span_limit = uint32_t(std::max(16, std::min(64, wanted_spans)));
    const uint32_t pages_per_span = (step_pages + span_limit - 1) / span_limit;
    const uint32_t spans = (step_pages + pages_per_span - 1) / pages_per_span;

    out->rows = uint32_t(count); out->run_count = uint32_t(runs.size() / 3); out->logit_rows = uint32_t(gather_index.size());
    out->attn_block_count = uint32_t(blocks); out->step_pages = step_pages; out->live_rows = live;
    out->spans = spans; out->pages_per_span = pages_per_span;
    out->tokens = tokens.data(); out->row_slot = row_slot.data(); out->row_pos = row_pos.data();
    out->runs = runs.data(); out->run_info = run_info.data(); out->row_read = row_read.data(); out->row_write = row_write.data();
    out->gather_index = gather_index.data(); out->attn_blocks = attn_blocks.data(); out->page_table = page_table.data();
    return SPL_OK;
}

void spl_host::finish_step(const spl_tables *t) {
    for (uint32_t r = 0; r < t->run_count; ++r) journal_pending[t->runs[r * 3]] = 0;
}

extern "C" {

spl_status spl_host_create(const spl_geometry *geometry, const spl_config *config, spl_host **out) {
    if (!geometry || !config || !out) return SPL_ERR_INVALID_ARGUMENT;
    if (config->max_slots <= 0 || config->max_rows <= 0 || config->kv_pages <= 0 || config->max_context <= 0) return SPL_ERR_INVALID_ARGUMENT;
    if (config->state_units > 0 && config->state_units < config->max_slots) return SPL_ERR_INVALID_ROWS;   // Engine.swift:627
    *out = new spl_host(*geometry, *config);
    return SPL_OK;
}
void spl_host_destroy(spl_host *host) { delete host; }
spl_status spl_host_build_tables(spl_host *host, const spl_row *rows, int32_t count, spl_tables *out) { return host->build(rows, count, out); }
void spl_host_finish_step(spl_host *host, const spl_tables *tables) { host->finish_step(tables); }
int32_t spl_host_reset_slot(spl_host *host, int32_t slot) { return host->reset_slot(slot); }
void spl_host_discard_verify(spl_host *host, int32_t slot) { host->discard_verify(slot); }
spl_status spl_host_accept_verify(spl_host *host, int32_t slot, int32_t rows, int32_t token_count) { return host->accept_verify(slot, rows, token_count); }
void spl_host_truncate(spl_host *host, int32_t slot, int32_t token_count) { host->truncate(slot, token_count); }
int32_t spl_host_pages_held(const spl_host *host, int32_t slot) { return int32_t(host->slot_pages[slot].size()); }
int32_t spl_host_free_page_count(const spl_host *host) { return int32_t(host->free_pages.size()); }
int32_t spl_host_slot_unit(const spl_host *host, int32_t slot) { return int32_t(host->slot_unit[slot]); }
int32_t spl_host_journal_pending(const spl_host *host, int32_t slot) { return int32_t(host->journal_pending[slot]); }
int32_t spl_host_max_pages(const spl_host *host) { return host->max_pages; }
const char *spl_host_last_error(const spl_host *host) { return host->error.c_str(); }

int32_t spl_greedy_accept(const int32_t *argmax_ids, const int32_t *drafts, int32_t draft_count, int32_t *bonus) {
    int32_t agreed = 0;
    while (agreed < draft_count && argmax_ids[agreed] == drafts[agreed]) ++agreed;
    if (bonus) *bonus = argmax_ids[agreed];
    return agreed;
}

// ---- width planner (BatchScheduler.swift:646-669, 735-789) -----------------------------------------
// The algorithm is the reference's; its cost table is a property of the machine, so it is an argument.
void spl_plan_costs_reference(spl_plan_costs *c) {
    if (!c) return;
    const double tiers[5] = {62, 86, 165, 230, 295};                    // tierMilliseconds, BatchScheduler.swift:740
    for (int i = 0; i < 5; ++i) c->tier_ms[i] = tiers[i];
    c->beyond_ms_per_row = 2.3; c->per_row_ms = 0.45; c->fixed_ms = 10;  // cycleMilliseconds, :743-745
    c->attention_first = 0.29; c->attention_second = 0.22;              // attentionMilliseconds, :750
    c->prefill_attention = 0.022;                                       // per row and thousand tokens, :659
    c->tier_margin = 0.88;                                              // :779
}
// The same table measured with this library on a B200 (27B shape, MLX 4-bit, 8 sessions): steps of 16, 32, 64, 96 and
// 128 rows at 1K context took 7.5, 8.1, 9.1, 15.6 and 16.4 ms; 64 rows at 40K took 11.3 ms and 128 rows 20.8 ms,
// i.e. 0.0072 ms per thousand context tokens for a session's first block of eight rows and 0.0070 for its second; the host's share of a step
// (tables, launches, ids back) was 0.3 ms. A draft pass is the caller's to add.
void spl_plan_costs_b200(spl_plan_costs *c) {
    if (!c) return;
    const double tiers[5] = {7.5, 8.1, 9.1, 15.6, 16.4};       // steps of 16, 32, 64, 96, 128 rows over 8 sessions at 1K context
    for (int i = 0; i < 5; ++i) c->tier_ms[i] = tiers[i];
    c->beyond_ms_per_row = 0.13; c->per_row_ms = 0.0; c->fixed_ms = 0.3;
    c->attention_first = 0.0072; c->attention_second = 0.0070;      // (64 rows at 40K - at 1K) / (8 x 39K tokens); the same for the second block of 8 rows
    c->prefill_attention = 0.001;
    c->tier_margin = 0.88;
}
int32_t spl_plan_tier(int32_t rows) { return rows <= 16 ? 16 : ((rows + 31) / 32) * 32; }
double spl_plan_cycle_ms(const spl_plan_costs *c, int32_t rows) {
    const int tier = spl_plan_tier(rows);
    const int index = tier == 16 ? 0 : tier / 32;
    const double step = index <= 4 ? c->tier_ms[index] : double(rows) * c->beyond_ms_per_row;
    return step + c->per_row_ms * double(rows) + c->fixed_ms;
}
// prefillCap: the width (16, 32, 64, 96, 128) that makes the most progress per millisecond, a generated token counting
// as `decode_weight` prompt tokens. backlog = prompt tokens still to feed; first_fed = tokens already fed of the prompt
// with least left.
int32_t spl_plan_prefill_cap(const spl_plan_costs *c, int32_t max_rows, int32_t decode_rows, double decode_tokens, double decode_attention_ms,
                             double decode_weight, int32_t backlog, int32_t first_fed, int32_t prefill_rows_while_decoding) {
    if (backlog <= 0) return decode_rows;
    const double per_row = c->prefill_attention * double(first_fed) / 1000.0;
    int32_t best_cap = std::min(max_rows, spl_plan_tier(decode_rows + prefill_rows_while_decoding));
    double best_rate = 0.0;
    const int widths[5] = {16, 32, 64, 96, 128};
    for (int width : widths) {
        if (!(width <= max_rows && width > decode_rows)) continue;
        const int prefill = std::min(backlog, width - decode_rows);
        const double ms = spl_plan_cycle_ms(c, decode_rows + prefill) + decode_attention_ms + per_row * double(prefill);
        const double rate = (decode_weight * decode_tokens + double(prefill)) / ms;
        if (rate > best_rate) { best_cap = width; best_rate = rate; }
    }
    return best_cap;
}
// planBlocks: which speculating sessions get a double block. Per session: tail = wholeRate * tailYield and block_yield
// (SpeculationState.BlockStats, LookupIndex.swift:175-183), context_tokens. blocks_out[i] = block or 2 * block; returns
// how many were doubled.
int32_t spl_plan_blocks(const spl_plan_costs *c, int32_t sessions, const double *tail, const double *block_yield, const int32_t *context_tokens,
                        int32_t other_rows, int32_t block, int32_t max_rows, int32_t max_logit_rows, int32_t max_verify_rows, int32_t max_context,
                        int32_t *blocks_out) {
    for (int i = 0; i < sessions; ++i) blocks_out[i] = block;
    const int base = sessions * block + other_rows;
    auto thousands = [&](int i) { return double(context_tokens[i]) / 1000.0; };
    auto tail_cost = [&](int i) { return c->per_row_ms * double(block) + c->attention_second * thousands(i); };      // 0.45 per row in the reference, its cycle's per-row cost
    std::vector<int> candidates;
    for (int i = 0; i < sessions; ++i) if (context_tokens[i] + 2 * block < max_context) candidates.push_back(i);
    std::stable_sort(candidates.begin(), candidates.end(), [&](int a, int b) { return tail[a] / tail_cost(a) > tail[b] / tail_cost(b); });
    double tokens = double(other_rows), attention = 0.0;
    for (int i = 0; i < sessions; ++i) { tokens += block_yield[i]; attention += c->attention_first * thousands(i); }
    int best_count = 0;
    double best_rate = tokens / (spl_plan_cycle_ms(c, base) + attention);
    for (size_t index = 0; index < candidates.size(); ++index) {
        const int rows = base + int(index + 1) * block;
        if (!(rows <= max_rows && rows <= max_logit_rows && (sessions + int(index) + 1) * block <= max_verify_rows)) break;
        tokens += tail[candidates[index]];
        attention += c->attention_second * thousands(candidates[index]);
        const double rate = tokens / (spl_plan_cycle_ms(c, rows) + attention) * (spl_plan_tier(rows) == spl_plan_tier(base) ? 1.0 : c->tier_margin);
        if (rate > best_rate) { best_count = int(index) + 1; best_rate = rate; }
    }
    for (int i = 0; i < best_count; ++i) blocks_out[candidates[i]] = 2 * block;
    return best_count;
}

// ---- row packer (BatchScheduler.buildRows, BatchScheduler.swift:1323-1442) ------------------------------------
int32_t spl_host_pack_rows(const spl_host *host, const spl_session *sessions, int32_t session_count, const spl_pack_config *config,
                           spl_row *rows, spl_planned *plan, int32_t *plan_count, int32_t *waiting, int32_t *waiting_count) {
    if (!host || !sessions || session_count < 0 || !config || !config->costs || !rows || !plan || !plan_count || !waiting || !waiting_count ||
        config->block < 1) return -1;
    const spl_config &c = host->config;
    const int block = config->block;
    int row_count = 0, plans = 0, waits = 0, logit_rows = 0, reserved = 0;
    double decode_tokens = 0.0, decode_attention = 0.0;
    // KV pages this step's rows will take (:1336-1343); eviction of idle slots is the caller's policy.
    auto reserve = [&](int index, int position) {
        const spl_session &s = sessions[index];
        const int need = position / kPageTokens + 1 - int(host->slot_pages[s.slot].size());
        if (need <= 0) return true;
        if (need > int(host->free_pages.size()) - reserved) { waiting[waits++] = index; return false; }
        reserved += need;
        return true;
    };
    auto put = [&](int slot, int token, int position, bool logits, bool verify) {
        spl_row &r = rows[row_count++];
        r.slot = slot; r.token = token; r.position = position; r.want_logits = logits ? 1 : 0; r.verify = verify ? 1 : 0; r.reserved[0] = r.reserved[1] = 0;
    };
    std::vector<int> decoders, speculative, plain, prefillers;
    for (int i = 0; i < session_count; ++i) {
        if (sessions[i].slot < 0 || sessions[i].slot >= c.max_slots) return -1;
        if (sessions[i].pending >= 0 && int(decoders.size()) < c.max_slots) decoders.push_back(i);
    }
    // Speculative sessions verify a drafted block; the rest decode one token (:1347-1361).
    for (int i : decoders) {
        const spl_session &s = sessions[i];
        const int position = s.evaluated, ahead = int(speculative.size()) + 1;
        const bool fits = ahead * block <= config->max_verify_rows && row_count + ahead * block + int(plain.size()) <= c.max_rows &&
                          logit_rows + ahead * block + int(plain.size()) <= c.max_logit_rows;
        if (config->speculate && position + block < c.max_context) {
            if (fits && reserve(i, position + 2 * block - 1)) speculative.push_back(i);      // otherwise it waits for the next step
        } else if (reserve(i, position)) {
            plain.push_back(i);
        }
    }
    for (int i : speculative) {
        const spl_session &s = sessions[i];
        decode_tokens += s.block_yield;
        decode_attention += config->costs->attention_first * double(s.evaluated) / 1000.0;
    }
    for (int i : speculative) {
        const spl_session &s = sessions[i];
        if (row_count + 1 + s.proposal_count > c.max_rows) return -1;
        put(s.slot, s.pending, s.evaluated, true, true);
        for (int k = 0; k < s.proposal_count; ++k) put(s.slot, s.proposal[k], s.evaluated + 1 + k, true, true);
        logit_rows += s.proposal_count + 1;
        plan[plans++] = {SPL_PLAN_VERIFY, i, s.proposal_count, 0};
    }
    for (int i : plain) {
        const spl_session &s = sessions[i];
        if (row_count + 1 > c.max_rows) return -1;
        put(s.slot, s.pending, s.evaluated, true, false);
        logit_rows += 1;
        plan[plans++] = {SPL_PLAN_DECODE, i, 0, 0};
    }
    // Prompt chunks, the prompt with least left first (:1403-1440).
    for (int i = 0; i < session_count; ++i) if (sessions[i].pending < 0) prefillers.push_back(i);
    std::stable_sort(prefillers.begin(), prefillers.end(), [&](int a, int b) {
        return sessions[a].prompt_count - sessions[a].fed < sessions[b].prompt_count - sessions[b].fed; });
    int cap = c.max_rows;
    if (!decoders.empty()) {
        int backlog = 0;
        for (int i : prefillers) backlog += sessions[i].prompt_count - sessions[i].fed;
        cap = spl_plan_prefill_cap(config->costs, c.max_rows, row_count, decode_tokens + double(plain.size()), decode_attention, config->decode_weight,
                                   backlog, prefillers.empty() ? 0 : sessions[prefillers[0]].fed, config->prefill_rows_while_decoding);
    }
    for (int i : prefillers) {
        const spl_session &s = sessions[i];
        const int budget = cap - row_count;
        if (budget <= 0) break;
        int count = std::min(s.prompt_count - s.fed, budget);
        // A step ends exactly where the state is to be kept.
        int mark = -1;
        for (int k = 0; k < s.mark_count; ++k) if (s.marks[k] > s.fed && (mark < 0 || s.marks[k] < mark)) mark = s.marks[k];
        if (mark >= 0 && mark < s.fed + count) count = mark - s.fed;
        if (!reserve(i, s.fed + count - 1)) {
            // Whatever still fits in the pages the slot has.
            count = std::min(count, int(host->slot_pages[s.slot].size()) * kPageTokens - s.fed);
            if (count <= 0) continue;
            --waits;      // it takes part after all (the entry reserve() just made is the last one)
        }
        const bool complete = s.fed + count == s.prompt_count;
        if (complete && logit_rows >= c.max_logit_rows) continue;
        for (int offset = 0; offset < count; ++offset) put(s.slot, s.prompt[s.fed + offset], s.fed + offset, complete && offset == count - 1, false);
        if (complete) logit_rows += 1;
        plan[plans++] = {SPL_PLAN_PREFILL, i, count, complete ? 1 : 0};
    }
    *plan_count = plans; *waiting_count = waits;
    return row_count;
}

// ---- sampling from the k largest logits (Sampler.swift:68-156) -----------------------------------
// The generator is SplitMix64 kept in `*state`; one uniform = the top 24 bits of an output over 2^24.
static float sampler_uniform(uint64_t *state) {
    *state += 0x9E3779B97F4A7C15ull;
    uint64_t z = *state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return float(z >> 40) / float(1 << 24);
}

float spl_sampler_uniform(uint64_t *state) { return state ? sampler_uniform(state) : 0.0f; }

// Sampler.sample after TopK.select: ids/values are the k largest logits in descending order. Temperature softmax over
// them, the smallest prefix whose mass reaches top_p, one uniform draw scaled by the kept mass (Sampler.swift:128-156).
int32_t spl_sample_topk(const int32_t *ids, const float *values, int32_t k, float temperature, float top_p, uint64_t *state) {
    if (!ids || !values || k < 1 || !state) return -1;
    if (temperature <= 0.0f) return ids[0];
    std::vector<float> probabilities(k);
    const float top = values[0];
    float total = 0.0f;
    for (int i = 0; i < k; ++i) { probabilities[i] = expf((values[i] - top) / temperature); total += probabilities[i]; }
    for (int i = 0; i < k; ++i) probabilities[i] /= total;
    int kept = k;
    if (top_p < 1.0f) {
        float mass = 0.0f;
        for (int i = 0; i < k; ++i) { mass += probabilities[i]; if (mass >= top_p) { kept = i + 1; break; } }
    }
    float kept_mass = 0.0f;
    for (int i = 0; i < kept; ++i) kept_mass += probabilities[i];
    float draw = sampler_uniform(state) * kept_mass;
    for (int i = 0; i < kept; ++i) { draw -= probabilities[i]; if (draw <= 0.0f) return ids[i]; }
    return ids[kept - 1];
}

// Sampler.distribution (Sampler.swift:100-116): probabilities over the kept candidates, renormalised; returns how many are kept.
int32_t spl_sampler_distribution(const float *values, int32_t k, float temperature, float top_p, float *probabilities) {
    if (!values || !probabilities || k < 1) return 0;
    const float top = values[0], t = temperature > 1e-6f ? temperature : 1e-6f;
    float total = 0.0f;
    for (int i = 0; i < k; ++i) { probabilities[i] = expf((values[i] - top) / t); total += probabilities[i]; }
    for (int i = 0; i < k; ++i) probabilities[i] /= total;
    int kept = k;
    if (top_p < 1.0f) {
        float mass = 0.0f;
        for (int i = 0; i < k; ++i) { mass += probabilities[i]; if (mass >= top_p) { kept = i + 1; break; } }
    }
    total = 0.0f;
    for (int i = 0; i < kept; ++i) total += probabilities[i];
    for (int i = 0; i < kept; ++i) probabilities[i] /= total;
    return kept;
}

// SpeculativeSampling.resolve (Sampler.swift:163-179): -1 when the draft token is kept, else the token that replaces it.
int32_t spl_speculative_resolve(int32_t draft, const int32_t *candidates, const float *draft_probabilities, int32_t candidate_count,
                                const int32_t *target_ids, const float *target_probabilities, int32_t target_count, uint64_t *state) {
    if (!candidates || !draft_probabilities || !target_ids || !target_probabilities || !state || target_count < 1) return -2;
    float q = 0.0f, p = 0.0f;
    for (int i = 0; i < candidate_count; ++i) if (candidates[i] == draft) { q = draft_probabilities[i]; break; }
    for (int i = 0; i < target_count; ++i) if (target_ids[i] == draft) { p = target_probabilities[i]; break; }
    if (sampler_uniform(state) * q < p) return -1;
    std::vector<float> residual(target_probabilities, target_probabilities + target_count);
    for (int slot = 0; slot < target_count; ++slot)
        for (int c = 0; c < candidate_count; ++c)
            if (candidates[c] == target_ids[slot]) { residual[slot] = std::max(0.0f, residual[slot] - draft_probabilities[c]); break; }
    float total = 0.0f;
    for (float r : residual) total += r;
    if (total > 0.0f) { for (float &r : residual) r /= total; } else { residual.assign(target_probabilities, target_probabilities + target_count); }
    float remaining = sampler_uniform(state);
    for (int i = 0; i < target_count; ++i) { remaining -= residual[i]; if (remaining <= 0.0f) return target_ids[i]; }
    return target_ids[target_count - 1];
}

}  // extern "C"
