// spl_host.cpp — the host-side bookkeeping of a step: paged-KV block allocator, state-unit pool,
// row validation and the per-step index tables. Plain C++; nothing here touches the GPU.
//
// In the reference this lives inside Engine (Sources/SploshRuntime/Engine.swift:625-632 free lists,
// :810-868 slot lifecycle, :1316-1398 the table build at the top of step()). Page ids come off the
// end of a free list that starts reversed, so a fresh engine hands out ascending ids and freed
// pages are reused last-in first-out; slot i starts on state unit i and speculative rows take
// fresh units from max_slots upward.
#include "spl_host.h"

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

}  // extern "C"
