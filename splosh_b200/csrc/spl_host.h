// spl_host.h — host bookkeeping object behind the spl_host_* entry points.
#pragma once
#include <string>
#include <vector>

#include "../../include/splosh_cuda.h"

struct spl_host {
    spl_geometry geometry;
    spl_config config;
    int max_pages = 0;
    std::vector<uint32_t> free_pages, free_units, slot_unit, journal_pending, page_table;
    std::vector<std::vector<uint32_t>> slot_pages, pending_verify;
    // The last build's tables (spl_tables points into these).
    std::vector<uint32_t> tokens, row_slot, row_pos, runs, run_info, row_read, row_write, gather_index, attn_blocks;
    std::string error;

    spl_host(const spl_geometry &g, const spl_config &c);
    int32_t reset_slot(int slot);
    void discard_verify(int slot);
    spl_status accept_verify(int slot, int rows, int token_count);
    void truncate(int slot, int token_count);
    spl_status ensure_page(int slot, int position);
    spl_status build(const spl_row *rows, int count, spl_tables *out);
    void finish_step(const spl_tables *t);
    spl_status fail(spl_status code, const std::string &text);
};
