// spl_gguf_file.cpp — a llama.cpp GGUF file of a Qwen3.5-family hybrid model into an engine (host code only).
//
// Stands in for the reference's reader and converter of such a file (Sources/SploshModel/GgufFile.swift: the container;
// GgufNames.swift:13-44: the tensor names; GgufNames.swift:73-84 and GgufConvert.swift:15-32: the order of the gated-delta
// value heads, the dense tensors' rounding, A_log). The reference writes an SPLW artifact its engine maps; here the tensors
// go straight to the engine through spl_weights_set_gguf / spl_weights_set_vector.
//
// The container (GGUF versions 2 and 3, little endian): magic "GGUF", u32 version, u64 tensor count, u64 metadata count;
// metadata pairs (string key, u32 value type, value); tensor records (string name, u32 dimensions, u64 extents with the
// fastest first, u32 ggml type, u64 offset into the data section); the data section starts at the next multiple of
// `general.alignment` (32 when the key is absent).
//
// What is changed on the way:
//   - A file orders the value heads of a gated-delta block differently from the engine: its head i is the engine's
//     ratio * (i % key heads) + i / key heads. Rows of attn_gate (128 a head), ssm_alpha and ssm_beta (one a head), the value
//     rows of attn_qkv (from row 2 x key heads x 128), the value channels of ssm_conv1d, and ssm_a / ssm_dt.bias are moved;
//     a row of a packed weight is whole blocks, so that is lossless. ssm_out has the heads as columns and stays as it is:
//     the engine is told to write the blocks' outputs in file order (spl_weights_gguf_file_order).
//   - Dense tensors (F32, F16 or BF16 in the file) become bf16, round to nearest even; ssm_a holds -exp(A_log) and the engine
//     reads A_log.
//   - The tensors of an MTP block (the last blk.<n> of a file that has `.nextn.` tensors) are left out.
#include <fcntl.h>
#include <math.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/splosh_cuda.h"

namespace {

struct Record { std::vector<uint64_t> extent; uint32_t type = 0; uint64_t offset = 0; };

struct Reader {
    const uint8_t *base = nullptr; size_t size = 0, at = 0; bool ok = true;
    template <typename T> T get() { T v{}; if (at + sizeof(T) > size) { ok = false; return v; } memcpy(&v, base + at, sizeof(T)); at += sizeof(T); return v; }
    std::string str() { const uint64_t n = get<uint64_t>(); if (!ok || n > size - at) { ok = false; return ""; } std::string s(reinterpret_cast<const char *>(base + at), size_t(n)); at += size_t(n); return s; }
    // Skips a metadata value of `type`; returns it as an integer when it is one (for general.alignment).
    uint64_t value(uint32_t type) {
        switch (type) {
        case 0: return get<uint8_t>(); case 1: return uint64_t(get<int8_t>()); case 2: return get<uint16_t>(); case 3: return uint64_t(get<int16_t>());
        case 4: return get<uint32_t>(); case 5: return uint64_t(get<int32_t>()); case 6: get<float>(); return 0; case 7: return get<uint8_t>();
        case 8: str(); return 0;
        case 9: { const uint32_t inner = get<uint32_t>(); const uint64_t n = get<uint64_t>(); for (uint64_t i = 0; i < n && ok; ++i) value(inner); return 0; }
        case 10: return get<uint64_t>(); case 11: return uint64_t(get<int64_t>()); case 12: get<double>(); return 0;
        }
        ok = false; return 0;
    }
};

uint16_t to_bf16(float v) { uint32_t bits; memcpy(&bits, &v, 4); return uint16_t((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16); }
float half_to_float(uint16_t h) { _Float16 x; memcpy(&x, &h, 2); return float(x); }
int block_bytes(uint32_t type) { return type == 14 ? 210 : type == 13 ? 176 : type == 12 ? 144 : 0; }

struct Loader {
    spl_engine *engine; spl_geometry g; std::string error;
    const uint8_t *data = nullptr; size_t data_size = 0;
    std::map<std::string, Record> records;
    int D() const { return g.gdn_head_dim; }
    int engine_head(int file_head) const { const int ratio = g.gdn_value_heads / g.gdn_key_heads; return ratio * (file_head % g.gdn_key_heads) + file_head / g.gdn_key_heads; }

    bool fail(const std::string &what) { if (error.empty()) error = what; return false; }
    const Record *find(const std::string &name) { auto it = records.find(name); return it == records.end() ? nullptr : &it->second; }
    bool payload(const Record &r, size_t bytes, const uint8_t **out) {
        if (r.offset > data_size || bytes > data_size - r.offset) return fail("a tensor's data lies outside the file");
        *out = data + r.offset; return true;
    }
    // A dense tensor as floats.
    bool dense(const std::string &name, size_t count, std::vector<float> *out) {
        const Record *r = find(name);
        if (!r) return fail("missing tensor " + name);
        size_t have = 1; for (uint64_t e : r->extent) have *= size_t(e);
        if (have != count) return fail("tensor " + name + " has the wrong number of elements");
        const uint8_t *src;
        out->resize(count);
        if (r->type == 0) { if (!payload(*r, count * 4, &src)) return false; memcpy(out->data(), src, count * 4); }
        else if (r->type == 1) { if (!payload(*r, count * 2, &src)) return false; for (size_t i = 0; i < count; ++i) { uint16_t h; memcpy(&h, src + 2 * i, 2); (*out)[i] = half_to_float(h); } }
        else if (r->type == 30) { if (!payload(*r, count * 2, &src)) return false; for (size_t i = 0; i < count; ++i) { uint16_t h; memcpy(&h, src + 2 * i, 2); uint32_t bits = uint32_t(h) << 16; memcpy(&(*out)[i], &bits, 4); } }
        else return fail("tensor " + name + " is not F32, F16 or BF16");
        return true;
    }
    bool set_vector(int layer, int kind, const std::vector<float> &values) {
        std::vector<uint16_t> bits(values.size());
        for (size_t i = 0; i < values.size(); ++i) bits[i] = to_bf16(values[i]);
        if (spl_weights_set_vector(engine, layer, kind, bits.data(), int32_t(bits.size())) != SPL_OK) return fail(spl_last_error_string(engine));
        return true;
    }
    // Units (rows, channels, elements) [first, first + heads x span) of `values`, `width` items a unit, moved from the file's head order to the engine's.
    template <typename T> void reorder(std::vector<T> &values, size_t first, size_t span, size_t width) {
        const std::vector<T> old(values);
        for (int i = 0; i < g.gdn_value_heads; ++i) {
            const size_t from = (first + size_t(i) * span) * width, to = (first + size_t(engine_head(i)) * span) * width;
            memcpy(values.data() + to, old.data() + from, span * width * sizeof(T));
        }
    }
    // A packed 2-D weight [rows][inner]; heads_first >= 0: the value heads are rows from there, `span` rows a head.
    bool packed(const std::string &name, int layer, int kind, int rows, int inner, long heads_first, int span) {
        const Record *r = find(name);
        if (!r) return fail("missing tensor " + name);
        const int bytes = block_bytes(r->type);
        if (!bytes) return fail("tensor " + name + " is not Q4_K, Q5_K or Q6_K");
        if (r->extent.size() != 2 || int(r->extent[0]) != inner || int(r->extent[1]) != rows) return fail("tensor " + name + " does not have the geometry's shape");
        const size_t row_bytes = size_t(inner / 256) * bytes;
        const uint8_t *src;
        if (!payload(*r, row_bytes * rows, &src)) return false;
        std::vector<uint8_t> moved;
        if (heads_first >= 0) { moved.assign(src, src + row_bytes * rows); reorder(moved, size_t(heads_first), size_t(span), row_bytes); src = moved.data(); }
        if (spl_weights_set_gguf(engine, layer, kind, int32_t(r->type), rows, inner, src) != SPL_OK) return fail(spl_last_error_string(engine));
        return true;
    }

    bool load() {
        const int H = g.hidden, Dh = D(), KH = g.gdn_key_heads, VH = g.gdn_value_heads, C = (2 * KH + VH) * Dh, VD = VH * Dh, AD = g.heads * g.head_dim, KV = g.kv_heads * g.head_dim;
        std::vector<float> v;
        for (int layer = 0; layer < g.layers; ++layer) {
            const std::string b = "blk." + std::to_string(layer) + ".";
            if (!dense(b + "attn_norm.weight", H, &v) || !set_vector(layer, SPL_VEC_INPUT_NORM, v)) return false;
            if (!dense(b + "post_attention_norm.weight", H, &v) || !set_vector(layer, SPL_VEC_POST_NORM, v)) return false;
            if (layer % 4 == 3) {        // gated attention (Sources/SploshModel/LayerGraph.swift:22)
                if (!packed(b + "attn_q.weight", layer, SPL_Q4_Q, 2 * AD, H, -1, 0) || !packed(b + "attn_k.weight", layer, SPL_Q4_K, KV, H, -1, 0) ||
                    !packed(b + "attn_v.weight", layer, SPL_Q4_V, KV, H, -1, 0) || !packed(b + "attn_output.weight", layer, SPL_Q4_O, H, AD, -1, 0)) return false;
                if (!dense(b + "attn_q_norm.weight", g.head_dim, &v) || !set_vector(layer, SPL_VEC_Q_NORM, v)) return false;
                if (!dense(b + "attn_k_norm.weight", g.head_dim, &v) || !set_vector(layer, SPL_VEC_K_NORM, v)) return false;
            } else {
                if (!packed(b + "attn_qkv.weight", layer, SPL_Q4_QKV, C, H, 2L * KH * Dh, Dh) || !packed(b + "attn_gate.weight", layer, SPL_Q4_Z, VD, H, 0, Dh) ||
                    !packed(b + "ssm_alpha.weight", layer, SPL_Q4_A, VH, H, 0, 1) || !packed(b + "ssm_beta.weight", layer, SPL_Q4_B, VH, H, 0, 1) ||
                    !packed(b + "ssm_out.weight", layer, SPL_Q4_OUT, H, VD, -1, 0)) return false;
                if (!dense(b + "ssm_conv1d.weight", size_t(C) * 4, &v)) return false;
                { const Record *r = find(b + "ssm_conv1d.weight"); if (r->extent.empty() || r->extent[0] != 4) return fail("ssm_conv1d.weight is not [channels][4]"); }
                reorder(v, size_t(2) * KH * Dh, size_t(Dh), 4);
                if (!set_vector(layer, SPL_VEC_CONV, v)) return false;
                if (!dense(b + "ssm_a", VH, &v)) return false;
                for (float &x : v) { if (!(x < 0.0f)) return fail("ssm_a holds -exp(A_log): a value is not negative"); x = logf(-x); }
                reorder(v, 0, 1, 1);
                if (!set_vector(layer, SPL_VEC_A_LOG, v)) return false;
                if (!dense(b + "ssm_dt.bias", VH, &v)) return false;
                reorder(v, 0, 1, 1);
                if (!set_vector(layer, SPL_VEC_DT_BIAS, v)) return false;
                if (!dense(b + "ssm_norm.weight", Dh, &v) || !set_vector(layer, SPL_VEC_GDN_NORM, v)) return false;
            }
            if (!packed(b + "ffn_gate.weight", layer, SPL_Q4_GATE, g.inter, H, -1, 0) || !packed(b + "ffn_up.weight", layer, SPL_Q4_UP, g.inter, H, -1, 0) ||
                !packed(b + "ffn_down.weight", layer, SPL_Q4_DOWN, H, g.inter, -1, 0)) return false;
        }
        if (!packed("token_embd.weight", -1, SPL_Q4_EMBED, g.vocab, H, -1, 0)) return false;
        // A file without an output tensor ties the head to the embedding.
        if (!packed(find("output.weight") ? "output.weight" : "token_embd.weight", -1, SPL_Q4_HEAD, g.vocab, H, -1, 0)) return false;
        if (!dense("output_norm.weight", H, &v) || !set_vector(-1, SPL_VEC_FINAL_NORM, v)) return false;
        if (spl_weights_gguf_file_order(engine, 1) != SPL_OK) return fail(spl_last_error_string(engine));
        return true;
    }
};

}  // namespace

extern "C" spl_status spl_weights_load_gguf_file(spl_engine *engine, const char *path, char *message, size_t message_bytes) {
    auto say = [&](const std::string &text, spl_status status) {
        if (message && message_bytes) { const size_t n = std::min(text.size(), message_bytes - 1); memcpy(message, text.data(), n); message[n] = 0; }
        return status;
    };
    if (!engine || !path) return say("null argument", SPL_ERR_INVALID_ARGUMENT);
    Loader loader;
    loader.engine = engine;
    if (spl_engine_geometry(engine, &loader.g) != SPL_OK) return say("no geometry", SPL_ERR_INVALID_ARGUMENT);
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return say(std::string("cannot open ") + path, SPL_ERR_INVALID_ARGUMENT);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) { close(fd); return say("not a GGUF file", SPL_ERR_INVALID_ARGUMENT); }
    void *map = mmap(nullptr, size_t(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) return say("cannot map the file", SPL_ERR_ALLOCATION_FAILED);
    Reader in; in.base = static_cast<const uint8_t *>(map); in.size = size_t(st.st_size);
    spl_status status = SPL_OK;
    std::string text;
    do {
        if (in.get<uint32_t>() != 0x46554747u) { text = "not a GGUF file"; status = SPL_ERR_INVALID_ARGUMENT; break; }
        const uint32_t version = in.get<uint32_t>();
        if (version != 2 && version != 3) { text = "GGUF version " + std::to_string(version) + " is not 2 or 3"; status = SPL_ERR_INVALID_ARGUMENT; break; }
        const uint64_t tensors = in.get<uint64_t>(), pairs = in.get<uint64_t>();
        uint64_t alignment = 32;
        for (uint64_t i = 0; i < pairs && in.ok; ++i) {
            const std::string key = in.str();
            const uint32_t type = in.get<uint32_t>();
            const uint64_t value = in.value(type);
            if (key == "general.alignment" && value) alignment = value;
        }
        int last_block = -1; bool has_nextn = false;
        std::vector<std::pair<std::string, Record>> all;
        for (uint64_t i = 0; i < tensors && in.ok; ++i) {
            Record r;
            const std::string name = in.str();
            const uint32_t dims = in.get<uint32_t>();
            if (dims > 4) { in.ok = false; break; }
            for (uint32_t d = 0; d < dims; ++d) r.extent.push_back(in.get<uint64_t>());
            r.type = in.get<uint32_t>(); r.offset = in.get<uint64_t>();
            if (name.find(".nextn.") != std::string::npos) has_nextn = true;
            if (name.compare(0, 4, "blk.") == 0) last_block = std::max(last_block, atoi(name.c_str() + 4));
            all.emplace_back(name, r);
        }
        if (!in.ok) { text = "the file's directory is cut short or malformed"; status = SPL_ERR_INVALID_ARGUMENT; break; }
        // The MTP block (GgufNames.mtpBlock): the last blk.<n> of a file that has `.nextn.` tensors; the engine does not run it.
        const std::string mtp = has_nextn ? "blk." + std::to_string(last_block) + "." : "";
        for (auto &entry : all)
            if (mtp.empty() || entry.first.compare(0, mtp.size(), mtp) != 0) loader.records[entry.first] = entry.second;
        const size_t start = (in.at + alignment - 1) / alignment * alignment;
        if (start > in.size) { text = "the file has no data section"; status = SPL_ERR_INVALID_ARGUMENT; break; }
        loader.data = in.base + start; loader.data_size = in.size - start;
        if (!loader.load()) { text = loader.error; status = SPL_ERR_INVALID_ARGUMENT; }
    } while (false);
    munmap(map, size_t(st.st_size));
    return say(text, status);
}
