// spl_splw_file.cpp — an SPLW artifact (the reference's own weight container) into an engine (host code only).
//
// Stands in for the reference's reader of such a file and the model loader over it (Sources/SploshModel/WeightFile.swift:88-141:
// the container and its checks; Sources/SploshModel/Converter.swift:46-82: the header; Sources/SploshModel/Retile.swift:1-36,
// 137-153: the tiled layout; Sources/SploshModel/ModelWeights.swift:181-248: the tensor names and shapes). The reference maps
// the file and hands spans of it to its kernels; here the tensors go to the engine through spl_weights_set_q4 /
// spl_weights_set_vector, which copies them into its own device layout.
//
// The container: "SPLW", u32 version 1, u64 header length (little endian), a JSON header of that length, zero padding to
// the next multiple of the header's pointer alignment, then the payload: every tensor at its recorded offset, the offsets
// ascending, aligned, with no unaccounted bytes between or after them. The header names the format: "mlxAffine4"
// (row-major MLX affine-4 triplets: packed u32 [rows][inner / 8], bf16 scales and biases [rows][inner / 64]) or
// "mlxAffine4.tiled128" (the same tensors with the triplets of eligible weights permuted to [tile of 128 rows][group][row in
// tile][32 bytes of codes] and [tile][group][row] for the sidecars; eligible = name under "language_model." ending in
// ".weight", not the embedding, rows a multiple of 128). Both are read; the tiled form is put back in rows on the way.
// A GGUF-derived artifact ("gguf.tiled128", Sources/SploshModel/GgufConvert.swift:1-33) has the same names and dense tensors
// (value heads already in the engine's order, the out projection's columns in the file's) and holds every 2-D weight as the
// three planes of Sources/SploshModel/GgufPlanes.swift, records <base>.weight (plane 0, with the ggml type and the logical
// shape), <base>.plane1 and <base>.meta, rows padded to whole tiles of 128 with zero blocks; the planes are put back into
// llama.cpp's native blocks (spl_gguf_planes_unpack) and go in through spl_weights_set_gguf, and the engine is told that
// the out projections are in file order. Q4_K, Q5_K and Q6_K weights; the 8-bit affine packs ("mlxAffine8...") are refused
// with a message: the engine's affine tensors are 4-bit.
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "../../include/splosh_cuda.h"

namespace {

// ---- a JSON value: what the header needs (objects, arrays, strings, numbers, true / false / null) ----
struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool truth = false;
    double number = 0.0;
    uint64_t integer = 0;          // the number as an unsigned integer when it is written as one
    bool is_integer = false;
    std::string text;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> fields;
    const Json *get(const char *key) const {
        for (const auto &f : fields) if (f.first == key) return &f.second;
        return nullptr;
    }
};

struct JsonReader {
    const char *p, *end; bool ok = true; int depth = 0;
    void space() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool take(char c) { space(); if (p < end && *p == c) { ++p; return true; } return false; }
    bool word(const char *w) { const size_t n = strlen(w); if (size_t(end - p) >= n && memcmp(p, w, n) == 0) { p += n; return true; } return false; }
    std::string string() {
        std::string out;
        if (!take('"')) { ok = false; return out; }
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (++p >= end) break;
                switch (*p) {
                case 'n': out += '\n'; break; case 't': out += '\t'; break; case 'r': out += '\r'; break; case 'b': out += '\b'; break; case 'f': out += '\f'; break;
                case 'u': {      // a basic-plane code point as UTF-8 (names are ASCII; this keeps any other header text intact)
                    if (end - p < 5) { ok = false; return out; }
                    unsigned code = 0;
                    for (int i = 1; i <= 4; ++i) { const char h = p[i]; code = code * 16 + unsigned(h >= '0' && h <= '9' ? h - '0' : h >= 'a' && h <= 'f' ? h - 'a' + 10 : h >= 'A' && h <= 'F' ? h - 'A' + 10 : 0); }
                    p += 4;
                    if (code < 0x80) out += char(code);
                    else if (code < 0x800) { out += char(0xC0 | (code >> 6)); out += char(0x80 | (code & 0x3F)); }
                    else { out += char(0xE0 | (code >> 12)); out += char(0x80 | ((code >> 6) & 0x3F)); out += char(0x80 | (code & 0x3F)); }
                    break;
                }
                default: out += *p;       // \" \\ \/
                }
                ++p;
            } else out += *p++;
        }
        if (p >= end) { ok = false; return out; }
        ++p;
        return out;
    }
    Json value() {
        Json v;
        if (++depth > 32) { ok = false; return v; }
        space();
        if (p >= end) { ok = false; }
        else if (*p == '{') {
            ++p; v.kind = Json::Object;
            if (!take('}')) {
                do {
                    std::string key = string();
                    if (!ok || !take(':')) { ok = false; break; }
                    v.fields.emplace_back(std::move(key), value());
                } while (ok && take(','));
                if (ok && !take('}')) ok = false;
            }
        } else if (*p == '[') {
            ++p; v.kind = Json::Array;
            if (!take(']')) {
                do v.items.push_back(value()); while (ok && take(','));
                if (ok && !take(']')) ok = false;
            }
        } else if (*p == '"') { v.kind = Json::String; v.text = string(); }
        else if (word("true")) { v.kind = Json::Bool; v.truth = true; }
        else if (word("false")) { v.kind = Json::Bool; }
        else if (word("null")) { }
        else {
            const char *start = p;
            bool integral = true;
            if (p < end && *p == '-') { ++p; integral = false; }
            while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '+' || *p == '-')) { if (*p < '0' || *p > '9') integral = false; ++p; }
            if (p == start) ok = false;
            else {
                v.kind = Json::Number;
                const std::string digits(start, p);
                v.number = strtod(digits.c_str(), nullptr);
                if (integral && digits.size() <= 19) { v.is_integer = true; v.integer = strtoull(digits.c_str(), nullptr, 10); }
            }
        }
        --depth;
        return v;
    }
};

struct Record {
    std::string name, dtype;
    std::vector<int64_t> shape, physical, logical;
    bool has_logical = false, has_type = false;
    uint64_t offset = 0, bytes = 0, padding = 0, gguf_type = 0;
};

bool integer_of(const Json *j, uint64_t *out) { if (!j || j->kind != Json::Number || !j->is_integer) return false; *out = j->integer; return true; }
bool shape_of(const Json *j, std::vector<int64_t> *out) {
    if (!j || j->kind != Json::Array) return false;
    out->clear();
    for (const Json &item : j->items) { if (item.kind != Json::Number || !item.is_integer) return false; out->push_back(int64_t(item.integer)); }
    return true;
}
uint64_t align_up(uint64_t n, uint64_t a) { return n + ((a - n % a) % a); }

// The checked container: the header's records in payload order.
struct Container {
    std::string format, error;
    std::vector<Record> records;
    std::map<std::string, const Record *> by_name;
    bool fail(const std::string &what) { if (error.empty()) error = what; return false; }

    // The checks of WeightFile.init(splwURL:) (WeightFile.swift:88-141), in its order and with its messages.
    bool parse(const uint8_t *base, uint64_t size) {
        if (size < 16) return fail("truncated framing");
        if (memcmp(base, "SPLW", 4) != 0) return fail("bad magic");
        uint32_t version; memcpy(&version, base + 4, 4);
        if (version != 1) return fail("unsupported version");
        uint64_t header_length; memcpy(&header_length, base + 8, 8);
        if (header_length > size - 16) return fail("header length overflow");
        JsonReader reader{reinterpret_cast<const char *>(base + 16), reinterpret_cast<const char *>(base + 16 + header_length)};
        const Json header = reader.value();
        reader.space();
        if (!reader.ok || reader.p != reader.end || header.kind != Json::Object) return fail("malformed header");
        const Json *magic = header.get("magic"), *fmt = header.get("format"), *quant = header.get("quantization"), *alignment = header.get("alignment"), *list = header.get("tensorRecords");
        uint64_t declared_version = 0, declared_length = 0, payload_length = 0;
        if (!magic || magic->kind != Json::String || !fmt || fmt->kind != Json::String || !quant || quant->kind != Json::Object || !alignment || alignment->kind != Json::Object ||
            !list || list->kind != Json::Array || !integer_of(header.get("version"), &declared_version) || !integer_of(header.get("headerLength"), &declared_length) ||
            !integer_of(header.get("payloadLength"), &payload_length)) return fail("malformed header");
        if (magic->text != "SPLW" || declared_version != 1 || declared_length != header_length) return fail("contradictory header framing");
        format = fmt->text;
        uint64_t bits = 0, group = 0, pointer_alignment = 0;
        const Json *mode = quant->get("mode");
        if (!integer_of(quant->get("bits"), &bits) || !integer_of(quant->get("groupSize"), &group) || !mode || mode->kind != Json::String) return fail("malformed header");
        const bool affine = (bits == 4 || bits == 8) && group == 64 && mode->text == "affine";
        const bool gguf = bits == 0 && group == 32 && mode->text == "gguf";
        if (format == "gguf.tiled128" ? !gguf : !affine) return fail("unsupported quantization");
        if (!integer_of(alignment->get("pointerAlignmentBytes"), &pointer_alignment) || pointer_alignment == 0) return fail("invalid alignment");
        const uint64_t payload_start = align_up(16 + header_length, pointer_alignment);
        if (payload_start > size || payload_length > size - payload_start || payload_start + payload_length != size) return fail("payload size mismatch");
        uint64_t previous = payload_start;
        std::set<std::string> names;
        records.reserve(list->items.size());
        for (const Json &item : list->items) {
            Record r;
            const Json *name = item.get("name"), *dtype = item.get("dtype");
            if (item.kind != Json::Object || !name || name->kind != Json::String || !dtype || dtype->kind != Json::String || !shape_of(item.get("shape"), &r.shape) ||
                !shape_of(item.get("physicalShape"), &r.physical) || !integer_of(item.get("payloadOffset"), &r.offset) || !integer_of(item.get("rawByteLength"), &r.bytes) ||
                !integer_of(item.get("alignmentPadding"), &r.padding)) return fail("malformed header");
            r.name = name->text; r.dtype = dtype->text;
            const Json *logical = item.get("logicalShape");
            if (logical && logical->kind != Json::Null) { if (!shape_of(logical, &r.logical)) return fail("malformed header"); r.has_logical = true; }
            const Json *type = item.get("ggufType");
            if (type && type->kind != Json::Null) { if (!integer_of(type, &r.gguf_type)) return fail("malformed header"); r.has_type = true; }
            if (!names.insert(r.name).second) return fail("duplicate tensor: " + r.name);
            static const char *const known[] = {"BF16", "F32", "F16", "U32", "I32", "I64", "U8"};
            if (std::find_if(known, known + 7, [&](const char *k) { return r.dtype == k; }) == known + 7) return fail("unknown dtype: " + r.name);
            if (r.name.empty() || r.offset < payload_start || r.offset < previous || r.offset > size || r.bytes > size - r.offset) return fail("tensor bounds: " + r.name);
            if (r.offset % pointer_alignment != 0) return fail("unaligned tensor: " + r.name);
            if (r.padding != r.offset - previous) return fail("padding mismatch: " + r.name);
            previous = r.offset + r.bytes;
            records.push_back(std::move(r));
        }
        if (previous > size || (!records.empty() && previous != size)) return fail("unaccounted payload bytes");
        for (const Record &r : records) by_name[r.name] = &r;
        return true;
    }
};

// Whether a packed weight of a tiled artifact is stored in tiles (Retile.swift:31-36).
bool tiled_weight(const std::string &name, int64_t rows) {
    const std::string prefix = "language_model.", suffix = ".weight";
    return name.compare(0, prefix.size(), prefix) == 0 && name.size() >= suffix.size() && name.compare(name.size() - suffix.size(), suffix.size(), suffix) == 0 &&
           name.find("embed_tokens") == std::string::npos && rows % 128 == 0;
}
// [tile][group][row in tile][element] -> [row][group][element]: the inverse of Converter.tile (Retile.swift:137-153).
void untile(const uint8_t *src, uint8_t *dst, int64_t rows, int64_t groups, int element_bytes) {
    for (int64_t tile = 0; tile < rows / 128; ++tile)
        for (int64_t group = 0; group < groups; ++group) {
            const int64_t base = (tile * groups + group) * 128;
            for (int64_t n = 0; n < 128; ++n) memcpy(dst + ((tile * 128 + n) * groups + group) * element_bytes, src + (base + n) * element_bytes, size_t(element_bytes));
        }
}

// ---- the planes of a GGUF weight (GgufPlanes.swift:1-20) back into native blocks ----
// A weight of `rows` x `inner` is held as records per (row, group of 32 inputs) in two code planes and per (row, native
// block of 256) in a meta plane, each plane in tiles of 128 rows: record (row, b of n a row) sits at
// ((row / 128) * n + b) * 128 + row % 128. Inside a group element e has slot 8 ((e >> 2) & 3) + 4 (e >> 4) + (e & 3).
// Plane 0 holds a slot's low four bits: word s / 8 of the record's four, at bit 16 (s & 1) + 4 ((s & 7) >> 1). Plane 1 holds
// the bits above them as a little-endian string of fields (one bit a slot for Q5_K, two for Q6_K). The meta record is the
// block's scale fields: bytes 0-15 of a Q4_K or Q5_K block; a Q6_K block's sixteen scales (its bytes 192-207), then d (208-209)
// and two zero bytes.
struct PlaneShape { int plane1_bytes, meta_bytes, block_bytes, high_width; };
bool plane_shape(int type, PlaneShape *out) {
    switch (type) {
    case 12: *out = {0, 16, 144, 0}; return true;
    case 13: *out = {4, 16, 176, 1}; return true;
    case 14: *out = {8, 20, 210, 2}; return true;
    }
    return false;
}
size_t plane_record(int64_t row, int64_t index, int64_t per_row) { return size_t(((row / 128) * per_row + index) * 128 + row % 128); }
int plane_slot(int e) { return 8 * ((e >> 2) & 3) + 4 * (e >> 4) + (e & 3); }

// `rows` logical rows out of planes that hold `stored_rows` (a multiple of 128); native: [rows][inner / 256][block bytes].
bool planes_unpack(int type, const uint8_t *plane0, const uint8_t *plane1, const uint8_t *meta, int64_t rows, int64_t inner, uint8_t *native) {
    PlaneShape shape;
    if (!plane_shape(type, &shape) || rows <= 0 || inner <= 0 || inner % 256 != 0) return false;
    const int64_t groups = inner / 32, blocks = inner / 256;
    memset(native, 0, size_t(rows * blocks * shape.block_bytes));
    for (int64_t row = 0; row < rows; ++row)
        for (int64_t group = 0; group < groups; ++group) {
            const int64_t block = group / 8; const int j = int(group % 8);
            uint8_t *b = native + (row * blocks + block) * shape.block_bytes;
            const uint8_t *codes = plane0 + plane_record(row, group, groups) * 16;
            const uint8_t *high = shape.plane1_bytes ? plane1 + plane_record(row, group, groups) * size_t(shape.plane1_bytes) : nullptr;
            uint32_t words[4], high_words[2] = {0, 0};
            memcpy(words, codes, 16);
            if (high) memcpy(high_words, high, size_t(shape.plane1_bytes));
            for (int e = 0; e < 32; ++e) {
                const int s = plane_slot(e);
                const uint8_t low = uint8_t((words[s >> 3] >> (16 * (s & 1) + 4 * ((s & 7) >> 1))) & 15u);
                uint8_t top = 0;
                if (shape.high_width) { const int per_word = 32 / shape.high_width; top = uint8_t((high_words[s / per_word] >> (shape.high_width * (s % per_word))) & ((1u << shape.high_width) - 1u)); }
                if (type == 14) {
                    const int half = j / 4, quarter = j % 4;
                    b[64 * half + 32 * (quarter & 1) + e] |= uint8_t(low << (4 * (quarter >> 1)));
                    b[128 + 32 * half + e] |= uint8_t(top << (2 * quarter));
                } else {
                    b[(type == 13 ? 48 : 16) + 32 * (j / 2) + e] |= uint8_t(low << (4 * (j % 2)));
                    if (type == 13) b[16 + e] |= uint8_t(top << j);
                }
            }
            if (j == 0) {
                const uint8_t *fields = meta + plane_record(row, block, blocks) * size_t(shape.meta_bytes);
                if (type == 14) { memcpy(b + 192, fields, 16); memcpy(b + 208, fields + 16, 2); }
                else memcpy(b, fields, 16);
            }
        }
    return true;
}

struct Loader {
    spl_engine *engine; spl_geometry g; Container *file; const uint8_t *base; bool tiled = false, gguf = false; std::string error;
    bool fail(const std::string &what) { if (error.empty()) error = what; return false; }
    const Record *find(const std::string &name) { auto it = file->by_name.find("language_model." + name); return it == file->by_name.end() ? nullptr : it->second; }

    // One MLX affine-4 triplet by the name of its weight (WeightFile.q4, WeightFile.swift:202-240) into the engine.
    // One GGUF weight by the name of its plane 0 (WeightFile.gguf, WeightFile.swift:155-199) into the engine as native blocks.
    bool planes(const std::string &name, int layer, int kind, int64_t rows, int64_t inner) {
        const Record *w = find(name + ".weight"), *m = find(name + ".meta"), *h = find(name + ".plane1");
        if (!w) return fail("missing tensor language_model." + name + ".weight");
        if (w->dtype != "U8") return fail(name + ".weight is " + w->dtype + ", not U8");
        PlaneShape shape;
        if (!w->has_type || !plane_shape(int(w->gguf_type), &shape)) return fail(name + ".weight is not a GGUF weight of a type the engine takes (Q4_K, Q5_K, Q6_K)");
        if (!w->has_logical || w->logical.size() != 2 || w->logical[0] <= 0 || w->logical[1] <= 0) return fail(name + ".weight has no logical shape [rows, inner]");
        if (w->logical[0] != rows || w->logical[1] != inner) return fail(name + " does not have the geometry's shape");
        if (inner % 256 != 0) return fail(name + ": a row of " + std::to_string(inner) + " is not a whole number of blocks");
        const int64_t stored = (rows + 127) / 128 * 128, groups = inner / 32;
        auto plane = [&](const Record *r, const std::string &which, int64_t bytes) {
            if (!r) return fail(name + ".weight has no " + which);
            const std::vector<int64_t> expected = {stored, bytes / stored};
            if (r->dtype != "U8" || r->bytes != uint64_t(bytes) || r->shape != expected) return fail(which + " does not have the size its type and logical shape give it");
            return true;
        };
        if (!plane(w, name + ".weight", stored * groups * 16) || !plane(m, name + ".meta", stored * (groups / 8) * shape.meta_bytes)) return false;
        if (shape.plane1_bytes ? !plane(h, name + ".plane1", stored * groups * shape.plane1_bytes) : h != nullptr) return fail(shape.plane1_bytes ? error : name + ".weight has no second plane, yet " + name + ".plane1 exists");
        std::unique_ptr<uint8_t[]> native(new uint8_t[size_t(rows * (inner / 256) * shape.block_bytes)]);
        if (!planes_unpack(int(w->gguf_type), base + w->offset, h ? base + h->offset : nullptr, base + m->offset, rows, inner, native.get())) return fail(name + ": the planes cannot be unpacked");
        if (spl_weights_set_gguf(engine, layer, kind, int32_t(w->gguf_type), int32_t(rows), int32_t(inner), native.get()) != SPL_OK) return fail(name + ": " + spl_last_error_string(engine));
        return true;
    }
    bool q4(const std::string &name, int layer, int kind, int64_t rows, int64_t inner) {
        if (gguf) return planes(name, layer, kind, rows, inner);
        const Record *w = find(name + ".weight"), *s = find(name + ".scales"), *b = find(name + ".biases");
        if (!w) return fail("missing tensor language_model." + name + ".weight");
        if (w->dtype != "U32") return fail(name + ".weight is " + w->dtype + ", not U32");
        if (w->physical != w->shape || w->physical.size() != 2 || !w->has_logical || w->logical.size() != 2 || w->logical[0] != w->physical[0] || w->logical[1] != w->physical[1] * 8 ||
            w->physical[0] <= 0 || w->physical[1] <= 0) return fail("invalid physical/logical shape metadata for " + name + ".weight");
        if (!s || !b) return fail("missing sidecar for " + name + ".weight; expected " + name + ".scales and " + name + ".biases");
        if (s->dtype != "BF16" || b->dtype != "BF16") return fail("sidecars for " + name + ".weight must be BF16");
        const int64_t groups = (w->logical[1] + 63) / 64;
        const std::vector<int64_t> expected = {w->logical[0], groups};
        if (s->shape != expected || b->shape != expected) return fail("sidecar shape for " + name + ".weight is not [rows, groups]");
        if (w->logical[0] != rows || w->logical[1] != inner || groups * 64 != inner) return fail(name + " does not have the geometry's shape");
        if (w->bytes != uint64_t(rows * (inner / 8) * 4) || s->bytes != uint64_t(rows * groups * 2) || b->bytes != s->bytes) return fail(name + ": a record's byte length does not match its shape");
        const uint8_t *codes = base + w->offset, *scales = base + s->offset, *biases = base + b->offset;
        std::unique_ptr<uint8_t[]> moved;
        if (tiled && tiled_weight("language_model." + name + ".weight", rows)) {
            moved.reset(new uint8_t[w->bytes + 2 * s->bytes]);
            untile(codes, moved.get(), rows, groups, 32);
            untile(scales, moved.get() + w->bytes, rows, groups, 2);
            untile(biases, moved.get() + w->bytes + s->bytes, rows, groups, 2);
            codes = moved.get(); scales = codes + w->bytes; biases = scales + s->bytes;
        }
        if (spl_weights_set_q4(engine, layer, kind, int32_t(rows), int32_t(inner), reinterpret_cast<const uint32_t *>(codes), reinterpret_cast<const uint16_t *>(scales),
                               reinterpret_cast<const uint16_t *>(biases)) != SPL_OK) return fail(name + ": " + spl_last_error_string(engine));
        return true;
    }
    // A dense bf16 tensor of the given shape (WeightFile.denseBF16, ModelWeights.swift:201-207).
    bool dense(const std::string &name, int layer, int kind, const std::vector<int64_t> &shape) {
        const Record *r = find(name);
        if (!r) return fail("missing tensor language_model." + name);
        if (r->dtype != "BF16") return fail(name + " is " + r->dtype + ", not BF16");
        if (r->shape != shape) return fail(name + " does not have the geometry's shape");
        int64_t count = 1; for (int64_t e : shape) count *= e;
        if (r->bytes != uint64_t(count * 2)) return fail(name + ": the record's byte length does not match its shape");
        if (spl_weights_set_vector(engine, layer, kind, reinterpret_cast<const uint16_t *>(base + r->offset), int32_t(count)) != SPL_OK) return fail(name + ": " + spl_last_error_string(engine));
        return true;
    }
    // Every tensor of the model by name, each checked against the geometry (ModelWeights.resolve, ModelWeights.swift:181-248).
    bool load() {
        const int64_t H = g.hidden, D = g.gdn_head_dim, KH = g.gdn_key_heads, VH = g.gdn_value_heads, C = (2 * KH + VH) * D, VD = VH * D, AD = int64_t(g.heads) * g.head_dim, KV = int64_t(g.kv_heads) * g.head_dim;
        for (int layer = 0; layer < g.layers; ++layer) {
            const std::string p = "model.layers." + std::to_string(layer) + ".";
            if (layer % 4 == 3) {        // gated attention (Sources/SploshModel/LayerGraph.swift:22)
                if (!q4(p + "self_attn.q_proj", layer, SPL_Q4_Q, 2 * AD, H) || !q4(p + "self_attn.k_proj", layer, SPL_Q4_K, KV, H) || !q4(p + "self_attn.v_proj", layer, SPL_Q4_V, KV, H) ||
                    !q4(p + "self_attn.o_proj", layer, SPL_Q4_O, H, AD) || !dense(p + "self_attn.q_norm.weight", layer, SPL_VEC_Q_NORM, {g.head_dim}) ||
                    !dense(p + "self_attn.k_norm.weight", layer, SPL_VEC_K_NORM, {g.head_dim})) return false;
            } else {
                if (!q4(p + "linear_attn.in_proj_qkv", layer, SPL_Q4_QKV, C, H) || !q4(p + "linear_attn.in_proj_a", layer, SPL_Q4_A, VH, H) || !q4(p + "linear_attn.in_proj_b", layer, SPL_Q4_B, VH, H) ||
                    !q4(p + "linear_attn.in_proj_z", layer, SPL_Q4_Z, VD, H) || !q4(p + "linear_attn.out_proj", layer, SPL_Q4_OUT, H, VD) ||
                    !dense(p + "linear_attn.conv1d.weight", layer, SPL_VEC_CONV, {C, 4, 1}) || !dense(p + "linear_attn.A_log", layer, SPL_VEC_A_LOG, {VH}) ||
                    !dense(p + "linear_attn.dt_bias", layer, SPL_VEC_DT_BIAS, {VH}) || !dense(p + "linear_attn.norm.weight", layer, SPL_VEC_GDN_NORM, {D})) return false;
            }
            if (!dense(p + "input_layernorm.weight", layer, SPL_VEC_INPUT_NORM, {H}) || !dense(p + "post_attention_layernorm.weight", layer, SPL_VEC_POST_NORM, {H}) ||
                !q4(p + "mlp.gate_proj", layer, SPL_Q4_GATE, g.inter, H) || !q4(p + "mlp.up_proj", layer, SPL_Q4_UP, g.inter, H) || !q4(p + "mlp.down_proj", layer, SPL_Q4_DOWN, H, g.inter)) return false;
        }
        if (!q4("model.embed_tokens", -1, SPL_Q4_EMBED, g.vocab, H) || !q4("lm_head", -1, SPL_Q4_HEAD, g.vocab, H) || !dense("model.norm.weight", -1, SPL_VEC_FINAL_NORM, {H})) return false;
        // A GGUF-derived artifact leaves the out projections' columns in the file's order of the value heads (GgufConvert.swift:18-24).
        if (gguf && spl_weights_gguf_file_order(engine, 1) != SPL_OK) return fail(spl_last_error_string(engine));
        return true;
    }
};

struct Mapping {
    void *map = MAP_FAILED; size_t size = 0;
    ~Mapping() { if (map != MAP_FAILED) munmap(map, size); }
    // 0: mapped; 1: cannot open; 2: cannot map
    int open_file(const char *path) {
        const int fd = open(path, O_RDONLY);
        if (fd < 0) return 1;
        struct stat st;
        if (fstat(fd, &st) != 0) { close(fd); return 1; }
        size = size_t(st.st_size);
        if (size == 0) { close(fd); return 0; }
        map = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
        close(fd);
        return map == MAP_FAILED ? 2 : 0;
    }
};

spl_status say(char *message, size_t message_bytes, const std::string &text, spl_status status) {
    if (message && message_bytes) { const size_t n = std::min(text.size(), message_bytes - 1); memcpy(message, text.data(), n); message[n] = 0; }
    return status;
}

}  // namespace

extern "C" spl_status spl_gguf_planes_unpack(int32_t type, const uint8_t *plane0, const uint8_t *plane1, const uint8_t *meta, int32_t rows, int32_t inner, uint8_t *native) {
    PlaneShape shape;
    if (!plane_shape(type, &shape) || !plane0 || !meta || !native || (shape.plane1_bytes && !plane1)) return SPL_ERR_INVALID_ARGUMENT;
    return planes_unpack(type, plane0, plane1, meta, rows, inner, native) ? SPL_OK : SPL_ERR_INVALID_ARGUMENT;
}

extern "C" spl_status spl_splw_check(const char *path, int32_t *tensors, char *message, size_t message_bytes) {
    if (tensors) *tensors = 0;
    if (!path) return say(message, message_bytes, "null argument", SPL_ERR_INVALID_ARGUMENT);
    Mapping file;
    const int opened = file.open_file(path);
    if (opened == 1) return say(message, message_bytes, std::string("weight file missing: ") + path, SPL_ERR_INVALID_ARGUMENT);
    if (opened == 2) return say(message, message_bytes, "cannot map the file", SPL_ERR_ALLOCATION_FAILED);
    Container container;
    if (!container.parse(static_cast<const uint8_t *>(file.map == MAP_FAILED ? nullptr : file.map), file.size)) return say(message, message_bytes, "weight file invalid: " + container.error, SPL_ERR_INVALID_ARGUMENT);
    if (tensors) *tensors = int32_t(container.records.size());
    return say(message, message_bytes, container.format, SPL_OK);
}

extern "C" spl_status spl_weights_load_splw_file(spl_engine *engine, const char *path, char *message, size_t message_bytes) {
    if (!engine || !path) return say(message, message_bytes, "null argument", SPL_ERR_INVALID_ARGUMENT);
    Loader loader;
    loader.engine = engine;
    if (spl_engine_geometry(engine, &loader.g) != SPL_OK) return say(message, message_bytes, "no geometry", SPL_ERR_INVALID_ARGUMENT);
    Mapping file;
    const int opened = file.open_file(path);
    if (opened == 1) return say(message, message_bytes, std::string("weight file missing: ") + path, SPL_ERR_INVALID_ARGUMENT);
    if (opened == 2) return say(message, message_bytes, "cannot map the file", SPL_ERR_ALLOCATION_FAILED);
    Container container;
    if (!container.parse(static_cast<const uint8_t *>(file.map == MAP_FAILED ? nullptr : file.map), file.size)) return say(message, message_bytes, "weight file invalid: " + container.error, SPL_ERR_INVALID_ARGUMENT);
    if (container.format == "mlxAffine4") loader.tiled = false;
    else if (container.format == "mlxAffine4.tiled128") loader.tiled = true;
    else if (container.format == "gguf.tiled128") loader.gguf = true;
    else return say(message, message_bytes, "format " + container.format + " is not mlxAffine4, mlxAffine4.tiled128 or gguf.tiled128", SPL_ERR_INVALID_ARGUMENT);
    loader.file = &container; loader.base = static_cast<const uint8_t *>(file.map);
    if (!loader.load()) return say(message, message_bytes, loader.error, SPL_ERR_INVALID_ARGUMENT);
    return say(message, message_bytes, "", SPL_OK);
}

// The drafter's checkpoint, a bf16 safetensors file (MappedFile and SafetensorsHeader, Sources/SploshRuntime/DraftModel.swift:742-794):
// an 8-byte little-endian header length, a JSON object of {dtype, shape, data_offsets} per tensor name ("__metadata__" aside),
// then the data. Every tensor the drafter asks for is handed to spl_draft_set_tensor; refusals carry the reference's reasons.
extern "C" spl_status spl_draft_load_safetensors(spl_draft *draft, const char *path, char *message, size_t message_bytes) {
    if (!draft || !path) return say(message, message_bytes, "null argument", SPL_ERR_INVALID_ARGUMENT);
    Mapping file;
    const int opened = file.open_file(path);
    if (opened == 1) return say(message, message_bytes, std::string("draft model: cannot open ") + path, SPL_ERR_INVALID_ARGUMENT);
    if (opened == 2 || file.size <= 16 || file.map == MAP_FAILED) return say(message, message_bytes, std::string("draft model: cannot map ") + path, SPL_ERR_INVALID_ARGUMENT);
    const uint8_t *base = static_cast<const uint8_t *>(file.map);
    uint64_t header_length = 0;
    memcpy(&header_length, base, 8);
    if (header_length == 0 || header_length > file.size - 8) return say(message, message_bytes, "draft model: bad safetensors header", SPL_ERR_INVALID_ARGUMENT);
    JsonReader reader{reinterpret_cast<const char *>(base + 8), reinterpret_cast<const char *>(base + 8 + header_length)};
    const Json header = reader.value();
    reader.space();
    if (!reader.ok || reader.p != reader.end || header.kind != Json::Object) return say(message, message_bytes, "draft model: safetensors header is not an object", SPL_ERR_INVALID_ARGUMENT);
    struct Entry { std::string dtype; std::vector<int64_t> shape; uint64_t offset = 0, length = 0; };
    std::vector<std::pair<std::string, Entry>> entries;
    for (const auto &field : header.fields) {
        if (field.first == "__metadata__") continue;
        const Json &t = field.second;
        Entry en;
        uint64_t begin = 0, end = 0;
        const Json *dtype = t.kind == Json::Object ? t.get("dtype") : nullptr, *offsets = t.kind == Json::Object ? t.get("data_offsets") : nullptr;
        if (!dtype || dtype->kind != Json::String || !shape_of(t.get("shape"), &en.shape) || !offsets || offsets->kind != Json::Array || offsets->items.size() != 2 ||
            !integer_of(&offsets->items[0], &begin) || !integer_of(&offsets->items[1], &end) || end < begin || 8 + header_length + end > file.size)
            return say(message, message_bytes, "draft model: malformed tensor entry " + field.first, SPL_ERR_INVALID_ARGUMENT);
        en.dtype = dtype->text; en.offset = 8 + header_length + begin; en.length = end - begin;
        entries.emplace_back(field.first, std::move(en));
    }
    auto shape_text = [](const std::vector<int64_t> &shape) {
        std::string out = "[";
        for (size_t i = 0; i < shape.size(); ++i) out += (i ? ", " : "") + std::to_string(shape[i]);
        return out + "]";
    };
    const int count = spl_draft_tensor_count(draft);
    for (int index = 0; index < count; ++index) {
        char name[160]; int64_t dims[4]; int32_t nd = 0;
        if (spl_draft_tensor_expected(draft, index, name, sizeof name, dims, &nd) != SPL_OK) return say(message, message_bytes, "draft model: no such tensor", SPL_ERR_INVALID_ARGUMENT);
        const std::vector<int64_t> want(dims, dims + nd);
        const Entry *found = nullptr;
        for (const auto &en : entries) if (en.first == name) { found = &en.second; break; }
        if (!found) return say(message, message_bytes, std::string("draft model: missing tensor ") + name, SPL_ERR_INVALID_ARGUMENT);
        int64_t elements = 1;
        for (int64_t v : want) elements *= v;
        if (found->dtype != "BF16" || found->shape != want || found->length != uint64_t(elements) * 2)
            return say(message, message_bytes, std::string("draft model: ") + name + " is " + found->dtype + " " + shape_text(found->shape) + "; expected BF16 " + shape_text(want), SPL_ERR_INVALID_ARGUMENT);
        const int64_t rows = nd == 1 ? 1 : want[0];
        const spl_status s = spl_draft_set_tensor(draft, name, reinterpret_cast<const uint16_t *>(base + found->offset), int32_t(rows), int32_t(elements / rows));
        if (s != SPL_OK) return say(message, message_bytes, std::string("draft model: ") + name + " was refused", s);
    }
    return say(message, message_bytes, "", SPL_OK);
}
