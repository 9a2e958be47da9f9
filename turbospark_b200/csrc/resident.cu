// The resident weight file's leading index region, and a loader that hands its block tensors to a model.
//
// File layout (crates/model-io/src/resident_index.rs:19-67, written by crates/repack/src/resident_writer.rs:375-470):
//   header  24 B: u64 index_size (whole index region, header included), u64 resident_size, u64 entry_count
//   entries 72 B each: u32 name_offset, u16 name_length, u8 dtype, u8 reserved, u64 file_offset, u64 size_bytes,
//           u32 shape[4], u64 scale_offset, u64 scale_size, u64 bias_offset, u64 bias_size
//   string table, zero padding to the writer's page size, and in the last 16 bytes of the region an optional
//   trailer: "GTURBIDX", u32 format version, u32 reserved.  Tensor bytes start at file byte index_size.
// Everything here is host code: the parser needs no device, the loader copies verbatim block rows to the model.
#include "model.cuh"

#include <cinttypes>
#include <cstdarg>
#include <cstring>
#include <memory>
#include <cstdio>
#include <map>

namespace {

constexpr uint64_t HEADER_BYTES = 24, ENTRY_BYTES = 72, TRAILER_BYTES = 16;
constexpr uint32_t FORMAT_VERSION = 1;
const char INDEX_MAGIC[9] = "GTURBIDX";

thread_local std::string g_resident_error;

int32_t fail(int32_t code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_resident_error = buf;
    return code;
}

uint64_t rd64(const uint8_t* p) {
    uint64_t v = 0;
    for (int i = 7; i >= 0; i--) v = (v << 8) | p[i];
    return v;
}
uint32_t rd32(const uint8_t* p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }

bool add_overflows(uint64_t a, uint64_t b, uint64_t* out) { return __builtin_add_overflow(a, b, out); }
bool mul_overflows(uint64_t a, uint64_t b, uint64_t* out) { return __builtin_mul_overflow(a, b, out); }

}  // namespace

struct tsb_resident {
    std::string path;
    uint64_t index_size = 0, resident_size = 0;
    std::vector<std::string> names;
    std::vector<tsb_resident_entry> entries;
    std::map<std::string, size_t> by_name;
};

// resident_index.rs:83-127: the fixed 4-bit / 8-bit affine entries must carry planes of exactly the declared shape
static int32_t validate_affine(const std::string& name, const tsb_resident_entry& e) {
    uint64_t bits;
    if (e.dtype == 4) bits = 4;
    else if (e.dtype == 5) bits = 8;
    else return TSB_OK;
    const uint64_t rows = e.shape[0], cols = e.shape[1];
    if (rows == 0 || cols == 0 || cols % 64 != 0)
        return fail(TSB_ERR_INVALID, "index corrupt: tensor %s has invalid affine shape %" PRIu64 "x%" PRIu64, name.c_str(), rows, cols);
    uint64_t elements, packed_bits, companions;
    if (mul_overflows(rows, cols, &elements) || mul_overflows(elements, bits, &packed_bits))
        return fail(TSB_ERR_INVALID, "index corrupt: tensor %s shape overflows", name.c_str());
    if (mul_overflows(rows, cols / 64, &companions) || mul_overflows(companions, 2, &companions))
        return fail(TSB_ERR_INVALID, "index corrupt: tensor %s companion size overflows", name.c_str());
    if (e.size_bytes != packed_bits / 8 || e.scale_size != companions || e.bias_size != companions)
        return fail(TSB_ERR_INVALID, "index corrupt: tensor %s affine planes are %" PRIu64 ", %" PRIu64 " and %" PRIu64 " bytes; shape requires %" PRIu64 ", %" PRIu64 " and %" PRIu64,
                    name.c_str(), e.size_bytes, e.scale_size, e.bias_size, packed_bits / 8, companions, companions);
    if (e.scale_offset % 2 != 0 || e.bias_offset % 2 != 0)
        return fail(TSB_ERR_INVALID, "index corrupt: tensor %s affine companion offsets are not 2-byte aligned", name.c_str());
    return TSB_OK;
}

extern "C" {

const char* tsb_resident_last_error(void) { return g_resident_error.c_str(); }

// resident_index.rs:131-317 (load + check_trailer): every offset an entry names is checked against the file here,
// because no later consumer re-checks it.
int32_t tsb_resident_open(const char* path, tsb_resident** out) {
    if (!path || !out) return fail(TSB_ERR_INVALID, "null argument");
    *out = nullptr;
    FILE* f = fopen(path, "rb");
    if (!f) return fail(TSB_ERR_INVALID, "open failed: %s", path);
    struct Closer {
        FILE* f;
        ~Closer() { fclose(f); }
    } closer{f};
    if (fseeko(f, 0, SEEK_END) != 0) return fail(TSB_ERR_INVALID, "stat failed: %s", path);
    const uint64_t file_len = (uint64_t)ftello(f);
    if (fseeko(f, 0, SEEK_SET) != 0) return fail(TSB_ERR_INVALID, "seek failed: %s", path);
    uint8_t hb[HEADER_BYTES];
    if (fread(hb, 1, HEADER_BYTES, f) != HEADER_BYTES) return fail(TSB_ERR_INVALID, "index corrupt: short read for IndexHeader");
    const uint64_t index_size = rd64(hb), resident_size = rd64(hb + 8), entry_count = rd64(hb + 16);
    if (index_size < HEADER_BYTES) return fail(TSB_ERR_INVALID, "index corrupt: indexSize %" PRIu64 " < header size 24", index_size);
    uint64_t table_bytes, table_end, region_end;
    if (mul_overflows(entry_count, ENTRY_BYTES, &table_bytes))
        return fail(TSB_ERR_INVALID, "index corrupt: entryCount %" PRIu64 " overflows the entry table", entry_count);
    if (add_overflows(HEADER_BYTES, table_bytes, &table_end)) return fail(TSB_ERR_INVALID, "index corrupt: header + entry table size overflows");
    if (table_end > index_size)
        return fail(TSB_ERR_INVALID, "index corrupt: header+entries (%" PRIu64 ") > indexSize %" PRIu64, table_end, index_size);
    if (add_overflows(index_size, resident_size, &region_end)) return fail(TSB_ERR_INVALID, "index corrupt: indexSize + residentSize overflows");
    if (region_end > file_len)
        return fail(TSB_ERR_INVALID, "index corrupt: indexSize %" PRIu64 " + residentSize %" PRIu64 " = %" PRIu64 " exceeds file length %" PRIu64,
                    index_size, resident_size, region_end, file_len);
    std::vector<uint8_t> buf;
    try {
        buf.resize((size_t)index_size);
    } catch (...) {
        return fail(TSB_ERR_OOM, "index region of %" PRIu64 " bytes does not fit in memory", index_size);
    }
    if (fseeko(f, 0, SEEK_SET) != 0 || fread(buf.data(), 1, buf.size(), f) != buf.size())
        return fail(TSB_ERR_INVALID, "index corrupt: short read for index region");

    std::unique_ptr<tsb_resident> idx(new (std::nothrow) tsb_resident());
    if (!idx) return fail(TSB_ERR_OOM, "out of memory");
    idx->path = path, idx->index_size = index_size, idx->resident_size = resident_size;
    uint64_t string_table_end = table_end;
    auto in_region = [&](uint64_t off, uint64_t size) {
        uint64_t end;
        return size == 0 || (off >= index_size && !add_overflows(off, size, &end) && end <= region_end);
    };
    for (uint64_t i = 0; i < entry_count; i++) {
        const uint8_t* p = buf.data() + HEADER_BYTES + i * ENTRY_BYTES;
        const uint64_t name_off = rd32(p), name_len = (uint64_t)p[4] | ((uint64_t)p[5] << 8);
        tsb_resident_entry e{};
        e.dtype = p[6];
        e.file_offset = rd64(p + 8), e.size_bytes = rd64(p + 16);
        for (int k = 0; k < 4; k++) e.shape[k] = rd32(p + 24 + 4 * k);
        e.scale_offset = rd64(p + 40), e.scale_size = rd64(p + 48), e.bias_offset = rd64(p + 56), e.bias_size = rd64(p + 64);
        if (name_off < HEADER_BYTES || name_off + name_len > index_size)
            return fail(TSB_ERR_INVALID, "index corrupt: entry %" PRIu64 " name range [%" PRIu64 ", %" PRIu64 ") out of index region [24, %" PRIu64 ")",
                        i, name_off, name_off + name_len, index_size);
        std::string name((const char*)buf.data() + name_off, (size_t)name_len);
        string_table_end = std::max(string_table_end, name_off + name_len);
        if (!in_region(e.file_offset, e.size_bytes))
            return fail(TSB_ERR_INVALID, "index corrupt: entry %" PRIu64 " (%s) payload [%" PRIu64 ", +%" PRIu64 ") outside the resident region [%" PRIu64 ", %" PRIu64 ")",
                        i, name.c_str(), e.file_offset, e.size_bytes, index_size, region_end);
        if (!in_region(e.scale_offset, e.scale_size))
            return fail(TSB_ERR_INVALID, "index corrupt: entry %" PRIu64 " (%s) scale plane [%" PRIu64 ", +%" PRIu64 ") outside the resident region [%" PRIu64 ", %" PRIu64 ")",
                        i, name.c_str(), e.scale_offset, e.scale_size, index_size, region_end);
        if (!in_region(e.bias_offset, e.bias_size))
            return fail(TSB_ERR_INVALID, "index corrupt: entry %" PRIu64 " (%s) bias plane [%" PRIu64 ", +%" PRIu64 ") outside the resident region [%" PRIu64 ", %" PRIu64 ")",
                        i, name.c_str(), e.bias_offset, e.bias_size, index_size, region_end);
        int32_t rc = validate_affine(name, e);
        if (rc) return rc;
        if (idx->by_name.count(name)) return fail(TSB_ERR_INVALID, "index corrupt: duplicate tensor name %s", name.c_str());
        idx->by_name[name] = idx->entries.size();
        idx->names.push_back(name);
        idx->entries.push_back(e);
    }
    // the trailer counts only past the string table, so a legacy name ending in the magic bytes is not one
    if (index_size >= TRAILER_BYTES && index_size - TRAILER_BYTES >= string_table_end) {
        const uint8_t* t = buf.data() + (index_size - TRAILER_BYTES);
        if (memcmp(t, INDEX_MAGIC, 8) == 0) {
            const uint32_t found = rd32(t + 8);
            if (found != FORMAT_VERSION)
                return fail(TSB_ERR_UNSUPPORTED, "index format %u is not supported (this reader implements format %u)", found, FORMAT_VERSION);
        }
    }
    *out = idx.release();
    return TSB_OK;
}

void tsb_resident_close(tsb_resident* idx) { delete idx; }

int64_t tsb_resident_count(const tsb_resident* idx) { return idx ? (int64_t)idx->entries.size() : 0; }
uint64_t tsb_resident_index_size(const tsb_resident* idx) { return idx ? idx->index_size : 0; }
uint64_t tsb_resident_data_size(const tsb_resident* idx) { return idx ? idx->resident_size : 0; }

int32_t tsb_resident_entry_at(const tsb_resident* idx, int64_t i, tsb_resident_entry* out, char* name_buf, int32_t name_cap) {
    if (!idx || !out || i < 0 || i >= (int64_t)idx->entries.size()) return fail(TSB_ERR_INVALID, "entry index out of range");
    *out = idx->entries[(size_t)i];
    if (name_buf && name_cap > 0) snprintf(name_buf, (size_t)name_cap, "%s", idx->names[(size_t)i].c_str());
    return TSB_OK;
}

int32_t tsb_resident_find(const tsb_resident* idx, const char* name, tsb_resident_entry* out) {
    if (!idx || !name || !out) return fail(TSB_ERR_INVALID, "null argument");
    auto it = idx->by_name.find(name);
    if (it == idx->by_name.end()) return fail(TSB_ERR_INVALID, "tensor %s is not in the index", name);
    *out = idx->entries[it->second];
    return TSB_OK;
}

// dtype tags of the block formats (crates/repack/src/resident_writer.rs:103-162)
int32_t tsb_resident_qtype_of(int32_t dtype_tag) {
    switch (dtype_tag) {
        case 7: return TSB_Q4_K;
        case 8: return TSB_Q6_K;
        case 14: return TSB_MXFP4;
        case 13: return TSB_Q5_K;
        case 6: return TSB_Q8_0;
        default: return -1;
    }
}

// Reads the Llama-family tensor set the reference's runner looks up by name
// (crates/runtime/src/families/llama/mod.rs:49-51,99,371-386; attn.rs:173-197,438; dense.rs:60-62) into `m`:
// embedding, per layer input_layernorm / q,k,v,o / post_attention_layernorm / gate,up,down, final norm, head
// (the embedding again when tied).  Sizes are checked against the model's shape as encode_gemm_any does
// (real_forward_dispatch.rs:1008-1016): a dtype/byte-count mismatch is refused, never reinterpreted.
int32_t tsb_model_load_resident(tsb_model* m, const tsb_resident* idx, int32_t tie_word_embeddings) {
    if (!m || !idx) return TSB_ERR_INVALID;
    tsb_ctx* ctx = m->ctx;
    const tsb_model_config& c = m->cfg;
    FILE* f = fopen(idx->path.c_str(), "rb");
    if (!f) return tsb_fail(ctx, TSB_ERR_INVALID, "open failed: %s", idx->path.c_str());
    struct Closer {
        FILE* f;
        ~Closer() { fclose(f); }
    } closer{f};
    std::vector<uint8_t> host;
    auto read_entry = [&](const std::string& name, const tsb_resident_entry** e_out) -> int32_t {
        auto it = idx->by_name.find(name);
        if (it == idx->by_name.end()) return tsb_fail(ctx, TSB_ERR_INVALID, "tensor %s is not in the index", name.c_str());
        const tsb_resident_entry& e = idx->entries[it->second];
        try {
            host.resize((size_t)e.size_bytes);
        } catch (...) {
            return tsb_fail(ctx, TSB_ERR_OOM, "tensor %s (%" PRIu64 " bytes) does not fit in host memory", name.c_str(), e.size_bytes);
        }
        if (fseeko(f, (off_t)e.file_offset, SEEK_SET) != 0 || fread(host.data(), 1, host.size(), f) != host.size())
            return tsb_fail(ctx, TSB_ERR_INVALID, "short read for tensor %s", name.c_str());
        *e_out = &e;
        return TSB_OK;
    };
    auto matrix = [&](const std::string& name, int layer, int which, int64_t rows, int64_t cols) -> int32_t {
        const tsb_resident_entry* e;
        int32_t rc = read_entry(name, &e);
        if (rc) return rc;
        const int qt = tsb_resident_qtype_of(e->dtype);
        if (qt < 0) return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "tensor %s has dtype tag %d, which is not one of the block formats", name.c_str(), (int)e->dtype);
        const int64_t expected = tsb_row_bytes(qt, cols) * rows;
        if ((int64_t)e->size_bytes != expected)
            return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "tensor %s: %" PRIu64 " bytes does not match %lld x %lld of its block format (%lld bytes)",
                            name.c_str(), e->size_bytes, (long long)rows, (long long)cols, (long long)expected);
        return tsb_model_set_matrix(m, layer, which, qt, host.data(), rows, cols);
    };
    auto norm = [&](const std::string& name, int layer, int which) -> int32_t {
        const tsb_resident_entry* e;
        int32_t rc = read_entry(name, &e);
        if (rc) return rc;
        if (e->size_bytes != (uint64_t)c.d_model * 2)  // real_forward_utils.rs:241-256: norms are BF16 [d_model]
            return tsb_fail(ctx, TSB_ERR_UNSUPPORTED, "tensor %s: %" PRIu64 " bytes does not match expected BF16 [%d]", name.c_str(), e->size_bytes, c.d_model);
        return tsb_model_set_norm(m, layer, which, host.data(), c.d_model);
    };
    const int64_t qd = (int64_t)c.n_q_heads * c.head_dim, kd = (int64_t)c.n_kv_heads * c.head_dim;
    const std::string embed = "language_model.model.embed_tokens.weight";
    int32_t rc;
    if ((rc = matrix(embed, 0, TSB_W_EMBED, c.vocab, c.d_model))) return rc;
    for (int L = 0; L < c.n_layers; L++) {
        const std::string p = "language_model.model.layers." + std::to_string(L) + ".";
        if ((rc = norm(p + "input_layernorm.weight", L, TSB_N_ATTN)) || (rc = matrix(p + "self_attn.q_proj.weight", L, TSB_W_Q, qd, c.d_model)) ||
            (rc = matrix(p + "self_attn.k_proj.weight", L, TSB_W_K, kd, c.d_model)) || (rc = matrix(p + "self_attn.v_proj.weight", L, TSB_W_V, kd, c.d_model)) ||
            (rc = matrix(p + "self_attn.o_proj.weight", L, TSB_W_O, c.d_model, qd)) || (rc = norm(p + "post_attention_layernorm.weight", L, TSB_N_FFN)) ||
            (rc = matrix(p + "mlp.gate_proj.weight", L, TSB_W_GATE, c.ffn, c.d_model)) || (rc = matrix(p + "mlp.up_proj.weight", L, TSB_W_UP, c.ffn, c.d_model)) ||
            (rc = matrix(p + "mlp.down_proj.weight", L, TSB_W_DOWN, c.d_model, c.ffn)))
            return rc;
    }
    if ((rc = norm("language_model.model.norm.weight", 0, TSB_N_OUT))) return rc;
    return matrix(tie_word_embeddings ? embed : std::string("language_model.lm_head.weight"), 0, TSB_W_LM_HEAD, c.vocab, c.d_model);
}

}  // extern "C"
