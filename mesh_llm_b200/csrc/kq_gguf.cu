// GGUF container reader and the per-stage selective load (host code only).
//
// A mesh-llm worker is started with the path of its local GGUF file and pulls exactly the tensors
// it owns out of that file by name instead of receiving them over the wire (SET_TENSOR_GGUF,
// third_party/llama.cpp/patches/0001 lines 179-266: look the tensor name up in the file's index,
// seek to data_offset + tensor_offset, read ggml_nbytes, hand the bytes to the backend's
// set_tensor).  The header scan follows the limits and the derived fields of the reference's own
// scanner (mesh-client/src/models/gguf.rs:4-9 limits, :319-421 compact metadata, :476-572 byte
// profile by offset differences).
#include "kq_common.cuh"

#include <errno.h>
#include <fcntl.h>
#include <stdio.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

namespace {

constexpr uint64_t MAX_STRING_BYTES = 1000000, MAX_ARRAY_ELEMENTS = 1000000, MAX_KV_COUNT = 1000000,
                   MAX_TENSOR_COUNT = 1000000;
constexpr uint32_t MAX_ARRAY_DEPTH = 64, MAX_TENSOR_DIMS = 8;

enum GgufVal : uint32_t {
    V_U8 = 0, V_I8, V_U16, V_I16, V_U32, V_I32, V_F32, V_BOOL, V_STRING, V_ARRAY, V_U64, V_I64, V_F64, V_COUNT
};

struct TensorInfo {
    std::string name;
    uint32_t type = 0, n_dims = 0;
    int64_t ne[4] = {1, 1, 1, 1};
    uint64_t offset = 0; // relative to the data section
    uint64_t nbytes = 0; // from type and shape; 0 if the type is not known
    uint64_t pos_dims = 0, pos_offset = 0; // where the shape and the offset sit in the file
};

// elements per block and bytes per block of the ggml tensor types
bool type_size(uint32_t t, uint32_t &blck, uint32_t &bytes) {
    switch (t) {
    case 0: blck = 1; bytes = 4; return true;     // F32
    case 1: blck = 1; bytes = 2; return true;     // F16
    case 2: blck = 32; bytes = 18; return true;   // Q4_0
    case 3: blck = 32; bytes = 20; return true;   // Q4_1
    case 6: blck = 32; bytes = 22; return true;   // Q5_0
    case 7: blck = 32; bytes = 24; return true;   // Q5_1
    case 8: blck = 32; bytes = 34; return true;   // Q8_0
    case 10: blck = 256; bytes = 84; return true; // Q2_K
    case 11: blck = 256; bytes = 110; return true;
    case 12: blck = 256; bytes = 144; return true; // Q4_K
    case 13: blck = 256; bytes = 176; return true;
    case 14: blck = 256; bytes = 210; return true; // Q6_K
    case 15: blck = 256; bytes = 292; return true; // Q8_K
    case 24: blck = 1; bytes = 1; return true;
    case 25: blck = 1; bytes = 2; return true;
    case 26: blck = 1; bytes = 4; return true;
    case 27: blck = 1; bytes = 8; return true;
    case 28: blck = 1; bytes = 8; return true;
    case 30: blck = 1; bytes = 2; return true; // BF16
    default: return false;
    }
}

struct Reader {
    int fd = -1;
    uint64_t pos = 0, len = 0;
    std::string err;
    bool fail(const char *what) {
        if (err.empty()) err = what;
        return false;
    }
    bool read(void *dst, size_t n) {
        if (pos + n > len) return fail("unexpected end of file");
        size_t done = 0;
        while (done < n) {
            const ssize_t r = pread(fd, (char *)dst + done, n - done, (off_t)(pos + done));
            if (r <= 0) return fail("read failed");
            done += (size_t)r;
        }
        pos += n;
        return true;
    }
    template <typename T>
    bool get(T &v) { return read(&v, sizeof(T)); }
    bool skip(uint64_t n) {
        if (pos + n > len) return fail("unexpected end of file");
        pos += n;
        return true;
    }
    bool str(std::string &s) {
        uint64_t n = 0;
        if (!get(n)) return false;
        if (n > MAX_STRING_BYTES) return fail("string too long");
        s.resize((size_t)n);
        return n == 0 || read(&s[0], (size_t)n);
    }
    bool count(uint64_t max, const char *neg, const char *big, uint64_t &out) { // header counts are signed
        int64_t v = 0;
        if (!get(v)) return false;
        if (v < 0) return fail(neg);
        if ((uint64_t)v > max) return fail(big);
        out = (uint64_t)v;
        return true;
    }
    static int scalar_bytes(uint32_t t) {
        switch (t) {
        case V_U8: case V_I8: case V_BOOL: return 1;
        case V_U16: case V_I16: return 2;
        case V_U32: case V_I32: case V_F32: return 4;
        case V_U64: case V_I64: case V_F64: return 8;
        default: return 0;
        }
    }
    bool skip_value(uint32_t t, uint32_t depth) {
        if (t >= V_COUNT) return fail("unknown value type");
        if (t == V_STRING) {
            uint64_t n = 0;
            if (!get(n)) return false;
            if (n > MAX_STRING_BYTES) return fail("string too long");
            return skip(n);
        }
        if (t == V_ARRAY) {
            if (depth >= MAX_ARRAY_DEPTH) return fail("nesting too deep");
            uint32_t et = 0;
            uint64_t n = 0;
            if (!get(et) || !get(n)) return false;
            if (et >= V_COUNT) return fail("unknown value type");
            if (n > MAX_ARRAY_ELEMENTS) return fail("array too long");
            if (const int sb = scalar_bytes(et)) return skip(n * (uint64_t)sb);
            for (uint64_t i = 0; i < n; i++)
                if (!skip_value(et, depth + 1)) return false;
            return true;
        }
        return skip((uint64_t)scalar_bytes(t));
    }
    // integer value as u32; negative or too large values are invalid; other types are skipped
    bool as_u32(uint32_t t, bool &have, uint32_t &out) {
        have = false;
        int64_t v = 0;
        switch (t) {
        case V_U8: { uint8_t x; if (!get(x)) return false; v = x; break; }
        case V_I8: { int8_t x; if (!get(x)) return false; v = x; break; }
        case V_U16: { uint16_t x; if (!get(x)) return false; v = x; break; }
        case V_I16: { int16_t x; if (!get(x)) return false; v = x; break; }
        case V_U32: { uint32_t x; if (!get(x)) return false; v = x; break; }
        case V_I32: { int32_t x; if (!get(x)) return false; v = x; break; }
        case V_U64: { uint64_t x; if (!get(x)) return false; if (x > 0xFFFFFFFFull) return fail("value does not fit u32"); v = (int64_t)x; break; }
        case V_I64: { int64_t x; if (!get(x)) return false; v = x; break; }
        default: return skip_value(t, 0);
        }
        if (v < 0) return fail("negative value where an unsigned one is expected");
        if (v > 0xFFFFFFFFll) return fail("value does not fit u32");
        have = true;
        out = (uint32_t)v;
        return true;
    }
    bool as_f32(uint32_t t, bool &have, float &out) {
        have = false;
        if (t == V_F32) { if (!get(out)) return false; have = true; return true; }
        if (t == V_F64) { double d; if (!get(d)) return false; out = (float)d; have = true; return true; }
        return skip_value(t, 0);
    }
};

bool ends_with(const std::string &s, const char *suffix) {
    const size_t n = strlen(suffix);
    return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}

bool expert_partitioned(const std::string &name) { // mesh-client/src/models/gguf.rs:455-469
    std::string l = name;
    std::transform(l.begin(), l.end(), l.begin(), [](unsigned char c) { return (char)tolower(c); });
    if (l.find("shared_expert") != std::string::npos || l.find("sharedexpert") != std::string::npos ||
        l.find("shexp") != std::string::npos)
        return false;
    for (const char *k : {"ffn_gate_exps", "ffn_up_exps", "ffn_down_exps", "exp_probs", ".expert", "_expert"})
        if (l.find(k) != std::string::npos) return true;
    return false;
}

} // namespace

struct b200_gguf {
    int fd = -1;
    uint64_t file_len = 0, data_start = 0, tensor_info_end = 0;
    uint32_t version = 0, alignment = 32;
    b200_gguf_meta meta;
    // file position and value type of the two counts a shard writer has to change (0: key absent)
    uint64_t pos_expert_count = 0, pos_expert_used = 0;
    uint32_t vt_expert_count = 0, vt_expert_used = 0;
    std::vector<TensorInfo> tensors;
    std::map<std::string, int> index;
};

b200_status b200_gguf_open(const char *path, b200_gguf **out) {
    KQ_REQUIRE(path && out, "gguf_open: null argument");
    *out = nullptr;
    const int fd = open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) {
        kq_set_error("gguf_open: cannot open %s: %s", path, strerror(errno));
        return B200_ERR_INVALID;
    }
    struct stat sb;
    if (fstat(fd, &sb) != 0) {
        close(fd);
        kq_set_error("gguf_open: cannot stat %s", path);
        return B200_ERR_INVALID;
    }
    b200_gguf *g = new b200_gguf();
    g->fd = fd;
    g->file_len = (uint64_t)sb.st_size;
    memset(&g->meta, 0, sizeof(g->meta));
    Reader r;
    r.fd = fd;
    r.len = g->file_len;
    auto bad = [&](const char *what) {
        kq_set_error("gguf_open: %s: %s", path, what);
        close(fd);
        delete g;
        return B200_ERR_INVALID;
    };
    char magic[4];
    if (!r.read(magic, 4) || memcmp(magic, "GGUF", 4) != 0) return bad("not a GGUF file");
    if (!r.get(g->version)) return bad(r.err.c_str());
    if (g->version < 2) return bad("GGUF version below 2");
    uint64_t n_tensors = 0, n_kv = 0;
    if (!r.count(MAX_TENSOR_COUNT, "negative tensor count", "tensor count too large", n_tensors)) return bad(r.err.c_str());
    if (!r.count(MAX_KV_COUNT, "negative KV count", "KV count too large", n_kv)) return bad(r.err.c_str());

    b200_gguf_meta &m = g->meta;
    for (uint64_t i = 0; i < n_kv; i++) {
        std::string key;
        uint32_t vt = 0;
        if (!r.str(key) || !r.get(vt)) return bad(r.err.c_str());
        if (vt >= V_COUNT) return bad("unknown value type");
        bool have = false;
        uint32_t u = 0;
        float f = 0.f;
        bool ok = true;
        if (key == "general.architecture" || key == "tokenizer.ggml.model") {
            if (vt != V_STRING) return bad("string value expected");
            std::string s;
            ok = r.str(s);
            if (ok) snprintf(key == "general.architecture" ? m.architecture : m.tokenizer_model, 64, "%s", s.c_str());
        } else if (key == "general.alignment") {
            ok = r.as_u32(vt, have, u);
            if (have) g->alignment = u ? u : 1;
        } else if (ends_with(key, ".context_length")) { ok = r.as_u32(vt, have, u); if (have) m.context_length = u; }
        else if (ends_with(key, ".embedding_length")) { ok = r.as_u32(vt, have, u); if (have) m.embedding_length = u; }
        else if (ends_with(key, ".attention.head_count_kv")) { ok = r.as_u32(vt, have, u); if (have) m.head_count_kv = u; }
        else if (ends_with(key, ".head_count")) { ok = r.as_u32(vt, have, u); if (have) m.head_count = u; }
        else if (ends_with(key, ".block_count")) { ok = r.as_u32(vt, have, u); if (have) m.block_count = u; }
        else if (ends_with(key, ".expert_feed_forward_length")) { ok = r.as_u32(vt, have, u); if (have) m.expert_feed_forward_length = u; }
        else if (ends_with(key, ".feed_forward_length")) { ok = r.as_u32(vt, have, u); if (have) m.feed_forward_length = u; }
        else if (ends_with(key, ".attention.key_length")) { ok = r.as_u32(vt, have, u); if (have) m.key_length = u; }
        else if (ends_with(key, ".attention.value_length")) { ok = r.as_u32(vt, have, u); if (have) m.value_length = u; }
        else if (ends_with(key, ".vocab_size")) { ok = r.as_u32(vt, have, u); if (have) m.vocab_size = u; }
        else if (ends_with(key, ".expert_used_count")) {
            g->pos_expert_used = r.pos; g->vt_expert_used = vt;
            ok = r.as_u32(vt, have, u); if (have) m.expert_used_count = u;
        } else if (ends_with(key, ".expert_count")) {
            g->pos_expert_count = r.pos; g->vt_expert_count = vt;
            ok = r.as_u32(vt, have, u); if (have) m.expert_count = u;
        }
        else if (ends_with(key, ".rope.freq_base")) { ok = r.as_f32(vt, have, f); if (have) m.rope_freq_base = f; }
        else if (ends_with(key, ".rope.scale")) { ok = r.as_f32(vt, have, f); if (have) m.rope_scale = f; }
        else if (ends_with(key, ".attention.layer_norm_rms_epsilon")) { ok = r.as_f32(vt, have, f); if (have) m.rms_epsilon = f; }
        else ok = r.skip_value(vt, 0);
        if (!ok) return bad(r.err.c_str());
    }
    if (m.head_count > 0) { // derived lengths, as the reference derives them
        if (m.key_length == 0) m.key_length = m.embedding_length / m.head_count;
    }
    if (m.value_length == 0) {
        const uint32_t kv = m.head_count_kv ? m.head_count_kv : m.head_count;
        if (kv) m.value_length = m.embedding_length / kv;
    }

    g->tensors.reserve((size_t)n_tensors);
    for (uint64_t i = 0; i < n_tensors; i++) {
        TensorInfo t;
        if (!r.str(t.name) || !r.get(t.n_dims)) return bad(r.err.c_str());
        if (t.n_dims > MAX_TENSOR_DIMS) return bad("too many tensor dimensions");
        uint64_t elems = 1;
        t.pos_dims = r.pos;
        for (uint32_t d = 0; d < t.n_dims; d++) {
            uint64_t ne = 0;
            if (!r.get(ne)) return bad(r.err.c_str());
            if (d < 4) t.ne[d] = (int64_t)ne;
            else if (ne != 1) t.ne[3] = -1; // more than four real dimensions: not addressable here
            if (ne != 0 && elems > (1ull << 62) / ne) return bad("tensor too large");
            elems *= ne;
        }
        if (!r.get(t.type)) return bad(r.err.c_str());
        t.pos_offset = r.pos;
        if (!r.get(t.offset)) return bad(r.err.c_str());
        uint32_t blck = 0, bytes = 0;
        if (type_size(t.type, blck, bytes) && t.n_dims > 0 && t.ne[0] % blck == 0) t.nbytes = elems / blck * bytes;
        g->index[t.name] = (int)g->tensors.size();
        g->tensors.push_back(std::move(t));
    }
    g->tensor_info_end = r.pos;
    const uint64_t al = g->alignment;
    g->data_start = (r.pos + al - 1) / al * al;
    if (n_tensors > 0 && g->data_start > g->file_len) return bad("data section starts past the end of the file");
    for (const TensorInfo &t : g->tensors)
        if (t.offset > g->file_len - std::min(g->file_len, g->data_start) ||
            (t.nbytes && t.offset + t.nbytes > g->file_len - g->data_start))
            return bad("tensor data outside the file");
    if (m.vocab_size == 0) { // not every architecture stores it: the embedding matrix has it
        auto it = g->index.find("token_embd.weight");
        if (it != g->index.end()) m.vocab_size = (uint32_t)g->tensors[it->second].ne[1];
    }
    *out = g;
    return B200_OK;
}

void b200_gguf_close(b200_gguf *g) {
    if (!g) return;
    if (g->fd >= 0) close(g->fd);
    delete g;
}

b200_status b200_gguf_get_meta(const b200_gguf *g, b200_gguf_meta *out) {
    KQ_REQUIRE(g && out, "gguf_get_meta: null argument");
    *out = g->meta;
    return B200_OK;
}

int64_t b200_gguf_tensor_count(const b200_gguf *g) { return g ? (int64_t)g->tensors.size() : -1; }

b200_status b200_gguf_tensor_info(const b200_gguf *g, int64_t i, b200_gguf_tensor *out) {
    KQ_REQUIRE(g && out, "gguf_tensor_info: null argument");
    KQ_REQUIRE(i >= 0 && i < (int64_t)g->tensors.size(), "gguf_tensor_info: index %lld out of range", (long long)i);
    const TensorInfo &t = g->tensors[(size_t)i];
    memset(out, 0, sizeof(*out));
    snprintf(out->name, sizeof(out->name), "%s", t.name.c_str());
    out->type = t.type;
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; d++) out->ne[d] = t.ne[d];
    out->file_offset = g->data_start + t.offset;
    out->nbytes = t.nbytes;
    return B200_OK;
}

int64_t b200_gguf_find_tensor(const b200_gguf *g, const char *name) {
    if (!g || !name) return -1;
    auto it = g->index.find(name);
    return it == g->index.end() ? -1 : it->second;
}

b200_status b200_gguf_read_tensor(const b200_gguf *g, int64_t i, void *dst, size_t nbytes) {
    KQ_REQUIRE(g && dst, "gguf_read_tensor: null argument");
    KQ_REQUIRE(i >= 0 && i < (int64_t)g->tensors.size(), "gguf_read_tensor: index %lld out of range", (long long)i);
    const TensorInfo &t = g->tensors[(size_t)i];
    KQ_REQUIRE(t.nbytes != 0, "gguf_read_tensor: %s has a type (%u) whose size is not known", t.name.c_str(), t.type);
    if (nbytes != t.nbytes) {
        kq_set_error("gguf_read_tensor: %s holds %llu bytes, caller asked for %zu", t.name.c_str(),
                     (unsigned long long)t.nbytes, nbytes);
        return B200_ERR_BOUNDS;
    }
    size_t done = 0;
    while (done < nbytes) {
        const ssize_t r = pread(g->fd, (char *)dst + done, nbytes - done, (off_t)(g->data_start + t.offset + done));
        if (r <= 0) {
            kq_set_error("gguf_read_tensor: short read for %s: got %zu of %zu bytes", t.name.c_str(), done, nbytes);
            return B200_ERR_INVALID;
        }
        done += (size_t)r;
    }
    return B200_OK;
}

b200_status b200_gguf_byte_profile(const b200_gguf *g, b200_gguf_byte_profile_t *out) {
    KQ_REQUIRE(g && out, "gguf_byte_profile: null argument");
    memset(out, 0, sizeof(*out));
    out->expert_count = g->meta.expert_count;
    out->expert_used_count = g->meta.expert_used_count;
    out->full_model_bytes = g->file_len;
    if (g->tensors.empty()) {
        out->file_overhead_bytes = g->file_len;
        return B200_OK;
    }
    const uint64_t data_len = g->file_len - g->data_start;
    std::vector<const TensorInfo *> order;
    for (const TensorInfo &t : g->tensors) order.push_back(&t);
    std::stable_sort(order.begin(), order.end(), [](const TensorInfo *a, const TensorInfo *b) { return a->offset < b->offset; });
    for (size_t i = 0; i < order.size(); i++) {
        const uint64_t next = i + 1 < order.size() ? order[i + 1]->offset : data_len;
        KQ_REQUIRE(next >= order[i]->offset && next <= data_len, "gguf_byte_profile: tensor offsets are not consistent");
        const uint64_t bytes = next - order[i]->offset; // padding up to the next tensor counts with the tensor
        (expert_partitioned(order[i]->name) ? out->expert_tensor_bytes : out->base_resident_bytes) += bytes;
    }
    out->file_overhead_bytes = g->file_len - (out->base_resident_bytes + out->expert_tensor_bytes);
    return B200_OK;
}

void b200_kv_types_for_model_bytes(uint64_t model_bytes, uint32_t *k_type, uint32_t *v_type) {
    const uint64_t GB = 1000000000ull; // decimal, as the tiers are defined
    uint32_t k = B200_TYPE_F16, v = B200_TYPE_F16;
    if (model_bytes >= 50 * GB) {
        k = B200_TYPE_Q4_0;
        v = B200_TYPE_Q4_0;
    } else if (model_bytes >= 5 * GB) {
        k = B200_TYPE_Q8_0;
        v = B200_TYPE_Q4_0;
    }
    if (k_type) *k_type = k;
    if (v_type) *v_type = v;
}

b200_status b200_gguf_stage_config(const b200_gguf *g, int32_t layer_begin, int32_t layer_end, int32_t n_ctx,
                                   int32_t n_seq, int32_t n_ubatch, int32_t device, b200_stage_config *cfg) {
    KQ_REQUIRE(g && cfg, "gguf_stage_config: null argument");
    const b200_gguf_meta &m = g->meta;
    KQ_REQUIRE(m.block_count > 0 && m.embedding_length > 0 && m.head_count > 0,
               "gguf_stage_config: the file lacks block_count / embedding_length / head_count");
    memset(cfg, 0, sizeof(*cfg));
    cfg->n_layer = (int32_t)m.block_count;
    cfg->layer_begin = layer_begin;
    cfg->layer_end = layer_end < 0 ? cfg->n_layer : layer_end;
    KQ_REQUIRE(cfg->layer_begin >= 0 && cfg->layer_begin <= cfg->layer_end && cfg->layer_end <= cfg->n_layer,
               "gguf_stage_config: layer range [%d, %d) outside [0, %d)", layer_begin, layer_end, cfg->n_layer);
    cfg->n_embd = (int32_t)m.embedding_length;
    cfg->n_head = (int32_t)m.head_count;
    cfg->n_head_kv = (int32_t)(m.head_count_kv ? m.head_count_kv : m.head_count);
    cfg->head_dim = (int32_t)(m.key_length ? m.key_length : m.embedding_length / m.head_count);
    cfg->n_vocab = (int32_t)m.vocab_size;
    cfg->n_expert = (int32_t)m.expert_count;
    cfg->n_expert_used = (int32_t)m.expert_used_count;
    cfg->n_ff_exp = (int32_t)m.expert_feed_forward_length;
    cfg->n_ff = cfg->n_expert > 0 ? 0 : (int32_t)m.feed_forward_length;
    cfg->n_ctx = n_ctx;
    cfg->n_seq = n_seq;
    cfg->n_ubatch = n_ubatch;
    cfg->device = device;
    cfg->rms_eps = m.rms_epsilon > 0.f ? m.rms_epsilon : 1e-5f;
    cfg->rope_theta = m.rope_freq_base > 0.f ? m.rope_freq_base : 10000.f;
    // rotary pairing by architecture family: llama-style adjacent pairs, everything Qwen-like (i, i + hd/2)
    const std::string arch = m.architecture;
    cfg->rope_neox = !(arch == "llama" || arch == "mistral" || arch == "llama4");
    char probe[64];
    snprintf(probe, sizeof(probe), "blk.%d.attn_q.bias", cfg->layer_begin < cfg->n_layer ? cfg->layer_begin : 0);
    cfg->qkv_bias = g->index.count(probe) ? 1 : (g->index.count("blk.0.attn_q.bias") ? 1 : 0);
    cfg->qk_norm = g->index.count("blk.0.attn_q_norm.weight") ? 1 : 0;
    cfg->has_embd = cfg->layer_begin == 0;
    cfg->has_output = cfg->layer_end == cfg->n_layer;
    return B200_OK;
}

b200_status b200_stage_load_gguf(b200_stage *st, const b200_gguf *g, int64_t *n_loaded, int64_t *bytes_read) {
    KQ_REQUIRE(st && g, "stage_load_gguf: null argument");
    int64_t loaded = 0, total = 0;
    std::vector<uint8_t> host;
    const int64_t n = b200_stage_tensor_count(st);
    for (int64_t i = 0; i < n; i++) {
        char name[96];
        uint32_t want_type = 0;
        int64_t ne[3];
        b200_status rc = b200_stage_tensor_info(st, i, name, sizeof(name), &want_type, ne);
        if (rc != B200_OK) return rc;
        auto it = g->index.find(name);
        if (it == g->index.end() && strcmp(name, "output.weight") == 0) it = g->index.find("token_embd.weight"); // tied head
        if (it == g->index.end()) {
            kq_set_error("stage_load_gguf: the file has no tensor %s", name);
            return B200_ERR_STATE;
        }
        const TensorInfo &t = g->tensors[(size_t)it->second];
        if (t.type != B200_TYPE_F32 && t.type != B200_TYPE_Q4_K && t.type != B200_TYPE_Q6_K) {
            kq_set_error("stage_load_gguf: %s is stored as ggml type %u; this path takes F32, Q4_K and Q6_K", name, t.type);
            return B200_ERR_UNSUPPORTED;
        }
        const int64_t rows_file = t.ne[1] * t.ne[2] * (t.ne[3] > 0 ? t.ne[3] : 1);
        if (t.ne[0] != ne[0] || rows_file != ne[1] * ne[2]) {
            kq_set_error("stage_load_gguf: %s is [%lld x %lld] in the file, the stage expects [%lld x %lld]", name,
                         (long long)t.ne[0], (long long)rows_file, (long long)ne[0], (long long)(ne[1] * ne[2]));
            return B200_ERR_INVALID;
        }
        host.resize((size_t)t.nbytes);
        rc = b200_gguf_read_tensor(g, it->second, host.data(), (size_t)t.nbytes);
        if (rc != B200_OK) return rc;
        rc = b200_stage_set_tensor(st, name, t.type, host.data(), (size_t)t.nbytes);
        if (rc != B200_OK) return rc;
        loaded++;
        total += (int64_t)t.nbytes;
    }
    if (n_loaded) *n_loaded = loaded;
    if (bytes_read) *bytes_read = total;
    return B200_OK;
}

// ---- expert shards ---------------------------------------------------------------------------
// Which experts each node of a group holds.  The ranking lists expert ids from the most to the
// least used.  mode 0 (mesh-llm/src/inference/moe.rs:535-591): the first min_experts are a shared
// core on every node, the others go round-robin, each to `overlap` consecutive nodes.  mode 1
// (moe.rs:597-636): shared core of min_experts, the others dealt in snake order.  The node's list
// comes back sorted, without duplicates.
b200_status b200_moe_assign(const uint32_t *ranking, int32_t n_expert, int32_t n_nodes, int32_t min_experts,
                            int32_t overlap, int32_t mode, int32_t node, uint32_t *experts_out, int32_t cap,
                            int32_t *n_out, int32_t *n_shared, int32_t *n_unique) {
    KQ_REQUIRE(ranking && experts_out && n_out, "moe_assign: null argument");
    KQ_REQUIRE(n_expert >= 1 && min_experts >= 0 && (mode == 0 || mode == 1), "moe_assign: bad argument");
    if (n_nodes < 1) n_nodes = 1;
    KQ_REQUIRE(node >= 0 && node < n_nodes, "moe_assign: node %d of %d", node, n_nodes);
    std::vector<uint32_t> mine;
    int shared = 0, unique = 0;
    if (n_nodes <= 1 || min_experts >= n_expert) { // one node, or the core covers everything
        mine.assign(ranking, ranking + n_expert); // in ranking order, as the reference returns it
        shared = n_expert;
    } else {
        mine.assign(ranking, ranking + min_experts);
        shared = min_experts;
        const int ov = mode == 0 ? std::max(1, std::min(overlap, n_nodes)) : 1;
        for (int i = 0; i < n_expert - min_experts; i++) {
            const uint32_t e = ranking[min_experts + i];
            if (mode == 0) {
                for (int j = 0; j < ov; j++)
                    if ((i + j) % n_nodes == node) { mine.push_back(e); unique++; }
            } else {
                const int round = i / n_nodes, pos = i % n_nodes;
                if ((round % 2 == 0 ? pos : n_nodes - 1 - pos) == node) { mine.push_back(e); unique++; }
            }
        }
        std::sort(mine.begin(), mine.end());
        mine.erase(std::unique(mine.begin(), mine.end()), mine.end());
    }
    KQ_REQUIRE((int)mine.size() <= cap, "moe_assign: %zu experts do not fit the caller's %d slots", mine.size(), cap);
    for (size_t i = 0; i < mine.size(); i++) experts_out[i] = mine[i];
    *n_out = (int32_t)mine.size();
    if (n_shared) *n_shared = shared;
    if (n_unique) *n_unique = unique;
    return B200_OK;
}

namespace {
bool expert_packed(const std::string &n) { // llama-moe-split: patches/0003 lines 945-955
    return n.find("ffn_gate_exps") != std::string::npos || n.find("ffn_up_exps") != std::string::npos ||
           n.find("ffn_down_exps") != std::string::npos || n.find("ffn_gate_inp") != std::string::npos;
}
bool copy_range(int fd_in, uint64_t src, int fd_out, uint64_t dst, uint64_t n, std::vector<uint8_t> &buf) {
    buf.resize(1 << 22);
    while (n > 0) {
        const size_t c = (size_t)std::min<uint64_t>(n, buf.size());
        size_t done = 0;
        while (done < c) {
            const ssize_t r = pread(fd_in, buf.data() + done, c - done, (off_t)(src + done));
            if (r <= 0) return false;
            done += (size_t)r;
        }
        done = 0;
        while (done < c) {
            const ssize_t w = pwrite(fd_out, buf.data() + done, c - done, (off_t)(dst + done));
            if (w <= 0) return false;
            done += (size_t)w;
        }
        src += c;
        dst += c;
        n -= c;
    }
    return true;
}
} // namespace

// Writes a GGUF file that holds the trunk of `src` and only the listed experts: the expert-packed
// tensors are cut on their last dimension, the rows of the router gate are gathered in the same
// order, expert_count becomes the number of experts kept and expert_used_count is clamped to it
// (llama-moe-split, patches/0003 lines 1040-1113 and 1142-1191).  Every other byte of the header is
// carried over unchanged.
b200_status b200_gguf_write_expert_shard(const b200_gguf *g, const int32_t *expert_ids, int32_t n_ids,
                                         const char *dst_path, uint64_t *bytes_written) {
    KQ_REQUIRE(g && expert_ids && dst_path, "write_expert_shard: null argument");
    const uint32_t E = g->meta.expert_count;
    KQ_REQUIRE(E > 1 && g->pos_expert_count != 0, "write_expert_shard: the file is not a mixture-of-experts model");
    KQ_REQUIRE(n_ids >= 1 && (uint32_t)n_ids <= E, "write_expert_shard: %d experts of %u", n_ids, E);
    for (int i = 0; i < n_ids; i++) {
        KQ_REQUIRE(expert_ids[i] >= 0 && (uint32_t)expert_ids[i] < E, "write_expert_shard: expert id %d out of range", expert_ids[i]);
        for (int j = 0; j < i; j++) KQ_REQUIRE(expert_ids[j] != expert_ids[i], "write_expert_shard: expert id %d listed twice", expert_ids[i]);
    }
    auto four_byte_int = [](uint32_t vt) { return vt == V_U32 || vt == V_I32; };
    KQ_REQUIRE(four_byte_int(g->vt_expert_count) && (g->pos_expert_used == 0 || four_byte_int(g->vt_expert_used)),
               "write_expert_shard: expert counts are not stored as 32-bit integers");
    std::vector<uint8_t> head((size_t)g->tensor_info_end);
    {
        size_t done = 0;
        while (done < head.size()) {
            const ssize_t r = pread(g->fd, head.data() + done, head.size() - done, (off_t)done);
            KQ_REQUIRE(r > 0, "write_expert_shard: cannot re-read the header");
            done += (size_t)r;
        }
    }
    auto put32 = [&](uint64_t pos, uint32_t v) { memcpy(head.data() + pos, &v, 4); };
    auto put64 = [&](uint64_t pos, uint64_t v) { memcpy(head.data() + pos, &v, 8); };
    put32(g->pos_expert_count, (uint32_t)n_ids);
    if (g->pos_expert_used) put32(g->pos_expert_used, std::min<uint32_t>(g->meta.expert_used_count, (uint32_t)n_ids));

    struct Plan { uint64_t new_off, new_bytes, per_expert; bool cut; };
    std::vector<Plan> plan(g->tensors.size());
    uint64_t off = 0;
    const uint64_t al = g->alignment;
    for (size_t i = 0; i < g->tensors.size(); i++) {
        const TensorInfo &t = g->tensors[i];
        KQ_REQUIRE(t.nbytes != 0, "write_expert_shard: %s has a type (%u) whose size is not known", t.name.c_str(), t.type);
        Plan &p = plan[i];
        const uint32_t ed = t.n_dims ? t.n_dims - 1 : 0;
        const int64_t ne_last = t.n_dims == 0 ? 1 : (ed < 4 ? t.ne[ed] : 1);
        p.cut = expert_packed(t.name) && t.n_dims >= 2 && ed < 4 && ne_last == (int64_t)E; // other shapes are copied as they are
        p.per_expert = p.cut ? t.nbytes / E : 0;
        p.new_bytes = p.cut ? p.per_expert * (uint64_t)n_ids : t.nbytes;
        p.new_off = off;
        off += (p.new_bytes + al - 1) / al * al;
        put64(t.pos_offset, p.new_off);
        if (p.cut) put64(t.pos_dims + 8ull * ed, (uint64_t)n_ids);
    }
    const int fd = open(dst_path, O_WRONLY | O_CREAT | O_TRUNC | O_CLOEXEC, 0644);
    if (fd < 0) {
        kq_set_error("write_expert_shard: cannot create %s: %s", dst_path, strerror(errno));
        return B200_ERR_INVALID;
    }
    std::vector<uint8_t> buf;
    bool ok = pwrite(fd, head.data(), head.size(), 0) == (ssize_t)head.size();
    const uint64_t total = g->data_start + off;
    if (ok) ok = ftruncate(fd, (off_t)total) == 0; // alignment gaps read back as zeros
    for (size_t i = 0; ok && i < g->tensors.size(); i++) {
        const TensorInfo &t = g->tensors[i];
        const Plan &p = plan[i];
        const uint64_t src = g->data_start + t.offset, dst = g->data_start + p.new_off;
        if (!p.cut) {
            ok = copy_range(g->fd, src, fd, dst, t.nbytes, buf);
        } else {
            for (int e = 0; ok && e < n_ids; e++)
                ok = copy_range(g->fd, src + (uint64_t)expert_ids[e] * p.per_expert, fd, dst + (uint64_t)e * p.per_expert,
                                p.per_expert, buf);
        }
    }
    if (close(fd) != 0) ok = false;
    if (!ok) {
        kq_set_error("write_expert_shard: I/O error while writing %s", dst_path);
        return B200_ERR_INVALID;
    }
    if (bytes_written) *bytes_written = total;
    return B200_OK;
}
