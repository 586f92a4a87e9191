// Direct GGUF -> device load of a gpt2-architecture model: the tensors go to the GPU as they
// are stored (raw Q8_0 blocks, f32 vectors), with no f32 expansion of the matrices in between.
//
// Follows the reference's reader: container layout gguf/header.rs:9-66 (magic, version 2 or 3,
// metadata, tensor directory, aligned data section; general.alignment, default 32), value tags
// gguf/format.rs:60-90, and the gpt2 tensor contract loader/gpt2.rs:201-262 (gpt2.* keys,
// layer_norm_epsilon must be 1e-5, token rows permuted by the tokenizer's id layout, tied
// head when output.weight is absent). The reference expands every matrix to f32
// (loader/decode.rs) and names the direct path as future work (loader/decode.rs:99-100).
// Host code only: parsing and validation need no GPU (fc_gguf_probe).
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/ferrum_cuda.h"
#include "llama_native.h"

namespace fc {
int fail(int code, const char* fmt, ...);
}
using fc::fail;

namespace {

constexpr uint32_t kMagic = 0x46554747u;   // "GGUF"
constexpr uint32_t T_F32 = 0, T_Q8_0 = 8;   // the types this engine computes on; the others are converted at load
enum : uint32_t { VT_U8, VT_I8, VT_U16, VT_I16, VT_U32, VT_I32, VT_F32, VT_BOOL, VT_STRING, VT_ARRAY, VT_U64, VT_I64, VT_F64 };

struct Tensor {
    uint32_t type = 0;
    std::vector<uint64_t> dims;   // ne0 first (the contiguous dimension)
    uint64_t offset = 0;          // relative to the data section
    uint64_t nbytes = 0;
};

struct Meta {
    uint32_t type = 0;
    uint64_t u = 0;
    double f = 0.0;
    std::string s;                // VT_STRING values shorter than 256 bytes (names, not vocabularies)
};

struct File {
    // matrices stored in another block format, brought to Q8_0 on first use: Q4_0 / Q5_0 re-blocked exactly (same scale,
    // integer levels), the formats with minima or sub-block scales (Q4_1, Q5_1, Q8_1, the K-quants) and f16 / f32
    // matrices decoded and re-encoded with the Q8_0 block encoder
    mutable std::map<std::string, std::vector<uint8_t>> reblocked;
    std::vector<uint8_t> bytes;
    std::map<std::string, Meta> meta;        // scalars and short strings (arrays are skipped)
    std::map<std::string, Tensor> tensors;
    uint64_t data = 0;                        // absolute offset of the data section
    uint64_t align = 32;                      // general.alignment: every tensor offset is a multiple of it
};

struct Cursor {
    const uint8_t* p;
    size_t n, pos = 0;
    bool ok = true;
    bool need(size_t k) {
        if (!ok || k > n - pos) { ok = false; return false; }
        return true;
    }
    template <class T>
    T get() {
        T v{};
        if (need(sizeof(T))) { memcpy(&v, p + pos, sizeof(T)); pos += sizeof(T); }
        return v;
    }
    std::string str() {
        const uint64_t len = get<uint64_t>();
        if (!need((size_t)len) || len > (1u << 24)) { ok = false; return std::string(); }
        std::string s((const char*)p + pos, (size_t)len);
        pos += (size_t)len;
        return s;
    }
};

size_t scalar_size(uint32_t t) {
    switch (t) {
        case VT_U8: case VT_I8: case VT_BOOL: return 1;
        case VT_U16: case VT_I16: return 2;
        case VT_U32: case VT_I32: case VT_F32: return 4;
        case VT_U64: case VT_I64: case VT_F64: return 8;
        default: return 0;
    }
}

// Reads one metadata value; scalars are kept, strings and arrays are walked over.
bool read_value(Cursor& c, uint32_t type, Meta* out) {
    out->type = type;
    switch (type) {
        case VT_U8: out->u = c.get<uint8_t>(); break;
        case VT_I8: out->u = (uint64_t)(int64_t)c.get<int8_t>(); break;
        case VT_U16: out->u = c.get<uint16_t>(); break;
        case VT_I16: out->u = (uint64_t)(int64_t)c.get<int16_t>(); break;
        case VT_U32: out->u = c.get<uint32_t>(); break;
        case VT_I32: out->u = (uint64_t)(int64_t)c.get<int32_t>(); break;
        case VT_F32: out->f = c.get<float>(); break;
        case VT_BOOL: out->u = c.get<uint8_t>(); break;
        case VT_U64: out->u = c.get<uint64_t>(); break;
        case VT_I64: out->u = (uint64_t)c.get<int64_t>(); break;
        case VT_F64: out->f = c.get<double>(); break;
        case VT_STRING: out->s = c.str(); if (out->s.size() >= 256) out->s.clear(); break;
        case VT_ARRAY: {
            const uint32_t et = c.get<uint32_t>();
            const uint64_t count = c.get<uint64_t>();
            if (et == VT_STRING) {
                for (uint64_t i = 0; i < count && c.ok; ++i) c.str();
            } else if (et == VT_ARRAY) {
                c.ok = false;   // nested arrays do not occur in model files
            } else {
                const size_t sz = scalar_size(et);
                if (!sz || count > (c.n - c.pos) / sz) c.ok = false;
                else c.pos += (size_t)count * sz;
            }
            break;
        }
        default: c.ok = false;
    }
    return c.ok;
}

// gguf/format.rs:107-130: every tensor type the reference's importer reads; 0 for the others
uint64_t type_nbytes(uint32_t type, uint64_t n) { return (uint64_t)fc_ggml_type_bytes((int)type, (size_t)n); }

int read_file(const char* path, File* f) {
    FILE* fp = fopen(path, "rb");
    if (!fp) return fail(FC_E_FORMAT, "cannot open %s", path);
    fseek(fp, 0, SEEK_END);
    const long size = ftell(fp);
    fseek(fp, 0, SEEK_SET);
    if (size <= 0) { fclose(fp); return fail(FC_E_FORMAT, "%s is empty", path); }
    f->bytes.resize((size_t)size);
    const size_t got = fread(f->bytes.data(), 1, (size_t)size, fp);
    fclose(fp);
    if (got != (size_t)size) return fail(FC_E_FORMAT, "short read of %s", path);

    Cursor c{f->bytes.data(), f->bytes.size()};
    if (c.get<uint32_t>() != kMagic) return fail(FC_E_FORMAT, "not a GGUF file (bad magic)");
    const uint32_t version = c.get<uint32_t>();
    if (version != 2 && version != 3) return fail(FC_E_FORMAT, "unsupported GGUF version %u (need 2 or 3)", version);
    const uint64_t n_tensors = c.get<uint64_t>(), n_meta = c.get<uint64_t>();
    if (!c.ok || n_tensors > (1u << 20) || n_meta > (1u << 20)) return fail(FC_E_FORMAT, "GGUF header is truncated or implausible");
    for (uint64_t i = 0; i < n_meta; ++i) {
        const std::string key = c.str();
        const uint32_t type = c.get<uint32_t>();
        Meta m;
        if (!read_value(c, type, &m)) return fail(FC_E_FORMAT, "GGUF metadata entry %llu (%s) is malformed", (unsigned long long)i, key.c_str());
        if (type != VT_ARRAY) f->meta[key] = m;
    }
    for (uint64_t i = 0; i < n_tensors; ++i) {
        const std::string name = c.str();
        Tensor t;
        const uint32_t nd = c.get<uint32_t>();
        if (!c.ok || nd == 0 || nd > 4) return fail(FC_E_FORMAT, "GGUF tensor %s has %u dimensions", name.c_str(), nd);
        uint64_t n = 1;
        for (uint32_t k = 0; k < nd; ++k) {
            t.dims.push_back(c.get<uint64_t>());
            if (t.dims.back() == 0 || t.dims.back() > (1ull << 40) || n > (1ull << 50) / t.dims.back()) c.ok = false;
            else n *= t.dims.back();
        }
        t.type = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        if (!c.ok) return fail(FC_E_FORMAT, "GGUF tensor directory is truncated at %s", name.c_str());
        t.nbytes = type_nbytes(t.type, n);
        if (!f->tensors.emplace(name, t).second) return fail(FC_E_FORMAT, "GGUF tensor %s appears twice in the directory", name.c_str());
    }
    uint64_t align = 32;
    auto it = f->meta.find("general.alignment");
    if (it != f->meta.end()) align = it->second.u;
    if (align == 0 || (align & (align - 1))) return fail(FC_E_FORMAT, "general.alignment %llu is not a power of two", (unsigned long long)align);
    f->data = (c.pos + align - 1) / align * align;
    f->align = align;
    return FC_OK;
}

int meta_int(const File& f, const char* key, int* out) {
    auto it = f.meta.find(key);
    if (it == f.meta.end()) return fail(FC_E_FORMAT, "GGUF metadata key %s is missing", key);
    const Meta& m = it->second;
    if (m.type == VT_F32 || m.type == VT_F64 || m.type == VT_BOOL || m.type == VT_STRING || m.u > (1u << 30)) return fail(FC_E_FORMAT, "GGUF metadata key %s is not a small integer", key);
    *out = (int)m.u;
    return FC_OK;
}

// The tensor `name` with the given type and dims (ne0, ne1); returns its bytes.
int tensor(const File& f, const std::string& name, uint32_t type, uint64_t ne0, uint64_t ne1, const uint8_t** out) {
    auto it = f.tensors.find(name);
    if (it == f.tensors.end()) return fail(FC_E_FORMAT, "GGUF tensor %s is missing", name.c_str());
    const Tensor& t = it->second;
    const bool reblock = type == T_Q8_0 && t.type != T_Q8_0 && type_nbytes(t.type, 256) != 0;
    if (t.type != type && !reblock)
        return fail(FC_E_FORMAT, "GGUF tensor %s has ggml type %u, this engine needs %u (%s)", name.c_str(), t.type, type,
                    type == T_Q8_0 ? "matrices are Q8_0, or one of the block formats of gguf/dequant.rs brought to it" : "vectors are F32");
    const uint64_t d0 = t.dims[0], d1 = t.dims.size() > 1 ? t.dims[1] : 1;
    for (size_t k = 2; k < t.dims.size(); ++k)
        if (t.dims[k] != 1) return fail(FC_E_FORMAT, "GGUF tensor %s has more than two dimensions", name.c_str());
    if (d0 != ne0 || d1 != ne1)
        return fail(FC_E_FORMAT, "GGUF tensor %s is [%llu][%llu], expected [%llu][%llu]", name.c_str(), (unsigned long long)d1,
                    (unsigned long long)d0, (unsigned long long)ne1, (unsigned long long)ne0);
    // compared without additions, so that a crafted offset near 2^64 cannot wrap
    const uint64_t size = f.bytes.size();
    if (t.nbytes == 0 || f.data > size || t.offset > size - f.data || t.nbytes > size - f.data - t.offset)
        return fail(FC_E_FORMAT, "GGUF tensor %s runs past the end of the file", name.c_str());
    if (t.offset % f.align)
        return fail(FC_E_FORMAT, "GGUF tensor %s starts at offset %llu, not a multiple of general.alignment %llu", name.c_str(),
                    (unsigned long long)t.offset, (unsigned long long)f.align);
    *out = f.bytes.data() + f.data + t.offset;
    if (reblock) {
        std::vector<uint8_t>& store = f.reblocked[name];
        if (store.empty()) {
            const uint64_t n = d0 * d1;
            store.resize((size_t)(n / 32 * 34));
            if (n % 32 || fc_ggml_requantize_q8_0((int)t.type, *out, (size_t)t.nbytes, (size_t)n, store.data()) != FC_OK)
                return fail(FC_E_FORMAT, "GGUF tensor %s (ggml type %u) could not be brought to Q8_0", name.c_str(), t.type);
        }
        *out = store.data();
    }
    return FC_OK;
}

struct Parsed {
    fc_config cfg{};
    std::vector<fc_layer_weights> layers;
    fc_weights w{};
    std::vector<std::vector<float>> owned_f32;       // vectors copied out of the file (alignment)
    std::vector<uint8_t> tok_perm, head_perm;         // row-permuted copies of the token / head tables
};

// F32 tensor copied into owned storage: file offsets are only guaranteed 32-byte aligned
// relative to the data section, which is enough for floats, but a copy keeps the file buffer
// free to go away independently of the pointers handed on.
int f32_vec(const File& f, Parsed* p, const std::string& name, uint64_t ne0, uint64_t ne1, const float** out) {
    const uint8_t* b = nullptr;
    int rc = tensor(f, name, T_F32, ne0, ne1, &b);
    if (rc != FC_OK) return rc;
    p->owned_f32.emplace_back((size_t)(ne0 * ne1));
    memcpy(p->owned_f32.back().data(), b, (size_t)(ne0 * ne1) * 4);
    *out = p->owned_f32.back().data();
    return FC_OK;
}

int parse_model(const File& f, const int32_t* row_perm, int n_perm, int math_mode, Parsed* p) {
    int ctx = 0, d = 0, L = 0, F = 0, H = 0;
    int rc;
    if ((rc = meta_int(f, "gpt2.context_length", &ctx)) != FC_OK) return rc;
    if ((rc = meta_int(f, "gpt2.embedding_length", &d)) != FC_OK) return rc;
    if ((rc = meta_int(f, "gpt2.block_count", &L)) != FC_OK) return rc;
    if ((rc = meta_int(f, "gpt2.feed_forward_length", &F)) != FC_OK) return rc;
    if ((rc = meta_int(f, "gpt2.attention.head_count", &H)) != FC_OK) return rc;
    auto eps = f.meta.find("gpt2.attention.layer_norm_epsilon");
    if (eps == f.meta.end() || (eps->second.type != VT_F32 && eps->second.type != VT_F64))
        return fail(FC_E_FORMAT, "GGUF metadata key gpt2.attention.layer_norm_epsilon is missing");
    if (eps->second.f < 1e-5 - 1e-9 || eps->second.f > 1e-5 + 1e-9)
        return fail(FC_E_FORMAT, "gpt2.attention.layer_norm_epsilon is %g; the LayerNorm here uses 1e-5", eps->second.f);
    if (ctx <= 0 || d <= 0 || L <= 0 || F <= 0 || H <= 0) return fail(FC_E_FORMAT, "gpt2.* dimensions must be positive");
    auto te = f.tensors.find("token_embd.weight");
    if (te == f.tensors.end() || te->second.dims.size() < 2) return fail(FC_E_FORMAT, "GGUF tensor token_embd.weight is missing");
    const uint64_t v_file = te->second.dims[1];
    const int V = row_perm ? n_perm : (int)v_file;
    if (V <= 0 || (uint64_t)V > v_file) return fail(FC_E_FORMAT, "row permutation has %d entries, the file holds %llu token rows", V, (unsigned long long)v_file);
    const bool tied = f.tensors.find("output.weight") == f.tensors.end();

    const size_t row_bytes = (size_t)d / 32 * 34;
    // perm[ferrum_id] = file_id (loader/gpt2.rs:189-199 permute_rows)
    auto permuted = [&](const std::string& name, std::vector<uint8_t>* store, const void** out) -> int {
        const uint8_t* b = nullptr;
        int r = tensor(f, name, T_Q8_0, (uint64_t)d, v_file, &b);
        if (r != FC_OK) return r;
        if (!row_perm) { *out = b; return FC_OK; }
        store->resize((size_t)V * row_bytes);
        for (int i = 0; i < V; ++i) {
            if (row_perm[i] < 0 || (uint64_t)row_perm[i] >= v_file) return fail(FC_E_DIM, "row permutation entry %d = %d is outside the %llu token rows", i, row_perm[i], (unsigned long long)v_file);
            memcpy(store->data() + (size_t)i * row_bytes, b + (size_t)row_perm[i] * row_bytes, row_bytes);
        }
        *out = store->data();
        return FC_OK;
    };
    if (d % 32) return fail(FC_E_FORMAT, "embedding_length %d is not a multiple of 32: its matrices cannot be Q8_0 (loader/mod.rs:147-154)", d);
    if ((rc = permuted("token_embd.weight", &p->tok_perm, &p->w.token_embd_q8)) != FC_OK) return rc;
    if (!tied && (rc = permuted("output.weight", &p->head_perm, &p->w.output_q8)) != FC_OK) return rc;
    if ((rc = f32_vec(f, p, "position_embd.weight", d, ctx, &p->w.position_embd)) != FC_OK) return rc;
    p->layers.resize(L);
    for (int i = 0; i < L; ++i) {
        fc_layer_weights& lw = p->layers[i];
        const std::string n = "blk." + std::to_string(i) + ".";
        const uint8_t* b = nullptr;
        if ((rc = tensor(f, n + "attn_qkv.weight", T_Q8_0, d, 3ull * d, &b)) != FC_OK) return rc;
        lw.attn_qkv_q8 = b;
        if ((rc = tensor(f, n + "attn_output.weight", T_Q8_0, d, d, &b)) != FC_OK) return rc;
        lw.attn_out_q8 = b;
        if ((rc = tensor(f, n + "ffn_up.weight", T_Q8_0, d, F, &b)) != FC_OK) return rc;
        lw.ffn_up_q8 = b;
        if ((rc = tensor(f, n + "ffn_down.weight", T_Q8_0, F, d, &b)) != FC_OK) return rc;
        lw.ffn_down_q8 = b;
        if ((rc = f32_vec(f, p, n + "attn_qkv.bias", 3ull * d, 1, &lw.attn_qkv_b)) != FC_OK) return rc;
        if ((rc = f32_vec(f, p, n + "attn_output.bias", d, 1, &lw.attn_out_b)) != FC_OK) return rc;
        if ((rc = f32_vec(f, p, n + "ffn_up.bias", F, 1, &lw.ffn_up_b)) != FC_OK) return rc;
        if ((rc = f32_vec(f, p, n + "ffn_down.bias", d, 1, &lw.ffn_down_b)) != FC_OK) return rc;
        if ((rc = f32_vec(f, p, n + "attn_norm.weight", d, 1, &lw.ln1_g)) != FC_OK) return rc;
        if ((rc = f32_vec(f, p, n + "attn_norm.bias", d, 1, &lw.ln1_b)) != FC_OK) return rc;
        if ((rc = f32_vec(f, p, n + "ffn_norm.weight", d, 1, &lw.ln2_g)) != FC_OK) return rc;
        if ((rc = f32_vec(f, p, n + "ffn_norm.bias", d, 1, &lw.ln2_b)) != FC_OK) return rc;
    }
    if ((rc = f32_vec(f, p, "output_norm.weight", d, 1, &p->w.out_norm_g)) != FC_OK) return rc;
    if ((rc = f32_vec(f, p, "output_norm.bias", d, 1, &p->w.out_norm_b)) != FC_OK) return rc;
    p->w.layers = p->layers.data();
    p->cfg.n_layer = L; p->cfg.d_model = d; p->cfg.n_head = H; p->cfg.d_ff = F; p->cfg.ctx = ctx; p->cfg.vocab = V;
    p->cfg.tied = tied ? 1 : 0;
    p->cfg.math_mode = math_mode;
    return FC_OK;
}


// ---------------------------------------------------------------- llama / qwen2 files
// Gguf::load_llama_prec (gguf/llama.rs:171-339): metadata keys, defaults and refusals as there;
// the projections must be Q8_0 and stay packed, the norms F32.
struct ParsedLlama {
    fc_llama_config cfg{};
    std::vector<fc_llama_layer> layers;
    fc_llama_weights w{};
    std::vector<std::vector<float>> owned_f32;
    // the same matrices as the file stores them (for the model that keeps them in their block formats)
    fc::RawTensor raw_tok, raw_out;
    std::vector<fc::RawLlamaLayer> raw_layers;
};

// The stored form of a tensor that tensor() has already validated.
fc::RawTensor raw_of(const File& f, const std::string& name) {
    const Tensor& t = f.tensors.find(name)->second;
    fc::RawTensor r;
    r.type = (int)t.type;
    r.data = f.bytes.data() + f.data + t.offset;
    r.nbytes = (size_t)t.nbytes;
    return r;
}

bool has_tensor(const File& f, const std::string& name) { return f.tensors.find(name) != f.tensors.end(); }

int opt_int(const File& f, const std::string& key, int fallback, int* out) {
    if (f.meta.find(key) == f.meta.end()) { *out = fallback; return FC_OK; }
    return meta_int(f, key.c_str(), out);
}

double meta_f32_or(const File& f, const std::string& key, double fallback) {
    auto it = f.meta.find(key);
    if (it == f.meta.end()) return fallback;
    const Meta& m = it->second;
    if (m.type == VT_F32 || m.type == VT_F64) return m.f;
    if (m.type == VT_STRING || m.type == VT_BOOL) return fallback;
    return (double)(int64_t)m.u;
}

int f32_owned(const File& f, ParsedLlama* p, const std::string& name, uint64_t n, const float** out) {
    const uint8_t* b = nullptr;
    const int rc = tensor(f, name, T_F32, n, 1, &b);
    if (rc != FC_OK) return rc;
    p->owned_f32.emplace_back((size_t)n);
    memcpy(p->owned_f32.back().data(), b, (size_t)n * 4);
    *out = p->owned_f32.back().data();
    return FC_OK;
}

int parse_llama(const File& f, int math_mode, int ctx_cap, ParsedLlama* p) {
    auto at = f.meta.find("general.architecture");
    if (at == f.meta.end() || at->second.type != VT_STRING) return fail(FC_E_FORMAT, "GGUF missing general.architecture");
    const std::string arch = at->second.s;
    if (arch != "llama" && arch != "qwen2")
        return fail(FC_E_FORMAT, "architecture '%s' is not supported by load_llama (llama / qwen2 only)", arch.c_str());
    auto key = [&](const char* k) { return arch + "." + k; };
    int d = 0, L = 0, H = 0, KV = 0, F = 0, hd = 0, rope_dim = 0, ctx = 0;
    int rc;
    if ((rc = meta_int(f, key("embedding_length").c_str(), &d)) != FC_OK) return rc;
    if ((rc = meta_int(f, key("block_count").c_str(), &L)) != FC_OK) return rc;
    if ((rc = meta_int(f, key("attention.head_count").c_str(), &H)) != FC_OK) return rc;
    if ((rc = opt_int(f, key("attention.head_count_kv"), H, &KV)) != FC_OK) return rc;
    if ((rc = meta_int(f, key("feed_forward_length").c_str(), &F)) != FC_OK) return rc;
    if (d <= 0 || L <= 0 || H <= 0 || F <= 0) return fail(FC_E_FORMAT, "%s.* dimensions must be positive", arch.c_str());
    if ((size_t)L > f.tensors.size()) return fail(FC_E_FORMAT, "block_count %d exceeds the %zu tensors of the file", L, f.tensors.size());
    if ((rc = opt_int(f, key("attention.key_length"), d / H, &hd)) != FC_OK) return rc;
    if ((rc = opt_int(f, key("rope.dimension_count"), hd, &rope_dim)) != FC_OK) return rc;
    if ((rc = opt_int(f, key("context_length"), 2048, &ctx)) != FC_OK) return rc;
    const double rope_base = meta_f32_or(f, key("rope.freq_base"), 10000.0);
    const double eps = meta_f32_or(f, key("attention.layer_norm_rms_epsilon"), 1e-5);
    // rope_scaling (gguf/llama.rs:51-103): linear (also when no type is given) and
    // rope_freqs.weight; yarn, longrope and a non-1 attn_factor are refused
    double factor = 1.0;
    {
        auto it = f.meta.find(key("rope.scaling.factor"));
        if (it == f.meta.end()) it = f.meta.find(key("rope.scale_linear"));
        if (it != f.meta.end()) factor = meta_f32_or(f, it->first, 1.0);
        if (factor == 0.0) factor = 1.0;
        std::string ty = "linear";
        auto tt = f.meta.find(key("rope.scaling.type"));
        if (tt != f.meta.end()) {
            if (tt->second.type != VT_STRING) return fail(FC_E_FORMAT, "'%s' is not a string", key("rope.scaling.type").c_str());
            ty = tt->second.s;
        }
        if (ty == "none") {
            if (factor != 1.0) return fail(FC_E_FORMAT, "'%s' is \"none\" but the scaling factor is %g", key("rope.scaling.type").c_str(), factor);
        } else if (ty != "linear") {
            return fail(FC_E_FORMAT, "RoPE scaling type '%s' is not supported: none, linear and rope_freqs.weight are (yarn and longrope are refused)", ty.c_str());
        }
        const double attn = meta_f32_or(f, key("rope.scaling.attn_factor"), 1.0);
        if (attn != 1.0) return fail(FC_E_FORMAT, "RoPE scaling attn_factor %g is not supported (only 1.0)", attn);
    }
    if (has_tensor(f, "rope_freqs.weight")) {
        if (rope_dim < 2) return fail(FC_E_FORMAT, "rope_freqs.weight without a rotary dimension");
        if ((rc = f32_owned(f, p, "rope_freqs.weight", (uint64_t)rope_dim / 2, &p->w.rope_freqs)) != FC_OK) return rc;
    }
    auto te = f.tensors.find("token_embd.weight");
    if (te == f.tensors.end()) return fail(FC_E_FORMAT, "GGUF missing token_embd.weight");
    if (te->second.dims.size() != 2 || te->second.dims[0] != (uint64_t)d) return fail(FC_E_FORMAT, "token_embd.weight size does not match vocab x dim");
    const uint64_t V = te->second.dims[1];
    if (V == 0 || V > (1u << 30)) return fail(FC_E_FORMAT, "token_embd.weight size does not match vocab x dim");
    if (d % 32 || F % 32 || ((long long)H * hd) % 32)
        return fail(FC_E_FORMAT, "embedding_length, feed_forward_length and head_count x key_length must be multiples of 32 for Q8_0 rows");
    const uint64_t q_dim = (uint64_t)H * hd, kv_dim = (uint64_t)KV * hd;
    const uint8_t* b = nullptr;
    if ((rc = tensor(f, "token_embd.weight", T_Q8_0, d, V, &b)) != FC_OK) return rc;
    p->w.token_embd_q8 = b;
    p->raw_tok = raw_of(f, "token_embd.weight");
    p->layers.resize(L);
    p->raw_layers.resize(L);
    for (int i = 0; i < L; ++i) {
        fc_llama_layer& lw = p->layers[i];
        const std::string n = "blk." + std::to_string(i) + ".";
        // biases other than q / k / v are refused, not dropped (gguf/llama.rs:252-263)
        for (const char* stem : {"attn_output", "ffn_gate", "ffn_up", "ffn_down"})
            if (has_tensor(f, n + stem + ".bias"))
                return fail(FC_E_FORMAT, "GGUF tensor '%s%s.bias' is not supported: biases are loaded only for attn_q/attn_k/attn_v", n.c_str(), stem);
        if ((rc = f32_owned(f, p, n + "attn_norm.weight", d, &lw.attn_norm)) != FC_OK) return rc;
        if ((rc = tensor(f, n + "attn_q.weight", T_Q8_0, d, q_dim, &b)) != FC_OK) return rc;
        lw.wq_q8 = b;
        p->raw_layers[i].wq = raw_of(f, n + "attn_q.weight");
        if ((rc = tensor(f, n + "attn_k.weight", T_Q8_0, d, kv_dim, &b)) != FC_OK) return rc;
        lw.wk_q8 = b;
        p->raw_layers[i].wk = raw_of(f, n + "attn_k.weight");
        if ((rc = tensor(f, n + "attn_v.weight", T_Q8_0, d, kv_dim, &b)) != FC_OK) return rc;
        lw.wv_q8 = b;
        p->raw_layers[i].wv = raw_of(f, n + "attn_v.weight");
        if ((rc = tensor(f, n + "attn_output.weight", T_Q8_0, q_dim, d, &b)) != FC_OK) return rc;
        lw.wo_q8 = b;
        p->raw_layers[i].wo = raw_of(f, n + "attn_output.weight");
        if (has_tensor(f, n + "attn_q.bias") && (rc = f32_owned(f, p, n + "attn_q.bias", q_dim, &lw.bq)) != FC_OK) return rc;
        if (has_tensor(f, n + "attn_k.bias") && (rc = f32_owned(f, p, n + "attn_k.bias", kv_dim, &lw.bk)) != FC_OK) return rc;
        if (has_tensor(f, n + "attn_v.bias") && (rc = f32_owned(f, p, n + "attn_v.bias", kv_dim, &lw.bv)) != FC_OK) return rc;
        if ((rc = f32_owned(f, p, n + "ffn_norm.weight", d, &lw.ffn_norm)) != FC_OK) return rc;
        if ((rc = tensor(f, n + "ffn_gate.weight", T_Q8_0, d, F, &b)) != FC_OK) return rc;
        lw.gate_q8 = b;
        p->raw_layers[i].gate = raw_of(f, n + "ffn_gate.weight");
        if ((rc = tensor(f, n + "ffn_up.weight", T_Q8_0, d, F, &b)) != FC_OK) return rc;
        lw.up_q8 = b;
        p->raw_layers[i].up = raw_of(f, n + "ffn_up.weight");
        if ((rc = tensor(f, n + "ffn_down.weight", T_Q8_0, F, d, &b)) != FC_OK) return rc;
        lw.down_q8 = b;
        p->raw_layers[i].down = raw_of(f, n + "ffn_down.weight");
    }
    if ((rc = f32_owned(f, p, "output_norm.weight", d, &p->w.output_norm)) != FC_OK) return rc;
    if (has_tensor(f, "output.bias"))
        return fail(FC_E_FORMAT, "GGUF tensor 'output.bias' is not supported: biases are loaded only for attn_q/attn_k/attn_v");
    const bool tied = !has_tensor(f, "output.weight");
    if (!tied) {
        if ((rc = tensor(f, "output.weight", T_Q8_0, d, V, &b)) != FC_OK) return rc;
        p->w.output_q8 = b;
        p->raw_out = raw_of(f, "output.weight");
    }
    p->w.layers = p->layers.data();
    fc_llama_config& c = p->cfg;
    c.vocab = (int)V; c.d_model = d; c.n_layer = L; c.n_head = H; c.n_kv_head = KV; c.head_dim = hd; c.d_ff = F;
    c.rope_dim = rope_dim; c.rope_base = (float)rope_base;
    c.rope_type = arch == "qwen2" ? FC_ROPE_NEOX : FC_ROPE_NORM;   // gguf/llama.rs:181-186
    c.rope_linear_factor = (float)factor; c.norm_eps = (float)eps;
    c.ctx = ctx_cap > 0 && ctx_cap < ctx ? ctx_cap : ctx;
    c.tied = tied ? 1 : 0; c.math_mode = math_mode;
    return FC_OK;
}

}  // namespace

extern "C" {

int fc_gguf_probe(const char* path, const int32_t* row_perm, int n_perm, fc_config* out) {
    if (!path || !out || (row_perm && n_perm <= 0)) return fail(FC_E_ARG, "fc_gguf_probe: bad argument");
    File f;
    int rc = read_file(path, &f);
    if (rc != FC_OK) return rc;
    Parsed p;
    rc = parse_model(f, row_perm, n_perm, FC_MATH_FP32, &p);
    if (rc != FC_OK) return rc;
    *out = p.cfg;
    return FC_OK;
}

int fc_model_load_gguf(const char* path, const int32_t* row_perm, int n_perm, int device, int math_mode, fc_model** out) {
    if (!path || !out || (row_perm && n_perm <= 0)) return fail(FC_E_ARG, "fc_model_load_gguf: bad argument");
    *out = nullptr;
    File f;
    int rc = read_file(path, &f);
    if (rc != FC_OK) return rc;
    Parsed p;
    rc = parse_model(f, row_perm, n_perm, math_mode, &p);
    if (rc != FC_OK) return rc;
    return fc_model_create(&p.cfg, &p.w, device, out);   // copies everything it needs
}

int fc_llama_gguf_probe(const char* path, fc_llama_config* out) {
    if (!path || !out) return fail(FC_E_ARG, "fc_llama_gguf_probe: bad argument");
    File f;
    int rc = read_file(path, &f);
    if (rc != FC_OK) return rc;
    ParsedLlama p;
    rc = parse_llama(f, FC_MATH_FP32, 0, &p);
    if (rc != FC_OK) return rc;
    *out = p.cfg;
    return FC_OK;
}

static int load_llama_file(const char* path, int device, int math_mode, int ctx_cap, int kind, fc_llama** out) {
    if (!path || !out) return fail(FC_E_ARG, "fc_llama_load_gguf: bad argument");
    *out = nullptr;
    File f;
    int rc = read_file(path, &f);
    if (rc != FC_OK) return rc;
    ParsedLlama p;
    rc = parse_llama(f, math_mode, ctx_cap, &p);
    if (rc != FC_OK) return rc;
    // copies everything it needs
    return kind < 0 ? fc_llama_create(&p.cfg, &p.w, device, out) : fc_llama_create_packed(&p.cfg, &p.w, device, kind, out);
}

int fc_llama_load_gguf(const char* path, int device, int math_mode, int ctx_cap, fc_llama** out) {
    return load_llama_file(path, device, math_mode, ctx_cap, -1, out);
}

int fc_llama_load_gguf_native(const char* path, int device, int ctx_cap, fc_llama** out) {
    if (!path || !out) return fail(FC_E_ARG, "fc_llama_load_gguf_native: bad argument");
    *out = nullptr;
    File f;
    int rc = read_file(path, &f);
    if (rc != FC_OK) return rc;
    ParsedLlama p;
    rc = parse_llama(f, FC_MATH_FP32, ctx_cap, &p);
    if (rc != FC_OK) return rc;
    return fc::llama_create_native(&p.cfg, &p.w, p.raw_tok, p.raw_out, p.raw_layers.data(), device, out);
}

int fc_llama_load_gguf_packed(const char* path, int device, int ctx_cap, int kind, fc_llama** out) {
    if (kind != FC_Q_INT8 && kind != FC_Q_INT4) return fail(FC_E_ARG, "fc_llama_load_gguf_packed: kind %d", kind);
    return load_llama_file(path, device, FC_MATH_FP32, ctx_cap, kind, out);
}

}  // extern "C"
