// SafeTensors ingest and adapter save / load for the step engine (host code).
//
// Container: 8-byte little-endian header length, a JSON header {"name": {"dtype", "shape", "data_offsets"}, ...,
// "__metadata__": {...}}, then the raw tensor bytes.  A model is one file, or a directory holding
// model.safetensors, or a HuggingFace sharded snapshot with model.safetensors.index.json
// (SafeTensorsReader / SafeTensorsModelReader, graph/safetensors_loader.h:35-124).
// Model load: the HuggingFace key of every frozen parameter (GPT2KeyMapper / GemmaKeyMapper / QwenKeyMapper,
// graph/safetensors_loader.cpp:470-590) is read as f32 (F32, F16 and BF16 sources), HF Linear weights [out,in] are
// transposed to the engine's [in,out] (GPT-2's Conv1D weights already are), and installed through the engine's
// staging path.  Adapter files: keys layer.{i}.{target}.lora_A / lora_B, F32, sorted, with rank / alpha /
// dropout / targets in __metadata__ (LoraSaver::make_peft_key graph/lora_saver.cpp:123-126,
// GemmaLoraInjector::save_lora_safetensors graph/gemma_lora_injector.cpp:179-264).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "common.cuh"
#include "engine.h"

using namespace mft;

namespace {

struct TensorEntry {
    std::string dtype;
    std::vector<int64_t> shape;
    uint64_t begin = 0, end = 0;      // relative to the data section
    int file = 0;
};

struct StFile {
    std::string path;
    uint64_t data_offset = 0;
};

// ---- a JSON reader for the subset the container uses: objects, arrays, strings, integers
struct Json {
    const std::string& s;
    size_t i = 0;
    explicit Json(const std::string& str) : s(str) {}
    void ws() { while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i; }
    bool eat(char c) { ws(); if (i < s.size() && s[i] == c) { ++i; return true; } return false; }
    bool peek(char c) { ws(); return i < s.size() && s[i] == c; }
    bool string(std::string* out) {
        ws();
        if (i >= s.size() || s[i] != '"') return false;
        ++i;
        out->clear();
        while (i < s.size() && s[i] != '"') {
            if (s[i] == '\\' && i + 1 < s.size()) {
                const char e = s[i + 1];
                if (e == 'u' && i + 5 < s.size()) { out->push_back('?'); i += 6; continue; }
                out->push_back(e == 'n' ? '\n' : e == 't' ? '\t' : e);
                i += 2;
            } else {
                out->push_back(s[i++]);
            }
        }
        if (i >= s.size()) return false;
        ++i;
        return true;
    }
    bool integer(int64_t* out) {
        ws();
        size_t j = i;
        if (j < s.size() && (s[j] == '-' || s[j] == '+')) ++j;
        const size_t d0 = j;
        while (j < s.size() && s[j] >= '0' && s[j] <= '9') ++j;
        if (j == d0) return false;
        *out = std::strtoll(s.c_str() + i, nullptr, 10);
        i = j;
        return true;
    }
    // skips any value (used for fields this reader does not need)
    bool skip() {
        ws();
        if (i >= s.size()) return false;
        if (s[i] == '"') { std::string t; return string(&t); }
        if (s[i] == '{' || s[i] == '[') {
            const char open = s[i], close = open == '{' ? '}' : ']';
            ++i;
            if (eat(close)) return true;
            while (true) {
                if (open == '{') { std::string k; if (!string(&k) || !eat(':')) return false; }
                if (!skip()) return false;
                if (eat(',')) continue;
                return eat(close);
            }
        }
        while (i < s.size() && s[i] != ',' && s[i] != '}' && s[i] != ']') ++i;
        return true;
    }
};

}  // namespace

struct mft_safetensors {
    std::vector<StFile> files;
    std::map<std::string, TensorEntry> tensors;
    std::vector<std::string> names;
    std::map<std::string, std::string> metadata;
};

namespace {

int32_t parse_one_file(mft_safetensors* h, const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) return fail(MFT_ERR_INVALID_ARG, "safetensors: cannot open " + path);
    uint8_t lenb[8];
    f.read(reinterpret_cast<char*>(lenb), 8);
    if (!f) return fail(MFT_ERR_INVALID_ARG, "safetensors: " + path + " is shorter than its header length field");
    uint64_t hlen = 0;
    for (int b = 7; b >= 0; --b) hlen = (hlen << 8) | lenb[b];
    f.seekg(0, std::ios::end);
    const uint64_t fsize = (uint64_t)f.tellg();
    if (hlen == 0 || hlen > fsize - 8 || hlen > (1ull << 31)) return fail(MFT_ERR_INVALID_ARG, "safetensors: bad header length in " + path);
    std::string header(hlen, '\0');
    f.seekg(8);
    f.read(&header[0], (std::streamsize)hlen);
    if (!f) return fail(MFT_ERR_INVALID_ARG, "safetensors: truncated header in " + path);
    const int file_index = (int)h->files.size();
    h->files.push_back(StFile{path, 8 + hlen});
    const uint64_t data_bytes = fsize - 8 - hlen;
    Json j(header);
    if (!j.eat('{')) return fail(MFT_ERR_INVALID_ARG, "safetensors: header of " + path + " is not a JSON object");
    if (j.eat('}')) return MFT_OK;
    while (true) {
        std::string name;
        if (!j.string(&name) || !j.eat(':')) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed header in " + path);
        if (name == "__metadata__") {
            if (!j.eat('{')) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed __metadata__ in " + path);
            if (!j.eat('}')) {
                while (true) {
                    std::string k, v;
                    if (!j.string(&k) || !j.eat(':')) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed __metadata__ in " + path);
                    if (j.peek('"')) { if (!j.string(&v)) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed __metadata__ in " + path); }
                    else if (!j.skip()) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed __metadata__ in " + path);
                    h->metadata[k] = v;
                    if (j.eat(',')) continue;
                    if (j.eat('}')) break;
                    return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed __metadata__ in " + path);
                }
            }
        } else {
            TensorEntry e;
            e.file = file_index;
            if (!j.eat('{')) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed entry " + name);
            while (true) {
                std::string k;
                if (!j.string(&k) || !j.eat(':')) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed entry " + name);
                if (k == "dtype") {
                    if (!j.string(&e.dtype)) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed dtype of " + name);
                } else if (k == "shape" || k == "data_offsets") {
                    std::vector<int64_t> v;
                    if (!j.eat('[')) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed " + k + " of " + name);
                    if (!j.eat(']')) {
                        while (true) {
                            int64_t x;
                            if (!j.integer(&x)) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed " + k + " of " + name);
                            v.push_back(x);
                            if (j.eat(',')) continue;
                            if (j.eat(']')) break;
                            return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed " + k + " of " + name);
                        }
                    }
                    if (k == "shape") e.shape = v;
                    else {
                        if (v.size() != 2 || v[0] < 0 || v[1] < v[0]) return fail(MFT_ERR_INVALID_ARG, "safetensors: bad data_offsets of " + name);
                        e.begin = (uint64_t)v[0]; e.end = (uint64_t)v[1];
                    }
                } else if (!j.skip()) {
                    return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed entry " + name);
                }
                if (j.eat(',')) continue;
                if (j.eat('}')) break;
                return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed entry " + name);
            }
            if (e.end > data_bytes) return fail(MFT_ERR_INVALID_ARG, "safetensors: " + name + " points past the end of " + path);
            if (h->tensors.emplace(name, e).second) h->names.push_back(name);
        }
        if (j.eat(',')) continue;
        if (j.eat('}')) break;
        return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed header in " + path);
    }
    return MFT_OK;
}

bool file_exists(const std::string& p) { std::ifstream f(p, std::ios::binary); return (bool)f; }

int dtype_size(const std::string& d) {
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    if (d == "I8" || d == "U8" || d == "BOOL") return 1;
    return 0;
}

float half_to_float(uint16_t hv) {
    const uint32_t sign = (uint32_t)(hv & 0x8000u) << 16;
    uint32_t exp = (hv >> 10) & 0x1Fu, man = hv & 0x3FFu, out;
    if (exp == 0) {
        if (man == 0) out = sign;
        else {
            int e = -1;
            do { ++e; man <<= 1; } while ((man & 0x400u) == 0);
            out = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) out = sign | 0x7F800000u | (man << 13);
    else out = sign | ((exp + 112) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &out, 4);
    return f;
}

int32_t read_f32(const mft_safetensors* h, const std::string& name, float* out, bool transpose2d, int64_t expect_elems) {
    auto it = h->tensors.find(name);
    if (it == h->tensors.end()) return fail(MFT_ERR_INVALID_ARG, "safetensors: no tensor named " + name);
    const TensorEntry& e = it->second;
    int64_t n = 1;
    for (int64_t d : e.shape) {      // a header is untrusted input: no negative extents, no product that wraps
        if (d < 0 || (d > 0 && n > (int64_t)(1ull << 40) / d)) return fail(MFT_ERR_INVALID_ARG, "safetensors: implausible shape of " + name);
        n *= d;
    }
    const int es = dtype_size(e.dtype);
    if (!(e.dtype == "F32" || e.dtype == "F16" || e.dtype == "BF16")) return fail(MFT_ERR_UNSUPPORTED, "safetensors: " + name + " has dtype " + e.dtype + " (F32, F16 or BF16 expected)");
    if ((uint64_t)n * es != e.end - e.begin) return fail(MFT_ERR_INVALID_ARG, "safetensors: byte size of " + name + " does not match its shape");
    if (expect_elems >= 0 && n != expect_elems) return fail(MFT_ERR_INVALID_ARG, "safetensors: " + name + " has " + std::to_string(n) + " elements, " + std::to_string(expect_elems) + " expected");
    if (transpose2d && e.shape.size() != 2) return fail(MFT_ERR_INVALID_ARG, "safetensors: " + name + " is not 2-D, cannot transpose");
    std::ifstream f(h->files[(size_t)e.file].path, std::ios::binary);
    if (!f) return fail(MFT_ERR_INVALID_ARG, "safetensors: cannot reopen " + h->files[(size_t)e.file].path);
    f.seekg((std::streamoff)(h->files[(size_t)e.file].data_offset + e.begin));
    std::vector<uint8_t> raw((size_t)n * es);
    f.read(reinterpret_cast<char*>(raw.data()), (std::streamsize)raw.size());
    if (!f) return fail(MFT_ERR_INVALID_ARG, "safetensors: short read of " + name);
    auto value = [&](int64_t idx) -> float {
        if (es == 4) { float v; std::memcpy(&v, raw.data() + idx * 4, 4); return v; }
        uint16_t hv;
        std::memcpy(&hv, raw.data() + idx * 2, 2);
        if (e.dtype == "BF16") { const uint32_t u = (uint32_t)hv << 16; float v; std::memcpy(&v, &u, 4); return v; }
        return half_to_float(hv);
    };
    if (!transpose2d) {
        for (int64_t i = 0; i < n; ++i) out[i] = value(i);
    } else {
        const int64_t R = e.shape[0], Cc = e.shape[1];
        for (int64_t r = 0; r < R; ++r)
            for (int64_t c = 0; c < Cc; ++c) out[c * R + r] = value(r * Cc + c);
    }
    return MFT_OK;
}

// The stored bytes of a tensor, unconverted.
int32_t read_raw(const mft_safetensors* h, const std::string& name, std::vector<uint8_t>& raw, int64_t expect_elems) {
    auto it = h->tensors.find(name);
    if (it == h->tensors.end()) return fail(MFT_ERR_INVALID_ARG, "safetensors: no tensor named " + name);
    const TensorEntry& e = it->second;
    int64_t n = 1;
    for (int64_t d : e.shape) {
        if (d < 0 || (d > 0 && n > (int64_t)(1ull << 40) / d)) return fail(MFT_ERR_INVALID_ARG, "safetensors: implausible shape of " + name);
        n *= d;
    }
    const int es = dtype_size(e.dtype);
    if (es <= 0 || (uint64_t)n * es != e.end - e.begin) return fail(MFT_ERR_INVALID_ARG, "safetensors: byte size of " + name + " does not match its shape");
    if (expect_elems >= 0 && n != expect_elems) return fail(MFT_ERR_INVALID_ARG, "safetensors: " + name + " has " + std::to_string(n) + " elements, " + std::to_string(expect_elems) + " expected");
    std::ifstream f(h->files[(size_t)e.file].path, std::ios::binary);
    if (!f) return fail(MFT_ERR_INVALID_ARG, "safetensors: cannot reopen " + h->files[(size_t)e.file].path);
    f.seekg((std::streamoff)(h->files[(size_t)e.file].data_offset + e.begin));
    raw.resize((size_t)n * es);
    f.read(reinterpret_cast<char*>(raw.data()), (std::streamsize)raw.size());
    if (!f) return fail(MFT_ERR_INVALID_ARG, "safetensors: short read of " + name);
    return MFT_OK;
}

// HuggingFace key and orientation of frozen parameter `idx` (engine names are set in mft_model_create)
struct HfKey { std::string key; bool transpose; bool skip; };

HfKey hf_key_of(const mft_model* m, const ParamInfo& p) {
    const int fam = m->cfg.family;
    const std::string& n = p.name;
    auto layer_split = [&](std::string* rest) -> int {
        if (n.compare(0, 5, "layer") != 0) return -1;
        const size_t dot = n.find('.');
        *rest = n.substr(dot + 1);
        return std::atoi(n.substr(5, dot - 5).c_str());
    };
    std::string rest;
    const int l = layer_split(&rest);
    if (fam == MFT_FAMILY_GPT2) {
        if (n == "wte") return {"wte.weight", false, false};
        if (n == "wpe") return {"wpe.weight", false, false};
        if (n == "ln_f.weight" || n == "ln_f.bias") return {n, false, false};
        if (l >= 0) return {"h." + std::to_string(l) + "." + rest, false, false};        // Conv1D weights are [in,out] already
        return {"", false, true};
    }
    if (p.kind == ParamInfo::LM_HEAD_COPY) return {"", false, true};                      // tied: follows embed_tokens
    if (n == "embed_tokens") return {"model.embed_tokens.weight", false, false};
    if (n == "final_norm" || n == "norm") return {"model.norm.weight", false, false};
    if (l >= 0) {
        const std::string pre = "model.layers." + std::to_string(l) + ".";
        if (p.kind == ParamInfo::NORM) {
            if (rest == "q_norm" || rest == "k_norm") return {pre + "self_attn." + rest + ".weight", false, false};
            return {pre + rest + ".weight", false, false};
        }
        const bool attn = rest.compare(0, 2, "q_") == 0 || rest.compare(0, 2, "k_") == 0 || rest.compare(0, 2, "v_") == 0 || rest.compare(0, 2, "o_") == 0;
        return {pre + (attn ? "self_attn." : "mlp.") + rest, p.kind == ParamInfo::LINEAR, false};
    }
    return {"", false, true};
}

// adapter target names in get_lora_parameters() order, per family
std::vector<std::string> lora_targets_of(const mft_model* m) {
    const uint32_t tg = m->cfg.lora_targets;
    std::vector<std::string> t;
    if (m->cfg.family == MFT_FAMILY_GPT2) {
        if (tg & MFT_LORA_Q) t.push_back("attn.qkv");
        if (tg & MFT_LORA_O) t.push_back("attn.proj");
        if (tg & MFT_LORA_GATE) t.push_back("mlp.fc_in");
        if (tg & MFT_LORA_DOWN) t.push_back("mlp.fc_out");
    } else if (m->cfg.family == MFT_FAMILY_QWEN) {
        if (tg & MFT_LORA_Q) t.push_back("attn.q");
        if (tg & MFT_LORA_V) t.push_back("attn.v");
        if (tg & MFT_LORA_K) t.push_back("attn.k");
        if (tg & MFT_LORA_O) t.push_back("attn.proj");
    } else {
        if (tg & MFT_LORA_Q) t.push_back("attn.q");
        if (tg & MFT_LORA_K) t.push_back("attn.k");
        if (tg & MFT_LORA_V) t.push_back("attn.v");
        if (tg & MFT_LORA_O) t.push_back("attn.proj");
        if (tg & MFT_LORA_GATE) t.push_back("mlp.gate");
        if (tg & MFT_LORA_UP) t.push_back("mlp.up");
        if (tg & MFT_LORA_DOWN) t.push_back("mlp.down");
    }
    return t;
}

std::string fmt_float(float v) {
    std::ostringstream o;
    o << v;
    return o.str();
}

}  // namespace

extern "C" int32_t mft_safetensors_open(const char* path_or_dir, mft_safetensors_t** out) {
    MFT_CHECK_ARG(path_or_dir && out, "mft_safetensors_open: null argument");
    auto h = std::make_unique<mft_safetensors>();
    const std::string p(path_or_dir);
    std::vector<std::string> files;
    if (p.size() > 12 && p.compare(p.size() - 12, 12, ".safetensors") == 0) {
        files.push_back(p);
    } else if (file_exists(p + "/model.safetensors")) {
        files.push_back(p + "/model.safetensors");
    } else if (file_exists(p + "/model.safetensors.index.json")) {
        // sharded snapshot: {"weight_map": {"tensor": "model-0000x-of-0000y.safetensors", ...}}
        std::ifstream f(p + "/model.safetensors.index.json", std::ios::binary);
        std::stringstream ss;
        ss << f.rdbuf();
        const std::string text = ss.str();
        Json j(text);
        if (!j.eat('{')) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed index in " + p);
        while (!j.peek('}')) {
            std::string k;
            if (!j.string(&k) || !j.eat(':')) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed index in " + p);
            if (k == "weight_map") {
                if (!j.eat('{')) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed weight_map in " + p);
                while (!j.peek('}')) {
                    std::string t, shard;
                    if (!j.string(&t) || !j.eat(':') || !j.string(&shard)) return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed weight_map in " + p);
                    if (std::find(files.begin(), files.end(), p + "/" + shard) == files.end()) files.push_back(p + "/" + shard);
                    j.eat(',');
                }
                j.eat('}');
            } else if (!j.skip()) {
                return fail(MFT_ERR_INVALID_ARG, "safetensors: malformed index in " + p);
            }
            j.eat(',');
        }
        std::sort(files.begin(), files.end());
    } else {
        return fail(MFT_ERR_INVALID_ARG, "safetensors: " + p + " is neither a .safetensors file nor a directory with model.safetensors(.index.json)");
    }
    for (const auto& f : files)
        if (int32_t s = parse_one_file(h.get(), f)) return s;
    *out = h.release();
    return MFT_OK;
}

extern "C" int32_t mft_safetensors_close(mft_safetensors_t* h) { delete h; return MFT_OK; }
extern "C" int64_t mft_safetensors_count(const mft_safetensors_t* h) { return h ? (int64_t)h->names.size() : 0; }
extern "C" const char* mft_safetensors_name(const mft_safetensors_t* h, int64_t i) {
    return (h && i >= 0 && i < (int64_t)h->names.size()) ? h->names[(size_t)i].c_str() : nullptr;
}
extern "C" const char* mft_safetensors_metadata(const mft_safetensors_t* h, const char* key) {
    if (!h || !key) return nullptr;
    auto it = h->metadata.find(key);
    return it == h->metadata.end() ? nullptr : it->second.c_str();
}
extern "C" int32_t mft_safetensors_info(const mft_safetensors_t* h, const char* name, char* dtype8, int32_t* ndim, int64_t* shape8) {
    MFT_CHECK_ARG(h && name && dtype8 && ndim && shape8, "mft_safetensors_info: null argument");
    auto it = h->tensors.find(name);
    if (it == h->tensors.end()) return fail(MFT_ERR_INVALID_ARG, std::string("safetensors: no tensor named ") + name);
    MFT_CHECK_ARG(it->second.shape.size() <= 8, "mft_safetensors_info: more than 8 dimensions");
    std::snprintf(dtype8, 8, "%s", it->second.dtype.c_str());
    *ndim = (int32_t)it->second.shape.size();
    for (size_t d = 0; d < it->second.shape.size(); ++d) shape8[d] = it->second.shape[d];
    return MFT_OK;
}
extern "C" int32_t mft_safetensors_read_f32(const mft_safetensors_t* h, const char* name, float* out_host, int32_t transpose2d) {
    MFT_CHECK_ARG(h && name && out_host, "mft_safetensors_read_f32: null argument");
    return read_f32(h, name, out_host, transpose2d != 0, -1);
}

extern "C" int32_t mft_safetensors_write_f32(const char* path, int32_t n, const char* const* names, const int32_t* ndims,
                                             const int64_t* shapes8, const float* const* data, int32_t n_meta,
                                             const char* const* meta_keys, const char* const* meta_values) {
    MFT_CHECK_ARG(path && n >= 0 && (n == 0 || (names && ndims && shapes8 && data)), "mft_safetensors_write_f32: bad argument");
    std::vector<int> order((size_t)n);
    for (int i = 0; i < n; ++i) order[(size_t)i] = i;
    std::sort(order.begin(), order.end(), [&](int a, int b) { return std::strcmp(names[a], names[b]) < 0; });
    std::ostringstream header;
    header << "{";
    uint64_t offset = 0;
    std::vector<uint64_t> bytes((size_t)n);
    for (int k = 0; k < n; ++k) {
        const int i = order[(size_t)k];
        uint64_t elems = 1;
        for (int d = 0; d < ndims[i]; ++d) elems *= (uint64_t)shapes8[i * 8 + d];
        bytes[(size_t)i] = elems * 4;
        if (k > 0) header << ",";
        header << "\"" << names[i] << "\":{\"dtype\":\"F32\",\"shape\":[";
        for (int d = 0; d < ndims[i]; ++d) header << (d ? "," : "") << shapes8[i * 8 + d];
        header << "],\"data_offsets\":[" << offset << "," << offset + bytes[(size_t)i] << "]}";
        offset += bytes[(size_t)i];
    }
    if (n_meta > 0) {
        header << (n > 0 ? "," : "") << "\"__metadata__\":{";
        for (int k = 0; k < n_meta; ++k) header << (k ? "," : "") << "\"" << meta_keys[k] << "\":\"" << meta_values[k] << "\"";
        header << "}";
    }
    header << "}";
    std::string hs = header.str();
    while (hs.size() % 8 != 0) hs.push_back(' ');               // the data section starts 8-byte aligned
    std::ofstream f(path, std::ios::binary | std::ios::trunc);
    if (!f) return fail(MFT_ERR_INVALID_ARG, std::string("safetensors: cannot open ") + path + " for writing");
    const uint64_t hlen = hs.size();
    uint8_t lenb[8];
    for (int b = 0; b < 8; ++b) lenb[b] = (uint8_t)(hlen >> (8 * b));
    f.write(reinterpret_cast<const char*>(lenb), 8);
    f.write(hs.data(), (std::streamsize)hs.size());
    for (int k = 0; k < n; ++k) {
        const int i = order[(size_t)k];
        f.write(reinterpret_cast<const char*>(data[i]), (std::streamsize)bytes[(size_t)i]);
    }
    if (!f) return fail(MFT_ERR_INVALID_ARG, std::string("safetensors: write to ") + path + " failed");
    return MFT_OK;
}

// ---------------------------------------------------------------- model level
extern "C" int32_t mft_model_hf_key(const mft_model_t* m, int32_t idx, char* key_out, int32_t key_cap, int32_t* transpose) {
    MFT_CHECK_ARG(m && idx >= 0 && idx < (int)m->params.size() && key_out && key_cap > 0, "mft_model_hf_key: bad argument");
    const HfKey k = hf_key_of(m, m->params[(size_t)idx]);
    std::snprintf(key_out, (size_t)key_cap, "%s", k.skip ? "" : k.key.c_str());
    if (transpose) *transpose = k.transpose ? 1 : 0;
    return MFT_OK;
}

extern "C" int32_t mft_model_load_safetensors(mft_model_t* m, const char* path_or_dir) {
    MFT_CHECK_ARG(m && path_or_dir, "mft_model_load_safetensors: null argument");
    mft_safetensors_t* h = nullptr;
    if (int32_t s = mft_safetensors_open(path_or_dir, &h)) return s;
    std::unique_ptr<mft_safetensors> guard(h);
    std::vector<float> host;
    std::vector<uint8_t> raw;
    for (size_t i = 0; i < m->params.size(); ++i) {
        const ParamInfo& p = m->params[i];
        HfKey k = hf_key_of(m, p);
        if (k.skip) continue;
        // GPT-2 checkpoints come with or without the "transformer." prefix
        if (m->cfg.family == MFT_FAMILY_GPT2 && !h->tensors.count(k.key) && h->tensors.count("transformer." + k.key)) k.key = "transformer." + k.key;
        if (!h->tensors.count(k.key)) return fail(MFT_ERR_INVALID_ARG, "safetensors: checkpoint has no tensor " + k.key + " (parameter " + p.name + ")");
        const TensorEntry& entry = h->tensors[k.key];
        if (k.transpose) {                                  // HF Linear weight [out, in]
            if (entry.shape.size() != 2 || entry.shape[0] != p.cols || entry.shape[1] != p.rows)
                return fail(MFT_ERR_INVALID_ARG, "safetensors: shape of " + k.key + " does not fit parameter " + p.name);
        }
        if (entry.dtype == "BF16") {
            // the stored bits are what the device keeps: no f32 detour on the host
            if (int32_t s = read_raw(h, k.key, raw, p.rows * p.cols)) return s;
            const int32_t st = mft_model_set_param_host_bf16(m, (int32_t)i, raw.data(), k.transpose ? 1 : 0);
            if (st == MFT_OK) continue;
            if (st != MFT_ERR_UNSUPPORTED) return st;       // larger than the staging area: the f32 path below chunks it
        }
        host.resize((size_t)(p.rows * p.cols));
        if (int32_t s = read_f32(h, k.key, host.data(), k.transpose, p.rows * p.cols)) return s;
        if (int32_t s = mft_model_set_param_host(m, (int32_t)i, host.data())) return s;
    }
    return MFT_OK;
}

extern "C" int32_t mft_model_save_lora_safetensors(mft_model_t* m, const char* path) {
    MFT_CHECK_ARG(m && path, "mft_model_save_lora_safetensors: null argument");
    const std::vector<std::string> targets = lora_targets_of(m);
    const size_t per_layer = targets.size() * 2;
    MFT_CHECK_ARG(per_layer > 0 && m->loras.size() == per_layer * (size_t)m->cfg.layers, "mft_model_save_lora_safetensors: model has no LoRA tensors");
    std::vector<std::string> names;
    std::vector<std::vector<float>> bufs(m->loras.size());
    std::vector<int32_t> ndims(m->loras.size(), 2);
    std::vector<int64_t> shapes(m->loras.size() * 8, 0);
    for (size_t i = 0; i < m->loras.size(); ++i) {
        const size_t layer = i / per_layer, t = (i % per_layer) / 2;
        names.push_back("layer." + std::to_string(layer) + "." + targets[t] + ((i & 1) ? ".lora_B" : ".lora_A"));
        bufs[i].resize((size_t)(m->loras[i].rows * m->loras[i].cols));
        shapes[i * 8] = m->loras[i].rows; shapes[i * 8 + 1] = m->loras[i].cols;
        if (int32_t s = mft_model_get_lora_host(m, (int32_t)i, bufs[i].data())) return s;
    }
    std::vector<const char*> name_ptrs, meta_k, meta_v;
    std::vector<const float*> data_ptrs;
    for (size_t i = 0; i < names.size(); ++i) { name_ptrs.push_back(names[i].c_str()); data_ptrs.push_back(bufs[i].data()); }
    // the metadata lists the targets sorted for Gemma adapters (GemmaLoraInjector::save_lora_safetensors,
    // graph/gemma_lora_injector.cpp:218) and in injection order otherwise (LoraSaver::join_targets, graph/lora_saver.cpp:74-82)
    std::vector<std::string> listed = targets;
    if (m->cfg.family == MFT_FAMILY_GEMMA) std::sort(listed.begin(), listed.end());
    std::string joined;
    for (size_t t = 0; t < listed.size(); ++t) joined += (t ? "," : "") + listed[t];
    // the step engine applies no LoRA dropout, so "0" is what was trained with (the operator API's injectors write their
    // configured value through their own writer)
    const std::string rank = std::to_string(m->cfg.lora_rank), alpha = fmt_float(m->cfg.lora_alpha), dropout = "0";
    const char* keys[4] = {"rank", "alpha", "dropout", "targets"};
    const char* vals[4] = {rank.c_str(), alpha.c_str(), dropout.c_str(), joined.c_str()};
    return mft_safetensors_write_f32(path, (int32_t)names.size(), name_ptrs.data(), ndims.data(), shapes.data(), data_ptrs.data(), 4, keys, vals);
}

extern "C" int32_t mft_model_load_lora_safetensors(mft_model_t* m, const char* path) {
    MFT_CHECK_ARG(m && path, "mft_model_load_lora_safetensors: null argument");
    mft_safetensors_t* h = nullptr;
    if (int32_t s = mft_safetensors_open(path, &h)) return s;
    std::unique_ptr<mft_safetensors> guard(h);
    const std::vector<std::string> targets = lora_targets_of(m);
    const size_t per_layer = targets.size() * 2;
    MFT_CHECK_ARG(per_layer > 0 && m->loras.size() == per_layer * (size_t)m->cfg.layers, "mft_model_load_lora_safetensors: model has no LoRA tensors");
    if (const char* r = mft_safetensors_metadata(h, "rank"))
        if (std::atoi(r) != m->cfg.lora_rank) return fail(MFT_ERR_INVALID_ARG, std::string("adapter rank ") + r + " does not match the model's " + std::to_string(m->cfg.lora_rank));
    std::vector<float> host;
    for (size_t i = 0; i < m->loras.size(); ++i) {
        const size_t layer = i / per_layer, t = (i % per_layer) / 2;
        const std::string name = "layer." + std::to_string(layer) + "." + targets[t] + ((i & 1) ? ".lora_B" : ".lora_A");
        auto it = h->tensors.find(name);
        if (it == h->tensors.end()) return fail(MFT_ERR_INVALID_ARG, "adapter file has no tensor " + name);
        if (it->second.shape.size() != 2 || it->second.shape[0] != m->loras[i].rows || it->second.shape[1] != m->loras[i].cols)
            return fail(MFT_ERR_INVALID_ARG, "adapter tensor " + name + " has the wrong shape");
        host.resize((size_t)(m->loras[i].rows * m->loras[i].cols));
        if (int32_t s = read_f32(h, name, host.data(), false, (int64_t)host.size())) return s;
        if (int32_t s = mft_model_set_lora_host(m, (int32_t)i, host.data())) return s;
    }
    return MFT_OK;
}
