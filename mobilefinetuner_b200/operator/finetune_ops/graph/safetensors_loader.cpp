#include "safetensors_loader.h"

#include <cstring>
#include <fstream>
#include <iostream>
#include <stdexcept>

#include "mft_cuda.h"
#include "mft_step.h"

namespace ops {

namespace {
[[noreturn]] void raise(const std::string& what) { throw std::runtime_error(what + ": " + mft_last_error()); }
bool has(const std::string& s, const char* needle) { return s.find(needle) != std::string::npos; }
}  // namespace

SafeTensorsReader::SafeTensorsReader(const std::string& filepath) : filepath_(filepath) {}
SafeTensorsReader::~SafeTensorsReader() { if (handle_) mft_safetensors_close(handle_); }

void SafeTensorsReader::parse_header() {
    if (handle_) return;
    if (mft_safetensors_open(filepath_.c_str(), &handle_) != MFT_OK) raise("SafeTensorsReader: cannot open " + filepath_);
}

void SafeTensorsReader::require_parsed() const {
    if (!handle_) throw std::logic_error("SafeTensorsReader: parse_header must be called first");
}

std::vector<std::string> SafeTensorsReader::get_tensor_names() const {
    require_parsed();
    std::vector<std::string> names;
    const int64_t n = mft_safetensors_count(handle_);
    for (int64_t i = 0; i < n; ++i) names.emplace_back(mft_safetensors_name(handle_, i));
    return names;
}

SafeTensorInfo SafeTensorsReader::get_tensor_info(const std::string& name) const {
    require_parsed();
    char dtype[8];
    int32_t nd = 0;
    int64_t shape[8];
    if (mft_safetensors_info(handle_, name.c_str(), dtype, &nd, shape) != MFT_OK) raise("SafeTensorsReader: " + name);
    SafeTensorInfo info;
    info.dtype = dtype;
    info.shape.assign(shape, shape + nd);
    return info;
}

TensorPtr SafeTensorsReader::read(const std::string& name, bool transpose, bool preserve_low_precision) {
    const SafeTensorInfo info = get_tensor_info(name);
    std::vector<int64_t> shape = info.shape;
    if (transpose && shape.size() == 2) std::swap(shape[0], shape[1]);
    auto f32 = std::make_shared<Tensor>(shape, kFloat32, kCPU);
    if (mft_safetensors_read_f32(handle_, name.c_str(), f32->data<float>(), (transpose && shape.size() == 2) ? 1 : 0) != MFT_OK)
        raise("SafeTensorsReader: " + name);
    if (preserve_low_precision && (info.dtype == "F16" || info.dtype == "BF16"))
        return cast(f32, info.dtype == "F16" ? DType::kFloat16 : DType::kBFloat16);     // exact: the values came from that format
    return f32;
}

TensorPtr SafeTensorsReader::load_tensor(const std::string& name, bool transpose) {
    require_parsed();
    return read(name, transpose, false);
}

std::unordered_map<std::string, TensorPtr>
SafeTensorsReader::load_tensors_mapped(const std::unordered_map<std::string, std::string>& key_mapping,
                                       const SafeTensorsLoadOptions& options) {
    require_parsed();
    std::unordered_map<std::string, bool> present;
    for (const auto& n : get_tensor_names()) present[n] = true;
    std::unordered_map<std::string, TensorPtr> out;
    for (const auto& kv : key_mapping) {
        const std::string& internal = kv.first;
        const std::string& hf = kv.second;
        if (!present.count(hf)) {
            if (options.verbose) std::cerr << "[WARN] HF key not found: " << hf << std::endl;
            continue;
        }
        const SafeTensorInfo info = get_tensor_info(hf);
        const bool embedding = has(hf, "wte") || has(hf, "wpe") || has(hf, "embed_tokens");
        const bool transpose = options.transpose_linear && has(hf, "weight") && !has(hf, "ln") && !embedding && info.shape.size() == 2;
        bool keep_low = !options.auto_promote_fp16;
        if (options.auto_promote_fp16)
            for (const auto& needle : options.preserve_low_precision_key_substrings)
                if (!needle.empty() && (has(internal, needle.c_str()) || has(hf, needle.c_str()))) { keep_low = true; break; }
        out[internal] = read(hf, transpose, keep_low);
        if (options.verbose) {
            std::cout << "[Loaded] " << internal << " <- " << hf << " shape=[";
            const auto& sh = out[internal]->shape();
            for (size_t i = 0; i < sh.size(); ++i) std::cout << sh[i] << (i + 1 < sh.size() ? ", " : "");
            std::cout << "]" << (transpose ? " (transposed)" : "") << std::endl;
        }
    }
    return out;
}

SafeTensorsModelReader::SafeTensorsModelReader(const std::string& model_dir_or_file)
    : SafeTensorsReader(model_dir_or_file), files_(resolve_weight_files(model_dir_or_file)) {}

std::vector<std::string> SafeTensorsModelReader::resolve_weight_files(const std::string& p) {
    auto exists = [](const std::string& f) { std::ifstream s(f, std::ios::binary); return (bool)s; };
    const std::string ext = ".safetensors";
    if (p.size() > ext.size() && p.compare(p.size() - ext.size(), ext.size(), ext) == 0) return {p};
    if (exists(p + "/model.safetensors")) return {p + "/model.safetensors"};
    if (!exists(p + "/model.safetensors.index.json")) throw std::runtime_error("no SafeTensors weights under " + p);
    // the shard names are the values of "weight_map" in the index
    std::ifstream f(p + "/model.safetensors.index.json");
    std::string text((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    std::vector<std::string> files;
    size_t pos = 0;
    while ((pos = text.find(ext + "\"", pos)) != std::string::npos) {
        const size_t q = text.rfind('"', pos);
        const std::string shard = p + "/" + text.substr(q + 1, pos + ext.size() - q - 1);
        bool seen = false;
        for (const auto& s : files) seen = seen || s == shard;
        if (!seen) files.push_back(shard);
        pos += ext.size();
    }
    return files;
}

std::unordered_map<std::string, std::string> GPT2KeyMapper::generate_gpt2_mapping(int num_layers) {
    std::unordered_map<std::string, std::string> m;
    for (const char* k : {"wte.weight", "wpe.weight", "ln_f.weight", "ln_f.bias"}) m[k] = k;
    static const char* pairs[][2] = {{"ln_1", "ln_1"}, {"attn.qkv", "attn.c_attn"}, {"attn.proj", "attn.c_proj"},
                                     {"ln_2", "ln_2"}, {"mlp.fc_in", "mlp.c_fc"}, {"mlp.fc_out", "mlp.c_proj"}};
    for (int l = 0; l < num_layers; ++l)
        for (const auto& pr : pairs)
            for (const char* leaf : {".weight", ".bias"})
                m["blocks." + std::to_string(l) + "." + pr[0] + leaf] = "h." + std::to_string(l) + "." + pr[1] + leaf;
    return m;
}

void GPT2KeyMapper::print_mapping(const std::unordered_map<std::string, std::string>& mapping) {
    std::cout << "\n[GPT2 Key Mapping] Total: " << mapping.size() << " entries\n";
    for (const auto& kv : mapping) std::cout << "  " << kv.first << " <- " << kv.second << std::endl;
}

std::unordered_map<std::string, std::string> GemmaKeyMapper::generate_gemma_mapping(int num_layers) {
    std::unordered_map<std::string, std::string> m;
    m["embed_tokens.weight"] = "model.embed_tokens.weight";
    m["norm.weight"] = "model.norm.weight";
    m["lm_head.weight"] = "lm_head.weight";
    static const char* leaves[] = {"input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm",
                                   "self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "self_attn.q_norm",
                                   "self_attn.k_norm", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"};
    for (int l = 0; l < num_layers; ++l)
        for (const char* leaf : leaves) {
            const std::string tail = "layers." + std::to_string(l) + "." + leaf + ".weight";
            m[tail] = "model." + tail;
        }
    return m;
}

void GemmaKeyMapper::print_mapping(const std::unordered_map<std::string, std::string>& mapping) {
    for (const auto& kv : mapping) std::cout << kv.first << " -> " << kv.second << std::endl;
}

std::unordered_map<std::string, std::string> QwenKeyMapper::generate_qwen_mapping(int num_layers) {
    std::unordered_map<std::string, std::string> m;
    m["embed_tokens.weight"] = "model.embed_tokens.weight";
    m["final_norm.weight"] = "model.norm.weight";
    for (int l = 0; l < num_layers; ++l) {
        const std::string in = "layers." + std::to_string(l) + ".", hf = "model." + in;
        m[in + "input_norm.weight"] = hf + "input_layernorm.weight";
        m[in + "post_norm.weight"] = hf + "post_attention_layernorm.weight";
        for (const char* proj : {"q_proj", "k_proj", "v_proj"})
            for (const char* leaf : {".weight", ".bias"}) m[in + "self_attn." + proj + leaf] = hf + "self_attn." + proj + leaf;
        m[in + "self_attn.o_proj.weight"] = hf + "self_attn.o_proj.weight";
        for (const char* proj : {"gate_proj", "up_proj", "down_proj"}) m[in + "mlp." + proj + ".weight"] = hf + "mlp." + proj + ".weight";
    }
    return m;
}

}  // namespace ops
