// SafeTensors readers and HuggingFace key maps with the reference's class surface
// (graph/safetensors_loader.h), implemented over the container code of libmft_cuda.so
// (mft_safetensors_*): header parsing, F32 / F16 / BF16 decoding and the optional
// transpose happen there; this file only shapes the results into ops::Tensor.
#pragma once

#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../core/tensor.h"

struct mft_safetensors;

namespace ops {

struct SafeTensorInfo {
    std::string dtype;                  // "F32", "F16", "BF16", "I64", ...
    std::vector<int64_t> shape;
    std::vector<size_t> data_offsets;   // not exposed by the container layer: left empty
};

struct SafeTensorsLoadOptions {
    bool transpose_linear = true;       // 2-D "weight" tensors other than embeddings / LayerNorm come back [in,out]
    bool auto_promote_fp16 = true;      // F16 / BF16 -> F32
    bool verbose = true;
    bool strict_shape_check = true;
    // keys (internal or HF) containing one of these keep F16 / BF16 storage even when auto_promote_fp16 is set
    std::vector<std::string> preserve_low_precision_key_substrings;
};

class SafeTensorsReader {
public:
    explicit SafeTensorsReader(const std::string& filepath);
    ~SafeTensorsReader();
    SafeTensorsReader(const SafeTensorsReader&) = delete;
    SafeTensorsReader& operator=(const SafeTensorsReader&) = delete;

    void parse_header();
    std::vector<std::string> get_tensor_names() const;
    SafeTensorInfo get_tensor_info(const std::string& name) const;
    TensorPtr load_tensor(const std::string& name, bool transpose = false);
    std::unordered_map<std::string, TensorPtr>
    load_tensors_mapped(const std::unordered_map<std::string, std::string>& key_mapping,
                        const SafeTensorsLoadOptions& options = SafeTensorsLoadOptions());

protected:
    std::string filepath_;
    mft_safetensors* handle_ = nullptr;
    TensorPtr read(const std::string& name, bool transpose, bool preserve_low_precision);
    void require_parsed() const;
};

// One model.safetensors file, a directory holding it, or a sharded snapshot with model.safetensors.index.json.
class SafeTensorsModelReader : private SafeTensorsReader {
public:
    explicit SafeTensorsModelReader(const std::string& model_dir_or_file);
    void parse_headers() { parse_header(); }
    using SafeTensorsReader::get_tensor_names;
    using SafeTensorsReader::load_tensors_mapped;
    const std::vector<std::string>& files() const { return files_; }
    static std::vector<std::string> resolve_weight_files(const std::string& model_dir_or_file);

private:
    std::vector<std::string> files_;
};

// {"internal_key": "hf_key"} tables of the three model families
class GPT2KeyMapper {
public:
    static std::unordered_map<std::string, std::string> generate_gpt2_mapping(int num_layers = 12);
    static void print_mapping(const std::unordered_map<std::string, std::string>& mapping);
};
class GemmaKeyMapper {
public:
    static std::unordered_map<std::string, std::string> generate_gemma_mapping(int num_layers = 18);
    static void print_mapping(const std::unordered_map<std::string, std::string>& mapping);
};
class QwenKeyMapper {
public:
    static std::unordered_map<std::string, std::string> generate_qwen_mapping(int num_layers = 24);
};

}  // namespace ops
