// Adapter files: named f32 tensors plus string metadata in one .safetensors container (keys sorted, F32), written
// and read through the container code of libmft_cuda.so.  Shared by LoraSaver, LoraInjector and GemmaLoraInjector.
#pragma once
#include <map>
#include <string>

#include "../core/tensor.h"

namespace ops {
namespace detail {

void write_adapter_file(const std::string& path, const std::map<std::string, TensorPtr>& tensors, const std::map<std::string, std::string>& metadata);
// Reads every tensor (as f32) and the metadata entries named in `metadata` (left untouched when absent).
std::map<std::string, TensorPtr> read_adapter_file(const std::string& path, std::map<std::string, std::string>* metadata);

}  // namespace detail
}  // namespace ops
