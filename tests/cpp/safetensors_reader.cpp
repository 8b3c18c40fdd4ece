// The SafeTensors reader classes and key maps of the source-level mirror, used as reference code uses them:
// write a small checkpoint, open it through SafeTensorsModelReader, load it with a key mapping and the default
// options (HF Linear weights come back transposed, embeddings and 1-D tensors do not).  Host only.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <string>
#include <vector>

#include "finetune_ops/graph/safetensors_loader.h"
#include "mft_cuda.h"
#include "mft_step.h"

using namespace ops;

#define CHECK(cond)                                                              \
    do {                                                                         \
        if (!(cond)) { std::printf("FAILED: %s (line %d)\n", #cond, __LINE__); return 1; } \
    } while (0)

int main(int argc, char** argv) {
    const std::string dir = argc > 1 ? argv[1] : "/tmp";
    const std::string path = dir + "/model.safetensors";
    // q_proj.weight [out = 3, in = 2], embed [4, 2], a norm vector [2]
    const float q[6] = {1, 2, 3, 4, 5, 6}, e[8] = {0, 1, 2, 3, 4, 5, 6, 7}, n[2] = {0.5f, -0.5f};
    const char* names[3] = {"model.layers.0.self_attn.q_proj.weight", "model.embed_tokens.weight", "model.layers.0.input_layernorm.weight"};
    const int32_t ndims[3] = {2, 2, 1};
    int64_t shapes[24] = {0};
    shapes[0] = 3; shapes[1] = 2; shapes[8] = 4; shapes[9] = 2; shapes[16] = 2;
    const float* data[3] = {q, e, n};
    CHECK(mft_safetensors_write_f32(path.c_str(), 3, names, ndims, shapes, data, 0, nullptr, nullptr) == MFT_OK);

    SafeTensorsModelReader reader(dir);
    reader.parse_headers();
    CHECK(reader.files().size() == 1 && reader.get_tensor_names().size() == 3);
    auto mapping = GemmaKeyMapper::generate_gemma_mapping(1);
    CHECK(mapping.size() == 3 + 13);
    CHECK(mapping["layers.0.self_attn.q_proj.weight"] == "model.layers.0.self_attn.q_proj.weight");
    SafeTensorsLoadOptions opt;
    opt.verbose = false;
    auto loaded = reader.load_tensors_mapped(mapping, opt);
    CHECK(loaded.size() == 3);                                    // the keys the file does not have are skipped
    auto w = loaded["layers.0.self_attn.q_proj.weight"];
    CHECK(w->shape() == (std::vector<int64_t>{2, 3}));             // [in, out]
    const float* wd = w->data<float>();
    CHECK(wd[0] == 1 && wd[1] == 3 && wd[2] == 5 && wd[3] == 2 && wd[4] == 4 && wd[5] == 6);
    auto emb = loaded["embed_tokens.weight"];
    CHECK(emb->shape() == (std::vector<int64_t>{4, 2}) && emb->data<float>()[3] == 3);      // embeddings are not transposed
    CHECK(loaded["layers.0.input_layernorm.weight"]->data<float>()[1] == -0.5f);

    SafeTensorsReader single(path);
    single.parse_header();
    CHECK(single.get_tensor_info(names[0]).dtype == "F32");
    auto raw = single.load_tensor(names[0], false);
    CHECK(raw->shape() == (std::vector<int64_t>{3, 2}) && raw->data<float>()[5] == 6);

    CHECK(GPT2KeyMapper::generate_gpt2_mapping(12).size() == 4 + 12 * 12);
    CHECK(GPT2KeyMapper::generate_gpt2_mapping(2)["blocks.1.attn.qkv.bias"] == "h.1.attn.c_attn.bias");
    auto qm = QwenKeyMapper::generate_qwen_mapping(24);
    CHECK(qm.size() == 2 + 24 * 12 && qm["layers.23.post_norm.weight"] == "model.layers.23.post_attention_layernorm.weight");
    std::printf("safetensors reader: all checks passed\n");
    return 0;
}
