// Test program for the C++ operator API: drives one LoRA step exactly the way the reference's
// graph/test_auto_model.cpp drives its AutoTrainer (config.json -> from_pretrained(load_weights=false) ->
// fill parameters() -> init_lora -> fill trainable_parameters() -> AutoTrainer::train_step), on inputs read
// from raw little-endian files, and dumps the loss, the LoRA gradients and the updated LoRA tensors.
//
//   auto_trainer_step <case_dir>     case.txt: batch, seq, lr, max_grad_norm, lora_rank, lora_alpha, lora_targets (comma separated)
#include <cstdio>
#include <fstream>
#include <iostream>
#include <map>
#include <sstream>
#include <stdexcept>
#include <string>
#include <sys/stat.h>
#include <vector>

#include "mobile_finetuner/mobile_finetuner.h"
#include "finetune_ops/graph/auto_model.h"
#include "finetune_ops/core/lm_loss.h"
#include "finetune_ops/optim/auto_trainer.h"

static void read_bin(const std::string& path, void* dst, size_t bytes) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open " + path);
    f.read(static_cast<char*>(dst), (std::streamsize)bytes);
    if ((size_t)f.gcount() != bytes) throw std::runtime_error("short read: " + path);
}
static void write_bin(const std::string& path, const void* src, size_t bytes) {
    std::ofstream f(path, std::ios::binary);
    f.write(static_cast<const char*>(src), (std::streamsize)bytes);
}
static std::string idx(size_t i) { char b[16]; std::snprintf(b, sizeof b, "%04zu", i); return b; }

int main(int argc, char** argv) {
    if (argc < 2) { std::fprintf(stderr, "usage: auto_trainer_step <case_dir>\n"); return 2; }
    try {
        const std::string dir = argv[1];
        std::map<std::string, std::string> kv;
        std::ifstream cf(dir + "/case.txt");
        std::string line;
        while (std::getline(cf, line)) { auto sp = line.find(' '); if (sp != std::string::npos) kv[line.substr(0, sp)] = line.substr(sp + 1); }
        const int B = std::stoi(kv.at("batch")), S = std::stoi(kv.at("seq"));
        mkdir((dir + "/out").c_str(), 0755);

        ops::AutoModelLoadOptions opt;
        opt.load_weights = false;
        auto model = ops::AutoModelForCausalLM::from_pretrained(dir, opt);
        auto params = model->parameters();
        for (size_t i = 0; i < params.size(); ++i) read_bin(dir + "/params/" + idx(i) + ".bin", params[i]->data<float>(), (size_t)params[i]->numel() * 4);

        ops::AutoLoraConfig lc;
        lc.rank = std::stoi(kv.at("lora_rank"));
        lc.alpha = std::stof(kv.at("lora_alpha"));
        std::stringstream ss(kv.at("lora_targets"));
        for (std::string t; std::getline(ss, t, ',');) if (!t.empty()) lc.target_modules.push_back(t);
        model->init_lora(lc);
        auto lora = model->trainable_parameters();
        for (size_t i = 0; i < lora.size(); ++i) read_bin(dir + "/lora/" + idx(i) + ".bin", lora[i]->data<float>(), (size_t)lora[i]->numel() * 4);

        auto ids = std::make_shared<ops::Tensor>(std::vector<int64_t>{B, S}, ops::kInt32, ops::kCPU);
        auto labels = std::make_shared<ops::Tensor>(std::vector<int64_t>{B, S}, ops::kInt32, ops::kCPU);
        auto mask = ops::ones({B, S});
        read_bin(dir + "/ids.bin", ids->data<int32_t>(), (size_t)B * S * 4);
        read_bin(dir + "/labels.bin", labels->data<int32_t>(), (size_t)B * S * 4);

        // gradients of the same batch first, through the reference's own sequence (forward -> lm_cross_entropy ->
        // backward); the trainer's step below starts from cleared gradients again
        {
            auto logits = model->forward(ids, mask);
            auto loss = ops::lm_cross_entropy(logits, labels, -100, "mean");
            loss->backward();
            const float loss0 = static_cast<const ops::Tensor&>(*loss).data<float>()[0];
            write_bin(dir + "/out/loss0.bin", &loss0, 4);
            for (size_t i = 0; i < lora.size(); ++i)
                if (auto g = lora[i]->grad()) write_bin(dir + "/out/grad_" + idx(i) + ".bin", static_cast<const ops::Tensor&>(*g).data<float>(), (size_t)g->numel() * 4);
            for (auto& p : lora) p->zero_grad();
        }

        ops::AutoTrainerConfig tc;
        tc.learning_rate = std::stof(kv.at("lr"));
        tc.max_grad_norm = std::stof(kv.at("max_grad_norm"));
        ops::AutoTrainer trainer(*model, tc);
        const auto res = trainer.train_step(ids, mask, labels);
        write_bin(dir + "/out/loss.bin", &res.loss, 4);
        auto after = model->trainable_parameters();
        for (size_t i = 0; i < after.size(); ++i) write_bin(dir + "/out/lora_" + idx(i) + ".bin", static_cast<const ops::Tensor&>(*after[i]).data<float>(), (size_t)after[i]->numel() * 4);
        std::printf("loss %.6f tensors %d\n", res.loss, res.trainable_tensor_count);
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "auto_trainer_step error: %s\n", e.what());
        return 1;
    }
}
