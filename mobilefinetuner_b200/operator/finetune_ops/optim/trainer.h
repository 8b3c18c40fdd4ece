// LoRATrainer for GPT-2 (the class surface of the reference's optim/trainer.h): epochs over a WikiText2Dataset with
// gradient accumulation, gradient clipping, a warm-up + linear / cosine schedule and periodic evaluation.
// The dataset types come from data/wikitext2_dataset.h (host code, built from the reference's sources).
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "../core/tensor.h"
#include "../graph/gpt2_model.h"
#include "../graph/lora_injector.h"
#include "adam.h"

namespace ops {
class WikiText2Dataset;
struct Batch;
namespace detail { class StepDriver; }

struct TrainerConfig {
    float learning_rate = 2e-4f;
    float weight_decay = 0.01f;            // ignored: adapters train without weight decay (as in the reference)
    float adam_beta1 = 0.9f;
    float adam_beta2 = 0.999f;
    float adam_eps = 1e-8f;
    int num_epochs = 3;
    int micro_batch_size = 1;
    int gradient_accumulation_steps = 1;
    float max_grad_norm = 1.0f;
    std::string lr_scheduler = "linear";   // "linear" or "cosine"
    float warmup_ratio = 0.03f;
    int logging_steps = 10;
    int eval_steps = 100;
    std::string output_dir = "./lora_checkpoints";
};

class LoRATrainer {
public:
    LoRATrainer(GPT2Model& model, LoraInjector& lora, WikiText2Dataset& train_data, WikiText2Dataset& eval_data, const TrainerConfig& config);
    ~LoRATrainer();
    void train();
    float train_step(const Batch& batch);      // mean loss of the window when it closed one, else -1
    float evaluate();                           // mean loss over the evaluation split
    void save_lora(const std::string& path);

private:
    GPT2Model& model_;
    LoraInjector& lora_;
    WikiText2Dataset& train_data_;
    WikiText2Dataset& eval_data_;
    TrainerConfig config_;
    std::unique_ptr<detail::StepDriver> driver_;
};

}  // namespace ops
