// GemmaLoRATrainer (the class surface of the reference's optim/gemma_trainer.h): epochs over a WikiText2Dataset with
// gradient accumulation, clipping, warm-up + linear / cosine schedule, periodic adapter checkpoints and evaluation.
// The dataset types come from data/wikitext2_dataset.h (host code, built from the reference's sources).
#pragma once
#include <chrono>
#include <memory>
#include <string>
#include <vector>

#include "../core/tensor.h"
#include "../graph/gemma_lora_injector.h"
#include "../graph/gemma_model.h"
#include "adam.h"

namespace ops {
class WikiText2Dataset;
struct Batch;
namespace detail { class StepDriver; }

struct GemmaTrainerConfig {
    float learning_rate = 2e-4f;
    float weight_decay = 0.0f;
    float adam_beta1 = 0.9f;
    float adam_beta2 = 0.999f;
    float adam_eps = 1e-8f;
    int num_epochs = 3;
    float max_grad_norm = 1.0f;
    std::string lr_scheduler = "linear";
    float warmup_ratio = 0.03f;
    int logging_steps = 10;
    int eval_steps = 100;
    std::string output_dir = "./gemma_lora_ckpt";
    int max_steps = -1;
    int micro_batch_size = 1;
    int grad_accum_steps = 1;
    int save_every = 0;                    // > 0: save the adapters every N optimizer steps
    bool dump_embedding = false;           // accepted; the fused device path has no embedding tensor to dump
    int dump_embedding_step = 1;
    std::string dump_embedding_dir = "./debug";
};

class GemmaLoRATrainer {
public:
    GemmaLoRATrainer(GemmaModel& model, GemmaLoraInjector& injector, WikiText2Dataset& train_data, WikiText2Dataset& eval_data,
                     const GemmaTrainerConfig& config);
    ~GemmaLoRATrainer();
    void train();
    float train_step(const Batch& batch);
    float evaluate();
    void save_lora(const std::string& path);

private:
    GemmaModel& model_;
    GemmaLoraInjector& injector_;
    WikiText2Dataset& train_data_;
    WikiText2Dataset& eval_data_;
    GemmaTrainerConfig config_;
    std::unique_ptr<detail::StepDriver> driver_;
    std::chrono::time_point<std::chrono::steady_clock> start_;
    bool started_ = false;
};

}  // namespace ops
