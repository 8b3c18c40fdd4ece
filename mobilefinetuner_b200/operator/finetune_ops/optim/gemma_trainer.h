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

struct GemmaTrainerConfig {                // field order as in the reference
    // optimizer (the reference's L2-style Adam)
    float learning_rate = 2e-4f, weight_decay = 0.0f;
    float adam_beta1 = 0.9f, adam_beta2 = 0.999f, adam_eps = 1e-8f;
    int num_epochs = 3;
    float max_grad_norm = 1.0f;
    std::string lr_scheduler = "linear";   // or "cosine"; both after a linear warm-up over warmup_ratio of the updates
    float warmup_ratio = 0.03f;
    int logging_steps = 10, eval_steps = 100;
    std::string output_dir = "./gemma_lora_ckpt";
    int max_steps = -1;                    // > 0: stop after this many optimizer steps
    int micro_batch_size = 1, grad_accum_steps = 1;
    int save_every = 0;                    // > 0: save the adapters every N optimizer steps
    bool dump_embedding = false;           // accepted; the fused device path has no embedding tensor to dump
    int dump_embedding_step = 1;
    std::string dump_embedding_dir = "./debug";
};

class GemmaLoRATrainer {
    GemmaModel& model_;
    GemmaLoraInjector& injector_;
    WikiText2Dataset &train_data_, &eval_data_;
    GemmaTrainerConfig config_;
    std::unique_ptr<detail::StepDriver> driver_;      // accumulation window, clip rule, schedule, Adam on the device
    std::chrono::time_point<std::chrono::steady_clock> start_;
    bool started_ = false;
public:
    GemmaLoRATrainer(GemmaModel& model, GemmaLoraInjector& injector, WikiText2Dataset& train_data, WikiText2Dataset& eval_data,
                     const GemmaTrainerConfig& config);
    ~GemmaLoRATrainer();
    void train();                               // epochs over train_data_, evaluation / checkpoints as configured
    float train_step(const Batch& batch);       // one micro-batch; -1 inside an accumulation window, else the window's mean loss
    float evaluate();                           // mean loss over eval_data_
    void save_lora(const std::string& path);
};

}  // namespace ops
