#include "trainer.h"

#include <iostream>

#include "../core/lm_loss.h"
#include "../core/memory_manager.h"
#include "../data/wikitext2_dataset.h"
#include "step_driver.h"

namespace ops {

LoRATrainer::LoRATrainer(GPT2Model& model, LoraInjector& lora, WikiText2Dataset& train_data, WikiText2Dataset& eval_data, const TrainerConfig& config)
    : model_(model), lora_(lora), train_data_(train_data), eval_data_(eval_data), config_(config) {
    AdamConfig a;
    a.learning_rate = config_.learning_rate; a.beta1 = config_.adam_beta1; a.beta2 = config_.adam_beta2; a.epsilon = config_.adam_eps;
    a.weight_decay = 0.0f;
    a.clip_grad_norm = config_.max_grad_norm;
    detail::StepDriverConfig d;
    d.learning_rate = config_.learning_rate; d.max_grad_norm = config_.max_grad_norm; d.warmup_ratio = config_.warmup_ratio;
    d.lr_scheduler = config_.lr_scheduler; d.constant_when_unknown = true;
    d.grad_accum_steps = config_.gradient_accumulation_steps; d.micro_batch_size = config_.micro_batch_size; d.num_epochs = config_.num_epochs;
    driver_ = std::make_unique<detail::StepDriver>([this](const TensorPtr& ids, const TensorPtr& mask) { return model_.forward(ids, mask); },
                                                   [this] { return lora_.get_trainable_params(); }, a, d);
    std::cout << "[Trainer] lr " << config_.learning_rate << ", epochs " << config_.num_epochs << ", micro batch " << config_.micro_batch_size
              << ", accumulation " << config_.gradient_accumulation_steps << ", max grad norm " << config_.max_grad_norm << std::endl;
}

LoRATrainer::~LoRATrainer() = default;

float LoRATrainer::train_step(const Batch& batch) {
    return driver_->micro_step(batch.input_ids, batch.attention_mask, batch.labels, (int64_t)train_data_.num_sequences());
}

float LoRATrainer::evaluate() {
    eval_data_.reset_cursor();
    float total = 0.0f;
    int n = 0;
    for (;;) {
        auto batch = eval_data_.next_batch(config_.micro_batch_size, false);
        if (!batch.input_ids) break;
        total += driver_->eval_loss(batch.input_ids, batch.attention_mask, batch.labels);
        ++n;
    }
    MemoryManager::instance().force_cleanup();
    const float mean = n > 0 ? total / n : 0.0f;
    std::cout << "[Eval] loss " << mean << ", perplexity " << perplexity_from_loss(mean) << std::endl;
    return mean;
}

void LoRATrainer::train() {
    for (int epoch = 0; epoch < config_.num_epochs; ++epoch) {
        std::cout << "--- Epoch " << (epoch + 1) << "/" << config_.num_epochs << " ---" << std::endl;
        train_data_.reset_cursor();
        float epoch_loss = 0.0f;
        int windows = 0;
        for (;;) {
            auto batch = train_data_.next_batch(config_.micro_batch_size, false);
            if (!batch.input_ids) break;
            const float loss = train_step(batch);
            if (loss < 0.0f) continue;
            epoch_loss += loss;
            ++windows;
            const int step = driver_->global_step();
            if (config_.logging_steps > 0 && step % config_.logging_steps == 0)
                std::cout << "[Step " << step << "] Loss: " << loss << ", PPL: " << perplexity_from_loss(loss) << ", LR: "
                          << driver_->lr_at(step, (int64_t)train_data_.num_sequences()) << std::endl;
            if (config_.eval_steps > 0 && step % config_.eval_steps == 0) {
                evaluate();
                train_data_.reset_cursor();        // as the reference: the training iterator restarts after an evaluation
            }
        }
        std::cout << "Epoch " << (epoch + 1) << " finished, Mean Loss: " << (windows > 0 ? epoch_loss / windows : 0.0f) << std::endl;
        MemoryManager::instance().force_cleanup();
    }
    MemoryManager::instance().print_memory_stats();
}

void LoRATrainer::save_lora(const std::string& path) { lora_.save_lora_safetensors(path); }

}  // namespace ops
