#include "gemma_trainer.h"

#include <filesystem>
#include <iomanip>
#include <iostream>

#include "../core/lm_loss.h"
#include "../core/memory_manager.h"
#include "../data/wikitext2_dataset.h"
#include "step_driver.h"

namespace ops {

GemmaLoRATrainer::GemmaLoRATrainer(GemmaModel& model, GemmaLoraInjector& injector, WikiText2Dataset& train_data, WikiText2Dataset& eval_data,
                                   const GemmaTrainerConfig& config)
    : model_(model), injector_(injector), train_data_(train_data), eval_data_(eval_data), config_(config) {
    AdamConfig a;
    a.learning_rate = config_.learning_rate; a.beta1 = config_.adam_beta1; a.beta2 = config_.adam_beta2; a.epsilon = config_.adam_eps;
    a.weight_decay = config_.weight_decay;
    a.clip_grad_norm = config_.max_grad_norm;
    detail::StepDriverConfig d;
    d.learning_rate = config_.learning_rate; d.max_grad_norm = config_.max_grad_norm; d.warmup_ratio = config_.warmup_ratio;
    d.lr_scheduler = config_.lr_scheduler; d.constant_when_unknown = false;
    d.grad_accum_steps = config_.grad_accum_steps; d.micro_batch_size = config_.micro_batch_size; d.num_epochs = config_.num_epochs;
    driver_ = std::make_unique<detail::StepDriver>([this](const TensorPtr& ids, const TensorPtr& mask) { return model_.forward(ids, mask); },
                                                   [this] { return injector_.get_trainable_params(); }, a, d);
    std::cout << "[GemmaTrainer] LR=" << config_.learning_rate << ", epochs=" << config_.num_epochs << ", grad_accum=" << config_.grad_accum_steps << std::endl;
}

GemmaLoRATrainer::~GemmaLoRATrainer() = default;

float GemmaLoRATrainer::train_step(const Batch& batch) {
    return driver_->micro_step(batch.input_ids, batch.attention_mask, batch.labels, (int64_t)train_data_.num_sequences());
}

float GemmaLoRATrainer::evaluate() {
    eval_data_.reset_cursor();
    float total = 0.0f;
    int n = 0;
    for (;;) {
        auto batch = eval_data_.next_batch(config_.micro_batch_size, false);
        if (!batch.input_ids) break;
        total += driver_->eval_loss(batch.input_ids, batch.attention_mask, batch.labels);
        ++n;
    }
    const float mean = n > 0 ? total / n : 0.0f;
    std::cout << "  Eval Loss: " << mean << " PPL: " << perplexity_from_loss(mean) << std::endl;
    MemoryManager::instance().force_cleanup();
    return mean;
}

void GemmaLoRATrainer::train() {
    if (!started_) { start_ = std::chrono::steady_clock::now(); started_ = true; }
    for (int epoch = 0; epoch < config_.num_epochs; ++epoch) {
        std::cout << "\n=== Gemma Epoch " << (epoch + 1) << "/" << config_.num_epochs << " ===" << std::endl;
        train_data_.reset_cursor();
        float epoch_loss = 0.0f;
        int windows = 0;
        bool stop = false;
        for (;;) {
            auto batch = train_data_.next_batch(config_.micro_batch_size, false);
            if (!batch.input_ids) break;
            const float loss = train_step(batch);
            if (loss < 0.0f) continue;
            epoch_loss += loss;
            ++windows;
            const int step = driver_->global_step();
            if (config_.logging_steps > 0 && step % config_.logging_steps == 0) {
                const double s = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - start_).count() / 1000.0;
                std::cout << "[Step " << step << "] Loss=" << loss << " PPL=" << perplexity_from_loss(loss) << " LR="
                          << driver_->lr_at(step, (int64_t)train_data_.num_sequences()) << " | time_cum=" << std::fixed << std::setprecision(3) << s
                          << "s" << std::defaultfloat << std::endl;
            }
            if (config_.save_every > 0 && step % config_.save_every == 0) {
                try {
                    std::filesystem::create_directories(config_.output_dir);
                    const std::string ckpt = config_.output_dir + "/gemma_lora_step" + std::to_string(step) + ".safetensors";
                    save_lora(ckpt);
                    std::cout << "[Checkpoint] Saved LoRA at step " << step << " -> " << ckpt << std::endl;
                } catch (const std::exception& e) {
                    std::cerr << "[Checkpoint] Failed to save at step " << step << ": " << e.what() << std::endl;
                }
            }
            if (config_.eval_steps > 0 && step % config_.eval_steps == 0) evaluate();
            if (config_.max_steps > 0 && step >= config_.max_steps) { stop = true; break; }
        }
        std::cout << "Epoch " << (epoch + 1) << " avg loss: " << (windows > 0 ? epoch_loss / windows : 0.0f) << std::endl;
        MemoryManager::instance().clear_unused_memory();
        if (stop) {
            std::cout << "[GemmaTrainer] Reached max_steps=" << config_.max_steps << ", stopping early." << std::endl;
            break;
        }
    }
    MemoryManager::instance().force_cleanup();
}

void GemmaLoRATrainer::save_lora(const std::string& path) { injector_.save_lora_safetensors(path); }

}  // namespace ops
