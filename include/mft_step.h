/*
 * mft_step.h - C ABI of the LoRA fine-tuning step engine in libmft_cuda.so.
 *
 * The engine is the device-side counterpart of the reference's model graphs and
 * step driver: GPT2Model / QwenModel / GemmaModel ::forward
 * (operator/finetune_ops/graph/gpt2_model.cpp:320-406, qwen_model.cpp:335-394,
 * gemma_model.cpp:579-646), lm_cross_entropy + Tensor::backward
 * (core/lm_loss.cpp:268-382, core/autograd_engine.cpp:144-273) and
 * Optimizer::clip_grad_norm + Adam::step + zero_grad
 * (optim/auto_trainer.cpp:20-46).  It schedules the kernels of mft_cuda.h on one
 * stream over preallocated activations; nothing here runs on the CPU.
 *
 * Parameter order and layouts are the reference's: mft_model_param_* walks
 * XModel::parameters(), mft_model_lora_* walks get_lora_parameters() (A then B
 * per LoRA'd linear; GPT-2/Qwen A[in,r], B[r,out]; Gemma A[r,in], B[out,r]).
 * Host-side values are fp32; frozen weights are rounded to bf16 on upload.
 */
#ifndef MFT_STEP_H
#define MFT_STEP_H

#include <stdint.h>

#include "mft_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

#define MFT_FAMILY_GPT2 0
#define MFT_FAMILY_QWEN 1
#define MFT_FAMILY_GEMMA 2

/* LoRA target bits.  GPT-2: c_attn, c_proj, c_fc, mlp_c_proj reuse Q, O, GATE, DOWN. */
#define MFT_LORA_Q 1
#define MFT_LORA_K 2
#define MFT_LORA_V 4
#define MFT_LORA_O 8
#define MFT_LORA_GATE 16
#define MFT_LORA_UP 32
#define MFT_LORA_DOWN 64

typedef struct {
    int32_t family;
    int32_t vocab, hidden, inter, layers, n_heads, n_kv_heads, head_dim;
    int32_t n_positions;        /* GPT-2 learned positions */
    float norm_eps;
    float rope_theta;           /* Qwen; Gemma global layers */
    float rope_local_theta;     /* Gemma sliding layers */
    float attn_scale;           /* 1/sqrt(head_dim), or query_pre_attn_scalar^-0.5 for Gemma */
    int32_t sliding_window;     /* Gemma: keys i-j < window on sliding layers */
    int32_t global_every;       /* Gemma: layer i is global iff (i+1) % global_every == 0; 0 = all sliding */
    int32_t lora_rank;
    float lora_alpha;
    uint32_t lora_targets;
    int32_t gpt2_detach_attn;   /* 1 = reproduce the reference: no gradient through GPT-2 attention */
    int32_t max_batch, max_seq;
} mft_model_config_t;

typedef struct mft_model mft_model_t;

int32_t mft_model_create(const mft_model_config_t* cfg, mft_stream_t stream, mft_model_t** out);
int32_t mft_model_destroy(mft_model_t* m);

/* Frozen parameters, in XModel::parameters() order. */
int32_t mft_model_param_count(const mft_model_t* m);
int32_t mft_model_param_shape(const mft_model_t* m, int32_t idx, int64_t* rows, int64_t* cols);
int32_t mft_model_set_param_host(mft_model_t* m, int32_t idx, const float* data_host);
/* The same from bf16 bits (a BF16 checkpoint: graph/safetensors_loader.h:35-46 of the reference converts such
 * tensors to f32 on the host; here they go up as stored, which is exact and half the bytes).  stored_transposed != 0:
 * a linear weight stored [out, in] (HuggingFace) instead of the API's [in, out]. */
int32_t mft_model_set_param_host_bf16(mft_model_t* m, int32_t idx, const void* data_bf16_host, int32_t stored_transposed);
/* Same, from a device f32 buffer (weights generated on the device). */
int32_t mft_model_set_param_dev(mft_model_t* m, int32_t idx, const float* data_dev);

/* Trainable LoRA tensors, in get_lora_parameters() order. */
int32_t mft_model_lora_count(const mft_model_t* m);
int32_t mft_model_lora_shape(const mft_model_t* m, int32_t idx, int64_t* rows, int64_t* cols);
int32_t mft_model_set_lora_host(mft_model_t* m, int32_t idx, const float* data_host);
int32_t mft_model_get_lora_host(mft_model_t* m, int32_t idx, float* data_host);
int32_t mft_model_get_lora_grad_host(mft_model_t* m, int32_t idx, float* data_host);
/* 1 if the reference's graph delivers a gradient to this tensor (GPT-2 c_attn does not). */
int32_t mft_model_lora_has_grad(const mft_model_t* m, int32_t idx);
/* Offset (in floats) of a LoRA tensor inside the flat buckets below. */
int32_t mft_model_lora_offset(const mft_model_t* m, int32_t idx, int64_t* offset);
/* Tells the model that the f32 LoRA values in the parameter bucket were changed
 * from outside (an optimizer that works on the bucket memory directly, as
 * ops::Adam over tensors bound to it does): the bf16 panels the GEMMs read are
 * re-packed before the next forward pass. */
int32_t mft_model_mark_lora_dirty(mft_model_t* m);
/* The flat f32 buckets every LoRA tensor lives in (params, grads): what a
 * data-parallel caller all-reduces between backward and the optimizer. */
int32_t mft_model_buckets(mft_model_t* m, float** params_dev, float** grads_dev, int64_t* n);

/* forward + shifted cross-entropy + backward for one batch.  ids / labels are
 * int32 [batch, seq] HOST buffers (pinned for overlap); they are copied to the
 * device inside the call.  Gradients are ACCUMULATED into the grad bucket.
 * n_valid_global > 0 overrides the local count of scored tokens in the 1/n
 * coefficient (data parallel).  loss_host receives the local mean loss. */
int32_t mft_model_forward_backward(mft_model_t* m, const int32_t* ids_host, const int32_t* labels_host,
                                   int32_t batch, int32_t seq, int64_t n_valid_global,
                                   float* loss_host, int32_t* n_valid_host);
/* Same with ids/labels already in device memory; the loss stays on the device
 * (loss_dev, n_valid_dev may be read later) and nothing synchronises. */
int32_t mft_model_forward_backward_dev(mft_model_t* m, const int32_t* ids_dev, const int32_t* labels_dev,
                                       int32_t batch, int32_t seq, int64_t n_valid_global,
                                       float** loss_dev, int32_t** n_valid_dev);
/* Forward only: mean loss for a batch (evaluation). */
int32_t mft_model_forward_loss(mft_model_t* m, const int32_t* ids_host, const int32_t* labels_host,
                               int32_t batch, int32_t seq, float* loss_host);
/* XModel::forward of the reference (gpt2_model.cpp:320-406, qwen_model.cpp:335-394,
 * gemma_model.cpp:579-646) with the logits written out: f32 [batch*seq, vocab]
 * on the device.  The loss paths above never need this tensor; it exists for
 * callers that read logits directly. */
int32_t mft_model_forward_logits(mft_model_t* m, const int32_t* ids_host, int32_t batch, int32_t seq, float* logits_dev);
/* QwenModel::forward_hidden (qwen_model.cpp:335-386): the final-norm output, f32 [batch*seq, hidden] on the device. */
int32_t mft_model_forward_hidden(mft_model_t* m, const int32_t* ids_host, int32_t batch, int32_t seq, float* hidden_dev);
/* ---- SafeTensors ingest and adapter files (host code; SafeTensorsReader / SafeTensorsModelReader
 *      graph/safetensors_loader.h:35-124, key mappers graph/safetensors_loader.cpp:470-590, LoraSaver
 *      graph/lora_saver.cpp:123-198, GemmaLoraInjector::save_lora_safetensors graph/gemma_lora_injector.cpp:179-264).
 * A container is one .safetensors file, a directory holding model.safetensors, or a sharded HuggingFace snapshot
 * (model.safetensors.index.json).  F32, F16 and BF16 tensors are read as f32; transpose2d returns a 2-D tensor
 * transposed (HF Linear weights are [out, in], the graphs use [in, out]). */
typedef struct mft_safetensors mft_safetensors_t;
int32_t mft_safetensors_open(const char* path_or_dir, mft_safetensors_t** out);
int32_t mft_safetensors_close(mft_safetensors_t* h);
int64_t mft_safetensors_count(const mft_safetensors_t* h);
const char* mft_safetensors_name(const mft_safetensors_t* h, int64_t i);
const char* mft_safetensors_metadata(const mft_safetensors_t* h, const char* key);     /* NULL when absent */
int32_t mft_safetensors_info(const mft_safetensors_t* h, const char* name, char* dtype8, int32_t* ndim, int64_t* shape8);
int32_t mft_safetensors_read_f32(const mft_safetensors_t* h, const char* name, float* out_host, int32_t transpose2d);
/* Writes n f32 tensors (shapes8: 8 extents per tensor, ndims[i] used) sorted by name, plus string metadata. */
int32_t mft_safetensors_write_f32(const char* path, int32_t n, const char* const* names, const int32_t* ndims,
                                  const int64_t* shapes8, const float* const* data, int32_t n_meta,
                                  const char* const* meta_keys, const char* const* meta_values);
/* HuggingFace key of frozen parameter idx ("" for a tensor the checkpoint does not carry, e.g. a tied lm_head)
 * and whether the file's tensor is the transpose of the parameter. */
int32_t mft_model_hf_key(const mft_model_t* m, int32_t idx, char* key_out, int32_t key_cap, int32_t* transpose);
/* Loads every frozen parameter from a HuggingFace checkpoint of the model's family (GPT-2 keys with or without
 * the "transformer." prefix) through the staging path (host f32 -> device, cast / fused-group packing there). */
int32_t mft_model_load_safetensors(mft_model_t* m, const char* path_or_dir);
/* Adapter file: keys layer.{i}.{target}.lora_A / .lora_B in the reference's tensor layouts, F32, sorted, with
 * rank / alpha / dropout / targets in __metadata__.  Load checks rank and shapes. */
int32_t mft_model_save_lora_safetensors(mft_model_t* m, const char* path);
int32_t mft_model_load_lora_safetensors(mft_model_t* m, const char* path);

/* ---- double-buffered input (the Batch tensors of WikiText2Dataset::get_batch, data/wikitext2_dataset.cpp:451-519,
 *      are rebuilt in the same host buffers for every batch): batch k+1 is copied to the device on a copy stream
 *      while step k computes, and the loss of step k is read back without stalling step k+1.
 *      mft_model_stage_batch(slot): asynchronous copy of ids / labels ([batch, seq] int32, PAGE-LOCKED host memory,
 *      e.g. from mft_host_alloc) into device slot 0 or 1; the host buffers may be refilled once
 *      mft_model_stage_wait(slot) returned (or after the step that consumes the slot was queued and synchronised).
 *      mft_model_step_staged(slot): forward + backward on the staged batch; the mean loss and the count of scored
 *      tokens are copied asynchronously to page-locked host words that are valid after mft_model_sync (or after
 *      any later synchronising call on the model). */
int32_t mft_model_stage_batch(mft_model_t* m, int32_t slot, const int32_t* ids_pinned, const int32_t* labels_pinned,
                              int32_t batch, int32_t seq);
int32_t mft_model_stage_wait(mft_model_t* m, int32_t slot);
int32_t mft_model_step_staged(mft_model_t* m, int32_t slot, int32_t batch, int32_t seq, int64_t n_valid_global,
                              float* loss_pinned, int32_t* n_valid_pinned);
int32_t mft_model_sync(mft_model_t* m);

/* ---- evaluation drivers (no gradients, same forward kernels).
 * Perplexity, the loop body of examples/gpt2_small_lora_finetune/src/eval_ppl.cpp:170-210: one batch's mean loss
 * is weighted by the number of labels != -100 in the WHOLE labels tensor (the reference counts them unshifted),
 * summed in double; mean_nll = sum_loss / sum_tokens, ppl = expf(mean_nll). */
typedef struct {
    double sum_loss;
    int64_t sum_tokens;
    int64_t n_batches;
} mft_ppl_accum_t;
int32_t mft_model_eval_ppl_batch(mft_model_t* m, mft_ppl_accum_t* acc, const int32_t* ids_host, const int32_t* labels_host,
                                 int32_t batch, int32_t seq);
int32_t mft_ppl_result(const mft_ppl_accum_t* acc, float* mean_nll, float* ppl);
/* Letter scoring, MMLURunner::predict_letter (examples/common/mmlu/mmlu_runner.cpp:141-192): forward of ONE prompt
 * (seq >= 2 token ids), log_softmax of the logits at its last position, read at n_cand candidate token ids
 * (<= 64).  logprob_host[c] = log p(cand[c] | prompt); an id outside the vocabulary gets -1e30 as in the
 * reference.  The [seq, V] logits are never formed: only the last position is projected. */
int32_t mft_model_score_tokens(mft_model_t* m, const int32_t* ids_host, int32_t seq, const int32_t* cand_host,
                               int32_t n_cand, float* logprob_host);
/* LoRALinear::merge_to_base / unmerge_from_base (nn/lora_linear.cpp:470-508; LoraInjector::merge / unmerge and
 * GemmaLoraInjector::merge_all / unmerge_all call them per layer): fold scale * A B of every adapted slice into the
 * device copies of the frozen weights, W[i, col0+o] += scale * float(sum_r double(A[i,r]) double(B[r,o])), rounded
 * to the weights' bf16 storage as the reference rounds to its weight dtype.  While merged, forward / evaluation
 * calls skip the adapter products and training calls (forward_backward, optimizer_step, set_lora) return
 * MFT_ERR_INVALID_ARG.  Unmerge restores the saved weights byte for byte, as the reference's backup does. */
int32_t mft_model_merge_lora(mft_model_t* m);
int32_t mft_model_unmerge_lora(mft_model_t* m);
int32_t mft_model_is_merged(const mft_model_t* m);
/* clip (max_norm <= 0: none; clip_eps 0 = Optimizer::clip_grad_norm, 1e-6 = trainers) + Adam + zero_grad. */
int32_t mft_model_optimizer_step(mft_model_t* m, float lr, float beta1, float beta2, float eps,
                                 float weight_decay, float max_norm, float clip_eps);
int32_t mft_model_zero_grad(mft_model_t* m);
/* Factor applied to d(loss) in the next forward_backward calls (default 1): a driver that accumulates
 * gradients over several micro-batches passes 1 / grad_accum_steps, as the reference's trainers do by
 * back-propagating mul(loss, 1 / grad_accum_steps). */
int32_t mft_model_set_loss_scale(mft_model_t* m, float scale);

/* ---- step driver: the loop body of GemmaLoRATrainer::train_step (optim/gemma_trainer.cpp:85-147) and
 *      LoRATrainer::train_step (optim/trainer.cpp:102-146) with everything after the batch upload on the device:
 *      micro-batch forward + loss + backward with the loss scaled by 1/grad_accum_steps, gradients accumulated
 *      in the LoRA bucket; every grad_accum_steps-th call clips (if ||g|| > max_grad_norm: g *= max / (||g|| + 1e-6),
 *      the trainers' rule), sets the learning rate from the schedule, runs Adam and clears the gradients.
 *      The LoRA gradients never leave the GPU. */
enum { MFT_LR_LINEAR = 0, MFT_LR_COSINE = 1, MFT_LR_CONSTANT = 2 };
typedef struct {
    float learning_rate, weight_decay, adam_beta1, adam_beta2, adam_eps;
    float max_grad_norm;         /* <= 0: no clipping */
    float warmup_ratio;
    int32_t lr_scheduler;        /* MFT_LR_*: GemmaLoRATrainer treats every name but "cosine" as linear; LoRATrainer
                                    keeps the rate constant after the warm-up for a name it does not know */
    int32_t grad_accum_steps;
    int64_t total_updates;       /* optimizer steps of the run: ceil(ceil(num_sequences / micro_batch) * epochs / grad_accum) */
} mft_trainer_config_t;
typedef struct mft_trainer mft_trainer_t;
/* Learning rate of optimizer step `step` (1-based), get_lr of both trainers.  Pure host arithmetic. */
float mft_trainer_lr(const mft_trainer_config_t* cfg, int64_t step);
int32_t mft_trainer_create(mft_model_t* model, const mft_trainer_config_t* cfg, mft_trainer_t** out);
int32_t mft_trainer_destroy(mft_trainer_t* t);
/* One micro-batch (host ids / labels, as Batch carries them).  *stepped = 1 and *avg_loss = mean of the window's
 * micro-batch losses when this call closed an accumulation window (the reference returns that mean), else
 * *stepped = 0 (the reference returns -1).  n_valid_global as in mft_model_forward_backward.
 * *lr_used (optional) receives the learning rate of the step taken. */
int32_t mft_trainer_train_step(mft_trainer_t* t, const int32_t* ids_host, const int32_t* labels_host,
                               int32_t batch, int32_t seq, int64_t n_valid_global,
                               int32_t* stepped, float* avg_loss, float* lr_used);
int64_t mft_trainer_global_step(const mft_trainer_t* t);
/* Debug/parity taps: copy the final hidden states (f32 [batch*seq, hidden], after the last norm). */
int32_t mft_model_get_final_hidden_host(mft_model_t* m, float* out_host, int64_t n_elements);
int64_t mft_model_activation_bytes(const mft_model_t* m);

#ifdef __cplusplus
}
#endif
#endif /* MFT_STEP_H */
