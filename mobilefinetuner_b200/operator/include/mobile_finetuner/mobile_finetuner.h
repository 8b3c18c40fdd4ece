// Umbrella header of the operator API: everything the reference's include/mobile_finetuner/mobile_finetuner.h pulls
// in.  Tokenizers and datasets are host code that this repository takes from the reference's tree at build time (see
// operator/CMakeLists.txt, MFT_REFERENCE_OPERATOR_DIR); their headers are included when the build has staged them.
#pragma once

#include "finetune_ops/core/autograd_engine.h"
#include "finetune_ops/core/dtype.h"
#include "finetune_ops/core/lm_loss.h"
#include "finetune_ops/core/memory_efficient_attention.h"
#include "finetune_ops/core/memory_manager.h"
#include "finetune_ops/core/ops.h"
#include "finetune_ops/core/tensor.h"
#if __has_include("finetune_ops/core/tokenizer.h")
#include "finetune_ops/core/tokenizer.h"
#endif

#if __has_include("finetune_ops/data/wikitext2_dataset.h")
#include "finetune_ops/data/mmlu_dataset.h"
#include "finetune_ops/data/wikitext2_dataset.h"
#endif

#include "finetune_ops/graph/auto_model.h"
#include "finetune_ops/graph/gemma_lora_injector.h"
#include "finetune_ops/graph/gemma_model.h"
#include "finetune_ops/graph/gpt2_model.h"
#include "finetune_ops/graph/lora_injector.h"
#include "finetune_ops/graph/lora_saver.h"
#include "finetune_ops/graph/model_registry.h"
#include "finetune_ops/graph/qwen_model.h"
#include "finetune_ops/graph/safetensors_loader.h"

#include "finetune_ops/nn/lora_linear.h"

#include "finetune_ops/optim/adam.h"
#include "finetune_ops/optim/auto_trainer.h"
#include "finetune_ops/optim/gemma_trainer.h"
#include "finetune_ops/optim/optimizer.h"
#include "finetune_ops/optim/trainer.h"
