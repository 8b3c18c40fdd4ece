// Umbrella header of the operator API as far as the LoRA step's path goes.
#pragma once
#include "finetune_ops/core/autograd_engine.h"
#include "finetune_ops/core/lm_loss.h"
#include "finetune_ops/core/memory_efficient_attention.h"
#include "finetune_ops/core/memory_manager.h"
#include "finetune_ops/core/ops.h"
#include "finetune_ops/core/tensor.h"
#include "finetune_ops/nn/lora_linear.h"
#include "finetune_ops/optim/adam.h"
