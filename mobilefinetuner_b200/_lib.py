"""ctypes binding of libmft_cuda.so (the C ABI declared in include/mft_cuda.h).

There is no fallback: if the shared object is missing or a call fails, an
exception is raised.  PyTorch is only used by callers for device memory and
streams; pointers cross this boundary as plain integers.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libmft_cuda.so"

MFT_F32, MFT_BF16, MFT_I32 = 0, 1, 2
ACT_GELU, ACT_SWIGLU, ACT_GEGLU = 0, 1, 2
MFT_ERR_UNSUPPORTED = -7


class MftError(RuntimeError):
    pass


class Strides(C.Structure):
    _fields_ = [("stride_b", C.c_int64), ("stride_s", C.c_int64), ("stride_h", C.c_int64)]


class BlockCopy(C.Structure):
    _fields_ = [("src", C.c_void_p), ("dst", C.c_void_p), ("rows", C.c_int32), ("cols", C.c_int32),
                ("src_ld", C.c_int32), ("dst_ld", C.c_int32), ("transpose", C.c_int32), ("pad", C.c_int32)]


class TrainerConfig(C.Structure):
    """mft_trainer_config_t of include/mft_step.h (fields of GemmaTrainerConfig / TrainerConfig that drive a step)."""
    _fields_ = [("learning_rate", C.c_float), ("weight_decay", C.c_float), ("adam_beta1", C.c_float), ("adam_beta2", C.c_float),
                ("adam_eps", C.c_float), ("max_grad_norm", C.c_float), ("warmup_ratio", C.c_float), ("lr_scheduler", C.c_int32),
                ("grad_accum_steps", C.c_int32), ("total_updates", C.c_int64)]


LR_SCHEDULERS = {"linear": 0, "cosine": 1, "constant": 2}


class PplAccum(C.Structure):
    """mft_ppl_accum_t of include/mft_step.h."""
    _fields_ = [("sum_loss", C.c_double), ("sum_tokens", C.c_int64), ("n_batches", C.c_int64)]


class ModelConfig(C.Structure):
    """mft_model_config_t of include/mft_step.h."""
    _fields_ = [("family", C.c_int32), ("vocab", C.c_int32), ("hidden", C.c_int32), ("inter", C.c_int32),
                ("layers", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32),
                ("n_positions", C.c_int32), ("norm_eps", C.c_float), ("rope_theta", C.c_float),
                ("rope_local_theta", C.c_float), ("attn_scale", C.c_float), ("sliding_window", C.c_int32),
                ("global_every", C.c_int32), ("lora_rank", C.c_int32), ("lora_alpha", C.c_float),
                ("lora_targets", C.c_uint32), ("gpt2_detach_attn", C.c_int32), ("max_batch", C.c_int32),
                ("max_seq", C.c_int32)]


_lib = None

i32, i64, f32, vp, sz = C.c_int32, C.c_int64, C.c_float, C.c_void_p, C.c_size_t

# name -> argument types (every function returns int32 unless listed in _RET)
_SIGS = {
    "mft_init": [i32],
    "mft_shutdown": [],
    "mft_version": [],
    "mft_stream_sync": [vp],
    "mft_device_status": [vp, C.POINTER(i32)],
    "mft_malloc": [sz, vp, C.POINTER(vp)],
    "mft_free": [vp, vp],
    "mft_comm_unique_id": [vp],
    "mft_comm_init": [i32, i32, vp],
    "mft_comm_info": [C.POINTER(i32), C.POINTER(i32), C.POINTER(i32)],
    "mft_allreduce_sum_f32": [vp, i64, vp],
    "mft_allreduce_sum_i64": [vp, i64, vp],
    "mft_comm_async_error": [C.POINTER(i32)],
    "mft_comm_wait": [vp, i32],
    "mft_comm_abort": [],
    "mft_comm_destroy": [],
    "mft_empty_cache": [],
    "mft_trim_cache": [i64],
    "mft_mem_stats": [C.POINTER(i64)],
    "mft_host_alloc": [C.c_size_t, vp],
    "mft_host_free": [vp],
    "mft_memcpy_h2d": [vp, vp, sz, vp],
    "mft_memcpy_d2h": [vp, vp, sz, vp],
    "mft_memcpy_d2d": [vp, vp, sz, vp],
    "mft_memset": [vp, i32, sz, vp],
    "mft_cast_f32_to_bf16": [vp, vp, i64, vp],
    "mft_cast_bf16_to_f32": [vp, vp, i64, vp],
    "mft_transpose_f32_to_bf16": [vp, vp, i64, i64, vp],
    "mft_transpose_bf16": [vp, vp, i64, i64, vp],
    "mft_transpose_bf16_ld": [vp, vp, i64, i64, i64, vp],
    "mft_embedding_gather": [vp, vp, vp, vp, i64, i64, i64, i64, f32, vp, vp],
    "mft_rmsnorm_fwd": [vp, i32, vp, f32, i32, vp, i32, vp, vp, vp, i64, i64, vp],
    "mft_rmsnorm_bwd": [vp, i32, vp, i32, vp, vp, f32, i32, vp, i32, i32, vp, i64, i64, vp],
    "mft_rmsnorm_add_norm_fwd": [vp, vp, i32, vp, vp, i32, f32, vp, vp, vp, vp, i64, i64, vp],
    "mft_rmsnorm_pair_bwd": [vp, vp, vp, i32, vp, vp, vp, vp, i32, vp, vp, i64, i64, vp],
    "mft_layernorm_fwd": [vp, i32, vp, vp, f32, vp, i32, vp, vp, i64, i64, vp],
    "mft_layernorm_bwd": [vp, i32, vp, i32, vp, vp, vp, vp, i32, i32, vp, vp, i64, i64, vp],
    "mft_act_fwd": [i32, vp, vp, i64, vp, i64, i64, vp],
    "mft_act_bwd": [i32, vp, vp, vp, i64, vp, vp, i64, i64, vp],
    "mft_add_f32": [vp, vp, vp, i64, vp],
    "mft_add_f32_bf16": [vp, vp, vp, i64, vp],
    "mft_scale_f32": [vp, f32, i64, vp],
    "mft_rope_table_host": [vp, vp, i64, i64, f32],
    "mft_headnorm_rope_fwd": [vp, i64, vp, f32, vp, vp, vp, i64, vp, i64, i64, i64, i64, vp],
    "mft_headnorm_rope_bwd": [vp, i64, vp, i64, vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, vp],
    "mft_repeat_kv": [vp, i32, vp, i64, i64, i64, i64, i64, vp],
    "mft_repeat_kv_bwd": [vp, vp, i64, i64, i64, i64, i64, vp],
    "mft_gemm_nt": [vp, i64, vp, i64, i64, i64, i64, vp, i64, vp, i64, i64, vp, f32, vp, i64, i32, i32, vp],
    "mft_gemm_nt_tile_cols": [i64, i64, i64, i64, i32, C.POINTER(i32)],
    "mft_glu_linear_fwd": [i32, vp, i64, vp, i64, i64, i64, i64, vp, i64, vp, i64, i64, vp, vp, i64, vp, i64, vp],
    "mft_glu_linear_bwd": [i32, vp, i64, vp, i64, i64, i64, i64, vp, i64, vp, i64, i64, vp, i64, vp, i64, vp],
    "mft_probe_tma_delivery": [i32, i32, i32, i32, C.POINTER(C.c_double), C.POINTER(C.c_double), vp],
    "mft_profile_gemm": [i32],
    "mft_profile_gemm_report": [C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(i64)],
    "mft_profile_gemm_report_epi": [i32, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(i64)],
    "mft_profile_gemm_launch": [i64, C.POINTER(i64), C.POINTER(i32), C.POINTER(i32), C.POINTER(C.c_double)],
    "mft_gemm_tn_acc": [vp, i64, vp, i64, i64, i64, i64, f32, vp, i64, vp],
    "mft_pack_blocks_bf16": [vp, i32, vp],
    "mft_accumulate_blocks_f32": [vp, i32, vp],
    "mft_attn_fwd": [vp, Strides, vp, Strides, vp, Strides, vp, Strides, vp, i64, i64, i64, i64, i64, f32, i64, vp],
    "mft_attn_bwd": [vp, Strides, vp, Strides, vp, Strides, vp, Strides, vp, Strides, vp, vp, vp, vp, vp, vp,
                     i64, i64, i64, i64, i64, f32, i64, vp],
    "mft_attn_bwd_noalloc": [vp, Strides, vp, Strides, vp, Strides, vp, Strides, vp, Strides, vp, vp, vp, vp,
                             i64, i64, i64, i64, i64, f32, i64, vp],
    "mft_lmhead_ce_workspace_bytes": [i64, i64, i64],
    "mft_lmhead_ce_set_panel_budget": [i64],
    "mft_lmhead_ce_fwd": [vp, vp, vp, i64, i64, i64, i64, i32, vp, vp, vp, vp, vp, i64, vp],
    "mft_lmhead_ce_bwd": [vp, vp, vp, i64, vp, i64, i64, i64, i64, i32, vp, vp, i64, f32, vp, vp, i64, vp],
    "mft_lmhead_ce_fused": [vp, vp, vp, i64, vp, i64, i64, i64, i64, i32, i64, f32, vp, vp, vp, vp, vp, vp, i64, vp],
    "mft_ce_dense_fwd": [vp, vp, i64, i64, i64, i32, vp, vp, vp, vp, vp, vp, vp],
    "mft_ce_dense_bwd": [vp, vp, i64, i64, i64, vp, vp, f32, vp, vp],
    "mft_grad_sqnorm": [vp, i64, vp, vp],
    "mft_ew_binary_f32": [i32, vp, vp, i32, vp, vp, i32, vp, vp, i32, vp],
    "mft_ew_scalar_f32": [i32, vp, f32, i32, vp, i64, vp],
    "mft_ew_unary_f32": [i32, vp, f32, vp, i64, vp],
    "mft_reduce_sum_f32": [vp, vp, i64, i64, i64, f32, vp],
    "mft_permute_b32": [vp, vp, vp, vp, i32, vp],
    "mft_matmul_f32": [vp, vp, vp, i64, i64, i64, i64, i64, i64, i64, i32, vp],
    "mft_softmax_f32": [vp, vp, i64, i64, vp],
    "mft_softmax_bwd_f32": [vp, vp, vp, i64, i64, vp],
    "mft_rope_f32": [vp, vp, vp, vp, i64, i64, i64, i32, vp],
    "mft_swiglu_f32": [vp, vp, vp, vp, vp, i64, vp],
    # ---- include/mft_step.h
    "mft_model_create": [C.POINTER(ModelConfig), vp, C.POINTER(vp)],
    "mft_model_destroy": [vp],
    "mft_model_param_count": [vp],
    "mft_model_param_shape": [vp, i32, C.POINTER(i64), C.POINTER(i64)],
    "mft_model_set_param_host": [vp, i32, vp],
    "mft_model_set_param_host_bf16": [vp, i32, vp, i32],
    "mft_model_set_param_dev": [vp, i32, vp],
    "mft_model_lora_count": [vp],
    "mft_model_lora_shape": [vp, i32, C.POINTER(i64), C.POINTER(i64)],
    "mft_model_set_lora_host": [vp, i32, vp],
    "mft_model_get_lora_host": [vp, i32, vp],
    "mft_model_get_lora_grad_host": [vp, i32, vp],
    "mft_model_lora_has_grad": [vp, i32],
    "mft_model_lora_offset": [vp, i32, C.POINTER(i64)],
    "mft_model_mark_lora_dirty": [vp],
    "mft_model_forward_logits": [vp, vp, i32, i32, vp],
    "mft_model_forward_hidden": [vp, vp, i32, i32, vp],
    "mft_model_buckets": [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(i64)],
    "mft_model_forward_backward": [vp, vp, vp, i32, i32, i64, C.POINTER(f32), C.POINTER(i32)],
    "mft_model_forward_backward_dev": [vp, vp, vp, i32, i32, i64, C.POINTER(vp), C.POINTER(vp)],
    "mft_model_forward_loss": [vp, vp, vp, i32, i32, C.POINTER(f32)],
    "mft_model_optimizer_step": [vp, f32, f32, f32, f32, f32, f32, f32],
    "mft_model_zero_grad": [vp],
    "mft_model_set_loss_scale": [vp, f32],
    "mft_safetensors_open": [C.c_char_p, vp],
    "mft_safetensors_close": [vp],
    "mft_safetensors_count": [vp],
    "mft_safetensors_name": [vp, i64],
    "mft_safetensors_metadata": [vp, C.c_char_p],
    "mft_safetensors_info": [vp, C.c_char_p, vp, vp, vp],
    "mft_safetensors_read_f32": [vp, C.c_char_p, vp, i32],
    "mft_safetensors_write_f32": [C.c_char_p, i32, vp, vp, vp, vp, i32, vp, vp],
    "mft_model_hf_key": [vp, i32, vp, i32, vp],
    "mft_model_load_safetensors": [vp, C.c_char_p],
    "mft_model_save_lora_safetensors": [vp, C.c_char_p],
    "mft_model_load_lora_safetensors": [vp, C.c_char_p],
    "mft_model_stage_batch": [vp, i32, vp, vp, i32, i32],
    "mft_model_stage_wait": [vp, i32],
    "mft_model_step_staged": [vp, i32, i32, i32, i64, vp, vp],
    "mft_model_sync": [vp],
    "mft_model_eval_ppl_batch": [vp, vp, vp, vp, i32, i32],
    "mft_ppl_result": [vp, vp, vp],
    "mft_model_score_tokens": [vp, vp, i32, vp, i32, vp],
    "mft_model_merge_lora": [vp],
    "mft_model_unmerge_lora": [vp],
    "mft_model_is_merged": [vp],
    "mft_trainer_lr": [vp, i64],
    "mft_trainer_create": [vp, vp, vp],
    "mft_trainer_destroy": [vp],
    "mft_trainer_train_step": [vp, vp, vp, i32, i32, i64, vp, vp, vp],
    "mft_trainer_global_step": [vp],
    "mft_model_get_final_hidden_host": [vp, vp, i64],
    "mft_model_activation_bytes": [vp],
    "mft_grad_sqnorm_add": [vp, i64, vp, vp],
    "mft_adam_step": [vp, vp, vp, vp, i64, i64, f32, f32, f32, f32, f32, vp, f32, f32, i32, vp],
}
_RET = {"mft_launch_count": i64, "mft_last_error": C.c_char_p, "mft_lmhead_ce_workspace_bytes": i64,
        "mft_lmhead_ce_set_panel_budget": i64,
        "mft_model_activation_bytes": i64, "mft_trainer_lr": f32, "mft_trainer_global_step": i64,
        "mft_safetensors_count": i64, "mft_safetensors_name": C.c_char_p, "mft_safetensors_metadata": C.c_char_p}
_NO_STATUS = {"mft_version", "mft_lmhead_ce_workspace_bytes", "mft_lmhead_ce_set_panel_budget", "mft_model_param_count", "mft_model_lora_count",
              "mft_model_lora_has_grad", "mft_trainer_lr", "mft_trainer_global_step",
              "mft_safetensors_count", "mft_safetensors_name", "mft_safetensors_metadata"}


def exported_names() -> list[str]:
    return sorted(set(_SIGS) | {"mft_launch_count", "mft_launch_count_reset", "mft_last_error"})


def load() -> C.CDLL:
    """Load the shared object (building nothing: see mobilefinetuner_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise MftError(f"{_LIB_PATH} is missing: run `python -m mobilefinetuner_b200.build` (there is no CPU fallback)")
    lib = C.CDLL(str(_LIB_PATH))
    for name, args in _SIGS.items():
        fn = getattr(lib, name, None)
        if fn is None:   # reported by missing_symbols(); calling it raises
            continue
        fn.argtypes = args
        fn.restype = _RET.get(name, i32)
    lib.mft_launch_count.argtypes = []
    lib.mft_launch_count.restype = i64
    lib.mft_launch_count_reset.argtypes = []
    lib.mft_launch_count_reset.restype = None
    lib.mft_last_error.argtypes = []
    lib.mft_last_error.restype = C.c_char_p
    _lib = lib
    return lib


def missing_symbols() -> list[str]:
    lib = load()
    return [n for n in exported_names() if getattr(lib, n, None) is None]


def call(name: str, *args):
    """Call an entry point and raise MftError on a non-zero status."""
    lib = load()
    fn = getattr(lib, name)
    rc = fn(*args)
    if name in _NO_STATUS or name in _RET:
        return rc
    if rc != 0:
        raise MftError(f"{name} failed with status {rc}: {lib.mft_last_error().decode(errors='replace')}")
    return rc


_initialised = set()


def init(device: int = 0) -> None:
    if device not in _initialised:
        call("mft_init", device)
        _initialised.add(device)
