/*
 * mft_cuda.h - C ABI of libmft_cuda.so, the sm_100a kernel library behind the
 * LoRA fine-tuning step (forward + backward + Adam) of MobileFineTuner's
 * operator API.
 *
 * The reference has no FFI for this path: its boundary is the C++ source API of
 * the `operators` target (operator/finetune_ops/core/ops.h, lm_loss.h,
 * nn/lora_linear.h, optim/adam.h).  Each entry point below names the reference
 * function whose arithmetic it replaces; a C++ host layer (or any FFI: ctypes,
 * cgo, JNI) binds these symbols.
 *
 * Conventions
 *  - every function returns an int32 status: 0 = ok, negative = MFT_ERR_*;
 *    mft_last_error() gives the message of the calling thread's last failure;
 *  - all tensor pointers are DEVICE pointers unless the name ends in `_host`;
 *  - tensors are contiguous row-major; `bf16` buffers hold raw IEEE bfloat16;
 *  - every launch is asynchronous on the given stream (a cudaStream_t passed as
 *    void*; NULL = the default stream); nothing synchronises except
 *    mft_stream_sync and the *_host copies;
 *  - there is no CPU fallback: without a CUDA device every call fails.
 */
#ifndef MFT_CUDA_H
#define MFT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MFT_OK 0
#define MFT_ERR_INVALID_ARG (-1)
#define MFT_ERR_OOM (-2)
#define MFT_ERR_CUDA (-3)
#define MFT_ERR_NCCL (-4)
#define MFT_ERR_TIMEOUT (-5)
#define MFT_ERR_BOUNDS (-6)
#define MFT_ERR_UNSUPPORTED (-7)

typedef void* mft_stream_t;

/* ---- runtime ------------------------------------------------------------ */
/* Selects the device for the calling thread, creates library state (the
 * TMA-descriptor encoder, the device status word).  Idempotent. */
int32_t mft_init(int32_t device);
int32_t mft_shutdown(void);
const char* mft_last_error(void);
int32_t mft_version(void);
/* Number of kernels this library has launched since the last reset. */
int64_t mft_launch_count(void);
void mft_launch_count_reset(void);
int32_t mft_stream_sync(mft_stream_t stream);
/* Reads and clears the device status word that kernels with bounded waits set
 * when a wait ran out (0 = no error).  Synchronises the stream. */
int32_t mft_device_status(mft_stream_t stream, int32_t* status_host);

/* ---- memory: the device analogue of MemoryManager / MemoryPool
 *      (operator/finetune_ops/core/memory_manager.h:103-153; allocate
 *      memory_manager.cpp:34-73, deallocate :75-97, clear_unused :99-145) ---
 * Size-bucketed, stream-ordered caching allocator: freed blocks are kept for
 * reuse and only returned to the driver by mft_empty_cache (what force_cleanup
 * maps to).  mft_free(ptr, stream) states that every use of the block has been
 * queued on `stream`; the block may be handed out again at once, and a request
 * from ANOTHER stream is ordered after those uses on the device (an event
 * wait), never by blocking the host.  A block used on several streams must be
 * made visible to the stream it is freed on first (event wait or sync). */
int32_t mft_malloc(size_t bytes, mft_stream_t stream, void** ptr);
int32_t mft_free(void* ptr, mft_stream_t stream);
int32_t mft_empty_cache(void);
/* Returns cached blocks to the driver, largest first, until at most keep_bytes
 * stay cached: the per-step MemoryManager::force_cleanup() / clear_unused_memory()
 * of the reference's training loops (trainer.cpp:143, gemma_trainer.cpp:137) maps
 * to this with a high-water mark, so a steady-state step allocates nothing. */
int32_t mft_trim_cache(int64_t keep_bytes);
/* stats_host[0..5] = bytes in use, bytes cached, peak bytes in use, #cudaMalloc
 * calls, #requests served from the cache, #of those that had to be ordered
 * behind another stream. */
int32_t mft_mem_stats(int64_t* stats_host);
int32_t mft_memcpy_h2d(void* dst, const void* src_host, size_t bytes, mft_stream_t stream);
/* Page-locked host memory (asynchronous copies need it to overlap with kernels). */
int32_t mft_host_alloc(size_t bytes, void** out_host);
int32_t mft_host_free(void* host);
int32_t mft_memcpy_d2h(void* dst_host, const void* src, size_t bytes, mft_stream_t stream);
int32_t mft_memcpy_d2d(void* dst, const void* src, size_t bytes, mft_stream_t stream);
int32_t mft_memset(void* dst, int32_t byte_value, size_t bytes, mft_stream_t stream);

/* ---- casts (ops::cast, operator/finetune_ops/core/ops.cpp:2894-2952;
 *      bf16 conversion is round-to-nearest-even as core/dtype.h:114-121) ---- */
int32_t mft_cast_f32_to_bf16(const float* src, void* dst_bf16, int64_t n, mft_stream_t stream);
int32_t mft_cast_bf16_to_f32(const void* src_bf16, float* dst, int64_t n, mft_stream_t stream);
/* dst[c, r] = src[r, c] with conversion f32 -> bf16 (weight packing: the
 * reference stores linears as [in, out]; the GEMMs here want K-major [out, in]). */
int32_t mft_transpose_f32_to_bf16(const float* src, void* dst_bf16, int64_t rows, int64_t cols,
                                  mft_stream_t stream);
int32_t mft_transpose_bf16(const void* src_bf16, void* dst_bf16, int64_t rows, int64_t cols,
                           mft_stream_t stream);
/* Same with a padded destination: dst[c * dst_ld + r] = src[r, c], dst_ld >= rows. */
int32_t mft_transpose_bf16_ld(const void* src_bf16, void* dst_bf16, int64_t rows, int64_t cols,
                              int64_t dst_ld, mft_stream_t stream);

/* ---- embedding gather
 *      (GPT2Model::embedding_lookup gpt2_model.cpp:464-492 + positions :349-369,
 *       QwenModel::embedding_lookup qwen_model.cpp:249-272,
 *       GemmaModel::embedding_lookup gemma_model.cpp:222-259) ---------------
 * out[t, :] = table[ids[t], :] * scale (+ pos_table[t % seq_len, :]).
 * table is bf16 [vocab, hidden]; pos_table (may be NULL) bf16 [n_pos, hidden];
 * out is f32 [n_tokens, hidden].  An id outside [0, vocab) sets status
 * MFT_ERR_BOUNDS in *status_dev (device int32, may be NULL) and writes zeros. */
int32_t mft_embedding_gather(const int32_t* ids, const void* table_bf16, const void* pos_table_bf16,
                             float* out, int64_t n_tokens, int64_t seq_len, int64_t hidden,
                             int64_t vocab, float scale, int32_t* status_dev, mft_stream_t stream);

/* ---- normalisation
 *      rms_norm (1+w)   ops.cpp:1677-1725, RMSNormBackward backward_functions.cpp:492-532
 *      rms_norm_affine  ops.cpp:1728-1762, RMSNormAffineBackward        :534-570
 *      layer_norm       ops.cpp:1592-1646, LayerNormBackward            :434-490 --------
 * x is [rows, dim] in x_dtype (MFT_F32 or MFT_BF16); y in y_dtype; weights f32.
 * rstd (f32 [rows], may be NULL) receives 1/sqrt(mean(x^2)+eps) for the backward.
 * unit_offset = 1 multiplies by (1 + w) (Gemma), 0 by w (Qwen).
 * If residual != NULL (f32 [rows, dim]) the forward also writes
 * sum_out = residual + y (f32), the fused "norm then residual add". */
#define MFT_F32 0
#define MFT_BF16 1
#define MFT_I32 2
int32_t mft_rmsnorm_fwd(const void* x, int32_t x_dtype, const float* weight, float eps,
                        int32_t unit_offset, void* y, int32_t y_dtype, float* rstd,
                        const float* residual, float* sum_out,
                        int64_t rows, int64_t dim, mft_stream_t stream);
/* dx = rms-norm backward of dy; dx_dtype f32 or bf16.  If accumulate != 0
 * (f32 dx only) the result is added to dx.  dweight (f32 [dim], may be NULL)
 * is accumulated with atomics (only needed for trainable norms). */
int32_t mft_rmsnorm_bwd(const void* dy, int32_t dy_dtype, const void* x, int32_t x_dtype,
                        const float* weight, const float* rstd, float eps, int32_t unit_offset,
                        void* dx, int32_t dx_dtype, int32_t accumulate, float* dweight,
                        int64_t rows, int64_t dim, mft_stream_t stream);
/* Gemma's block wrapper in one pass per row (rows up to 2048 wide; MFT_ERR_UNSUPPORTED beyond):
 *   forward : sum_out = residual + rms_norm(y; w_post) ,  h_next = rms_norm(sum_out; w_next)
 *             (post-norm of one block + residual add + pre-norm of the next, gemma_model.cpp:615-640), the row
 *             stays in registers between the two norms; both rstd vectors are stored for the backward.
 *   backward: dx_inout += d rms_norm(x_sum; w_next)(dy_next)   then   d_branch = d rms_norm(y_branch; w_post)(dx_inout)
 * Results are bit-identical to the two separate mft_rmsnorm_* calls. */
int32_t mft_rmsnorm_add_norm_fwd(const void* y_bf16, const float* w_post, int32_t unit_post, const float* residual,
                                 const float* w_next, int32_t unit_next, float eps, float* sum_out, float* rstd_post,
                                 void* h_next_bf16, float* rstd_next, int64_t rows, int64_t dim, mft_stream_t stream);
int32_t mft_rmsnorm_pair_bwd(const void* dy_next_bf16, const float* x_sum, const float* w_next, int32_t unit_next,
                             const float* rstd_next, float* dx_inout, const void* y_branch_bf16, const float* w_post,
                             int32_t unit_post, const float* rstd_post, void* d_branch_bf16, int64_t rows, int64_t dim,
                             mft_stream_t stream);
int32_t mft_layernorm_fwd(const void* x, int32_t x_dtype, const float* weight, const float* bias,
                          float eps, void* y, int32_t y_dtype, float* mean, float* rstd,
                          int64_t rows, int64_t dim, mft_stream_t stream);
int32_t mft_layernorm_bwd(const void* dy, int32_t dy_dtype, const void* x, int32_t x_dtype,
                          const float* weight, const float* mean, const float* rstd,
                          void* dx, int32_t dx_dtype, int32_t accumulate,
                          float* dweight, float* dbias,
                          int64_t rows, int64_t dim, mft_stream_t stream);

/* ---- activations and residuals
 *      gelu ops.cpp:1243-1267 / GeluBackward backward_functions.cpp:164-186
 *      swiglu ops.cpp:2416-2452 / SwiGLUBackward :277-295
 *      Gemma GeGLU = mul(gelu(gate), up), gemma_model.cpp:538-546
 *      add ops.cpp:415-442 ------------------------------------------------ */
#define MFT_ACT_GELU 0    /* y = gelu_tanh(x)               (x = gate, up unused)   */
#define MFT_ACT_SWIGLU 1  /* y = silu(gate) * up                                      */
#define MFT_ACT_GEGLU 2   /* y = gelu_tanh(gate) * up                                 */
/* gate/up are bf16 [rows, ld] slices: element (r, c) at base[r*ld + c], c < cols.
 * y is bf16 [rows, cols] contiguous. */
int32_t mft_act_fwd(int32_t kind, const void* gate_bf16, const void* up_bf16, int64_t ld,
                    void* y_bf16, int64_t rows, int64_t cols, mft_stream_t stream);
int32_t mft_act_bwd(int32_t kind, const void* dy_bf16, const void* gate_bf16, const void* up_bf16,
                    int64_t ld, void* dgate_bf16, void* dup_bf16, int64_t rows, int64_t cols,
                    mft_stream_t stream);
/* out = a + b (f32, n elements); a may alias out. */
int32_t mft_add_f32(const float* a, const float* b, float* out, int64_t n, mft_stream_t stream);
/* out(f32) = a(f32) + b(bf16) */
int32_t mft_add_f32_bf16(const float* a, const void* b_bf16, float* out, int64_t n, mft_stream_t stream);
int32_t mft_scale_f32(float* x, float alpha, int64_t n, mft_stream_t stream);

/* ---- RoPE (apply_rope ops.cpp:2337-2414, ApplyRoPEBackward
 *      backward_functions.cpp:728-774) and Gemma's per-head QK RMSNorm ------
 * mft_rope_table fills cos/sin f32 [seq_len, head_dim/2] on the HOST with the
 * reference's own expression (freq = 1/powf(theta, 2d/hd); angle = pos*freq in
 * fp32; std::cos/std::sin of float), so device angles are bit-identical. */
int32_t mft_rope_table_host(float* cos_host, float* sin_host, int64_t seq_len, int64_t head_dim, float theta);
/* x: bf16 rows of `n_heads` heads of `head_dim`, token-major: element
 * (token, head, d) at x[token*ld + head*head_dim + d]; token position =
 * token % seq_len.  norm_weight (f32 [head_dim], may be NULL) applies
 * rms_norm(1+w) per head BEFORE the rotation (Gemma, gemma_model.cpp:459-482);
 * rstd (f32 [n_tokens*n_heads]) is then written for the backward.
 * cos/sin may be NULL to skip the rotation. */
int32_t mft_headnorm_rope_fwd(const void* x_bf16, int64_t ld, const float* norm_weight, float eps,
                              const float* cos_tab, const float* sin_tab,
                              void* y_bf16, int64_t ld_y, float* rstd,
                              int64_t n_tokens, int64_t seq_len, int64_t n_heads, int64_t head_dim,
                              mft_stream_t stream);
int32_t mft_headnorm_rope_bwd(const void* dy_bf16, int64_t ld_dy, const void* x_bf16, int64_t ld,
                              const float* norm_weight, const float* rstd,
                              const float* cos_tab, const float* sin_tab,
                              void* dx_bf16, int64_t ld_dx,
                              int64_t n_tokens, int64_t seq_len, int64_t n_heads, int64_t head_dim,
                              mft_stream_t stream);

/* ---- repeat_kv_heads (ops.cpp:2260-2335, RepeatKVHeadsBackward
 *      backward_functions.cpp:693-726): standalone gather, [B,nkv,S,hd] ->
 *      [B,nkv*rep,S,hd]; the attention kernels never call it (h -> h/rep). -- */
int32_t mft_repeat_kv(const void* kv, int32_t dtype, void* out, int64_t batch, int64_t n_kv,
                      int64_t seq, int64_t head_dim, int64_t repeat, mft_stream_t stream);
int32_t mft_repeat_kv_bwd(const float* dout, float* dkv, int64_t batch, int64_t n_kv,
                          int64_t seq, int64_t head_dim, int64_t repeat, mft_stream_t stream);

/* ---- GEMM (ops::matmul ops.cpp:619-822, ops::matmul_rhs_T :824-988,
 *      MatmulBackward backward_functions.cpp:94-147, and the LoRA branch of
 *      LoRALinear::forward nn/lora_linear.cpp:336-468) ----------------------
 * "NT" product on the tcgen05 tensor cores, bf16 operands, fp32 accumulation
 * in tensor memory:
 *     D[m,n] = alpha * ( sum_k A[m,k]*B[n,k] + sum_j A2[m,j]*B2[n,j] ) + bias[n] (+ D[m,n])
 * A [M,K] and B [N,K] are bf16 with the contraction index contiguous (row
 * strides lda/ldb in elements, multiples of 8; base pointers 16-byte aligned).
 * The optional second segment (A2 [M,K2], B2 [N,K2], K2 <= 64) is how the
 * rank-r LoRA update rides in the same accumulator: A2 = scale*(X*A),
 * B2 = B^T, so Y = X*W + scale*(X*A)*B costs one extra 64-wide k-block.
 * bias is f32 [N] or NULL.  D is bf16 or f32 (d_dtype), row stride ldd.
 * accumulate != 0 adds the previous contents of D (f32 D only). */
int32_t mft_gemm_nt(const void* a_bf16, int64_t lda, const void* b_bf16, int64_t ldb,
                    int64_t m, int64_t n, int64_t k,
                    const void* a2_bf16, int64_t lda2, const void* b2_bf16, int64_t ldb2, int64_t k2,
                    const float* bias, float alpha,
                    void* d, int64_t ldd, int32_t d_dtype, int32_t accumulate,
                    mft_stream_t stream);
/* Tile plan of mft_gemm_nt for a plain call (no accumulate) of this shape: *tile_cols_host = columns of the CTA-pair
 * kernel's tile - 256, or 384 when the width is a multiple of 384, m a multiple of 256 and the cost model (waves of
 * tiles x k-blocks per tile) prefers the wider tile; f32 outputs take it only under at least 64 k-blocks per tile - or
 * 0 when another kernel takes the call.  Needs an initialised device (the SM count enters the plan). */
int32_t mft_gemm_nt_tile_cols(int64_t m, int64_t n, int64_t k, int64_t k2, int32_t d_dtype, int32_t* tile_cols_host);
/* Measurement aid: bytes per clock that one SM takes in from L2 through its TMA unit when nothing else uses its shared
 * memory (one CTA per SM loads an L2-resident 64 MiB matrix into a ring of `stages` 32 KB stages that a second thread
 * releases at once).  mode 0: two tensor boxes of 128 rows x 128 bytes per stage (what the GEMMs load); 1: two bulk
 * copies of 16 KB; 2: one of each.  Results: bytes per clock of the slowest CTA, and TB/s over all `ctas`.  Allocates
 * its own scratch and synchronises; not for use inside a step. */
int32_t mft_probe_tma_delivery(int32_t mode, int32_t stages, int32_t ctas, int32_t iters, double* bytes_per_clock_per_sm_host,
                               double* tb_per_s_host, mft_stream_t stream);
/* Measurement aid: while enabled, every tensor-core GEMM launch (mft_gemm_nt and the GEMMs inside
 * the lm-head routines) is bracketed by CUDA events on its stream.  The report sums the
 * executed MACs*2 (including the LoRA k-block) and the device time over the launches recorded
 * since the last call of mft_profile_gemm. */
int32_t mft_profile_gemm(int32_t enable);
int32_t mft_profile_gemm_report(double* flops_host, double* ms_host, int64_t* launches_host);
/* The same sums over the launches whose epilogue is selected by bit e of `epilogue_mask`: 0 plain store, 1..3 the
 * lm-head cross-entropy epilogues (row statistics, gradient, probabilities), 4 / 5 the gated-MLP forward / backward
 * epilogues.  A fused launch's time contains its epilogue's element-wise work, its flops only the product. */
int32_t mft_profile_gemm_report_epi(int32_t epilogue_mask, double* flops_host, double* ms_host, int64_t* launches_host);
/* One recorded launch, 0 <= index < launches of mft_profile_gemm_report: its shape (m, n, k, k of the LoRA block),
 * epilogue, output type and device time. */
int32_t mft_profile_gemm_launch(int64_t index, int64_t* shape_mnk_k2_host, int32_t* epilogue_host, int32_t* d_is_f32_host, double* ms_host);

/* "TN" product with the long dimension contracted (the LoRA weight gradients
 * dA = s*X^T*(dY*B^T), dB = s*(X*A)^T*dY of the generic MatmulBackward):
 *     out[p,q] (+)= alpha * sum_t U[t,p]*V[t,q]
 * U [T,P], V [T,Q] bf16 row-major (ldu, ldv); out f32 [P,Q] with row stride
 * ldo.  Split over T across CTAs with fp32 atomics, so `out` must hold the
 * value to accumulate onto (zero for a fresh result). */
int32_t mft_gemm_tn_acc(const void* u_bf16, int64_t ldu, const void* v_bf16, int64_t ldv,
                        int64_t t, int64_t p, int64_t q, float alpha,
                        float* out, int64_t ldo, mft_stream_t stream);

/* Table-driven block copies between the fp32 LoRA tensors (reference layouts:
 * GPT-2/Qwen A[in,r], B[r,out]; Gemma A[r,in], B[out,r]) and the bf16 / f32
 * operand panels the GEMMs use.  One launch handles every entry. */
typedef struct {
    const void* src;   /* f32 (pack) */
    void* dst;         /* bf16 (pack) or f32 (unpack-accumulate) */
    int32_t rows;      /* rows of the source block */
    int32_t cols;      /* cols of the source block */
    int32_t src_ld;
    int32_t dst_ld;
    int32_t transpose; /* 1: dst[c, r] = src[r, c] */
    int32_t pad;
} mft_block_copy_t;
/* dst(bf16) = src(f32) for every table entry (table lives in device memory). */
int32_t mft_pack_blocks_bf16(const mft_block_copy_t* table_dev, int32_t n_entries, mft_stream_t stream);
/* dst(f32) += src(f32) for every table entry. */
int32_t mft_accumulate_blocks_f32(const mft_block_copy_t* table_dev, int32_t n_entries, mft_stream_t stream);

/* ---- gated MLP with the gating fused into the GEMM epilogues
 *      (GemmaModel::apply_mlp gemma_model.cpp:538-546: down(mul(gelu(gate(x)), up(x)));
 *       QwenModel::mlp qwen_model.cpp:320-332: down(swiglu(gate(x), up(x)));
 *       backward: MulBackward backward_functions.cpp:74-83, GeluBackward :164-186, SwiGLUBackward :277-295) ----
 * kind = MFT_ACT_GEGLU or MFT_ACT_SWIGLU.  w_nk is the K-major gate|up weight [2*inter, k] (gate rows first), b_nk the
 * matching LoRA panel [2*inter, 64], xa = scale * x A [m, 64] (k2 used columns; k2 = 0: no LoRA).
 *   forward : gu[m, 2*inter] = x W (+ bias) + xa B   (kept for the backward pass)  and  act[m, inter] = f(gate) * up
 *             in ONE launch: a CTA pair owns 128 gate columns and the 128 matching up columns of a tile.
 *   backward: d_act = dy W_down^T + a2 b2^T is formed tile by tile in tensor memory and never stored; the epilogue loads
 *             the saved gate|up tile and writes dgu[m, 2*inter] = (d_gate | d_up) directly.  w_kn = K-major [inter, k].
 * Both return MFT_ERR_UNSUPPORTED (without an error message) when the shape does not qualify (m < 256, inter not a
 * multiple of 128 / 64, unaligned operands): the caller then runs mft_gemm_nt followed by mft_act_fwd / mft_act_bwd,
 * whose results these calls reproduce bit for bit. */
int32_t mft_glu_linear_fwd(int32_t kind, const void* x_bf16, int64_t ldx, const void* w_nk_bf16, int64_t ldw, int64_t m,
                           int64_t inter, int64_t k, const void* xa_bf16, int64_t ldxa, const void* b_nk_bf16, int64_t ldb2,
                           int64_t k2, const float* bias, void* gu_bf16, int64_t ld_gu, void* act_bf16, int64_t ld_act,
                           mft_stream_t stream);
int32_t mft_glu_linear_bwd(int32_t kind, const void* dy_bf16, int64_t lddy, const void* w_kn_bf16, int64_t ldw, int64_t m,
                           int64_t inter, int64_t k, const void* a2_bf16, int64_t lda2, const void* b2_bf16, int64_t ldb2,
                           int64_t k2, const void* gu_bf16, int64_t ld_gu, void* dgu_bf16, int64_t ld_dgu,
                           mft_stream_t stream);

/* ---- attention: the chain repeat_kv_heads -> transpose -> matmul ->
 *      mul(scale) -> add(mask) -> softmax -> matmul of the model graphs
 *      (qwen_model.cpp:311-318, gemma_model.cpp:487-505, gpt2_model.cpp:630-657;
 *      softmax ops.cpp:1307-1363, SoftmaxBackward backward_functions.cpp:306-349;
 *      masks ops.cpp:2167-2180 and gemma_model.cpp:272-285) -----------------
 * Fused causal / sliding-window GQA attention.  Element (b, s, h, d) of a
 * tensor lives at base[b*stride_b + s*stride_s + h*stride_h + d] (bf16).
 * Query head h reads KV head h / (n_heads / n_kv_heads): repeat_kv is an index
 * remap, never a copy.  Key j is visible to query i iff j <= i and
 * (window <= 0 or i - j < window).  lse is f32 [batch, n_heads, seq].
 * head_dim 64 / 128 / 256 with seq a multiple of 128 and token-major tensors
 * (stride_b == seq * stride_s) runs on tensor-memory (tcgen05) kernels
 * (head_dim 64 / 128 only from seq 512 forward / 256 backward on, where they
 * are the faster ones); other shapes of those head sizes on mma.sync kernels,
 * any other even head_dim <= 256 on generic kernels, all with the same results
 * to bf16 rounding.  MFT_ATTN_TC=0 in the environment selects the mma.sync
 * kernels everywhere, MFT_ATTN_TC=2 the tensor-memory kernels at every shape
 * they take. */
typedef struct {
    int64_t stride_b, stride_s, stride_h;
} mft_strides_t;
int32_t mft_attn_fwd(const void* q, mft_strides_t sq, const void* k, mft_strides_t sk,
                     const void* v, mft_strides_t sv, void* o, mft_strides_t so, float* lse,
                     int64_t batch, int64_t seq, int64_t n_heads, int64_t n_kv_heads, int64_t head_dim,
                     float scale, int64_t window, mft_stream_t stream);
/* dq/dk/dv are bf16 with the strides of q/k/v; dk/dv are per KV head (the sum
 * over the query heads of a group, RepeatKVHeadsBackward).  `delta` is an f32
 * [batch, n_heads, seq] scratch buffer supplied by the caller (the call fills
 * it with rowsum(O * dO)); dk/dv accumulate in f32 scratch `dkv_acc` of
 * 2*batch*seq*n_kv_heads*head_dim floats supplied by the caller.  `dkv_acc`
 * may be NULL: dk/dv are then produced by one CTA per KV head without scratch
 * (slower for grouped KV heads, and the tensor-memory dK/dV kernel needs it). */
int32_t mft_attn_bwd(const void* q, mft_strides_t sq, const void* k, mft_strides_t sk,
                     const void* v, mft_strides_t sv, const void* o, mft_strides_t so,
                     const void* d_o, mft_strides_t sdo, const float* lse,
                     void* dq, void* dk, void* dv, float* delta, float* dkv_acc,
                     int64_t batch, int64_t seq, int64_t n_heads, int64_t n_kv_heads, int64_t head_dim,
                     float scale, int64_t window, mft_stream_t stream);

/* Allocation-free variant of mft_attn_bwd.  It has no counterpart in the reference.
 * Some hosts of this library may not create device memory at the point where they run a
 * backward pass: code executing inside a memory-budgeted or real-time section, a plugin whose
 * embedding application owns every allocation, or a caller that simply holds no allocator
 * handle.  For them the `delta` scratch of mft_attn_bwd ([batch, n_heads, seq] floats) lives in
 * a fixed 4 MiB array compiled into the library (one copy on every GPU that loads it, kept until
 * the process exits) and `dkv_acc` is not needed.  Inputs and outputs are still the caller's.
 *  - limit: batch * n_heads * seq <= 1,048,576; larger problems are rejected with
 *    MFT_ERR_INVALID_ARG and a message naming mft_attn_bwd as the alternative;
 *  - the first call on each device looks up the array's device address (no allocation); make
 *    that first call outside any stream capture;
 *  - all calls on a device share the one array: calls that may overlap on the GPU (different
 *    streams, or the same stream from two threads) race on it and must be serialised by the
 *    caller.  The array keeps the previous call's contents between calls; each call overwrites
 *    the rows it uses before reading them, so no clearing is required;
 *  - it calls no cudaMalloc / cudaFree and no allocating library routine. */
int32_t mft_attn_bwd_noalloc(const void* q, mft_strides_t sq, const void* k, mft_strides_t sk,
                             const void* v, mft_strides_t sv, const void* o, mft_strides_t so,
                             const void* d_o, mft_strides_t sdo, const float* lse,
                             void* dq, void* dk, void* dv,
                             int64_t batch, int64_t seq, int64_t n_heads, int64_t n_kv_heads, int64_t head_dim,
                             float scale, int64_t window, mft_stream_t stream);

/* ---- lm head + shifted cross-entropy (lm_cross_entropy core/lm_loss.cpp:268-382,
 *      LMCrossEntropyBackward :75-163, streaming variant :384-481 / :165-266) -
 * hidden bf16 [batch*seq, H]; table bf16 [V, H] (tied embedding); labels int32
 * [batch, seq] UNSHIFTED: row (b, s < seq-1) is scored against labels[b, s+1],
 * labels equal to ignore_index are skipped, the mean runs over the valid rows.
 * The [T, V] logits never reach memory: the vocabulary is processed in panels.
 * Forward writes loss_dev[0] (f32 mean NLL; NaN when nothing is valid),
 * n_valid_dev[0] (int32) and lse (f32 [batch*seq]).  A label >= V or < 0 (other
 * than ignore_index) sets *status_dev = MFT_ERR_BOUNDS.
 * Backward writes dhidden (bf16 [T,H]) = dloss * d(mean NLL)/d(hidden), with the
 * 1/n_valid coefficient read from n_valid_dev, or 1/n_valid_override if > 0
 * (data-parallel runs pass the global count).  table_t is the transposed table,
 * bf16 [H, table_t_ld] with table_t_ld >= V a multiple of 8 (built once at load).
 * workspace: mft_lmhead_ce_workspace_bytes() bytes of device scratch. */
int64_t mft_lmhead_ce_workspace_bytes(int64_t n_tokens, int64_t hidden, int64_t vocab);
/* The panel width is the largest multiple of 8192 columns whose bf16 [n_tokens, panel]
 * buffer fits a byte budget (default 12 GiB; the whole vocabulary when it fits).  Sets
 * the budget (bytes > 0) and returns the previous one; changes workspace_bytes, so call
 * it before sizing the workspace. */
int64_t mft_lmhead_ce_set_panel_budget(int64_t bytes);
int32_t mft_lmhead_ce_fwd(const void* hidden_bf16, const void* table_bf16, const int32_t* labels,
                          int64_t batch, int64_t seq, int64_t hidden, int64_t vocab, int32_t ignore_index,
                          float* loss_dev, int32_t* n_valid_dev, float* lse, int32_t* status_dev,
                          void* workspace, int64_t workspace_bytes, mft_stream_t stream);
int32_t mft_lmhead_ce_bwd(const void* hidden_bf16, const void* table_bf16, const void* table_t_bf16,
                          int64_t table_t_ld, const int32_t* labels, int64_t batch, int64_t seq, int64_t hidden, int64_t vocab,
                          int32_t ignore_index, const float* lse, const int32_t* n_valid_dev,
                          int64_t n_valid_override, float dloss, void* dhidden_bf16,
                          void* workspace, int64_t workspace_bytes, mft_stream_t stream);
/* Forward AND backward in one sweep over the vocabulary, for a training step
 * (the reference runs lm_cross_entropy and, from loss->backward(),
 * LMCrossEntropyBackward; both recompute or re-read the logits): the logits
 * are formed once, as un-normalised softmax numerators relative to a per-row
 * reference value, and folded straight into dHidden; the normalisation is
 * applied at the end.  Outputs are those of mft_lmhead_ce_fwd (loss_dev,
 * n_valid_dev, lse) plus dhidden of mft_lmhead_ce_bwd, with the same meaning
 * of n_valid_override and dloss.  Rows whose logits leave the range the sweep
 * can represent are detected and recomputed exactly, so results do not depend
 * on the logits' magnitude.  hidden must be a multiple of 8. */
int32_t mft_lmhead_ce_fused(const void* hidden_bf16, const void* table_bf16, const void* table_t_bf16,
                            int64_t table_t_ld, const int32_t* labels, int64_t batch, int64_t seq, int64_t hidden,
                            int64_t vocab, int32_t ignore_index, int64_t n_valid_override, float dloss,
                            float* loss_dev, int32_t* n_valid_dev, float* lse, void* dhidden_bf16,
                            int32_t* status_dev, void* workspace, int64_t workspace_bytes, mft_stream_t stream);
/* Dense-logits variants (API completeness: lm_cross_entropy on a materialised
 * [batch, seq, V] f32 tensor).  tgt_scratch is int32 [batch*seq] and
 * loss_scratch one double, both device scratch; the forward fills tgt_scratch
 * with the shifted labels, which the backward then reads. */
int32_t mft_ce_dense_fwd(const float* logits, const int32_t* labels, int64_t batch, int64_t seq, int64_t vocab,
                         int32_t ignore_index, float* loss_dev, int32_t* n_valid_dev, float* lse,
                         int32_t* tgt_scratch, double* loss_scratch, int32_t* status_dev, mft_stream_t stream);
int32_t mft_ce_dense_bwd(const float* logits, const int32_t* tgt_scratch, int64_t batch, int64_t seq, int64_t vocab,
                         const float* lse, const int32_t* n_valid_dev, float dloss, float* dlogits,
                         mft_stream_t stream);

/* ---- optimizer (Adam::step optim/adam.cpp:25-90, Optimizer::clip_grad_norm
 *      optim/optimizer.cpp:6-38, Tensor::zero_grad core/tensor.cpp:602-607) ---
 * All LoRA parameters live in one flat f32 bucket (params / grads / m / v of n
 * elements).  mft_grad_sqnorm writes sum(g^2) to sqnorm_dev[0].
 * mft_adam_step applies, per element (the reference's L2-style rule):
 *     g = clip * grads[i] + wd * p;  m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g
 *     p -= lr * (m / (1 - b1^step)) / (sqrt(v / (1 - b2^step)) + eps)
 * where clip = 1 if max_norm <= 0 or norm <= max_norm, else
 * max_norm / (norm + clip_eps) with norm = sqrt(sqnorm_dev[0]) (clip_eps = 0
 * for Optimizer::clip_grad_norm, 1e-6 for the trainers' variant).
 * zero_grad != 0 clears grads in the same pass. */
int32_t mft_grad_sqnorm(const float* grads, int64_t n, float* sqnorm_dev, mft_stream_t stream);
/* Same without clearing sqnorm_dev first: sums over several tensors with one read-back at the end. */
int32_t mft_grad_sqnorm_add(const float* grads, int64_t n, float* sqnorm_dev, mft_stream_t stream);
int32_t mft_adam_step(float* params, float* grads, float* m, float* v, int64_t n, int64_t step,
                      float lr, float beta1, float beta2, float eps, float weight_decay,
                      const float* sqnorm_dev, float max_norm, float clip_eps, int32_t zero_grad,
                      mft_stream_t stream);

/* ---- data-parallel exchange -------------------------------------------------
 * The reference is a single-device library (no collective call sites); the
 * sharded job built on it runs one process per GPU, each with a full replica
 * and its own slice of the batch, and exchanges exactly one thing per step:
 * the sum of the flat f32 LoRA-gradient bucket (what Optimizer::clip_grad_norm
 * optim/optimizer.cpp:6-38 and Adam::step optim/adam.cpp:25-90 then consume on
 * every rank).  These entry points are that exchange over NCCL, one
 * communicator per process.  NCCL is opened at run time (libnccl.so.2, or the
 * path in MFT_NCCL_LIB), so hosts that stay on one GPU need no NCCL at all.
 *
 * Rendezvous is the host's job: rank 0 calls mft_comm_unique_id and sends the
 * 128 bytes to the other ranks by any means (a file, a socket, MPI, a store);
 * every rank then calls mft_comm_init with its own device current.  world = 1
 * is legal and makes every call below a no-op.
 *
 * Failure handling: none of these calls blocks on a peer.  A rank that knows a
 * peer has left (heartbeat, store) calls mft_comm_abort before its next launch;
 * afterwards every exchange returns MFT_ERR_NCCL.  mft_comm_async_error reports
 * what NCCL's watchdog has seen.  mft_comm_wait polls the stream until the
 * queued work has finished, an asynchronous NCCL error shows up, or the
 * deadline passes; in the last two cases it aborts the communicator (which
 * releases a collective that waits for a missing peer) and returns
 * MFT_ERR_NCCL / MFT_ERR_TIMEOUT. */
#define MFT_COMM_ID_BYTES 128
int32_t mft_comm_unique_id(uint8_t* id_host);
int32_t mft_comm_init(int32_t rank, int32_t world, const uint8_t* id_host);
int32_t mft_comm_info(int32_t* rank, int32_t* world, int32_t* nccl_version);
/* In-place sum over all ranks, asynchronous on `stream`. */
int32_t mft_allreduce_sum_f32(float* buf, int64_t n, mft_stream_t stream);
int32_t mft_allreduce_sum_i64(int64_t* buf, int64_t n, mft_stream_t stream);
int32_t mft_comm_async_error(int32_t* nccl_result_host);
int32_t mft_comm_wait(mft_stream_t stream, int32_t timeout_ms);
int32_t mft_comm_abort(void);
int32_t mft_comm_destroy(void);

/* ---- generic fp32 operators behind the eager ops:: surface (add/sub/mul/div with broadcasting
 *      ops.cpp:299-560, unary maps :1221-1305, sum/mean :1970-2127, transpose/permute :990-1149,
 *      matmul :619-988 in full fp32, softmax :1307-1363 / SoftmaxBackward backward_functions.cpp:306-349,
 *      apply_rope on [B,H,S,D] :2337-2414, swiglu :2416-2452).  Contiguous tensors, fp32 accuracy. ---- */
#define MFT_EW_ADD 0
#define MFT_EW_SUB 1
#define MFT_EW_MUL 2
#define MFT_EW_DIV 3
#define MFT_UN_GELU 0
#define MFT_UN_GELU_GRAD 1
#define MFT_UN_SILU 2
#define MFT_UN_SIGMOID 3
#define MFT_UN_TANH 4
#define MFT_UN_RELU 5
#define MFT_UN_EXP 6
#define MFT_UN_LOG 7
#define MFT_UN_SQRT 8
#define MFT_UN_ABS 9
#define MFT_UN_POW 10
#define MFT_UN_NEG 11
#define MFT_UN_COPY 12
/* out = a (op) b with right-aligned (numpy-style) broadcasting; at most 6 dimensions. */
int32_t mft_ew_binary_f32(int32_t op, const float* a, const int64_t* a_shape_host, int32_t a_nd,
                          const float* b, const int64_t* b_shape_host, int32_t b_nd,
                          float* out, const int64_t* out_shape_host, int32_t out_nd, mft_stream_t stream);
int32_t mft_ew_scalar_f32(int32_t op, const float* a, float scalar, int32_t scalar_first, float* out, int64_t n, mft_stream_t stream);
int32_t mft_ew_unary_f32(int32_t op, const float* a, float param, float* out, int64_t n, mft_stream_t stream);
/* out[o, i] = scale * sum_r in[o, r, i] */
int32_t mft_reduce_sum_f32(const float* in, float* out, int64_t outer, int64_t reduce, int64_t inner, float scale, mft_stream_t stream);
/* out = in permuted: out dim k is in dim perm[k]; 32-bit elements of any type. */
int32_t mft_permute_b32(const void* in, void* out, const int64_t* in_shape_host, const int32_t* perm_host, int32_t nd, mft_stream_t stream);
/* C[b] (m x n) = A[b] (m x k) * B[b] with B [k,n] (trans_b = 0) or [n,k] (trans_b = 1); batch strides in elements (0 = shared). */
int32_t mft_matmul_f32(const float* a, const float* b, float* c, int64_t batch, int64_t m, int64_t n, int64_t k,
                       int64_t stride_a, int64_t stride_b, int64_t stride_c, int32_t trans_b, mft_stream_t stream);
int32_t mft_softmax_f32(const float* x, float* y, int64_t rows, int64_t dim, mft_stream_t stream);
int32_t mft_softmax_bwd_f32(const float* y, const float* dy, float* dx, int64_t rows, int64_t dim, mft_stream_t stream);
/* x, y: [rows, seq, head_dim] f32 (rows = batch*heads); backward != 0 applies the transposed rotation. */
int32_t mft_rope_f32(const float* x, float* y, const float* cos_tab, const float* sin_tab, int64_t rows, int64_t seq,
                     int64_t head_dim, int32_t backward, mft_stream_t stream);
/* dy == NULL: out1 = silu(gate)*up.  Otherwise out1 = d(gate), out2 = d(up). */
int32_t mft_swiglu_f32(const float* gate, const float* up, const float* dy, float* out1, float* out2, int64_t n, mft_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MFT_CUDA_H */
