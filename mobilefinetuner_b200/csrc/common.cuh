// Shared helpers for the kernels of libmft_cuda.so: status handling, launch
// accounting, bf16 vector access and warp/block reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string>

#include "../../include/mft_cuda.h"

namespace mft {

// One flag per device for set-up that CUDA keeps per device (cudaFuncSetAttribute): `here()` is the current device's.
struct PerDeviceFlag {
    bool v[64] = {};
    bool& here() {
        int d = 0;
        cudaGetDevice(&d);
        return v[(d >= 0 && d < 64) ? d : 0];
    }
};


// Thread-local last-error message plus the process-wide launch counter.
void set_error(const std::string& msg);
void count_launch(int n = 1);
// With MFT_LAUNCH_REPORT=<file> in the environment the library also counts launches per kernel family (the name given
// to MFT_LAUNCH_CHECK; kernels captured into a step graph are counted once, at capture) and writes "name count" lines
// to that file when the process exits: a way to see from outside which kernels a host program ran.
void note_launch(const char* name);
int32_t* device_status_word();   // int32 in device memory, set by kernels whose bounded waits ran out

int32_t fail(int32_t code, const std::string& msg);
int32_t check_cuda(cudaError_t e, const char* what);

// ---- programmatic dependent launch.  A kernel launched through launch_dep() may become resident while the
// kernel before it in the stream is still draining: it runs its set-up (barrier init, tensor-memory allocation,
// descriptor prefetch), then dep_wait() blocks until the previous kernel has completed and its writes are
// visible.  Such a kernel must not touch global memory before dep_wait().  dep_trigger() tells the scheduler
// that the NEXT kernel may start its own set-up.  Both are no-ops in a kernel launched the ordinary way.
// Whether it pays depends on the step: a large step that sits at the power cap measured 1 % SLOWER with it (118.5 vs
// 117.1 ms, alternating runs on one GPU), steps of a few thousand tokens, whose kernels are short against their own
// set-up, measured faster (Qwen2.5-0.5B at 8 x 512: 16.63 -> 16.40 ms; GPT-2 small at 4 x 128: 2.30 -> 2.22 ms).  The
// step engine therefore turns it on for its own launches when a step has at most 8192 tokens (DepLaunchScope);
// MFT_PDL=0 / 1 in the environment overrides that for the whole process.
bool dep_launch_enabled();
bool set_dep_launch_hint(bool on);      // returns the previous hint of this host thread
struct DepLaunchScope {
    bool active = false, previous = false;
    DepLaunchScope() = default;
    DepLaunchScope(const DepLaunchScope&) = delete;
    DepLaunchScope& operator=(const DepLaunchScope&) = delete;
    void set(bool on) { if (!active) { previous = set_dep_launch_hint(on); active = true; } else set_dep_launch_hint(on); }
    ~DepLaunchScope() { if (active) set_dep_launch_hint(previous); }
};
__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dep_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dep_launch_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define MFT_CHECK_ARG(cond, msg)                                   \
    do {                                                           \
        if (!(cond)) return ::mft::fail(MFT_ERR_INVALID_ARG, msg); \
    } while (0)

#define MFT_LAUNCH_CHECK(name)                                                 \
    do {                                                                       \
        ::mft::count_launch();                                                 \
        ::mft::note_launch(name);                                              \
        cudaError_t e__ = cudaGetLastError();                                  \
        if (e__ != cudaSuccess) return ::mft::check_cuda(e__, name);           \
    } while (0)

static inline cudaStream_t as_stream(mft_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// ---------------------------------------------------------------- device helpers
__device__ __forceinline__ float bf16_to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 f32_to_bf16(float v) { return __float2bfloat16_rn(v); }

// 8 bf16 values = 16 bytes
struct __align__(16) bf16x8 {
    __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&out)[8]) {
    bf16x8 r = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(r.v[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void load8(const float* p, float (&out)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *reinterpret_cast<const float4*>(p + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&in)[8]) {
    bf16x8 r;
#pragma unroll
    for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
    *reinterpret_cast<bf16x8*>(p) = r;
}
__device__ __forceinline__ void store8(float* p, const float (&in)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(in[4], in[5], in[6], in[7]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block-wide sum; `scratch` is 32 floats of shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float r = (lane < nwarps) ? scratch[lane] : 0.0f;
    r = warp_sum(r);
    return r;
}

__device__ __forceinline__ float gelu_tanh_f(float x) {
    float t = 0.7978845608f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(t));
}
__device__ __forceinline__ float gelu_tanh_grad_f(float x) {
    float x2 = x * x;
    float t = tanhf(0.7978845608f * (x + 0.044715f * x * x2));
    float dt = 0.7978845608f * (1.0f + 3.0f * 0.044715f * x2);
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * dt;
}

}  // namespace mft
