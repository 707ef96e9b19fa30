// Shared helpers for the carrier kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pragnosia_b200.h"

namespace pgb {

// thread-local text of the last CUDA error this library saw
void set_cuda_error(cudaError_t e, const char *where);

inline int check_launch(const char *where) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_cuda_error(e, where);
        return PGB_ERR_CUDA;
    }
    return PGB_OK;
}

inline bool aligned(const void *p, size_t n) { return (reinterpret_cast<uintptr_t>(p) % n) == 0; }

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ void from_f32(float &d, float x) { d = x; }
__device__ __forceinline__ void from_f32(__nv_bfloat16 &d, float x) { d = __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// softplus with torch's threshold (x > 20 -> x)
__device__ __forceinline__ float softplusf_(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// cheap forms for gate logits that arrive in bf16 (8 bits of mantissa): ex2/lg2-based, ~1e-6 relative
// Programmatic dependent launch. A kernel launched with pdl_launch() may start while the kernel before it in the stream
// is still running; pdl_wait() blocks until that kernel has completed and its writes are visible (a no-op when the launch
// carried no such dependency), so everything that reads activations or writes anything comes after it, and only
// constants (weights) are touched before. pdl_launch_dependents() lets the next kernel in the stream start likewise.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <typename... KArgs, typename... Args>
inline cudaError_t pdl_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// 2^x by the hardware approximation (relative error about 2^-22; results below 2^-126 flush to zero)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float fast_softplus(float x) { return x > 20.0f ? x : __logf(1.0f + __expf(x)); }

// launch arguments shared between the C ABI layer and the kernels' translation units
struct PrefillArgs {
    const void *q, *k, *v; const float *la, *beta, *S0; void *o; float *S_out; __nv_bfloat16 *sent;
    const float *theta; const float *shift_dev; float shift_host;      // rebase of S0's key axis (theta NULL: none)
    int B, H, T;
    // fused layer pieces, tensor-core kernel only (zero / NULL = off)
    const void *la_raw = nullptr; long long la_sb = 0, la_st = 0; const float *decay_A = nullptr;
    const float *rms_w = nullptr; float rms_eps = 0.f; int o_token_major = 0;
    // raw mode: q, k, v are (B,T,H*D) views of the projection output with strides (raw_sb, raw_st); the kernel does the
    // normalise / gate / rotate itself (gate_raw: write-gate logits with la_raw's strides; rot: table [H][rot_T][D/2])
    int raw = 0; long long raw_sb = 0, raw_st = 0; const void *gate_raw = nullptr; const float *rot = nullptr; int rot_T = 0;
};
struct DecodeArgs {
    const void *qp, *kp, *vp; long long in_sb; int normalize;
    const void *gate; long long gate_sb; int gate_is_logit;
    const void *decay; long long decay_sb; const float *decay_A;
    const float *theta; const float *shift_dev; float shift_host;
    const float *S_in; float *S_out; const float *rms_w; float rms_eps;
    void *o; long long out_sb; int B, H;
};

}  // namespace pgb
