// One recurrent decode step of the associative carrier, fused: one CTA per (sequence, head).
//
// HBM traffic is the state: D*D fp32 read and written once (2*D*D*4 bytes per head), plus ~1 KB of vectors. Every
// state access is a 128-bit load/store; a thread owns 4 adjacent value columns of whole ROW PAIRS (2i, 2i+1), so the
// rebase rotation of the key axis (pairs of rows) is thread-local. The state slice stays in registers between the
// delta rule's two passes; q, k, v and the partial sums go through shared memory.
//
// Per (b,h), with shift the number of positions the carried state is rotated back by (reference src/assoc.py:399-402):
//   S <- R(-shift*theta) S (rows 2i,2i+1 rotated);  Sd = alpha S
//   plain:  S' = Sd + k v^T                          delta:  r = beta (v - Sd^T k),  S' = Sd + k r^T
//   o = S'^T q    [optionally o <- o * rsqrt(mean(o^2) + eps) * w, the carrier's per-head RMS norm, src/assoc.py:505]
#include "decode_step.cuh"

namespace pgb {

template <typename TIN, typename TOUT, int D, bool DELTA>
__global__ void __launch_bounds__(DEC_THREADS) decode_step_kernel(DecodeArgs a) {
    // Launched as a programmatic dependent: nothing is read before the kernel ahead (the projection) has completed, and the
    // kernel behind (the output projection) may start requesting its weights now.
    pdl_wait();
    pdl_launch_dependents();
    decode_step_body<TIN, TOUT, D, DELTA>(a, blockIdx.x / a.H, blockIdx.x % a.H, [] { return true; });
}

template <typename TIN, typename TOUT>
static int decode_dispatch(const DecodeArgs &a, int D, int delta, cudaStream_t stream) {
    const unsigned grid = (unsigned)(a.B * a.H);
    cudaError_t e;
    if (D == 64) {
        if (delta) e = pdl_launch(decode_step_kernel<TIN, TOUT, 64, true>, dim3(grid), dim3(DEC_THREADS), 0, stream, a);
        else e = pdl_launch(decode_step_kernel<TIN, TOUT, 64, false>, dim3(grid), dim3(DEC_THREADS), 0, stream, a);
    } else {
        if (delta) e = pdl_launch(decode_step_kernel<TIN, TOUT, 128, true>, dim3(grid), dim3(DEC_THREADS), 0, stream, a);
        else e = pdl_launch(decode_step_kernel<TIN, TOUT, 128, false>, dim3(grid), dim3(DEC_THREADS), 0, stream, a);
    }
    if (e != cudaSuccess) { set_cuda_error(e, "decode_step launch"); return PGB_ERR_CUDA; }
    return check_launch("decode_step_kernel");
}

int decode_launch(const DecodeArgs &a, int in_dtype, int out_dtype, int D, int delta, cudaStream_t stream) {
    if (in_dtype == PGB_F32 && out_dtype == PGB_F32) return decode_dispatch<float, float>(a, D, delta, stream);
    if (in_dtype == PGB_F32 && out_dtype == PGB_BF16) return decode_dispatch<float, __nv_bfloat16>(a, D, delta, stream);
    if (in_dtype == PGB_BF16 && out_dtype == PGB_F32) return decode_dispatch<__nv_bfloat16, float>(a, D, delta, stream);
    return decode_dispatch<__nv_bfloat16, __nv_bfloat16>(a, D, delta, stream);
}

}  // namespace pgb
