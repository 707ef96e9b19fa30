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

// ---- head dim 64, one WARP per (sequence, head)
// A lane owns two adjacent value columns of ALL 64 key rows (128 registers of state, 64 eight-byte loads in flight per
// lane, 256 contiguous bytes per row and warp), so everything a column needs -- the delta rule's K^T S, the read S^T q --
// is a sum inside one thread and the rotation of row pairs is thread-local as before: no partial sums through shared
// memory and no block barrier anywhere; q, k and the rotation constants are handed round through the warp's own lines of
// shared memory. With enough pairs to fill the SMs with warps (configuration 2's 64 sequences: 768) the step is one round
// of loads, a few hundred instructions and one round of stores and is a seventh shorter than the block-per-head kernel
// above with its three barriers; at large batches both run at the HBM rate; with few pairs the block kernel is quicker.
constexpr int DW_WARPS = 4;                                           // (sequence, head) units per CTA

template <typename TIN, typename TOUT, bool DELTA>
__global__ void __launch_bounds__(DW_WARPS * 32) decode_step_warp_kernel(DecodeArgs a) {
    constexpr int D = 64;
    __shared__ __align__(16) float sq[DW_WARPS][D], sk[DW_WARPS][D];
    __shared__ __align__(16) float2 srot[DW_WARPS][D / 2];            // alpha * (cos, sin) of the rebase rotation, per row pair
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int unit = blockIdx.x * DW_WARPS + w;
    pdl_wait();                                                       // nothing is read before the kernel ahead has completed
    pdl_launch_dependents();
    if (unit >= a.B * a.H) return;                                    // whole warps leave; the warps of a CTA never meet
    const int b = unit / a.H, h = unit - b * a.H;

    // ---- the state first: its loads are the long latency
    const float2 *Sin = reinterpret_cast<const float2 *>(a.S_in + (size_t)unit * D * D) + lane;
    float2 *Sout = reinterpret_cast<float2 *>(a.S_out + (size_t)unit * D * D) + lane;
    float2 s[D];
#pragma unroll
    for (int i = 0; i < D; ++i) s[i] = __ldcs(Sin + i * (D / 2));

    // ---- vectors and scalars
    const TIN *qp = (const TIN *)a.qp + (size_t)b * a.in_sb + (size_t)h * D;
    const TIN *kp = (const TIN *)a.kp + (size_t)b * a.in_sb + (size_t)h * D;
    const TIN *vp = (const TIN *)a.vp + (size_t)b * a.in_sb + (size_t)h * D;
    float q0 = to_f32(qp[lane]), q1 = to_f32(qp[lane + 32]);
    float k0 = to_f32(kp[lane]), k1 = to_f32(kp[lane + 32]);
    float2 vv = make_float2(to_f32(vp[2 * lane]), to_f32(vp[2 * lane + 1]));   // this lane's two columns
    float dl = to_f32(((const TIN *)a.decay)[(size_t)b * a.decay_sb + h]);
    if (a.decay_A != nullptr) dl = -softplusf_(dl) * expf(a.decay_A[h]);
    const float alpha = expf(dl);
    float g = 1.f;
    if (a.gate != nullptr) {
        g = to_f32(((const TIN *)a.gate)[(size_t)b * a.gate_sb + h]);
        if (a.gate_is_logit) g = sigmoidf_(g);
    }
    if (a.normalize) {
        const float iq = 1.0f / fmaxf(sqrtf(warp_sum(q0 * q0 + q1 * q1)), 1e-12f);
        const float ik = 1.0f / fmaxf(sqrtf(warp_sum(k0 * k0 + k1 * k1)), 1e-12f);
        const float iv = 1.0f / fmaxf(sqrtf(warp_sum(vv.x * vv.x + vv.y * vv.y)), 1e-12f);
        q0 *= iq; q1 *= iq; k0 *= ik; k1 *= ik; vv.x *= iv; vv.y *= iv;
    }
    const float kscale = DELTA ? 1.f : g;                             // plain rule: the write gate scales k; delta rule: g is beta
    sq[w][lane] = q0; sq[w][lane + 32] = q1;
    sk[w][lane] = k0 * kscale; sk[w][lane + 32] = k1 * kscale;
    {
        const float shift = a.shift_dev != nullptr ? *a.shift_dev : a.shift_host;
        float sn = 0.f, cs = 1.f;
        if (shift != 0.f) sincosf(-shift * a.theta[(size_t)h * (D / 2) + lane], &sn, &cs);   // lane = row pair
        srot[w][lane] = make_float2(alpha * cs, alpha * sn);
    }
    __syncwarp();

    float2 acc = make_float2(0.f, 0.f);                               // delta: sum_r k_r Sd[r][j];  plain: sum_r q_r S'[r][j]
#pragma unroll
    for (int p = 0; p < D / 2; ++p) {
        const float2 r = srot[w][p];
        const float2 kk = *reinterpret_cast<const float2 *>(&sk[w][2 * p]);
        const float2 x0 = s[2 * p], x1 = s[2 * p + 1];
        float2 d0, d1;                                                // alpha * rotated rows
        d0.x = x0.x * r.x - x1.x * r.y; d1.x = x0.x * r.y + x1.x * r.x;
        d0.y = x0.y * r.x - x1.y * r.y; d1.y = x0.y * r.y + x1.y * r.x;
        if constexpr (DELTA) {
            acc.x += kk.x * d0.x + kk.y * d1.x; acc.y += kk.x * d0.y + kk.y * d1.y;
        } else {
            const float2 qq = *reinterpret_cast<const float2 *>(&sq[w][2 * p]);
            d0.x += kk.x * vv.x; d0.y += kk.x * vv.y; d1.x += kk.y * vv.x; d1.y += kk.y * vv.y;
            acc.x += qq.x * d0.x + qq.y * d1.x; acc.y += qq.x * d0.y + qq.y * d1.y;
            Sout[(2 * p) * (D / 2)] = d0; Sout[(2 * p + 1) * (D / 2)] = d1;
        }
        s[2 * p] = d0; s[2 * p + 1] = d1;
    }
    if constexpr (DELTA) {
        const float2 rr = make_float2(g * (vv.x - acc.x), g * (vv.y - acc.y));    // what is written: beta (v - Sd^T k), whole in this lane
        acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int p = 0; p < D / 2; ++p) {
            const float2 kk = *reinterpret_cast<const float2 *>(&sk[w][2 * p]);
            const float2 qq = *reinterpret_cast<const float2 *>(&sq[w][2 * p]);
            float2 d0 = s[2 * p], d1 = s[2 * p + 1];
            d0.x += kk.x * rr.x; d0.y += kk.x * rr.y; d1.x += kk.y * rr.x; d1.y += kk.y * rr.y;
            acc.x += qq.x * d0.x + qq.y * d1.x; acc.y += qq.x * d0.y + qq.y * d1.y;
            Sout[(2 * p) * (D / 2)] = d0; Sout[(2 * p + 1) * (D / 2)] = d1;
        }
    }
    // ---- the read: optional per-head RMS norm, store
    if (a.rms_w != nullptr) {
        const float sc = rsqrtf(warp_sum(acc.x * acc.x + acc.y * acc.y) / (float)D + a.rms_eps);
        acc.x = acc.x * sc * a.rms_w[2 * lane]; acc.y = acc.y * sc * a.rms_w[2 * lane + 1];   // two loads: the weight need only be 4-byte aligned
    }
    TOUT *o = (TOUT *)a.o + (size_t)b * a.out_sb + (size_t)h * D + 2 * lane;
    from_f32(o[0], acc.x); from_f32(o[1], acc.y);
}

// 0: head dim 64 takes the warp-per-head kernel from DW_MIN_UNITS (sequence, head) pairs up; 1: always the block-per-head
// kernel; 2: the warp-per-head kernel at any size (A/B timing, tests). Measured inside the configuration-2 decode step
// (graph replay, ms per token, block / warp kernel): batch 64 (768 pairs) 0.507 / 0.494, the kernel itself 8.9 / 7.6 us
// against 3.9 us of bytes; batch 16 (192 pairs) 0.467 / 0.477 and batch 8 0.476 / 0.491 -- with few pairs a pair is better
// served by 256 threads than by one warp's few hundred instructions in a row; batch 1024: the same 70 us (the HBM rate).
constexpr int DW_MIN_UNITS = 512;
static int g_decode_variant = 0;
int decode_set_variant(int v) {
    if (v < 0 || v > 2) return PGB_ERR_BAD_SHAPE;
    g_decode_variant = v;
    return PGB_OK;
}

template <typename TIN, typename TOUT>
static int decode_dispatch(const DecodeArgs &a, int D, int delta, cudaStream_t stream) {
    const unsigned grid = (unsigned)(a.B * a.H);
    cudaError_t e;
    if (D == 64 && (g_decode_variant == 2 || (g_decode_variant == 0 && grid >= (unsigned)DW_MIN_UNITS))) {
        const unsigned gw = (grid + DW_WARPS - 1) / DW_WARPS;
        if (delta) e = pdl_launch(decode_step_warp_kernel<TIN, TOUT, true>, dim3(gw), dim3(DW_WARPS * 32), 0, stream, a);
        else e = pdl_launch(decode_step_warp_kernel<TIN, TOUT, false>, dim3(gw), dim3(DW_WARPS * 32), 0, stream, a);
        if (e != cudaSuccess) { set_cuda_error(e, "decode_step launch"); return PGB_ERR_CUDA; }
        return check_launch("decode_step_warp_kernel");
    }
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
