// The reference's op-level pieces of the chunked scan as stand-alone kernels, so that code written against its custom
// ops (src/assoc_kernel.py: membrae::assoc_out :128, prefix_scan :231, delta_loop_fwd :363) finds the same operators
// with the same argument lists here. The product path does not use them -- one fused walk replaces all three and never
// writes the per-chunk states to memory unless asked -- so these are plain fp32 FFMA kernels built for exactness, not
// speed: every product is formed in fp32 (the reference rounds its operands to bf16 first), the state entering each
// chunk is stored as bf16 exactly as the reference stores it.
//
//   assoc_out       one CTA per (sequence-head, chunk):   o = ((q k^T) * dec) v + (q e^L) S_entering[c]
//   prefix_scan     one CTA per (sequence-head, 16 state columns), walking chunks:  S_ent[c] = S;  S = e^{a_c} S + (k w)^T v
//   delta_loop_fwd  one CTA per (sequence-head, 16 state columns), walking chunks:
//                   rhs = beta (v - e^L k S);  W = X rhs;  S = e^{L_C} S + (k w)^T W        (X from delta_inv)
#include "common.cuh"

namespace pgb {

constexpr int SO_C = 64, SO_NT = 256, SO_BV = 16;

template <typename T_> __device__ __forceinline__ float so_ld(const T_ *p) {
    if constexpr (sizeof(T_) == 2) return __bfloat162float(*p); else return *p;
}
template <typename T_> __device__ __forceinline__ void so_st(T_ *p, float x) {
    if constexpr (sizeof(T_) == 2) *p = __float2bfloat16_rn(x); else *p = x;
}

// inclusive cumulative log-decay of one chunk: thread t < 64 sums la[0..t] (64 adds; this is not the hot path)
__device__ __forceinline__ void so_cumsum(const float *la_sm, float *L_sm, int tid) {
    if (tid < SO_C) {
        float s = 0.f;
        for (int i = 0; i <= tid; ++i) s += la_sm[i];
        L_sm[tid] = s;
    }
}

// ---------------------------------------------------------------------------------------------------- assoc_out
template <typename TIO, int D>
__global__ void __launch_bounds__(SO_NT) assoc_out_kernel(const TIO *__restrict__ q, const TIO *__restrict__ k, const TIO *__restrict__ v,
                                                          const float *__restrict__ la, const __nv_bfloat16 *__restrict__ sent,
                                                          TIO *__restrict__ o, int T, int NC) {
    constexpr int P = D + 1;                                          // row pitch: rows of different tokens hit different banks
    extern __shared__ float so_smem[];
    float *qs = so_smem, *ks = qs + SO_C * P, *vs = ks + SO_C * P, *A = vs + SO_C * P, *las = A + SO_C * (SO_C + 1), *L = las + SO_C;
    const int tid = threadIdx.x, c = blockIdx.x, bh = blockIdx.y, t0 = c * SO_C;
    const size_t base = ((size_t)bh * T + t0) * D;
    for (int idx = tid; idx < SO_C * D; idx += SO_NT) {
        const int r = idx / D, i = idx % D;
        const bool live = t0 + r < T;
        qs[r * P + i] = live ? so_ld(q + base + idx) : 0.f;
        ks[r * P + i] = live ? so_ld(k + base + idx) : 0.f;
        vs[r * P + i] = live ? so_ld(v + base + idx) : 0.f;
    }
    if (tid < SO_C) las[tid] = t0 + tid < T ? la[(size_t)bh * T + t0 + tid] : 0.f;
    __syncthreads();
    so_cumsum(las, L, tid);
    __syncthreads();
    {   // decayed causal scores: thread (t, 16 consecutive s)
        const int t = tid >> 2, s0 = (tid & 3) * 16;
        for (int s = s0; s < s0 + 16; ++s) {
            float acc = 0.f;
            if (s <= t) {
                for (int i = 0; i < D; ++i) acc = fmaf(qs[t * P + i], ks[s * P + i], acc);
                acc *= expf(fminf(L[t] - L[s], 0.f));
            }
            A[t * (SO_C + 1) + s] = acc;
        }
    }
    __syncthreads();
    // output: thread (column j, a group of NT token rows)
    constexpr int NG = SO_NT / D, NT = SO_C / NG;
    const int j = tid % D, tg = tid / D;
    float acc[NT];
#pragma unroll
    for (int tt = 0; tt < NT; ++tt) acc[tt] = 0.f;
    for (int s = 0; s < SO_C; ++s) {
        const float vv = vs[s * P + j];
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) acc[tt] = fmaf(A[(tg * NT + tt) * (SO_C + 1) + s], vv, acc[tt]);
    }
    const __nv_bfloat16 *Sc = sent + ((size_t)bh * NC + c) * D * D;
    float rd[NT];
#pragma unroll
    for (int tt = 0; tt < NT; ++tt) rd[tt] = 0.f;
    for (int i = 0; i < D; ++i) {
        const float sv = __bfloat162float(Sc[(size_t)i * D + j]);
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) rd[tt] = fmaf(qs[(tg * NT + tt) * P + i], sv, rd[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < NT; ++tt) {
        const int t = tg * NT + tt;
        if (t0 + t < T) so_st(o + base + (size_t)t * D + j, fmaf(expf(L[t]), rd[tt], acc[tt]));
    }
}

// ---------------------------------------------------------------------------------------------------- prefix_scan
// k, v: whole chunks, [BH][NC*64][D];  w [BH][NC][64];  a_log [BH][NC]
template <typename TIO, int D>
__global__ void __launch_bounds__(SO_NT) prefix_scan_kernel(const TIO *__restrict__ k, const TIO *__restrict__ v, const float *__restrict__ w,
                                                            const float *__restrict__ a_log, const float *__restrict__ S0,
                                                            __nv_bfloat16 *__restrict__ sent, float *__restrict__ sfin, int NC) {
    constexpr int P = D + 1, NR = D / 16;                            // NR state rows per thread
    extern __shared__ float so_smem[];
    float *kw = so_smem, *vs = kw + SO_C * P;                         // [64][P], [64][16]
    const int tid = threadIdx.x, j = tid % SO_BV, i0 = tid / SO_BV, col0 = blockIdx.x * SO_BV, bh = blockIdx.y;
    float S[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) S[r] = S0 != nullptr ? S0[((size_t)bh * D + i0 + 16 * r) * D + col0 + j] : 0.f;
    for (int c = 0; c < NC; ++c) {
        const size_t base = ((size_t)bh * NC + c) * SO_C * D;
        __syncthreads();
        for (int idx = tid; idx < SO_C * D; idx += SO_NT) {
            const int r = idx / D, i = idx % D;
            kw[r * P + i] = so_ld(k + base + idx) * w[((size_t)bh * NC + c) * SO_C + r];
        }
        for (int idx = tid; idx < SO_C * SO_BV; idx += SO_NT) {
            const int r = idx / SO_BV, jj = idx % SO_BV;
            vs[idx] = so_ld(v + base + (size_t)r * D + col0 + jj);
        }
        __syncthreads();
        const float a = expf(a_log[(size_t)bh * NC + c]);
        __nv_bfloat16 *dst = sent + ((size_t)bh * NC + c) * D * D;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const int i = i0 + 16 * r;
            dst[(size_t)i * D + col0 + j] = __float2bfloat16_rn(S[r]);
            float acc = 0.f;
            for (int s = 0; s < SO_C; ++s) acc = fmaf(kw[s * P + i], vs[s * SO_BV + j], acc);
            S[r] = fmaf(a, S[r], acc);
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) sfin[((size_t)bh * D + i0 + 16 * r) * D + col0 + j] = S[r];
}

// ---------------------------------------------------------------------------------------------------- delta_loop_fwd
// k, v [BH][T][D] (ragged last chunk masked);  X [BH][NC][64][64] bf16;  W out [BH][T][D] bf16
template <typename TIO, int D>
__global__ void __launch_bounds__(SO_NT) delta_loop_kernel(const TIO *__restrict__ k, const TIO *__restrict__ v, const float *__restrict__ la,
                                                           const float *__restrict__ be, const __nv_bfloat16 *__restrict__ X,
                                                           const float *__restrict__ S0, __nv_bfloat16 *__restrict__ W,
                                                           __nv_bfloat16 *__restrict__ sent, float *__restrict__ sfin, int T, int NC) {
    constexpr int P = D + 1, NR = D / 16, XP = SO_C + 1;
    extern __shared__ float so_smem[];
    float *ks = so_smem, *Xs = ks + SO_C * P, *Ss = Xs + SO_C * XP, *vs = Ss + D * SO_BV, *rhs = vs + SO_C * SO_BV,
          *Ws = rhs + SO_C * SO_BV, *las = Ws + SO_C * SO_BV, *L = las + SO_C, *bes = L + SO_C;
    const int tid = threadIdx.x, j = tid % SO_BV, i0 = tid / SO_BV, col0 = blockIdx.x * SO_BV, bh = blockIdx.y;
#pragma unroll
    for (int r = 0; r < NR; ++r)
        Ss[(i0 + 16 * r) * SO_BV + j] = S0 != nullptr ? S0[((size_t)bh * D + i0 + 16 * r) * D + col0 + j] : 0.f;
    for (int c = 0; c < NC; ++c) {
        const int t0 = c * SO_C;
        const size_t base = ((size_t)bh * T + t0) * D;
        __syncthreads();
        for (int idx = tid; idx < SO_C * D; idx += SO_NT) {
            const int r = idx / D, i = idx % D;
            ks[r * P + i] = t0 + r < T ? so_ld(k + base + idx) : 0.f;
        }
        for (int idx = tid; idx < SO_C * SO_C; idx += SO_NT)
            Xs[(idx / SO_C) * XP + idx % SO_C] = __bfloat162float(X[((size_t)bh * NC + c) * SO_C * SO_C + idx]);
        for (int idx = tid; idx < SO_C * SO_BV; idx += SO_NT) {
            const int r = idx / SO_BV, jj = idx % SO_BV;
            vs[idx] = t0 + r < T ? so_ld(v + base + (size_t)r * D + col0 + jj) : 0.f;
        }
        if (tid < SO_C) {
            las[tid] = t0 + tid < T ? la[(size_t)bh * T + t0 + tid] : 0.f;
            bes[tid] = t0 + tid < T ? be[(size_t)bh * T + t0 + tid] : 0.f;
        }
        __nv_bfloat16 *dst = sent + ((size_t)bh * NC + c) * D * D;
#pragma unroll
        for (int r = 0; r < NR; ++r) dst[(size_t)(i0 + 16 * r) * D + col0 + j] = __float2bfloat16_rn(Ss[(i0 + 16 * r) * SO_BV + j]);
        __syncthreads();
        so_cumsum(las, L, tid);
        __syncthreads();
        // rhs = beta (v - e^L k S): thread (column j, token rows tr + 16 m)
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int t = i0 + 16 * m;
            float acc = 0.f;
            for (int i = 0; i < D; ++i) acc = fmaf(ks[t * P + i], Ss[i * SO_BV + j], acc);
            rhs[t * SO_BV + j] = bes[t] * (vs[t * SO_BV + j] - expf(L[t]) * acc);
        }
        __syncthreads();
        // W = X rhs (X is unit lower triangular: the sum stops at the diagonal)
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int t = i0 + 16 * m;
            float acc = 0.f;
            for (int s = 0; s <= t; ++s) acc = fmaf(Xs[t * XP + s], rhs[s * SO_BV + j], acc);
            Ws[t * SO_BV + j] = acc;
            if (t0 + t < T) W[base + (size_t)t * D + col0 + j] = __float2bfloat16_rn(acc);
        }
        __syncthreads();
        // S = e^{L_C} S + (k w)^T W,  w_s = e^{L_C - L_s}
        const float LC = L[SO_C - 1], aC = expf(LC);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const int i = i0 + 16 * r;
            float acc = 0.f;
            for (int s = 0; s < SO_C; ++s) acc = fmaf(ks[s * P + i] * expf(fminf(LC - L[s], 0.f)), Ws[s * SO_BV + j], acc);
            Ss[i * SO_BV + j] = fmaf(aC, Ss[i * SO_BV + j], acc);     // read and written by this thread only
        }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < NR; ++r) sfin[((size_t)bh * D + i0 + 16 * r) * D + col0 + j] = Ss[(i0 + 16 * r) * SO_BV + j];
}

// ---------------------------------------------------------------------------------------------------- host side
template <typename K>
static int so_attr(K kern, size_t smem, const char *what) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e, what); return PGB_ERR_CUDA; }
    return PGB_OK;
}

template <typename TIO, int D>
static int assoc_out_go(const void *q, const void *k, const void *v, const float *la, const void *sent, void *o, int BH, int T, cudaStream_t st) {
    const int NC = (T + SO_C - 1) / SO_C;
    const size_t smem = (size_t)(3 * SO_C * (D + 1) + SO_C * (SO_C + 1) + 2 * SO_C) * sizeof(float);
    int rc = so_attr(assoc_out_kernel<TIO, D>, smem, "assoc_out smem attribute");
    if (rc != PGB_OK) return rc;
    assoc_out_kernel<TIO, D><<<dim3(NC, BH), SO_NT, smem, st>>>((const TIO *)q, (const TIO *)k, (const TIO *)v, la,
                                                               (const __nv_bfloat16 *)sent, (TIO *)o, T, NC);
    return check_launch("assoc_out_kernel");
}

int assoc_out_launch(const void *q, const void *k, const void *v, int io_dtype, const float *la, const void *sent, void *o, int BH, int T,
                     int D, cudaStream_t st) {
    if (io_dtype == PGB_BF16)
        return D == 64 ? assoc_out_go<__nv_bfloat16, 64>(q, k, v, la, sent, o, BH, T, st) : assoc_out_go<__nv_bfloat16, 128>(q, k, v, la, sent, o, BH, T, st);
    return D == 64 ? assoc_out_go<float, 64>(q, k, v, la, sent, o, BH, T, st) : assoc_out_go<float, 128>(q, k, v, la, sent, o, BH, T, st);
}

template <typename TIO, int D>
static int prefix_scan_go(const void *k, const void *v, const float *w, const float *a_log, const float *S0, void *sent, float *sfin, int BH,
                          int NC, cudaStream_t st) {
    const size_t smem = (size_t)(SO_C * (D + 1) + SO_C * SO_BV) * sizeof(float);
    int rc = so_attr(prefix_scan_kernel<TIO, D>, smem, "prefix_scan smem attribute");
    if (rc != PGB_OK) return rc;
    prefix_scan_kernel<TIO, D><<<dim3(D / SO_BV, BH), SO_NT, smem, st>>>((const TIO *)k, (const TIO *)v, w, a_log, S0,
                                                                       (__nv_bfloat16 *)sent, sfin, NC);
    return check_launch("prefix_scan_kernel");
}

int prefix_scan_launch(const void *k, const void *v, int io_dtype, const float *w, const float *a_log, const float *S0, void *sent,
                       float *sfin, int BH, int NC, int D, cudaStream_t st) {
    if (io_dtype == PGB_BF16)
        return D == 64 ? prefix_scan_go<__nv_bfloat16, 64>(k, v, w, a_log, S0, sent, sfin, BH, NC, st)
                       : prefix_scan_go<__nv_bfloat16, 128>(k, v, w, a_log, S0, sent, sfin, BH, NC, st);
    return D == 64 ? prefix_scan_go<float, 64>(k, v, w, a_log, S0, sent, sfin, BH, NC, st)
                   : prefix_scan_go<float, 128>(k, v, w, a_log, S0, sent, sfin, BH, NC, st);
}

template <typename TIO, int D>
static int delta_loop_go(const void *k, const void *v, const float *la, const float *be, const void *X, const float *S0, void *W, void *sent,
                         float *sfin, int BH, int T, cudaStream_t st) {
    const int NC = (T + SO_C - 1) / SO_C;
    const size_t smem = (size_t)(SO_C * (D + 1) + SO_C * (SO_C + 1) + D * SO_BV + 3 * SO_C * SO_BV + 3 * SO_C) * sizeof(float);
    int rc = so_attr(delta_loop_kernel<TIO, D>, smem, "delta_loop smem attribute");
    if (rc != PGB_OK) return rc;
    delta_loop_kernel<TIO, D><<<dim3(D / SO_BV, BH), SO_NT, smem, st>>>((const TIO *)k, (const TIO *)v, la, be, (const __nv_bfloat16 *)X, S0,
                                                                      (__nv_bfloat16 *)W, (__nv_bfloat16 *)sent, sfin, T, NC);
    return check_launch("delta_loop_kernel");
}

int delta_loop_launch(const void *k, const void *v, int io_dtype, const float *la, const float *be, const void *X, const float *S0, void *W,
                      void *sent, float *sfin, int BH, int T, int D, cudaStream_t st) {
    if (io_dtype == PGB_BF16)
        return D == 64 ? delta_loop_go<__nv_bfloat16, 64>(k, v, la, be, X, S0, W, sent, sfin, BH, T, st)
                       : delta_loop_go<__nv_bfloat16, 128>(k, v, la, be, X, S0, W, sent, sfin, BH, T, st);
    return D == 64 ? delta_loop_go<float, 64>(k, v, la, be, X, S0, W, sent, sfin, BH, T, st)
                   : delta_loop_go<float, 128>(k, v, la, be, X, S0, W, sent, sfin, BH, T, st);
}

}  // namespace pgb
