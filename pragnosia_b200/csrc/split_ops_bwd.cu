// Backward of the plain rule's two split operators (the reference's _bwd_chunk, src/assoc_kernel.py:75-126, and
// _prefix_bwd, :206-228, with their register_autograd wiring at :179 and :299), so that code written against
// membrae::assoc_out / membrae::prefix_scan can train through this library. Like the forward kernels in split_ops.cu
// these are plain fp32 FFMA kernels built for exactness, not speed; every gradient leaves in fp32 and every sum is taken
// in a fixed order (no atomics).
//
// assoc_out   o_t = sum_{s<=t} (q_t.k_s) e^{L_t-L_s} v_s + e^{L_t} q_t S,   L = inclusive cumulative sum of la in the chunk
//   one CTA per (sequence-head, chunk):   A = (q k^T) dec,  dA = (do v^T) masked,  dP = dA dec
//   dv = A^T do;  dk = dP^T q;  dq = dP k + e^{L} (do S^T);  dS = (q e^{L})^T do
//   dL_t = sum_s dA A [t,s] - sum_t' dA A [t',t] + e^{L_t} q_t.(do_t S^T);   dla = reverse cumulative sum of dL
//
// prefix_scan S_{c+1} = e^{a_c} S_c + sum_s (w_s k_s) v_s^T,  sent[c] = S_c
//   one CTA per sequence-head, walking the chunks backwards with G = dLoss/dS_{c+1} in shared memory:
//   dk_s = w_s G v_s;  dw_s = k_s.(G v_s);  dv_s = (w_s k_s) G;  da_c = e^{a_c} <G, S_c>;  G <- e^{a_c} G + dsent[c]
#include "common.cuh"

namespace pgb {

constexpr int SB_C = 64, SB_NT = 256;

template <typename T_> __device__ __forceinline__ float sb_ld(const T_ *p) {
    if constexpr (sizeof(T_) == 2) return __bfloat162float(*p); else return *p;
}

// ---------------------------------------------------------------------------------------------------- assoc_out backward
template <typename TIO, int D>
__global__ void __launch_bounds__(SB_NT) assoc_out_bwd_kernel(const TIO *__restrict__ q, const TIO *__restrict__ k, const TIO *__restrict__ v,
                                                              const float *__restrict__ la, const __nv_bfloat16 *__restrict__ sent,
                                                              const TIO *__restrict__ dout, float *__restrict__ dq, float *__restrict__ dk,
                                                              float *__restrict__ dv, float *__restrict__ dla, float *__restrict__ dsent,
                                                              int T, int NC) {
    constexpr int P = D + 1, MP = SB_C + 1;
    extern __shared__ float sb_smem[];
    float *qs = sb_smem, *ks = qs + SB_C * P, *vs = ks + SB_C * P, *ds = vs + SB_C * P, *R = ds + SB_C * P;
    float *A = R + SB_C * P, *dP = A + SB_C * MP, *Gm = dP + SB_C * MP, *las = Gm + SB_C * MP, *L = las + SB_C, *eL = L + SB_C,
          *dL = eL + SB_C;
    const int tid = threadIdx.x, c = blockIdx.x, bh = blockIdx.y, t0 = c * SB_C;
    const size_t base = ((size_t)bh * T + t0) * D;
    for (int idx = tid; idx < SB_C * D; idx += SB_NT) {
        const int r = idx / D, i = idx % D;
        const bool live = t0 + r < T;
        qs[r * P + i] = live ? sb_ld(q + base + idx) : 0.f;
        ks[r * P + i] = live ? sb_ld(k + base + idx) : 0.f;
        vs[r * P + i] = live ? sb_ld(v + base + idx) : 0.f;
        ds[r * P + i] = live ? sb_ld(dout + base + idx) : 0.f;
    }
    if (tid < SB_C) las[tid] = t0 + tid < T ? la[(size_t)bh * T + t0 + tid] : 0.f;
    __syncthreads();
    if (tid < SB_C) {
        float s = 0.f;
        for (int i = 0; i <= tid; ++i) s += las[i];
        L[tid] = s; eL[tid] = expf(s);
    }
    __syncthreads();
    {   // the three 64 x 64 matrices: thread (t, 16 consecutive s)
        const int t = tid >> 2, s0 = (tid & 3) * 16;
        for (int s = s0; s < s0 + 16; ++s) {
            float a = 0.f, dp = 0.f, g = 0.f;
            if (s <= t) {
                float p = 0.f, da = 0.f;
                for (int i = 0; i < D; ++i) { p = fmaf(qs[t * P + i], ks[s * P + i], p); da = fmaf(ds[t * P + i], vs[s * P + i], da); }
                const float dec = expf(fminf(L[t] - L[s], 0.f));
                a = p * dec; dp = da * dec; g = da * a;
            }
            A[t * MP + s] = a; dP[t * MP + s] = dp; Gm[t * MP + s] = g;
        }
    }
    // R[t][i] = sum_j do[t][j] S[i][j]: thread (i, a group of token rows)
    constexpr int NG = SB_NT / D, NT = SB_C / NG;
    const int col = tid % D, grp = tid / D;
    const __nv_bfloat16 *Sc = sent + ((size_t)bh * NC + c) * D * D;
    {
        float acc[NT];
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) acc[tt] = 0.f;
        for (int j = 0; j < D; ++j) {
            const float sv = __bfloat162float(Sc[(size_t)col * D + j]);
#pragma unroll
            for (int tt = 0; tt < NT; ++tt) acc[tt] = fmaf(ds[(grp * NT + tt) * P + j], sv, acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) R[(grp * NT + tt) * P + col] = acc[tt];
    }
    __syncthreads();
    // dv[s][j] = sum_t A[t][s] do[t][j];  dk[s][i] = sum_t dP[t][s] q[t][i];  dq[t][i] = sum_s dP[t][s] k[s][i] + e^{L_t} R[t][i]
    {
        float av[NT], ak[NT], aq[NT];
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) { av[tt] = 0.f; ak[tt] = 0.f; aq[tt] = 0.f; }
        for (int u = 0; u < SB_C; ++u) {
            const float dv_u = ds[u * P + col], q_u = qs[u * P + col], k_u = ks[u * P + col];
#pragma unroll
            for (int tt = 0; tt < NT; ++tt) {
                const int r = grp * NT + tt;
                av[tt] = fmaf(A[u * MP + r], dv_u, av[tt]);           // u runs over t, r is s
                ak[tt] = fmaf(dP[u * MP + r], q_u, ak[tt]);
                aq[tt] = fmaf(dP[r * MP + u], k_u, aq[tt]);           // u runs over s, r is t
            }
        }
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) {
            const int r = grp * NT + tt;
            if (t0 + r < T) {
                dv[base + (size_t)r * D + col] = av[tt];
                dk[base + (size_t)r * D + col] = ak[tt];
                dq[base + (size_t)r * D + col] = fmaf(eL[r], R[r * P + col], aq[tt]);
            }
        }
    }
    // dS[i][j] = sum_t e^{L_t} q[t][i] do[t][j]: thread (j, a group of rows i)
    {
        constexpr int NI = D / NG;
        float *dst = dsent + ((size_t)bh * NC + c) * D * D;
        for (int ii = 0; ii < NI; ++ii) {
            const int i = grp * NI + ii;
            float acc = 0.f;
            for (int t = 0; t < SB_C; ++t) acc = fmaf(eL[t] * qs[t * P + i], ds[t * P + col], acc);
            dst[(size_t)i * D + col] = acc;
        }
    }
    // dL, then dla as its reverse cumulative sum
    if (tid < SB_C) {
        const int t = tid;
        float s = 0.f;
        for (int u = 0; u < SB_C; ++u) s += Gm[t * MP + u] - Gm[u * MP + t];
        float r = 0.f;
        for (int i = 0; i < D; ++i) r = fmaf(qs[t * P + i], R[t * P + i], r);
        dL[t] = fmaf(eL[t], r, s);
    }
    __syncthreads();
    if (tid < SB_C && t0 + tid < T) {
        float s = 0.f;
        for (int u = SB_C - 1; u >= tid; --u) s += dL[u];
        dla[(size_t)bh * T + t0 + tid] = s;
    }
}

// ---------------------------------------------------------------------------------------------------- prefix_scan backward
template <typename TIO, int D>
__global__ void __launch_bounds__(SB_NT) prefix_scan_bwd_kernel(const TIO *__restrict__ k, const TIO *__restrict__ v, const float *__restrict__ w,
                                                                const float *__restrict__ a_log, const __nv_bfloat16 *__restrict__ sent,
                                                                const float *__restrict__ dsent, const float *__restrict__ dsfin,
                                                                float *__restrict__ dk, float *__restrict__ dv, float *__restrict__ dw,
                                                                float *__restrict__ da_log, float *__restrict__ dS0, int NC) {
    constexpr int P = D + 1, NG = SB_NT / D, NT = SB_C / NG;
    extern __shared__ float sb_smem[];
    float *G = sb_smem, *ks = G + D * P, *vs = ks + SB_C * P, *T1 = vs + SB_C * P, *ws = T1 + SB_C * P, *red = ws + SB_C;
    const int tid = threadIdx.x, bh = blockIdx.x, col = tid % D, grp = tid / D, lane = tid & 31, warp = tid >> 5;
    for (int idx = tid; idx < D * D; idx += SB_NT)
        G[(idx / D) * P + idx % D] = dsfin != nullptr ? dsfin[(size_t)bh * D * D + idx] : 0.f;
    for (int c = NC - 1; c >= 0; --c) {
        const size_t base = ((size_t)bh * NC + c) * SB_C * D;
        __syncthreads();
        for (int idx = tid; idx < SB_C * D; idx += SB_NT) {
            ks[(idx / D) * P + idx % D] = sb_ld(k + base + idx);
            vs[(idx / D) * P + idx % D] = sb_ld(v + base + idx);
        }
        if (tid < SB_C) ws[tid] = w[((size_t)bh * NC + c) * SB_C + tid];
        __syncthreads();
        // g[s][i] = sum_j G[i][j] v[s][j] (thread: i = col);  dk = w g;  T1 = k g (summed over i below for dw)
        // dv[s][j] = w_s sum_i k[s][i] G[i][j] (thread: j = col)
        {
            float ag[NT], avv[NT];
#pragma unroll
            for (int tt = 0; tt < NT; ++tt) { ag[tt] = 0.f; avv[tt] = 0.f; }
            for (int u = 0; u < D; ++u) {
                const float g_iu = G[col * P + u], g_ui = G[u * P + col];
#pragma unroll
                for (int tt = 0; tt < NT; ++tt) {
                    const int s = grp * NT + tt;
                    ag[tt] = fmaf(g_iu, vs[s * P + u], ag[tt]);
                    avv[tt] = fmaf(ks[s * P + u], g_ui, avv[tt]);
                }
            }
#pragma unroll
            for (int tt = 0; tt < NT; ++tt) {
                const int s = grp * NT + tt;
                dk[base + (size_t)s * D + col] = ws[s] * ag[tt];
                dv[base + (size_t)s * D + col] = ws[s] * avv[tt];
                T1[s * P + col] = ks[s * P + col] * ag[tt];
            }
        }
        // da_c = e^{a_c} <G, S_c>, summed in a fixed order: thread partial, warp, then the eight warps
        const float a = expf(a_log[(size_t)bh * NC + c]);
        const __nv_bfloat16 *Sc = sent + ((size_t)bh * NC + c) * D * D;
        float part = 0.f;
        for (int idx = tid; idx < D * D; idx += SB_NT) part = fmaf(G[(idx / D) * P + idx % D], __bfloat162float(Sc[idx]), part);
        part = warp_sum(part);
        if (lane == 0) red[warp] = part;
        __syncthreads();
        if (tid < SB_C) {
            float s = 0.f;
            for (int i = 0; i < D; ++i) s += T1[tid * P + i];
            dw[((size_t)bh * NC + c) * SB_C + tid] = s;
        }
        if (tid == 0) {
            float s = 0.f;
            for (int i = 0; i < SB_NT / 32; ++i) s += red[i];
            da_log[(size_t)bh * NC + c] = a * s;
        }
        // G <- e^{a_c} G + dsent[c]
        const float *dsc = dsent != nullptr ? dsent + ((size_t)bh * NC + c) * D * D : nullptr;
        for (int idx = tid; idx < D * D; idx += SB_NT) {
            float *g = &G[(idx / D) * P + idx % D];
            *g = fmaf(a, *g, dsc != nullptr ? dsc[idx] : 0.f);
        }
    }
    __syncthreads();
    if (dS0 != nullptr)
        for (int idx = tid; idx < D * D; idx += SB_NT) dS0[(size_t)bh * D * D + idx] = G[(idx / D) * P + idx % D];
}

// ---------------------------------------------------------------------------------------------------- host side
template <typename K>
static int sb_attr(K kern, size_t smem, const char *what) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e, what); return PGB_ERR_CUDA; }
    return PGB_OK;
}

template <typename TIO, int D>
static int assoc_out_bwd_go(const void *q, const void *k, const void *v, const float *la, const void *sent, const void *dout, float *dq,
                            float *dk, float *dv, float *dla, float *dsent, int BH, int T, cudaStream_t st) {
    const int NC = (T + SB_C - 1) / SB_C;
    const size_t smem = (size_t)(5 * SB_C * (D + 1) + 3 * SB_C * (SB_C + 1) + 4 * SB_C) * sizeof(float);
    int rc = sb_attr(assoc_out_bwd_kernel<TIO, D>, smem, "assoc_out_bwd smem attribute");
    if (rc != PGB_OK) return rc;
    assoc_out_bwd_kernel<TIO, D><<<dim3(NC, BH), SB_NT, smem, st>>>((const TIO *)q, (const TIO *)k, (const TIO *)v, la,
                                                                   (const __nv_bfloat16 *)sent, (const TIO *)dout, dq, dk, dv, dla, dsent, T, NC);
    return check_launch("assoc_out_bwd_kernel");
}

int assoc_out_bwd_launch(const void *q, const void *k, const void *v, int io_dtype, const float *la, const void *sent, const void *dout,
                         float *dq, float *dk, float *dv, float *dla, float *dsent, int BH, int T, int D, cudaStream_t st) {
    if (io_dtype == PGB_BF16)
        return D == 64 ? assoc_out_bwd_go<__nv_bfloat16, 64>(q, k, v, la, sent, dout, dq, dk, dv, dla, dsent, BH, T, st)
                       : assoc_out_bwd_go<__nv_bfloat16, 128>(q, k, v, la, sent, dout, dq, dk, dv, dla, dsent, BH, T, st);
    return D == 64 ? assoc_out_bwd_go<float, 64>(q, k, v, la, sent, dout, dq, dk, dv, dla, dsent, BH, T, st)
                   : assoc_out_bwd_go<float, 128>(q, k, v, la, sent, dout, dq, dk, dv, dla, dsent, BH, T, st);
}

template <typename TIO, int D>
static int prefix_scan_bwd_go(const void *k, const void *v, const float *w, const float *a_log, const void *sent, const float *dsent,
                              const float *dsfin, float *dk, float *dv, float *dw, float *da_log, float *dS0, int BH, int NC,
                              cudaStream_t st) {
    const size_t smem = (size_t)(D * (D + 1) + 3 * SB_C * (D + 1) + SB_C + 8) * sizeof(float);
    int rc = sb_attr(prefix_scan_bwd_kernel<TIO, D>, smem, "prefix_scan_bwd smem attribute");
    if (rc != PGB_OK) return rc;
    prefix_scan_bwd_kernel<TIO, D><<<dim3(BH), SB_NT, smem, st>>>((const TIO *)k, (const TIO *)v, w, a_log, (const __nv_bfloat16 *)sent, dsent,
                                                                 dsfin, dk, dv, dw, da_log, dS0, NC);
    return check_launch("prefix_scan_bwd_kernel");
}

int prefix_scan_bwd_launch(const void *k, const void *v, int io_dtype, const float *w, const float *a_log, const void *sent,
                           const float *dsent, const float *dsfin, float *dk, float *dv, float *dw, float *da_log, float *dS0, int BH,
                           int NC, int D, cudaStream_t st) {
    if (io_dtype == PGB_BF16)
        return D == 64 ? prefix_scan_bwd_go<__nv_bfloat16, 64>(k, v, w, a_log, sent, dsent, dsfin, dk, dv, dw, da_log, dS0, BH, NC, st)
                       : prefix_scan_bwd_go<__nv_bfloat16, 128>(k, v, w, a_log, sent, dsent, dsfin, dk, dv, dw, da_log, dS0, BH, NC, st);
    return D == 64 ? prefix_scan_bwd_go<float, 64>(k, v, w, a_log, sent, dsent, dsfin, dk, dv, dw, da_log, dS0, BH, NC, st)
                   : prefix_scan_bwd_go<float, 128>(k, v, w, a_log, sent, dsent, dsfin, dk, dv, dw, da_log, dS0, BH, NC, st);
}

}  // namespace pgb
