// Backward of the split operators (the reference's _bwd_chunk, src/assoc_kernel.py:75-126, _prefix_bwd, :206-221,
// _delta_loop_bwd, :390-459, and _inv_bwd, :626-656, with their register_autograd wiring at :179, :299, :509, :704), so that
// code written against membrae::assoc_out / prefix_scan / delta_loop_fwd / delta_inv can train through this library.
// Like the forward kernels in split_ops.cu these are plain fp32 FFMA kernels built for exactness, not speed; every gradient leaves in fp32 and every sum is taken
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

// ---------------------------------------------------------------------------------------------------- delta_inv backward
// X = (I + N)^-1,  N[t][s] = beta_t (k_t.k_s) e^{L_t-L_s} for s < t.   dN = -X^T dX X^T restricted to s < t, then
//   dbeta_t = sum_s dN (k_t.k_s) dec;   dk_t = sum_s c[t][s] k_s + sum_t' c[t'][t] k_t'  with c = dN beta dec;
//   dL_t = sum_s dN N [t,s] - sum_t' dN N [t',t];   dla = reverse cumulative sum of dL.
// (the reference's _inv_bwd, src/assoc_kernel.py:626-656, wired at :704)
template <typename TIO, int D>
__global__ void __launch_bounds__(SB_NT) delta_inv_bwd_kernel(const TIO *__restrict__ k, const float *__restrict__ la, const float *__restrict__ be,
                                                              const __nv_bfloat16 *__restrict__ X, const float *__restrict__ dX,
                                                              float *__restrict__ dk, float *__restrict__ dla, float *__restrict__ dbe,
                                                              int T, int NC) {
    constexpr int P = D + 1, MP = SB_C + 1;
    extern __shared__ float sb_smem[];
    float *ks = sb_smem, *Xs = ks + SB_C * P, *M1 = Xs + SB_C * MP, *M2 = M1 + SB_C * MP, *M3 = M2 + SB_C * MP, *las = M3 + SB_C * MP,
          *L = las + SB_C, *bes = L + SB_C, *dL = bes + SB_C;
    const int tid = threadIdx.x, c = blockIdx.x, bh = blockIdx.y, t0 = c * SB_C;
    const size_t base = ((size_t)bh * T + t0) * D, xb = ((size_t)bh * NC + c) * SB_C * SB_C;
    for (int idx = tid; idx < SB_C * D; idx += SB_NT) ks[(idx / D) * P + idx % D] = t0 + idx / D < T ? sb_ld(k + base + idx) : 0.f;
    for (int idx = tid; idx < SB_C * SB_C; idx += SB_NT) {
        Xs[(idx / SB_C) * MP + idx % SB_C] = __bfloat162float(X[xb + idx]);
        M1[(idx / SB_C) * MP + idx % SB_C] = dX[xb + idx];                       // M1 = dX
    }
    if (tid < SB_C) {
        las[tid] = t0 + tid < T ? la[(size_t)bh * T + t0 + tid] : 0.f;
        bes[tid] = t0 + tid < T ? be[(size_t)bh * T + t0 + tid] : 0.f;
    }
    __syncthreads();
    if (tid < SB_C) {
        float s = 0.f;
        for (int i = 0; i <= tid; ++i) s += las[i];
        L[tid] = s;
    }
    const int r = tid >> 2, c0 = (tid & 3) * 16;                      // thread (row, 16 consecutive columns) of a 64 x 64 matrix
    for (int b = c0; b < c0 + 16; ++b) {                              // M2 = X^T dX
        float acc = 0.f;
        for (int t = 0; t < SB_C; ++t) acc = fmaf(Xs[t * MP + r], M1[t * MP + b], acc);
        M2[r * MP + b] = acc;
    }
    __syncthreads();
    for (int b = c0; b < c0 + 16; ++b) {                              // M3 = dN = -(X^T dX) X^T, strictly lower
        float acc = 0.f;
        if (b < r)
            for (int u = 0; u < SB_C; ++u) acc = fmaf(M2[r * MP + u], Xs[b * MP + u], acc);
        M3[r * MP + b] = -acc;
    }
    __syncthreads();
    for (int b = c0; b < c0 + 16; ++b) {                              // M1 = c (dk coefficient), M2 = dN N, Xs = dN (k.k) dec
        float cc = 0.f, g = 0.f, nb = 0.f;
        if (b < r) {
            float kk = 0.f;
            for (int i = 0; i < D; ++i) kk = fmaf(ks[r * P + i], ks[b * P + i], kk);
            const float dec = expf(fminf(L[r] - L[b], 0.f)), dn = M3[r * MP + b];
            nb = dn * kk * dec; cc = dn * bes[r] * dec; g = nb * bes[r];
        }
        M1[r * MP + b] = cc; M2[r * MP + b] = g; Xs[r * MP + b] = nb;
    }
    __syncthreads();
    {   // dk[t][i] = sum_s c[t][s] k[s][i] + sum_t' c[t'][t] k[t'][i]
        constexpr int NG = SB_NT / D, NT = SB_C / NG;
        const int col = tid % D, grp = tid / D;
        float acc[NT];
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) acc[tt] = 0.f;
        for (int u = 0; u < SB_C; ++u) {
            const float ku = ks[u * P + col];
#pragma unroll
            for (int tt = 0; tt < NT; ++tt) {
                const int t = grp * NT + tt;
                acc[tt] = fmaf(M1[t * MP + u] + M1[u * MP + t], ku, acc[tt]);
            }
        }
#pragma unroll
        for (int tt = 0; tt < NT; ++tt)
            if (t0 + grp * NT + tt < T) dk[base + (size_t)(grp * NT + tt) * D + col] = acc[tt];
    }
    if (tid < SB_C) {
        float s = 0.f, b = 0.f;
        for (int u = 0; u < SB_C; ++u) { s += M2[tid * MP + u] - M2[u * MP + tid]; b += Xs[tid * MP + u]; }
        dL[tid] = s;
        if (t0 + tid < T) dbe[(size_t)bh * T + t0 + tid] = b;
    }
    __syncthreads();
    if (tid < SB_C && t0 + tid < T) {
        float s = 0.f;
        for (int u = SB_C - 1; u >= tid; --u) s += dL[u];
        dla[(size_t)bh * T + t0 + tid] = s;
    }
}

// ---------------------------------------------------------------------------------------------------- delta_loop backward
// Forward per chunk:  rhs = beta (v - e^L (k S));  W = X rhs;  S' = e^{L_C} S + (k w)^T W,  w_s = e^{L_C - L_s}.
// One CTA per (sequence-head, 64 value columns) walks the chunks backwards with G = dLoss/dS' (its columns) in shared
// memory. Sums over value columns (dk, dla, dbeta, dX) leave as one partial per column slab; the caller adds the slabs.
// (the reference's _delta_loop_bwd, src/assoc_kernel.py:390-459, wired at :509)
template <typename TIO, int D>
__global__ void __launch_bounds__(SB_NT) delta_loop_bwd_kernel(const TIO *__restrict__ k, const TIO *__restrict__ v, const float *__restrict__ la,
                                                               const float *__restrict__ be, const __nv_bfloat16 *__restrict__ X,
                                                               const __nv_bfloat16 *__restrict__ sent, const float *__restrict__ dW,
                                                               const float *__restrict__ dsent, const float *__restrict__ dsfin,
                                                               float *__restrict__ dk_part, float *__restrict__ dv, float *__restrict__ dla_part,
                                                               float *__restrict__ dbe_part, float *__restrict__ dX_part, float *__restrict__ dS0,
                                                               int BH, int T, int NC) {
    constexpr int P = D + 1, MP = SB_C + 1, SL = 64;                  // SL: value columns of this CTA
    extern __shared__ float sb_smem[];
    float *G = sb_smem, *S = G + D * MP, *ks = S + D * MP, *Xs = ks + SB_C * P, *RH = Xs + SB_C * MP, *Wm = RH + SB_C * MP,
          *KS = Wm + SB_C * MP, *KG = KS + SB_C * MP, *DW = KG + SB_C * MP, *DR = DW + SB_C * MP, *las = DR + SB_C * MP, *L = las + SB_C,
          *eL = L + SB_C, *wt = eL + SB_C, *bes = wt + SB_C, *dwv = bes + SB_C, *dLa = dwv + SB_C, *red = dLa + SB_C;
    const int tid = threadIdx.x, slab = blockIdx.x, bh = blockIdx.y, j0 = slab * SL, lane = tid & 31, warp = tid >> 5;
    const int r = tid >> 2, c0 = (tid & 3) * 16;                      // (token row, 16 slab columns)
    constexpr int NG = SB_NT / D, NT = SB_C / NG;                     // (state row / k column i, group of token rows)
    const int col = tid % D, grp = tid / D;
    const size_t part = (size_t)slab * BH + bh;
    for (int idx = tid; idx < D * SL; idx += SB_NT) {
        const int i = idx / SL, j = idx % SL;
        G[i * MP + j] = dsfin != nullptr ? dsfin[((size_t)bh * D + i) * D + j0 + j] : 0.f;
    }
    for (int c = NC - 1; c >= 0; --c) {
        const int t0 = c * SB_C;
        const size_t base = ((size_t)bh * T + t0) * D, xb = ((size_t)bh * NC + c) * SB_C * SB_C, sb = ((size_t)bh * NC + c) * D * D;
        __syncthreads();
        for (int idx = tid; idx < SB_C * D; idx += SB_NT) ks[(idx / D) * P + idx % D] = t0 + idx / D < T ? sb_ld(k + base + idx) : 0.f;
        for (int idx = tid; idx < SB_C * SB_C; idx += SB_NT) Xs[(idx / SB_C) * MP + idx % SB_C] = __bfloat162float(X[xb + idx]);
        for (int idx = tid; idx < D * SL; idx += SB_NT) S[(idx / SL) * MP + idx % SL] = __bfloat162float(sent[sb + (size_t)(idx / SL) * D + j0 + idx % SL]);
        for (int idx = tid; idx < SB_C * SL; idx += SB_NT) {
            const int t = idx / SL, j = idx % SL;
            const bool live = t0 + t < T;
            RH[t * MP + j] = live ? sb_ld(v + base + (size_t)t * D + j0 + j) : 0.f;                 // v for now
            DW[t * MP + j] = (live && dW != nullptr) ? dW[base + (size_t)t * D + j0 + j] : 0.f;
        }
        if (tid < SB_C) {
            las[tid] = t0 + tid < T ? la[(size_t)bh * T + t0 + tid] : 0.f;
            bes[tid] = t0 + tid < T ? be[(size_t)bh * T + t0 + tid] : 0.f;
        }
        __syncthreads();
        if (tid < SB_C) {
            float s = 0.f, tot = 0.f;
            for (int i = 0; i < SB_C; ++i) { tot += las[i]; if (i <= tid) s += las[i]; }
            L[tid] = s; eL[tid] = expf(s);
            wt[tid] = t0 + tid < T ? expf(fminf(tot - s, 0.f)) : 0.f;
        }
        __syncthreads();
        // 1. KS = k S;  KG = k G;  rhs = beta (v - e^L KS)
        for (int j = c0; j < c0 + 16; ++j) {
            float a = 0.f, g = 0.f;
            for (int i = 0; i < D; ++i) { a = fmaf(ks[r * P + i], S[i * MP + j], a); g = fmaf(ks[r * P + i], G[i * MP + j], g); }
            KS[r * MP + j] = a; KG[r * MP + j] = g;
            RH[r * MP + j] = bes[r] * (RH[r * MP + j] - eL[r] * a);
        }
        __syncthreads();
        // 2. W = X rhs;  dWtot = dW + w (k G)
        for (int j = c0; j < c0 + 16; ++j) {
            float a = 0.f;
            for (int s = 0; s <= r; ++s) a = fmaf(Xs[r * MP + s], RH[s * MP + j], a);
            Wm[r * MP + j] = a;
            DW[r * MP + j] = fmaf(wt[r], KG[r * MP + j], DW[r * MP + j]);
        }
        __syncthreads();
        // 3. drhs = X^T dWtot;  dX[t][s] = sum_j dWtot[t][j] rhs[s][j] (s <= t);  dw_s = sum_j W[s][j] KG[s][j]
        for (int j = c0; j < c0 + 16; ++j) {
            float a = 0.f;
            for (int t = r; t < SB_C; ++t) a = fmaf(Xs[t * MP + r], DW[t * MP + j], a);
            DR[r * MP + j] = a;
        }
        for (int s = c0; s < c0 + 16; ++s) {
            float a = 0.f;
            if (s <= r)
                for (int j = 0; j < SL; ++j) a = fmaf(DW[r * MP + j], RH[s * MP + j], a);
            dX_part[(part * NC + c) * SB_C * SB_C + (size_t)r * SB_C + s] = a;
        }
        if (tid < SB_C) {
            float a = 0.f;
            for (int j = 0; j < SL; ++j) a = fmaf(Wm[tid * MP + j], KG[tid * MP + j], a);
            dwv[tid] = a;
        }
        __syncthreads();
        // 4. dv = beta drhs;  dbeta_t = sum_j drhs (v - e^L KS);  dL_t (first part) = sum_j dKS KS with dKS = -beta e^L drhs
        if (tid < SB_C) {
            const int t = tid;
            const bool live = t0 + t < T;
            float db = 0.f, dl = 0.f;
            for (int j = 0; j < SL; ++j) {
                const float dr = DR[t * MP + j], ksv = KS[t * MP + j];
                dl = fmaf(-bes[t] * eL[t] * dr, ksv, dl);
                if (live) db = fmaf(dr, sb_ld(v + base + (size_t)t * D + j0 + j) - eL[t] * ksv, db);   // v again: its tile now holds rhs
            }
            dLa[t] = dl;
            if (live) dbe_part[part * T + t0 + t] = db;
        }
        for (int j = c0; j < c0 + 16; ++j)
            if (t0 + r < T) dv[base + (size_t)r * D + j0 + j] = bes[r] * DR[r * MP + j];
        __syncthreads();
        for (int j = c0; j < c0 + 16; ++j) DR[r * MP + j] *= -bes[r] * eL[r];                      // DR = dKS
        __syncthreads();
        // 5. dk[t][i] = w_t sum_j G[i][j] W[t][j] + sum_j dKS[t][j] S[i][j]   (this slab's part)
        {
            float acc[NT];
#pragma unroll
            for (int tt = 0; tt < NT; ++tt) acc[tt] = 0.f;
            for (int j = 0; j < SL; ++j) {
                const float gj = G[col * MP + j], sj = S[col * MP + j];
#pragma unroll
                for (int tt = 0; tt < NT; ++tt) {
                    const int t = grp * NT + tt;
                    acc[tt] = fmaf(wt[t] * gj, Wm[t * MP + j], acc[tt]);
                    acc[tt] = fmaf(DR[t * MP + j], sj, acc[tt]);
                }
            }
#pragma unroll
            for (int tt = 0; tt < NT; ++tt)
                if (t0 + grp * NT + tt < T) dk_part[(part * T + t0 + grp * NT + tt) * D + col] = acc[tt];
        }
        // 6. <G, S> for dL_C, summed in a fixed order
        const float LC = L[SB_C - 1], aC = expf(LC);
        float pr = 0.f;
        for (int idx = tid; idx < D * SL; idx += SB_NT) pr = fmaf(G[(idx / SL) * MP + idx % SL], S[(idx / SL) * MP + idx % SL], pr);
        pr = warp_sum(pr);
        if (lane == 0) red[warp] = pr;
        __syncthreads();
        // 7. dL and dla (this slab's part): dL_t = dL_t(a) - dw_t w_t, plus dL_C on the chunk's last step
        if (tid == 0) {
            float gs = 0.f;
            for (int i = 0; i < SB_NT / 32; ++i) gs += red[i];
            float dLC = aC * gs;
            for (int s = 0; s < SB_C; ++s) dLC = fmaf(dwv[s], wt[s], dLC);
            float run = 0.f;
            for (int t = SB_C - 1; t >= 0; --t) {
                run += dLa[t] - dwv[t] * wt[t] + (t == SB_C - 1 ? dLC : 0.f);
                if (t0 + t < T) dla_part[part * T + t0 + t] = run;
            }
        }
        // 8. G <- e^{L_C} G + k^T dKS + dsent[c]
        for (int idx = tid; idx < D * SL; idx += SB_NT) {
            const int i = idx / SL, j = idx % SL;
            float a = dsent != nullptr ? dsent[sb + (size_t)i * D + j0 + j] : 0.f;
            for (int t = 0; t < SB_C; ++t) a = fmaf(ks[t * P + i], DR[t * MP + j], a);
            G[i * MP + j] = fmaf(aC, G[i * MP + j], a);
        }
    }
    __syncthreads();
    if (dS0 != nullptr)
        for (int idx = tid; idx < D * SL; idx += SB_NT) dS0[((size_t)bh * D + idx / SL) * D + j0 + idx % SL] = G[(idx / SL) * MP + idx % SL];
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

template <typename TIO, int D>
static int delta_inv_bwd_go(const void *k, const float *la, const float *be, const void *X, const float *dX, float *dk, float *dla, float *dbe,
                            int BH, int T, cudaStream_t st) {
    const int NC = (T + SB_C - 1) / SB_C;
    const size_t smem = (size_t)(SB_C * (D + 1) + 4 * SB_C * (SB_C + 1) + 4 * SB_C) * sizeof(float);
    int rc = sb_attr(delta_inv_bwd_kernel<TIO, D>, smem, "delta_inv_bwd smem attribute");
    if (rc != PGB_OK) return rc;
    delta_inv_bwd_kernel<TIO, D><<<dim3(NC, BH), SB_NT, smem, st>>>((const TIO *)k, la, be, (const __nv_bfloat16 *)X, dX, dk, dla, dbe, T, NC);
    return check_launch("delta_inv_bwd_kernel");
}

int delta_inv_bwd_launch(const void *k, int io_dtype, const float *la, const float *be, const void *X, const float *dX, float *dk, float *dla,
                         float *dbe, int BH, int T, int D, cudaStream_t st) {
    if (io_dtype == PGB_BF16)
        return D == 64 ? delta_inv_bwd_go<__nv_bfloat16, 64>(k, la, be, X, dX, dk, dla, dbe, BH, T, st)
                       : delta_inv_bwd_go<__nv_bfloat16, 128>(k, la, be, X, dX, dk, dla, dbe, BH, T, st);
    return D == 64 ? delta_inv_bwd_go<float, 64>(k, la, be, X, dX, dk, dla, dbe, BH, T, st)
                   : delta_inv_bwd_go<float, 128>(k, la, be, X, dX, dk, dla, dbe, BH, T, st);
}

template <typename TIO, int D>
static int delta_loop_bwd_go(const void *k, const void *v, const float *la, const float *be, const void *X, const void *sent, const float *dW,
                             const float *dsent, const float *dsfin, float *dk_part, float *dv, float *dla_part, float *dbe_part,
                             float *dX_part, float *dS0, int BH, int T, cudaStream_t st) {
    const int NC = (T + SB_C - 1) / SB_C;
    const size_t smem = (size_t)(2 * D * (SB_C + 1) + SB_C * (D + 1) + 7 * SB_C * (SB_C + 1) + 7 * SB_C + 8) * sizeof(float);
    int rc = sb_attr(delta_loop_bwd_kernel<TIO, D>, smem, "delta_loop_bwd smem attribute");
    if (rc != PGB_OK) return rc;
    delta_loop_bwd_kernel<TIO, D><<<dim3(D / 64, BH), SB_NT, smem, st>>>((const TIO *)k, (const TIO *)v, la, be, (const __nv_bfloat16 *)X,
                                                                       (const __nv_bfloat16 *)sent, dW, dsent, dsfin, dk_part, dv, dla_part,
                                                                       dbe_part, dX_part, dS0, BH, T, NC);
    return check_launch("delta_loop_bwd_kernel");
}

int delta_loop_bwd_launch(const void *k, const void *v, int io_dtype, const float *la, const float *be, const void *X, const void *sent,
                          const float *dW, const float *dsent, const float *dsfin, float *dk_part, float *dv, float *dla_part,
                          float *dbe_part, float *dX_part, float *dS0, int BH, int T, int D, cudaStream_t st) {
    if (io_dtype == PGB_BF16)
        return D == 64 ? delta_loop_bwd_go<__nv_bfloat16, 64>(k, v, la, be, X, sent, dW, dsent, dsfin, dk_part, dv, dla_part, dbe_part, dX_part, dS0, BH, T, st)
                       : delta_loop_bwd_go<__nv_bfloat16, 128>(k, v, la, be, X, sent, dW, dsent, dsfin, dk_part, dv, dla_part, dbe_part, dX_part, dS0, BH, T, st);
    return D == 64 ? delta_loop_bwd_go<float, 64>(k, v, la, be, X, sent, dW, dsent, dsfin, dk_part, dv, dla_part, dbe_part, dX_part, dS0, BH, T, st)
                   : delta_loop_bwd_go<float, 128>(k, v, la, be, X, sent, dW, dsent, dsfin, dk_part, dv, dla_part, dbe_part, dX_part, dS0, BH, T, st);
}

}  // namespace pgb
