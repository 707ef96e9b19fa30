// Chunked prefill of the associative carrier in full fp32 (FFMA): the precise mode.
//
// One CTA walks the 64-token chunks of one (sequence, head) for a slice of BV value columns; the state slice
// S[D][BV] lives in shared memory in fp32 for the whole sequence, so HBM sees q, k, v, o once (k and q once per
// slice) and the state only at the ends (plus the optional per-chunk entering states).
// Per chunk (reference src/assoc.py:118-165 plain, :207-251 delta; same masking as src/assoc_kernel.py:55-70):
//   L = cumsum(la) (left to right, fp32);  dec[t][s] = exp(min(L_t-L_s,0)) for s<=t
//   A = (Q K^T) * dec
//   delta only:  N = beta_t * (K K^T) * dec strictly lower;  rhs = beta_t (V - e^{L_t} K S);  W = (I+N)^-1 rhs by
//                blocked forward substitution (16-row blocks; inside a block one thread per column walks the rows)
//   plain:       W = V
//   O = A W + e^{L_t} (Q S);   S <- e^{L_C} S + (K * e^{L_C-L_s})^T W
// Rows past T are zero tokens with log-decay 0 and beta 0, as the reference pads.
#include "common.cuh"

namespace pgb {

constexpr int PF_C = 64;
constexpr int PF_THREADS = 256;


// acc[i][j] += sum_k A(m = ty+16i, k) * B(k, n = tx+16j).  AT: A stored [k][m]; BT: B stored [n][k].
template <int MI, int NJ, bool AT, bool BT>
__device__ __forceinline__ void mm_acc(float (&acc)[MI][NJ], const float *__restrict__ A, int lda,
                                       const float *__restrict__ B, int ldb, int ty, int tx, int k0, int k1) {
#pragma unroll 4
    for (int k = k0; k < k1; ++k) {
        float a[MI], bb[NJ];
#pragma unroll
        for (int i = 0; i < MI; ++i) a[i] = AT ? A[k * lda + ty + 16 * i] : A[(ty + 16 * i) * lda + k];
#pragma unroll
        for (int j = 0; j < NJ; ++j) bb[j] = BT ? B[(tx + 16 * j) * ldb + k] : B[k * ldb + tx + 16 * j];
#pragma unroll
        for (int i = 0; i < MI; ++i)
#pragma unroll
            for (int j = 0; j < NJ; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
}

template <int D, int BV, bool DELTA>
struct PfSmem {
    static constexpr int PD = D + 1, PV = BV + 1, PC = PF_C + 1;
    static constexpr int off_q = 0;
    static constexpr int off_k = off_q + PF_C * PD;
    static constexpr int off_v = off_k + PF_C * PD;
    static constexpr int off_s = off_v + PF_C * PV;
    static constexpr int off_a = off_s + D * PV;
    static constexpr int off_n = off_a + PF_C * PC;
    static constexpr int off_w = off_n + (DELTA ? PF_C * PC : 0);
    static constexpr int off_vec = off_w + (DELTA ? PF_C * PV : 0);
    static constexpr int floats = off_vec + 5 * PF_C;
    static constexpr size_t bytes = (size_t)floats * sizeof(float);
};

template <typename TIO, typename TOUT, int D, int BV, bool DELTA>
__global__ void __launch_bounds__(PF_THREADS) prefill_fp32_kernel(PrefillArgs a) {
    using SM = PfSmem<D, BV, DELTA>;
    constexpr int PD = SM::PD, PV = SM::PV, PC = SM::PC;
    constexpr int MI_D = D / 16, NJ_V = BV / 16;
    extern __shared__ float smem[];
    float *Qs = smem + SM::off_q, *Ks = smem + SM::off_k, *Vs = smem + SM::off_v, *Ss = smem + SM::off_s;
    float *As = smem + SM::off_a, *Ns = smem + SM::off_n, *Ws = DELTA ? smem + SM::off_w : Vs;
    float *las = smem + SM::off_vec, *Ls = las + PF_C, *eLs = Ls + PF_C, *wts = eLs + PF_C, *bes = wts + PF_C;

    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int j0 = blockIdx.x * BV;
    const size_t bh = blockIdx.y;
    const int T = a.T;
    const int NC = (T + PF_C - 1) / PF_C;
    const TIO *q = (const TIO *)a.q + bh * T * D, *k = (const TIO *)a.k + bh * T * D, *v = (const TIO *)a.v + bh * T * D;
    TOUT *o = (TOUT *)a.o + bh * T * D;
    const float *la = a.la + bh * T;
    const float *beta = DELTA ? a.beta + bh * T : nullptr;

    {
        // entering state, with the key axis (row pairs 2i, 2i+1) rotated back by shift*theta when a rebase is asked for
        const float shift = a.theta == nullptr ? 0.f : (a.shift_dev != nullptr ? *a.shift_dev : a.shift_host);
        const int h = (int)(bh % a.H);
        for (int idx = tid; idx < (D / 2) * BV; idx += PF_THREADS) {
            const int i = idx / BV, j = idx % BV;
            float x0 = 0.f, x1 = 0.f;
            if (a.S0 != nullptr) {
                x0 = a.S0[(bh * D + 2 * i) * D + j0 + j];
                x1 = a.S0[(bh * D + 2 * i + 1) * D + j0 + j];
                if (shift != 0.f) {
                    float sn, cs;
                    sincosf(-shift * a.theta[(size_t)h * (D / 2) + i], &sn, &cs);
                    const float r0 = x0 * cs - x1 * sn, r1 = x0 * sn + x1 * cs;
                    x0 = r0; x1 = r1;
                }
            }
            Ss[(2 * i) * PV + j] = x0;
            Ss[(2 * i + 1) * PV + j] = x1;
        }
    }

    for (int c = 0; c < NC; ++c) {
        const int t0 = c * PF_C;
        __syncthreads();                                               // previous chunk done with every buffer
        // ---- load the chunk (zero rows past T); the entering state goes out if asked for
        for (int idx = tid; idx < PF_C * D; idx += PF_THREADS) {
            const int r = idx / D, d = idx % D;
            const bool ok = t0 + r < T;
            Qs[r * PD + d] = ok ? to_f32(q[(size_t)(t0 + r) * D + d]) : 0.f;
            Ks[r * PD + d] = ok ? to_f32(k[(size_t)(t0 + r) * D + d]) : 0.f;
        }
        for (int idx = tid; idx < PF_C * BV; idx += PF_THREADS) {
            const int r = idx / BV, j = idx % BV;
            Vs[r * PV + j] = (t0 + r < T) ? to_f32(v[(size_t)(t0 + r) * D + j0 + j]) : 0.f;
        }
        if (a.sent != nullptr) {
            __nv_bfloat16 *dst = a.sent + ((bh * NC + c) * D) * D;
            for (int idx = tid; idx < D * BV; idx += PF_THREADS) {
                const int d = idx / BV, j = idx % BV;
                dst[(size_t)d * D + j0 + j] = __float2bfloat16_rn(Ss[d * PV + j]);
            }
        }
        if (tid < PF_C) {
            const bool ok = t0 + tid < T;
            las[tid] = ok ? la[t0 + tid] : 0.f;
            bes[tid] = (DELTA && ok) ? beta[t0 + tid] : 0.f;
        }
        __syncthreads();
        if (tid < PF_C) {
            float L = 0.f;
            for (int r = 0; r <= tid; ++r) L += las[r];                // left-to-right, as a cumulative sum does
            Ls[tid] = L;
            eLs[tid] = expf(L);
        }
        __syncthreads();
        if (tid < PF_C) wts[tid] = expf(fminf(Ls[PF_C - 1] - Ls[tid], 0.f));
        // ---- scores: A = (Q K^T) dec ; N = beta (K K^T) dec, strictly lower
        {
            float pa[4][4] = {}, pn[4][4] = {};
#pragma unroll 2
            for (int d = 0; d < D; ++d) {
                float aq[4], ak[4], bk[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) { aq[i] = Qs[(ty + 16 * i) * PD + d]; ak[i] = DELTA ? Ks[(ty + 16 * i) * PD + d] : 0.f; }
#pragma unroll
                for (int j = 0; j < 4; ++j) bk[j] = Ks[(tx + 16 * j) * PD + d];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        pa[i][j] = fmaf(aq[i], bk[j], pa[i][j]);
                        if (DELTA) pn[i][j] = fmaf(ak[i], bk[j], pn[i][j]);
                    }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int t = ty + 16 * i, s = tx + 16 * j;
                    const float dec = (s <= t) ? expf(fminf(Ls[t] - Ls[s], 0.f)) : 0.f;
                    As[t * PC + s] = pa[i][j] * dec;
                    if (DELTA) Ns[t * PC + s] = (s < t) ? bes[t] * pn[i][j] * dec : 0.f;
                }
        }
        __syncthreads();
        if constexpr (DELTA) {
            // ---- rhs = beta (V - e^L K S)
            {
                float ks[4][NJ_V] = {};
                mm_acc<4, NJ_V, false, false>(ks, Ks, PD, Ss, PV, ty, tx, 0, D);
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < NJ_V; ++j) {
                        const int t = ty + 16 * i, jj = tx + 16 * j;
                        Ws[t * PV + jj] = bes[t] * (Vs[t * PV + jj] - eLs[t] * ks[i][j]);
                    }
            }
            __syncthreads();
            // ---- W = (I + N)^-1 rhs, blocked forward substitution
            for (int blk = 0; blk < 4; ++blk) {
                const int r0 = 16 * blk;
                if (blk > 0) {
                    float up[1][NJ_V] = {};
                    // rows r0+ty: the helper's row index is ty + 16*i with i = 0, so shift A by r0 rows
                    mm_acc<1, NJ_V, false, false>(up, Ns + r0 * PC, PC, Ws, PV, ty, tx, 0, r0);
#pragma unroll
                    for (int j = 0; j < NJ_V; ++j) Ws[(r0 + ty) * PV + tx + 16 * j] -= up[0][j];
                    __syncthreads();
                }
                if (tid < BV) {
                    float wr[16];
#pragma unroll
                    for (int r = 0; r < 16; ++r) {
                        float x = Ws[(r0 + r) * PV + tid];
#pragma unroll
                        for (int s = 0; s < r; ++s) x = fmaf(-Ns[(r0 + r) * PC + r0 + s], wr[s], x);
                        wr[r] = x;
                        Ws[(r0 + r) * PV + tid] = x;
                    }
                }
                __syncthreads();
            }
        }
        // ---- output rows and the chunk's contribution to the state
        float upd[MI_D][NJ_V] = {};
        {
            float oi[4][NJ_V] = {}, oc[4][NJ_V] = {};
            mm_acc<4, NJ_V, false, false>(oi, As, PC, Ws, PV, ty, tx, 0, PF_C);
            mm_acc<4, NJ_V, false, false>(oc, Qs, PD, Ss, PV, ty, tx, 0, D);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int t = ty + 16 * i;
                if (t0 + t < T) {
#pragma unroll
                    for (int j = 0; j < NJ_V; ++j)
                        from_f32(o[(size_t)(t0 + t) * D + j0 + tx + 16 * j], oi[i][j] + eLs[t] * oc[i][j]);
                }
            }
            // (K * w)^T W: scale W's rows once through a register copy of w
#pragma unroll 4
            for (int s = 0; s < PF_C; ++s) {
                const float ws = wts[s];
                float ak[MI_D], bw[NJ_V];
#pragma unroll
                for (int i = 0; i < MI_D; ++i) ak[i] = Ks[s * PD + ty + 16 * i] * ws;
#pragma unroll
                for (int j = 0; j < NJ_V; ++j) bw[j] = Ws[s * PV + tx + 16 * j];
#pragma unroll
                for (int i = 0; i < MI_D; ++i)
#pragma unroll
                    for (int j = 0; j < NJ_V; ++j) upd[i][j] = fmaf(ak[i], bw[j], upd[i][j]);
            }
        }
        __syncthreads();                                               // every read of the entering state is done
        {
            const float aC = eLs[PF_C - 1];
#pragma unroll
            for (int i = 0; i < MI_D; ++i)
#pragma unroll
                for (int j = 0; j < NJ_V; ++j) {
                    float *p = &Ss[(ty + 16 * i) * PV + tx + 16 * j];
                    *p = aC * (*p) + upd[i][j];
                }
        }
    }
    __syncthreads();
    for (int idx = tid; idx < D * BV; idx += PF_THREADS) {
        const int d = idx / BV, j = idx % BV;
        a.S_out[(bh * D + d) * D + j0 + j] = Ss[d * PV + j];
    }
}

template <typename TIO, typename TOUT, int D, bool DELTA>
static int prefill_fp32_go(const PrefillArgs &a, cudaStream_t stream) {
    constexpr int BV = 64;
    using SM = PfSmem<D, BV, DELTA>;
    auto kern = prefill_fp32_kernel<TIO, TOUT, D, BV, DELTA>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SM::bytes);
    if (e != cudaSuccess) { set_cuda_error(e, "prefill_fp32 smem attribute"); return PGB_ERR_CUDA; }
    dim3 grid(D / BV, (unsigned)(a.B * a.H));
    kern<<<grid, PF_THREADS, SM::bytes, stream>>>(a);
    return check_launch("prefill_fp32_kernel");
}

template <typename TIO, typename TOUT>
static int prefill_fp32_io(const PrefillArgs &a, int D, cudaStream_t stream) {
    const bool delta = a.beta != nullptr;
    if (D == 64) return delta ? prefill_fp32_go<TIO, TOUT, 64, true>(a, stream) : prefill_fp32_go<TIO, TOUT, 64, false>(a, stream);
    return delta ? prefill_fp32_go<TIO, TOUT, 128, true>(a, stream) : prefill_fp32_go<TIO, TOUT, 128, false>(a, stream);
}

int prefill_fp32_launch(const PrefillArgs &a, int io_dtype, int o_dtype, int D, cudaStream_t stream) {
    if (io_dtype == PGB_F32)
        return o_dtype == PGB_F32 ? prefill_fp32_io<float, float>(a, D, stream) : prefill_fp32_io<float, __nv_bfloat16>(a, D, stream);
    return o_dtype == PGB_F32 ? prefill_fp32_io<__nv_bfloat16, float>(a, D, stream)
                              : prefill_fp32_io<__nv_bfloat16, __nv_bfloat16>(a, D, stream);
}

}  // namespace pgb
