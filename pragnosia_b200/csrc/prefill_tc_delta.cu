// Delta-rule chunked prefill on the tensor cores (tcgen05.mma, TMEM accumulators, TMA-fed tiles): two kernels.
//
// The delta rule writes v minus what the memory already returns for the key: S_t = a_t S_{t-1} + k_t [b_t (v_t - a_t S_{t-1}^T k_t)]^T.
// In a 64-token chunk the residuals actually written, W, solve (I + N) W = rhs with
//     N = diag(beta) strictly_lower((K K^T) * dec),   rhs = diag(beta) (V - e^{L} K S_entering),
// (reference src/assoc.py:207-251). N does not depend on the state, so
//
//   delta_inv_kernel   (chunk-parallel, one CTA per (sequence-head, chunk)): K K^T on the tensor core, N in fp32, then
//                      X = (I + N)^-1 by forward substitution in true fp32 FFMA -- one thread per column of X, every
//                      intermediate bounded (the reduced-precision Neumann doubling the reference warns about at
//                      src/assoc_kernel.py:577-582 is never formed). X goes to a scratch buffer as bf16 head + tail.
//   prefill_tc_delta_kernel (one CTA per (sequence-head, 64 value columns), walking the chunks): per chunk
//        P  = Q K^T,  KS = K S_c,  O2 = Q S_c                (state-dependent: KS, O2)
//        A  = P * dec ;  rhs = beta (V - e^{L_t} KS)          registers -> shared memory
//        W  = X rhs                                           the solve, as one product
//        O1 = A W,   U = (K w)^T W
//        o  = O1 + e^{L_t} O2 ;   S_{c+1} = e^{L_C} S_c + U   fp32 registers
//      Three tensor-core round trips per chunk are sequential (KS -> W -> U); everything fp32 that re-enters the tensor
//      core (S, rhs, X, A, W, K w) is split into bf16 head + tail and multiplied as head*head + head*tail + tail*head.
//
// Layouts and fragment geometry are those of prefill_tc.cu (128-byte swizzled tiles, M=64 accumulators read with
// 16x256b loads by 8 warps). Every mbarrier wait is bounded.
#include "tc_common.cuh"

namespace pgb {

constexpr int TD_NT = 256;
constexpr float TD_LOG2E = 1.4426950408889634f;

// decay statistics of one 64-token chunk by warps 0 and 1 (tid < 64): L (inclusive cumulative log-decay), e^L,
// w = e^{L_C - L} (0 past T) and beta (0 past T)
__device__ __forceinline__ void chunk_stats(const float *la, const float *beta, int t0, int T, int tid, int lane, int warp,
                                            float *Ls, float *eLs, float *wts, float *bes) {
    const int t = t0 + tid, tx = t0 + (tid ^ 32);
    const float own = t < T ? la[t] : 0.f, other = tx < T ? la[tx] : 0.f;
    float sc = own;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, sc, o);
        if (lane >= o) sc += n;
    }
    const float sum_other = warp_sum(other), sum_own = __shfl_sync(0xffffffffu, sc, 31);
    const float L = sc + (warp == 1 ? sum_other : 0.f), Ltot = sum_own + sum_other;
    Ls[tid] = L;
    if (eLs != nullptr) eLs[tid] = expf(L);
    if (wts != nullptr) wts[tid] = t < T ? expf(fminf(Ltot - L, 0.f)) : 0.f;
    bes[tid] = t < T ? beta[t] : 0.f;
}

// ------------------------------------------------------------------------------------------------ X = (I + N)^-1
template <int D>
struct InvSmem {
    static constexpr int off_k = 0;                                   // K tile, TC_C x D bf16
    static constexpr int NP = 68;                                     // row pitch of N in floats (16-byte aligned, spreads banks)
    static constexpr int off_n = TC_C * D * 2;                        // N fp32 [64][NP]
    static constexpr int off_x = off_n + TC_C * NP * 4;               // X head, X tail: [64][64] bf16 each
    static constexpr int off_misc = off_x + 2 * TC_C * TC_C * 2;
    static constexpr int bytes = off_misc + 1024 + 1024;
};

template <int D>
__global__ void __launch_bounds__(128) delta_inv_kernel(const __grid_constant__ CUtensorMap mk, const float *__restrict__ la_all,
                                                        const float *__restrict__ beta_all, __nv_bfloat16 *__restrict__ X, int T,
                                                        int with_tail) {
    using SM = InvSmem<D>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - smem_u32(smem_raw));
    float *Nf = reinterpret_cast<float *>(sm + SM::off_n);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + SM::off_misc + 32);
    float *Ls = reinterpret_cast<float *>(sm + SM::off_misc + 64), *bes = Ls + 64;
    const uint32_t bar_k = base + SM::off_misc, bar_m = bar_k + 8;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int c = blockIdx.x, bh = blockIdx.y, NC = gridDim.x, t0 = c * TC_C;

    if (tid == 0) {
        mbar_init(bar_k, 1); mbar_init(bar_m, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(bar_k, TC_C * D * 2);
#pragma unroll
        for (int s = 0; s < D / 64; ++s) tma_load_3d(base + SM::off_k + s * 8192, &mk, bar_k, 64 * s, t0, bh);
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), 64);
    if (warp < 2) chunk_stats(la_all + (size_t)bh * T, beta_all + (size_t)bh * T, t0, T, tid, lane, warp, Ls, nullptr, nullptr, bes);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool ok = mbar_wait(bar_k, 0, 11);
    if (tid == 0 && ok) {
        constexpr uint32_t I_KK = idesc_bf16(64, 64, 0, 0);
        const uint64_t dk = smem_desc(base + SM::off_k, 16, 1024);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
            const uint32_t ko = ((uint32_t)(k >> 2) * 8192u + (uint32_t)(k & 3) * 32u) >> 4;
            mma_bf16(tmem, dk + ko, dk + ko, I_KK, k > 0);
        }
        mma_commit(bar_m);
    }
    if (ok && !mbar_wait(bar_m, 0, 12)) ok = false;
    tc_fence_after();
    // ---- N = beta_t (k_t . k_s) exp(min(L_t - L_s, 0)) for s < t, else 0.   Each warp: its 16 rows, all 64 columns.
    {
        const int fr = lane >> 2, fq = lane & 3, r0 = 16 * warp + fr, r1 = r0 + 8;
        float kk[32];
        tmem_ld_frag8(tmem + ((uint32_t)(32 * warp) << 16), kk);
        tmem_ld_wait();
        const float L0 = Ls[r0] * TD_LOG2E, L1 = Ls[r1] * TD_LOG2E, b0 = bes[r0], b1 = bes[r1];
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int s = 8 * j + 2 * fq + e;
                const float Lsv = Ls[s] * TD_LOG2E;
                Nf[r0 * SM::NP + s] = (s < r0) ? b0 * kk[4 * j + e] * exp2f(fminf(L0 - Lsv, 0.f)) : 0.f;
                Nf[r1 * SM::NP + s] = (s < r1) ? b1 * kk[4 * j + 2 + e] * exp2f(fminf(L1 - Lsv, 0.f)) : 0.f;
            }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 64);
    // ---- column j of X: x_t = [t == j] - sum_{s<t} N[t][s] x_s   (x_s = 0 above the diagonal, so one code path for all j)
    __nv_bfloat16 *Xh = reinterpret_cast<__nv_bfloat16 *>(sm + SM::off_x), *Xl = Xh + TC_C * TC_C;
    if (tid < TC_C) {
        float x[TC_C];
#pragma unroll
        for (int t = 0; t < TC_C; ++t) {
            float acc0 = (t == tid) ? 1.f : 0.f, acc1 = 0.f;
            const float4 *row = reinterpret_cast<const float4 *>(Nf + t * SM::NP);
#pragma unroll
            for (int s4 = 0; s4 < (t + 3) / 4; ++s4) {
                const float4 n = row[s4];                             // the same address for every thread: a broadcast
                if (4 * s4 + 0 < t) acc0 = fmaf(-n.x, x[4 * s4 + 0], acc0);
                if (4 * s4 + 1 < t) acc1 = fmaf(-n.y, x[4 * s4 + 1], acc1);
                if (4 * s4 + 2 < t) acc0 = fmaf(-n.z, x[4 * s4 + 2], acc0);
                if (4 * s4 + 3 < t) acc1 = fmaf(-n.w, x[4 * s4 + 3], acc1);
            }
            x[t] = acc0 + acc1;
            __nv_bfloat16 hi, lo;
            split_bf16(x[t], hi, lo);
            Xh[t * 64 + tid] = hi;
            Xl[t * 64 + tid] = lo;
        }
    }
    __syncthreads();
    // ---- head then tail, 8 KB each, to the scratch buffer; or the head alone, densely packed (the stand-alone operator)
    {
        uint4 *dst = reinterpret_cast<uint4 *>(X + ((size_t)bh * NC + c) * ((with_tail ? 2 : 1) * TC_C * TC_C));
        const uint4 *src = reinterpret_cast<const uint4 *>(Xh);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (with_tail || i < 4) dst[tid + 128 * i] = src[tid + 128 * i];
    }
}

// ------------------------------------------------------------------------------------------------ the chunk walk

struct TdParams {
    const float *la, *beta, *S0, *theta, *shift_dev;
    float shift_host;
    void *o; float *S_out; __nv_bfloat16 *sent;
    int H, T, o_is_f32;
};

template <int D>
struct TdSmem {
    static constexpr int QK = TC_C * D * 2;                           // Q or K tile
    static constexpr int SQ = TC_C * TC_C * 2;                        // a 64 x 64 bf16 tile (V slice, X, A, rhs / W)
    static constexpr int STAGE = 2 * QK + 3 * SQ;                     // Q, K, V slice, X head, X tail
    static constexpr int off_stage = 0;                               // [2]
    // Head dim 128 double-buffers the tiles and fills the SM with one CTA. Head dim 64 keeps ONE stage (its next load is
    // issued as soon as the second product group has consumed the tiles and lands under the rest of the chunk), which
    // brings the CTA to 108 KiB: two CTAs share an SM and fill each other's tensor-core and barrier waits.
    static constexpr int NSTAGE = D == 64 ? 1 : 2;
    static constexpr int off_kwh = NSTAGE * STAGE;
    static constexpr int off_kwl = off_kwh + QK;
    static constexpr int off_ah = off_kwl + QK;
    static constexpr int off_al = off_ah + SQ;
    static constexpr int off_wh = off_al + SQ;                        // rhs, then W (same layout, reused)
    static constexpr int off_wl = off_wh + SQ;
    static constexpr int off_sh = off_wl + SQ;                        // S slice [D key rows][64 value columns]
    static constexpr int off_sl = off_sh + D * 128;
    static constexpr int off_misc = off_sl + D * 128;
    static constexpr int bytes = off_misc + 3072 + 1024;             // barriers, tensor-memory slot, two statistics slots
};

template <int D>
__global__ void __launch_bounds__(TD_NT) prefill_tc_delta_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                                                                 const __grid_constant__ CUtensorMap mv, const __grid_constant__ CUtensorMap mx,
                                                                 TdParams p) {
    using SM = TdSmem<D>;
    constexpr int SUB = D / 64;
    constexpr int NSG = D / 64;                                       // 16-row groups of the state per warp
    constexpr uint32_t TM_P = 0, TM_KS = 64, TM_O1 = 128, TM_O2 = 192;  // KS, then W, then U share columns 64..127
    constexpr uint32_t TM_COLS = 256;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - smem_u32(smem_raw));
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + SM::off_misc + 64);
    float *stats = reinterpret_cast<float *>(sm + SM::off_misc + 128);    // [2 chunks][L, e^L, w, beta][64]
    const uint32_t bar_full0 = base + SM::off_misc, bar_full1 = bar_full0 + 8, bar_a = bar_full0 + 16, bar_b = bar_full0 + 24,
                   bar_c = bar_full0 + 32;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, wg = warp >> 2, sub = warp & 3;
    const int vs0 = blockIdx.x * 64;                                  // first value column of this CTA's slice
    const int bh = blockIdx.y, h = bh % p.H;
    const int T = p.T, NC = (T + TC_C - 1) / TC_C;
    const float *la = p.la + (size_t)bh * T, *beta = p.beta + (size_t)bh * T;

    if (tid == 0) {
        mbar_init(bar_full0, 1); mbar_init(bar_full1, 1); mbar_init(bar_a, 3); mbar_init(bar_b, 1); mbar_init(bar_c, 2);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), TM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int fr = lane >> 2, fq = lane & 3;
    const int trow0 = 16 * sub + fr, trow1 = trow0 + 8;
    const uint32_t lane_base = (uint32_t)(32 * sub) << 16;
    const int col0 = 32 * wg;                                         // this warp's 32 columns of every 64-column accumulator
    auto state_row = [&](int g, int hi8) { return (D == 128 ? 32 * sub + 16 * g : 16 * sub) + fr + 8 * hi8; };

    // ---- entering state slice in fragment order (rows = key index, this CTA's 64 value columns), rebased
    float S[NSG][16];
#pragma unroll
    for (int g = 0; g < NSG; ++g)
#pragma unroll
        for (int j = 0; j < 16; ++j) S[g][j] = 0.f;
    if (p.S0 != nullptr) {
        const float shift = p.theta == nullptr ? 0.f : (p.shift_dev != nullptr ? *p.shift_dev : p.shift_host);
#pragma unroll
        for (int g = 0; g < NSG; ++g)
#pragma unroll
            for (int hi8 = 0; hi8 < 2; ++hi8) {
                const int row = state_row(g, hi8);
                const float *src = p.S0 + ((size_t)bh * D + row) * D + vs0 + col0 + 2 * fq;
                float sn = 0.f, cs = 1.f;
                if (shift != 0.f) sincosf(-shift * p.theta[(size_t)h * (D / 2) + (row >> 1)], &sn, &cs);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 t = *reinterpret_cast<const float2 *>(src + 8 * j);
                    float x0 = t.x, x1 = t.y;
                    if (shift != 0.f) {
                        const float y0 = __shfl_xor_sync(0xffffffffu, x0, 4), y1 = __shfl_xor_sync(0xffffffffu, x1, 4);
                        x0 = (row & 1) ? y0 * sn + x0 * cs : x0 * cs - y0 * sn;
                        x1 = (row & 1) ? y1 * sn + x1 * cs : x1 * cs - y1 * sn;
                    }
                    S[g][4 * j + 2 * hi8] = x0; S[g][4 * j + 2 * hi8 + 1] = x1;
                }
            }
    }

    auto load_stage = [&](int c, int st) {                            // thread 0: one chunk's tiles into stage st
        const uint32_t bar = st ? bar_full1 : bar_full0, sb = base + SM::off_stage + st * SM::STAGE;
        mbar_expect_tx(bar, SM::STAGE);
#pragma unroll
        for (int s = 0; s < SUB; ++s) {
            tma_load_3d(sb + s * 8192, &mq, bar, 64 * s, c * TC_C, bh);
            tma_load_3d(sb + SM::QK + s * 8192, &mk, bar, 64 * s, c * TC_C, bh);
        }
        tma_load_3d(sb + 2 * SM::QK, &mv, bar, vs0, c * TC_C, bh);
        tma_load_3d(sb + 2 * SM::QK + SM::SQ, &mx, bar, 0, 0, (bh * NC + c) * 2);
        tma_load_3d(sb + 2 * SM::QK + 2 * SM::SQ, &mx, bar, 0, 0, (bh * NC + c) * 2 + 1);
    };
    bool ok = true;
    if (tid == 0) load_stage(0, 0);
    // The decay statistics do not depend on the state: warps 6 and 7, idle while a tensor-core round is in flight, prepare
    // the next chunk's one iteration ahead (a global load plus a dependent shuffle scan, ~2.5k cycles otherwise exposed).
    auto stats_of = [&](int c) {
        float *L = stats + (c & 1) * 256;
        chunk_stats(la, beta, c * TC_C, T, tid - 192, lane, warp - 6, L, L + 64, L + 128, L + 192);
    };
    if (warp >= 6) stats_of(0);

    for (int c = 0; c < NC && ok; ++c) {
        const int t0 = c * TC_C, st = SM::NSTAGE == 2 ? (c & 1) : 0;
        const uint32_t sb = base + SM::off_stage + st * SM::STAGE;
        const uint32_t qs = sb, ks = sb + SM::QK, vs = sb + 2 * SM::QK, xh = vs + SM::SQ, xl = xh + SM::SQ;
        uint8_t *ks_ptr = sm + SM::off_stage + st * SM::STAGE + SM::QK, *vs_ptr = ks_ptr + SM::QK;
        if (SM::NSTAGE == 2 && tid == 0 && c + 1 < NC) load_stage(c + 1, st ^ 1);
        const float *Ls = stats + (c & 1) * 256, *eLs = Ls + 64, *wts = eLs + 64, *bes = wts + 64;
        // ---- entering state slice as an MN-major B operand (rows = key index), head and tail
        {
#pragma unroll
            for (int g = 0; g < NSG; ++g)
#pragma unroll
                for (int hi8 = 0; hi8 < 2; ++hi8) {
                    const int row = state_row(g, hi8);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t hi, lo;
                        split2(S[g][4 * j + 2 * hi8], S[g][4 * j + 2 * hi8 + 1], hi, lo);
                        const uint32_t off = swz(row, 4 * wg + j) + 4 * fq;
                        *reinterpret_cast<uint32_t *>(sm + SM::off_sh + off) = hi;
                        *reinterpret_cast<uint32_t *>(sm + SM::off_sl + off) = lo;
                        if (p.sent != nullptr)
                            *reinterpret_cast<uint32_t *>(p.sent + (((size_t)bh * NC + c) * D + row) * D + vs0 + col0 + 8 * j + 2 * fq) = hi;
                    }
                }
        }
        if (!mbar_wait(st ? bar_full1 : bar_full0, (SM::NSTAGE == 2 ? (c >> 1) : c) & 1, 21)) ok = false;
        ok = __syncthreads_and(ok);                                   // one verdict for the whole CTA: every thread leaves the loop at the same point
        const float aC = expf(Ls[TC_C - 1]);
        // ---- K * w, head and tail, in K's own layout (an MN-major A operand)
        if (ok) {
            for (int idx = tid; idx < TC_C * (D / 8); idx += TD_NT) {
                const int r = idx / (D / 8), jj = idx % (D / 8);
                const uint32_t off = (uint32_t)(jj >> 3) * 8192u + swz(r, jj & 7);
                const uint4 raw = *reinterpret_cast<const uint4 *>(ks_ptr + off);
                const __nv_bfloat162 *b2 = reinterpret_cast<const __nv_bfloat162 *>(&raw);
                const float w = wts[r];
                float x[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(b2[i]); x[2 * i] = f.x * w; x[2 * i + 1] = f.y * w; }
                uint4 hi, lo;
                split8(x, hi, lo);
                *reinterpret_cast<uint4 *>(sm + SM::off_kwh + off) = hi;
                *reinterpret_cast<uint4 *>(sm + SM::off_kwl + off) = lo;
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- first product group: P = Q K^T, KS = K S, O2 = Q S
        const uint64_t dsh = smem_desc(base + SM::off_sh, 16, 1024), dsl = smem_desc(base + SM::off_sl, 16, 1024);
        // Everyone waits for the round, so issue time counts: the three products go out from three warps (one accumulator
        // each, so no ordering between them is needed), each through one elected lane of the converged warp, which keeps the
        // descriptors in the uniform datapath (measured: about 33 cycles per tcgen05.mma against 65-100 from a lone thread).
        if (warp < 3 && __all_sync(0xffffffffu, ok)) {                // whole warps, converged: one elected lane each issues
            tc_fence_after();
            constexpr uint32_t I_P = idesc_bf16(64, 64, 0, 0), I_S = idesc_bf16(64, 64, 0, 1);
            const uint64_t dq = smem_desc(qs, 16, 1024), dk = smem_desc(ks, 16, 1024);
            if (warp == 0) {
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint32_t ko = ((uint32_t)(k >> 2) * 8192u + (uint32_t)(k & 3) * 32u) >> 4;
                    mma_bf16_elect(tmem + TM_P, dq + ko, dk + ko, I_P, k > 0);
                }
            } else {
                const uint64_t da = warp == 1 ? dk : dq;
                const uint32_t acc = warp == 1 ? TM_KS : TM_O2;
#pragma unroll
                for (int half = 0; half < 2; ++half)
#pragma unroll
                    for (int k = 0; k < D / 16; ++k) {                // S rows (key index) advance 16 rows = 2048 B per step
                        const uint32_t ko = ((uint32_t)(k >> 2) * 8192u + (uint32_t)(k & 3) * 32u) >> 4;
                        mma_bf16_elect(tmem + acc, da + ko, (half ? dsl : dsh) + k * 128, I_S, half | (k > 0));
                    }
            }
            mma_commit_elect(bar_a);
        }
        if (warp >= 6 && c + 1 < NC) stats_of(c + 1);
        if (ok && !mbar_wait(bar_a, c & 1, 22)) ok = false;
        ok = __syncthreads_and(ok);
        tc_fence_after();
        if (ok) {
            // ---- A = P * decay (causal), head and tail; rhs = beta (V - e^{L_t} K S), head and tail
            float pv[16], kv[16];
            tmem_ld_frag4(tmem + lane_base + TM_P + col0, pv);
            tmem_ld_frag4(tmem + lane_base + TM_KS + col0, kv);
            tmem_ld_wait();
            const float Lt0 = Ls[trow0] * TD_LOG2E, Lt1 = Ls[trow1] * TD_LOG2E;
            const float e0 = eLs[trow0], e1 = eLs[trow1], b0 = bes[trow0], b1 = bes[trow1];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int s0 = col0 + 8 * j + 2 * fq;
                const float Ls0 = Ls[s0] * TD_LOG2E, Ls1 = Ls[s0 + 1] * TD_LOG2E;
                const float a00 = (s0 <= trow0) ? pv[4 * j] * exp2f(fminf(Lt0 - Ls0, 0.f)) : 0.f;
                const float a01 = (s0 + 1 <= trow0) ? pv[4 * j + 1] * exp2f(fminf(Lt0 - Ls1, 0.f)) : 0.f;
                const float a10 = (s0 <= trow1) ? pv[4 * j + 2] * exp2f(fminf(Lt1 - Ls0, 0.f)) : 0.f;
                const float a11 = (s0 + 1 <= trow1) ? pv[4 * j + 3] * exp2f(fminf(Lt1 - Ls1, 0.f)) : 0.f;
                const uint32_t o0 = swz(trow0, 4 * wg + j) + 4 * fq, o1 = swz(trow1, 4 * wg + j) + 4 * fq;
                uint32_t hi, lo;
                split2(a00, a01, hi, lo);
                *reinterpret_cast<uint32_t *>(sm + SM::off_ah + o0) = hi; *reinterpret_cast<uint32_t *>(sm + SM::off_al + o0) = lo;
                split2(a10, a11, hi, lo);
                *reinterpret_cast<uint32_t *>(sm + SM::off_ah + o1) = hi; *reinterpret_cast<uint32_t *>(sm + SM::off_al + o1) = lo;
                // the same (row, column pair) of V: the value slice tile has the identical swizzled layout
                const float2 v0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(vs_ptr + o0));
                const float2 v1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(vs_ptr + o1));
                split2(b0 * (v0.x - e0 * kv[4 * j]), b0 * (v0.y - e0 * kv[4 * j + 1]), hi, lo);
                *reinterpret_cast<uint32_t *>(sm + SM::off_wh + o0) = hi; *reinterpret_cast<uint32_t *>(sm + SM::off_wl + o0) = lo;
                split2(b1 * (v1.x - e1 * kv[4 * j + 2]), b1 * (v1.y - e1 * kv[4 * j + 3]), hi, lo);
                *reinterpret_cast<uint32_t *>(sm + SM::off_wh + o1) = hi; *reinterpret_cast<uint32_t *>(sm + SM::off_wl + o1) = lo;
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- second product group: W = X rhs  (head*head + head*tail + tail*head)
        const uint64_t dwh = smem_desc(base + SM::off_wh, 16, 1024), dwl = smem_desc(base + SM::off_wl, 16, 1024);
        if (warp == 0 && __all_sync(0xffffffffu, ok)) {               // the whole warp, converged: one elected lane issues
            tc_fence_after();
            constexpr uint32_t I_W = idesc_bf16(64, 64, 0, 1);
            const uint64_t dxh = smem_desc(xh, 16, 1024), dxl = smem_desc(xl, 16, 1024);
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_bf16_elect(tmem + TM_KS, dxh + k * 2, dwh + k * 128, I_W, k > 0);
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_bf16_elect(tmem + TM_KS, dxh + k * 2, dwl + k * 128, I_W, 1);
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_bf16_elect(tmem + TM_KS, dxl + k * 2, dwh + k * 128, I_W, 1);
            mma_commit_elect(bar_b);
        }
        if (ok && !mbar_wait(bar_b, c & 1, 23)) ok = false;
        ok = __syncthreads_and(ok);
        tc_fence_after();
        // single stage: Q, K, V and X of this chunk are consumed (the first two product groups are complete, the generic
        // reads of K and V ended before the barrier ahead of the second), so the next chunk's tiles may overwrite them
        if (SM::NSTAGE == 1 && tid == 0 && ok && c + 1 < NC) load_stage(c + 1, 0);
        if (ok) {
            // ---- W back to shared memory (over rhs), head and tail
            float wv[16];
            tmem_ld_frag4(tmem + lane_base + TM_KS + col0, wv);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t o0 = swz(trow0, 4 * wg + j) + 4 * fq, o1 = swz(trow1, 4 * wg + j) + 4 * fq;
                uint32_t hi, lo;
                split2(wv[4 * j], wv[4 * j + 1], hi, lo);
                *reinterpret_cast<uint32_t *>(sm + SM::off_wh + o0) = hi; *reinterpret_cast<uint32_t *>(sm + SM::off_wl + o0) = lo;
                split2(wv[4 * j + 2], wv[4 * j + 3], hi, lo);
                *reinterpret_cast<uint32_t *>(sm + SM::off_wh + o1) = hi; *reinterpret_cast<uint32_t *>(sm + SM::off_wl + o1) = lo;
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- third product group: O1 = A W, U = (K w)^T W
        if (warp < 2 && __all_sync(0xffffffffu, ok)) {                // O1 from one warp's elected lane, U from another's
            tc_fence_after();
            constexpr uint32_t I_O = idesc_bf16(64, 64, 0, 1), I_U = idesc_bf16(D, 64, 1, 1);
            if (warp == 0) {
                const uint64_t dah = smem_desc(base + SM::off_ah, 16, 1024), dal = smem_desc(base + SM::off_al, 16, 1024);
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16_elect(tmem + TM_O1, dah + k * 2, dwh + k * 128, I_O, k > 0);
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16_elect(tmem + TM_O1, dah + k * 2, dwl + k * 128, I_O, 1);
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16_elect(tmem + TM_O1, dal + k * 2, dwh + k * 128, I_O, 1);
            } else {
                const uint64_t dkwh = smem_desc(base + SM::off_kwh, 8192, 1024), dkwl = smem_desc(base + SM::off_kwl, 8192, 1024);
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16_elect(tmem + TM_KS, dkwh + k * 128, dwh + k * 128, I_U, k > 0);
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16_elect(tmem + TM_KS, dkwh + k * 128, dwl + k * 128, I_U, 1);
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16_elect(tmem + TM_KS, dkwl + k * 128, dwh + k * 128, I_U, 1);
            }
            mma_commit_elect(bar_c);
        }
        if (ok && !mbar_wait(bar_c, c & 1, 24)) ok = false;
        ok = __syncthreads_and(ok);
        tc_fence_after();
        if (ok) {
            float ov[16], o2v[16], uv[NSG][16];
            tmem_ld_frag4(tmem + lane_base + TM_O1 + col0, ov);
            tmem_ld_frag4(tmem + lane_base + TM_O2 + col0, o2v);
#pragma unroll
            for (int g = 0; g < NSG; ++g) tmem_ld_frag4(tmem + lane_base + ((uint32_t)(16 * g) << 16) + TM_KS + col0, uv[g]);
            tmem_ld_wait();
            const float e0 = eLs[trow0], e1 = eLs[trow1];
#pragma unroll
            for (int hi8 = 0; hi8 < 2; ++hi8) {
                const int trow = hi8 ? trow1 : trow0;
                if (t0 + trow < T) {
                    const float e = hi8 ? e1 : e0;
                    const size_t off = ((size_t)bh * T + t0 + trow) * D + vs0 + col0 + 2 * fq;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float x0 = fmaf(e, o2v[4 * j + 2 * hi8], ov[4 * j + 2 * hi8]);
                        const float x1 = fmaf(e, o2v[4 * j + 2 * hi8 + 1], ov[4 * j + 2 * hi8 + 1]);
                        if (p.o_is_f32) *reinterpret_cast<float2 *>((float *)p.o + off + 8 * j) = make_float2(x0, x1);
                        else *reinterpret_cast<__nv_bfloat162 *>((__nv_bfloat16 *)p.o + off + 8 * j) = __floats2bfloat162_rn(x0, x1);
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < NSG; ++g)
#pragma unroll
                for (int j = 0; j < 16; ++j) S[g][j] = fmaf(aC, S[g][j], uv[g][j]);
        }
        tc_fence_before();
        __syncthreads();
    }
    if (ok) {
#pragma unroll
        for (int g = 0; g < NSG; ++g)
#pragma unroll
            for (int hi8 = 0; hi8 < 2; ++hi8) {
                float *dst = p.S_out + ((size_t)bh * D + state_row(g, hi8)) * D + vs0 + col0 + 2 * fq;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *reinterpret_cast<float2 *>(dst + 8 * j) = make_float2(S[g][4 * j + 2 * hi8], S[g][4 * j + 2 * hi8 + 1]);
            }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, TM_COLS);
}

// ------------------------------------------------------------------------------------------------ host side
template <int D>
static int delta_go(const PrefillArgs &a, int o_dtype, void *x_scratch, cudaStream_t stream) {
    const int BH = a.B * a.H, NC = (a.T + TC_C - 1) / TC_C;
    CUtensorMap mq, mk, mv, mx;
    if (!tc_make_map(&mq, a.q, BH, a.T, D, D, (long long)a.T * D) || !tc_make_map(&mk, a.k, BH, a.T, D, D, (long long)a.T * D) ||
        !tc_make_map(&mv, a.v, BH, a.T, D, D, (long long)a.T * D) ||
        !tc_make_map(&mx, x_scratch, (long long)BH * NC * 2, TC_C, TC_C, TC_C, TC_C * TC_C)) {
        set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled");
        return PGB_ERR_CUDA;
    }
    auto inv = delta_inv_kernel<D>;
    auto walk = prefill_tc_delta_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(inv, cudaFuncAttributeMaxDynamicSharedMemorySize, InvSmem<D>::bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(walk, cudaFuncAttributeMaxDynamicSharedMemorySize, TdSmem<D>::bytes);
    if (e != cudaSuccess) { set_cuda_error(e, "prefill_tc_delta smem attribute"); return PGB_ERR_CUDA; }
    inv<<<dim3(NC, BH), 128, InvSmem<D>::bytes, stream>>>(mk, a.la, a.beta, (__nv_bfloat16 *)x_scratch, a.T, 1);
    int rc = check_launch("delta_inv_kernel");
    if (rc != PGB_OK) return rc;
    TdParams p{a.la, a.beta, a.S0, a.theta, a.shift_dev, a.shift_host, a.o, a.S_out, a.sent, a.H, a.T, o_dtype == PGB_F32};
    walk<<<dim3(D / 64, BH), TD_NT, TdSmem<D>::bytes, stream>>>(mq, mk, mv, mx, p);
    return check_launch("prefill_tc_delta_kernel");
}

// bytes of scratch the delta path needs for X (head and tail, 64 x 64 bf16 each, per (sequence-head, chunk))
size_t prefill_tc_delta_scratch_bytes(int B, int H, int T) {
    return (size_t)B * H * ((T + TC_C - 1) / TC_C) * 2 * TC_C * TC_C * sizeof(__nv_bfloat16);
}

int prefill_tc_delta_launch(const PrefillArgs &a, int o_dtype, int D, void *x_scratch, cudaStream_t stream) {
    return D == 64 ? delta_go<64>(a, o_dtype, x_scratch, stream) : delta_go<128>(a, o_dtype, x_scratch, stream);
}

int tc_delta_error_flag(int *out) { return tc_read_error_flag(out); }

// The inverse alone, as the reference's stand-alone operator returns it (src/assoc_kernel.py:658-667 membrae::delta_inv):
// X [B*H][NC][64][64] bf16, the rounded heads only.
template <int D>
static int delta_inv_go(const void *k, const float *la, const float *beta, void *X, int BH, int T, cudaStream_t stream) {
    const int NC = (T + TC_C - 1) / TC_C;
    CUtensorMap mk;
    if (!tc_make_map(&mk, k, BH, T, D, D, (long long)T * D)) { set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled"); return PGB_ERR_CUDA; }
    auto inv = delta_inv_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(inv, cudaFuncAttributeMaxDynamicSharedMemorySize, InvSmem<D>::bytes);
    if (e != cudaSuccess) { set_cuda_error(e, "delta_inv smem attribute"); return PGB_ERR_CUDA; }
    inv<<<dim3(NC, BH), 128, InvSmem<D>::bytes, stream>>>(mk, la, beta, (__nv_bfloat16 *)X, T, 0);
    return check_launch("delta_inv_kernel");
}
int delta_inv_launch(const void *k, const float *la, const float *beta, void *X, int BH, int T, int D, cudaStream_t stream) {
    return D == 64 ? delta_inv_go<64>(k, la, beta, X, BH, T, stream) : delta_inv_go<128>(k, la, beta, X, BH, T, stream);
}

// ------------------------------------------------------------------------------------------------ built-in scratch
// The same delta prefill for callers that have no way to hand over a scratch buffer. The chunk inverses then live in
// this file-scope device array: PGB_STATIC_SCRATCH_BYTES of device memory that every GPU which loads the library keeps
// reserved until the process exits. In host code the array's name is only a stand-in for the device object, so its
// device address is asked for once per device (cudaGetSymbolAddress, with that device current) and cached.
constexpr size_t PGB_STATIC_SCRATCH_BYTES = 32u << 20;                 // 2048 (sequence-head, chunk) pairs of 16 KiB
static __device__ __align__(256) unsigned char g_static_scratch[PGB_STATIC_SCRATCH_BYTES];

static void *static_scratch_ptr() {
    constexpr int MAX_DEV = 64;
    static void *cache[MAX_DEV] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return nullptr;
    void *ptr = __atomic_load_n(&cache[dev], __ATOMIC_ACQUIRE);
    if (ptr == nullptr) {
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) { set_cuda_error(e, "cudaGetSymbolAddress(static scratch)"); return nullptr; }
        __atomic_store_n(&cache[dev], ptr, __ATOMIC_RELEASE);         // the same value whoever gets here first
    }
    return ptr;
}

long long prefill_tc_delta_static_capacity() { return (long long)PGB_STATIC_SCRATCH_BYTES; }

int prefill_tc_delta_static_launch(const PrefillArgs &a, int o_dtype, int D, cudaStream_t stream) {
    if (prefill_tc_delta_scratch_bytes(a.B, a.H, a.T) > PGB_STATIC_SCRATCH_BYTES) return PGB_ERR_TOO_LARGE;
    void *scratch = static_scratch_ptr();
    if (scratch == nullptr) return PGB_ERR_CUDA;
    return prefill_tc_delta_launch(a, o_dtype, D, scratch, stream);
}

}  // namespace pgb
