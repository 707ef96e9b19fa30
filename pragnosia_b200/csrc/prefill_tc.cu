// Chunked prefill of the associative carrier on the 5th-generation tensor cores: tcgen05.mma with TMEM accumulators,
// operands staged in shared memory by TMA, bf16 operands with fp32 accumulation and an fp32 state.
//
// One CTA walks the 64-token chunks of one (sequence, head). Per chunk c, with L the within-chunk cumulative log-decay:
//   P  = Q K^T                                   (M=64 tokens, N=64 tokens, K=D)        state-independent
//   U  = (K*w)^T V,  w_s = exp(L_C - L_s)        (M=D, N=D, K=64 tokens)               state-independent
//   O2 = Q S_c                                   (M=64, N=D, K=D)                       reads the entering state
//   A  = P * exp(min(L_t - L_s, 0)) [s<=t]       in registers (tcgen05.ld), written back to shared memory
//   O1 = A V                                     (M=64, N=D, K=64)
//   o_t = O1_t + exp(L_t) O2_t ;   S_{c+1} = exp(L_C) S_c + U      (fp32, in registers)
// Only the last line is sequential across chunks, and it is one FMA per state element.
//
// Precision. Every fp32 operand that has to re-enter the tensor core (A, K*w, S) is split into a bf16 head and a bf16
// tail (x = hi + lo to 2^-17) and multiplied as two MMAs into the same accumulator, so the only roundings left are the
// callers' bf16 q, k, v. The row scaling exp(L_t) of the state read is applied to the fp32 accumulator, not the operand.
// This is HBM-bound work (64 FLOP/B at D=64), so the second MMA per product is free.
//
// Shared-memory operand layouts (all 128-byte swizzled, tiles 1024-byte aligned):
//   Q, K   [64 tokens][D]  rows of 128 B, K-major operands (K = head dim); D=128 is two 64-column sub-tiles.  From TMA.
//   V      [64 tokens][D]  the same bytes read as an MN-major B operand (N = value dim contiguous).            From TMA.
//   KW     like K, rows scaled by w, hi and lo copies: MN-major A operand (M = key dim contiguous).           Threads.
//   A      [64 t][64 s]    K-major A operand, hi and lo.                                                      Threads.
//   S      [D key][D value] MN-major B operand (rows = key index = K), hi and lo; D=128: two value sub-tiles. Threads.
// TMEM (columns): P 64 | U D | O1 D | O2 D.  M=64 accumulators live in lanes 0-15 of each 32-lane subpartition; they are
// read with 16x256b loads, so all 32 threads of a warp share those 16 rows (thread: rows l/4 and l/4+8, column pairs).
// 8 warps: warp%4 picks the subpartition (rows), warp/4 the column half.
//
// RAW mode takes the layer's projections as they leave the GEMM ((B,T,H,D) views) and does the plumbing in place in
// shared memory after the TMA lands: L2-normalise q, k, v, scale k by the write gate, rotate q and k (cos/sin from a
// per-layer table), so the separate prep pass and its HBM round trip disappear.
//
// Every mbarrier wait is bounded; a wait that runs out sets g_tc_error, and the CTA still frees its TMEM and returns.
#include "tc_common.cuh"

namespace pgb {


template <int D>
struct TcSmem {
    static constexpr int TILE = TC_C * D * 2;                         // one Q / K / V tile, bytes
    static constexpr int off_q = 0;                                   // [2 stages]
    static constexpr int off_k = off_q + 2 * TILE;
    static constexpr int off_v = off_k + 2 * TILE;
    static constexpr int off_kwh = off_v + 2 * TILE;
    static constexpr int off_kwl = off_kwh + TILE;
    static constexpr int off_ah = off_kwl + TILE;                     // [64][64] bf16
    static constexpr int off_al = off_ah + TC_C * TC_C * 2;
    static constexpr int off_sh = off_al + TC_C * TC_C * 2;           // [D][D] bf16
    static constexpr int off_sl = off_sh + D * D * 2;
    static constexpr int off_misc = off_sl + D * D * 2;               // barriers, tmem base, L / eL / w, ...
    static constexpr int bytes = off_misc + 3072 + 1024;              // misc (2.2 KB used) + slack for the 1024-byte alignment
};

constexpr int TC_NT = 256;

template <int D, bool RAW>
__global__ void __launch_bounds__(TC_NT) prefill_tc_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                                                           const __grid_constant__ CUtensorMap mv, TcParams p) {
    using SM = TcSmem<D>;
    constexpr int NT = TC_NT;
    constexpr int SUB = D / 64;                                       // 64-column sub-tiles per Q/K/V tile
    constexpr int HALF = D / 2;                                       // accumulator columns one warp reads (N = D)
    constexpr int NBO = HALF / 8;                                     // 8-column blocks per thread for O1 / O2 / U
    constexpr int NSG = D / 64;                                       // 16-row groups of the state per warp
    constexpr uint32_t TM_P = 0, TM_U = 64, TM_O1 = 64 + D, TM_O2 = 64 + 2 * D;
    constexpr uint32_t TM_COLS = (D == 64) ? 256 : 512;
    constexpr uint32_t STAGE_BYTES = 3 * SM::TILE;
    constexpr float LOG2E = 1.4426950408889634f;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - smem_u32(smem_raw));
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + SM::off_misc + 64);
    float *Ls = reinterpret_cast<float *>(sm + SM::off_misc + 128);            // L[64]
    float *eLs = Ls + 64, *wts = eLs + 64, *red = wts + 64, *rmsw = red + 128; // red[2][64], rmsw[D]
    float *gts = rmsw + 128;                                                   // sigmoid(write gate) of the chunk's tokens
    const uint32_t bar_full0 = base + SM::off_misc, bar_full1 = bar_full0 + 8, bar_a = bar_full0 + 16, bar_b = bar_full0 + 24,
                   bar_rot = bar_full0 + 32;
    // RAW, D = 64: the chunk's 64 x 32 (cos, sin) pairs are bulk-copied into the A-operand buffers, which are idle
    // between one chunk's O1 product and the next chunk's score pass
    constexpr bool ROT_SMEM = RAW && D == 64;
    constexpr uint32_t ROT_BYTES = TC_C * (D / 2) * 8;
    const float2 *rot_sm = reinterpret_cast<const float2 *>(sm + SM::off_ah);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, wg = warp >> 2, sub = warp & 3;
    const int bh = blockIdx.x, h = bh % p.H, b = bh / p.H;
    const int T = p.T, NC = (T + TC_C - 1) / TC_C;
    const float *la = p.la != nullptr ? p.la + (size_t)bh * T : nullptr;
    const int tma_c0 = RAW ? h * D : 0, tma_c2 = RAW ? b : bh;

    if (tid == 0) {
        mbar_init(bar_full0, 1); mbar_init(bar_full1, 1); mbar_init(bar_a, 1); mbar_init(bar_b, 1); mbar_init(bar_rot, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc(smem_u32(tmem_slot), TM_COLS);
    if (p.rms_w != nullptr && tid < D) rmsw[tid] = p.rms_w[tid];
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // ---- fragment geometry (16x256b loads): rows l/4 and l/4+8 of the warp's 16-row group, column pairs 2(l%4)
    const int fr = lane >> 2, fq = lane & 3;
    const int trow0 = 16 * sub + fr, trow1 = trow0 + 8;               // token rows of the M=64 accumulators
    const uint32_t lane_base = (uint32_t)(32 * sub) << 16;
    const int pcol0 = 32 * wg;                                        // first score column of this warp
    const int ocol0 = HALF * wg;                                      // first value column of this warp (O1, O2, U, S)
    auto state_row = [&](int g, int hi8) { return (D == 128 ? 32 * sub + 16 * g : 16 * sub) + fr + 8 * hi8; };

    // ---- entering state in fragment order, rotated back by shift*theta (key rows 2i, 2i+1 are lanes l, l^4)
    float S[NSG][4 * NBO];
#pragma unroll
    for (int g = 0; g < NSG; ++g)
#pragma unroll
        for (int j = 0; j < 4 * NBO; ++j) S[g][j] = 0.f;
    if (p.S0 != nullptr) {
        const float shift = p.theta == nullptr ? 0.f : (p.shift_dev != nullptr ? *p.shift_dev : p.shift_host);
#pragma unroll
        for (int g = 0; g < NSG; ++g)
#pragma unroll
            for (int hi8 = 0; hi8 < 2; ++hi8) {
                const int row = state_row(g, hi8);
                const float *src = p.S0 + ((size_t)bh * D + row) * D + ocol0 + 2 * fq;
                float sn = 0.f, cs = 1.f;
                if (shift != 0.f) sincosf(-shift * p.theta[(size_t)h * (D / 2) + (row >> 1)], &sn, &cs);
#pragma unroll
                for (int j = 0; j < NBO; ++j) {
                    const float2 t = *reinterpret_cast<const float2 *>(src + 8 * j);
                    float x0 = t.x, x1 = t.y;
                    if (shift != 0.f) {                               // uniform across the CTA
                        const float y0 = __shfl_xor_sync(0xffffffffu, x0, 4), y1 = __shfl_xor_sync(0xffffffffu, x1, 4);
                        // even key row: x c - partner s ; odd key row: partner s + x c
                        x0 = (row & 1) ? y0 * sn + x0 * cs : x0 * cs - y0 * sn;
                        x1 = (row & 1) ? y1 * sn + x1 * cs : x1 * cs - y1 * sn;
                    }
                    S[g][4 * j + 2 * hi8] = x0; S[g][4 * j + 2 * hi8 + 1] = x1;
                }
            }
    }

    bool ok = true;
    if (tid == 0) {                                                   // first chunk's tiles
        mbar_expect_tx(bar_full0, STAGE_BYTES);
#pragma unroll
        for (int s = 0; s < SUB; ++s) {
            tma_load_3d(base + SM::off_q + s * 8192, &mq, bar_full0, tma_c0 + 64 * s, 0, tma_c2);
            tma_load_3d(base + SM::off_k + s * 8192, &mk, bar_full0, tma_c0 + 64 * s, 0, tma_c2);
            tma_load_3d(base + SM::off_v + s * 8192, &mv, bar_full0, tma_c0 + 64 * s, 0, tma_c2);
        }
        if constexpr (ROT_SMEM) {
            mbar_expect_tx(bar_rot, ROT_BYTES);
            bulk_load_1d(base + SM::off_ah, p.rot + (size_t)h * p.rot_T * (D / 2), ROT_BYTES, bar_rot);
        }
    }
    // decay (and write-gate) inputs of the first chunk, fetched one chunk ahead from here on
    auto fetch_decay = [&](int t) -> float {
        if (t >= T) return 0.f;
        if (p.la_raw != nullptr) return __bfloat162float(p.la_raw[(size_t)b * p.aux_sb + (size_t)t * p.aux_st + h]);
        return la[t];
    };
    auto fetch_gate = [&](int t) -> float {
        if (!RAW || p.gate_raw == nullptr || t >= T) return 0.f;
        return __bfloat162float(p.gate_raw[(size_t)b * p.aux_sb + (size_t)t * p.aux_st + h]);
    };
    const float expA = p.decay_A != nullptr ? expf(p.decay_A[h]) : 1.f;
    float nx_own = 0.f, nx_other = 0.f, nx_gate = 0.f;
    if (warp < 2) { nx_own = fetch_decay(tid); nx_other = fetch_decay(tid ^ 32); nx_gate = fetch_gate(tid); }

    for (int c = 0; c < NC && ok; ++c) {
        const int t0 = c * TC_C, st = c & 1;
        const uint32_t qs = base + SM::off_q + st * SM::TILE, ks = base + SM::off_k + st * SM::TILE, vs = base + SM::off_v + st * SM::TILE;
        uint8_t *qs_ptr = sm + SM::off_q + st * SM::TILE, *ks_ptr = sm + SM::off_k + st * SM::TILE, *vs_ptr = sm + SM::off_v + st * SM::TILE;
        if (tid == 0 && c + 1 < NC) {                                 // next chunk's tiles into the other stage
            const uint32_t nb = (st ? bar_full0 : bar_full1), o2 = (st ^ 1) * SM::TILE;
            mbar_expect_tx(nb, STAGE_BYTES);
#pragma unroll
            for (int s = 0; s < SUB; ++s) {
                tma_load_3d(base + SM::off_q + o2 + s * 8192, &mq, nb, tma_c0 + 64 * s, t0 + TC_C, tma_c2);
                tma_load_3d(base + SM::off_k + o2 + s * 8192, &mk, nb, tma_c0 + 64 * s, t0 + TC_C, tma_c2);
                tma_load_3d(base + SM::off_v + o2 + s * 8192, &mv, nb, tma_c0 + 64 * s, t0 + TC_C, tma_c2);
            }
        }
        // ---- decay statistics of the chunk: warps 0 and 1 each scan their 32 tokens and reduce the other half
        if (warp < 2) {
            // -softplus(gate logit) * exp(A_h) when the decay comes as logits (src/assoc.py:355-356); padding tokens: alpha = 1
            auto log_decay = [&](float raw, int r) -> float {
                if (t0 + r >= T) return 0.f;
                return p.la_raw != nullptr ? -fast_softplus(raw) * expA : raw;
            };
            const float own = log_decay(nx_own, tid), other = log_decay(nx_other, tid ^ 32);
            if (RAW) gts[tid] = p.gate_raw != nullptr ? fast_sigmoid(nx_gate) : 1.f;
            nx_own = fetch_decay(t0 + TC_C + tid); nx_other = fetch_decay(t0 + TC_C + (tid ^ 32)); nx_gate = fetch_gate(t0 + TC_C + tid);
            float sc = own;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float n = __shfl_up_sync(0xffffffffu, sc, o);
                if (lane >= o) sc += n;
            }
            const float sum_other = warp_sum(other), sum_own = __shfl_sync(0xffffffffu, sc, 31);
            const float L = sc + (warp == 1 ? sum_other : 0.f), Ltot = sum_own + sum_other;
            Ls[tid] = L;
            eLs[tid] = expf(L);
            wts[tid] = (t0 + tid < T) ? expf(fminf(Ltot - L, 0.f)) : 0.f;
        }
        // ---- the entering state as an MN-major B operand, hi and lo (and to HBM if asked for)
        {
            uint8_t *sh = sm + SM::off_sh + (D == 128 ? wg * (D * 128) : 0), *sl = sm + SM::off_sl + (D == 128 ? wg * (D * 128) : 0);
#pragma unroll
            for (int g = 0; g < NSG; ++g)
#pragma unroll
                for (int hi8 = 0; hi8 < 2; ++hi8) {
                    const int row = state_row(g, hi8);
#pragma unroll
                    for (int j = 0; j < NBO; ++j) {
                        uint32_t hi, lo;
                        split2(S[g][4 * j + 2 * hi8], S[g][4 * j + 2 * hi8 + 1], hi, lo);
                        const uint32_t off = swz(row, (D == 128 ? j : 4 * wg + j)) + 4 * fq;
                        *reinterpret_cast<uint32_t *>(sh + off) = hi;
                        *reinterpret_cast<uint32_t *>(sl + off) = lo;
                        if (p.sent != nullptr)
                            *reinterpret_cast<uint32_t *>(p.sent + (((size_t)bh * NC + c) * D + row) * D + ocol0 + 8 * j + 2 * fq) = hi;
                    }
                }
        }
        if (!mbar_wait(st ? bar_full1 : bar_full0, (c >> 1) & 1, 1)) { ok = false; }
        if (ROT_SMEM && ok && !mbar_wait(bar_rot, c & 1, 4)) ok = false;
        ok = __syncthreads_and(ok);                                   // one verdict for the whole CTA: every thread leaves the loop at the same point
        __syncthreads();                                              // L, e^L, w are visible; the tiles have landed for everyone
        const float aC = expf(Ls[TC_C - 1]);
        if (ok) {
            if constexpr (RAW) {
                // ---- plumbing in place: 8 lanes share a token row (one 16-byte piece per 64-column sub-tile each)
                const int cp = lane & 7;
#pragma unroll
                for (int which = 0; which < 3; ++which) {
                    uint8_t *tile = which == 0 ? qs_ptr : (which == 1 ? ks_ptr : vs_ptr);
#pragma unroll
                    for (int pass = 0; pass < 2; ++pass) {
                        const int row = 32 * pass + 4 * warp + (lane >> 3);
                        float x[SUB][8];
                        float ss = 0.f;
#pragma unroll
                        for (int s2 = 0; s2 < SUB; ++s2) {
                            const uint4 raw = *reinterpret_cast<const uint4 *>(tile + s2 * 8192 + swz(row, cp));
                            const __nv_bfloat162 *b2 = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 f = __bfloat1622float2(b2[i]);
                                x[s2][2 * i] = f.x; x[s2][2 * i + 1] = f.y;
                                ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
                            }
                        }
                        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
                        float inv = 1.0f / fmaxf(sqrtf(ss), 1e-12f);
                        const int t = min(t0 + row, T - 1);
                        if (which == 1) inv *= gts[row];
                        const float w = wts[row];
#pragma unroll
                        for (int s2 = 0; s2 < SUB; ++s2) {
                            float y[8];
                            if (which < 2) {
                                const float4 *rt = ROT_SMEM
                                    ? reinterpret_cast<const float4 *>(rot_sm + row * (D / 2) + cp * 4)
                                    : reinterpret_cast<const float4 *>(p.rot + ((size_t)h * p.rot_T + min(t, p.rot_T - 1)) * (D / 2) + s2 * 32 + cp * 4);
                                const float4 r01 = rt[0], r23 = rt[1];                 // (c0,s0,c1,s1), (c2,s2,c3,s3)
                                const float cs[4] = {r01.x, r01.z, r23.x, r23.z}, sn[4] = {r01.y, r01.w, r23.y, r23.w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    y[2 * i] = (x[s2][2 * i] * cs[i] - x[s2][2 * i + 1] * sn[i]) * inv;
                                    y[2 * i + 1] = (x[s2][2 * i] * sn[i] + x[s2][2 * i + 1] * cs[i]) * inv;
                                }
                            } else {
#pragma unroll
                                for (int i = 0; i < 8; ++i) y[i] = x[s2][i] * inv;
                            }
                            __nv_bfloat162 o2[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
                            const uint32_t off = s2 * 8192 + swz(row, cp);
                            *reinterpret_cast<uint4 *>(tile + off) = *reinterpret_cast<uint4 *>(o2);
                            if (which == 1) {                         // K * w from the ROUNDED k, hi and lo
                                float kw[8];
#pragma unroll
                                for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(o2[i]); kw[2 * i] = f.x * w; kw[2 * i + 1] = f.y * w; }
                                uint4 hi, lo;
                                split8(kw, hi, lo);
                                *reinterpret_cast<uint4 *>(sm + SM::off_kwh + off) = hi;
                                *reinterpret_cast<uint4 *>(sm + SM::off_kwl + off) = lo;
                            }
                        }
                    }
                }
            } else {
                // ---- K * w, hi and lo, in K's own layout
                for (int idx = tid; idx < TC_C * (D / 8); idx += NT) {
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
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- P, U, O2
        if (tid == 0 && ok) {
            tc_fence_after();
            constexpr uint32_t I_P = idesc_bf16(64, 64, 0, 0), I_U = idesc_bf16(D, D, 1, 1), I_O = idesc_bf16(64, D, 0, 1);
            // a descriptor's start-address field counts 16-byte units: stepping is an add on the low word
            const uint64_t dq = smem_desc(qs, 16, 1024), dk = smem_desc(ks, 16, 1024), dv = smem_desc(vs, 8192, 1024);
            const uint64_t dkwh = smem_desc(base + SM::off_kwh, 8192, 1024), dkwl = smem_desc(base + SM::off_kwl, 8192, 1024);
            const uint64_t dsh = smem_desc(base + SM::off_sh, D * 128, 1024), dsl = smem_desc(base + SM::off_sl, D * 128, 1024);
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {                        // P = Q K^T, K-major steps of 32 B inside a sub-tile
                const uint32_t ko = ((uint32_t)(k >> 2) * 8192u + (uint32_t)(k & 3) * 32u) >> 4;
                mma_bf16(tmem + TM_P, dq + ko, dk + ko, I_P, k > 0);
            }
#pragma unroll
            for (int k = 0; k < TC_C / 16; ++k)                       // U = (K w)^T V over the 64 tokens, 16 rows (2048 B) a step
                mma_bf16(tmem + TM_U, dkwh + k * 128, dv + k * 128, I_U, k > 0);
#pragma unroll
            for (int k = 0; k < TC_C / 16; ++k) mma_bf16(tmem + TM_U, dkwl + k * 128, dv + k * 128, I_U, 1);
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {                        // O2 = Q S (hi then lo); S rows are the key index
                const uint32_t qo = ((uint32_t)(k >> 2) * 8192u + (uint32_t)(k & 3) * 32u) >> 4;
                mma_bf16(tmem + TM_O2, dq + qo, dsh + k * 128, I_O, k > 0);
            }
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
                const uint32_t qo = ((uint32_t)(k >> 2) * 8192u + (uint32_t)(k & 3) * 32u) >> 4;
                mma_bf16(tmem + TM_O2, dq + qo, dsl + k * 128, I_O, 1);
            }
            mma_commit(bar_a);
        }
        if (ok && !mbar_wait(bar_a, c & 1, 2)) ok = false;
        ok = __syncthreads_and(ok);
        tc_fence_after();
        if (ok) {
            // ---- A = P * decay, causal; hi and lo rows of the K-major A operand
            float pv[16];
            tmem_ld_frag4(tmem + lane_base + TM_P + pcol0, pv);
            // ---- and the state leaving the chunk: S <- e^{L_C} S + U
            float uv[NSG][4 * NBO];
#pragma unroll
            for (int g = 0; g < NSG; ++g) tmem_ld_frag<NBO>(tmem + lane_base + ((uint32_t)(16 * g) << 16) + TM_U + ocol0, uv[g]);
            tmem_ld_wait();
            const float Lt0 = Ls[trow0] * LOG2E, Lt1 = Ls[trow1] * LOG2E;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int s0 = pcol0 + 8 * j + 2 * fq;
                const float Ls0 = Ls[s0] * LOG2E, Ls1 = Ls[s0 + 1] * LOG2E;
                const float a00 = (s0 <= trow0) ? pv[4 * j] * exp2f(fminf(Lt0 - Ls0, 0.f)) : 0.f;
                const float a01 = (s0 + 1 <= trow0) ? pv[4 * j + 1] * exp2f(fminf(Lt0 - Ls1, 0.f)) : 0.f;
                const float a10 = (s0 <= trow1) ? pv[4 * j + 2] * exp2f(fminf(Lt1 - Ls0, 0.f)) : 0.f;
                const float a11 = (s0 + 1 <= trow1) ? pv[4 * j + 3] * exp2f(fminf(Lt1 - Ls1, 0.f)) : 0.f;
                uint32_t hi, lo;
                split2(a00, a01, hi, lo);
                *reinterpret_cast<uint32_t *>(sm + SM::off_ah + swz(trow0, 4 * wg + j) + 4 * fq) = hi;
                *reinterpret_cast<uint32_t *>(sm + SM::off_al + swz(trow0, 4 * wg + j) + 4 * fq) = lo;
                split2(a10, a11, hi, lo);
                *reinterpret_cast<uint32_t *>(sm + SM::off_ah + swz(trow1, 4 * wg + j) + 4 * fq) = hi;
                *reinterpret_cast<uint32_t *>(sm + SM::off_al + swz(trow1, 4 * wg + j) + 4 * fq) = lo;
            }
#pragma unroll
            for (int g = 0; g < NSG; ++g)
#pragma unroll
                for (int j = 0; j < 4 * NBO; ++j) S[g][j] = fmaf(aC, S[g][j], uv[g][j]);
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- O1 = A V
        if (tid == 0 && ok) {
            tc_fence_after();
            constexpr uint32_t I_O = idesc_bf16(64, D, 0, 1);
            const uint64_t dah = smem_desc(base + SM::off_ah, 16, 1024), dal = smem_desc(base + SM::off_al, 16, 1024);
            const uint64_t dv = smem_desc(vs, 8192, 1024);
#pragma unroll
            for (int k = 0; k < TC_C / 16; ++k) mma_bf16(tmem + TM_O1, dah + k * 2, dv + k * 128, I_O, k > 0);
#pragma unroll
            for (int k = 0; k < TC_C / 16; ++k) mma_bf16(tmem + TM_O1, dal + k * 2, dv + k * 128, I_O, 1);
            mma_commit(bar_b);
        }
        if (ok && !mbar_wait(bar_b, c & 1, 3)) ok = false;
        ok = __syncthreads_and(ok);
        tc_fence_after();
        if (ROT_SMEM && tid == 0 && ok && c + 1 < NC) {              // A buffers are idle again: next chunk's (cos, sin) rows
            mbar_expect_tx(bar_rot, ROT_BYTES);
            bulk_load_1d(base + SM::off_ah, p.rot + ((size_t)h * p.rot_T + t0 + TC_C) * (D / 2), ROT_BYTES, bar_rot);
        }
        // ---- o = O1 + e^{L_t} O2 [* rsqrt(mean(o^2) + eps) * w]
        float ov[4 * NBO];
        {
            float o2v[4 * NBO];
            if (ok) {
                tmem_ld_frag<NBO>(tmem + lane_base + TM_O1 + ocol0, ov);
                tmem_ld_frag<NBO>(tmem + lane_base + TM_O2 + ocol0, o2v);
                tmem_ld_wait();
            }
            const float e0 = eLs[trow0], e1 = eLs[trow1];
#pragma unroll
            for (int j = 0; j < NBO; ++j) {
                ov[4 * j] = fmaf(e0, o2v[4 * j], ov[4 * j]);         ov[4 * j + 1] = fmaf(e0, o2v[4 * j + 1], ov[4 * j + 1]);
                ov[4 * j + 2] = fmaf(e1, o2v[4 * j + 2], ov[4 * j + 2]); ov[4 * j + 3] = fmaf(e1, o2v[4 * j + 3], ov[4 * j + 3]);
            }
        }
        float sc0 = 1.f, sc1 = 1.f;
        if (p.rms_w != nullptr) {                                     // uniform
            float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
            for (int j = 0; j < NBO; ++j) {
                ss0 = fmaf(ov[4 * j], ov[4 * j], fmaf(ov[4 * j + 1], ov[4 * j + 1], ss0));
                ss1 = fmaf(ov[4 * j + 2], ov[4 * j + 2], fmaf(ov[4 * j + 3], ov[4 * j + 3], ss1));
            }
            ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1); ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
            ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1); ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
            if (fq == 0) { red[wg * 64 + trow0] = ss0; red[wg * 64 + trow1] = ss1; }
            __syncthreads();                                          // a row's other half belongs to the other warpgroup
            sc0 = rsqrtf((red[trow0] + red[64 + trow0]) * (1.0f / D) + p.rms_eps);
            sc1 = rsqrtf((red[trow1] + red[64 + trow1]) * (1.0f / D) + p.rms_eps);
        }
        if (ok) {
#pragma unroll
            for (int hi8 = 0; hi8 < 2; ++hi8) {
                const int trow = hi8 ? trow1 : trow0;
                if (t0 + trow < T) {
                    const float sc = hi8 ? sc1 : sc0;
                    const size_t row = p.o_token_major ? ((size_t)b * T + t0 + trow) * p.H + h : (size_t)bh * T + t0 + trow;
                    const size_t off = row * D + ocol0 + 2 * fq;
#pragma unroll
                    for (int j = 0; j < NBO; ++j) {
                        float x0 = ov[4 * j + 2 * hi8] * sc, x1 = ov[4 * j + 2 * hi8 + 1] * sc;
                        if (p.rms_w != nullptr) { x0 *= rmsw[ocol0 + 8 * j + 2 * fq]; x1 *= rmsw[ocol0 + 8 * j + 2 * fq + 1]; }
                        if (p.o_is_f32) *reinterpret_cast<float2 *>((float *)p.o + off + 8 * j) = make_float2(x0, x1);
                        else *reinterpret_cast<__nv_bfloat162 *>((__nv_bfloat16 *)p.o + off + 8 * j) = __floats2bfloat162_rn(x0, x1);
                    }
                }
            }
        }
        tc_fence_before();
        __syncthreads();                                              // every TMEM read of this chunk is done before the next MMAs
    }
    // ---- final state
    if (ok) {
#pragma unroll
        for (int g = 0; g < NSG; ++g)
#pragma unroll
            for (int hi8 = 0; hi8 < 2; ++hi8) {
                float *dst = p.S_out + ((size_t)bh * D + state_row(g, hi8)) * D + ocol0 + 2 * fq;
#pragma unroll
                for (int j = 0; j < NBO; ++j)
                    *reinterpret_cast<float2 *>(dst + 8 * j) = make_float2(S[g][4 * j + 2 * hi8], S[g][4 * j + 2 * hi8 + 1]);
            }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, TM_COLS);
}

// ---------------------------------------------------------------------------------------------- host side
namespace {

template <int D, bool RAW>
int tc_go(const PrefillArgs &a, int o_dtype, cudaStream_t stream) {
    using SM = TcSmem<D>;
    CUtensorMap mq, mk, mv;
    const int BH = a.B * a.H;
    bool made;
    if (RAW)       // (B,T,H*D) views into the projection GEMM's output
        made = tc_make_map(&mq, a.q, a.B, a.T, (long long)a.H * D, a.raw_st, a.raw_sb) &&
               tc_make_map(&mk, a.k, a.B, a.T, (long long)a.H * D, a.raw_st, a.raw_sb) &&
               tc_make_map(&mv, a.v, a.B, a.T, (long long)a.H * D, a.raw_st, a.raw_sb);
    else           // contiguous (B*H, T, D)
        made = tc_make_map(&mq, a.q, BH, a.T, D, D, (long long)a.T * D) && tc_make_map(&mk, a.k, BH, a.T, D, D, (long long)a.T * D) &&
               tc_make_map(&mv, a.v, BH, a.T, D, D, (long long)a.T * D);
    if (!made) {
        set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled");
        return PGB_ERR_CUDA;
    }
    auto kern = prefill_tc_kernel<D, RAW>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::bytes);
    if (e != cudaSuccess) { set_cuda_error(e, "prefill_tc smem attribute"); return PGB_ERR_CUDA; }
    TcParams p{a.la, a.S0, a.theta, a.shift_dev, a.shift_host, a.o, a.S_out, a.sent, a.H, a.T, o_dtype == PGB_F32,
               (const __nv_bfloat16 *)a.la_raw, a.la_sb, a.la_st, a.decay_A, a.rms_w, a.rms_eps, a.o_token_major,
               (const __nv_bfloat16 *)a.gate_raw, (const float2 *)a.rot, a.rot_T};
    kern<<<(unsigned)BH, TC_NT, SM::bytes, stream>>>(mq, mk, mv, p);
    return check_launch("prefill_tc_kernel");
}

}  // namespace

// bf16 inputs, plain rule. (The delta rule runs in the fp32 kernel.)
bool prefill_tc_supported(int io_dtype, int D, bool delta) { return io_dtype == PGB_BF16 && !delta && (D == 64 || D == 128); }

int prefill_tc_launch(const PrefillArgs &a, int o_dtype, int D, cudaStream_t stream) {
    if (a.raw) return D == 64 ? tc_go<64, true>(a, o_dtype, stream) : tc_go<128, true>(a, o_dtype, stream);
    return D == 64 ? tc_go<64, false>(a, o_dtype, stream) : tc_go<128, false>(a, o_dtype, stream);
}

// table[h][t][i] = (cos, sin)(t * theta[h][i]) for t in [0, T): the rotation phases of one layer, built once
__global__ void rot_table_kernel(const float *__restrict__ theta, float2 *__restrict__ table, int H, int T, int half) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)H * T * half) return;
    const int pi = (int)(i % half), t = (int)((i / half) % T), h = (int)(i / ((long long)half * T));
    float sn, cs;
    sincosf((float)t * theta[(size_t)h * half + pi], &sn, &cs);
    table[i] = make_float2(cs, sn);
}

int rot_table_launch(const float *theta, float *table, int H, int T, int D, cudaStream_t stream) {
    const long long n = (long long)H * T * (D / 2);
    rot_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(theta, reinterpret_cast<float2 *>(table), H, T, D / 2);
    return check_launch("rot_table_kernel");
}


int tc_error_flag(int *out) { return tc_read_error_flag(out); }

// Self-test of the failure path every tensor-core kernel here relies on: one thread waits, with the same bounded loop, on
// an mbarrier that nothing ever arrives at; the wait runs out after `limit_cycles` of the SM clock, the error flag is set
// to 99 and the kernel returns normally, leaving the context usable.
__global__ void tc_wait_selftest_kernel(long long limit_cycles) {
    __shared__ __align__(8) unsigned long long bar;
    if (threadIdx.x != 0) return;
    const uint32_t b = smem_u32(&bar);
    mbar_init(b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const long long t0 = clock64();
    bool flipped = false;
    do {
        for (int i = 0; i < 32 && !flipped; ++i) flipped = mbar_try(b, 0);
    } while (!flipped && clock64() - t0 < limit_cycles);
    if (!flipped) atomicExch(&g_tc_error, 99);
}

int tc_wait_selftest_launch(long long limit_cycles, cudaStream_t stream) {
    tc_wait_selftest_kernel<<<1, 32, 0, stream>>>(limit_cycles);
    return check_launch("tc_wait_selftest_kernel");
}

}  // namespace pgb
