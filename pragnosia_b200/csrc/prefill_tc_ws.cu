// Plain-rule chunked prefill at head dim 64 as a warp-specialised pipeline: the chunk loop of prefill_tc.cu cut into
// roles that work on DIFFERENT chunks at the same time inside one CTA (one CTA per (sequence, head)).
//
//   stats  (warps 25-26) chunks c+2..c+4, alternating: the decay statistics (L, e^L, w and the key gate) -- a long dependent
//                        chain of shuffles and exponentials that nothing has to wait for when it runs ahead.
//   front  (warps 0-7)   chunk c+1: the plumbing on the TMA tiles (RAW mode: normalise, gate, rotate) and K*w head/tail --
//                        all shared memory to shared memory, no tensor-memory access.
//   issuer (warp 24)     one thread: TMA loads three chunks ahead, and the tcgen05.mma stream
//                        P(c+1) = Q K^T, U(c+1) = (K w)^T V   as soon as the front is done with chunk c+1.
//   issuer (warp 27)     one thread (a single thread issues an MMA only every few tens of cycles):
//                        O2(c) = Q S_c                         as soon as S_c is in shared memory,
//                        O1(c) = A V                           as soon as A(c) is.
//   back   (warps 8-15)  chunk c: scores -> A (decay mask, head/tail), S_{c+1} = e^{L_C} S_c + U in registers and to shared
//                        memory for the next chunk's O2.
//   tail   (warps 16-23) chunk c-1: o = O1 + e^{L} O2 with the per-head RMS norm, stores.
//
// Only S_{c+1} = e^{L_C} S_c + U is sequential across chunks; P, U, O1 and O2 are double-buffered in tensor memory, the
// Q/K/V tiles triple-buffered, K*w / A / S operand / rotation rows double-buffered, the statistics four deep. The roles
// meet only at mbarriers (every wait bounded; a wait that runs out sets g_tc_error and the CTA winds down). A waiter never
// falls two phases behind a barrier: each barrier's next completion depends on the waiter having passed. Arithmetic,
// operand layouts, precision (bf16 head + tail for every fp32 operand) and results are those of
// prefill_tc_kernel<64, RAW>; that kernel remains the head-dim-128 path.
#include "tc_common.cuh"

namespace pgb {

constexpr int WS_FRONT = 8, WS_BACK = 8, WS_TAIL = 8;                 // warps per role; a warp reaches tensor-memory lanes 32*(warp%4)..
constexpr int WS_ISSUER = WS_FRONT + WS_BACK + WS_TAIL;               // warp 24
constexpr int WS_STATS = WS_ISSUER + 1;                               // warps 25, 26
constexpr int WS_ISSUER_O = WS_STATS + 2;                             // warp 27
constexpr int WS_NT = (WS_ISSUER_O + 1) * 32;                         // 896 threads
constexpr int WS_D = 64;
constexpr float WS_LOG2E = 1.4426950408889634f;

struct WsSmem {
    static constexpr int TILE = 8192;                                 // one 64 x 64 bf16 tile
    static constexpr int off_stage = 0;                               // [3][Q, K, V]
    static constexpr int off_kw = off_stage + 3 * 3 * TILE;           // [2][head, tail]
    static constexpr int off_rot = off_kw + 2 * 2 * TILE;             // [2] 64 rows x 32 (cos, sin) pairs, fp32
    static constexpr int off_a = off_rot + 2 * 16384;                 // [2][head, tail]
    static constexpr int off_s = off_a + 2 * 2 * TILE;                // [2][head, tail]
    static constexpr int off_misc = off_s + 2 * 2 * TILE;
    static constexpr int bytes = off_misc + 6144 + 1024;
    // inside misc
    static constexpr int bar_full = 0, bar_empty = 24, bar_rot = 48, bar_ready = 64, bar_pu = 80, bar_s = 96, bar_a = 112,
                         bar_o = 128, bar_stats = 144, bar_done = 176, tmem_slot = 208, abort_tail = 216, bar_free = 232, bar_q = 256,
                         stats = 512, red = 4608, rmsw = 5632;
};

__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void named_sync(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }
// bounded wait whose verdict is the same for every lane of the warp (the lanes leave the chunk loop together)
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, int code) {
    if (__all_sync(0xffffffffu, mbar_test(bar, parity))) return true;     // the common case: already complete, no suspension
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, code)) != 0;
}
// one arrival per warp, after every lane's shared-memory writes are visible to the async proxy
__device__ __forceinline__ void warp_arrive(uint32_t bar, int lane) {
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}


template <bool RAW>
__global__ void __launch_bounds__(WS_NT, 1) prefill_tc_ws_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                                                                const __grid_constant__ CUtensorMap mv, TcParams p) {
    using SM = WsSmem;
    constexpr int D = WS_D;
    constexpr uint32_t TM_P = 0, TM_U = 128, TM_O1 = 256, TM_O2 = 384, TM_COLS = 512;   // each: two slots of 64 columns
    constexpr uint32_t STAGE_BYTES = 3 * SM::TILE, ROT_BYTES = 16384;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - smem_u32(smem_raw));
    uint8_t *misc = sm + SM::off_misc;
    const uint32_t mb = base + SM::off_misc;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(misc + SM::tmem_slot);
    float *stats = reinterpret_cast<float *>(misc + SM::stats);       // [4 chunks][L, e^L, w, gate][64]
    float *red = reinterpret_cast<float *>(misc + SM::red);           // [2 chunks][2 column halves][64]
    float *rmsw = reinterpret_cast<float *>(misc + SM::rmsw);         // [64]
    // The only named barriers are between the two tail warps that share a row (RMS norm). Such a pair leaves its chunk loop
    // together: a warp whose wait ran out raises the pair's flag before the barrier, both read it after. (A lone exit would
    // strand the partner at that barrier.) Every other meeting is an mbarrier with a bounded wait.
    volatile int *abort_tail = reinterpret_cast<volatile int *>(misc + SM::abort_tail);   // [4]
    auto bar_full = [&](int s) { return mb + SM::bar_full + 8 * s; };     // TMA -> front            stage c%3
    auto bar_empty = [&](int s) { return mb + SM::bar_empty + 8 * s; };   // products of c done      stage c%3
    auto bar_rot = [&](int s) { return mb + SM::bar_rot + 8 * s; };       // rotation rows -> front  slot c&1
    auto bar_ready = [&](int s) { return mb + SM::bar_ready + 8 * s; };   // front -> issuer         slot c&1
    auto bar_pu = [&](int s) { return mb + SM::bar_pu + 8 * s; };         // P, U done -> back       slot c&1
    auto bar_s = [&](int s) { return mb + SM::bar_s + 8 * s; };           // S_c published -> issuer slot c&1
    auto bar_a = [&](int s) { return mb + SM::bar_a + 8 * s; };           // A(c) written -> issuer  slot c&1
    auto bar_free = [&](int s) { return mb + SM::bar_free + 8 * s; };     // P, U read; P/U/K*w slot free     c&1
    auto bar_o = [&](int s) { return mb + SM::bar_o + 8 * s; };           // O1, O2 done -> tail, back        c&1
    auto bar_stats = [&](int s) { return mb + SM::bar_stats + 8 * s; };   // statistics -> everyone  slot c&3
    auto bar_done = [&](int s) { return mb + SM::bar_done + 8 * s; };     // tail through with chunk c        c&3
    auto bar_q = [&](int s) { return mb + SM::bar_q + 8 * s; };           // P, U issued: tiles of c final    c&3

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int bh = blockIdx.x, h = bh % p.H, b = bh / p.H;
    const int T = p.T, NC = (T + TC_C - 1) / TC_C;
    const int tma_c0 = RAW ? h * D : 0, tma_c2 = RAW ? b : bh;

    if (tid == 0) {
        for (int s = 0; s < 3; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 2); }   // empty: one commit per issuer
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_rot(s), 1); mbar_init(bar_ready(s), WS_FRONT); mbar_init(bar_pu(s), 1);
            mbar_init(bar_s(s), WS_BACK); mbar_init(bar_a(s), WS_BACK); mbar_init(bar_o(s), 1); mbar_init(bar_free(s), WS_BACK);
        }
        for (int s = 0; s < 4; ++s) { mbar_init(bar_stats(s), 1); mbar_init(bar_done(s), WS_TAIL); mbar_init(bar_q(s), 1); abort_tail[s] = 0; }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == WS_ISSUER) tmem_alloc(smem_u32(tmem_slot), TM_COLS);
    // Launched as a programmatic dependent: the set-up above (barriers, tensor memory) may overlap the tail of the kernel
    // before this one on the stream. No global memory is read or written before this wait -- not even the small constant
    // vectors, which that kernel may have produced (a dtype cast of the norm weight, say).
    pdl_wait();
    if (p.rms_w != nullptr && tid < D) rmsw[tid] = p.rms_w[tid];
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_launch_dependents();

    if (warp < WS_FRONT) {
        // =========================================================================================== front
        for (int c = 0; c < NC; ++c) {
            const int s2 = c & 1, s3 = c % 3;
            const float *wts = stats + (c & 3) * 256 + 128, *gts = wts + 64;
            // the K*w slot and the P / U accumulators were last used by chunk c-2: free once the back has read U(c-2)
            bool fine = c < 2 || mbar_wait_warp(bar_free(s2), ((c >> 1) + 1) & 1, 31);
            fine = fine && mbar_wait_warp(bar_stats(c & 3), (c >> 2) & 1, 34);
            fine = fine && mbar_wait_warp(bar_full(s3), (c / 3) & 1, 32);
            if (RAW) fine = fine && mbar_wait_warp(bar_rot(s2), (c >> 1) & 1, 33);
            if (!fine) break;                                         // the other roles run out of their own waits
            uint8_t *qs_ptr = sm + SM::off_stage + s3 * STAGE_BYTES, *ks_ptr = qs_ptr + SM::TILE, *vs_ptr = ks_ptr + SM::TILE;
            uint8_t *kwh = sm + SM::off_kw + s2 * 2 * SM::TILE, *kwl = kwh + SM::TILE;
            if constexpr (RAW) {
                const float2 *rot_sm = reinterpret_cast<const float2 *>(sm + SM::off_rot + s2 * ROT_BYTES);
                const int cp = lane & 7;
#pragma unroll 1                                                      // rolled: five roles share the instruction cache
                for (int pass = 0; pass < 2; ++pass) {
                    // every load of the pass first: the stores below may alias anything as far as the compiler can tell,
                    // and would otherwise chain the three tiles one behind the other
                    const int row = 32 * pass + 4 * warp + (lane >> 3);
                    const uint32_t off = swz(row, cp);
                    uint4 raw[3];
                    raw[0] = *reinterpret_cast<const uint4 *>(qs_ptr + off);
                    raw[1] = *reinterpret_cast<const uint4 *>(ks_ptr + off);
                    raw[2] = *reinterpret_cast<const uint4 *>(vs_ptr + off);
                    const float4 *rt = reinterpret_cast<const float4 *>(rot_sm + row * (D / 2) + cp * 4);
                    const float4 r01 = rt[0], r23 = rt[1];
                    const float cs[4] = {r01.x, r01.z, r23.x, r23.z}, sn[4] = {r01.y, r01.w, r23.y, r23.w};
                    const float wrow = wts[row], grow = gts[row];
                    uint4 outv[3], kwhi, kwlo;
#pragma unroll
                    for (int which = 0; which < 3; ++which) {
                        const __nv_bfloat162 *b2 = reinterpret_cast<const __nv_bfloat162 *>(&raw[which]);
                        float x[8], ss = 0.f;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 f = __bfloat1622float2(b2[i]);
                            x[2 * i] = f.x; x[2 * i + 1] = f.y;
                            ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
                        }
                        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
                        float inv = rsqrtf(fmaxf(ss, 1e-24f));        // 1 / max(|x|, 1e-12)
                        if (which == 1) inv *= grow;
                        float y[8];
                        if (which < 2) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                y[2 * i] = (x[2 * i] * cs[i] - x[2 * i + 1] * sn[i]) * inv;
                                y[2 * i + 1] = (x[2 * i] * sn[i] + x[2 * i + 1] * cs[i]) * inv;
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) y[i] = x[i] * inv;
                        }
                        __nv_bfloat162 *o2 = reinterpret_cast<__nv_bfloat162 *>(&outv[which]);
#pragma unroll
                        for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
                        if (which == 1) {                             // K * w from the ROUNDED k
                            float kw[8];
#pragma unroll
                            for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(o2[i]); kw[2 * i] = f.x * wrow; kw[2 * i + 1] = f.y * wrow; }
                            split8(kw, kwhi, kwlo);
                        }
                    }
                    *reinterpret_cast<uint4 *>(qs_ptr + off) = outv[0];
                    *reinterpret_cast<uint4 *>(ks_ptr + off) = outv[1];
                    *reinterpret_cast<uint4 *>(vs_ptr + off) = outv[2];
                    *reinterpret_cast<uint4 *>(kwh + off) = kwhi;
                    *reinterpret_cast<uint4 *>(kwl + off) = kwlo;
                }
            } else {
#pragma unroll
                for (int pass = 0; pass < 2; ++pass) {
                    const int idx = tid + pass * WS_FRONT * 32, r = idx >> 3;
                    const uint32_t off = swz(r, idx & 7);
                    const uint4 raw = *reinterpret_cast<const uint4 *>(ks_ptr + off);
                    const __nv_bfloat162 *b2 = reinterpret_cast<const __nv_bfloat162 *>(&raw);
                    const float w = wts[r];
                    float x[8];
#pragma unroll
                    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(b2[i]); x[2 * i] = f.x * w; x[2 * i + 1] = f.y * w; }
                    uint4 hi, lo;
                    split8(x, hi, lo);
                    *reinterpret_cast<uint4 *>(kwh + off) = hi;
                    *reinterpret_cast<uint4 *>(kwl + off) = lo;
                }
            }
            warp_arrive(bar_ready(s2), lane);
        }
    } else if (warp < WS_FRONT + WS_BACK) {
        // =========================================================================================== back
        const int bw = warp - WS_FRONT, wg = bw >> 2, sub = bw & 3;
        const int fr = lane >> 2, fq = lane & 3;
        const int row0 = 16 * sub + fr, row1 = row0 + 8;              // token rows of P and key rows of U / S
        const uint32_t lane_base = (uint32_t)(32 * sub) << 16;
        const int col0 = 32 * wg;                                     // this warp's half of every 64-column accumulator
        float S[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) S[j] = 0.f;
        if (p.S0 != nullptr) {
            const float shift = p.theta == nullptr ? 0.f : (p.shift_dev != nullptr ? *p.shift_dev : p.shift_host);
#pragma unroll
            for (int hi8 = 0; hi8 < 2; ++hi8) {
                const int row = hi8 ? row1 : row0;
                const float *src = p.S0 + ((size_t)bh * D + row) * D + col0 + 2 * fq;
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
                    S[4 * j + 2 * hi8] = x0; S[4 * j + 2 * hi8 + 1] = x1;
                }
            }
        }
        auto publish_state = [&](int c) {                             // S_c as the MN-major B operand of O2(c), head and tail
            uint8_t *sh = sm + SM::off_s + (c & 1) * 2 * SM::TILE, *sl = sh + SM::TILE;
#pragma unroll
            for (int hi8 = 0; hi8 < 2; ++hi8) {
                const int row = hi8 ? row1 : row0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t hi, lo;
                    split2(S[4 * j + 2 * hi8], S[4 * j + 2 * hi8 + 1], hi, lo);
                    const uint32_t off = swz(row, 4 * wg + j) + 4 * fq;
                    *reinterpret_cast<uint32_t *>(sh + off) = hi;
                    *reinterpret_cast<uint32_t *>(sl + off) = lo;
                    if (p.sent != nullptr)
                        *reinterpret_cast<uint32_t *>(p.sent + (((size_t)bh * NC + c) * D + row) * D + col0 + 8 * j + 2 * fq) = hi;
                }
            }
            warp_arrive(bar_s(c & 1), lane);
        };
        publish_state(0);
        bool ok = true;
        for (int c = 0; c < NC; ++c) {
            const int s2 = c & 1;
            const float *Ls = stats + (c & 3) * 256;
            ok = mbar_wait_warp(bar_stats(c & 3), (c >> 2) & 1, 41) && mbar_wait_warp(bar_pu(s2), (c >> 1) & 1, 42);
            if (!ok) break;
            tc_fence_after();
            float pv[16];
            tmem_ld_frag4(tmem + lane_base + TM_P + 64 * s2 + col0, pv);
            // every statistics load before the stores (which the compiler must assume alias them), and U only after the
            // scores pass: both keep the sixteen score chains independent and within the register budget
            float2 Lp[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                Lp[j] = *reinterpret_cast<const float2 *>(Ls + col0 + 8 * j + 2 * fq);
                Lp[j].x *= WS_LOG2E; Lp[j].y *= WS_LOG2E;
            }
            const float Lt0 = Ls[row0] * WS_LOG2E, Lt1 = Ls[row1] * WS_LOG2E;
            const float aC = expf(Ls[TC_C - 1]);
            tmem_ld_wait();
            {
                uint8_t *ah = sm + SM::off_a + s2 * 2 * SM::TILE, *al = ah + SM::TILE;
                uint32_t hi[8], lo[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int s0 = col0 + 8 * j + 2 * fq;
                    const float a00 = (s0 <= row0) ? pv[4 * j] * fast_exp2(fminf(Lt0 - Lp[j].x, 0.f)) : 0.f;
                    const float a01 = (s0 + 1 <= row0) ? pv[4 * j + 1] * fast_exp2(fminf(Lt0 - Lp[j].y, 0.f)) : 0.f;
                    const float a10 = (s0 <= row1) ? pv[4 * j + 2] * fast_exp2(fminf(Lt1 - Lp[j].x, 0.f)) : 0.f;
                    const float a11 = (s0 + 1 <= row1) ? pv[4 * j + 3] * fast_exp2(fminf(Lt1 - Lp[j].y, 0.f)) : 0.f;
                    split2(a00, a01, hi[2 * j], lo[2 * j]);
                    split2(a10, a11, hi[2 * j + 1], lo[2 * j + 1]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t o0 = swz(row0, 4 * wg + j) + 4 * fq, o1 = swz(row1, 4 * wg + j) + 4 * fq;
                    *reinterpret_cast<uint32_t *>(ah + o0) = hi[2 * j];     *reinterpret_cast<uint32_t *>(al + o0) = lo[2 * j];
                    *reinterpret_cast<uint32_t *>(ah + o1) = hi[2 * j + 1]; *reinterpret_cast<uint32_t *>(al + o1) = lo[2 * j + 1];
                }
            }
            warp_arrive(bar_a(s2), lane);                             // A(c) is there: O1(c) may go
            float uv[16];
            tmem_ld_frag4(tmem + lane_base + TM_U + 64 * s2 + col0, uv);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_free(s2));                 // P / U / K*w slot c&1 may be refilled
#pragma unroll
            for (int j = 0; j < 16; ++j) S[j] = fmaf(aC, S[j], uv[j]);
            if (c + 1 < NC) {
                // S slot (c+1)&1 was the operand of O2(c-1): finished once O1(c-1), issued after it, is
                if (c >= 1 && !mbar_wait_warp(bar_o((c - 1) & 1), ((c - 1) >> 1) & 1, 44)) { ok = false; break; }
                publish_state(c + 1);
            }
        }
        if (ok) {
#pragma unroll
            for (int hi8 = 0; hi8 < 2; ++hi8) {
                float *dst = p.S_out + ((size_t)bh * D + (hi8 ? row1 : row0)) * D + col0 + 2 * fq;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *reinterpret_cast<float2 *>(dst + 8 * j) = make_float2(S[4 * j + 2 * hi8], S[4 * j + 2 * hi8 + 1]);
            }
        }
    } else if (warp < WS_ISSUER) {
        // =========================================================================================== tail
        const int tw = warp - WS_FRONT - WS_BACK, wg = tw >> 2, sub = tw & 3;
        const int fr = lane >> 2, fq = lane & 3;
        const int row0 = 16 * sub + fr, row1 = row0 + 8;              // token rows of O1 / O2
        const uint32_t lane_base = (uint32_t)(32 * sub) << 16;
        const int col0 = 32 * wg;
        bool alive = true;                                            // false once a wait of this warp ran out: no more waiting
        for (int c = 0; c < NC; ++c) {
            const int t0 = c * TC_C, s2 = c & 1;
            const float *eLs = stats + (c & 3) * 256 + 64;
            bool fine = alive && mbar_wait_warp(bar_stats(c & 3), (c >> 2) & 1, 45) && mbar_wait_warp(bar_o(s2), (c >> 1) & 1, 43);
            if (!fine) { alive = false; abort_tail[sub] = 1; }
            tc_fence_after();
            float ov[16], o2v[16];
            tmem_ld_frag4(tmem + lane_base + TM_O1 + 64 * s2 + col0, ov);
            tmem_ld_frag4(tmem + lane_base + TM_O2 + 64 * s2 + col0, o2v);
            tmem_ld_wait();
            tc_fence_before();
            const float e0 = eLs[row0], e1 = eLs[row1];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                ov[4 * j] = fmaf(e0, o2v[4 * j], ov[4 * j]);             ov[4 * j + 1] = fmaf(e0, o2v[4 * j + 1], ov[4 * j + 1]);
                ov[4 * j + 2] = fmaf(e1, o2v[4 * j + 2], ov[4 * j + 2]); ov[4 * j + 3] = fmaf(e1, o2v[4 * j + 3], ov[4 * j + 3]);
            }
            float sc0 = 1.f, sc1 = 1.f;
            if (p.rms_w != nullptr) {
                float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    ss0 = fmaf(ov[4 * j], ov[4 * j], fmaf(ov[4 * j + 1], ov[4 * j + 1], ss0));
                    ss1 = fmaf(ov[4 * j + 2], ov[4 * j + 2], fmaf(ov[4 * j + 3], ov[4 * j + 3], ss1));
                }
                ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1); ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
                ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1); ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
                float *rd = red + s2 * 128;                           // two slots: chunk c+1 does not overwrite what c still reads
                if (fq == 0) { rd[wg * 64 + row0] = ss0; rd[wg * 64 + row1] = ss1; }
                named_sync(2 + sub, 64);                              // a row's other half belongs to warp sub of the other group
                sc0 = rsqrtf((rd[row0] + rd[64 + row0]) * (1.0f / D) + p.rms_eps);
                sc1 = rsqrtf((rd[row1] + rd[64 + row1]) * (1.0f / D) + p.rms_eps);
                if (abort_tail[sub]) fine = false;                    // read after the barrier: the same for both warps of the pair
            }
            if (!fine) break;
#pragma unroll
            for (int hi8 = 0; hi8 < 2; ++hi8) {
                const int trow = hi8 ? row1 : row0;
                if (t0 + trow < T) {
                    const float sc = hi8 ? sc1 : sc0;
                    const size_t row = p.o_token_major ? ((size_t)b * T + t0 + trow) * p.H + h : (size_t)bh * T + t0 + trow;
                    const size_t off = row * D + col0 + 2 * fq;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float x0 = ov[4 * j + 2 * hi8] * sc, x1 = ov[4 * j + 2 * hi8 + 1] * sc;
                        if (p.rms_w != nullptr) { x0 *= rmsw[col0 + 8 * j + 2 * fq]; x1 *= rmsw[col0 + 8 * j + 2 * fq + 1]; }
                        if (p.o_is_f32) *reinterpret_cast<float2 *>((float *)p.o + off + 8 * j) = make_float2(x0, x1);
                        else *reinterpret_cast<__nv_bfloat162 *>((__nv_bfloat16 *)p.o + off + 8 * j) = __floats2bfloat162_rn(x0, x1);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_done(c & 3));
        }
    } else if (warp == WS_STATS || warp == WS_STATS + 1) {
        // =========================================================================================== statistics
        // two warps take alternate chunks; lane l owns tokens l and l + 32 of the chunk: two interleaved warp scans
        const float *la = p.la != nullptr ? p.la + (size_t)bh * T : nullptr;
        const float expA = p.decay_A != nullptr ? expf(p.decay_A[h]) : 1.f;
        auto fetch_decay = [&](int t) -> float {
            if (t >= T) return 0.f;
            if (p.la_raw != nullptr) return __bfloat162float(p.la_raw[(size_t)b * p.aux_sb + (size_t)t * p.aux_st + h]);
            return la[t];
        };
        auto fetch_gate = [&](int t) -> float {
            if (!RAW || p.gate_raw == nullptr || t >= T) return 0.f;
            return __bfloat162float(p.gate_raw[(size_t)b * p.aux_sb + (size_t)t * p.aux_st + h]);
        };
        const int first = warp - WS_STATS;
        float nx_lo = fetch_decay(first * TC_C + lane), nx_hi = fetch_decay(first * TC_C + lane + 32);
        float ng_lo = fetch_gate(first * TC_C + lane), ng_hi = fetch_gate(first * TC_C + lane + 32);
        for (int c = first; c < NC; c += 2) {
            const int t0 = c * TC_C;
            float *Ls = stats + (c & 3) * 256, *eLs = Ls + 64, *wts = eLs + 64, *gts = wts + 64;
            // the slot was last used by chunk c-4: the tail, its last reader, is through with it
            if (c >= 4 && !mbar_wait_warp(bar_done(c & 3), ((c >> 2) + 1) & 1, 61)) break;
            auto log_decay = [&](float raw, int r) -> float {
                if (t0 + r >= T) return 0.f;
                return p.la_raw != nullptr ? -fast_softplus(raw) * expA : raw;
            };
            float sl = log_decay(nx_lo, lane), sh = log_decay(nx_hi, lane + 32);
            if (RAW) {
                gts[lane] = p.gate_raw != nullptr ? fast_sigmoid(ng_lo) : 1.f;
                gts[lane + 32] = p.gate_raw != nullptr ? fast_sigmoid(ng_hi) : 1.f;
            }
            nx_lo = fetch_decay(t0 + 2 * TC_C + lane); nx_hi = fetch_decay(t0 + 2 * TC_C + lane + 32);
            ng_lo = fetch_gate(t0 + 2 * TC_C + lane);  ng_hi = fetch_gate(t0 + 2 * TC_C + lane + 32);
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float nl = __shfl_up_sync(0xffffffffu, sl, o), nh = __shfl_up_sync(0xffffffffu, sh, o);
                if (lane >= o) { sl += nl; sh += nh; }
            }
            const float tot_lo = __shfl_sync(0xffffffffu, sl, 31);
            sh += tot_lo;
            const float Ltot = __shfl_sync(0xffffffffu, sh, 31);
            Ls[lane] = sl; Ls[lane + 32] = sh;
            eLs[lane] = expf(sl); eLs[lane + 32] = expf(sh);
            wts[lane] = (t0 + lane < T) ? expf(fminf(Ltot - sl, 0.f)) : 0.f;
            wts[lane + 32] = (t0 + lane + 32 < T) ? expf(fminf(Ltot - sh, 0.f)) : 0.f;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_stats(c & 3));
        }
    } else if (warp == WS_ISSUER && lane == 0) {
        // =========================================================================================== issuer: loads, P, U
        constexpr uint32_t I_P = idesc_bf16(64, 64, 0, 0), I_U = idesc_bf16(64, 64, 1, 1);
        auto load_chunk = [&](int c) {
            const int s3 = c % 3;
            const uint32_t sb = base + SM::off_stage + s3 * STAGE_BYTES;
            mbar_expect_tx(bar_full(s3), STAGE_BYTES);
            tma_load_3d(sb, &mq, bar_full(s3), tma_c0, c * TC_C, tma_c2);
            tma_load_3d(sb + SM::TILE, &mk, bar_full(s3), tma_c0, c * TC_C, tma_c2);
            tma_load_3d(sb + 2 * SM::TILE, &mv, bar_full(s3), tma_c0, c * TC_C, tma_c2);
        };
        auto load_rot = [&](int c) {
            if (!RAW) return;
            mbar_expect_tx(bar_rot(c & 1), ROT_BYTES);
            bulk_load_1d(base + SM::off_rot + (c & 1) * ROT_BYTES, p.rot + ((size_t)h * p.rot_T + (size_t)c * TC_C) * (D / 2), ROT_BYTES,
                         bar_rot(c & 1));
        };
        int tma_c = 0, pu_c = 0;
        for (; tma_c < 3 && tma_c < NC; ++tma_c) load_chunk(tma_c);
        for (int c = 0; c < 2 && c < NC; ++c) load_rot(c);
        uint32_t idle = 0;
        while (pu_c < NC) {
            bool progress = false;
            if (tma_c < NC && mbar_test(bar_empty(tma_c % 3), ((tma_c / 3) + 1) & 1)) { load_chunk(tma_c); ++tma_c; progress = true; }
            if (mbar_test(bar_ready(pu_c & 1), (pu_c >> 1) & 1)) {
                const int c = pu_c, s2 = c & 1;
                const uint32_t sb = base + SM::off_stage + (c % 3) * STAGE_BYTES;
                const uint64_t dq = smem_desc(sb, 16, 1024), dk = smem_desc(sb + SM::TILE, 16, 1024), dv = smem_desc(sb + 2 * SM::TILE, 8192, 1024);
                const uint64_t dkwh = smem_desc(base + SM::off_kw + s2 * 2 * SM::TILE, 8192, 1024), dkwl = dkwh + (SM::TILE >> 4);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16(tmem + TM_P + 64 * s2, dq + k * 2, dk + k * 2, I_P, k > 0);
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16(tmem + TM_U + 64 * s2, dkwh + k * 128, dv + k * 128, I_U, k > 0);
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16(tmem + TM_U + 64 * s2, dkwl + k * 128, dv + k * 128, I_U, 1);
                mma_commit(bar_pu(s2));
                mma_commit(bar_empty(c % 3));                         // this issuer's half: P and U have read the chunk's tiles
                mbar_arrive(bar_q(c & 3));                            // the other issuer may use the chunk's Q and V tiles
                if (c + 2 < NC) load_rot(c + 2);                      // the front is done with this slot's rotation rows
                ++pu_c; progress = true;
            }
            if (progress) idle = 0;
            else {
                if (++idle > (TC_WAIT_LIMIT >> 2)) { atomicExch(&g_tc_error, 51); break; }
                __nanosleep(20);                                      // leave the issue slots to the working warps
            }
        }
        // the last loads were issued inside the loop: tma_c == NC by the time pu_c == NC (a chunk's P, U need its tiles)
    } else if (warp == WS_ISSUER_O && lane == 0) {
        // =========================================================================================== issuer: O2, O1
        constexpr uint32_t I_O = idesc_bf16(64, 64, 0, 1);
        int q_c = 0, o2_c = 0, o1_c = 0;
        uint32_t idle = 0;
        while (o1_c < NC) {
            bool progress = false;
            // bar_q has four slots: its completion c+4 needs the back at chunk c+2, which needs O1(c) from this loop,
            // so this thread is never two phases behind it
            if (q_c < NC && mbar_test(bar_q(q_c & 3), (q_c >> 2) & 1)) { ++q_c; progress = true; }
            // O2(c) and O1(c) go to tensor-memory slot c&1, which the tail has drained once chunk c-2 is finished
            if (o2_c < q_c && mbar_test(bar_s(o2_c & 1), (o2_c >> 1) & 1) &&
                (o2_c < 2 || mbar_test(bar_done((o2_c - 2) & 3), ((o2_c - 2) >> 2) & 1))) {
                const int c = o2_c;
                const uint64_t dq = smem_desc(base + SM::off_stage + (c % 3) * STAGE_BYTES, 16, 1024);
                const uint64_t dsh = smem_desc(base + SM::off_s + (c & 1) * 2 * SM::TILE, 16, 1024), dsl = dsh + (SM::TILE >> 4);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16(tmem + TM_O2 + 64 * (c & 1), dq + k * 2, dsh + k * 128, I_O, k > 0);
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16(tmem + TM_O2 + 64 * (c & 1), dq + k * 2, dsl + k * 128, I_O, 1);
                ++o2_c; progress = true;
            }
            if (o1_c < o2_c && mbar_test(bar_a(o1_c & 1), (o1_c >> 1) & 1)) {
                const int c = o1_c;
                const uint64_t dv = smem_desc(base + SM::off_stage + (c % 3) * STAGE_BYTES + 2 * SM::TILE, 8192, 1024);
                const uint64_t dah = smem_desc(base + SM::off_a + (c & 1) * 2 * SM::TILE, 16, 1024), dal = dah + (SM::TILE >> 4);
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16(tmem + TM_O1 + 64 * (c & 1), dah + k * 2, dv + k * 128, I_O, k > 0);
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_bf16(tmem + TM_O1 + 64 * (c & 1), dal + k * 2, dv + k * 128, I_O, 1);
                mma_commit(bar_o(c & 1));
                mma_commit(bar_empty(c % 3));                         // this issuer's half: O2 and O1 have read the chunk's tiles
                ++o1_c; progress = true;
            }
            if (progress) idle = 0;
            else {
                if (++idle > (TC_WAIT_LIMIT >> 2)) { atomicExch(&g_tc_error, 52); break; }
                __nanosleep(20);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == WS_ISSUER) tmem_dealloc(tmem, TM_COLS);
}

int prefill_tc_ws_launch(const PrefillArgs &a, int o_dtype, cudaStream_t stream) {
    constexpr int D = WS_D;
    CUtensorMap mq, mk, mv;
    const int BH = a.B * a.H;
    bool made;
    if (a.raw)
        made = tc_make_map(&mq, a.q, a.B, a.T, (long long)a.H * D, a.raw_st, a.raw_sb) &&
               tc_make_map(&mk, a.k, a.B, a.T, (long long)a.H * D, a.raw_st, a.raw_sb) &&
               tc_make_map(&mv, a.v, a.B, a.T, (long long)a.H * D, a.raw_st, a.raw_sb);
    else
        made = tc_make_map(&mq, a.q, BH, a.T, D, D, (long long)a.T * D) && tc_make_map(&mk, a.k, BH, a.T, D, D, (long long)a.T * D) &&
               tc_make_map(&mv, a.v, BH, a.T, D, D, (long long)a.T * D);
    if (!made) { set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled"); return PGB_ERR_CUDA; }
    TcParams p{a.la, a.S0, a.theta, a.shift_dev, a.shift_host, a.o, a.S_out, a.sent, a.H, a.T, o_dtype == PGB_F32,
               (const __nv_bfloat16 *)a.la_raw, a.la_sb, a.la_st, a.decay_A, a.rms_w, a.rms_eps, a.o_token_major,
               (const __nv_bfloat16 *)a.gate_raw, (const float2 *)a.rot, a.rot_T};
    cudaError_t e;
    if (a.raw) {
        e = cudaFuncSetAttribute(prefill_tc_ws_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, WsSmem::bytes);
        if (e != cudaSuccess) { set_cuda_error(e, "prefill_tc_ws smem attribute"); return PGB_ERR_CUDA; }
        e = pdl_launch(prefill_tc_ws_kernel<true>, dim3((unsigned)BH), dim3(WS_NT), (size_t)WsSmem::bytes, stream, mq, mk, mv, p);
    } else {
        e = cudaFuncSetAttribute(prefill_tc_ws_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, WsSmem::bytes);
        if (e != cudaSuccess) { set_cuda_error(e, "prefill_tc_ws smem attribute"); return PGB_ERR_CUDA; }
        e = pdl_launch(prefill_tc_ws_kernel<false>, dim3((unsigned)BH), dim3(WS_NT), (size_t)WsSmem::bytes, stream, mq, mk, mv, p);
    }
    if (e != cudaSuccess) { set_cuda_error(e, "prefill_tc_ws launch"); return PGB_ERR_CUDA; }
    return check_launch("prefill_tc_ws_kernel");
}

int tc_ws_error_flag(int *out) { return tc_read_error_flag(out); }

}  // namespace pgb
