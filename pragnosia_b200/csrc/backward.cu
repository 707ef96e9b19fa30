// Backward kernels of the two simplest operators on the path, for callers that train through them:
//
//   lambda_scan_bwd   the adjoint of h_t = lambda_t h_{t-1} + u_t (reference: src/scan_kernel.py:54-101 _bwd, wired by
//                     _Scan.backward :121-140). The adjoint state obeys the same kind of recurrence run backwards in time,
//                     a_{t-1} = conj(lambda_t) a_t + g_{t-1}, so it is the forward kernel's chunked shuffle scan on the
//                     reversed sequence; with R_t h_{t-1} = h_t - (u_t, 0) the three per-token gradients are
//                         du_t = Re a_t,   dlogmag_t = a_t . (h_t - u_t),   dang_t = a_t . i (h_t - u_t).
//   prep_bwd          the gradient of the normalise / gate / rotate plumbing (reference: src/assoc_kernel.py:774-826
//                     _prep_bwd): with u = x / |x|, r = R(ang) u and g the gradient on r: du = R^T g,
//                     dx = (du - u (u . du)) / |x|, d ang = g2 r1 - g1 r2 per pair; theta's gradient is the sum of
//                     pos * d ang over batch and time, written as one partial per CTA and summed by the caller.
#include "common.cuh"

namespace pgb {

// ---------------------------------------------------------------------------------------------------- lambda scan adjoint
constexpr int LB_SEG = 4, LB_WARPS = 4;

template <int TS>
__global__ void __launch_bounds__(LB_WARPS * 32)
lambda_scan_bwd_kernel(const float *__restrict__ g, const float *__restrict__ u, const float *__restrict__ lm, const float *__restrict__ an,
                       long long an_sb, long long an_st, const float *__restrict__ hr_all, const float *__restrict__ hi_all,
                       const float *__restrict__ gli, float *__restrict__ du, float *__restrict__ dlm, float *__restrict__ dan,
                       float *__restrict__ dh0r, float *__restrict__ dh0i, int B, int T, int D) {
    constexpr int CQ = 32 / TS;
    constexpr unsigned FULL = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int wpb = (D + CQ - 1) / CQ;                                // warps per batch row
    const long long wg = (long long)blockIdx.x * LB_WARPS + (threadIdx.x >> 5);
    if (wg >= (long long)B * wpb) return;                             // a whole warp leaves together
    const int b = (int)(wg / wpb), cq = lane % CQ, seg = lane / CQ;
    const int d = (int)(wg % wpb) * CQ + cq;
    const bool live = d < D;
    const size_t row0 = (size_t)b * T;
    float ar = 0.f, ai = (live && gli != nullptr) ? gli[(size_t)b * D + d] : 0.f;   // adjoint state entering the tile (from later times)

    for (int r0 = 0; r0 < T; r0 += TS * LB_SEG) {
        const int rb = r0 + seg * LB_SEG;                             // reversed step index; time t = T - 1 - r
        float c[LB_SEG], s[LB_SEG], x[LB_SEG];
#pragma unroll
        for (int i = 0; i < LB_SEG; ++i) {
            const int t = T - 1 - (rb + i);
            c[i] = 1.f; s[i] = 0.f; x[i] = 0.f;                       // steps before time 0, and the first (latest) step: the identity
            if (live && t >= 0) {
                x[i] = g[(row0 + t) * D + d];
                if (t + 1 < T) {
                    const float mag = expf(lm[(row0 + t + 1) * D + d]);
                    float sn, cs;
                    sincosf(an[(size_t)b * an_sb + (size_t)(t + 1) * an_st + d], &sn, &cs);
                    c[i] = mag * cs; s[i] = -mag * sn;                 // conj(lambda_{t+1})
                }
            }
        }
        float hsr = ar, hsi = ai;
        if constexpr (TS > 1) {
            float Ar = 1.f, Ai = 0.f, Br = 0.f, Bi = 0.f;             // this segment's affine map a -> A a + B
#pragma unroll
            for (int i = 0; i < LB_SEG; ++i) {
                const float nbr = c[i] * Br - s[i] * Bi + x[i], nbi = s[i] * Br + c[i] * Bi;
                const float nar = c[i] * Ar - s[i] * Ai, nai = s[i] * Ar + c[i] * Ai;
                Br = nbr; Bi = nbi; Ar = nar; Ai = nai;
            }
#pragma unroll
            for (int off = 1; off < TS; off <<= 1) {
                const float par = __shfl_up_sync(FULL, Ar, off * CQ), pai = __shfl_up_sync(FULL, Ai, off * CQ);
                const float pbr = __shfl_up_sync(FULL, Br, off * CQ), pbi = __shfl_up_sync(FULL, Bi, off * CQ);
                if (seg >= off) {
                    const float nbr = Ar * pbr - Ai * pbi + Br, nbi = Ai * pbr + Ar * pbi + Bi;
                    const float nar = Ar * par - Ai * pai, nai = Ai * par + Ar * pai;
                    Br = nbr; Bi = nbi; Ar = nar; Ai = nai;
                }
            }
            float ear = __shfl_up_sync(FULL, Ar, CQ), eai = __shfl_up_sync(FULL, Ai, CQ);
            float ebr = __shfl_up_sync(FULL, Br, CQ), ebi = __shfl_up_sync(FULL, Bi, CQ);
            if (seg == 0) { ear = 1.f; eai = 0.f; ebr = 0.f; ebi = 0.f; }
            hsr = ear * ar - eai * ai + ebr;
            hsi = eai * ar + ear * ai + ebi;
        }
#pragma unroll
        for (int i = 0; i < LB_SEG; ++i) {
            const int t = T - 1 - (rb + i);
            const float nr = c[i] * hsr - s[i] * hsi + x[i], ni = s[i] * hsr + c[i] * hsi;
            hsr = nr; hsi = ni;
            if (live && t >= 0) {
                const size_t off = (row0 + t) * D + d;
                const float rr = hr_all[off] - u[off], ri = hi_all[off];      // lambda_t h_{t-1}
                du[off] = nr;
                dlm[off] = nr * rr + ni * ri;
                dan[off] = ni * rr - nr * ri;
            }
        }
        if constexpr (TS > 1) {
            ar = __shfl_sync(FULL, hsr, (TS - 1) * CQ + cq);
            ai = __shfl_sync(FULL, hsi, (TS - 1) * CQ + cq);
        } else {
            ar = hsr; ai = hsi;
        }
    }
    if (live && seg == 0 && dh0r != nullptr) {                        // a_{-1} = conj(lambda_0) a_0
        const float mag = expf(lm[row0 * D + d]);
        float sn, cs;
        sincosf(an[(size_t)b * an_sb + d], &sn, &cs);
        dh0r[(size_t)b * D + d] = mag * (cs * ar + sn * ai);
        dh0i[(size_t)b * D + d] = mag * (cs * ai - sn * ar);
    }
}

int lambda_scan_bwd_launch(const float *g, const float *u, const float *lm, const float *an, long long sb, long long st,
                           const float *hr_all, const float *hi_all, const float *gli, float *du, float *dlm, float *dan,
                           float *dh0r, float *dh0i, int B, int T, int D, cudaStream_t stream) {
    // many channels: one lane per channel walks its sequence; few: 8 time segments per warp share the walk
    const bool wide = (long long)B * D >= 148LL * 8 * 32 || T <= 2 * LB_SEG;
    const int cq = wide ? 32 : 4;
    const long long warps = (long long)B * ((D + cq - 1) / cq), ctas = (warps + LB_WARPS - 1) / LB_WARPS;
    if (ctas > 0x7fffffffLL) return PGB_ERR_TOO_LARGE;
    if (wide)
        lambda_scan_bwd_kernel<1><<<(unsigned)ctas, LB_WARPS * 32, 0, stream>>>(g, u, lm, an, sb, st, hr_all, hi_all, gli, du, dlm, dan, dh0r, dh0i, B, T, D);
    else
        lambda_scan_bwd_kernel<8><<<(unsigned)ctas, LB_WARPS * 32, 0, stream>>>(g, u, lm, an, sb, st, hr_all, hi_all, gli, du, dlm, dan, dh0r, dh0i, B, T, D);
    return check_launch("lambda_scan_bwd_kernel");
}

// ---------------------------------------------------------------------------------------------------- prep backward
constexpr int PB_WARPS = 8;                                           // consecutive tokens of one (sequence, head) per CTA

template <typename T_, int PER>
__device__ __forceinline__ void pb_ld(float (&d)[PER], const T_ *p) {
#pragma unroll
    for (int i = 0; i < PER; ++i) d[i] = to_f32(p[i]);
}
template <typename T_, int PER>
__device__ __forceinline__ void pb_st(T_ *p, const float (&d)[PER]) {
#pragma unroll
    for (int i = 0; i < PER; ++i) from_f32(p[i], d[i]);
}

// qp, kp, vp: TIN views (B,T,H,D) with element strides (sb, st, sh);  dq, dk, dv: TG, contiguous (B,H,T,D)
// dqp, dkp, dvp: TIN, contiguous (B,T,H,D);  dgl fp32 (B,T,H);  dth_part fp32 [B * NT][H][D/2], NT = ceil(T / PB_WARPS)
template <typename TIN, typename TG, int D>
__global__ void __launch_bounds__(PB_WARPS * 32)
prep_bwd_kernel(const TIN *__restrict__ qp, const TIN *__restrict__ kp, const TIN *__restrict__ vp, long long sb, long long st, long long sh,
                const TIN *__restrict__ gate, long long gsb, long long gst, const float *__restrict__ theta, const long long *__restrict__ pos,
                const TG *__restrict__ dq, const TG *__restrict__ dk, const TG *__restrict__ dv, TIN *__restrict__ dqp, TIN *__restrict__ dkp,
                TIN *__restrict__ dvp, float *__restrict__ dgl, float *__restrict__ dth_part, int T, int H, int NT) {
    constexpr int PER = D / 32, NP = PER / 2;
    __shared__ float part[PB_WARPS][D / 2];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pt = blockIdx.x, bh = blockIdx.y, b = bh / H, h = bh % H;
    const int t = pt * PB_WARPS + warp;
    float dang[NP];
#pragma unroll
    for (int i = 0; i < NP; ++i) dang[i] = 0.f;
    float p = 0.f;
    if (t < T) {
        const size_t in_off = (size_t)b * sb + (size_t)t * st + (size_t)h * sh + lane * PER;
        const size_t g_off = ((size_t)bh * T + t) * D + lane * PER;
        const size_t o_off = (((size_t)b * T + t) * H + h) * D + lane * PER;
        p = (float)pos[t];
        float cs[NP], sn[NP];
#pragma unroll
        for (int i = 0; i < NP; ++i) sincosf(p * theta[(size_t)h * (D / 2) + lane * NP + i], &sn[i], &cs[i]);
        float x[PER], gr[PER], out[PER];
        // ---- q and k: normalise, (gate,) rotate
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            pb_ld<TIN, PER>(x, (which ? kp : qp) + in_off);
            pb_ld<TG, PER>(gr, (which ? dk : dq) + g_off);
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < PER; ++i) ss = fmaf(x[i], x[i], ss);
            const float inv = 1.0f / fmaxf(sqrtf(warp_sum(ss)), 1e-12f);
            float r1[NP], r2[NP], u1[NP], u2[NP];
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                u1[i] = x[2 * i] * inv; u2[i] = x[2 * i + 1] * inv;
                r1[i] = u1[i] * cs[i] - u2[i] * sn[i]; r2[i] = u1[i] * sn[i] + u2[i] * cs[i];
            }
            if (which == 1 && gate != nullptr) {
                const float sg = sigmoidf_(to_f32(gate[(size_t)b * gsb + (size_t)t * gst + h]));
                float dsg = 0.f;
#pragma unroll
                for (int i = 0; i < NP; ++i) dsg += gr[2 * i] * r1[i] + gr[2 * i + 1] * r2[i];
                dsg = warp_sum(dsg);
                if (lane == 0) dgl[((size_t)b * T + t) * H + h] = dsg * sg * (1.0f - sg);
#pragma unroll
                for (int i = 0; i < PER; ++i) gr[i] *= sg;
            }
            float du1[NP], du2[NP], dot = 0.f;
#pragma unroll
            for (int i = 0; i < NP; ++i) {
                dang[i] += gr[2 * i + 1] * r1[i] - gr[2 * i] * r2[i];
                du1[i] = gr[2 * i] * cs[i] + gr[2 * i + 1] * sn[i];
                du2[i] = gr[2 * i + 1] * cs[i] - gr[2 * i] * sn[i];
                dot += u1[i] * du1[i] + u2[i] * du2[i];
            }
            dot = warp_sum(dot);
#pragma unroll
            for (int i = 0; i < NP; ++i) { out[2 * i] = (du1[i] - u1[i] * dot) * inv; out[2 * i + 1] = (du2[i] - u2[i] * dot) * inv; }
            pb_st<TIN, PER>((which ? dkp : dqp) + o_off, out);
        }
        // ---- v: normalise only
        pb_ld<TIN, PER>(x, vp + in_off);
        pb_ld<TG, PER>(gr, dv + g_off);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) ss = fmaf(x[i], x[i], ss);
        const float inv = 1.0f / fmaxf(sqrtf(warp_sum(ss)), 1e-12f);
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) dot = fmaf(x[i] * inv, gr[i], dot);
        dot = warp_sum(dot);
#pragma unroll
        for (int i = 0; i < PER; ++i) out[i] = (gr[i] - x[i] * inv * dot) * inv;
        pb_st<TIN, PER>(dvp + o_off, out);
    }
    // ---- theta: this CTA's share of the sum over batch and time, tokens added in a fixed order
#pragma unroll
    for (int i = 0; i < NP; ++i) part[warp][lane * NP + i] = dang[i] * p;
    __syncthreads();
    if (threadIdx.x < D / 2) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < PB_WARPS; ++w) s += part[w][threadIdx.x];
        dth_part[(((size_t)b * NT + pt) * H + h) * (D / 2) + threadIdx.x] = s;
    }
}

int prep_bwd_tiles(int T) { return (T + PB_WARPS - 1) / PB_WARPS; }

template <typename TIN, typename TG>
static int prep_bwd_go(const void *qp, const void *kp, const void *vp, long long sb, long long st, long long sh, const void *gate,
                       long long gsb, long long gst, const float *theta, const long long *pos, const void *dq, const void *dk,
                       const void *dv, void *dqp, void *dkp, void *dvp, float *dgl, float *dth_part, int B, int T, int H, int D,
                       cudaStream_t stream) {
    const int NT = prep_bwd_tiles(T);
    auto go = [&](auto kern) {
        kern<<<dim3(NT, B * H), PB_WARPS * 32, 0, stream>>>((const TIN *)qp, (const TIN *)kp, (const TIN *)vp, sb, st, sh, (const TIN *)gate,
                                                           gsb, gst, theta, pos, (const TG *)dq, (const TG *)dk, (const TG *)dv, (TIN *)dqp,
                                                           (TIN *)dkp, (TIN *)dvp, dgl, dth_part, T, H, NT);
    };
    if (D == 64) go(prep_bwd_kernel<TIN, TG, 64>); else go(prep_bwd_kernel<TIN, TG, 128>);
    return check_launch("prep_bwd_kernel");
}

int prep_bwd_launch(const void *qp, const void *kp, const void *vp, int in_dtype, long long sb, long long st, long long sh, const void *gate,
                    long long gsb, long long gst, const float *theta, const long long *pos, const void *dq, const void *dk, const void *dv,
                    int g_dtype, void *dqp, void *dkp, void *dvp, float *dgl, float *dth_part, int B, int T, int H, int D,
                    cudaStream_t stream) {
#define PB_ARGS qp, kp, vp, sb, st, sh, gate, gsb, gst, theta, pos, dq, dk, dv, dqp, dkp, dvp, dgl, dth_part, B, T, H, D, stream
    if (in_dtype == PGB_F32) return g_dtype == PGB_F32 ? prep_bwd_go<float, float>(PB_ARGS) : prep_bwd_go<float, __nv_bfloat16>(PB_ARGS);
    return g_dtype == PGB_F32 ? prep_bwd_go<__nv_bfloat16, float>(PB_ARGS) : prep_bwd_go<__nv_bfloat16, __nv_bfloat16>(PB_ARGS);
#undef PB_ARGS
}

}  // namespace pgb
