// One recurrent decode step of the associative carrier for one (sequence, head), as a device function: the stand-alone
// kernel (decode_step.cu) and the one-launch-per-token kernel (decode_token.cu) both run exactly this arithmetic.
#pragma once
#include "common.cuh"

namespace pgb {

constexpr int DEC_THREADS = 256;


// One (sequence, head) by the calling CTA of DEC_THREADS threads; every thread of the CTA must call it (it synchronises).
// between(): called by every thread once the loads of the state slice are in flight and before anything of this token's
// projection is read -- the place for a wait on whoever produces the projection. False from it (the same for the whole
// CTA) abandons the step with nothing written.
template <typename TIN, typename TOUT, int D, bool DELTA, typename Between>
__device__ __forceinline__ void decode_step_body(const DecodeArgs &a, int b, int h, Between &&between) {
    constexpr int NCG = D / 4;                    // column groups (4 value columns each)
    constexpr int NRG = DEC_THREADS / NCG;        // row groups
    constexpr int NPAIR = (D / 2) / NRG;          // row pairs per thread
    __shared__ __align__(16) float sq[D], sk[D], sv[D];             // read and written four floats at a time
    __shared__ __align__(16) float part[NRG][D];
    __shared__ float red[8];
    __shared__ float sc[4];                        // alpha, gate/beta, inv-rms

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int bhx = b * a.H + h;
    const TIN *qp = (const TIN *)a.qp + (size_t)b * a.in_sb + (size_t)h * D;
    const TIN *kp = (const TIN *)a.kp + (size_t)b * a.in_sb + (size_t)h * D;
    const TIN *vp = (const TIN *)a.vp + (size_t)b * a.in_sb + (size_t)h * D;

    // ---- the state slice first: its loads are the long latency, everything below overlaps with them
    const int cg = tid % NCG, rg = tid / NCG;
    const int col = cg * 4;
    const float *Sin = a.S_in + (size_t)bhx * D * D;
    float *Sout = a.S_out + (size_t)bhx * D * D;
    float4 s0[NPAIR], s1[NPAIR];
#pragma unroll
    for (int p = 0; p < NPAIR; ++p) {
        const int pr = rg + p * NRG;                                 // pair index: rows 2pr, 2pr+1
        s0[p] = __ldcs(reinterpret_cast<const float4 *>(Sin + (size_t)(2 * pr) * D + col));
        s1[p] = __ldcs(reinterpret_cast<const float4 *>(Sin + (size_t)(2 * pr + 1) * D + col));
    }
    const float shift = a.shift_dev != nullptr ? *a.shift_dev : a.shift_host;
    float rcs[NPAIR], rsn[NPAIR];                                    // rebase rotation of this thread's row pairs
#pragma unroll
    for (int p = 0; p < NPAIR; ++p) {
        rcs[p] = 1.f; rsn[p] = 0.f;
        if (shift != 0.f) sincosf(-shift * a.theta[(size_t)h * (D / 2) + rg + p * NRG], &rsn[p], &rcs[p]);
    }

    if (!between()) return;

    // ---- vectors: load, normalise (warps 0,1,2 take q,k,v), scalars (warp 3)
    if (warp < 3) {
        const TIN *src = warp == 0 ? qp : (warp == 1 ? kp : vp);
        float *dst = warp == 0 ? sq : (warp == 1 ? sk : sv);
        float x[D / 32]; float ss = 0.f;
#pragma unroll
        for (int i = 0; i < D / 32; ++i) { x[i] = to_f32(src[lane + 32 * i]); ss += x[i] * x[i]; }
        float inv = 1.f;
        if (a.normalize) { ss = warp_sum(ss); inv = 1.0f / fmaxf(sqrtf(ss), 1e-12f); }
#pragma unroll
        for (int i = 0; i < D / 32; ++i) dst[lane + 32 * i] = x[i] * inv;
    } else if (warp == 3 && lane == 0) {
        float d = to_f32(((const TIN *)a.decay)[(size_t)b * a.decay_sb + h]);
        if (a.decay_A != nullptr) d = -softplusf_(d) * expf(a.decay_A[h]);
        sc[0] = expf(d);
        float g = 1.f;
        if (a.gate != nullptr) {
            g = to_f32(((const TIN *)a.gate)[(size_t)b * a.gate_sb + h]);
            if (a.gate_is_logit) g = sigmoidf_(g);
        }
        sc[1] = g;
    }
    __syncthreads();
    const float alpha = sc[0];
    const float g = sc[1];
    // plain rule: the write gate scales k.  delta rule: g is beta.
    const float kscale = DELTA ? 1.f : g;

    const float4 vv = *reinterpret_cast<const float4 *>(sv + col);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);                    // delta: sum_r k_r Sd[r][j];  plain: sum_r q_r S'[r][j]
#pragma unroll
    for (int p = 0; p < NPAIR; ++p) {
        const int pr = rg + p * NRG;
        const float cs = alpha * rcs[p], sn = alpha * rsn[p];
        const float4 x0 = s0[p], x1 = s1[p];
        float4 d0, d1;                                               // alpha * rotated rows
        d0.x = x0.x * cs - x1.x * sn; d1.x = x0.x * sn + x1.x * cs;
        d0.y = x0.y * cs - x1.y * sn; d1.y = x0.y * sn + x1.y * cs;
        d0.z = x0.z * cs - x1.z * sn; d1.z = x0.z * sn + x1.z * cs;
        d0.w = x0.w * cs - x1.w * sn; d1.w = x0.w * sn + x1.w * cs;
        const float k0 = sk[2 * pr] * kscale, k1 = sk[2 * pr + 1] * kscale;
        if constexpr (DELTA) {
            acc.x += k0 * d0.x + k1 * d1.x; acc.y += k0 * d0.y + k1 * d1.y;
            acc.z += k0 * d0.z + k1 * d1.z; acc.w += k0 * d0.w + k1 * d1.w;
        } else {
            const float q0 = sq[2 * pr], q1 = sq[2 * pr + 1];
            d0.x += k0 * vv.x; d0.y += k0 * vv.y; d0.z += k0 * vv.z; d0.w += k0 * vv.w;
            d1.x += k1 * vv.x; d1.y += k1 * vv.y; d1.z += k1 * vv.z; d1.w += k1 * vv.w;
            acc.x += q0 * d0.x + q1 * d1.x; acc.y += q0 * d0.y + q1 * d1.y;
            acc.z += q0 * d0.z + q1 * d1.z; acc.w += q0 * d0.w + q1 * d1.w;
            *reinterpret_cast<float4 *>(Sout + (size_t)(2 * pr) * D + col) = d0;
            *reinterpret_cast<float4 *>(Sout + (size_t)(2 * pr + 1) * D + col) = d1;
        }
        s0[p] = d0; s1[p] = d1;
    }
    *reinterpret_cast<float4 *>(&part[rg][col]) = acc;
    __syncthreads();
    if constexpr (DELTA) {
        // r_j = beta (v_j - sum over row groups), computed redundantly by every thread for its 4 columns
        float4 ks = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < NRG; ++r) {
            const float4 t = *reinterpret_cast<const float4 *>(&part[r][col]);
            ks.x += t.x; ks.y += t.y; ks.z += t.z; ks.w += t.w;
        }
        const float4 rr = make_float4(g * (vv.x - ks.x), g * (vv.y - ks.y), g * (vv.z - ks.z), g * (vv.w - ks.w));
        acc = make_float4(0.f, 0.f, 0.f, 0.f);
        __syncthreads();                                             // everyone has read part[] before it is reused
#pragma unroll
        for (int p = 0; p < NPAIR; ++p) {
            const int pr = rg + p * NRG;
            const float k0 = sk[2 * pr], k1 = sk[2 * pr + 1];
            const float q0 = sq[2 * pr], q1 = sq[2 * pr + 1];
            float4 d0 = s0[p], d1 = s1[p];
            d0.x += k0 * rr.x; d0.y += k0 * rr.y; d0.z += k0 * rr.z; d0.w += k0 * rr.w;
            d1.x += k1 * rr.x; d1.y += k1 * rr.y; d1.z += k1 * rr.z; d1.w += k1 * rr.w;
            acc.x += q0 * d0.x + q1 * d1.x; acc.y += q0 * d0.y + q1 * d1.y;
            acc.z += q0 * d0.z + q1 * d1.z; acc.w += q0 * d0.w + q1 * d1.w;
            *reinterpret_cast<float4 *>(Sout + (size_t)(2 * pr) * D + col) = d0;
            *reinterpret_cast<float4 *>(Sout + (size_t)(2 * pr + 1) * D + col) = d1;
        }
        *reinterpret_cast<float4 *>(&part[rg][col]) = acc;
        __syncthreads();
    }
    // ---- the read: sum the row groups' partials, optional per-head RMS norm, store
    float oj = 0.f;
    if (tid < D) {
#pragma unroll
        for (int r = 0; r < NRG; ++r) oj += part[r][tid];
    }
    if (a.rms_w != nullptr) {
        float ss = (tid < D) ? oj * oj : 0.f;
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (tid == 0) {
            float tot = 0.f;
#pragma unroll
            for (int w = 0; w < D / 32; ++w) tot += red[w];
            sc[2] = rsqrtf(tot / (float)D + a.rms_eps);
        }
        __syncthreads();
        if (tid < D) oj = oj * sc[2] * a.rms_w[tid];
    }
    if (tid < D) {
        TOUT *o = (TOUT *)a.o + (size_t)b * a.out_sb + (size_t)h * D;
        from_f32(o[tid], oj);
    }
}


}  // namespace pgb
