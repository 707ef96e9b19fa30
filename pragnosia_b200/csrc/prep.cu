// Plumbing between the projections and the scan, one pass: L2-normalise q, k, v per head, scale k by the write gate,
// rotate q and k by pos * theta per channel pair, cast, and go from the projections' (B,T,H,D) to the scan's (B,H,T,D).
// HBM-bound: reads 3 rows and writes 3 rows per (b,t,h). One warp per (b,h,t) row; a lane owns D/32 adjacent
// channels (whole rotation pairs), so the norm is one shuffle reduction and the rotation is lane-local.
// Arithmetic order follows the reference kernel (src/assoc_kernel.py:742-769): rotate the raw pair, then multiply by
// 1/max(|x|,1e-12) (times sigmoid(gate) for k, in fp32), then round.
#include "common.cuh"

namespace pgb {

constexpr int PREP_WARPS = 8;

template <typename TIN, int PER>
__device__ __forceinline__ void ld_row(float (&d)[PER], const TIN *p) {
    if constexpr (sizeof(TIN) == 4) {
        if constexpr (PER == 2) { float2 t = *reinterpret_cast<const float2 *>(p); d[0] = t.x; d[1] = t.y; }
        else { float4 t = *reinterpret_cast<const float4 *>(p); d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w; }
    } else {
        const __nv_bfloat162 *q = reinterpret_cast<const __nv_bfloat162 *>(p);
#pragma unroll
        for (int i = 0; i < PER / 2; ++i) { float2 t = __bfloat1622float2(q[i]); d[2 * i] = t.x; d[2 * i + 1] = t.y; }
    }
}
template <typename TOUT, int PER>
__device__ __forceinline__ void st_row(TOUT *p, const float (&d)[PER]) {
    if constexpr (sizeof(TOUT) == 4) {
        if constexpr (PER == 2) *reinterpret_cast<float2 *>(p) = make_float2(d[0], d[1]);
        else *reinterpret_cast<float4 *>(p) = make_float4(d[0], d[1], d[2], d[3]);
    } else {
        __nv_bfloat162 *q = reinterpret_cast<__nv_bfloat162 *>(p);
#pragma unroll
        for (int i = 0; i < PER / 2; ++i) q[i] = __floats2bfloat162_rn(d[2 * i], d[2 * i + 1]);
    }
}

template <typename TIN, typename TOUT, int D>
__global__ void __launch_bounds__(PREP_WARPS * 32)
prep_kernel(const TIN *__restrict__ qp, const TIN *__restrict__ kp, const TIN *__restrict__ vp, long long sb, long long st,
            long long sh, const TIN *__restrict__ gate, long long gsb, long long gst, const float *__restrict__ theta,
            const long long *__restrict__ pos, TOUT *__restrict__ q, TOUT *__restrict__ k, TOUT *__restrict__ v, int B,
            int T, int H) {
    constexpr int PER = D / 32;                                    // 2 or 4 channels per lane
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * PREP_WARPS + (threadIdx.x >> 5);     // over (b,h,t), t fastest
    if (row >= (long long)B * H * T) return;
    const int t = (int)(row % T);
    const int h = (int)((row / T) % H);
    const int b = (int)(row / ((long long)T * H));
    const size_t in_off = (size_t)b * sb + (size_t)t * st + (size_t)h * sh + lane * PER;
    const size_t out_off = (size_t)row * D + lane * PER;

    float xq[PER], xk[PER], xv[PER];
    ld_row<TIN, PER>(xq, qp + in_off);
    ld_row<TIN, PER>(xk, kp + in_off);
    ld_row<TIN, PER>(xv, vp + in_off);
    const float p = (float)pos[t];
    float cs[PER / 2], sn[PER / 2];
#pragma unroll
    for (int i = 0; i < PER / 2; ++i) {
        const float th = theta[(size_t)h * (D / 2) + lane * (PER / 2) + i];
        sincosf(p * th, &sn[i], &cs[i]);
    }
    float sq = 0.f, sk = 0.f, sv = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) { sq += xq[i] * xq[i]; sk += xk[i] * xk[i]; sv += xv[i] * xv[i]; }
    sq = warp_sum(sq); sk = warp_sum(sk); sv = warp_sum(sv);
    const float iq = 1.0f / fmaxf(sqrtf(sq), 1e-12f);
    float ik = 1.0f / fmaxf(sqrtf(sk), 1e-12f);
    const float iv = 1.0f / fmaxf(sqrtf(sv), 1e-12f);
    if (gate != nullptr) ik *= sigmoidf_(to_f32(gate[(size_t)b * gsb + (size_t)t * gst + h]));
    float oq[PER], ok[PER], ov[PER];
#pragma unroll
    for (int i = 0; i < PER / 2; ++i) {
        oq[2 * i] = (xq[2 * i] * cs[i] - xq[2 * i + 1] * sn[i]) * iq;
        oq[2 * i + 1] = (xq[2 * i] * sn[i] + xq[2 * i + 1] * cs[i]) * iq;
        ok[2 * i] = (xk[2 * i] * cs[i] - xk[2 * i + 1] * sn[i]) * ik;
        ok[2 * i + 1] = (xk[2 * i] * sn[i] + xk[2 * i + 1] * cs[i]) * ik;
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) ov[i] = xv[i] * iv;
    st_row<TOUT, PER>(q + out_off, oq);
    st_row<TOUT, PER>(k + out_off, ok);
    st_row<TOUT, PER>(v + out_off, ov);
}

template <typename TIN, typename TOUT>
static int prep_dispatch(const void *qp, const void *kp, const void *vp, long long sb, long long st, long long sh,
                         const void *gate, long long gsb, long long gst, const float *theta, const long long *pos,
                         void *q, void *k, void *v, int B, int T, int H, int D, cudaStream_t stream) {
    const long long rows = (long long)B * H * T;
    const long long ctas = (rows + PREP_WARPS - 1) / PREP_WARPS;
    if (ctas > 0x7fffffffLL) return PGB_ERR_TOO_LARGE;
    auto a = [&](auto kern) {
        kern<<<(unsigned)ctas, PREP_WARPS * 32, 0, stream>>>((const TIN *)qp, (const TIN *)kp, (const TIN *)vp, sb, st, sh,
                                                             (const TIN *)gate, gsb, gst, theta, pos, (TOUT *)q, (TOUT *)k,
                                                             (TOUT *)v, B, T, H);
    };
    if (D == 64) a(prep_kernel<TIN, TOUT, 64>); else a(prep_kernel<TIN, TOUT, 128>);
    return check_launch("prep_kernel");
}

int prep_launch(const void *qp, const void *kp, const void *vp, int in_dtype, long long sb, long long st, long long sh,
                const void *gate, long long gsb, long long gst, const float *theta, const long long *pos, void *q, void *k,
                void *v, int out_dtype, int B, int T, int H, int D, cudaStream_t stream) {
    if (in_dtype == PGB_F32 && out_dtype == PGB_F32)
        return prep_dispatch<float, float>(qp, kp, vp, sb, st, sh, gate, gsb, gst, theta, pos, q, k, v, B, T, H, D, stream);
    if (in_dtype == PGB_F32 && out_dtype == PGB_BF16)
        return prep_dispatch<float, __nv_bfloat16>(qp, kp, vp, sb, st, sh, gate, gsb, gst, theta, pos, q, k, v, B, T, H, D, stream);
    if (in_dtype == PGB_BF16 && out_dtype == PGB_F32)
        return prep_dispatch<__nv_bfloat16, float>(qp, kp, vp, sb, st, sh, gate, gsb, gst, theta, pos, q, k, v, B, T, H, D, stream);
    return prep_dispatch<__nv_bfloat16, __nv_bfloat16>(qp, kp, vp, sb, st, sh, gate, gsb, gst, theta, pos, q, k, v, B, T, H, D, stream);
}

// ---- plain rotation of channel pairs (src/assoc.py:34-39): one thread per pair
template <typename T_>
__global__ void rotate_pairs_kernel(const T_ *__restrict__ x, const float *__restrict__ theta, const float *__restrict__ pos,
                                    T_ *__restrict__ out, long long npairs, int H, int T, int half) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= npairs) return;
    const int pi = (int)(i % half);
    const long long row = i / half;                                   // over (b,h,t)
    const int t = (int)(row % T);
    const int h = (int)((row / T) % H);
    float sn, cs;
    sincosf(pos[t] * theta[(size_t)h * half + pi], &sn, &cs);
    const float a = to_f32(x[2 * i]), b = to_f32(x[2 * i + 1]);
    from_f32(out[2 * i], a * cs - b * sn);
    from_f32(out[2 * i + 1], a * sn + b * cs);
}

int rotate_launch(const void *x, int dtype, const float *theta, const float *pos, void *out, int B, int H, int T, int D,
                  cudaStream_t stream) {
    const long long npairs = (long long)B * H * T * (D / 2);
    const long long ctas = (npairs + 255) / 256;
    if (ctas > 0x7fffffffLL) return PGB_ERR_TOO_LARGE;
    if (dtype == PGB_F32)
        rotate_pairs_kernel<float><<<(unsigned)ctas, 256, 0, stream>>>((const float *)x, theta, pos, (float *)out, npairs, H, T, D / 2);
    else
        rotate_pairs_kernel<__nv_bfloat16><<<(unsigned)ctas, 256, 0, stream>>>((const __nv_bfloat16 *)x, theta, pos, (__nv_bfloat16 *)out, npairs, H, T, D / 2);
    return check_launch("rotate_pairs_kernel");
}

}  // namespace pgb
