// Residual add fused with the normalisation that follows it:  y = x + delta ;  z = norm(y) * w (+ b).
// One pass: reads x and delta, writes y (the new residual stream) and z (the normalised input of the next block).
// HBM-bound: 4 rows of d elements move per row. One warp per row, a lane owns 16-byte pieces 32 lanes apart, the whole
// row stays in registers (d <= 2048), the statistics are fp32. The norm is taken from y AS ROUNDED to the I/O dtype, so
// the result is identical to doing the add and the norm as two separate ops (reference src/model.py:552-560 MLP,
// src/assoc.py:388, 511: the layer norms and residual adds of the layer stack).
// kind 0: RMS norm  z = y * rsqrt(mean(y^2) + eps) * w          kind 1: layer norm  z = (y - mean) * rsqrt(var + eps) * w + b
#include "common.cuh"

namespace pgb {

constexpr int AN_WARPS = 8;
constexpr int AN_MAXCH = 8;      // 16-byte pieces a lane may own (bf16: d <= 2048, fp32: d <= 1024)

template <typename T_> struct Piece;
template <> struct Piece<__nv_bfloat16> { static constexpr int N = 8; };
template <> struct Piece<float> { static constexpr int N = 4; };

template <typename T_>
__device__ __forceinline__ void ld_piece(float (&d)[Piece<T_>::N], const T_ *p) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(p);
    if constexpr (sizeof(T_) == 2) {
        const __nv_bfloat162 *b = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(b[i]); d[2 * i] = f.x; d[2 * i + 1] = f.y; }
    } else {
        const float *f = reinterpret_cast<const float *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) d[i] = f[i];
    }
}
template <typename T_>
__device__ __forceinline__ void st_piece(T_ *p, const float (&d)[Piece<T_>::N]) {
    uint4 raw;
    if constexpr (sizeof(T_) == 2) {
        __nv_bfloat162 *b = reinterpret_cast<__nv_bfloat162 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(d[2 * i], d[2 * i + 1]);
    } else {
        float *f = reinterpret_cast<float *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = d[i];
    }
    *reinterpret_cast<uint4 *>(p) = raw;
}
template <typename T_> __device__ __forceinline__ float round_io(float x) {
    if constexpr (sizeof(T_) == 2) return __bfloat162float(__float2bfloat16_rn(x)); else return x;
}

template <typename T_, int KIND, int NCH>
__global__ void __launch_bounds__(AN_WARPS * 32)
add_norm_kernel(const T_ *__restrict__ x, const T_ *__restrict__ delta, const T_ *__restrict__ w, const T_ *__restrict__ b,
                float eps, T_ *__restrict__ y, T_ *__restrict__ z, long long rows, int d) {
    constexpr int N = Piece<T_>::N;
    pdl_wait();                                                    // launched as a programmatic dependent (a no-op otherwise)
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * AN_WARPS + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int npieces = d / N;
    const size_t base = (size_t)row * d;
    float v[NCH][N];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int pc = lane + 32 * c;
        if (pc < npieces) {
            ld_piece<T_>(v[c], x + base + (size_t)pc * N);
            if (delta != nullptr) {
                float dl[N];
                ld_piece<T_>(dl, delta + base + (size_t)pc * N);
#pragma unroll
                for (int i = 0; i < N; ++i) v[c][i] = round_io<T_>(v[c][i] + dl[i]);
                if (y != nullptr) st_piece<T_>(y + base + (size_t)pc * N, v[c]);
            }
#pragma unroll
            for (int i = 0; i < N; ++i) { s1 += v[c][i]; s2 = fmaf(v[c][i], v[c][i], s2); }
        }
    }
    float mean = 0.f, rstd;
    if constexpr (KIND == 0) {
        rstd = rsqrtf(warp_sum(s2) / (float)d + eps);
    } else {
        mean = warp_sum(s1) / (float)d;
        float sv = 0.f;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            if (lane + 32 * c < npieces) {
#pragma unroll
                for (int i = 0; i < N; ++i) { const float t = v[c][i] - mean; sv = fmaf(t, t, sv); }
            }
        }
        rstd = rsqrtf(warp_sum(sv) / (float)d + eps);
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int pc = lane + 32 * c;
        if (pc < npieces) {
            float ww[N], bb[N], out[N];
            ld_piece<T_>(ww, w + (size_t)pc * N);
            if constexpr (KIND == 1) ld_piece<T_>(bb, b + (size_t)pc * N);
#pragma unroll
            for (int i = 0; i < N; ++i) out[i] = KIND == 1 ? (v[c][i] - mean) * rstd * ww[i] + bb[i] : v[c][i] * rstd * ww[i];
            st_piece<T_>(z + base + (size_t)pc * N, out);
        }
    }
}

int add_norm_launch(const void *x, const void *delta, const void *w, const void *b, float eps, int kind, void *y, void *z,
                    long long rows, int d, int dtype, cudaStream_t stream) {
    const long long ctas = (rows + AN_WARPS - 1) / AN_WARPS;
    if (ctas > 0x7fffffffLL) return PGB_ERR_TOO_LARGE;
    // 16-byte pieces per lane: 1, 2, 3, 4 or 8 (the row stays in registers, so the buffer is sized to the row)
    const int n = dtype == PGB_BF16 ? 8 : 4, need = (d / n + 31) / 32;
    cudaError_t le = cudaSuccess;
#define PGB_AN2(T_, K_, C_) le = pdl_launch(add_norm_kernel<T_, K_, C_>, dim3((unsigned)ctas), dim3(AN_WARPS * 32), 0, stream, \
        (const T_ *)x, (const T_ *)delta, (const T_ *)w, (const T_ *)b, eps, (T_ *)y, (T_ *)z, rows, d)
#define PGB_AN(T_, K_) do { if (need <= 1) PGB_AN2(T_, K_, 1); else if (need <= 2) PGB_AN2(T_, K_, 2); else if (need <= 3) PGB_AN2(T_, K_, 3); \
        else if (need <= 4) PGB_AN2(T_, K_, 4); else PGB_AN2(T_, K_, 8); } while (0)
    if (dtype == PGB_BF16) { if (kind == 0) PGB_AN(__nv_bfloat16, 0); else PGB_AN(__nv_bfloat16, 1); }
    else { if (kind == 0) PGB_AN(float, 0); else PGB_AN(float, 1); }
#undef PGB_AN
#undef PGB_AN2
    if (le != cudaSuccess) { set_cuda_error(le, "add_norm launch"); return PGB_ERR_CUDA; }
    return check_launch("add_norm_kernel");
}

}  // namespace pgb
