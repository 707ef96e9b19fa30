// Linear layer for a handful of rows (decode at batch <= 8), fused with what surrounds it in the layer stack:
//
//     s = x + delta                     (residual add; optional; s is also the new residual stream, written once)
//     z = norm(s) * w (+ b)             (RMS or layer norm; optional)
//     y = act(z W^T + bias)             (W is [N][K] as torch.nn.Linear stores it; act: none or erf-GELU)
//
// One token per sequence makes every GEMM of the decode step a matrix-vector product: the time goes into streaming W
// once (HBM-bound, 2 bytes per weight) and into kernel boundaries. This kernel reads W exactly once with 128-bit loads,
// keeps the B normalised rows in shared memory as bf16, and folds the norm before and the activation after into the
// same launch, so a layer's decode step is five launches instead of eight. It replaces, for T = 1 and small batch, the
// F.linear / LayerNorm / GELU calls of src/assoc.py:384-512 and src/model.py:552-560; roundings are placed where the
// separate ops place them (s, z and the pre-activation are rounded to bf16), accumulation is fp32.
//
// Work split: a CTA of four warps first requests its rows of W, then builds z for all B rows (a warp per row; every CTA repeats this, B*K is a few
// thousand elements), then each warp owns SK_R consecutive output rows: lanes stride over K in 8-element pieces, each
// piece of W meets the same piece of all B rows of z, and a shuffle reduction finishes the dot products.
#include "common.cuh"

namespace pgb {

constexpr int SK_WARPS = 4;
constexpr int SK_R = 2;                                               // output rows per warp

__device__ __forceinline__ void unpack8(const uint4 &raw, float (&f)[8]) {
    const __nv_bfloat162 *b = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(b[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 raw;
    __nv_bfloat162 *b = reinterpret_cast<__nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return raw;
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

struct SkinnyArgs {
    const __nv_bfloat16 *x, *delta, *norm_w, *norm_b, *W, *bias;
    __nv_bfloat16 *y, *x_out;
    float eps;
    int norm_kind, act, K, N, nb;                                      // nb: rows actually present (<= the instantiation's B)
    int late_consts;                                                   // the norm vectors / bias may be the preceding kernel's output
};

// Launched with the programmatic-dependent-launch attribute: weights do not depend on the preceding kernel, so the first
// pieces of this warp's rows of W are requested before pdl_wait(); activations are read and results written after it.
// The norm vectors and the bias are requested early too. When the caller says (late_consts) that the kernel just before
// this one on the stream may have produced any of them (a dtype cast, a rebuilt fused weight), all of these loads move
// behind the wait: a predecessor's writes are visible only after it.
constexpr int SK_PRE = 3;                                             // pieces of each row of W requested before the wait (K <= 768: all)
constexpr int SK_ROWREG = 4;                                          // pieces of an activation row a lane keeps in registers (K <= 1024)

template <int B>
__global__ void __launch_bounds__(SK_WARPS * 32) skinny_linear_kernel(SkinnyArgs a) {
    extern __shared__ uint4 sk_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K8 = a.K >> 3;
    // [B][K / 8] pieces of 8 bf16. One row (B = 1): every warp builds the row for itself in a slice of its own, so no warp
    // ever reads a piece another warp is still rewriting (raw sum first, normalised value second, for rows longer than
    // the register buffer).
    uint4 *zs = sk_smem + (B == 1 ? warp * K8 : 0);
    const int n0 = (blockIdx.x * SK_WARPS + warp) * SK_R;
    const bool rows_live = n0 < a.N;
    const uint4 *w0 = reinterpret_cast<const uint4 *>(a.W + (size_t)(rows_live ? n0 : 0) * a.K);
    const uint4 *w1 = reinterpret_cast<const uint4 *>(a.W + (size_t)(n0 + 1 < a.N ? n0 + 1 : (rows_live ? n0 : 0)) * a.K);
    uint4 pw0[SK_PRE], pw1[SK_PRE];
    // the other constants this thread will need: its pieces of the norm vectors and the bias of the output it finishes
    uint4 pnw[SK_ROWREG], pnb[SK_ROWREG];
    float my_bias = 0.f;
    auto load_consts = [&]() {
#pragma unroll
        for (int i = 0; i < SK_PRE; ++i) {
            const int k8 = lane + 32 * i;
            pw0[i] = pw1[i] = make_uint4(0u, 0u, 0u, 0u);
            if (k8 < K8) { pw0[i] = w0[k8]; pw1[i] = w1[k8]; }
        }
#pragma unroll
        for (int i = 0; i < SK_ROWREG; ++i) {
            const int k8 = lane + 32 * i;
            pnw[i] = pnb[i] = make_uint4(0u, 0u, 0u, 0u);
            if (a.norm_kind != 0 && k8 < K8) pnw[i] = reinterpret_cast<const uint4 *>(a.norm_w)[k8];
            if (a.norm_kind == 2 && k8 < K8) pnb[i] = reinterpret_cast<const uint4 *>(a.norm_b)[k8];
        }
        if (a.bias != nullptr && lane < SK_R * B && n0 + lane / B < a.N) my_bias = __bfloat162float(a.bias[n0 + lane / B]);
    };
    if (!a.late_consts) load_consts();
    pdl_launch_dependents();
    pdl_wait();
    if (a.late_consts) load_consts();

    // ---- z for every row of the batch (skipped when there is nothing to add or normalise: z is x, read in place)
    const bool direct = a.delta == nullptr && a.norm_kind == 0 && a.x_out == nullptr;
    if (!direct) {
        // One row (B = 1): every warp builds the whole row for itself, in its own slice. More rows: a warp per row.
        for (int b = (B == 1 ? 0 : warp); b < a.nb; b += (B == 1 ? 1 : SK_WARPS)) {
            const uint4 *xr = reinterpret_cast<const uint4 *>(a.x + (size_t)b * a.K);
            const uint4 *dr = a.delta != nullptr ? reinterpret_cast<const uint4 *>(a.delta + (size_t)b * a.K) : nullptr;
            uint4 *xo = (a.x_out != nullptr && blockIdx.x == 0 && (B > 1 || warp == 0)) ? reinterpret_cast<uint4 *>(a.x_out + (size_t)b * a.K) : nullptr;
            float v[SK_ROWREG][8];                                    // the lane's pieces of the row (K <= 1024), else re-read from zs
            float s1 = 0.f, s2 = 0.f;
#pragma unroll
            for (int i = 0; i < SK_ROWREG; ++i) {
                const int k8 = lane + 32 * i;
                if (k8 < K8) {
                    uint4 keep = xr[k8];
                    unpack8(keep, v[i]);
                    if (dr != nullptr) {
                        float d[8];
                        unpack8(dr[k8], d);
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[i][j] = round_bf16(v[i][j] + d[j]);
                        keep = pack8(v[i]);
                    }
                    if (xo != nullptr) xo[k8] = keep;
                    if (a.norm_kind == 0) zs[b * K8 + k8] = keep;
#pragma unroll
                    for (int j = 0; j < 8; ++j) { s1 += v[i][j]; s2 = fmaf(v[i][j], v[i][j], s2); }
                }
            }
            for (int k8 = lane + 32 * SK_ROWREG; k8 < K8; k8 += 32) {  // rows longer than the register buffer
                float t[8];
                uint4 keep = xr[k8];
                unpack8(keep, t);
                if (dr != nullptr) {
                    float d[8];
                    unpack8(dr[k8], d);
#pragma unroll
                    for (int j = 0; j < 8; ++j) t[j] = round_bf16(t[j] + d[j]);
                    keep = pack8(t);
                }
                if (xo != nullptr) xo[k8] = keep;
                zs[b * K8 + k8] = keep;
#pragma unroll
                for (int j = 0; j < 8; ++j) { s1 += t[j]; s2 = fmaf(t[j], t[j], s2); }
            }
            if (a.norm_kind != 0) {
                float mean = 0.f, rstd;
                if (a.norm_kind == 1) {
                    rstd = rsqrtf(warp_sum(s2) / (float)a.K + a.eps);
                } else {
                    mean = warp_sum(s1) / (float)a.K;
                    float sv = 0.f;
#pragma unroll
                    for (int i = 0; i < SK_ROWREG; ++i)
                        if (lane + 32 * i < K8) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) { const float t = v[i][j] - mean; sv = fmaf(t, t, sv); }
                        }
                    for (int k8 = lane + 32 * SK_ROWREG; k8 < K8; k8 += 32) {
                        float t[8];
                        unpack8(zs[b * K8 + k8], t);
#pragma unroll
                        for (int j = 0; j < 8; ++j) { const float c = t[j] - mean; sv = fmaf(c, c, sv); }
                    }
                    rstd = rsqrtf(warp_sum(sv) / (float)a.K + a.eps);
                }
                const uint4 *wr = reinterpret_cast<const uint4 *>(a.norm_w);
                const uint4 *br = a.norm_kind == 2 ? reinterpret_cast<const uint4 *>(a.norm_b) : nullptr;
                auto norm_piece = [&](const float (&in)[8], int k8, const uint4 &wraw, const uint4 &braw) {
                    float w[8], o[8];
                    unpack8(wraw, w);
                    if (br != nullptr) {
                        float bb[8];
                        unpack8(braw, bb);
#pragma unroll
                        for (int j = 0; j < 8; ++j) o[j] = (in[j] - mean) * rstd * w[j] + bb[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) o[j] = in[j] * rstd * w[j];
                    }
                    zs[b * K8 + k8] = pack8(o);
                };
#pragma unroll
                for (int i = 0; i < SK_ROWREG; ++i)
                    if (lane + 32 * i < K8) norm_piece(v[i], lane + 32 * i, pnw[i], pnb[i]);
                for (int k8 = lane + 32 * SK_ROWREG; k8 < K8; k8 += 32) {
                    float t[8];
                    unpack8(zs[b * K8 + k8], t);
                    norm_piece(t, k8, wr[k8], br != nullptr ? br[k8] : make_uint4(0u, 0u, 0u, 0u));
                }
            }
        }
        if (B == 1) __syncwarp(); else __syncthreads();
    }

    // ---- this warp's output rows
    if (!rows_live) return;
    float acc[SK_R][B];
#pragma unroll
    for (int r = 0; r < SK_R; ++r)
#pragma unroll
        for (int b = 0; b < B; ++b) acc[r][b] = 0.f;
    const uint4 *xg = reinterpret_cast<const uint4 *>(a.x);
    auto piece = [&](const uint4 &ra, const uint4 &rb, int k8) {
        float wa[8], wb[8];
        unpack8(ra, wa);
        unpack8(rb, wb);
#pragma unroll
        for (int b = 0; b < B; ++b) {
            float z[8];
            unpack8(direct ? (b < a.nb ? xg[(size_t)b * K8 + k8] : make_uint4(0u, 0u, 0u, 0u)) : zs[b * K8 + k8], z);
#pragma unroll
            for (int i = 0; i < 8; ++i) { acc[0][b] = fmaf(wa[i], z[i], acc[0][b]); acc[1][b] = fmaf(wb[i], z[i], acc[1][b]); }
        }
    };
#pragma unroll
    for (int i = 0; i < SK_PRE; ++i)
        if (lane + 32 * i < K8) piece(pw0[i], pw1[i], lane + 32 * i);
    for (int k8 = lane + 32 * SK_PRE; k8 < K8; k8 += 32) piece(w0[k8], w1[k8], k8);
#pragma unroll
    for (int r = 0; r < SK_R; ++r)
#pragma unroll
        for (int b = 0; b < B; ++b) acc[r][b] = warp_sum(acc[r][b]);
    // lane (r * B + b) finishes and writes output (b, n0 + r)
#pragma unroll
    for (int r = 0; r < SK_R; ++r)
#pragma unroll
        for (int b = 0; b < B; ++b) {
            if (lane == r * B + b && b < a.nb && n0 + r < a.N) {
                float v = round_bf16(acc[r][b] + my_bias);
                if (a.act == 1) v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
                a.y[(size_t)b * a.N + n0 + r] = __float2bfloat16_rn(v);
            }
        }
}

template <int B>
static cudaError_t skinny_go(const SkinnyArgs &a, int ctas, size_t smem, cudaStream_t stream) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(skinny_linear_kernel<B>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return pdl_launch(skinny_linear_kernel<B>, dim3((unsigned)ctas), dim3(SK_WARPS * 32), smem, stream, a);
}

int skinny_linear_launch(const void *x, const void *delta, const void *norm_w, const void *norm_b, int norm_kind, float eps,
                         const void *W, const void *bias, int act, void *y, void *x_out, int B, int K, int N, int late_consts,
                         cudaStream_t stream) {
    SkinnyArgs a{(const __nv_bfloat16 *)x, (const __nv_bfloat16 *)delta, (const __nv_bfloat16 *)norm_w, (const __nv_bfloat16 *)norm_b,
                 (const __nv_bfloat16 *)W, (const __nv_bfloat16 *)bias, (__nv_bfloat16 *)y, (__nv_bfloat16 *)x_out, eps, norm_kind, act, K, N, B, late_consts};
    const int ctas = (N + SK_WARPS * SK_R - 1) / (SK_WARPS * SK_R);
    const int Bp = B <= 1 ? 1 : (B <= 2 ? 2 : (B <= 4 ? 4 : 8));          // kernel instantiation; its rows beyond B are computed
    const size_t smem = (size_t)(Bp == 1 ? SK_WARPS : Bp) * K * 2;        // on whatever shared memory holds and never written
    cudaError_t e;
    switch (Bp) {
        case 1: e = skinny_go<1>(a, ctas, smem, stream); break;
        case 2: e = skinny_go<2>(a, ctas, smem, stream); break;
        case 4: e = skinny_go<4>(a, ctas, smem, stream); break;
        default: e = skinny_go<8>(a, ctas, smem, stream); break;
    }
    if (e != cudaSuccess) { set_cuda_error(e, "skinny_linear launch"); return PGB_ERR_CUDA; }
    return check_launch("skinny_linear_kernel");
}

}  // namespace pgb
