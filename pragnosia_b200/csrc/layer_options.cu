// Optional steps of the associative carrier layer that sit between its projections and the scan
// (reference: src/assoc.py AssocCarrier.forward).
//
//   key_topk_mask   keep the key_topk largest-magnitude coordinates of every key (per token and head), zero the rest
//                   (src/assoc.py:435-439). One warp per (b,t,h) row; key_topk rounds of a warp arg-max.
//   short_conv      depthwise causal convolution over the last K tokens of the concatenated q|k|v projections, with the
//                   previous call's last K-1 inputs as left context (src/assoc.py:361-382 _sconv); also returns the new
//                   context. One thread per (b,t,channel), channels fastest.
#include "common.cuh"

namespace pgb {

constexpr int KT_WARPS = 8;

template <typename T_, int D>
__global__ void __launch_bounds__(KT_WARPS * 32)
key_topk_kernel(T_ *__restrict__ kp, long long sb, long long st, long long sh, int B, int T, int H, int topk) {
    constexpr int PER = D / 32;
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * KT_WARPS + (threadIdx.x >> 5);      // over (b,t,h)
    if (row >= (long long)B * T * H) return;
    const int h = (int)(row % H), t = (int)((row / H) % T), b = (int)(row / ((long long)H * T));
    T_ *p = kp + (size_t)b * sb + (size_t)t * st + (size_t)h * sh + lane * PER;
    float mag[PER];
    bool keep[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) { mag[i] = fabsf(to_f32(p[i])); keep[i] = false; }
    for (int round = 0; round < topk; ++round) {
        float best = -1.f; int bi = 0;
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (!keep[i] && mag[i] > best) { best = mag[i]; bi = i; }
        int idx = lane * PER + bi;
        float wv = best; int wi = idx;                                // warp arg-max; the lower index wins a tie
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, wv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
            if (ov > wv || (ov == wv && oi < wi)) { wv = ov; wi = oi; }
        }
        if (wv < 0.f) break;                                          // everything is already kept
        if (wi / PER == lane) {
#pragma unroll
            for (int i = 0; i < PER; ++i)
                if (i == wi % PER) keep[i] = true;
        }
    }
#pragma unroll
    for (int i = 0; i < PER; ++i)
        if (!keep[i]) from_f32(p[i], 0.f);
}

int key_topk_launch(void *kp, int dtype, long long sb, long long st, long long sh, int B, int T, int H, int D, int topk, cudaStream_t stream) {
    const long long rows = (long long)B * T * H, ctas = (rows + KT_WARPS - 1) / KT_WARPS;
    if (ctas > 0x7fffffffLL) return PGB_ERR_TOO_LARGE;
    auto go = [&](auto kern, auto *ptr) { kern<<<(unsigned)ctas, KT_WARPS * 32, 0, stream>>>(ptr, sb, st, sh, B, T, H, topk); };
    if (dtype == PGB_F32) { if (D == 64) go(key_topk_kernel<float, 64>, (float *)kp); else go(key_topk_kernel<float, 128>, (float *)kp); }
    else { if (D == 64) go(key_topk_kernel<__nv_bfloat16, 64>, (__nv_bfloat16 *)kp); else go(key_topk_kernel<__nv_bfloat16, 128>, (__nv_bfloat16 *)kp); }
    return check_launch("key_topk_kernel");
}

// x: (B,T,C) view, element strides (sb, st), unit over C = 3d;  w [C][K];  cache_in [B][C][K-1] or NULL (zeros)
// y [B][T][C] contiguous;  cache_out [B][C][K-1] = the last K-1 columns of [cache_in | x]
template <typename T_>
__global__ void short_conv_kernel(const T_ *__restrict__ x, long long sb, long long st, const T_ *__restrict__ w, const T_ *__restrict__ cache_in,
                                  T_ *__restrict__ y, T_ *__restrict__ cache_out, int B, int T, int C, int K) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)B * T * C) return;
    const int c = (int)(i % C), t = (int)((i / C) % T), b = (int)(i / ((long long)C * T));
    auto tap = [&](int tt) -> float {                                 // input at time tt; negative times come from the context
        if (tt >= 0) return to_f32(x[(size_t)b * sb + (size_t)tt * st + c]);
        const int j = K - 1 + tt;                                     // column of the context: -1 is its last
        return (cache_in != nullptr && j >= 0) ? to_f32(cache_in[((size_t)b * C + c) * (K - 1) + j]) : 0.f;
    };
    float acc = 0.f;
    for (int j = 0; j < K; ++j) acc = fmaf(to_f32(w[(size_t)c * K + j]), tap(t + j - (K - 1)), acc);
    from_f32(y[i], acc);
    if (t >= T - (K - 1)) {                                           // this thread's token is among the last K-1
        const int col = t - (T - (K - 1));
        from_f32(cache_out[((size_t)b * C + c) * (K - 1) + col], tap(t));
    }
    if (t == 0 && T < K - 1) {                                        // a short call: the head of the new context is old context
        for (int col = 0; col < K - 1 - T; ++col) from_f32(cache_out[((size_t)b * C + c) * (K - 1) + col], tap(col - (K - 1) + T));
    }
}

int short_conv_launch(const void *x, int dtype, long long sb, long long st, const void *w, const void *cache_in, void *y, void *cache_out,
                      int B, int T, int C, int K, cudaStream_t stream) {
    const long long n = (long long)B * T * C, ctas = (n + 255) / 256;
    if (ctas > 0x7fffffffLL) return PGB_ERR_TOO_LARGE;
    if (dtype == PGB_F32)
        short_conv_kernel<float><<<(unsigned)ctas, 256, 0, stream>>>((const float *)x, sb, st, (const float *)w, (const float *)cache_in,
                                                                     (float *)y, (float *)cache_out, B, T, C, K);
    else
        short_conv_kernel<__nv_bfloat16><<<(unsigned)ctas, 256, 0, stream>>>((const __nv_bfloat16 *)x, sb, st, (const __nv_bfloat16 *)w,
                                                                             (const __nv_bfloat16 *)cache_in, (__nv_bfloat16 *)y,
                                                                             (__nv_bfloat16 *)cache_out, B, T, C, K);
    return check_launch("short_conv_kernel");
}

}  // namespace pgb
