// The two ends of a decode step, each as one launch, so that a whole token (draw, bookkeeping, embedding, layers, head)
// is a fixed sequence of kernels with nothing left to the host (reference: the host-side loop and sampler of
// src/bench.py:79-86, 193-239, which syncs with the host for every token).
//
//   embed:   x[b][:] = E[tok[b]][:] + P[pos][:]                               (src/model.py:859: token + wrapped position)
//   sample:  tok[b] ~ softmax(logits[b] / temp)   (temp = 0: argmax), recorded in hist[b][count]; with min_p > 0 the ids
//            whose probability is below min_p times the largest are dropped first (src/bench.py:79-86). The position and the
//            rebase shift belong to the token being fed to the model, so from the second draw on (count > 0) the kernel
//            first advances them for the previous token: pos = (pos + 1) mod ctx, shift = 1; the CTA that finishes last
//            then does count += 1.
//
// The draw is the Gumbel-max form of categorical sampling, tok = argmax_v (logit_v / temp - log(-log u_v)), with u_v a
// counter-based uniform (a 64-bit mix of seed, step count, sequence and vocabulary index): reproducible from the seed,
// independent of launch geometry, and it needs no state. With few rows a row is shared by a thread-block cluster of up
// to eight CTAs (a single CTA walking 50k logits costs more than the rest of a small-batch step's kernels together).
#include <cooperative_groups.h>

#include "common.cuh"

namespace pgb {

__global__ void __launch_bounds__(128) decode_embed_kernel(const long long *__restrict__ tok, const long long *__restrict__ pos,
                                                           const __nv_bfloat16 *__restrict__ E, const __nv_bfloat16 *__restrict__ P,
                                                           __nv_bfloat16 *__restrict__ x, int d, int vocab, int ctx,
                                                           float *__restrict__ stats) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float red[2][4];
    float s1 = 0.f, s2 = 0.f;                                         // sum and sum of squares of the row (for a norm folded into the next GEMM)
    const int b = blockIdx.x;
    long long t = tok[b], p = pos[0];
    t = t < 0 ? 0 : (t >= vocab ? vocab - 1 : t);                     // ids outside the table are clamped, never dereferenced
    p = p < 0 ? 0 : (p >= ctx ? ctx - 1 : p);
    const uint4 *er = reinterpret_cast<const uint4 *>(E + (size_t)t * d), *pr = reinterpret_cast<const uint4 *>(P + (size_t)p * d);
    uint4 *xr = reinterpret_cast<uint4 *>(x + (size_t)b * d);
    for (int i = threadIdx.x; i < d / 8; i += blockDim.x) {
        const uint4 a = er[i], c = pr[i];
        const __nv_bfloat162 *a2 = reinterpret_cast<const __nv_bfloat162 *>(&a), *c2 = reinterpret_cast<const __nv_bfloat162 *>(&c);
        uint4 o;
        __nv_bfloat162 *o2 = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 fa = __bfloat1622float2(a2[j]), fc = __bfloat1622float2(c2[j]);
            o2[j] = __floats2bfloat162_rn(fa.x + fc.x, fa.y + fc.y);
            const float2 r = __bfloat1622float2(o2[j]);
            s1 += r.x + r.y; s2 = fmaf(r.x, r.x, fmaf(r.y, r.y, s2));
        }
        xr[i] = o;
    }
    if (stats != nullptr) {                                           // blockDim.x = 128: four warps
        s1 = warp_sum(s1); s2 = warp_sum(s2);
        if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = s1; red[1][threadIdx.x >> 5] = s2; }
        __syncthreads();
        if (threadIdx.x == 0)
            *reinterpret_cast<float2 *>(stats + 2 * b) = make_float2(red[0][0] + red[0][1] + red[0][2] + red[0][3],
                                                                     red[1][0] + red[1][1] + red[1][2] + red[1][3]);
    }
}

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {     // splitmix64 finaliser
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

constexpr int SAMPLE_NT = 512;
constexpr int SAMPLE_MAX_SPLIT = 8;                                   // CTAs that share a row: one thread-block cluster

__device__ __forceinline__ bool sample_better(float s, int v, float best, int arg) { return s > best || (s == best && v < arg); }

// One row of logits per thread-block cluster: with few rows (decode at small batch) a row is split over the cluster's
// CTAs, which combine their candidates through the first CTA's shared memory (distributed shared memory: no scratch in
// global memory, no second launch). The draw does not depend on the split: the uniform of (row, id) is a function of the
// seed, the step and the two indices only, and ties go to the smallest id.
template <typename T_>
__global__ void __launch_bounds__(SAMPLE_NT) decode_sample_kernel(const T_ *__restrict__ logits, float temp, float min_p, unsigned long long seed,
                                                                  long long *__restrict__ tok, long long *__restrict__ hist, int hist_cols,
                                                                  long long *__restrict__ count, long long *__restrict__ pos,
                                                                  float *__restrict__ shift, unsigned int *__restrict__ ticket,
                                                                  int V, int ctx) {
    pdl_wait();
    pdl_launch_dependents();
    namespace cg = cooperative_groups;
    cg::cluster_group cl = cg::this_cluster();
    const int S = (int)cl.num_blocks(), rank = (int)cl.block_rank();
    __shared__ float sval[SAMPLE_NT / 32];
    __shared__ int sidx[SAMPLE_NT / 32];
    __shared__ float cmax[SAMPLE_MAX_SPLIT], cval[SAMPLE_MAX_SPLIT];   // the cluster's per-CTA results, gathered in CTA 0
    __shared__ int cidx[SAMPLE_MAX_SPLIT];
    const int b = blockIdx.x / S, rows = gridDim.x / S, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long step = count[0];
    if (blockIdx.x == 0 && tid == 0 && step > 0) {                    // nobody in this kernel reads these two
        if (pos != nullptr) pos[0] = (pos[0] + 1) % ctx;
        if (shift != nullptr) shift[0] = 1.0f;
    }
    const T_ *row = logits + (size_t)b * V;
    const float inv_t = temp > 0.f ? 1.0f / temp : 1.0f;
    const unsigned long long key = mix64(seed ^ mix64((unsigned long long)step * 0x100000001b3ull + (unsigned long long)b));
    const int v0 = rank * SAMPLE_NT + tid, dv = S * SAMPLE_NT;
    float *cmax0 = cl.map_shared_rank(cmax, 0), *cval0 = cl.map_shared_rank(cval, 0);
    int *cidx0 = cl.map_shared_rank(cidx, 0);
    // min-p: p_v >= min_p * p_max  <=>  logit_v / temp >= max_w logit_w / temp + log(min_p); one extra pass for the maximum
    float floor_s = -INFINITY;
    if (temp > 0.f && min_p > 0.f) {
        float m = -INFINITY;
        for (int v = v0; v < V; v += dv) {
            float s;
            if constexpr (sizeof(T_) == 2) s = __bfloat162float(row[v]); else s = row[v];
            m = fmaxf(m, s * inv_t);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) sval[warp] = m;
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < SAMPLE_NT / 32; ++w) m = fmaxf(m, sval[w]);
            cmax0[rank] = m;
        }
        cl.sync();
        m = cmax0[0];
        for (int r = 1; r < S; ++r) m = fmaxf(m, cmax0[r]);
        floor_s = m + logf(min_p);
        __syncthreads();                                              // sval is reused below
    }
    float best = -INFINITY;
    int arg = V;                                                      // ties go to the smallest index
    for (int v = v0; v < V; v += dv) {
        float s;
        if constexpr (sizeof(T_) == 2) s = __bfloat162float(row[v]); else s = row[v];
        s *= inv_t;
        if (s < floor_s) continue;                                    // dropped by min-p
        if (temp > 0.f) {
            const unsigned long long r = mix64(key + (unsigned long long)v);
            const float u = ((float)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);          // (0, 1), 24 bits
            s -= logf(-logf(u));
        }
        if (sample_better(s, v, best, arg)) { best = s; arg = v; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (sample_better(ob, oa, best, arg)) { best = ob; arg = oa; }
    }
    if (lane == 0) { sval[warp] = best; sidx[warp] = arg; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < SAMPLE_NT / 32; ++w)
            if (sample_better(sval[w], sidx[w], best, arg)) { best = sval[w]; arg = sidx[w]; }
        cval0[rank] = best; cidx0[rank] = arg;
    }
    cl.sync();                                                        // every CTA's candidate is in CTA 0; nobody leaves before it is read
    if (rank == 0 && tid == 0) {
        best = cval[0]; arg = cidx[0];
        for (int r = 1; r < S; ++r)
            if (sample_better(cval[r], cidx[r], best, arg)) { best = cval[r]; arg = cidx[r]; }
        if (arg >= V) arg = 0;                                        // a row of NaNs: still a valid id
        tok[b] = arg;
        if (hist != nullptr && step >= 0 && step < hist_cols) hist[(size_t)b * hist_cols + step] = arg;
        __threadfence();
        if (atomicAdd(ticket, 1u) == (unsigned)rows - 1u) {           // every row has read the count: advance it
            count[0] = step + 1;
            *ticket = 0u;
        }
    }
}

// CTAs per row: as many as keep the whole launch within about two CTAs per SM, at most one portable cluster
static int sample_split(int B, int V) {
    int s = 1;
    while (s < SAMPLE_MAX_SPLIT && B * s * 2 <= 256 && V >= s * 2 * SAMPLE_NT * 4) s *= 2;
    return s;
}

template <typename T_>
static cudaError_t sample_go(const T_ *logits, float temp, float min_p, unsigned long long seed, long long *tok, long long *hist, int hist_cols,
                             long long *count, long long *pos, float *shift, unsigned int *ticket, int B, int V, int ctx, cudaStream_t stream) {
    const int S = sample_split(B, V);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(B * S)); cfg.blockDim = dim3(SAMPLE_NT); cfg.dynamicSmemBytes = 0; cfg.stream = stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    at[1].id = cudaLaunchAttributeClusterDimension;
    at[1].val.clusterDim.x = (unsigned)S; at[1].val.clusterDim.y = 1; at[1].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, decode_sample_kernel<T_>, logits, temp, min_p, seed, tok, hist, hist_cols, count, pos, shift, ticket, V, ctx);
}

int decode_embed_launch(const long long *tok, const long long *pos, const void *E, const void *P, void *x, int B, int d, int vocab,
                        int ctx, float *stats, cudaStream_t stream) {
    cudaError_t e = pdl_launch(decode_embed_kernel, dim3((unsigned)B), dim3(128), 0, stream, tok, pos, (const __nv_bfloat16 *)E,
                               (const __nv_bfloat16 *)P, (__nv_bfloat16 *)x, d, vocab, ctx, stats);
    if (e != cudaSuccess) { set_cuda_error(e, "decode_embed launch"); return PGB_ERR_CUDA; }
    return check_launch("decode_embed_kernel");
}

int decode_sample_launch(const void *logits, int dtype, float temp, float min_p, unsigned long long seed, long long *tok, long long *hist,
                         int hist_cols, long long *count, long long *pos, float *shift, unsigned int *ticket, int B, int V, int ctx,
                         cudaStream_t stream) {
    cudaError_t e;
    if (dtype == PGB_BF16)
        e = sample_go((const __nv_bfloat16 *)logits, temp, min_p, seed, tok, hist, hist_cols, count, pos, shift, ticket, B, V, ctx, stream);
    else
        e = sample_go((const float *)logits, temp, min_p, seed, tok, hist, hist_cols, count, pos, shift, ticket, B, V, ctx, stream);
    if (e != cudaSuccess) { set_cuda_error(e, "decode_sample launch"); return PGB_ERR_CUDA; }
    return check_launch("decode_sample_kernel");
}

}  // namespace pgb
