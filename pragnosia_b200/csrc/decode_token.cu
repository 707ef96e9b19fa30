// One decode step of the whole language model (every layer, the final norm and the head) as ONE launch, for a few
// sequences (batch <= 4, bf16 weights, fp32 state).
//
// The reference's decode step is one CUDA graph of about a thousand small launches (src/bench.py:242-317); the step built
// from this library's fused kernels is five launches a layer (decode_step.cu, skinny_linear.cu). At one token per sequence
// every launch moves a megabyte or so and lasts two to four microseconds, most of it ramp-up and drain, so the chain of
// kernel boundaries -- not HBM -- is what a token costs. Here the chain is one persistent kernel: one CTA per SM, launched
// cooperatively (so all of them are resident), walking the token through the phases
//
//     per layer   1. s = x + delta;  z = norm(s);  y = z Wqkv^T + b          (fused q | k | v | decay | gate projection)
//                 2. the recurrent state step per (sequence, head)            (decode_step.cuh: the stand-alone kernel's arithmetic)
//                 3. d1 = o Wo'^T                                             (output projection, gate folded into the weight)
//                 4. s = s + d1;  z = norm(s);  hmid = GELU(z Wa^T + ba)      (MLP up)
//                 5. delta = hmid Wb^T + bb                                   (MLP down)
//     at the end     z = norm(x + delta);  logits = z E^T                     (tied head)
//
// with a grid-wide barrier between phases (the embedding lookup is folded into the first phase 1). Every linear phase is a
// matrix-vector product per sequence: a warp owns groups of output rows (dealt round-robin over the grid's warps), keeps
// a dozen 128-bit pieces of them in flight, and meets each piece with the same piece of every sequence's normalised row
// held in shared memory. What a phase costs is a chain of dependent memory round trips, so everything that does not
// depend on the previous phase is requested between the two halves of the barrier that ends it (arrive, then wait): the
// first weights of the coming phase and their bias, the state slice of the recurrent step. Roundings sit where the
// separate ops put them (the residual sum, the normalised row, every linear output and the pre-activation are bf16), and
// the accumulation order of every dot product is the one of skinny_linear.cu.
//
// The barrier is one 64-bit arrival counter in global memory that only ever grows (nothing to reset between launches;
// the second word of the pair is reserved). Its wait is bounded: a CTA that gives up raises a flag every other waiter
// also watches, so the kernel winds down within about a second instead of hanging, and the host reads the flag.
#include "decode_step.cuh"

namespace pgb {

constexpr int DT_THREADS = DEC_THREADS;                               // 256: what decode_step_body is written for
constexpr int DT_WARPS = DT_THREADS / 32;
constexpr unsigned DT_SPIN_LIMIT = 1u << 20;                          // polls of about a microsecond each

static __device__ int g_dt_error = 0;

// One layer's pointers and norm settings; the host lays the table out as 18 64-bit words per layer.
struct DtLayer {
    const __nv_bfloat16 *Wc, *bc, *ln_w, *ln_b, *ow, *n_w, *n_b, *a_w, *a_b, *b_w, *b_b;
    const float *theta, *A, *on_w;
    float *S;
    int ln_kind, n_kind;
    float ln_eps, n_eps;
    float on_eps;                                                     // of the per-head RMS norm on the read
    int pad;
};
static_assert(sizeof(DtLayer) == 18 * 8, "the host writes 18 words per layer");

struct DtArgs {
    const DtLayer *layers;
    const __nv_bfloat16 *E, *P, *fn_w, *fn_b;
    const long long *tok, *pos;
    const float *shift;
    __nv_bfloat16 *xa, *xb, *y, *o, *hmid, *dl;
    float *logits;
    unsigned long long *sync;                                         // [0] arrivals, [1] reserved
    int L, B, d, H, NP, dff, V, ctx, fn_kind;
    float fn_eps;
};

__device__ __forceinline__ void dt_unpack8(const uint4 &raw, float (&f)[8]) {
    const __nv_bfloat162 *b = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(b[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 dt_pack8(const float (&f)[8]) {
    uint4 raw;
    __nv_bfloat162 *b = reinterpret_cast<__nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return raw;
}
__device__ __forceinline__ float dt_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// Grid-wide barrier number gen + 1 (every CTA passes the same barriers in the same order), in two halves so that work which
// does not depend on the other CTAs can sit between them. Arrive: one fire-and-forget add to the arrival counter once the
// whole CTA has written its results. Wait: polls of the counter itself; false when the wait ran out (or another CTA's
// did): the flag is up and the kernel winds down.
__device__ __forceinline__ void dt_arrive(unsigned long long *sync) {
    __syncthreads();
    // release: this CTA's writes (ordered before this by the CTA barrier above) are visible to whoever sees the count
    if (threadIdx.x == 0) asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(sync), "l"(1ull) : "memory");
}
__device__ __forceinline__ bool dt_wait(unsigned long long *sync, unsigned long long &gen, unsigned limit = DT_SPIN_LIMIT) {
    __shared__ int s_alive;
    if (threadIdx.x == 0) {
        int alive = 1;
        const unsigned long long target = (gen + 1) * gridDim.x;
        unsigned spins = 0;
        while (true) {
            unsigned long long c;
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(c) : "l"(sync) : "memory");
            if (c >= target) break;
            ++spins;
            if (spins > limit || ((spins & 63u) == 0u && *reinterpret_cast<volatile int *>(&g_dt_error) != 0)) {
                atomicExch(&g_dt_error, 81);
                alive = 0;
                break;
            }
        }
        s_alive = alive;
    }
    gen += 1;
    __syncthreads();
    return s_alive != 0;
}

// The rows a linear phase multiplies: copied as they are (mode 0), or norm(x + add) with the rounded sum written back as
// the new residual stream (mode 1), or the same with x = E[tok], add = P[pos] (mode 2: the embedding).
struct DtRows {
    int mode;
    const __nv_bfloat16 *x, *add;
    __nv_bfloat16 *x_out;
    int kind; float eps;
    const __nv_bfloat16 *nw, *nb;
    int K;
};
constexpr int DT_ROWREG = 2;                                          // pieces of a row a thread keeps in registers

// zs[b][:] = the phase's rows as bf16 in shared memory, built by the whole CTA: the warps are dealt to the rows (8, 4 or 2
// warps a row for 1, 2 or 3..4 rows) and every thread requests its pieces of the row, the addend and the norm vectors
// before it uses the first, so a build is one round trip to the L2 and a few dozen instructions per thread. The sums of
// the norm go through shared memory in a fixed order. CTA 0 writes the rounded sum to x_out.
__device__ __noinline__ void dt_build_rows(const DtArgs &a, const DtRows &rw, uint4 *zs) {
    const int K = rw.K, K8 = K >> 3;
    if (rw.mode == 0) {
        const uint4 *src = reinterpret_cast<const uint4 *>(rw.x);
        for (int i = threadIdx.x; i < a.B * K8; i += DT_THREADS) zs[i] = src[i];
        __syncthreads();
        return;
    }
    __shared__ float part[2][DT_WARPS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wpr = a.B == 1 ? DT_WARPS : (a.B == 2 ? DT_WARPS / 2 : DT_WARPS / 4);   // warps per row
    const int b = warp / wpr, li = (warp % wpr) * 32 + lane, stride = wpr * 32;
    const bool live = b < a.B;
    const uint4 *xr = nullptr, *dr = nullptr;
    if (live) {
        if (rw.mode == 2) {
            long long t = a.tok[b], p = a.pos[0];
            t = t < 0 ? 0 : (t >= a.V ? a.V - 1 : t);                 // ids outside the table are clamped, never dereferenced
            p = p < 0 ? 0 : (p >= a.ctx ? a.ctx - 1 : p);
            xr = reinterpret_cast<const uint4 *>(a.E + (size_t)t * K);
            dr = reinterpret_cast<const uint4 *>(a.P + (size_t)p * K);
        } else {
            xr = reinterpret_cast<const uint4 *>(rw.x + (size_t)b * K);
            dr = rw.add != nullptr ? reinterpret_cast<const uint4 *>(rw.add + (size_t)b * K) : nullptr;
        }
    }
    uint4 *xo = (live && rw.x_out != nullptr && blockIdx.x == 0) ? reinterpret_cast<uint4 *>(rw.x_out + (size_t)b * K) : nullptr;
    uint4 px[DT_ROWREG], pd[DT_ROWREG], pnw[DT_ROWREG], pnb[DT_ROWREG];
#pragma unroll
    for (int i = 0; i < DT_ROWREG; ++i) {
        const int k8 = li + stride * i;
        px[i] = pd[i] = pnw[i] = pnb[i] = make_uint4(0u, 0u, 0u, 0u);
        if (live && k8 < K8) {
            px[i] = xr[k8];
            if (dr != nullptr) pd[i] = dr[k8];
            pnw[i] = reinterpret_cast<const uint4 *>(rw.nw)[k8];
            if (rw.kind == 2) pnb[i] = reinterpret_cast<const uint4 *>(rw.nb)[k8];
        }
    }
    float s1 = 0.f, s2 = 0.f;
    float v[DT_ROWREG][8];
    auto sum_piece = [&](int k8, uint4 keep, const uint4 &draw, float (&t)[8]) {
        dt_unpack8(keep, t);
        if (dr != nullptr) {
            float dd[8];
            dt_unpack8(draw, dd);
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = dt_round(t[j] + dd[j]);
            keep = dt_pack8(t);
        }
        if (xo != nullptr) xo[k8] = keep;
        zs[b * K8 + k8] = keep;
#pragma unroll
        for (int j = 0; j < 8; ++j) { s1 += t[j]; s2 = fmaf(t[j], t[j], s2); }
    };
    if (live) {
#pragma unroll
        for (int i = 0; i < DT_ROWREG; ++i)
            if (li + stride * i < K8) sum_piece(li + stride * i, px[i], pd[i], v[i]);
        for (int k8 = li + stride * DT_ROWREG; k8 < K8; k8 += stride) {   // rows longer than the register buffer
            float t[8];
            sum_piece(k8, xr[k8], dr != nullptr ? dr[k8] : make_uint4(0u, 0u, 0u, 0u), t);
        }
    }
    // a row's sum: its warps' partials, added in warp order by every thread of the row
    auto row_sum = [&](float x, int slot) {
        x = warp_sum(x);
        if (lane == 0) part[slot][warp] = x;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < wpr; ++w) tot += part[slot][(live ? b : 0) * wpr + w];
        return tot;
    };
    float mean = 0.f, rstd;
    if (rw.kind == 1) {
        rstd = rsqrtf(row_sum(s2, 0) / (float)K + rw.eps);
    } else {
        mean = row_sum(s1, 0) / (float)K;
        float sv = 0.f;
        if (live) {
#pragma unroll
            for (int i = 0; i < DT_ROWREG; ++i)
                if (li + stride * i < K8) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) { const float c = v[i][j] - mean; sv = fmaf(c, c, sv); }
                }
            for (int k8 = li + stride * DT_ROWREG; k8 < K8; k8 += stride) {
                float t[8];
                dt_unpack8(zs[b * K8 + k8], t);
#pragma unroll
                for (int j = 0; j < 8; ++j) { const float c = t[j] - mean; sv = fmaf(c, c, sv); }
            }
        }
        rstd = rsqrtf(row_sum(sv, 1) / (float)K + rw.eps);
    }
    auto norm_piece = [&](int k8, const float (&t)[8], const uint4 &wraw, const uint4 &braw) {
        float w[8], o[8];
        dt_unpack8(wraw, w);
        if (rw.kind == 2) {
            float bb[8];
            dt_unpack8(braw, bb);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = (t[j] - mean) * rstd * w[j] + bb[j];
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = t[j] * rstd * w[j];
        }
        zs[b * K8 + k8] = dt_pack8(o);
    };
    if (live) {
#pragma unroll
        for (int i = 0; i < DT_ROWREG; ++i)
            if (li + stride * i < K8) norm_piece(li + stride * i, v[i], pnw[i], pnb[i]);
        for (int k8 = li + stride * DT_ROWREG; k8 < K8; k8 += stride) {
            float t[8];
            dt_unpack8(zs[b * K8 + k8], t);
            norm_piece(k8, t, reinterpret_cast<const uint4 *>(rw.nw)[k8],
                       rw.kind == 2 ? reinterpret_cast<const uint4 *>(rw.nb)[k8] : make_uint4(0u, 0u, 0u, 0u));
        }
    }
    __syncthreads();
}

__device__ __forceinline__ void dt_cp_async16(void *smem_dst, const void *gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void dt_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void dt_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

constexpr int DT_PIECES = 12;                                         // 128-bit pieces of weights a lane has in flight per item
constexpr int DT_DEPTH = 3;                                           // items a warp has in flight or in use
constexpr int DT_STAGE_U4 = DT_DEPTH * DT_PIECES * 32;                // a warp's staging buffers, in uint4

// One linear phase: out[b][n] = act(sum_k W[n][k] z[b][k] + bias[n]) with z the rows rw describes.
//
// Output rows go in groups of R consecutive rows, groups dealt round-robin to the grid's warps; a warp's work is a list of
// items (group, chunk of 32 * U pieces of K), U = 12 / R, so a lane moves twelve 128-bit pieces per item. Weights travel
// global -> shared memory by asynchronous copies into the warp's own two staging buffers (no registers held while they
// fly; a lane reads back only what it copied itself). The first three items -- constants, nothing another CTA writes -- are
// requested between the two halves of the barrier that ends the previous phase (wait_first), so they travel from HBM
// while the barrier completes; after it the rows are built from the previous phase's output, and a warp with more items
// (the head) keeps two of them in flight while it multiplies a third. OUT: bf16, or fp32 holding the bf16-rounded value (the logits).
// NB: rows of z the instantiation multiplies (>= the batch; the surplus is computed on whatever shared memory holds and
// never written). False: the barrier gave up.
template <typename OUT, int R, int NB>
__device__ __noinline__ bool dt_phase_rb(const DtArgs &a, const DtRows &rw, bool wait_first, unsigned long long &gen,
                                            const __nv_bfloat16 *W, const __nv_bfloat16 *bias, int N, bool gelu, OUT *out, uint4 *zs,
                                            uint4 *wstage) {
    constexpr int U = DT_PIECES / R;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int K = rw.K, K8 = K >> 3, nwarps = gridDim.x * DT_WARPS, groups = (N + R - 1) / R;
    const int nchunks = (K8 + 32 * U - 1) / (32 * U);
    const int first = blockIdx.x * DT_WARPS + warp;
    uint4 *wb = wstage + warp * DT_STAGE_U4 + lane;
    float bias_q[DT_DEPTH] = {0.f, 0.f, 0.f};                         // of the output this lane will finish, requested with the weights
    // the items in order, walked by two cursors (requests ahead, multiplications behind) with no division in sight
    int ig = first, ic = 0, issued = 0;                               // next item to request: group, chunk; items requested so far
    auto issue = [&](int buf) {
        const int n0 = ig * R, k0 = ic * 32 * U;
        if (++ic == nchunks) { ic = 0; ig += nwarps; }
        ++issued;
        if (bias != nullptr && lane < R * NB && n0 + lane / NB < N) {
            const float bv = __bfloat162float(bias[n0 + lane / NB]);
#pragma unroll
            for (int i = 0; i < DT_DEPTH; ++i) if (i == buf) bias_q[i] = bv;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint4 *wr = reinterpret_cast<const uint4 *>(W + (size_t)(n0 + r < N ? n0 + r : N - 1) * K);
#pragma unroll 1
            for (int u = 0; u < U; ++u) {
                const int k8 = k0 + lane + 32 * u;
                if (k8 < K8) dt_cp_async16(wb + (buf * DT_PIECES + r * U + u) * 32, wr + k8);
            }
        }
        dt_cp_async_commit();
    };
    if (wait_first) dt_arrive(a.sync);                                // the previous phase's results are out: tell the grid, then ...
#pragma unroll
    for (int i = 0; i < DT_DEPTH; ++i)
        if (ig < groups) issue(i);                                    // ... request weights while the other CTAs arrive
    if (wait_first && !dt_wait(a.sync, gen)) return false;
    dt_build_rows(a, rw, zs);

    float acc[R][NB];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[r][b] = 0.f;
    int ck = 0, buf = 0;
    for (int it = 0, cgp = first; cgp < groups; ++it, buf = (buf + 1 == DT_DEPTH ? 0 : buf + 1)) {
        if (it + 2 < issued) dt_cp_async_wait<2>(); else if (it + 1 < issued) dt_cp_async_wait<1>(); else dt_cp_async_wait<0>();
        const int n0 = cgp * R, k0 = ck * 32 * U;
        float my_bias = 0.f;
#pragma unroll
        for (int i = 0; i < DT_DEPTH; ++i) if (i == buf) my_bias = bias_q[i];
        auto piece = [&](int u, int k8) {
            float w[R][8];
#pragma unroll
            for (int r = 0; r < R; ++r) dt_unpack8(wb[(buf * DT_PIECES + r * U + u) * 32], w[r]);
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                float z[8];
                dt_unpack8(zs[b * K8 + k8], z);
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[r][b] = fmaf(w[r][i], z[i], acc[r][b]);
            }
        };
        if constexpr (sizeof(OUT) == 4) {
            // the head: dozens of items per warp, so its loop is worth unrolling (instruction-level overlap between pieces)
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (k0 + lane + 32 * u < K8) piece(u, k0 + lane + 32 * u);
        } else {
            // a layer's phase runs once per token: its code is fetched, not cached, so it stays rolled and small
#pragma unroll 1
            for (int u = 0; u < U; ++u) {
                if (k0 + lane + 32 * u >= K8) break;
                piece(u, k0 + lane + 32 * u);
            }
        }
        if (ig < groups) issue(buf);                                  // this lane's slots of the buffer are free again
        if (++ck == nchunks) {
            ck = 0; cgp += nwarps;
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int b = 0; b < NB; ++b) acc[r][b] = warp_sum(acc[r][b]);
            // lane (r * NB + b) finishes and writes output (b, n0 + r): pick the value with selects, finish it once
            float mine = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    if (lane == r * NB + b) mine = acc[r][b];
                    acc[r][b] = 0.f;
                }
            const int r_ = lane / NB, b_ = lane % NB;
            if (lane < R * NB && b_ < a.B && n0 + r_ < N) {
                float v = dt_round(mine + my_bias);                   // the linear layer's bf16 output
                if (gelu) v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
                if constexpr (sizeof(OUT) == 2) out[(size_t)b_ * N + n0 + r_] = __float2bfloat16_rn(v);
                else out[(size_t)b_ * N + n0 + r_] = v;
            }
        }
    }
    return true;
}

template <typename OUT, int NB>
__device__ __noinline__ bool dt_phase(const DtArgs &a, const DtRows &rw, bool wait_first, unsigned long long &gen, const __nv_bfloat16 *W,
                                         const __nv_bfloat16 *bias, int N, bool gelu, OUT *out, uint4 *zs, uint4 *wstage) {
    // rows per group: enough that every warp of the grid gets about one group, at most four
    const int nwarps = gridDim.x * DT_WARPS, want = (N + nwarps - 1) / nwarps;
    if (want <= 1) return dt_phase_rb<OUT, 1, NB>(a, rw, wait_first, gen, W, bias, N, gelu, out, zs, wstage);
    if (want == 2) return dt_phase_rb<OUT, 2, NB>(a, rw, wait_first, gen, W, bias, N, gelu, out, zs, wstage);
    if (want == 3) return dt_phase_rb<OUT, 3, NB>(a, rw, wait_first, gen, W, bias, N, gelu, out, zs, wstage);
    return dt_phase_rb<OUT, 4, NB>(a, rw, wait_first, gen, W, bias, N, gelu, out, zs, wstage);
}

template <int D, bool DELTA, int NB>
__global__ void __launch_bounds__(DT_THREADS, 1) decode_token_kernel(DtArgs a) {
    extern __shared__ uint4 dt_smem[];                                // the warps' weight staging, the rows, the layer table
    uint4 *wstage = dt_smem;
    uint4 *zs = dt_smem + DT_WARPS * DT_STAGE_U4;                     // [NB][max(d, dff) / 8] pieces of 8 bf16
    // The layer table comes into shared memory once: a pointer fetched from global memory in every phase would be one more
    // round trip in front of the weights it points at.
    const DtLayer *layers = reinterpret_cast<const DtLayer *>(zs + (size_t)NB * ((a.dff > a.d ? a.dff : a.d) >> 3));
    {
        const uint2 *src = reinterpret_cast<const uint2 *>(a.layers);
        uint2 *dst = reinterpret_cast<uint2 *>(const_cast<DtLayer *>(layers));
        for (int i = threadIdx.x; i < a.L * (int)(sizeof(DtLayer) / 8); i += DT_THREADS) dst[i] = src[i];
    }
    __shared__ unsigned long long s_gen;
    if (threadIdx.x == 0) {
        unsigned long long c;
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(c) : "l"(a.sync) : "memory");
        s_gen = c / gridDim.x;                                        // barriers completed by earlier launches (this CTA has not arrived yet)
    }
    __syncthreads();
    unsigned long long gen = s_gen;
    const int d = a.d;
    __nv_bfloat16 *xcur = a.xa, *xoth = a.xb;

    for (int l = 0; l < a.L; ++l) {
        const DtLayer &ly = layers[l];
        // 1. projection (layer 0: the embedding is the sum)
        {
            const DtRows rw{l == 0 ? 2 : 1, xcur, a.dl, l == 0 ? xcur : xoth, ly.ln_kind, ly.ln_eps, ly.ln_w, ly.ln_b, d};
            if (!dt_phase<__nv_bfloat16, NB>(a, rw, l != 0, gen, ly.Wc, ly.bc, a.NP, false, a.y, zs, wstage)) return;
            if (l != 0) { __nv_bfloat16 *t = xcur; xcur = xoth; xoth = t; }
        }
        // 2. the recurrent state step, one (sequence, head) per CTA; its state loads are in flight across the barrier
        {
            DecodeArgs da{a.y, a.y + d, a.y + 2 * d, (long long)a.NP, 1, a.y + 3 * d + a.H, (long long)a.NP, 1, a.y + 3 * d, (long long)a.NP,
                          ly.A, ly.theta, a.shift, 0.f, ly.S, ly.S, ly.on_w, ly.on_eps, a.o, (long long)d, a.B, a.H};
            bool waited = false, alive = true;
            dt_arrive(a.sync);
            for (int bh = blockIdx.x; bh < a.B * a.H && alive; bh += gridDim.x) {
                decode_step_body<__nv_bfloat16, __nv_bfloat16, D, DELTA>(da, bh / a.H, bh % a.H, [&]() {
                    if (!waited) { waited = true; alive = dt_wait(a.sync, gen); }
                    return alive;
                });
                __syncthreads();
            }
            if (!waited) alive = dt_wait(a.sync, gen);
            if (!alive) return;
        }
        // 3. output projection
        {
            const DtRows rw{0, a.o, nullptr, nullptr, 0, 0.f, nullptr, nullptr, d};
            if (!dt_phase<__nv_bfloat16, NB>(a, rw, true, gen, ly.ow, nullptr, d, false, a.dl, zs, wstage)) return;
        }
        // 4. MLP up
        {
            const DtRows rw{1, xcur, a.dl, xoth, ly.n_kind, ly.n_eps, ly.n_w, ly.n_b, d};
            if (!dt_phase<__nv_bfloat16, NB>(a, rw, true, gen, ly.a_w, ly.a_b, a.dff, true, a.hmid, zs, wstage)) return;
            __nv_bfloat16 *t = xcur; xcur = xoth; xoth = t;
        }
        // 5. MLP down
        {
            const DtRows rw{0, a.hmid, nullptr, nullptr, 0, 0.f, nullptr, nullptr, a.dff};
            if (!dt_phase<__nv_bfloat16, NB>(a, rw, true, gen, ly.b_w, ly.b_b, d, false, a.dl, zs, wstage)) return;
        }
    }
    // ---- final norm and the tied head
    const DtRows rw{1, xcur, a.dl, nullptr, a.fn_kind, a.fn_eps, a.fn_w, a.fn_b, d};
    dt_phase<float, NB>(a, rw, true, gen, a.E, nullptr, a.V, false, a.logits, zs, wstage);
}

// The barrier's failure path on its own: one CTA arrives at a barrier of a "grid" that it alone will never complete
// (the counter would have to reach twice the arrivals), so its wait runs out after `limit` polls, raises the flag and the
// kernel returns normally.
__global__ void __launch_bounds__(DT_THREADS) decode_token_wait_selftest_kernel(unsigned long long *sync, unsigned limit) {
    unsigned long long gen = 1;                                       // as if one barrier had completed: the target is 2 arrivals, one comes
    dt_arrive(sync);
    dt_wait(sync, gen, limit);
}

int decode_token_wait_selftest_launch(unsigned long long *sync, unsigned limit, cudaStream_t stream) {
    decode_token_wait_selftest_kernel<<<1, DT_THREADS, 0, stream>>>(sync, limit);
    return check_launch("decode_token_wait_selftest_kernel");
}

int decode_token_error_flag(int *out) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(out, g_dt_error, sizeof(int));
    if (e == cudaSuccess && *out != 0) e = cudaMemcpyToSymbol(g_dt_error, &zero, sizeof(int));
    if (e != cudaSuccess) { set_cuda_error(e, "decode_token error flag"); return PGB_ERR_CUDA; }
    return PGB_OK;
}

// bf16 scratch of one step: two residual streams, o, delta (B x d each), the projection (B x NP), the MLP's middle (B x dff)
size_t decode_token_work_bytes(int B, int d, int NP, int dff) {
    return (size_t)B * ((size_t)4 * d + NP + dff) * sizeof(__nv_bfloat16);
}

template <int D, bool DELTA, int NB>
static int decode_token_go(const DtArgs &a, cudaStream_t stream) {
    int dev = 0, sms = 0, per_sm = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t smem = (size_t)DT_WARPS * DT_STAGE_U4 * sizeof(uint4) + (size_t)NB * (size_t)(a.dff > a.d ? a.dff : a.d) * sizeof(__nv_bfloat16) +
                        (size_t)a.L * sizeof(DtLayer);
    auto kern = decode_token_kernel<D, DELTA, NB>;
    if (e == cudaSuccess && smem > 32 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, DT_THREADS, smem);
    if (e != cudaSuccess || sms <= 0 || per_sm <= 0) {
        set_cuda_error(e == cudaSuccess ? cudaErrorLaunchOutOfResources : e, "decode_token set-up");
        return PGB_ERR_CUDA;
    }
    DtArgs args = a;
    void *params[] = {&args};
    // cooperative: either every CTA is resident at once (what the grid-wide barrier needs) or the launch fails
    e = cudaLaunchCooperativeKernel((const void *)kern, dim3((unsigned)sms), dim3(DT_THREADS), params, smem, stream);
    if (e != cudaSuccess) { set_cuda_error(e, "decode_token launch"); return PGB_ERR_CUDA; }
    return check_launch("decode_token_kernel");
}

template <int D, bool DELTA>
static int decode_token_nb(const DtArgs &a, cudaStream_t stream) {
    if (a.B == 1) return decode_token_go<D, DELTA, 1>(a, stream);
    if (a.B == 2) return decode_token_go<D, DELTA, 2>(a, stream);
    return decode_token_go<D, DELTA, 4>(a, stream);
}

int decode_token_launch(const void *layers, int L, const void *E, const void *P, const void *fn_w, const void *fn_b, int fn_kind,
                        float fn_eps, const long long *tok, const long long *pos, const float *shift, void *work, float *logits,
                        unsigned long long *sync, int B, int d, int H, int D, int NP, int dff, int V, int ctx, int delta,
                        cudaStream_t stream) {
    __nv_bfloat16 *w = (__nv_bfloat16 *)work;
    DtArgs a{};
    a.layers = (const DtLayer *)layers; a.E = (const __nv_bfloat16 *)E; a.P = (const __nv_bfloat16 *)P;
    a.fn_w = (const __nv_bfloat16 *)fn_w; a.fn_b = (const __nv_bfloat16 *)fn_b; a.tok = tok; a.pos = pos; a.shift = shift;
    a.xa = w; a.xb = a.xa + (size_t)B * d; a.o = a.xb + (size_t)B * d; a.dl = a.o + (size_t)B * d; a.y = a.dl + (size_t)B * d;
    a.hmid = a.y + (size_t)B * NP;
    a.logits = logits; a.sync = sync; a.L = L; a.B = B; a.d = d; a.H = H; a.NP = NP; a.dff = dff; a.V = V; a.ctx = ctx;
    a.fn_kind = fn_kind; a.fn_eps = fn_eps;
    if (D == 64) return delta ? decode_token_nb<64, true>(a, stream) : decode_token_nb<64, false>(a, stream);
    return delta ? decode_token_nb<128, true>(a, stream) : decode_token_nb<128, false>(a, stream);
}

}  // namespace pgb
