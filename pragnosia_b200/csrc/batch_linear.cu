// y = act(x W^T + bias) for a batch of decode rows (9 .. 128 sequences, one token each): the linear layers of the decode
// step between the few-row kernel (skinny_linear.cu, at most 8 rows on the CUDA cores) and the prefill GEMMs.
//
// With one token per sequence a linear layer reads its weight once (a few MB) and does almost no arithmetic per byte, so
// what it costs is latency: the kernel ahead, the first bytes from HBM, the way out. This kernel is built around that:
//
//   * the rows of x are the M side of one tcgen05 tile (64 rows, or 128 for batches past 64; rows past the batch are
//     zero-filled by the TMA unit and never stored), a CTA owns BN = 16 / 32 / 64 rows of W (the N side) and the whole K, so the grid is
//     N / BN CTAs -- about one per SM for the layer's matrices, each streaming its slab of W exactly once;
//   * up to sixteen TMA stages of 64 K-columns are in flight at once; the slabs of W (constants) are requested BEFORE the
//     wait on the kernel that produces x (programmatic dependent launch), the tiles of x right after it;
//   * one elected thread issues the MMAs stage by stage; four warps take the accumulator out of tensor memory (a row per
//     thread), add the bias, round to bf16 where the separate Linear would, apply the erf-GELU if asked, and store 16-byte
//     pieces of their row.
//
// x [B][K] bf16 (K contiguous) is the K-major A operand, W [N][K] (torch.nn.Linear layout) the K-major B operand.
// Replaces, for T = 1 and 8 < batch <= 128, the F.linear (+ GELU) calls of src/assoc.py:384-512 and src/model.py:552-560.
// Every mbarrier wait is bounded; a wait that runs out sets the error flag and the CTA winds down.
#include "tc_common.cuh"

namespace pgb {

constexpr int BL_BK = 64;
constexpr int BL_NT = 6 * 32;                                         // producer, issuer, four epilogue warps

// What the kernel can take over from the add + norm launches on either side of a linear layer (all optional).
//
// Folded norm (norm_kind 1 RMS / 2 layer norm): x is the raw residual stream y and W already carries the norm's weight
// (W'[n][k] = W[n][k] w[k]), so with the row's mean mu and 1 / sqrt(var + eps) = r,
//     norm(y) W^T + b = r (y W'^T - mu c1) + c2,    c1[n] = sum_k W'[n][k],  c2[n] = sum_k beta[k] W[n][k] + b[n]
// and the normalised row never exists in memory. The row sums come as partial sums (sum y, sum y^2) from the kernel
// that produced y: stats_in [parts_in][B][2].
// Residual (resid != NULL): the output is resid + (x W^T + b), both roundings of the separate ops kept, written as the new
// residual stream, and this CTA's partial row sums of it go to stats_out [gridDim.x][B][2] for the next folded norm.
struct BlFused {
    const float *stats_in; int parts_in; const float *c1, *c2; int norm_kind; float eps;
    const __nv_bfloat16 *resid; float *stats_out;
    int late_consts;                 // W, bias, c1, c2 may be the output of the kernel just ahead: read nothing before the wait
};

// One ring of stages in shared memory, a stage = one x tile (64 K-columns of every row) and one slab of W, up to 16 stages
// and 192 KiB: what a CTA waits for after the kernel ahead is its x, all of which it needs, so the deeper the ring the
// fewer round trips to the L2 (measured: a 3-deep ring of x costs 2 us a launch over an 8-deep one; separate rings and
// barriers for x and W cost another microsecond in the issuer's loop).
template <int BM, int BN> struct BlSizes {
    static constexpr int A_BYTES = BM * BL_BK * 2, W_BYTES = BN * BL_BK * 2, STAGE = A_BYTES + W_BYTES;
    static constexpr int STAGES = 192 * 1024 / STAGE < 16 ? 192 * 1024 / STAGE : 16;
    static constexpr int SMEM = STAGES * STAGE + 1024 + 1024;         // stages, barriers, alignment slack
};

__device__ __forceinline__ void bl_tma_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(0) : "memory");
}
__device__ __forceinline__ bool bl_elect_one() {
    uint32_t e;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(e));
    return e != 0;
}

template <int BM, int BN>
__global__ void __launch_bounds__(BL_NT, 1) batch_linear_kernel(const __grid_constant__ CUtensorMap mx, const __grid_constant__ CUtensorMap mw,
                                                               const __nv_bfloat16 *__restrict__ bias, __nv_bfloat16 *__restrict__ y,
                                                               int B, int N, int K, int act, BlFused f) {
    constexpr int STAGE = BlSizes<BM, BN>::STAGE, STAGES = BlSizes<BM, BN>::STAGES, A_BYTES = BlSizes<BM, BN>::A_BYTES;
    constexpr int ACC = BN < 32 ? 32 : BN;                            // columns of one accumulator: loads come 32 columns at a time
    constexpr int TCOLS = 2 * ACC;                                    // two accumulators (see the issuer): a power of two, at least 32
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t mb = base + STAGES * STAGE;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + STAGES * STAGE + 512);
    auto bar_full = [&](int s) { return mb + 8 * s; };
    auto bar_empty = [&](int s) { return mb + 128 + 8 * s; };
    const uint32_t bar_acc = mb + 256;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n0 = blockIdx.x * BN;
    const int KB = (K + BL_BK - 1) / BL_BK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
        mbar_init(bar_acc, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TCOLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------------------------------------ producer
        const bool leader = bl_elect_one();
        const int pre = KB < STAGES ? KB : STAGES;
        // The weight slabs do not depend on the kernel ahead -- unless the caller says that kernel produced them (a cast, a
        // copy made contiguous just now): then they are requested after the wait like x.
        auto request_w = [&]() {
            for (int kb = 0; kb < pre; ++kb) {
                mbar_expect_tx(bar_full(kb), STAGE);
                bl_tma_2d(base + kb * STAGE + A_BYTES, &mw, bar_full(kb), kb * BL_BK, n0);
            }
        };
        if (leader && !f.late_consts) request_w();
        pdl_wait();                                                   // x is the kernel ahead's output
        if (leader) {
            if (f.late_consts) request_w();
            for (int kb = 0; kb < pre; ++kb) bl_tma_2d(base + kb * STAGE, &mx, bar_full(kb), kb * BL_BK, 0);
        }
        __syncwarp();
        bool ok = true;
        for (int kb = pre; kb < KB && ok; ++kb) {
            const int s = kb % STAGES;
            ok = __all_sync(0xffffffffu, mbar_wait(bar_empty(s), ((kb / STAGES) + 1) & 1, 75));
            if (ok && leader) {
                mbar_expect_tx(bar_full(s), STAGE);
                bl_tma_2d(base + s * STAGE + A_BYTES, &mw, bar_full(s), kb * BL_BK, n0);
                bl_tma_2d(base + s * STAGE, &mx, bar_full(s), kb * BL_BK, 0);
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------------------------------ MMA issuer
        constexpr uint32_t IDESC = idesc_bf16(BM, BN, 0, 0);
        bool ok = true;
        for (int kb = 0; kb < KB && ok; ++kb) {
            const int s = kb % STAGES;
            ok = __all_sync(0xffffffffu, mbar_wait(bar_full(s), (kb / STAGES) & 1, 76));
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = base + s * STAGE;
            const uint64_t da = smem_desc(sa, 16, 1024), db = smem_desc(sa + A_BYTES, 16, 1024);
            // consecutive MMAs alternate between two accumulators, so no MMA waits for the one just before it; the epilogue
            // adds the two
#pragma unroll
            for (int k = 0; k < BL_BK / 16; ++k)
                mma_bf16_elect(tmem + (k & 1) * ACC, da + k * 2, db + k * 2, IDESC, (kb != 0 || k >= 2) ? 1u : 0u);
            mma_commit_elect(bar_empty(s));                           // the stage is free once these MMAs have read it
        }
        if (ok) mma_commit_elect(bar_acc);
    } else {
        // ------------------------------------------------------------------------------------------ epilogue: a row per thread
        // 128 rows: tensor-memory lane = row. 64 rows: each quarter of the lanes holds 16 rows in its first 16 lanes.
        const int sub = warp & 3;
        const int row = BM == 128 ? 32 * sub + lane : (lane < 16 ? 16 * sub + lane : BM);
        const uint32_t lane_base = (uint32_t)(32 * sub) << 16;
        // the CTA's bias values (the same for every row), requested before the accumulator is waited for; the folded norm's
        // two vectors only as far as the L1 (after the wait on the kernel ahead if it may have produced them)
        if (f.late_consts) pdl_wait();
        uint4 braw[BN / 8];
#pragma unroll
        for (int g = 0; g < BN / 8; ++g) {
            braw[g] = make_uint4(0u, 0u, 0u, 0u);
            if (bias != nullptr && n0 + 8 * g < N) braw[g] = *reinterpret_cast<const uint4 *>(bias + n0 + 8 * g);
        }
        if (f.norm_kind != 0 && lane < BN / 8 && n0 + 8 * lane < N) {
            asm volatile("prefetch.global.L1 [%0];" ::"l"(f.c1 + n0 + 8 * lane));
            asm volatile("prefetch.global.L1 [%0];" ::"l"(f.c2 + n0 + 8 * lane));
        }
        float mu = 0.f, rstd = 1.f;
        uint4 rraw[BN <= 16 ? BN / 8 : 1];                            // the residual is taken with the narrowest slab only
        if (f.stats_in != nullptr || f.resid != nullptr) {
            pdl_wait();                                               // both are the work of kernels ahead
            if (f.norm_kind != 0 && row < B) {
                float s1 = 0.f, s2 = 0.f;
                for (int p = 0; p < f.parts_in; ++p) {                // fixed order: the same sums on every run
                    const float2 t = *reinterpret_cast<const float2 *>(f.stats_in + ((size_t)p * B + row) * 2);
                    s1 += t.x; s2 += t.y;
                }
                if (f.norm_kind == 2) mu = s1 / (float)K;
                rstd = rsqrtf(fmaxf(s2 / (float)K - mu * mu, 0.f) + f.eps);
            }
            if constexpr (BN <= 16) {
#pragma unroll
                for (int g = 0; g < BN / 8; ++g) {
                    rraw[g] = make_uint4(0u, 0u, 0u, 0u);
                    if (f.resid != nullptr && row < B && n0 + 8 * g < N) rraw[g] = *reinterpret_cast<const uint4 *>(f.resid + (size_t)row * N + n0 + 8 * g);
                }
            }
        }
        float q1 = 0.f, q2 = 0.f;                                     // this row's partial sums of the new residual stream
        const bool ok = __all_sync(0xffffffffu, mbar_wait(bar_acc, 0, 77));
        if (ok) {
            tc_fence_after();
#pragma unroll
            for (int c0 = 0; c0 < BN; c0 += 32) {
                float v[32], v1[32];
                tmem_ld32_nowait(tmem + lane_base + c0, v);           // BN = 16: the upper half of the 32 columns is never used
                tmem_ld32(tmem + lane_base + ACC + c0, v1);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] += v1[i];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int col = n0 + c0 + 8 * g;
                    if (c0 + 8 * g < BN && col < N && row < B) {
                        float bv[8];
                        {
                            const __nv_bfloat162 *b2 = reinterpret_cast<const __nv_bfloat162 *>(&braw[(c0 >> 3) + g < BN / 8 ? (c0 >> 3) + g : 0]);
#pragma unroll
                            for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(b2[i]); bv[2 * i] = t.x; bv[2 * i + 1] = t.y; }
                        }
                        float lin[8];
                        if (f.norm_kind != 0) {
                            const float4 ca = *reinterpret_cast<const float4 *>(f.c1 + col), cb = *reinterpret_cast<const float4 *>(f.c1 + col + 4);
                            const float4 da = *reinterpret_cast<const float4 *>(f.c2 + col), dd = *reinterpret_cast<const float4 *>(f.c2 + col + 4);
                            const float c1v[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
                            const float c2v[8] = {da.x, da.y, da.z, da.w, dd.x, dd.y, dd.z, dd.w};
#pragma unroll
                            for (int i = 0; i < 8; ++i) lin[i] = fmaf(rstd, v[8 * g + i] - mu * c1v[i], c2v[i]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) lin[i] = v[8 * g + i] + bv[i];
                        }
                        uint4 outv;
                        __nv_bfloat16 *o = reinterpret_cast<__nv_bfloat16 *>(&outv);
                        float rv[8];
                        if constexpr (BN <= 16) {
                            const __nv_bfloat162 *r2 = reinterpret_cast<const __nv_bfloat162 *>(&rraw[g < BN / 8 ? g : 0]);
#pragma unroll
                            for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(r2[i]); rv[2 * i] = t.x; rv[2 * i + 1] = t.y; }
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            // the pre-activation, rounded to bf16 as the separate Linear would hand it on
                            float x = __bfloat162float(__float2bfloat16_rn(lin[i]));
                            if (act == 1) x = 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
                            if constexpr (BN <= 16) {
                                if (f.resid != nullptr) {
                                    x = __bfloat162float(__float2bfloat16_rn(__bfloat162float(__float2bfloat16_rn(x)) + rv[i]));
                                    q1 += x; q2 = fmaf(x, x, q2);
                                }
                            }
                            o[i] = __float2bfloat16_rn(x);
                        }
                        *reinterpret_cast<uint4 *>(y + (size_t)row * N + col) = outv;
                    }
                }
            }
            if (f.stats_out != nullptr && row < B) *reinterpret_cast<float2 *>(f.stats_out + ((size_t)blockIdx.x * B + row) * 2) = make_float2(q1, q2);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TCOLS);
}

template <int BM, int BN>
static int batch_linear_go(const void *x, const void *W, const void *bias, void *y, int B, int N, int K, int act, const BlFused &f,
                           cudaStream_t stream) {
    CUtensorMap mx, mw;
    if (!tc_make_map(&mx, x, 1, B, K, K, (long long)B * K, BM) || !tc_make_map(&mw, W, 1, N, K, K, (long long)N * K, BN)) {
        set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled");
        return PGB_ERR_CUDA;
    }
    constexpr int SMEM = BlSizes<BM, BN>::SMEM;
    cudaError_t e = cudaFuncSetAttribute(batch_linear_kernel<BM, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) { set_cuda_error(e, "batch_linear smem attribute"); return PGB_ERR_CUDA; }
    e = pdl_launch(batch_linear_kernel<BM, BN>, dim3((unsigned)((N + BN - 1) / BN)), dim3(BL_NT), (size_t)SMEM, stream, mx, mw,
                   (const __nv_bfloat16 *)bias, (__nv_bfloat16 *)y, B, N, K, act, f);
    if (e != cudaSuccess) { set_cuda_error(e, "batch_linear launch"); return PGB_ERR_CUDA; }
    return check_launch("batch_linear_kernel");
}

// CTAs (= partial row sums written) a launch with a residual uses: the narrowest slab
int batch_linear_parts(int N) { return (N + 15) / 16; }

int batch_linear_launch(const void *x, const void *W, const void *bias, void *y, int B, int N, int K, int act, const float *stats_in,
                        int parts_in, const float *c1, const float *c2, int norm_kind, float eps, const void *resid, float *stats_out,
                        int late_consts, cudaStream_t stream) {
    const BlFused f{stats_in, parts_in, c1, c2, norm_kind, eps, (const __nv_bfloat16 *)resid, stats_out, late_consts};
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // the narrowest slab that still gives about one CTA per SM: every CTA re-reads x from the L2, so fewer, wider CTAs
    // once the grid would pass the SM count. A residual (and the row sums that go with it) is taken by the narrowest only.
    const int bn = (resid != nullptr || stats_out != nullptr || (N + 15) / 16 <= sms) ? 16 : ((N + 31) / 32 <= sms ? 32 : 64);
    if (B <= 64) {
        if (bn == 16) return batch_linear_go<64, 16>(x, W, bias, y, B, N, K, act, f, stream);
        if (bn == 32) return batch_linear_go<64, 32>(x, W, bias, y, B, N, K, act, f, stream);
        return batch_linear_go<64, 64>(x, W, bias, y, B, N, K, act, f, stream);
    }
    if (bn == 16) return batch_linear_go<128, 16>(x, W, bias, y, B, N, K, act, f, stream);
    if (bn == 32) return batch_linear_go<128, 32>(x, W, bias, y, B, N, K, act, f, stream);
    return batch_linear_go<128, 64>(x, W, bias, y, B, N, K, act, f, stream);
}

int batch_linear_error_flag(int *out) { return tc_read_error_flag(out); }

}  // namespace pgb
