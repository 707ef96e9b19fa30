// Per-token complex recurrence h_t = lambda_t h_{t-1} + u_t as a chunked parallel scan.
//
// Layout in HBM: u, logmag, y are [B][T][D] fp32 with D contiguous: 12 B read (8 B when the angle is one value per
// channel) and 4 B written per (b,t,d) element. Measured, the kernel is bound by instruction issue before HBM (accurate
// expf and sincosf per element), so the tile is kept small (SEG = 4 steps a lane) for 24 resident warps per SM.
//
// Work split. A lane owns VEC adjacent channels (VEC = 4: one 128-bit access). A warp is TS time-segments x CQ
// channel groups (TS * CQ = 32): lanes of one segment read 16*CQ contiguous bytes of one time row, so every 128-byte
// line is used whole. A tile is TS*SEG consecutive time steps; per tile each lane
//   1. loads its SEG steps (all loads issued before any is used) and forms c_t = |l_t| cos, s_t = |l_t| sin,
//   2. folds them into the segment's affine map h -> A h + Bv (complex A, Bv), starting from (1, 0),
//   3. combines the maps of the segments before it with a shuffle scan over the TS segment lanes
//      ((A2,B2) o (A1,B1) = (A2 A1, A2 B1 + B2)), which gives the state entering its segment,
//   4. replays the recurrence over its SEG steps from that state in the reference's operation order
//      (src/scan_kernel.py:42-48) and stores Re h.
// The state leaving the tile is broadcast from the last segment lane. With TS = 1 the kernel is the literal sequential
// recurrence; with TS > 1 only the state at segment boundaries is reassociated (fp32 rounding, no other difference).
#include "common.cuh"

namespace pgb {

constexpr int LS_SEG_VEC4 = 4;      // steps a lane owns per tile, 128-bit path: 12 values x 4 channels x 4 steps in registers
constexpr int LS_SEG_VEC1 = 8;      // scalar path (D not a multiple of 4, or unaligned)
constexpr int LS_WARPS = 4;
constexpr int LS_CTAS_PER_SM = 6;   // 24 warps an SM = 6 a scheduler, whose 16 K registers then allow 80 a thread

template <int VEC>
__device__ __forceinline__ void ld_vec(float (&d)[VEC], const float *p) {
    if constexpr (VEC == 4) {
        float4 t = *reinterpret_cast<const float4 *>(p);
        d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w;
    } else {
        d[0] = *p;
    }
}
template <int VEC>
__device__ __forceinline__ void st_vec(float *p, const float (&d)[VEC]) {
    if constexpr (VEC == 4) {
        *reinterpret_cast<float4 *>(p) = make_float4(d[0], d[1], d[2], d[3]);
    } else {
        *p = d[0];
    }
}

template <int VEC, int TS, bool ANG_BCAST, int SEG>
__global__ void __launch_bounds__(LS_WARPS * 32, TS == 32 ? LS_CTAS_PER_SM - 1 : LS_CTAS_PER_SM)   // 32 segments are chosen when warps are scarce: registers over occupancy
lambda_scan_kernel(const float *__restrict__ u, const float *__restrict__ lm, const float *__restrict__ an,
                   long long an_sb, long long an_st, const float *__restrict__ h0r, const float *__restrict__ h0i,
                   float *__restrict__ y, float *__restrict__ hr_out, float *__restrict__ hi_out, float *__restrict__ hi_all,
                   int B, int T, int D) {
    constexpr int CQ = 32 / TS;
    constexpr unsigned FULL = 0xffffffffu;
    const int lane = threadIdx.x & 31;
    const int ngroups = (D + VEC - 1) / VEC;
    const int wpb = (ngroups + CQ - 1) / CQ;                       // warps per batch row
    const long long wg = (long long)blockIdx.x * LS_WARPS + (threadIdx.x >> 5);
    if (wg >= (long long)B * wpb) return;                          // a whole warp leaves together
    const int b = (int)(wg / wpb);
    const int cq = lane % CQ;
    const int seg = lane / CQ;
    const int grp = (int)(wg % wpb) * CQ + cq;
    const bool live = grp < ngroups;
    const int d0 = live ? grp * VEC : 0;

    float hr[VEC], hi[VEC];                                        // state entering the current tile
#pragma unroll
    for (int v = 0; v < VEC; ++v) { hr[v] = 0.f; hi[v] = 0.f; }
    if (h0r != nullptr && live) {
        ld_vec<VEC>(hr, h0r + (size_t)b * D + d0);
        ld_vec<VEC>(hi, h0i + (size_t)b * D + d0);
    }
    float acs[VEC], asn[VEC];                                      // cos / sin of a per-channel angle
    if constexpr (ANG_BCAST) {
        float a[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) a[v] = 0.f;
        if (live) ld_vec<VEC>(a, an + d0);
#pragma unroll
        for (int v = 0; v < VEC; ++v) sincosf(a[v], &asn[v], &acs[v]);
    }

    const size_t row0 = (size_t)b * T;
    for (int t0 = 0; t0 < T; t0 += TS * SEG) {
        const int tb = t0 + seg * SEG;
        float c[SEG][VEC], s[SEG][VEC], x[SEG][VEC];
        // 1. loads first, all of them
#pragma unroll
        for (int i = 0; i < SEG; ++i) {
            const int t = tb + i;
            if (live && t < T) {
                const size_t off = (row0 + t) * D + d0;
                ld_vec<VEC>(x[i], u + off);
                ld_vec<VEC>(c[i], lm + off);
                if constexpr (!ANG_BCAST) ld_vec<VEC>(s[i], an + (size_t)b * an_sb + (size_t)t * an_st + d0);
            } else {
#pragma unroll
                for (int v = 0; v < VEC; ++v) { x[i][v] = 0.f; c[i][v] = 0.f; s[i][v] = 0.f; }
            }
        }
        // c, s of every step; steps past the end are the identity map
#pragma unroll
        for (int i = 0; i < SEG; ++i) {
            const bool ok = live && (tb + i) < T;
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                const float mag = expf(c[i][v]);
                float cs, sn;
                if constexpr (ANG_BCAST) { cs = acs[v]; sn = asn[v]; }
                else sincosf(s[i][v], &sn, &cs);
                c[i][v] = ok ? mag * cs : 1.f;
                s[i][v] = ok ? mag * sn : 0.f;
            }
        }
        float hsr[VEC], hsi[VEC];                                  // state entering this lane's segment
        if constexpr (TS > 1) {
            // 2. the segment's affine map
            float Ar[VEC], Ai[VEC], Br[VEC], Bi[VEC];
#pragma unroll
            for (int v = 0; v < VEC; ++v) { Ar[v] = 1.f; Ai[v] = 0.f; Br[v] = 0.f; Bi[v] = 0.f; }
#pragma unroll
            for (int i = 0; i < SEG; ++i) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    const float nbr = c[i][v] * Br[v] - s[i][v] * Bi[v] + x[i][v];
                    const float nbi = s[i][v] * Br[v] + c[i][v] * Bi[v];
                    const float nar = c[i][v] * Ar[v] - s[i][v] * Ai[v];
                    const float nai = s[i][v] * Ar[v] + c[i][v] * Ai[v];
                    Br[v] = nbr; Bi[v] = nbi; Ar[v] = nar; Ai[v] = nai;
                }
            }
            // 3. inclusive scan over the segment lanes (same cq, lanes CQ apart)
#pragma unroll
            for (int off = 1; off < TS; off <<= 1) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    const float par = __shfl_up_sync(FULL, Ar[v], off * CQ);
                    const float pai = __shfl_up_sync(FULL, Ai[v], off * CQ);
                    const float pbr = __shfl_up_sync(FULL, Br[v], off * CQ);
                    const float pbi = __shfl_up_sync(FULL, Bi[v], off * CQ);
                    if (seg >= off) {
                        const float nbr = Ar[v] * pbr - Ai[v] * pbi + Br[v];
                        const float nbi = Ai[v] * pbr + Ar[v] * pbi + Bi[v];
                        const float nar = Ar[v] * par - Ai[v] * pai;
                        const float nai = Ai[v] * par + Ar[v] * pai;
                        Br[v] = nbr; Bi[v] = nbi; Ar[v] = nar; Ai[v] = nai;
                    }
                }
            }
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                float ear = __shfl_up_sync(FULL, Ar[v], CQ);
                float eai = __shfl_up_sync(FULL, Ai[v], CQ);
                float ebr = __shfl_up_sync(FULL, Br[v], CQ);
                float ebi = __shfl_up_sync(FULL, Bi[v], CQ);
                if (seg == 0) { ear = 1.f; eai = 0.f; ebr = 0.f; ebi = 0.f; }
                hsr[v] = ear * hr[v] - eai * hi[v] + ebr;
                hsi[v] = eai * hr[v] + ear * hi[v] + ebi;
            }
        } else {
#pragma unroll
            for (int v = 0; v < VEC; ++v) { hsr[v] = hr[v]; hsi[v] = hi[v]; }
        }
        // 4. replay in the reference's order and store Re h
#pragma unroll
        for (int i = 0; i < SEG; ++i) {
            const int t = tb + i;
            float out[VEC];
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                const float nr = c[i][v] * hsr[v] - s[i][v] * hsi[v] + x[i][v];
                const float ni = s[i][v] * hsr[v] + c[i][v] * hsi[v];
                hsr[v] = nr; hsi[v] = ni; out[v] = nr;
            }
            if (live && t < T) {
                st_vec<VEC>(y + (row0 + t) * D + d0, out);
                if (hi_all != nullptr) st_vec<VEC>(hi_all + (row0 + t) * D + d0, hsi);   // Im h, kept only for a backward pass
            }
        }
        // state leaving the tile: the last segment's final state
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            if constexpr (TS > 1) {
                hr[v] = __shfl_sync(FULL, hsr[v], (TS - 1) * CQ + cq);
                hi[v] = __shfl_sync(FULL, hsi[v], (TS - 1) * CQ + cq);
            } else {
                hr[v] = hsr[v]; hi[v] = hsi[v];
            }
        }
    }
    if (live && seg == 0) {
        st_vec<VEC>(hr_out + (size_t)b * D + d0, hr);
        st_vec<VEC>(hi_out + (size_t)b * D + d0, hi);
    }
}

namespace {

struct DevInfo { int sms = 0; bool ok = false; };
DevInfo dev_info() {
    // queried per call: cheap, and correct when the caller switches devices
    DevInfo d; int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return d;
    if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return d;
    d.ok = true; return d;
}

template <int VEC, int TS, int SEG>
int launch_ts(const float *u, const float *lm, const float *an, long long sb, long long st, const float *h0r,
              const float *h0i, float *y, float *hro, float *hio, float *hia, int B, int T, int D, cudaStream_t stream) {
    constexpr int CQ = 32 / TS;
    const int ngroups = (D + VEC - 1) / VEC;
    const long long warps = (long long)B * ((ngroups + CQ - 1) / CQ);
    const long long ctas = (warps + LS_WARPS - 1) / LS_WARPS;
    if (ctas > 0x7fffffffLL) return PGB_ERR_TOO_LARGE;
    if (sb == 0 && st == 0)
        lambda_scan_kernel<VEC, TS, true, SEG><<<(unsigned)ctas, LS_WARPS * 32, 0, stream>>>(u, lm, an, sb, st, h0r, h0i, y, hro, hio, hia, B, T, D);
    else
        lambda_scan_kernel<VEC, TS, false, SEG><<<(unsigned)ctas, LS_WARPS * 32, 0, stream>>>(u, lm, an, sb, st, h0r, h0i, y, hro, hio, hia, B, T, D);
    return check_launch("lambda_scan_kernel");
}

template <int VEC, int SEG>
int launch_vec(int ts, const float *u, const float *lm, const float *an, long long sb, long long st, const float *h0r,
               const float *h0i, float *y, float *hro, float *hio, float *hia, int B, int T, int D, cudaStream_t stream) {
    switch (ts) {
        case 1:  return launch_ts<VEC, 1, SEG>(u, lm, an, sb, st, h0r, h0i, y, hro, hio, hia, B, T, D, stream);
        case 2:  return launch_ts<VEC, 2, SEG>(u, lm, an, sb, st, h0r, h0i, y, hro, hio, hia, B, T, D, stream);
        case 4:  return launch_ts<VEC, 4, SEG>(u, lm, an, sb, st, h0r, h0i, y, hro, hio, hia, B, T, D, stream);
        case 8:  return launch_ts<VEC, 8, SEG>(u, lm, an, sb, st, h0r, h0i, y, hro, hio, hia, B, T, D, stream);
        case 16: return launch_ts<VEC, 16, SEG>(u, lm, an, sb, st, h0r, h0i, y, hro, hio, hia, B, T, D, stream);
        default: return launch_ts<VEC, 32, SEG>(u, lm, an, sb, st, h0r, h0i, y, hro, hio, hia, B, T, D, stream);
    }
}

}  // namespace

// Number of time segments per warp. The kernel is bound by instruction issue (about 80 instructions per element with a
// per-token angle), every warp walks its whole time axis, and all warps of a launch take the same time, so the launch
// lasts rounds x tiles-per-warp x tile cost with rounds = ceil(warps / resident warps). More segments shorten a warp's
// walk but cost shuffle-scan rounds and, past the resident capacity, a whole extra round. Take the power of two with the
// smallest estimate. `force_ts` > 0 overrides (tests).
int lambda_scan_pick_ts(int B, int T, int D, int vec, int sms, int force_ts) {
    if (force_ts > 0) return force_ts;
    const int seg = vec == 4 ? LS_SEG_VEC4 : LS_SEG_VEC1;
    const int ngroups = (D + vec - 1) / vec;
    const long long cap = (long long)sms * LS_CTAS_PER_SM * LS_WARPS;           // resident warps
    int best = 1;
    double best_cost = 0.0;
    for (int ts = 1, lg = 0; ts <= 32; ts <<= 1, ++lg) {
        if (ts > 1 && (ts / 2) * seg >= T) break;                               // the sequence has no more pieces to hand out
        const int cq = 32 / ts;
        const long long warps = (long long)B * ((ngroups + cq - 1) / cq);
        const long long rounds = (warps + cap - 1) / cap;
        const long long tiles = (T + ts * seg - 1) / (ts * seg);
        const double tile = seg * 60.0 + lg * 14.0 + 12.0;                      // per lane and channel: steps, scan rounds, hand-over
        const double cost = (double)rounds * (double)tiles * tile;
        if (ts == 1 || cost < best_cost) { best = ts; best_cost = cost; }
    }
    return best;
}

int lambda_scan_launch(const float *u, const float *lm, const float *an, long long sb, long long st, const float *h0r,
                       const float *h0i, float *y, float *hro, float *hio, float *hia, int B, int T, int D, int force_ts,
                       cudaStream_t stream) {
    DevInfo di = dev_info();
    const int sms = di.ok ? di.sms : 148;
    const bool v4 = (D % 4 == 0) && aligned(u, 16) && aligned(lm, 16) && aligned(an, 16) && aligned(y, 16) && aligned(hia, 16) &&
                    aligned(hro, 16) && aligned(hio, 16) && (h0r == nullptr || (aligned(h0r, 16) && aligned(h0i, 16))) &&
                    (sb % 4 == 0) && (st % 4 == 0);
    const int ts = lambda_scan_pick_ts(B, T, D, v4 ? 4 : 1, sms, force_ts);
    return v4 ? launch_vec<4, LS_SEG_VEC4>(ts, u, lm, an, sb, st, h0r, h0i, y, hro, hio, hia, B, T, D, stream)
              : launch_vec<1, LS_SEG_VEC1>(ts, u, lm, an, sb, st, h0r, h0i, y, hro, hio, hia, B, T, D, stream);
}

}  // namespace pgb
