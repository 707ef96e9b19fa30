// The C ABI: argument checks on the host, then one launch. Declarations and contracts: include/pragnosia_b200.h.
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace pgb {

static thread_local char g_err[256] = "";

void set_cuda_error(cudaError_t e, const char *where) {
    snprintf(g_err, sizeof(g_err), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
}


int lambda_scan_launch(const float *, const float *, const float *, long long, long long, const float *, const float *,
                       float *, float *, float *, float *, int, int, int, int, cudaStream_t);
int lambda_scan_bwd_launch(const float *, const float *, const float *, const float *, long long, long long, const float *, const float *,
                           const float *, float *, float *, float *, float *, float *, int, int, int, cudaStream_t);
int prep_bwd_launch(const void *, const void *, const void *, int, long long, long long, long long, const void *, long long, long long,
                    const float *, const long long *, const void *, const void *, const void *, int, void *, void *, void *, float *,
                    float *, int, int, int, int, cudaStream_t);
int prep_bwd_tiles(int T);
int assoc_out_launch(const void *, const void *, const void *, int, const float *, const void *, void *, int, int, int, cudaStream_t);
int prefix_scan_launch(const void *, const void *, int, const float *, const float *, const float *, void *, float *, int, int, int,
                       cudaStream_t);
int delta_loop_launch(const void *, const void *, int, const float *, const float *, const void *, const float *, void *, void *, float *,
                      int, int, int, cudaStream_t);
int delta_inv_launch(const void *, const float *, const float *, void *, int, int, int, cudaStream_t);
int assoc_out_bwd_launch(const void *, const void *, const void *, int, const float *, const void *, const void *, float *, float *, float *,
                         float *, float *, int, int, int, cudaStream_t);
int delta_inv_bwd_launch(const void *, int, const float *, const float *, const void *, const float *, float *, float *, float *, int, int, int,
                         cudaStream_t);
int delta_loop_bwd_launch(const void *, const void *, int, const float *, const float *, const void *, const void *, const float *, const float *,
                          const float *, float *, float *, float *, float *, float *, float *, int, int, int, cudaStream_t);
int prefix_scan_bwd_launch(const void *, const void *, int, const float *, const float *, const void *, const float *, const float *, float *,
                           float *, float *, float *, float *, int, int, int, cudaStream_t);
int key_topk_launch(void *, int, long long, long long, long long, int, int, int, int, int, cudaStream_t);
int short_conv_launch(const void *, int, long long, long long, const void *, const void *, void *, void *, int, int, int, int, cudaStream_t);
int lambda_scan_pick_ts(int B, int T, int D, int vec, int sms, int force_ts);
int prep_launch(const void *, const void *, const void *, int, long long, long long, long long, const void *, long long,
                long long, const float *, const long long *, void *, void *, void *, int, int, int, int, int, cudaStream_t);
int prefill_fp32_launch(const PrefillArgs &, int, int, int, cudaStream_t);
int prefill_tc_launch(const PrefillArgs &, int, int, cudaStream_t);
bool prefill_tc_supported(int io_dtype, int D, bool delta);
int decode_launch(const DecodeArgs &, int, int, int, int, cudaStream_t);
int tc_error_flag(int *out);
int tc_wait_selftest_launch(long long, cudaStream_t);
int tc_delta_error_flag(int *out);
int tc_ws_error_flag(int *out);
int prefill_tc_ws_launch(const PrefillArgs &, int, cudaStream_t);
size_t prefill_tc_delta_scratch_bytes(int B, int H, int T);
int prefill_tc_delta_launch(const PrefillArgs &, int, int, void *, cudaStream_t);
int prefill_tc_delta_static_launch(const PrefillArgs &, int, int, cudaStream_t);
long long prefill_tc_delta_static_capacity();
int rot_table_launch(const float *, float *, int, int, int, cudaStream_t);
int decode_embed_launch(const long long *, const long long *, const void *, const void *, void *, int, int, int, int, float *, cudaStream_t);
int decode_sample_launch(const void *, int, float, float, unsigned long long, long long *, long long *, int, long long *, long long *, float *,
                         unsigned int *, int, int, int, cudaStream_t);
int linear_gelu_launch(const void *, const void *, const void *, void *, long long, int, int, int, cudaStream_t);
int linear_gelu_error_flag(int *);
int linear_gelu_set_variant(int);
int decode_set_variant(int);
int skinny_linear_launch(const void *, const void *, const void *, const void *, int, float, const void *, const void *, int, void *,
                         void *, int, int, int, int, cudaStream_t);
int add_norm_launch(const void *, const void *, const void *, const void *, float, int, void *, void *, long long, int, int,
                    cudaStream_t);
int rotate_launch(const void *, int, const float *, const float *, void *, int, int, int, int, cudaStream_t);
int decode_token_launch(const void *, int, const void *, const void *, const void *, const void *, int, float, const long long *,
                        const long long *, const float *, void *, float *, unsigned long long *, int, int, int, int, int, int, int, int,
                        int, cudaStream_t);
size_t decode_token_work_bytes(int B, int d, int NP, int dff);
int decode_token_error_flag(int *);
int batch_linear_launch(const void *, const void *, const void *, void *, int, int, int, int, const float *, int, const float *, const float *,
                        int, float, const void *, float *, int, cudaStream_t);
int batch_linear_parts(int N);
int batch_linear_error_flag(int *);
int decode_token_wait_selftest_launch(unsigned long long *, unsigned, cudaStream_t);

// PGB_PREFILL_AUTO sends bf16 plain-rule work to the tensor-core kernel only once this is on
static const bool kAutoUsesTensor = true;

// Plain-rule tensor-core prefill: head dim 64 runs the warp-specialised pipeline, head dim 128 the single-role kernel.
// variant: 0 = that choice, 1 = force the single-role kernel (kept reachable for A/B timing and tests).
static int g_tc_variant = 0;
static int tc_dispatch(const PrefillArgs &a, int o_dtype, int D, cudaStream_t stream) {
    if (D == 64 && g_tc_variant == 0) return prefill_tc_ws_launch(a, o_dtype, stream);
    return prefill_tc_launch(a, o_dtype, D, stream);
}

static inline size_t esize(int dt) { return dt == PGB_BF16 ? 2 : 4; }
static inline bool dtype_ok(int dt) { return dt == PGB_F32 || dt == PGB_BF16; }

}  // namespace pgb

using namespace pgb;

extern "C" {

const char *pgb_status_string(int s) {
    switch (s) {
        case PGB_OK: return "ok";
        case PGB_ERR_NULL_POINTER: return "a required pointer is NULL";
        case PGB_ERR_BAD_SHAPE: return "bad or inconsistent shape";
        case PGB_ERR_UNSUPPORTED_DIM: return "unsupported head dimension or chunk (D must be 64 or 128)";
        case PGB_ERR_MISALIGNED: return "pointer or stride breaks the alignment rule";
        case PGB_ERR_BAD_DTYPE: return "unknown dtype code";
        case PGB_ERR_CUDA: return "CUDA launch failed";
        case PGB_ERR_TOO_LARGE:
            return "size exceeds the documented maximum (for pgb_aspin_delta_prefill_noscratch_fwd: B*H*ceil(T/64) > 2048, the "
                   "built-in 32 MiB scratch; use pgb_aspin_delta_prefill_fwd with your own buffer)";
        default: return "unknown status";
    }
}

const char *pgb_last_cuda_error(void) { return g_err; }

int pgb_abi_version(void) { return 1; }

static int lambda_scan_checked(const float *u, const float *logmag, const float *ang, long long ang_stride_b,
                               long long ang_stride_t, const float *h0r, const float *h0i, float *y, float *hr_out,
                               float *hi_out, float *hi_all, int B, int T, int D, int time_segments, void *stream) {
    if (!u || !logmag || !ang || !y || !hr_out || !hi_out) return PGB_ERR_NULL_POINTER;
    if ((h0r == nullptr) != (h0i == nullptr)) return PGB_ERR_NULL_POINTER;
    if (B <= 0 || T <= 0 || D <= 0 || ang_stride_b < 0 || ang_stride_t < 0) return PGB_ERR_BAD_SHAPE;
    if (time_segments != 0 && (time_segments < 1 || time_segments > 32 || (time_segments & (time_segments - 1))))
        return PGB_ERR_BAD_SHAPE;
    if (!aligned(u, 4) || !aligned(logmag, 4) || !aligned(ang, 4) || !aligned(y, 4)) return PGB_ERR_MISALIGNED;
    return lambda_scan_launch(u, logmag, ang, ang_stride_b, ang_stride_t, h0r, h0i, y, hr_out, hi_out, hi_all, B, T, D,
                              time_segments, (cudaStream_t)stream);
}

int pgb_lambda_scan_fwd_ex(const float *u, const float *logmag, const float *ang, long long ang_stride_b,
                           long long ang_stride_t, const float *h0r, const float *h0i, float *y, float *hr_out,
                           float *hi_out, int B, int T, int D, int time_segments, void *stream) {
    return lambda_scan_checked(u, logmag, ang, ang_stride_b, ang_stride_t, h0r, h0i, y, hr_out, hi_out, nullptr, B, T, D,
                               time_segments, stream);
}

int pgb_lambda_scan_fwd_train(const float *u, const float *logmag, const float *ang, long long ang_stride_b,
                              long long ang_stride_t, const float *h0r, const float *h0i, float *y, float *hi_all, float *hr_out,
                              float *hi_out, int B, int T, int D, void *stream) {
    if (!hi_all) return PGB_ERR_NULL_POINTER;
    return lambda_scan_checked(u, logmag, ang, ang_stride_b, ang_stride_t, h0r, h0i, y, hr_out, hi_out, hi_all, B, T, D, 0, stream);
}

int pgb_lambda_scan_bwd(const float *g, const float *u, const float *logmag, const float *ang, long long ang_stride_b,
                        long long ang_stride_t, const float *hr_all, const float *hi_all, const float *g_last_i, float *du,
                        float *dlogmag, float *dang, float *dh0r, float *dh0i, int B, int T, int D, void *stream) {
    if (!g || !u || !logmag || !ang || !hr_all || !hi_all || !du || !dlogmag || !dang) return PGB_ERR_NULL_POINTER;
    if ((dh0r == nullptr) != (dh0i == nullptr)) return PGB_ERR_NULL_POINTER;
    if (B <= 0 || T <= 0 || D <= 0 || ang_stride_b < 0 || ang_stride_t < 0) return PGB_ERR_BAD_SHAPE;
    return lambda_scan_bwd_launch(g, u, logmag, ang, ang_stride_b, ang_stride_t, hr_all, hi_all, g_last_i, du, dlogmag, dang, dh0r,
                                  dh0i, B, T, D, (cudaStream_t)stream);
}

int pgb_lambda_scan_time_segments(int B, int T, int D, int sm_count) {
    if (B <= 0 || T <= 0 || D <= 0 || sm_count <= 0) return 0;
    return lambda_scan_pick_ts(B, T, D, (D % 4 == 0) ? 4 : 1, sm_count, 0);
}

int pgb_aspin_prep_bwd_tiles(int T) { return T > 0 ? prep_bwd_tiles(T) : 0; }

int pgb_aspin_prep_bwd(const void *qp, const void *kp, const void *vp, int in_dtype, long long in_stride_b, long long in_stride_t,
                       long long in_stride_h, const void *gate, long long gate_stride_b, long long gate_stride_t, const float *theta,
                       const long long *pos, const void *dq, const void *dk, const void *dv, int grad_dtype, void *dqp, void *dkp,
                       void *dvp, float *dgate, float *dtheta_partial, int B, int T, int H, int D, void *stream) {
    if (!qp || !kp || !vp || !theta || !pos || !dq || !dk || !dv || !dqp || !dkp || !dvp || !dtheta_partial) return PGB_ERR_NULL_POINTER;
    if (gate && !dgate) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(in_dtype) || !dtype_ok(grad_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || T <= 0 || H <= 0 || (long long)B * H > 65535) return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    return prep_bwd_launch(qp, kp, vp, in_dtype, in_stride_b, in_stride_t, in_stride_h, gate, gate_stride_b, gate_stride_t, theta, pos,
                           dq, dk, dv, grad_dtype, dqp, dkp, dvp, dgate, dtheta_partial, B, T, H, D, (cudaStream_t)stream);
}

int pgb_assoc_out_fwd(const void *q, const void *k, const void *v, int io_dtype, const float *la, const void *sent, void *o, int B,
                      int H, int T, int D, void *stream) {
    if (!q || !k || !v || !la || !sent || !o) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(io_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || T <= 0 || (long long)B * H > 65535) return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    return assoc_out_launch(q, k, v, io_dtype, la, sent, o, B * H, T, D, (cudaStream_t)stream);
}

int pgb_prefix_scan_fwd(const void *k, const void *v, int io_dtype, const float *w, const float *a_log, const float *S0, void *sent,
                        float *sfin, int B, int H, int NC, int D, void *stream) {
    if (!k || !v || !w || !a_log || !sent || !sfin) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(io_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || NC <= 0 || (long long)B * H > 65535) return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    return prefix_scan_launch(k, v, io_dtype, w, a_log, S0, sent, sfin, B * H, NC, D, (cudaStream_t)stream);
}

int pgb_assoc_out_bwd(const void *q, const void *k, const void *v, int io_dtype, const float *la, const void *sent, const void *dout,
                      float *dq, float *dk, float *dv, float *dla, float *dsent, int B, int H, int T, int D, void *stream) {
    if (!q || !k || !v || !la || !sent || !dout || !dq || !dk || !dv || !dla || !dsent) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(io_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || T <= 0 || (long long)B * H > 65535) return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    return assoc_out_bwd_launch(q, k, v, io_dtype, la, sent, dout, dq, dk, dv, dla, dsent, B * H, T, D, (cudaStream_t)stream);
}

int pgb_prefix_scan_bwd(const void *k, const void *v, int io_dtype, const float *w, const float *a_log, const void *sent,
                        const float *dsent, const float *dsfin, float *dk, float *dv, float *dw, float *da_log, float *dS0, int B, int H,
                        int NC, int D, void *stream) {
    if (!k || !v || !w || !a_log || !sent || !dk || !dv || !dw || !da_log) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(io_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || NC <= 0) return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    return prefix_scan_bwd_launch(k, v, io_dtype, w, a_log, sent, dsent, dsfin, dk, dv, dw, da_log, dS0, B * H, NC, D, (cudaStream_t)stream);
}

int pgb_delta_inv_bwd(const void *k, int io_dtype, const float *la, const float *beta, const void *X, const float *dX, float *dk, float *dla,
                      float *dbeta, int B, int H, int T, int D, void *stream) {
    if (!k || !la || !beta || !X || !dX || !dk || !dla || !dbeta) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(io_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || T <= 0 || (long long)B * H > 65535) return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    return delta_inv_bwd_launch(k, io_dtype, la, beta, X, dX, dk, dla, dbeta, B * H, T, D, (cudaStream_t)stream);
}

int pgb_delta_loop_bwd(const void *k, const void *v, int io_dtype, const float *la, const float *beta, const void *X, const void *sent,
                       const float *dW, const float *dsent, const float *dsfin, float *dk_part, float *dv, float *dla_part,
                       float *dbeta_part, float *dX_part, float *dS0, int B, int H, int T, int D, void *stream) {
    if (!k || !v || !la || !beta || !X || !sent || !dk_part || !dv || !dla_part || !dbeta_part || !dX_part) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(io_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || T <= 0 || (long long)B * H > 65535) return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    return delta_loop_bwd_launch(k, v, io_dtype, la, beta, X, sent, dW, dsent, dsfin, dk_part, dv, dla_part, dbeta_part, dX_part, dS0, B * H, T,
                                 D, (cudaStream_t)stream);
}

int pgb_delta_inv_fwd(const void *k, const float *la, const float *beta, void *X, int B, int H, int T, int D, void *stream) {
    if (!k || !la || !beta || !X) return PGB_ERR_NULL_POINTER;
    if (B <= 0 || H <= 0 || T <= 0) return PGB_ERR_BAD_SHAPE;
    if ((long long)B * H > 65535 || (T + 63) / 64 > 65535) return PGB_ERR_TOO_LARGE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    if (!aligned(k, 16) || !aligned(X, 16)) return PGB_ERR_MISALIGNED;
    return delta_inv_launch(k, la, beta, X, B * H, T, D, (cudaStream_t)stream);
}

int pgb_delta_loop_fwd(const void *k, const void *v, int io_dtype, const float *la, const float *beta, const void *X, const float *S0,
                       void *W, void *sent, float *sfin, int B, int H, int T, int D, void *stream) {
    if (!k || !v || !la || !beta || !X || !W || !sent || !sfin) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(io_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || T <= 0 || (long long)B * H > 65535) return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    return delta_loop_launch(k, v, io_dtype, la, beta, X, S0, W, sent, sfin, B * H, T, D, (cudaStream_t)stream);
}

int pgb_key_topk_mask(void *kp, int dtype, long long stride_b, long long stride_t, long long stride_h, int B, int T, int H, int D,
                      int topk, void *stream) {
    if (!kp) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || T <= 0 || H <= 0 || topk < 1 || topk > D) return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    return key_topk_launch(kp, dtype, stride_b, stride_t, stride_h, B, T, H, D, topk, (cudaStream_t)stream);
}

int pgb_short_conv_fwd(const void *x, int dtype, long long stride_b, long long stride_t, const void *w, const void *cache_in, void *y,
                       void *cache_out, int B, int T, int C, int K, void *stream) {
    if (!x || !w || !y || !cache_out) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || T <= 0 || C <= 0 || K < 2 || K > 64 || cache_in == cache_out) return PGB_ERR_BAD_SHAPE;
    return short_conv_launch(x, dtype, stride_b, stride_t, w, cache_in, y, cache_out, B, T, C, K, (cudaStream_t)stream);
}

int pgb_lambda_scan_fwd(const float *u, const float *logmag, const float *ang, long long ang_stride_b,
                        long long ang_stride_t, const float *h0r, const float *h0i, float *y, float *hr_out,
                        float *hi_out, int B, int T, int D, void *stream) {
    return pgb_lambda_scan_fwd_ex(u, logmag, ang, ang_stride_b, ang_stride_t, h0r, h0i, y, hr_out, hi_out, B, T, D, 0,
                                  stream);
}

int pgb_aspin_prep_fwd(const void *qp, const void *kp, const void *vp, int in_dtype, long long in_stride_b,
                       long long in_stride_t, long long in_stride_h, const void *gate, long long gate_stride_b,
                       long long gate_stride_t, const float *theta, const long long *pos, void *q, void *k, void *v,
                       int out_dtype, int B, int T, int H, int D, void *stream) {
    if (!qp || !kp || !vp || !theta || !pos || !q || !k || !v) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(in_dtype) || !dtype_ok(out_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || T <= 0 || H <= 0) return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    const int per = D / 32;                                           // channels a lane moves in one access
    const size_t ia = per * esize(in_dtype), oa = per * esize(out_dtype);
    if (!aligned(qp, ia) || !aligned(kp, ia) || !aligned(vp, ia) || !aligned(q, oa) || !aligned(k, oa) || !aligned(v, oa))
        return PGB_ERR_MISALIGNED;
    if (in_stride_b % per || in_stride_t % per || in_stride_h % per) return PGB_ERR_MISALIGNED;
    return prep_launch(qp, kp, vp, in_dtype, in_stride_b, in_stride_t, in_stride_h, gate, gate_stride_b, gate_stride_t,
                       theta, pos, q, k, v, out_dtype, B, T, H, D, (cudaStream_t)stream);
}

int pgb_aspin_prefill_fwd(const void *q, const void *k, const void *v, int io_dtype, const float *la, const float *beta,
                          const float *S0, const float *theta, const float *shift_dev, float shift_host, void *o,
                          int o_dtype, float *S_out, void *sent, int B, int H, int T, int D, int precision, void *stream) {
    if (!q || !k || !v || !la || !o || !S_out) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(io_dtype) || !dtype_ok(o_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || T <= 0 || (long long)B * H > 0x7fffffffLL) return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    if (precision < PGB_PREFILL_AUTO || precision > PGB_PREFILL_TENSOR) return PGB_ERR_BAD_SHAPE;
    if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(o, 16) || !aligned(S_out, 16) ||
        (S0 && !aligned(S0, 16)) || (sent && !aligned(sent, 16)))
        return PGB_ERR_MISALIGNED;
    PrefillArgs a{q, k, v, la, beta, S0, o, S_out, (__nv_bfloat16 *)sent, theta, shift_dev, shift_host, B, H, T};
    const bool tc_ok = prefill_tc_supported(io_dtype, D, beta != nullptr);
    if (precision == PGB_PREFILL_TENSOR && !tc_ok) return PGB_ERR_UNSUPPORTED_DIM;
    if (precision == PGB_PREFILL_TENSOR || (precision == PGB_PREFILL_AUTO && tc_ok && kAutoUsesTensor))
        return tc_dispatch(a, o_dtype, D, (cudaStream_t)stream);
    return prefill_fp32_launch(a, io_dtype, o_dtype, D, (cudaStream_t)stream);
}

int pgb_aspin_prefill_fused_fwd(const void *q, const void *k, const void *v, const void *decay_logits,
                                long long decay_stride_b, long long decay_stride_t, const float *decay_A, const float *S0,
                                const float *theta, const float *shift_dev, float shift_host, const float *rms_weight,
                                float rms_eps, void *o, int o_dtype, float *S_out, void *sent, int B, int H, int T, int D,
                                void *stream) {
    if (!q || !k || !v || !decay_logits || !decay_A || !o || !S_out) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(o_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || T <= 0 || (long long)B * H > 0x7fffffffLL || decay_stride_b < 0 || decay_stride_t < H)
        return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(o, 16) || !aligned(S_out, 16) ||
        (S0 && !aligned(S0, 16)) || (sent && !aligned(sent, 16)) || !aligned(decay_logits, 2))
        return PGB_ERR_MISALIGNED;
    PrefillArgs a{q, k, v, nullptr, nullptr, S0, o, S_out, (__nv_bfloat16 *)sent, theta, shift_dev, shift_host, B, H, T};
    a.la_raw = decay_logits; a.la_sb = decay_stride_b; a.la_st = decay_stride_t; a.decay_A = decay_A;
    a.rms_w = rms_weight; a.rms_eps = rms_eps; a.o_token_major = 1;
    return tc_dispatch(a, o_dtype, D, (cudaStream_t)stream);
}

int pgb_aspin_layer_prefill_fwd(const void *qp, const void *kp, const void *vp, long long in_stride_b, long long in_stride_t,
                                const void *gate_logits, const void *decay_logits, long long aux_stride_b,
                                long long aux_stride_t, const float *decay_A, const float *rot_table, int rot_T,
                                const float *S0, const float *theta, const float *shift_dev, float shift_host,
                                const float *rms_weight, float rms_eps, void *o, int o_dtype, float *S_out, void *sent,
                                int B, int H, int T, int D, void *stream) {
    if (!qp || !kp || !vp || !decay_logits || !decay_A || !rot_table || !o || !S_out) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(o_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || T <= 0 || (long long)B * H > 0x7fffffffLL || aux_stride_b < 0 || aux_stride_t < H ||
        in_stride_t < (long long)H * D || in_stride_b < 0 || rot_T < (T + 63) / 64 * 64)
        return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    if (!aligned(qp, 16) || !aligned(kp, 16) || !aligned(vp, 16) || in_stride_b % 8 || in_stride_t % 8 || !aligned(o, 16) ||
        !aligned(S_out, 16) || (S0 && !aligned(S0, 16)) || (sent && !aligned(sent, 16)) || !aligned(rot_table, 16))
        return PGB_ERR_MISALIGNED;
    PrefillArgs a{qp, kp, vp, nullptr, nullptr, S0, o, S_out, (__nv_bfloat16 *)sent, theta, shift_dev, shift_host, B, H, T};
    a.la_raw = decay_logits; a.la_sb = aux_stride_b; a.la_st = aux_stride_t; a.decay_A = decay_A;
    a.rms_w = rms_weight; a.rms_eps = rms_eps; a.o_token_major = 1;
    a.raw = 1; a.raw_sb = in_stride_b; a.raw_st = in_stride_t; a.gate_raw = gate_logits; a.rot = rot_table; a.rot_T = rot_T;
    return tc_dispatch(a, o_dtype, D, (cudaStream_t)stream);
}

int pgb_rot_table_build(const float *theta, float *table, int H, int T, int D, void *stream) {
    if (!theta || !table) return PGB_ERR_NULL_POINTER;
    if (H <= 0 || T <= 0 || D <= 0 || (D & 1)) return PGB_ERR_BAD_SHAPE;
    if (!aligned(table, 16)) return PGB_ERR_MISALIGNED;
    return rot_table_launch(theta, table, H, T, D, (cudaStream_t)stream);
}

int pgb_aspin_delta_prefill_noscratch_fwd(const void *q, const void *k, const void *v, const float *la, const float *beta,
                                          const float *S0, const float *theta, const float *shift_dev, float shift_host,
                                          void *o, int o_dtype, float *S_out, void *sent, int B, int H, int T, int D,
                                          void *stream) {
    if (!q || !k || !v || !la || !beta || !o || !S_out) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(o_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || T <= 0) return PGB_ERR_BAD_SHAPE;
    if ((long long)B * H > 65535 || (T + 63) / 64 > 65535) return PGB_ERR_TOO_LARGE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    if (pgb_aspin_delta_scratch_bytes(B, H, T) > prefill_tc_delta_static_capacity()) return PGB_ERR_TOO_LARGE;
    if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(o, 16) || !aligned(S_out, 16) ||
        (S0 && !aligned(S0, 16)) || (sent && !aligned(sent, 16)))
        return PGB_ERR_MISALIGNED;
    PrefillArgs a{q, k, v, la, beta, S0, o, S_out, (__nv_bfloat16 *)sent, theta, shift_dev, shift_host, B, H, T};
    return prefill_tc_delta_static_launch(a, o_dtype, D, (cudaStream_t)stream);
}

int pgb_decode_embed_ex(const long long *tok, const long long *pos, const void *E, const void *P, void *x, float *row_sums, int B, int d,
                        int vocab, int ctx, void *stream) {
    if (!tok || !pos || !E || !P || !x) return PGB_ERR_NULL_POINTER;
    if (B < 1 || d < 8 || (d % 8) != 0 || vocab < 1 || ctx < 1) return PGB_ERR_BAD_SHAPE;
    if (!aligned(E, 16) || !aligned(P, 16) || !aligned(x, 16) || !aligned(tok, 8) || !aligned(pos, 8) || (row_sums && !aligned(row_sums, 8)))
        return PGB_ERR_MISALIGNED;
    return decode_embed_launch(tok, pos, E, P, x, B, d, vocab, ctx, row_sums, (cudaStream_t)stream);
}

int pgb_decode_embed(const long long *tok, const long long *pos, const void *E, const void *P, void *x, int B, int d, int vocab,
                     int ctx, void *stream) {
    return pgb_decode_embed_ex(tok, pos, E, P, x, nullptr, B, d, vocab, ctx, stream);
}

int pgb_decode_token_wait_selftest(unsigned long long *sync, long long limit_polls, void *stream) {
    if (!sync) return PGB_ERR_NULL_POINTER;
    if (limit_polls < 1 || limit_polls > (1ll << 20)) return PGB_ERR_BAD_SHAPE;          // at most about a second
    if (!aligned(sync, 16)) return PGB_ERR_MISALIGNED;
    return decode_token_wait_selftest_launch(sync, (unsigned)limit_polls, (cudaStream_t)stream);
}

long long pgb_decode_token_work_bytes(int B, int d, int NP, int dff) {
    if (B < 1 || d < 1 || NP < 1 || dff < 1) return 0;
    return (long long)decode_token_work_bytes(B, d, NP, dff);
}

int pgb_decode_token_fwd(const void *layer_table, int L, const void *E, const void *P, const void *final_norm_weight,
                         const void *final_norm_bias, int final_norm_kind, float final_norm_eps, const long long *tok,
                         const long long *pos, const float *shift, void *work, long long work_bytes, float *logits,
                         unsigned long long *sync, int B, int d, int H, int D, int NP, int dff, int V, int ctx, int delta,
                         void *stream) {
    if (!layer_table || !E || !P || !final_norm_weight || !tok || !pos || !shift || !work || !logits || !sync) return PGB_ERR_NULL_POINTER;
    if (final_norm_kind != 1 && final_norm_kind != 2) return PGB_ERR_BAD_SHAPE;
    if (final_norm_kind == 2 && !final_norm_bias) return PGB_ERR_NULL_POINTER;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    if (L < 1 || B < 1 || H < 1 || d != H * D || (dff % 8) != 0 || dff < 8 || (NP % 8) != 0 || NP < 3 * d + 2 * H || V < 1 || ctx < 1)
        return PGB_ERR_BAD_SHAPE;
    if (B > 4 || (long long)4 * (dff > d ? dff : d) * 2 + (long long)L * 144 > 72 * 1024) return PGB_ERR_TOO_LARGE;   // shared memory
    if (work_bytes < pgb_decode_token_work_bytes(B, d, NP, dff)) return PGB_ERR_BAD_SHAPE;
    if (!aligned(layer_table, 8) || !aligned(E, 16) || !aligned(P, 16) || !aligned(final_norm_weight, 16) ||
        (final_norm_bias && !aligned(final_norm_bias, 16)) || !aligned(tok, 8) || !aligned(pos, 8) || !aligned(work, 16) ||
        !aligned(logits, 4) || !aligned(sync, 16))
        return PGB_ERR_MISALIGNED;
    return decode_token_launch(layer_table, L, E, P, final_norm_weight, final_norm_bias, final_norm_kind, final_norm_eps, tok, pos,
                               shift, work, logits, sync, B, d, H, D, NP, dff, V, ctx, delta ? 1 : 0,
                               (cudaStream_t)stream);
}

int pgb_decode_sample(const void *logits, int dtype, float temp, unsigned long long seed, long long *tok, long long *hist,
                      int hist_cols, long long *count, long long *pos, float *shift, unsigned int *ticket, int B, int V, int ctx,
                      void *stream) {
    return pgb_decode_sample_ex(logits, dtype, temp, 0.f, seed, tok, hist, hist_cols, count, pos, shift, ticket, B, V, ctx, stream);
}

int pgb_decode_sample_ex(const void *logits, int dtype, float temp, float min_p, unsigned long long seed, long long *tok,
                         long long *hist, int hist_cols, long long *count, long long *pos, float *shift, unsigned int *ticket,
                         int B, int V, int ctx, void *stream) {
    if (!logits || !tok || !count || !ticket) return PGB_ERR_NULL_POINTER;
    if (dtype != PGB_F32 && dtype != PGB_BF16) return PGB_ERR_BAD_DTYPE;
    if (B < 1 || V < 1 || ctx < 1 || hist_cols < 0 || !(temp >= 0.f) || !(min_p >= 0.f && min_p <= 1.f)) return PGB_ERR_BAD_SHAPE;
    if (!aligned(tok, 8) || !aligned(count, 8) || (hist && !aligned(hist, 8)) || (pos && !aligned(pos, 8)) || !aligned(ticket, 4))
        return PGB_ERR_MISALIGNED;
    return decode_sample_launch(logits, dtype, temp, min_p, seed, tok, hist, hist_cols, count, pos, shift, ticket, B, V, ctx,
                                (cudaStream_t)stream);
}

int pgb_linear_act(const void *x, const void *W, const void *bias, void *y, long long M, int N, int K, int act, void *stream) {
    if (!x || !W || !y) return PGB_ERR_NULL_POINTER;
    if (M < 1 || N < 8 || K < 8 || (N % 8) != 0 || (K % 8) != 0 || act < 0 || act > 1) return PGB_ERR_BAD_SHAPE;
    if (M > 0x7fffffffLL) return PGB_ERR_TOO_LARGE;
    if (!aligned(x, 16) || !aligned(W, 16) || !aligned(y, 16) || (bias && !aligned(bias, 16))) return PGB_ERR_MISALIGNED;
    return linear_gelu_launch(x, W, bias, y, M, N, K, act, (cudaStream_t)stream);
}

int pgb_linear_act_set_variant(int variant) { return linear_gelu_set_variant(variant); }

int pgb_decode_set_variant(int variant) { return decode_set_variant(variant); }

int pgb_batch_linear_ex(const void *x, const void *W, const void *bias, void *y, int B, int N, int K, int act, const float *row_sums_in,
                        int parts_in, const float *c1, const float *c2, int norm_kind, float eps, const void *resid, float *row_sums_out,
                        int flags, void *stream) {
    if (!x || !W || !y) return PGB_ERR_NULL_POINTER;
    if (act < 0 || act > 1 || B < 1 || N < 8 || K < 8 || (N % 8) != 0 || (K % 8) != 0) return PGB_ERR_BAD_SHAPE;
    if (norm_kind < 0 || norm_kind > 2 || parts_in < 0 || (flags & ~PGB_SKINNY_FRESH_CONSTANTS)) return PGB_ERR_BAD_SHAPE;
    if (norm_kind != 0 && (!row_sums_in || !c1 || !c2 || parts_in < 1 || bias)) return PGB_ERR_NULL_POINTER;   // the folded norm's c2 carries the bias
    if (B > 128) return PGB_ERR_TOO_LARGE;                            // the batch is one 128-row tensor-core tile
    if (!aligned(x, 16) || !aligned(W, 16) || !aligned(y, 16) || (bias && !aligned(bias, 16)) || (resid && !aligned(resid, 16)) ||
        (c1 && !aligned(c1, 16)) || (c2 && !aligned(c2, 16)) || (row_sums_in && !aligned(row_sums_in, 8)) ||
        (row_sums_out && !aligned(row_sums_out, 8)))
        return PGB_ERR_MISALIGNED;
    return batch_linear_launch(x, W, bias, y, B, N, K, act, row_sums_in, parts_in, c1, c2, norm_kind, eps, resid, row_sums_out,
                               (flags & PGB_SKINNY_FRESH_CONSTANTS) ? 1 : 0, (cudaStream_t)stream);
}

int pgb_batch_linear(const void *x, const void *W, const void *bias, void *y, int B, int N, int K, int act, void *stream) {
    return pgb_batch_linear_ex(x, W, bias, y, B, N, K, act, nullptr, 0, nullptr, nullptr, 0, 0.f, nullptr, nullptr, 0, stream);
}

int pgb_batch_linear_parts(int N) { return N < 1 ? 0 : batch_linear_parts(N); }

int pgb_skinny_linear_ex(const void *x, const void *delta, const void *norm_weight, const void *norm_bias, int norm_kind, float eps,
                         const void *W, const void *bias, int act, void *y, void *x_out, int B, int K, int N, int flags, void *stream) {
    if (!x || !W || !y) return PGB_ERR_NULL_POINTER;
    if (norm_kind < 0 || norm_kind > 2 || act < 0 || act > 1) return PGB_ERR_BAD_SHAPE;
    if ((norm_kind != 0 && !norm_weight) || (norm_kind == 2 && !norm_bias)) return PGB_ERR_NULL_POINTER;
    if (B < 1 || K < 8 || N < 1 || (K % 8) != 0) return PGB_ERR_BAD_SHAPE;
    if (B > 8 || K > 6144) return PGB_ERR_TOO_LARGE;                 // eight rows of K bf16 in shared memory: 96 KiB
    if (!aligned(x, 16) || !aligned(W, 16) || (delta && !aligned(delta, 16)) || (x_out && !aligned(x_out, 16)) ||
        (norm_weight && !aligned(norm_weight, 16)) || (norm_bias && !aligned(norm_bias, 16)))
        return PGB_ERR_MISALIGNED;
    if (flags & ~PGB_SKINNY_FRESH_CONSTANTS) return PGB_ERR_BAD_SHAPE;
    return skinny_linear_launch(x, delta, norm_weight, norm_bias, norm_kind, eps, W, bias, act, y, x_out, B, K, N,
                                (flags & PGB_SKINNY_FRESH_CONSTANTS) ? 1 : 0, (cudaStream_t)stream);
}

int pgb_skinny_linear(const void *x, const void *delta, const void *norm_weight, const void *norm_bias, int norm_kind, float eps,
                      const void *W, const void *bias, int act, void *y, void *x_out, int B, int K, int N, void *stream) {
    return pgb_skinny_linear_ex(x, delta, norm_weight, norm_bias, norm_kind, eps, W, bias, act, y, x_out, B, K, N, 0, stream);
}

int pgb_add_norm(const void *x, const void *delta, const void *weight, const void *bias, float eps, int kind, void *y, void *z,
                 long long rows, int d, int dtype, void *stream) {
    if (!x || !weight || !z || (kind == 1 && !bias)) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(dtype)) return PGB_ERR_BAD_DTYPE;
    if (kind != 0 && kind != 1) return PGB_ERR_BAD_SHAPE;
    const int n = dtype == PGB_BF16 ? 8 : 4;
    if (rows <= 0 || d <= 0 || d % n) return PGB_ERR_BAD_SHAPE;
    if (d > 32 * 8 * n) return PGB_ERR_TOO_LARGE;
    if (!aligned(x, 16) || !aligned(z, 16) || !aligned(weight, 16) || (delta && !aligned(delta, 16)) || (y && !aligned(y, 16)) ||
        (bias && !aligned(bias, 16)))
        return PGB_ERR_MISALIGNED;
    return add_norm_launch(x, delta, weight, bias, eps, kind, y, z, rows, d, dtype, (cudaStream_t)stream);
}

int pgb_tc_set_variant(int variant) {
    if (variant != 0 && variant != 1) return PGB_ERR_BAD_SHAPE;
    g_tc_variant = variant;
    return PGB_OK;
}

int pgb_tc_wait_selftest(long long limit_cycles, void *stream) {
    if (limit_cycles < 1 || limit_cycles > (1ll << 31)) return PGB_ERR_BAD_SHAPE;      // at most about a second of SM clock
    return tc_wait_selftest_launch(limit_cycles, (cudaStream_t)stream);
}

int pgb_tc_error_flag(int *out_host) {
    if (!out_host) return PGB_ERR_NULL_POINTER;
    int a = 0, b = 0;
    int rc = tc_error_flag(&a);
    if (rc == PGB_OK) rc = tc_delta_error_flag(&b);
    int c = 0;
    if (rc == PGB_OK) rc = tc_ws_error_flag(&c);
    int d = 0;
    if (rc == PGB_OK) rc = linear_gelu_error_flag(&d);
    int e = 0, f = 0;
    if (rc == PGB_OK) rc = decode_token_error_flag(&e);
    if (rc == PGB_OK) rc = batch_linear_error_flag(&f);
    e = e > f ? e : f;
    b = b > c ? b : c;
    b = b > d ? b : d;
    b = b > e ? b : e;
    *out_host = a > b ? a : b;
    return rc;
}

long long pgb_aspin_delta_scratch_bytes(int B, int H, int T) {
    if (B <= 0 || H <= 0 || T <= 0) return 0;
    return (long long)prefill_tc_delta_scratch_bytes(B, H, T);
}

int pgb_aspin_delta_prefill_fwd(const void *q, const void *k, const void *v, const float *la, const float *beta, const float *S0,
                                const float *theta, const float *shift_dev, float shift_host, void *o, int o_dtype,
                                float *S_out, void *sent, void *x_scratch, long long x_scratch_bytes, int B, int H, int T, int D,
                                void *stream) {
    if (!q || !k || !v || !la || !beta || !o || !S_out || !x_scratch) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(o_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || T <= 0) return PGB_ERR_BAD_SHAPE;
    if ((long long)B * H > 65535 || (T + 63) / 64 > 65535) return PGB_ERR_TOO_LARGE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    if (x_scratch_bytes < pgb_aspin_delta_scratch_bytes(B, H, T)) return PGB_ERR_BAD_SHAPE;
    if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(o, 16) || !aligned(S_out, 16) ||
        (S0 && !aligned(S0, 16)) || (sent && !aligned(sent, 16)) || !aligned(x_scratch, 16))
        return PGB_ERR_MISALIGNED;
    PrefillArgs a{q, k, v, la, beta, S0, o, S_out, (__nv_bfloat16 *)sent, theta, shift_dev, shift_host, B, H, T};
    return prefill_tc_delta_launch(a, o_dtype, D, x_scratch, (cudaStream_t)stream);
}

int pgb_rotate_pairs(const void *x, int dtype, const float *theta, const float *pos, void *out, int B, int H, int T, int D,
                     void *stream) {
    if (!x || !theta || !pos || !out) return PGB_ERR_NULL_POINTER;
    if (!dtype_ok(dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || T <= 0 || D <= 0 || (D & 1)) return PGB_ERR_BAD_SHAPE;
    if (!aligned(x, 2 * esize(dtype)) || !aligned(out, 2 * esize(dtype))) return PGB_ERR_MISALIGNED;
    return rotate_launch(x, dtype, theta, pos, out, B, H, T, D, (cudaStream_t)stream);
}

int pgb_aspin_decode_step(const void *qp, const void *kp, const void *vp, int in_dtype, long long in_stride_b,
                          int normalize, const void *gate, long long gate_stride_b, int gate_is_logit, int delta,
                          const void *decay, long long decay_stride_b, const float *decay_A, const float *theta,
                          const float *shift_dev, float shift_host, const float *S_in, float *S_out,
                          const float *rms_weight, float rms_eps, void *o, int out_dtype, long long out_stride_b, int B,
                          int H, int D, void *stream) {
    if (!qp || !kp || !vp || !decay || !theta || !S_in || !S_out || !o) return PGB_ERR_NULL_POINTER;
    if (delta && !gate) return PGB_ERR_NULL_POINTER;                  // the delta rule needs its beta
    if (!dtype_ok(in_dtype) || !dtype_ok(out_dtype)) return PGB_ERR_BAD_DTYPE;
    if (B <= 0 || H <= 0 || (long long)B * H > 0x7fffffffLL) return PGB_ERR_BAD_SHAPE;
    if (D != 64 && D != 128) return PGB_ERR_UNSUPPORTED_DIM;
    if (in_stride_b < (long long)H * D || out_stride_b < (long long)H * D || gate_stride_b < 0 || decay_stride_b < 0)
        return PGB_ERR_BAD_SHAPE;
    if (!aligned(S_in, 16) || !aligned(S_out, 16) || !aligned(qp, esize(in_dtype)) || !aligned(o, esize(out_dtype)))
        return PGB_ERR_MISALIGNED;
    DecodeArgs a{qp, kp, vp, in_stride_b, normalize, gate, gate_stride_b, gate_is_logit, decay, decay_stride_b, decay_A,
                 theta, shift_dev, shift_host, S_in, S_out, rms_weight, rms_eps, o, out_stride_b, B, H};
    return decode_launch(a, in_dtype, out_dtype, D, delta, (cudaStream_t)stream);
}

}  // extern "C"
