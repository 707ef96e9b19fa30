/*
 * pragnosia_b200 -- C ABI of the B200 (sm_100a) carrier kernels.
 *
 * The reference (ladkabiharihai/pragnosia) has no C/FFI boundary of its own: its operator boundary is Python
 * functions and torch custom ops that launch Triton kernels. Each entry point below is what a binding for one of
 * those operators calls; the comment on each names the reference operator it stands in for (path:line inside the
 * reference project).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its name ends in _host. The library never allocates, frees or
 *     synchronises; outputs are caller-allocated; launches go to the given stream (a cudaStream_t passed as void*,
 *     NULL = the legacy default stream), so every call can be captured in a CUDA graph.
 *   - Every function returns a pgb_status (0 = OK). Argument checks happen on the host before anything is
 *     launched, so a bad call never touches the GPU. pgb_status_string() names a code.
 *   - Tensors are row-major and contiguous unless a stride argument says otherwise; strides are in ELEMENTS.
 *   - dtype codes: PGB_F32 = 0, PGB_BF16 = 1. The recurrent state is always fp32, laid out [B][H][dk][dv]
 *     (key axis first), bit-compatible with the reference's carried state (src/assoc.py:512).
 */
#ifndef PRAGNOSIA_B200_H
#define PRAGNOSIA_B200_H

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    PGB_OK = 0,
    PGB_ERR_NULL_POINTER = 1,      /* a required pointer is NULL                                   */
    PGB_ERR_BAD_SHAPE = 2,         /* a size is zero/negative or inconsistent                      */
    PGB_ERR_UNSUPPORTED_DIM = 3,   /* head dimension / chunk the kernels are not built for         */
    PGB_ERR_MISALIGNED = 4,        /* a pointer or stride breaks the kernel's alignment rule       */
    PGB_ERR_BAD_DTYPE = 5,         /* unknown dtype code                                           */
    PGB_ERR_CUDA = 6,              /* the launch itself failed; see pgb_last_cuda_error()          */
    PGB_ERR_TOO_LARGE = 7          /* a size exceeds a documented maximum                          */
} pgb_status;

enum { PGB_F32 = 0, PGB_BF16 = 1 };

/* precision of the chunked prefill: AUTO = tensor cores for bf16 I/O, fp32 FFMA for fp32 I/O */
enum { PGB_PREFILL_AUTO = 0, PGB_PREFILL_FP32 = 1, PGB_PREFILL_TENSOR = 2 };

const char *pgb_status_string(int status);
const char *pgb_last_cuda_error(void);     /* text of the last CUDA error seen by this library (thread-local) */
int pgb_abi_version(void);

/* ---------------------------------------------------------------------------------------------------------
 * Per-token complex recurrence  h_t = lambda_t h_{t-1} + u_t,  lambda_t = exp(logmag_t + i ang_t).
 * Replaces src/scan_kernel.py:144-148 scan_triton (kernel _fwd :25-50); CPU definition src/spin.py:182-215.
 *   u, logmag [B][T][D] fp32.  ang: fp32 with element strides (ang_stride_b, ang_stride_t) and unit stride
 *   over D; strides (0,0) mean one angle per channel (the fspin layer's broadcast, src/spin.py:244).
 *   h0r, h0i [B][D] fp32 or both NULL (zero state).
 *   y [B][T][D] fp32 = Re h_t.  hr_out, hi_out [B][D] fp32 = final state.
 * ------------------------------------------------------------------------------------------------------- */
int pgb_lambda_scan_fwd(const float *u, const float *logmag, const float *ang, long long ang_stride_b,
                        long long ang_stride_t, const float *h0r, const float *h0i, float *y, float *hr_out,
                        float *hi_out, int B, int T, int D, void *stream);
/* Same, with the number of time segments a warp scans in parallel fixed by the caller (a power of two in 1..32;
 * 0 = choose from the shape). 1 is the literal sequential recurrence; used for tuning and by the parity tests. */
int pgb_lambda_scan_fwd_ex(const float *u, const float *logmag, const float *ang, long long ang_stride_b,
                           long long ang_stride_t, const float *h0r, const float *h0i, float *y, float *hr_out,
                           float *hi_out, int B, int T, int D, int time_segments, void *stream);

/* The number of time segments a warp scans in parallel that pgb_lambda_scan_fwd picks for this shape on a GPU with
 * sm_count multiprocessors (host arithmetic only; 0 for a bad shape): more segments when channels are too few to fill the
 * GPU, never more than the sequence has pieces to hand out. No counterpart in the reference. */
int pgb_lambda_scan_time_segments(int B, int T, int D, int sm_count);

/* The same forward pass for a caller that will differentiate through it: additionally stores Im h_t for every token
 * (hi_all [B][T][D] fp32), which the adjoint needs. Replaces _Scan.forward, src/scan_kernel.py:105-119, which saves both
 * components. */
int pgb_lambda_scan_fwd_train(const float *u, const float *logmag, const float *ang, long long ang_stride_b,
                              long long ang_stride_t, const float *h0r, const float *h0i, float *y, float *hi_all,
                              float *hr_out, float *hi_out, int B, int T, int D, void *stream);
/* Adjoint of the recurrence, run backwards in time as a chunked shuffle scan.
 * Replaces src/scan_kernel.py:54-101 _bwd (driven by _Scan.backward :121-140).
 *   g [B][T][D]: gradient on Re h_t (the caller has already added the gradient on the final Re state to g[:, T-1]);
 *   g_last_i [B][D] or NULL: gradient on the final Im state.  u, logmag, ang: the forward inputs; hr_all (= y), hi_all:
 *   the forward outputs of pgb_lambda_scan_fwd_train.
 *   du, dlogmag, dang [B][T][D] fp32 (dang is per token even when ang was one value per channel: the caller sums).
 *   dh0r, dh0i [B][D]: gradient on the entering state, or both NULL. */
int pgb_lambda_scan_bwd(const float *g, const float *u, const float *logmag, const float *ang, long long ang_stride_b,
                        long long ang_stride_t, const float *hr_all, const float *hi_all, const float *g_last_i, float *du,
                        float *dlogmag, float *dang, float *dh0r, float *dh0i, int B, int T, int D, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Fused plumbing before the scan: L2-normalise q, k, v per head, scale k by sigmoid(gate), rotate q and k by
 * pos[t] * theta[h][i] per channel pair, cast, and transpose (B,T,H,D) -> (B,H,T,D).
 * Replaces src/assoc_kernel.py:888-891 prep_kernel (op membrae::assoc_prep :828, kernel _prep_fwd :742-769).
 *   qp, kp, vp: in_dtype, logical shape (B,T,H,D), element strides (in_stride_b, in_stride_t, in_stride_h),
 *   unit stride over D (views into one fused projection are fine).
 *   gate: logits (B,T,H), same in_dtype, element strides (gate_stride_b, gate_stride_t), unit over H; NULL = none.
 *   theta [H][D/2] fp32.  pos [T] int64.   q, k, v out: out_dtype, contiguous (B,H,T,D).   D in {64,128}.
 * ------------------------------------------------------------------------------------------------------- */
int pgb_aspin_prep_fwd(const void *qp, const void *kp, const void *vp, int in_dtype, long long in_stride_b,
                       long long in_stride_t, long long in_stride_h, const void *gate, long long gate_stride_b,
                       long long gate_stride_t, const float *theta, const long long *pos, void *q, void *k,
                       void *v, int out_dtype, int B, int T, int H, int D, void *stream);

/* Gradient of pgb_aspin_prep_fwd. Replaces src/assoc_kernel.py:774-826 _prep_bwd (op membrae::assoc_prep_bwd :850).
 *   qp, kp, vp, gate, theta, pos: the forward inputs, same strides.  dq, dk, dv: grad_dtype, contiguous (B,H,T,D).
 *   dqp, dkp, dvp: in_dtype, contiguous (B,T,H,D).  dgate [B][T][H] fp32 (required when gate is given).
 *   dtheta_partial [B * pgb_aspin_prep_bwd_tiles(T)][H][D/2] fp32: one partial per CTA; theta's gradient is their sum
 *   over the first axis (a fixed summation order, so results repeat bit for bit). */
int pgb_aspin_prep_bwd(const void *qp, const void *kp, const void *vp, int in_dtype, long long in_stride_b, long long in_stride_t,
                       long long in_stride_h, const void *gate, long long gate_stride_b, long long gate_stride_t, const float *theta,
                       const long long *pos, const void *dq, const void *dk, const void *dv, int grad_dtype, void *dqp, void *dkp,
                       void *dvp, float *dgate, float *dtheta_partial, int B, int T, int H, int D, void *stream);
int pgb_aspin_prep_bwd_tiles(int T);

/* ---------------------------------------------------------------------------------------------------------
 * The reference's op-level pieces of the chunked scan as stand-alone operators with its argument lists. The fused
 * prefill above replaces all of them on the product path; these serve code written against the individual ops.
 * Plain fp32 arithmetic; sent / X / W are bf16 as the reference stores them. D in {64,128}; B*H <= 65535.
 *
 * pgb_assoc_out_fwd    replaces membrae::assoc_out (src/assoc_kernel.py:128-138, kernel _fwd_out :49-70):
 *   o = ((q k^T) * dec) v + (q e^L) sent[c] per 64-token chunk.  q, k, v, o [B][H][T][D] io_dtype; la [B][H][T];
 *   sent [B][H][ceil(T/64)][D][D] bf16 (the state entering each chunk).
 * pgb_prefix_scan_fwd  replaces membrae::prefix_scan (:231-244, kernels _chunk_kv :223, _prefix_fwd :189-202):
 *   sent[c] = S;  S = exp(a_log[c]) S + (k w)^T v.  k, v [B][H][NC*64][D] (whole chunks); w [B][H][NC][64];
 *   a_log [B][H][NC]; S0 [B][H][D][D] fp32 or NULL; outputs sent (bf16) and sfin [B][H][D][D] fp32.
 * pgb_delta_inv_fwd    replaces membrae::delta_inv (:658-667, kernels _inv_build :556, _inv_solve :571-622):
 *   X [B][H][ceil(T/64)][64][64] bf16 = (I + beta strictly_lower((k k^T) dec))^-1; k bf16 [B][H][T][D], 16-byte aligned.
 * pgb_delta_loop_fwd   replaces membrae::delta_loop_fwd (:363-378, kernel _delta_loop_fwd :333-360):
 *   per chunk rhs = beta (v - e^L k S), W = X rhs, S = e^{L_C} S + (k w)^T W; outputs W [B][H][T][D] bf16, sent, sfin.
 * ------------------------------------------------------------------------------------------------------- */
int pgb_assoc_out_fwd(const void *q, const void *k, const void *v, int io_dtype, const float *la, const void *sent, void *o, int B,
                      int H, int T, int D, void *stream);
int pgb_prefix_scan_fwd(const void *k, const void *v, int io_dtype, const float *w, const float *a_log, const float *S0, void *sent,
                        float *sfin, int B, int H, int NC, int D, void *stream);
/* Backward of the two plain-rule operators above (src/assoc_kernel.py:75-126 _bwd_chunk, :206-221 _prefix_bwd, wired with
 * register_autograd at :179 and :299). Every gradient is fp32; sums are taken in a fixed order.
 *   pgb_assoc_out_bwd:   dout [B][H][T][D] (io dtype) -> dq, dk, dv [B][H][T][D], dla [B][H][T], dsent [B][H][NC][D][D].
 *   pgb_prefix_scan_bwd: dsent [B][H][NC][D][D] and dsfin [B][H][D][D] (either may be NULL = zero), sent = the forward's
 *                        output -> dk, dv [B][H][NC*64][D], dw [B][H][NC][64], da_log [B][H][NC], dS0 [B][H][D][D] (or NULL). */
int pgb_assoc_out_bwd(const void *q, const void *k, const void *v, int io_dtype, const float *la, const void *sent, const void *dout,
                      float *dq, float *dk, float *dv, float *dla, float *dsent, int B, int H, int T, int D, void *stream);
int pgb_prefix_scan_bwd(const void *k, const void *v, int io_dtype, const float *w, const float *a_log, const void *sent,
                        const float *dsent, const float *dsfin, float *dk, float *dv, float *dw, float *da_log, float *dS0, int B, int H,
                        int NC, int D, void *stream);
/* Backward of the two delta-rule operators below (src/assoc_kernel.py:390-459 _delta_loop_bwd, :626-656 _inv_bwd, wired with
 * register_autograd at :509 and :704). fp32 gradients, fixed summation order.
 *   pgb_delta_inv_bwd:  dX [B][H][NC][64][64] -> dk [B][H][T][D], dla, dbeta [B][H][T].
 *   pgb_delta_loop_bwd: dW [B][H][T][D], dsent [B][H][NC][D][D], dsfin [B][H][D][D] (each may be NULL = zero); sent = the
 *     forward's output. Sums over value columns leave as one part per 64-column slab, P = D / 64, for the caller to add:
 *     dk_part [P][B][H][T][D], dla_part, dbeta_part [P][B][H][T], dX_part [P][B][H][NC][64][64]; dv [B][H][T][D] and
 *     dS0 [B][H][D][D] (or NULL) are complete. */
int pgb_delta_inv_bwd(const void *k, int io_dtype, const float *la, const float *beta, const void *X, const float *dX, float *dk, float *dla,
                      float *dbeta, int B, int H, int T, int D, void *stream);
int pgb_delta_loop_bwd(const void *k, const void *v, int io_dtype, const float *la, const float *beta, const void *X, const void *sent,
                       const float *dW, const float *dsent, const float *dsfin, float *dk_part, float *dv, float *dla_part,
                       float *dbeta_part, float *dX_part, float *dS0, int B, int H, int T, int D, void *stream);
int pgb_delta_inv_fwd(const void *k, const float *la, const float *beta, void *X, int B, int H, int T, int D, void *stream);
int pgb_delta_loop_fwd(const void *k, const void *v, int io_dtype, const float *la, const float *beta, const void *X, const float *S0,
                       void *W, void *sent, float *sfin, int B, int H, int T, int D, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Optional steps of the layer between its projections and the scan.
 * pgb_key_topk_mask  (src/assoc.py:435-439): in place, keep the topk largest-magnitude coordinates of every key row and
 *   zero the rest.  kp: dtype view (B,T,H,D) with element strides (stride_b, stride_t, stride_h), unit over D.
 * pgb_short_conv_fwd (src/assoc.py:361-382 _sconv): depthwise causal convolution over the last K tokens of the
 *   concatenated q|k|v projections.  x: view (B,T,C) with strides (stride_b, stride_t), C = 3d; w [C][K];
 *   cache_in [B][C][K-1] (the previous call's last K-1 inputs) or NULL; y [B][T][C]; cache_out [B][C][K-1] (must not be
 *   cache_in).  y[t] = sum_j w[:, j] x[t + j - (K-1)].
 * ------------------------------------------------------------------------------------------------------- */
int pgb_key_topk_mask(void *kp, int dtype, long long stride_b, long long stride_t, long long stride_h, int B, int T, int H, int D,
                      int topk, void *stream);
int pgb_short_conv_fwd(const void *x, int dtype, long long stride_b, long long stride_t, const void *w, const void *cache_in, void *y,
                       void *cache_out, int B, int T, int C, int K, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Chunked prefill of the associative carrier, plain rule (beta == NULL) or delta rule, one fused pass:
 *   o_t = sum_{s<=t} exp(L_t-L_s) (q_t.k_s) w_s + exp(L_t) q_t S_entering ;  S carried chunk to chunk in fp32.
 * Replaces src/assoc_kernel.py:302-323 assoc_scan_kernel (ops prefix_scan :231, assoc_out :128) and :512-546
 * delta_scan_kernel (ops delta_inv :658, delta_loop_fwd :363, assoc_out); CPU definition src/assoc.py:254-269.
 *   q, k, v [B][H][T][D] io_dtype (already normalised / gated / rotated).  la [B][H][T] fp32 log-decay <= 0.
 *   beta [B][H][T] fp32 or NULL.  S0 [B][H][D][D] fp32 or NULL (zero).
 *   theta [H][D/2] fp32 or NULL.  With theta given, S0's key axis is first rotated back by shift positions (the
 *   rebase of src/assoc.py:399-402); shift = *shift_dev if shift_dev != NULL else shift_host.
 *   o [B][H][T][D] o_dtype (fp32 output with bf16 inputs is allowed).  S_out [B][H][D][D] fp32.
 *   sent: optional [B][H][ceil(T/64)][D][D] bf16, the state ENTERING every 64-token chunk (NULL = not wanted).
 *   D in {64,128}.  precision: PGB_PREFILL_*.
 * ------------------------------------------------------------------------------------------------------- */
int pgb_aspin_prefill_fwd(const void *q, const void *k, const void *v, int io_dtype, const float *la,
                          const float *beta, const float *S0, const float *theta, const float *shift_dev,
                          float shift_host, void *o, int o_dtype, float *S_out, void *sent, int B, int H, int T,
                          int D, int precision, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Delta-rule chunked prefill on the tensor cores (bf16 operands): X = (I + beta strictly_lower(K K^T dec))^-1 for every
 * chunk by a chunk-parallel kernel (exact fp32 substitution), then the walk over chunks with W = X rhs.
 * Replaces src/assoc_kernel.py:512-546 delta_scan_kernel (ops delta_inv :658, delta_loop_fwd :363, assoc_out :128).
 *   Arguments as pgb_aspin_prefill_fwd with io dtype bf16 and beta required, plus
 *   x_scratch: device buffer of at least pgb_aspin_delta_scratch_bytes(B,H,T) bytes, 16-byte aligned, owned by the
 *   caller; its contents after the call are the X matrices (bf16 head and tail per chunk) and may be discarded.
 *   B*H and ceil(T/64) must each be at most 65535.
 * ------------------------------------------------------------------------------------------------------- */
int pgb_aspin_delta_prefill_fwd(const void *q, const void *k, const void *v, const float *la, const float *beta,
                                const float *S0, const float *theta, const float *shift_dev, float shift_host, void *o,
                                int o_dtype, float *S_out, void *sent, void *x_scratch, long long x_scratch_bytes, int B,
                                int H, int T, int D, void *stream);
long long pgb_aspin_delta_scratch_bytes(int B, int H, int T);

/* ---------------------------------------------------------------------------------------------------------
 * pgb_aspin_delta_prefill_fwd without the x_scratch argument. It has no counterpart in the reference.
 * It exists for callers that cannot get device memory at the moment they call: an operator hook inside a serving
 * runtime that owns every byte of device memory and hands the hook only tensor pointers and a stream (allocating there
 * would synchronise the device, can fail in the middle of a request, and is usually forbidden outright), or code that
 * is being recorded into a CUDA graph, where the ordinary allocation calls are not allowed. For them the chunk inverses
 * go to a fixed 32 MiB array that is part of the library's device image, so this call never allocates or frees.
 *   Limit: B * H * ceil(T/64) <= 2048 (16 KiB per (sequence-head, chunk)); larger problems return PGB_ERR_TOO_LARGE and
 *   must use pgb_aspin_delta_prefill_fwd. Every GPU that loads the library keeps those 32 MiB reserved until the process
 *   exits, whether or not this entry point is ever used.
 *   The first call on each device looks up the array's device address (a host-side query, cached afterwards). Make that
 *   first call outside any stream capture.
 *   All calls on a device share the one array and it keeps whatever the previous call left there (nothing in it has to
 *   start at zero: each call overwrites the part it reads). Two calls whose kernels can run at the same time on one
 *   device -- different streams, or different host threads -- would overwrite each other's inverses: serialise them.
 *   Inputs, outputs, dtype and dimension rules are exactly those of pgb_aspin_delta_prefill_fwd.
 * ------------------------------------------------------------------------------------------------------- */
int pgb_aspin_delta_prefill_noscratch_fwd(const void *q, const void *k, const void *v, const float *la, const float *beta,
                                          const float *S0, const float *theta, const float *shift_dev, float shift_host,
                                          void *o, int o_dtype, float *S_out, void *sent, int B, int H, int T, int D,
                                          void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * The same chunked prefill (plain rule, bf16 operands, tensor cores) with the layer's neighbouring elementwise steps
 * fused in, so a layer's prefill is: projection GEMM -> prep -> THIS -> output GEMM.
 * Replaces, in src/assoc.py AssocCarrier.forward: the decay gate (:355-356, :467), the scan (:498-499), the per-head
 * RMS norm and the (B,H,T,D)->(B,T,H*D) transpose (:505).
 *   q, k, v [B][H][T][D] bf16 as produced by pgb_aspin_prep_fwd.
 *   decay_logits: bf16 view (B,T,H) with element strides (decay_stride_b, decay_stride_t), unit over H: the output of
 *   the decay gate's linear layer; log alpha = -softplus(logit) * exp(decay_A[h]).  decay_A [H] fp32.
 *   S0, theta, shift_dev, shift_host, S_out, sent: as in pgb_aspin_prefill_fwd.
 *   rms_weight [D] fp32, rms_eps: o <- o * rsqrt(mean_D(o^2) + eps) * w per (token, head); NULL = no norm.
 *   o: o_dtype, TOKEN-major [B][T][H][D].     D in {64,128}.
 * ------------------------------------------------------------------------------------------------------- */
int pgb_aspin_prefill_fused_fwd(const void *q, const void *k, const void *v, const void *decay_logits,
                                long long decay_stride_b, long long decay_stride_t, const float *decay_A,
                                const float *S0, const float *theta, const float *shift_dev, float shift_host,
                                const float *rms_weight, float rms_eps, void *o, int o_dtype, float *S_out,
                                void *sent, int B, int H, int T, int D, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * A layer's whole prefill between its two GEMMs in ONE kernel (plain rule, bf16, tensor cores): the plumbing of
 * pgb_aspin_prep_fwd is done in shared memory on the tiles the TMA brings in, then pgb_aspin_prefill_fused_fwd.
 * Replaces src/assoc.py:440-451 (prep_kernel), :355-356/:467 (decay gate), :498-499 (scan), :505 (norm, transpose).
 *   qp, kp, vp: bf16 views (B,T,H*D) of the projection GEMM's output with element strides (in_stride_b, in_stride_t),
 *   unit stride inside a row; 16-byte aligned, strides multiples of 8.
 *   gate_logits (write gate, may be NULL) and decay_logits: bf16 views (B,T,H) with strides (aux_stride_b, aux_stride_t).
 *   rot_table: [H][rot_T][D/2] pairs (cos, sin) of position * theta from pgb_rot_table_build; rot_T >= T rounded up to
 *   a multiple of 64 (whole chunks of rows are bulk-copied).
 *   Everything else as in pgb_aspin_prefill_fused_fwd.  o is token-major [B][T][H][D].
 * ------------------------------------------------------------------------------------------------------- */
int pgb_aspin_layer_prefill_fwd(const void *qp, const void *kp, const void *vp, long long in_stride_b,
                                long long in_stride_t, const void *gate_logits, const void *decay_logits,
                                long long aux_stride_b, long long aux_stride_t, const float *decay_A,
                                const float *rot_table, int rot_T, const float *S0, const float *theta,
                                const float *shift_dev, float shift_host, const float *rms_weight, float rms_eps,
                                void *o, int o_dtype, float *S_out, void *sent, int B, int H, int T, int D,
                                void *stream);

/* table[h][t][i] = (cos, sin)(t * theta[h][i]), t in [0,T): the rotation phases of one layer (src/assoc.py:34-39 with
 * positions 0..T-1), built once per layer and reused by every pgb_aspin_layer_prefill_fwd call.
 *   theta [H][D/2] fp32;  table [H][T][D/2][2] fp32. */
int pgb_rot_table_build(const float *theta, float *table, int H, int T, int D, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Residual add fused with the norm that follows it:  y = x + delta ;  z = norm(y) * weight (+ bias).
 * Replaces, across the layer stack, the residual adds of src/assoc.py:511 and src/model.py:560 together with the norms
 * at src/assoc.py:388, src/model.py:560 (MLP.n) and the final norm (:863).
 *   x, delta, y, z: [rows][d], dtype (fp32 or bf16), contiguous.  delta may be NULL (norm only; y is then unused).
 *   y may be NULL (the sum is not kept).  weight, bias: [d], same dtype; bias only for kind 1.
 *   kind 0: RMS norm (eps inside the square root, as torch.nn.RMSNorm);  kind 1: layer norm.
 *   d must be a multiple of 8 (bf16) / 4 (fp32) and at most 2048 (bf16) / 1024 (fp32).
 * ------------------------------------------------------------------------------------------------------- */
int pgb_add_norm(const void *x, const void *delta, const void *weight, const void *bias, float eps, int kind, void *y,
                 void *z, long long rows, int d, int dtype, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * Linear layer for a few rows (decode at batch <= 8) with the residual add and norm before it and the activation
 * after it in the same launch:   s = x + delta ;  z = norm(s) ;  y = act(z W^T + bias).
 * Replaces, for T = 1 and small batch, the F.linear / LayerNorm / GELU calls of src/assoc.py:384-512 (projections,
 * output projection) and src/model.py:552-560 (MLP), and the tied head at src/model.py:863. bf16 only, fp32 accumulate;
 * s, z and the pre-activation are rounded to bf16 where the separate ops round them.
 *   x, delta [B][K]; delta may be NULL.  x_out [B][K] or NULL: receives s (must not alias x or delta).
 *   norm_kind 0: none, 1: RMS norm (norm_weight [K]), 2: layer norm (norm_weight, norm_bias [K]).
 *   W [N][K] (torch.nn.Linear layout), bias [N] or NULL;  act 0: none, 1: GELU (erf);  y [B][N].
 *   B <= 8, K a multiple of 8 and at most 6144; x, delta, x_out, W, norm vectors 16-byte aligned.
 * ------------------------------------------------------------------------------------------------------- */
int pgb_skinny_linear(const void *x, const void *delta, const void *norm_weight, const void *norm_bias, int norm_kind, float eps,
                      const void *W, const void *bias, int act, void *y, void *x_out, int B, int K, int N, void *stream);
/* The kernel is launched as a programmatic dependent of whatever precedes it on the stream and requests W, the norm
 * vectors and the bias BEFORE it waits for that predecessor: they must already be complete when the preceding kernel
 * was launched (model weights are). If the preceding kernel on the stream may have written any of them (a dtype cast, a
 * freshly concatenated weight), pass PGB_SKINNY_FRESH_CONSTANTS in flags and every such load moves behind the wait. */
enum { PGB_SKINNY_FRESH_CONSTANTS = 1 };
int pgb_skinny_linear_ex(const void *x, const void *delta, const void *norm_weight, const void *norm_bias, int norm_kind, float eps,
                         const void *W, const void *bias, int act, void *y, void *x_out, int B, int K, int N, int flags,
                         void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * The two ends of a decode step as single launches, so that a token is a fixed kernel sequence with no work on the host
 * (the reference samples on the host and syncs per token: src/bench.py:79-86, 193-239; embedding: src/model.py:859).
 *
 * pgb_decode_embed:  x[b][:] = E[tok[b]][:] + P[pos[0]][:]   (bf16; E [vocab][d], P [ctx][d], x [B][d]; tok [B] and pos [1]
 *   are int64 on the device; ids outside the tables are clamped).
 *
 * pgb_decode_sample: tok[b] ~ softmax(logits[b] / temp) (temp = 0: argmax) by Gumbel-max with a counter-based uniform
 *   mixed from (seed, count[0], b, v); logits [B][V] fp32 or bf16. Writes hist[b][count[0]] when hist != NULL and
 *   count[0] < hist_cols. The window position and the rebase shift belong to the token being fed to the model, so when
 *   count[0] > 0 the kernel first advances them for the previous token: pos[0] = (pos[0] + 1) mod ctx, shift[0] = 1
 *   (either may be NULL). Once every row has drawn, count[0] += 1. ticket is one zero-initialised uint32 the kernel uses
 *   and leaves at zero.
 * ------------------------------------------------------------------------------------------------------- */
int pgb_decode_embed(const long long *tok, const long long *pos, const void *E, const void *P, void *x, int B, int d, int vocab,
                     int ctx, void *stream);
int pgb_decode_sample(const void *logits, int dtype, float temp, unsigned long long seed, long long *tok, long long *hist,
                      int hist_cols, long long *count, long long *pos, float *shift, unsigned int *ticket, int B, int V, int ctx,
                      void *stream);
/* The same draw with min-p filtering (src/bench.py:38, 79-86 MEMBRAE_MIN_P): ids whose probability is below min_p times the
 * most likely id's are dropped before the draw; min_p in [0, 1], 0 = off. */
int pgb_decode_sample_ex(const void *logits, int dtype, float temp, float min_p, unsigned long long seed, long long *tok,
                         long long *hist, int hist_cols, long long *count, long long *pos, float *shift, unsigned int *ticket,
                         int B, int V, int ctx, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * y = act(x W^T + bias) for a batch of decode rows (one token per sequence, up to 128 sequences) as one tcgen05 launch: the
 * rows of x are one 128-row tile, a CTA owns 16 / 32 / 64 rows of W and streams them once by TMA (requested before the wait
 * on the kernel that produces x), bias and erf-GELU on the accumulator. Replaces, for T = 1 and batches too large for
 * pgb_skinny_linear, the F.linear (+ GELU) calls of src/assoc.py:384-512 and src/model.py:552-560. bf16, fp32 accumulate;
 * the pre-activation is rounded to bf16 first, as the separate Linear would.
 *   x [B][K], W [N][K] (torch.nn.Linear layout), bias [N] or NULL, y [B][N]; act 0: none, 1: GELU (erf).
 *   B <= 128; N and K multiples of 8; x, W, y, bias 16-byte aligned. Bounded waits (pgb_tc_error_flag).
 * ------------------------------------------------------------------------------------------------------- */
int pgb_batch_linear(const void *x, const void *W, const void *bias, void *y, int B, int N, int K, int act, void *stream);
/* The same launch taking over the add + norm kernels on either side of the layer (every extra argument optional):
 *   folded norm (norm_kind 1 RMS / 2 layer norm): x is the raw residual stream and W already carries the norm's weight,
 *     W'[n][k] = W[n][k] w[k]; with c1[n] = sum_k W'[n][k] and c2[n] = sum_k beta[k] W[n][k] + b[n] (fp32 [N], bias must be
 *     NULL) the epilogue forms r (acc - mu c1) + c2 from the row's mean mu and r = 1 / sqrt(var + eps), both taken from the
 *     partial row sums (sum, sum of squares) row_sums_in [parts_in][B][2] that the kernel producing x left behind;
 *   residual (resid [B][N] bf16): y = resid + act(x W^T + b) with the separate ops' roundings, i.e. the new residual
 *     stream, and row_sums_out [pgb_batch_linear_parts(N)][B][2] receives each CTA's partial row sums of y.
 * pgb_decode_embed_ex writes the row sums of the embedding (one part) for the first layer's folded norm.
 * The kernel requests W, bias, c1 and c2 before it waits for the kernel ahead of it on the stream: they must be complete
 * before that kernel was launched, or flags must carry PGB_SKINNY_FRESH_CONSTANTS (then nothing is read before the wait). */
int pgb_batch_linear_ex(const void *x, const void *W, const void *bias, void *y, int B, int N, int K, int act, const float *row_sums_in,
                        int parts_in, const float *c1, const float *c2, int norm_kind, float eps, const void *resid, float *row_sums_out,
                        int flags, void *stream);
int pgb_batch_linear_parts(int N);
int pgb_decode_embed_ex(const long long *tok, const long long *pos, const void *E, const void *P, void *x, float *row_sums, int B, int d,
                        int vocab, int ctx, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * One decode step of the whole language model -- embedding, every layer (norm + fused projection, recurrent state step,
 * output projection, norm + MLP), final norm, tied head -- as ONE cooperative launch of one CTA per SM, for 1..4 sequences
 * in bf16 with fp32 states updated in place. Replaces, for one token, the layer loop of src/model.py:859-884 over
 * src/assoc.py:384-512 (T = 1) and src/model.py:552-560 that the reference replays as a CUDA graph of about a thousand
 * launches (src/bench.py:242-317). Arithmetic and roundings are those of pgb_decode_embed, pgb_skinny_linear and
 * pgb_aspin_decode_step chained five launches a layer.
 *
 *   layer_table  [L][18] 64-bit words on the device, per layer: pointers Wc [NP][d] (rows q | k | v | decay | gate, padded),
 *                bc [NP], ln weight, ln bias (0 for RMS), Wo' [d][d] (output weight times sigmoid(gate)), MLP norm weight,
 *                MLP norm bias (0 for RMS), Wa [dff][d], ba [dff], Wb [d][dff], bb [d] (all bf16), theta [H][D/2], A [H],
 *                per-head RMS weight [D] (fp32), S [B][H][D][D] (fp32, in place); then word 15 = the two norm kinds as
 *                int32 (low: layer norm in front of the mixer, high: in front of the MLP; 1 = RMS, 2 = layer norm), word 16 =
 *                their epsilons as fp32 (same order), word 17 = the per-head RMS norm's epsilon as fp32 in its low half.
 *   E [V][d], P [ctx][d] bf16 (E is also the head); tok [B], pos [1] int64 and shift [1] fp32 on the device as for
 *   pgb_decode_embed / pgb_aspin_decode_step (shift_dev); logits [B][V] fp32 out (bf16-rounded values).
 *   work: pgb_decode_token_work_bytes(B, d, NP, dff) bytes of scratch, 16-byte aligned.
 *   sync: two 64-bit words, zero before the first launch and then left to the kernel (the grid barrier's counters); one
 *         pair per stream of launches, never shared by two launches in flight.
 *   B <= 4, D in {64, 128}, d = H * D, NP >= 3d + 2H, NP and dff multiples of 8; delta: 0 plain rule, 1 delta rule.
 * Every barrier wait is bounded; a wait that runs out makes the whole grid return and pgb_tc_error_flag reads 81 (zero the
 * sync words before the next launch).
 * ------------------------------------------------------------------------------------------------------- */
long long pgb_decode_token_work_bytes(int B, int d, int NP, int dff);
/* Self-test of that kernel's failure path: one CTA arrives at a grid barrier nobody else will reach; after `limit_polls`
 * polls (1 .. 2^20) its wait gives up, pgb_tc_error_flag reads 81 and the kernel returns normally -- nothing faults, traps
 * or hangs. sync: two 64-bit words holding zero (zero them again afterwards). No counterpart in the reference. */
int pgb_decode_token_wait_selftest(unsigned long long *sync, long long limit_polls, void *stream);
int pgb_decode_token_fwd(const void *layer_table, int L, const void *E, const void *P, const void *final_norm_weight,
                         const void *final_norm_bias, int final_norm_kind, float final_norm_eps, const long long *tok,
                         const long long *pos, const float *shift, void *work, long long work_bytes, float *logits,
                         unsigned long long *sync, int B, int d, int H, int D, int NP, int dff, int V, int ctx, int delta,
                         void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * y = act(x W^T + bias) as one tcgen05 GEMM with the bias and the activation applied on the accumulator in the epilogue.
 * Replaces the Linear(d, 4d) + GELU pair of the MLP block (src/model.py:552-560) in the prefill pass, where the separate
 * activation is a second pass over the hidden tensor. bf16, fp32 accumulate; the pre-activation is rounded to bf16 first,
 * as the separate Linear would.
 *   x [M][K], W [N][K] (torch.nn.Linear layout), bias [N] or NULL, y [M][N]; act 0: none, 1: GELU (erf).
 *   N and K multiples of 8; x, W, y, bias 16-byte aligned. Bounded waits as in the prefill kernels (pgb_tc_error_flag).
 * ------------------------------------------------------------------------------------------------------- */
int pgb_linear_act(const void *x, const void *W, const void *bias, void *y, long long M, int N, int K, int act, void *stream);

/* Which kernel pgb_linear_act uses. Bit 0: 0 (default) = one CTA per 128-row tile; 1 = pairs of SMs share one 256-row tile
 * (tcgen05.mma.cta_group::2: each CTA of a two-CTA cluster loads half of either operand, no multicast) whenever the
 * problem has more than 128 rows. Bits 1-2: the tile's width, 0 or 1 = 256 columns (default), 2 = 192. variant in 0..5.
 * Every choice gives the same results to the bit (and, timed at the MLP's shape, the same speed to within a few percent).
 * The pair is faster without an activation and slower with the GELU, whose epilogue then sets the pace. Process-wide; for
 * A/B timing and tests. No counterpart in the reference. */
int pgb_linear_act_set_variant(int variant);

/* Health check of the tensor-core prefill kernel: every wait inside it is bounded, and a wait that runs out sets a
 * device-side flag instead of hanging. This reads the flag into *out_host (0 = no wait ever ran out) and clears it.
 * Unlike every other entry point it SYNCHRONISES the device. No counterpart in the reference. */
int pgb_tc_error_flag(int *out_host);

/* Self-test of that failure path: launches one thread that waits, with the kernels' bounded loop, on an mbarrier nothing
 * arrives at. After `limit_cycles` of the SM clock (1 .. 2^31) the wait gives up, the flag reads 99 and the kernel returns
 * normally -- the context stays usable. Nothing faults, traps or hangs. No counterpart in the reference. */
int pgb_tc_wait_selftest(long long limit_cycles, void *stream);

/* Which plain-rule tensor-core kernel head dim 64 uses: 0 (default) = the warp-specialised pipeline, 1 = the single-role
 * kernel that head dim 128 always uses. Process-wide; for A/B timing and tests. No counterpart in the reference. */
int pgb_tc_set_variant(int variant);

/* ---------------------------------------------------------------------------------------------------------
 * Rotation of channel pairs (2i, 2i+1) of x (B,H,T,D) by pos[t] * theta[h][i]; any even D.
 * Replaces src/assoc.py:34-39 rotate.   x, out: dtype, contiguous.  theta [H][D/2] fp32.  pos [T] fp32.
 * ------------------------------------------------------------------------------------------------------- */
int pgb_rotate_pairs(const void *x, int dtype, const float *theta, const float *pos, void *out, int B, int H, int T,
                     int D, void *stream);

/* ---------------------------------------------------------------------------------------------------------
 * One recurrent decode step per (sequence, head), fully fused: normalise q,k,v; write gate or beta; rebase
 * rotation of the state's key axis by -shift*theta; decay; rank-1 write (plain or delta); read; optional per-head
 * RMS norm of the read.  Replaces the T=1 PyTorch path of src/assoc.py:384-512 (about 80 launches per layer in
 * the reference's graphed step, src/bench.py:281-288).
 *   qp, kp, vp: in_dtype, (B,H,D) with batch stride in_stride_b (elements), unit stride over (H,D).
 *   normalize != 0: L2-normalise q, k, v first (eps 1e-12 on the norm).
 *   gate (B,H) in_dtype, batch stride gate_stride_b, or NULL.  Plain rule: k *= sigmoid(gate).  Delta rule
 *   (delta != 0): beta = sigmoid(gate) if gate_is_logit else gate.
 *   decay (B,H) in_dtype, batch stride decay_stride_b.  decay_A == NULL: decay holds log alpha.  Otherwise
 *   log alpha = -softplus(decay) * exp(decay_A[h])  (src/assoc.py:355-356), decay_A [H] fp32.
 *   theta [H][D/2] fp32.  shift_dev: device fp32 scalar (may be NULL: then shift_host is used) = number of
 *   positions the carried state is rotated back by (the previous call's length).
 *   S_in, S_out [B][H][D][D] fp32; may be the same buffer (in-place).
 *   rms_weight [D] fp32 or NULL; rms_eps used only with rms_weight.
 *   o: out_dtype, (B,H,D) with batch stride out_stride_b.
 * ------------------------------------------------------------------------------------------------------- */
int pgb_aspin_decode_step(const void *qp, const void *kp, const void *vp, int in_dtype, long long in_stride_b,
                          int normalize, const void *gate, long long gate_stride_b, int gate_is_logit, int delta,
                          const void *decay, long long decay_stride_b, const float *decay_A, const float *theta,
                          const float *shift_dev, float shift_host, const float *S_in, float *S_out,
                          const float *rms_weight, float rms_eps, void *o, int out_dtype, long long out_stride_b,
                          int B, int H, int D, void *stream);

/* Which kernel pgb_aspin_decode_step uses at head dim 64: 0 (default) = from 512 (sequence, head) pairs up one warp per
 * pair, a lane owning two value columns of all key rows (no block barrier, no partial sums through shared memory), below
 * that one 256-thread CTA per pair (the kernel head dim 128 always uses); 1 = always the CTA per pair; 2 = always the warp
 * per pair. Process-wide; for A/B timing and tests. No counterpart in the reference. */
int pgb_decode_set_variant(int variant);

#ifdef __cplusplus
}
#endif
#endif /* PRAGNOSIA_B200_H */
