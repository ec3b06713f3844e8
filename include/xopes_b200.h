/*
 * xopes_b200 -- C ABI of the B200 (sm_100a) lightning-attention library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*,
 * i.e. a cudaStream_t), enqueues work on that stream and returns without waiting for it; nothing
 * here synchronises (except la_device_status and la_debug_lavd_unsafe, which read a word back) or
 * throws.  The caller owns every tensor and every workspace.  Two things the library creates for
 * itself, once per device and on first need: a stream-ordered memory pool from which a tcgen05
 * launch that splits (sequence, head) pairs across CTAs takes its hand-off scratch
 * (cudaMallocFromPoolAsync / cudaFreeAsync on the caller's stream, about 10 MB per launch in
 * flight), and two non-blocking side streams with three events on which independent gradient
 * passes of one backward call run beside each other.  la_lasd_bwd_noalloc uses neither.  The
 * return value is LA_OK or a negative LA_ERR_* code; la_status_string() turns it into text.
 *
 * Tensor layout (same as the reference operators): q, k are (B, N, H, D), v, o are (B, N, H, E),
 * row-major and contiguous; recurrent states are (B, H, D, E) fp32, contiguous.  `dtype` is the
 * element type of q, k, v, o, do, dq, dk, dv.  Log decays and states are always fp32.
 * With cu_seqlens (int64, device memory, M+1 entries, first 0, last N) B must be 1 and the M
 * documents are independent sequences: states are (M, H, D, E).
 *
 * Citations name files of the reference project (Doraemonzzz/xopes) by their path in that
 * project; they say which reference interface each entry point stands in for.
 */
#ifndef XOPES_B200_H_
#define XOPES_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define LA_API __attribute__((visibility("default")))
#else
#define LA_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define LA_OK 0
#define LA_ERR_NULL_POINTER (-1)   /* a required pointer is NULL                                  */
#define LA_ERR_BAD_SHAPE (-2)      /* a size is <= 0, B != 1 with cu_seqlens, or M != 0 without   */
#define LA_ERR_UNSUPPORTED (-3)    /* dtype / head dimension outside what the kernels cover        */
#define LA_ERR_CUDA (-4)           /* a CUDA runtime or driver call failed (launch, tensor map)    */
#define LA_ERR_TOO_LARGE (-5)      /* a size exceeds a documented fixed maximum                    */
#define LA_ERR_MISALIGNED (-6)     /* a pointer is not aligned as the chosen kernel requires       */
#define LA_ERR_WORKSPACE (-7)      /* workspace pointer NULL or too small                          */

enum la_dtype { LA_F32 = 0, LA_BF16 = 1, LA_F16 = 2 };

/* flags for the lasd/lavd entry points */
#define LA_FLAG_FORCE_RECURRENCE 1u /* never take the tcgen05 chunk kernels                       */
#define LA_FLAG_REQUIRE_TENSOR 2u   /* fail with LA_ERR_UNSUPPORTED instead of taking the scan     */
/* The decay tensors (ld; ldk, ldv) hold PRE-ACTIVATIONS x and the log decay is logsigmoid(x), the
 * usual producer of these decays (benchmarks/lightning_attention/benchmark.py:308-317): the
 * kernels apply it where they read the decay, and the backward returns d/dx in dld / dldk / dldv
 * (the chain-rule factor sigmoid(-x) is applied where the log-decay gradient is finished).  Saves
 * the producer's pass over the decay tensor and the elementwise pass of its backward. */
#define LA_FLAG_LD_LOGSIGMOID 4u
/* Vector decay only: ldk / ldv point to 16-bit values of the type of q, k, v (what the reference's
 * benchmark passes, benchmarks/lightning_attention/benchmark.py:315-316) although the parameters
 * are declared `const float *`; the kernels widen them where they read them, so the decay tensor
 * costs 2 bytes per value in every pass instead of a conversion pass plus 4.  dldk / dldv stay
 * fp32.  Rejected with LA_ERR_UNSUPPORTED for fp32 inputs and by the scalar-decay entry points
 * (ld is always fp32).  The decode entry points take fp32 decays only. */
#define LA_FLAG_LD_16BIT 8u

/* Library identification; bumps when the ABI changes. */
LA_API int la_abi_version(void);
LA_API const char *la_status_string(int status);

/* Which kernel family a call with these parameters runs: 1 = tcgen05/TMA chunk kernels,
 * 0 = fp32 CUDA-core scan kernels, negative = LA_ERR_*.  Pure host logic, no CUDA call. */
LA_API int la_lasd_path(int64_t N, int64_t D, int64_t E, int dtype, unsigned flags);

/* Device-side watchdog word.  The tcgen05 kernels bound every mbarrier wait; a wait that runs
 * out records a non-zero code here and the kernel returns early.  la_device_status() copies the
 * word of the current device to the host (this one call synchronises the stream it is given). */
LA_API int la_device_status(void *stream, int *status_out);
LA_API int la_device_status_clear(void *stream);

/* Reads (and synchronises the stream for) what the last vector-decay call on this GPU left behind:
 * 0 = it ran on the one-reference tensor-core kernels, 1 = a chunk decayed too fast for those and
 * the two-reference tensor-core kernels reran it, 2 = those gave up too and the scan kernels reran
 * it.  No counterpart in the reference. */
LA_API int la_debug_lavd_unsafe(void *stream, int *flag_out);

/* Text of the last CUDA error this library met on the calling thread (after an LA_ERR_CUDA return);
 * empty if none.  No counterpart in the reference. */
LA_API const char *la_debug_last_cuda_error(void);

/* Self-test of the watchdog (no counterpart in the reference): launches one CTA that waits, with
 * a limit of limit_us microseconds (1 .. 1,000,000), on an mbarrier nothing ever arrives on.  The
 * wait gives up, the kernel returns by itself and la_device_status() then reads 199. */
LA_API int la_debug_wait_probe(int64_t limit_us, void *stream);

/* Self-test of the tensor-core building blocks (no counterpart in the reference): one
 * 128x128x128 product D (fp32, row-major) from a, b (128x128, 16-bit, row-major, 16-byte aligned)
 * through one of the operand staging forms the chunk kernels use.  variant 0: D = a b^T;
 * 1, 2, 4: D = a b; 3: D = a^T b. */
LA_API int la_debug_umma_probe(int variant, const void *a, const void *b, float *d, int dtype,
                               void *stream);

/* ---------------------------------------------------------------------------------------------
 * Scalar decay (lasd).  ld is fp32 and addressed as ld[b*ld_sb + n*ld_sn + h*ld_sh] (element
 * strides), so (B,N,H) tensors, (H,) per-head vectors (strides 0,0,1) and expanded views all work.
 * ------------------------------------------------------------------------------------------- */

/* Forward: o and final_state from q, k, v, ld and an optional initial_state.
 * Stands in for lasd_parallel_fwd (xopes/ops/lightning_attn/scalar_decay/lasd_parallel_triton.py:474-565)
 * and, with LA_FLAG_FORCE_RECURRENCE or N == 1, lasd_recurrence_fwd
 * (xopes/ops/lightning_attn/scalar_decay/lasd_recurrence_triton.py:116-164).
 * initial_state and final_state may be NULL.  M is the number of documents (0 without cu_seqlens). */
LA_API int la_lasd_fwd(const void *q, const void *k, const void *v, const float *ld, int64_t ld_sb,
                int64_t ld_sn, int64_t ld_sh, const float *initial_state,
                const int64_t *cu_seqlens, void *o, float *final_state, int64_t B, int64_t N,
                int64_t H, int64_t D, int64_t E, int64_t M, int dtype, unsigned flags,
                void *stream);

/* Bytes of scratch la_lasd_bwd needs (0 when dld is not requested). */
LA_API int64_t la_lasd_bwd_workspace_bytes(int64_t B, int64_t N, int64_t H, int64_t D, int64_t E,
                                    int64_t M, int want_dld);

/* Backward: dq, dk, dv (dtype), and optionally dld (fp32, contiguous (B,N,H)) and dinitial_state
 * (fp32) from the forward inputs, do and an optional dfinal_state.  Recomputes the forward states.
 * Stands in for lasd_parallel_bwd (scalar_decay/lasd_parallel_triton.py:569-754) and
 * lasd_recurrence_bwd (scalar_decay/lasd_recurrence_triton.py:405-498).
 * dld == NULL skips the log-decay gradient; workspace may then be NULL. */
LA_API int la_lasd_bwd(const void *q, const void *k, const void *v, const float *ld, int64_t ld_sb,
                int64_t ld_sn, int64_t ld_sh, const float *initial_state, const void *d_o,
                const float *dfinal_state, const int64_t *cu_seqlens, void *dq, void *dk,
                void *dv, float *dld, float *dinitial_state, void *workspace,
                int64_t workspace_bytes, int64_t B, int64_t N, int64_t H, int64_t D, int64_t E,
                int64_t M, int dtype, unsigned flags, void *stream);

/* la_lasd_bwd for callers that cannot hand over scratch memory.  It has no counterpart in the
 * reference (whose Python drivers allocate freely with torch.empty).
 *
 * Some hosts of this library are not allowed to allocate device memory at the point where they
 * call it: a serving runtime whose whole memory budget was carved up at start-up, a plugin whose
 * "enqueue" hook is forbidden from touching the allocator, or a latency-critical loop where an
 * allocator call could stall the device.  For them this entry point takes the same arguments as
 * la_lasd_bwd minus workspace / workspace_bytes and keeps the scratch inside the library, in a
 * fixed device array of LA_NOALLOC_SCRATCH_BYTES that every GPU loading the library holds until
 * the process exits.  It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 *  - Limit: la_lasd_bwd_workspace_bytes(B, N, H, D, E, M, dld != NULL) must not exceed
 *    LA_NOALLOC_SCRATCH_BYTES, otherwise LA_ERR_TOO_LARGE is returned and nothing is launched.
 *    (Without dld the requirement is 0, so any size passes.)
 *  - The first call on each device looks up the array's device address (one runtime query, with
 *    that device current).  Make that first call before starting any stream capture.
 *  - All calls share the one array and it keeps the previous call's contents.  Nothing in it needs
 *    to be zero on entry (each call writes every word before reading it), but two calls whose
 *    kernels overlap on the GPU -- different streams, or different threads on one device -- race
 *    on it: serialise them. */
#define LA_NOALLOC_SCRATCH_BYTES (8u << 20)
LA_API int la_lasd_bwd_noalloc(const void *q, const void *k, const void *v, const float *ld,
                               int64_t ld_sb, int64_t ld_sn, int64_t ld_sh,
                               const float *initial_state, const void *d_o,
                               const float *dfinal_state, const int64_t *cu_seqlens, void *dq,
                               void *dk, void *dv, float *dld, float *dinitial_state, int64_t B,
                               int64_t N, int64_t H, int64_t D, int64_t E, int64_t M, int dtype,
                               unsigned flags, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Vector decay (lavd).  ldk (B,N,H,D) and ldv (B,N,H,E) are fp32, contiguous; either may be NULL
 * (not both).
 * ------------------------------------------------------------------------------------------- */

/* Which kernel family a vector-decay call runs: 1 = tcgen05/TMA chunk kernels (16-bit inputs,
 * D = E = 128, N >= 128, exactly one of ldk / ldv), 0 = fp32 scan kernels.  On path 1 the decay decides, on the
 * device, how far the call gets: the one-reference kernels handle chunks whose halves (64 tokens)
 * decay by at most 2^-64 per feature (bf16; 2^-10 for fp16); if a chunk exceeds that, the
 * two-reference kernels rerun the call (safe while every 32-token quarter decays by at most 2^-96;
 * the reference's own benchmark decay logsigmoid(N(0,1)) is about 2^-37 per quarter); if a chunk
 * exceeds that too, the scan kernels rerun it.  The two flag words behind those decisions are per
 * GPU: vector-decay calls whose kernels overlap on one GPU must be serialised. */
LA_API int la_lavd_path(int64_t N, int64_t D, int64_t E, int dtype, int has_ldk, int has_ldv,
                        unsigned flags);

/* Stands in for lavd_parallel_fwd (xopes/ops/lightning_attn/vector_decay/lavd_parallel_triton.py:879-992)
 * and lavd_recurrence_fwd (vector_decay/lavd_recurrence_triton.py:157-218). */
LA_API int la_lavd_fwd(const void *q, const void *k, const void *v, const float *ldk, const float *ldv,
                const float *initial_state, const int64_t *cu_seqlens, void *o,
                float *final_state, int64_t B, int64_t N, int64_t H, int64_t D, int64_t E,
                int64_t M, int dtype, unsigned flags, void *stream);

/* Bytes of scratch la_lavd_bwd needs when dfinal_state is given (one recomputed final state). */
LA_API int64_t la_lavd_bwd_workspace_bytes(int64_t B, int64_t N, int64_t H, int64_t D, int64_t E,
                                    int64_t M);

/* Stands in for lavd_parallel_bwd (vector_decay/lavd_parallel_triton.py:996-1290) and
 * lavd_recurrence_bwd (vector_decay/lavd_recurrence_triton.py:530-713).
 * dldk (B,N,H,D) / dldv (B,N,H,E) are fp32 outputs, required exactly when ldk / ldv is given;
 * they double as the kernels' accumulation buffers.  workspace is needed only with
 * dfinal_state (it receives the recomputed final state for the log-decay gradient). */
LA_API int la_lavd_bwd(const void *q, const void *k, const void *v, const float *ldk, const float *ldv,
                const float *initial_state, const void *d_o, const float *dfinal_state,
                const int64_t *cu_seqlens, void *dq, void *dk, void *dv, float *dldk, float *dldv,
                float *dinitial_state, void *workspace, int64_t workspace_bytes, int64_t B,
                int64_t N, int64_t H, int64_t D, int64_t E, int64_t M, int dtype, unsigned flags,
                void *stream);

/* ---------------------------------------------------------------------------------------------
 * Cutting long sequences into segments that run in parallel (no counterpart in the reference, whose
 * chunk kernels get their parallelism from materialised per-chunk states,
 * scalar_decay/lasd_parallel_triton.py:22-253; here the same associativity is used at segment
 * granularity so that nothing per-chunk is written to HBM).
 *
 * la_lasd_state_pass: for every (sequence, head) the state its own tokens build from a zero start,
 *     states[s,h] = sum_j w_j y_j^T z_j   (128 x 128 fp32, row = feature of y, column = feature of z)
 * and gsum[s,h] = the sequence's total log decay.  reverse = 0: w_j = exp(sum of ld after token j)
 * (state at the sequence's end, forward flow: (y,z) = (k,v) gives S, (v,k) gives S^T);
 * reverse = 1: w_j = exp(sum of ld up to and including token j) (state at the sequence's start for
 * the backward recurrences: (q,do) gives dS, (do,q) gives dS^T).  y, z are (B,N,H,128) 16-bit; ld as
 * in la_lasd_fwd (flags: LA_FLAG_LD_LOGSIGMOID only); with cu_seqlens the "sequences" are its M segments (ranges = 0: M + 1 boundaries;
 * ranges = 1: M explicit (begin, end) token pairs, so that a subset of segments can be given).
 * Reads 512 B per token and head.  D = E = 128, 16-bit only.
 *
 * la_lasd_fold_states: from the segments' own states `local` (nseg,H,D,E) and totals gsum (nseg,H),
 * the state ENTERING each segment (`incoming`, same shape): forward flow (reverse = 0) walks the
 * segments in order, a segment flagged first-of-document starts from ext[document] (or zero);
 * reverse flow walks them backwards, a segment flagged last-of-document starts from
 * ext[document].  seg_table is int32 (nseg,4): {document, first-of-document, last-of-document, row
 * of `local` / gsum with the segment's own state, or -1 if none was computed (counts as zero)}.
 * emit (optional, int32 (nseg)) names the row of `incoming` each segment's entering state goes to,
 * -1 for none: the state-only pass may run on finer pieces than the segments that need an entering
 * state.  `ends` (optional, one (H,D,E) row per document) receives the state after each
 * document's last segment in walking order: its end state (forward flow), the state before its first
 * token (reverse flow).  `incoming` may be NULL when only `ends` is wanted.
 * ------------------------------------------------------------------------------------------- */
LA_API int la_lasd_state_pass(const void *y, const void *z, const float *ld, int64_t ld_sb,
                              int64_t ld_sn, int64_t ld_sh, const int64_t *cu_seqlens, float *states,
                              float *gsum, int64_t B, int64_t N, int64_t H, int64_t D, int64_t E,
                              int64_t M, int dtype, int reverse, int ranges, unsigned flags, void *stream);
LA_API int la_lasd_fold_states(const float *local, const float *gsum, const int32_t *seg_table,
                               const int32_t *emit, const float *ext, float *incoming, float *ends, int64_t nseg, int64_t H,
                               int64_t D, int64_t E, int reverse, void *stream);

/* The same pair for vector decay on the features of y (ldk (B,N,H,128) fp32, contiguous):
 *     states[s,h][d][e] = sum_j w_jd y_jd z_je ,  gsum[s,h][d] = the sequence's total log decay of feature d
 * with w_jd = exp(sum of ldk[.,d] after token j) (reverse = 0) or exp(sum up to and including token j)
 * (reverse = 1); (y,z) = (k,v) forward gives S, (q,do) reverse gives dS.  Every factor is <= 1, so
 * this pass has no limit on the strength of the decay.  la_lavd_fold_states folds with the
 * per-feature decay on the state's rows: s = local + exp(gsum[d]) (.) s.  No counterpart in the
 * reference (its chunk-level states live in HBM, vector_decay/lavd_parallel_triton.py:25-316). */
LA_API int la_lavd_state_pass(const void *y, const void *z, const float *ldk, const int64_t *cu_seqlens,
                              float *states, float *gsum, int64_t B, int64_t N, int64_t H, int64_t D,
                              int64_t E, int64_t M, int dtype, int reverse, int ranges, unsigned flags,
                              void *stream);
LA_API int la_lavd_fold_states(const float *local, const float *gsum, const int32_t *seg_table,
                               const int32_t *emit, const float *ext, float *incoming, int64_t nseg,
                               int64_t H, int64_t D, int64_t E, int reverse, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Sequence-parallel scalar decay (no counterpart in the reference, which has no distributed code;
 * the math is lasd_torch's varlen recurrence, scalar_decay/lasd_torch.py:61-103, cut at a rank
 * boundary).  A rank whose first document started on an earlier rank runs la_lasd_fwd with a zero
 * incoming state and then adds the missing term in place:
 *     o[0,t,h,:] += exp(cum[t,h]) * q[0,t,h,:]^T s_in[h]      for t in [0, T1)
 * q, o are (1,N,H,D) / (1,N,H,E); cum is fp32 (T1,H), the inclusive cumulative log decay from the
 * rank's first token; s_in is fp32 (H,D,E), the document's true incoming state.
 * ------------------------------------------------------------------------------------------- */
/* The true state entering `rank` from the all-gathered per-rank summaries, each a row of
 * H*D*E + H + 2 floats [S_loc | G | open_end | spans]:
 *     S_in(r+1) = open_end(r) * (S_loc(r) + spans(r) * exp(G(r)) * S_in(r)),  S_in(0) = 0.
 * gathered is (world, H*D*E + H + 2) fp32, s_in (H,D,E) fp32.  No counterpart in the reference. */
LA_API int la_seqpar_fold(const float *gathered, float *s_in, int64_t rank, int64_t H, int64_t D,
                          int64_t E, void *stream);

/* Segmented forward inside one GPU: long sequences are cut into segments that run as independent
 * "documents" of la_lasd_fwd (zero incoming state), then stitched.  seg_table is int32 (nseg, 4):
 * {first token, length, index of the segment's first 128-token tile among all corrected tiles,
 * 1 if the segment starts a document}.  la_seqpar_fold_segments turns the segments' end states
 * (nseg,H,D,E) into true end states in place and writes each segment's incoming state to s_in,
 * given seg_decay (nseg,H) = the summed log decay of each segment.  la_seqpar_correct_multi then
 * adds exp(cum[t] - cum[start-1]) q_t^T s_in[seg] to every token of the listed segments (pass only
 * the segments that continue a document; their tile indices run from 0 to total_tiles), cum being
 * the inclusive cumulative log decay (N,H) of the whole stream.  16-bit, D = E = 128 only.
 * No counterpart in the reference. */
LA_API int la_seqpar_fold_segments(float *states, const float *seg_decay, const int32_t *seg_table,
                                   float *s_in, int64_t nseg, int64_t H, int64_t D, int64_t E,
                                   void *stream);
LA_API int la_seqpar_correct_multi(const void *q, void *o, const float *cum, const float *s_in,
                                   const int32_t *seg_table, int64_t nseg, int64_t total_tiles,
                                   int64_t N, int64_t H, int64_t D, int64_t E, int dtype, void *stream);

LA_API int la_seqpar_correct(const void *q, void *o, const float *cum, const float *s_in, int64_t T1,
                             int64_t N, int64_t H, int64_t D, int64_t E, int dtype, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Single-token decode: one new token per sequence, state read, updated and written once.
 * q, k (B,1,H,D), v, o (B,1,H,E); state_in / state_out (B,H,D,E) fp32 and MAY alias (in place).
 * Stand in for _lasd_recurrence_fwd with N == 1 (scalar_decay/lasd_recurrence_triton.py:28-113)
 * and _lavd_recurrence_fwd with N == 1 (vector_decay/lavd_recurrence_triton.py:28-154).
 * ------------------------------------------------------------------------------------------- */
LA_API int la_decode_scalar(const void *q, const void *k, const void *v, const float *ld, int64_t ld_sb,
                     int64_t ld_sh, const float *state_in, float *state_out, void *o, int64_t B,
                     int64_t H, int64_t D, int64_t E, int dtype, void *stream);

LA_API int la_decode_vector(const void *q, const void *k, const void *v, const float *ldk,
                     const float *ldv, const float *state_in, float *state_out, void *o,
                     int64_t B, int64_t H, int64_t D, int64_t E, int dtype, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Fused normalisation + gate: the op that follows lightning attention in a model block.  Stands in
 * for normalize_torch / normalize_triton with a gate and no residual
 * (xopes/ops/normalize/normalize/normalize_torch.py:9-111):
 *     a = act(gate);  z = x*a (gate_pos 0 = pre) or x;  zc = z - mean(z) if use_mean;
 *     y = c * zc / sqrt(sum zc^2 + eps) * weight + bias   per group of e features;
 *     o = y (pre / no gate) or y*a (gate_pos 1 = post).
 * x, gate, out, d_out, dx, dgate are (rows, G*e) in `dtype`, contiguous; gate may be NULL (plain
 * normalisation); weight, bias are fp32 (G*e) or NULL; act: 0 none, 1 relu, 2 sigmoid, 3 silu.
 * e must be a multiple of 4 and at most 512.  dweight / dbias (fp32, G*e, or NULL) are ACCUMULATED
 * into: zero them first.  One pass over the inputs each way, fp32 arithmetic.
 * ------------------------------------------------------------------------------------------- */
LA_API int la_normalize_gate_fwd(const void *x, const void *gate, const float *weight, const float *bias,
                                 void *out, int64_t rows, int64_t G, int64_t e, int dtype, int act,
                                 int gate_pos, float c, float eps, int use_mean, void *stream);
LA_API int la_normalize_gate_bwd(const void *x, const void *gate, const float *weight, const float *bias,
                                 const void *d_out, void *dx, void *dgate, float *dweight, float *dbias,
                                 int64_t rows, int64_t G, int64_t e, int dtype, int act, int gate_pos,
                                 float c, float eps, int use_mean, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* XOPES_B200_H_ */
