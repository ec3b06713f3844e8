// Host-visible interface of the tcgen05 / TMA chunk kernel for scalar decay (chunk_sm100.cu).
#pragma once
#include "common.cuh"

namespace la {

// One directional chunk-parallel pass over 128-token chunks, one CTA per (sequence, head),
// running state T (128x128 fp32) resident in tensor memory:
//
//   W_c = [(X_c Y_c^T) (.) M_c] Z_c + diag(s_c) X_c T ;   T <- e^{g_c} T + (Y_c (.) u_c)^T Z_c
//
// forward direction: M_ij = e^{c_i-c_j}[i>=j], s = e^{c}, u = e^{g-c}   (c = inclusive cumsum of ld)
// reverse direction: M_ij = e^{c_j-c_i}[j>=i], s = e^{g-c}, u = e^{c}, chunks visited last to first.
// (X,Y,Z) = (q,k,v) gives o; (do,v,k) with the state transposed gives dq; (v,do,q) reversed and
// transposed gives dk; (k,q,do) reversed gives dv
// (xopes/ops/lightning_attn/scalar_decay/lasd_parallel_triton.py:548-563,651-733).
struct ChunkPass {
  const void *x = nullptr, *y = nullptr, *z = nullptr;  // (B,N,H,fx), (B,N,H,fx), (B,N,H,fz) dtype
  void *out = nullptr;                                   // (B,N,H,fz) dtype
  const void *xrow = nullptr;                            // optional (B,N,H,fz): rowdot = sum_f xrow*W
  float *rowdot = nullptr;                               // (B,N,H) fp32
  const float *ld = nullptr;
  int64_t ld_sb = 0, ld_sn = 0, ld_sh = 0;
  const float *t0 = nullptr;                             // (nb,H,D,E) fp32 or null
  float *tfinal = nullptr;                               // (nb,H,D,E) fp32 or null
  int state_transposed = 0;                              // T[i][j] lives at state[j][i]
  int reverse = 0;
  const int64_t *cu = nullptr;
  int B = 0, N = 0, H = 0, M = 0;
  int ld_act = 0;          // 1: ld holds pre-activations, the log decay is logsigmoid(ld)
  int fx = 128, fz = 128;  // features per head of x, y (the contraction of X Y^T) and of z, out, xrow
  int no_scratch = 0;  // 1: never take hand-off scratch from the library's pool (one CTA per pair)
};

bool chunk_supported(int64_t N, int64_t D, int64_t E, int dtype);
// With more (sequence, head) pairs than SMs the launch runs one CTA per SM on an even split of
// the chunk space; the running state of a pair cut by a split crosses through scratch taken from
// a stream-ordered pool the library owns (and returned to it in stream order).
int launch_chunk_pass(const ChunkPass &p, int dtype, cudaStream_t stream);
// Two passes over the same tokens in one launch (even CTAs: p, odd CTAs: q), so that operand
// tiles both passes read are fetched from HBM once.  Sizes and cu_seqlens must be the same.
int launch_chunk_pass_pair(const ChunkPass &p, const ChunkPass &q, int dtype, cudaStream_t stream);
// One directional vector-decay (ldk) pass on tcgen05 (lavd_chunk_sm100.cu).  tmode = 0: the decay
// acts on the contraction dimension of X Y^T (o and dv passes); tmode = 1: on the output dimension
// (dq and dk passes, state transposed), with the optional log-decay-gradient accumulation
// dld (+)= xrow * W.  ref2 = 0: one reference row per chunk, safe while half a chunk decays by at
// most 2^-64 (bf16); ref2 = 1: two reference rows, safe while a 32-row quarter decays by at most
// 2^-96.  `unsafe` is raised when a chunk exceeds that range; the caller then reruns the next
// formulation (two references, then the scan kernels), each predicated on the previous one's word
// through `enable`.
struct LavdPass {
  const void *x = nullptr, *y = nullptr, *z = nullptr;
  const float *ldk = nullptr;
  void *out = nullptr;
  const void *xrow = nullptr;
  float *dld = nullptr;
  int dld_sub = 0;   // 1: the terms are subtracted from dld (dk pass) instead of stored (dq pass)
  int dld_add = 0;   // 1: dld starts at zero and both passes add to it atomically (they may overlap)
  const float *t0 = nullptr;
  float *tfinal = nullptr;
  int state_transposed = 0, reverse = 0, tmode = 0;
  const int64_t *cu = nullptr;
  int B = 0, N = 0, H = 0, M = 0;
  int *unsafe = nullptr;
  int ld_act = 0;    // 1: ldk holds pre-activations, the log decay is logsigmoid(ldk)
  int ld16 = 0;      // 1: ldk points to 16-bit values of the type of x, y, z
  int ref2 = 0;
  const int *enable = nullptr;  // optional device word: the launch does nothing while it reads 0
};
bool lavd_chunk_supported(int64_t N, int64_t D, int64_t E, int dtype, bool has_ldk, bool has_ldv);
int launch_lavd_pass(const LavdPass &p, int dtype, cudaStream_t stream);

// State-only pass (state_pass_sm100.cu): per (sequence, head) the state the sequence's own tokens
// build from a zero start, T = sum_j decay_j y_j^T z_j (row = feature of y, column = feature of z),
// and the sequence's total log decay.  reverse = 0: decay from token j (exclusive) to the end of the
// sequence (state at the end, forward flow); reverse = 1: decay from the start to token j
// (inclusive) (state at the start, reverse flow).  16-bit, 128 features.
struct StatePass {
  const void *y = nullptr, *z = nullptr;  // (B,N,H,128) dtype
  const float *ld = nullptr;               // scalar decay: strided fp32
  int64_t ld_sb = 0, ld_sn = 0, ld_sh = 0;
  const float *ldv = nullptr;              // vector decay: (B,N,H,128) fp32 on the features of y
  const int64_t *cu = nullptr;
  float *states = nullptr;                 // (nb,H,128,128) fp32
  float *gsum = nullptr;                   // (nb,H) fp32 (scalar) / (nb,H,128) (vector), optional
  int B = 0, N = 0, H = 0, M = 0, reverse = 0;
  int ld_act = 0;  // 1: ld / ldv hold pre-activations, the log decay is their logsigmoid
  int ld16 = 0;    // 1 (vector pass only): ldv points to 16-bit values of the type of y, z
  int ranges = 0;  // 1: cu holds M (begin, end) token ranges instead of M + 1 boundaries
};
int launch_state_pass(const StatePass &p, int dtype, cudaStream_t stream);
int launch_state_pass_vec(const StatePass &p, int dtype, cudaStream_t stream);
int launch_fold_states_vec(const float *local, const float *gsum, const int *seg, const int *emit, const float *ext,
                           float *out, int nseg, int H, int D, int E, int reverse, cudaStream_t st);
int launch_fold_states(const float *local, const float *gsum, const int *seg, const int *emit, const float *ext,
                       float *out, float *ends, int nseg, int H, int DE, int reverse, cudaStream_t st);

// o[0,t,h,:] += exp(cum[t,h]) * q[0,t,h,:] S_in[h] for t < T1 (sequence-parallel correction, seqpar.cu)
int launch_seqpar_correct(const void *q, void *o, const float *cum, const float *s_in, int T1, int N, int H,
                          int D, int E, int dtype, cudaStream_t st);
int launch_seqpar_fold(const float *gathered, float *s_in, int rank, int H, int DE, cudaStream_t st);
int launch_seqpar_fold_segments(float *states, const float *G, const int *seg, float *s_in, int nseg, int H, int DE,
                                cudaStream_t st);
int launch_seqpar_correct_multi(const void *q, void *o, const float *cum, const float *s_in, const int *seg,
                                int nseg, int total_tiles, int N, int H, int dtype, cudaStream_t st);
// One CTA waits on an mbarrier that nothing ever arrives on, with a limit of limit_us: the wait
// gives up, records its code in the device status word and the kernel returns (chunk_sm100.cu).
int wait_probe(uint32_t limit_us, cudaStream_t stream);
// one 128x128x128 product through one operand staging variant (see chunk_sm100.cu)
int umma_probe(int variant, const void *a, const void *b, float *d, int dtype, cudaStream_t stream);

}  // namespace la
