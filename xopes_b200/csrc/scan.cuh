// Host-visible interface of the fp32 CUDA-core scan kernels (scan.cu) and the small
// log-decay-gradient / decode kernels.  Internal to the library; the public ABI is
// include/xopes_b200.h.
#pragma once
#include "common.cuh"

namespace la {

// One directional pass of the linear-attention recurrence over a "row" operand a (R features),
// a "column" operand b (C features) and a contraction operand w (C features):
//
//   forward :  T <- dec_t * T ; T += a_t b_t^T ; out_t = T w_t
//   reverse :  T += a_t b_t^T ; out_t = T w_t ; T <- dec_t * T        (tokens visited last to first)
//
// dec_t[r][c] = exp(ld_t) * exp(ldr_t[r]) * exp(ldc_t[c]) (each factor optional).  With
// (a,b,w) = (v,k,q) this is the output pass (T = S^T), (k,v,do) gives dq (T = S),
// (q,do,v) reversed gives dk (T = dS) and (do,q,k) reversed gives dv (T = dS^T) -- the same
// role swap the reference performs with its TRANS / REVERSE kernel flags
// (xopes/ops/lightning_attn/scalar_decay/lasd_parallel_triton.py:651-733).
struct ScanParams {
  const void *a = nullptr, *b = nullptr, *w = nullptr;  // dtype tensors (B,N,H,R|C)
  void *out = nullptr;                                   // (B,N,H,R) dtype
  const void *x = nullptr;                               // optional (B,N,H,R) dtype
  float *xout = nullptr;                                 // see xmode
  int xmode = 0;  // 0 none; 1 xout[tile][b,n,h] = sum_r x*out; 2 xout[b,n,h,r] = x*out; 3 xout -= x*out
  const float *ld = nullptr;                             // scalar log decay, strided
  int64_t ld_sb = 0, ld_sn = 0, ld_sh = 0;
  const float *ldr = nullptr;                            // (B,N,H,R) fp32 row log decay
  const float *ldc = nullptr;                            // (B,N,H,C) fp32 column log decay
  const float *t0 = nullptr;                             // (nb,H,D,E) fp32 starting state, optional
  float *tfinal = nullptr;                               // (nb,H,D,E) fp32 end state, optional
  int64_t st_rs = 0, st_cs = 0;                          // element strides of T's row / column in the state
  const int64_t *cu = nullptr;                           // cu_seqlens (device) or null
  int B = 0, N = 0, H = 0, R = 0, C = 0, M = 0;
  int reverse = 0;
  int ld_act = 0;  // 1: ld / ldr / ldc hold pre-activations x and the decay factor is sigmoid(x) = exp(logsigmoid(x))
  int ld16 = 0;    // 1: ldr / ldc point to 16-bit values of the kernel's element type (ld stays fp32)
  const int *enable = nullptr;  // optional device word: the kernel does nothing while it is 0
};

// Number of row tiles launch_scan will use for these sizes (size of xout's leading dimension in
// xmode 1).  Deterministic function of the sizes only.
int scan_row_tiles(int R, int C, int H, int nb);
int launch_scan(const ScanParams &p, int dtype, cudaStream_t stream);

// dld[b,t,h] = sum_{s>=t in the same sequence} (sum_tiles A[.,s] - sum_tiles K[.,s]) + <S_fin, dS_fin>
// act_x (optional, with its element strides): the decay was logsigmoid(act_x); the result is then
// the gradient with respect to act_x (times sigmoid(-act_x)).
int launch_dld_scalar(const float *slots_q, int ntq, const float *slots_k, int ntk,
                      const float *final_state, const float *dfinal_state, const int64_t *cu,
                      float *dld, int B, int N, int H, int DE, int M, cudaStream_t stream,
                      const float *act_x = nullptr, int64_t x_sb = 0, int64_t x_sn = 0, int64_t x_sh = 0);

// In place: buf[b,t,h,f] <- sum_{s>=t} buf[b,s,h,f] + sum over the other state axis of S_fin*dS_fin.
// f_is_row: f indexes the state's D axis (sum over E) else its E axis (sum over D).
// act_x (optional, same layout as buf, elements of type act_dtype): the decay was
// logsigmoid(act_x); the result is then the gradient with respect to act_x.
int launch_revcumsum_vec(float *buf, const float *final_state, const float *dfinal_state,
                         const int64_t *cu, int B, int N, int H, int F, int D, int E, int f_is_row,
                         int M, cudaStream_t stream, const float *act_x = nullptr, int act_dtype = LA_F32);

int launch_decode(const void *q, const void *k, const void *v, const float *ld, int64_t ld_sb,
                  int64_t ld_sh, const float *ldk, const float *ldv, const float *state_in,
                  float *state_out, void *o, int B, int H, int D, int E, int dtype,
                  cudaStream_t stream);

}  // namespace la
