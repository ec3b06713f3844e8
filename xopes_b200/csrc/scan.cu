// fp32 CUDA-core kernels: the token-by-token scan (all dtypes, any head dimension up to 512),
// the single-token decode update and the log-decay-gradient reductions.
//
// These follow the recurrence exactly as the reference's torch operators state it
// (xopes/ops/lightning_attn/scalar_decay/lasd_torch.py:50-59,
//  xopes/ops/lightning_attn/vector_decay/lavd_torch.py:78-95) with every product and sum in fp32,
// so they are the path for fp32 inputs (tolerance 1e-5), odd head dimensions, single tokens and
// anything the tcgen05 chunk kernels do not cover.
#include "scan.cuh"

namespace la {

namespace {

constexpr int kMaxFeat = 512;

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }

// --------------------------------------------------------------------------------------------
// scan kernel
// --------------------------------------------------------------------------------------------
// Thread (rl, g): row rl of the CTA's row tile, lane group g of G.  It owns CC columns of that row
// of T, as CC/4 float4 chunks interleaved across the G lanes (chunk j*G+g), so that the G lanes of
// a row read consecutive 16-byte pieces of the shared b / w / decay vectors.
template <typename T, int CC, int G>
__global__ void __launch_bounds__(256) scan_kernel(ScanParams p, int TB) {
  constexpr int CP = CC * G;  // padded column count
  if (p.enable != nullptr && *p.enable == 0) return;
  const int tid = threadIdx.x;
  const int nthreads = blockDim.x;
  const int RT = nthreads / G;
  const int g = tid % G;
  const int rl = tid / G;
  const int row0 = blockIdx.x * RT;
  const int row = row0 + rl;
  const int h = blockIdx.y;
  const int seq = blockIdx.z;
  const int R = p.R, C = p.C, H = p.H;

  int64_t t_begin = 0, t_end = p.N;
  int64_t bidx = seq;
  if (p.cu != nullptr) {
    t_begin = p.cu[seq];
    t_end = p.cu[seq + 1];
    bidx = 0;
  }
  const int64_t len = t_end - t_begin;

  extern __shared__ __align__(16) float smem[];
  float *a_s = smem;                 // [TB][RT]
  float *dr_s = a_s + TB * RT;       // [TB][RT]
  float *x_s = dr_s + TB * RT;       // [TB][RT]
  float *out_s = x_s + TB * RT;      // [TB][RT]
  float *b_s = out_s + TB * RT;      // [TB][CP]
  float *w_s = b_s + TB * CP;        // [TB][CP]
  float *dc_s = w_s + TB * CP;       // [TB][CP]
  float *lam_s = dc_s + TB * CP;     // [TB]

  const T *a = static_cast<const T *>(p.a);
  const T *b = static_cast<const T *>(p.b);
  const T *w = static_cast<const T *>(p.w);
  const T *x = static_cast<const T *>(p.x);
  T *out = static_cast<T *>(p.out);

  // ---- starting state
  float Tst[CC];
  const int64_t st_base = ((int64_t)seq * H + h) * (int64_t)R * C;
#pragma unroll
  for (int j = 0; j < CC / 4; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = (j * G + g) * 4 + i;
      float val = 0.f;
      if (p.t0 != nullptr && row < R && c < C) val = p.t0[st_base + row * p.st_rs + c * p.st_cs];
      Tst[j * 4 + i] = val;
    }
  }

  const bool has_ld = p.ld != nullptr, has_ldr = p.ldr != nullptr, has_ldc = p.ldc != nullptr;
  const int64_t nblk = (len + TB - 1) / TB;
  for (int64_t kb = 0; kb < nblk; ++kb) {
    const int ntok = (int)min((int64_t)TB, len - kb * TB);
    // token visited i-th in this block
    auto tok = [&](int i) -> int64_t {
      const int64_t s = kb * TB + i;
      return p.reverse ? (t_end - 1 - s) : (t_begin + s);
    };
    // ---- load
    for (int idx = tid; idx < ntok * RT; idx += nthreads) {
      const int i = idx / RT, r = idx - i * RT;
      const int gr = row0 + r;
      const int64_t base = ((bidx * p.N + tok(i)) * H + h) * (int64_t)R + gr;
      float av = 0.f, xv = 0.f, dv = 1.f;
      if (gr < R) {
        av = Cvt<T>::to_f(a[base]);
        if (x != nullptr) xv = Cvt<T>::to_f(x[base]);
        if (has_ldr) {
          const float raw = p.ld16 ? Cvt<T>::to_f(reinterpret_cast<const T *>(p.ldr)[base]) : p.ldr[base];
          dv = p.ld_act ? 1.f / (1.f + expf(-raw)) : expf(raw);
        }
      }
      a_s[idx] = av;
      x_s[idx] = xv;
      dr_s[idx] = dv;
    }
    for (int idx = tid; idx < ntok * CP; idx += nthreads) {
      const int i = idx / CP, c = idx - i * CP;
      const int64_t base = ((bidx * p.N + tok(i)) * H + h) * (int64_t)C + c;
      float bv = 0.f, wv = 0.f, dv = 1.f;
      if (c < C) {
        bv = Cvt<T>::to_f(b[base]);
        wv = Cvt<T>::to_f(w[base]);
        if (has_ldc) {
          const float raw = p.ld16 ? Cvt<T>::to_f(reinterpret_cast<const T *>(p.ldc)[base]) : p.ldc[base];
          dv = p.ld_act ? 1.f / (1.f + expf(-raw)) : expf(raw);
        }
      }
      b_s[idx] = bv;
      w_s[idx] = wv;
      dc_s[idx] = dv;
    }
    if (tid < ntok) {
      float lam = 1.f;
      // exp in double, rounded once: a per-head constant decay is applied at every token, so an
      // ulp of error in it compounds linearly with the sequence length
      if (has_ld) {
        const double raw = (double)p.ld[bidx * p.ld_sb + tok(tid) * p.ld_sn + h * p.ld_sh];
        lam = (float)(p.ld_act ? 1.0 / (1.0 + exp(-raw)) : exp(raw));
      }
      lam_s[tid] = lam;
    }
    __syncthreads();

    // ---- recurrence over the block
    for (int i = 0; i < ntok; ++i) {
      const float rowfac = lam_s[i] * dr_s[i * RT + rl];
      const float av = a_s[i * RT + rl];
      const float *bi = b_s + i * CP, *wi = w_s + i * CP, *di = dc_s + i * CP;
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < CC / 4; ++j) {
        const int c0 = (j * G + g) * 4;
        const float4 bv = ld4(bi + c0), wv = ld4(wi + c0);
        float4 dc = make_float4(rowfac, rowfac, rowfac, rowfac);
        if (has_ldc) {
          const float4 d4 = ld4(di + c0);
          dc.x *= d4.x; dc.y *= d4.y; dc.z *= d4.z; dc.w *= d4.w;
        }
        float *t = Tst + j * 4;
        if (!p.reverse) {
          t[0] = fmaf(t[0], dc.x, av * bv.x);
          t[1] = fmaf(t[1], dc.y, av * bv.y);
          t[2] = fmaf(t[2], dc.z, av * bv.z);
          t[3] = fmaf(t[3], dc.w, av * bv.w);
          acc = fmaf(t[0], wv.x, acc);
          acc = fmaf(t[1], wv.y, acc);
          acc = fmaf(t[2], wv.z, acc);
          acc = fmaf(t[3], wv.w, acc);
        } else {
          t[0] = fmaf(av, bv.x, t[0]);
          t[1] = fmaf(av, bv.y, t[1]);
          t[2] = fmaf(av, bv.z, t[2]);
          t[3] = fmaf(av, bv.w, t[3]);
          acc = fmaf(t[0], wv.x, acc);
          acc = fmaf(t[1], wv.y, acc);
          acc = fmaf(t[2], wv.z, acc);
          acc = fmaf(t[3], wv.w, acc);
          t[0] *= dc.x; t[1] *= dc.y; t[2] *= dc.z; t[3] *= dc.w;
        }
      }
#pragma unroll
      for (int off = G / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (g == 0) out_s[i * RT + rl] = acc;
    }
    __syncthreads();

    // ---- store
    for (int idx = tid; idx < ntok * RT; idx += nthreads) {
      const int i = idx / RT, r = idx - i * RT;
      const int gr = row0 + r;
      if (gr < R) {
        const int64_t base = ((bidx * p.N + tok(i)) * H + h) * (int64_t)R + gr;
        const float ov = out_s[idx];
        if (out != nullptr) out[base] = Cvt<T>::from_f(ov);
        if (p.xmode == 2) p.xout[base] = x_s[idx] * ov;
        if (p.xmode == 3) p.xout[base] -= x_s[idx] * ov;
      }
    }
    if (p.xmode == 1) {
      const int wid = tid >> 5, lane = tid & 31, nw = nthreads >> 5;
      for (int i = wid; i < ntok; i += nw) {
        float s = 0.f;
        for (int r = lane; r < RT; r += 32) s += x_s[i * RT + r] * out_s[i * RT + r];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (lane == 0) {
          const int64_t slot = (int64_t)blockIdx.x * p.B * p.N * H;
          p.xout[slot + (bidx * p.N + tok(i)) * H + h] = s;
        }
      }
    }
    __syncthreads();
  }

  if (p.tfinal != nullptr && row < R) {
#pragma unroll
    for (int j = 0; j < CC / 4; ++j) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = (j * G + g) * 4 + i;
        if (c < C) p.tfinal[st_base + row * p.st_rs + c * p.st_cs] = Tst[j * 4 + i];
      }
    }
  }
}

struct ScanCfg {
  int cc, g, nwarps, tb;
};

ScanCfg pick_cfg(int R, int C, int H, int nb) {
  ScanCfg c;
  if (C <= 32) { c.cc = 8; c.g = 4; }
  else if (C <= 64) { c.cc = 16; c.g = 4; }
  else if (C <= 128) { c.cc = 32; c.g = 4; }
  else if (C <= 256) { c.cc = 32; c.g = 8; }
  else { c.cc = 32; c.g = 16; }
  const int rpw = 32 / c.g;
  int nw = 8;
  while (nw > 1 && nw * rpw / 2 >= R) nw >>= 1;  // do not exceed the row count by more than 2x
  while (nw > 1 && (int64_t)((R + nw * rpw - 1) / (nw * rpw)) * H * nb < 2 * 148) nw >>= 1;
  c.nwarps = nw;
  c.tb = (c.cc * c.g <= 256) ? 16 : 8;
  return c;
}

template <typename T, int CC, int G>
int launch_cfg(const ScanParams &p, const ScanCfg &c, cudaStream_t stream) {
  const int nthreads = c.nwarps * 32;
  const int RT = nthreads / G;
  const int nb = p.cu ? p.M : p.B;
  dim3 grid((p.R + RT - 1) / RT, p.H, nb);
  const size_t smem = sizeof(float) * ((size_t)c.tb * (4 * RT + 3 * CC * G) + c.tb);
  auto kern = scan_kernel<T, CC, G>;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return LA_ERR_CUDA;
  }
  kern<<<grid, nthreads, smem, stream>>>(p, c.tb);
  return launch_status();
}

template <typename T>
int launch_t(const ScanParams &p, const ScanCfg &c, cudaStream_t stream) {
  if (c.cc == 8) return launch_cfg<T, 8, 4>(p, c, stream);
  if (c.cc == 16) return launch_cfg<T, 16, 4>(p, c, stream);
  if (c.g == 4) return launch_cfg<T, 32, 4>(p, c, stream);
  if (c.g == 8) return launch_cfg<T, 32, 8>(p, c, stream);
  return launch_cfg<T, 32, 16>(p, c, stream);
}

}  // namespace

int scan_row_tiles(int R, int C, int H, int nb) {
  const ScanCfg c = pick_cfg(R, C, H, nb);
  const int RT = c.nwarps * 32 / c.g;
  return (R + RT - 1) / RT;
}

int launch_scan(const ScanParams &p, int dtype, cudaStream_t stream) {
  if (p.R <= 0 || p.C <= 0 || p.R > kMaxFeat || p.C > kMaxFeat) return LA_ERR_UNSUPPORTED;
  const int nb = p.cu ? p.M : p.B;
  if (nb <= 0 || p.H <= 0 || p.N <= 0) return LA_ERR_BAD_SHAPE;
  if (p.H > 65535 || nb > 65535) return LA_ERR_TOO_LARGE;
  const ScanCfg c = pick_cfg(p.R, p.C, p.H, nb);
  switch (dtype) {
    case LA_F32: return launch_t<float>(p, c, stream);
    case LA_BF16: return launch_t<__nv_bfloat16>(p, c, stream);
    case LA_F16: return launch_t<__half>(p, c, stream);
  }
  return LA_ERR_UNSUPPORTED;
}

// --------------------------------------------------------------------------------------------
// log-decay gradient reductions
// --------------------------------------------------------------------------------------------
namespace {

__device__ __forceinline__ float block_sum(float v, float *red) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float s = 0.f;
  for (int i = 0; i < nw; ++i) s += red[i];
  return s;
}

// One CTA per (sequence, head): reverse inclusive scan over tokens.
// Mirrors _compute_dld_cumsum_kernel + _compute_dld_state with sum_option = -1
// (xopes/ops/lightning_attn/log_decay/log_decay_with_cumsum/dld_with_cumsum_triton.py:20-285).
__global__ void __launch_bounds__(256) dld_scalar_kernel(const float *slots_q, int ntq,
                                                         const float *slots_k, int ntk,
                                                         const float *sfin, const float *dsfin,
                                                         const int64_t *cu, float *dld, int B, int N,
                                                         int H, int DE, const float *act_x, int64_t x_sb,
                                                         int64_t x_sn, int64_t x_sh) {
  __shared__ float red[32];
  __shared__ float wsum[8];
  const int h = blockIdx.x, seq = blockIdx.y, tid = threadIdx.x;
  int64_t t_begin = 0, t_end = N, bidx = seq;
  if (cu != nullptr) { t_begin = cu[seq]; t_end = cu[seq + 1]; bidx = 0; }
  float carry = 0.f;
  if (sfin != nullptr && dsfin != nullptr) {
    const int64_t base = ((int64_t)seq * H + h) * DE;
    float s = 0.f;
    for (int i = tid; i < DE; i += blockDim.x) s = fmaf(sfin[base + i], dsfin[base + i], s);
    carry = block_sum(s, red);
  }
  const int64_t slot = (int64_t)B * N * H;
  const int lane = tid & 31, wid = tid >> 5;
  for (int64_t hi = t_end; hi > t_begin; hi -= 256) {
    const int64_t t = hi - 1 - tid;  // thread 0 takes the last token
    float v = 0.f;
    if (t >= t_begin) {
      const int64_t idx = (bidx * N + t) * H + h;
      for (int s = 0; s < ntq; ++s) v += slots_q[s * slot + idx];
      for (int s = 0; s < ntk; ++s) v -= slots_k[s * slot + idx];
    }
    // inclusive scan in thread order (= reverse token order)
    float sc = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, sc, off);
      if (lane >= off) sc += n;
    }
    __syncthreads();
    if (lane == 31) wsum[wid] = sc;
    __syncthreads();
    float pre = carry;
    for (int i = 0; i < wid; ++i) pre += wsum[i];
    if (t >= t_begin) {
      float val = sc + pre;
      // d logsigmoid(x) / dx = sigmoid(-x)
      if (act_x != nullptr) val *= 1.f / (1.f + expf(act_x[bidx * x_sb + t * x_sn + h * x_sh]));
      dld[(bidx * N + t) * H + h] = val;
    }
    float tot = 0.f;
    for (int i = 0; i < 8; ++i) tot += wsum[i];
    carry += tot;
  }
}

// One CTA per (sequence, head): in-place reverse cumulative sum over tokens of every feature f,
// plus the state term (sum_option 0 / 1 of the reference kernel named above), in ONE read and one
// write of the buffer.  The CTA walks the sequence from its end in tiles of lanes x kRcRows tokens;
// group ln of Fpad threads owns kRcRows consecutive tokens of the tile (group 0 the latest), keeps
// them in registers, the groups' sums meet in shared memory, and every thread then writes its
// running sums.  The next tile is loaded before the current one is finished.  With few
// (sequence, head) pairs the features are split over blockIdx.z (Fpad features per CTA, a multiple
// of 32) so that the launch still fills the GPU.
constexpr int kRcRows = 16;

__global__ void __launch_bounds__(512, 2) revcumsum_vec_kernel(float *buf, const float *sfin, const float *dsfin,
                                                             const int64_t *cu, int N, int H, int F, int Fpad,
                                                             int D, int E, int f_is_row, const float *act_x,
                                                             int act_dtype) {
  extern __shared__ float part[];  // [2][lanes][Fpad] + [Fpad]
  const int h = blockIdx.x, seq = blockIdx.y;
  const int lanes = blockDim.x / Fpad;
  const int fl = threadIdx.x % Fpad, ln = threadIdx.x / Fpad;
  const int f = blockIdx.z * Fpad + fl;  // feature of this thread
  int64_t t_begin = 0, t_end = N, bidx = seq;
  if (cu != nullptr) { t_begin = cu[seq]; t_end = cu[seq + 1]; bidx = 0; }
  const int64_t stride = (int64_t)H * F;
  const bool on = f < F;
  const int fc = on ? f : 0;
  float *ptr = buf + ((bidx * N) * H + h) * (int64_t)F + fc;
  // element offset; the pre-activations may be fp32 or 16-bit
  const int64_t xoff = ((bidx * N) * H + h) * (int64_t)F + fc;
  auto xval = [&](int64_t idx) -> float {
    if (act_dtype == LA_F32) return act_x[idx];
    if (act_dtype == LA_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(act_x)[idx]);
    return __half2float(reinterpret_cast<const __half *>(act_x)[idx]);
  };

  // the state term starts the running sum: sum over the other index of final_state * d final_state,
  // formed by the whole CTA with coalesced reads and left in term[Fpad]
  float *term = part + 2 * lanes * Fpad;
  float carry = 0.f;
  if (sfin != nullptr && dsfin != nullptr) {
    const int64_t base = ((int64_t)seq * H + h) * (int64_t)D * E;
    if (f_is_row) {  // a warp per row f: E contiguous elements
      const int lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
      for (int r = threadIdx.x >> 5; r < Fpad; r += nwarps) {
        const int fr = blockIdx.z * Fpad + r;
        float a = 0.f;
        if (fr < F)
          for (int e = lane; e < E; e += 32) a = fmaf(sfin[base + (int64_t)fr * E + e], dsfin[base + (int64_t)fr * E + e], a);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
        if (lane == 0) term[r] = a;
      }
      __syncthreads();
    } else {  // column f: group ln takes rows ln, ln + lanes, ...
      float a = 0.f;
      if (on)
        for (int d = ln; d < D; d += lanes) a = fmaf(sfin[base + (int64_t)d * E + f], dsfin[base + (int64_t)d * E + f], a);
      part[ln * Fpad + fl] = a;
      __syncthreads();
      if (ln == 0) {
        float t = 0.f;
        for (int l = 0; l < lanes; ++l) t += part[l * Fpad + fl];
        term[fl] = t;
      }
      __syncthreads();
    }
    carry = term[fl];
  }

  // token positions are counted from t_begin in 32 bits; this thread's tokens of the tile that ends
  // at position `hi` are hi - 1 - ln kRcRows - i, i = 0 .. kRcRows - 1
  const int len = (int)(t_end - t_begin);
  const int tile = lanes * kRcRows;
  float *base = ptr + t_begin * stride;
  const int64_t xbase = xoff + t_begin * stride;
  auto load = [&](int r0, float (&v)[kRcRows]) {
    const float *pc = base + (int64_t)r0 * stride;
#pragma unroll
    for (int i = 0; i < kRcRows; ++i, pc -= stride) v[i] = (on && r0 - i >= 0) ? *pc : 0.f;
  };
  float cur[kRcRows], nxt[kRcRows];
  if (len > 0) load(len - 1 - ln * kRcRows, cur);
  int phase = 0;
  for (int hi = len; hi > 0; hi -= tile, phase ^= 1) {
    const int r0 = hi - 1 - ln * kRcRows;
    const bool more = hi > tile;
    if (more) load(r0 - tile, nxt);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kRcRows; ++i) s += cur[i];
    float *pp = part + phase * lanes * Fpad;
    pp[ln * Fpad + fl] = s;
    __syncthreads();  // the other buffer is written next, so one barrier per tile is enough
    float run = carry, tot = 0.f;
    for (int l = 0; l < lanes; ++l) {
      const float pv = pp[l * Fpad + fl];
      if (l < ln) run += pv;
      tot += pv;
    }
    carry += tot;
    if (on) {
      float *pc = base + (int64_t)r0 * stride;
      if (act_x == nullptr) {
#pragma unroll
        for (int i = 0; i < kRcRows; ++i, pc -= stride) {
          run += cur[i];
          if (r0 - i >= 0) *pc = run;
        }
      } else {  // d logsigmoid(x) / dx = sigmoid(-x)
        int64_t xc = xbase + (int64_t)r0 * stride;
#pragma unroll
        for (int i = 0; i < kRcRows; ++i, pc -= stride, xc -= stride) {
          run += cur[i];
          if (r0 - i >= 0) *pc = run / (1.f + expf(xval(xc)));
        }
      }
    }
    if (more) {
#pragma unroll
      for (int i = 0; i < kRcRows; ++i) cur[i] = nxt[i];
    }
  }
}

}  // namespace

int launch_dld_scalar(const float *slots_q, int ntq, const float *slots_k, int ntk,
                      const float *final_state, const float *dfinal_state, const int64_t *cu,
                      float *dld, int B, int N, int H, int DE, int M, cudaStream_t stream, const float *act_x,
                      int64_t x_sb, int64_t x_sn, int64_t x_sh) {
  const int nb = cu ? M : B;
  dim3 grid(H, nb);
  dld_scalar_kernel<<<grid, 256, 0, stream>>>(slots_q, ntq, slots_k, ntk, final_state, dfinal_state,
                                              cu, dld, B, N, H, DE, act_x, x_sb, x_sn, x_sh);
  return launch_status();
}

int launch_revcumsum_vec(float *buf, const float *final_state, const float *dfinal_state,
                         const int64_t *cu, int B, int N, int H, int F, int D, int E, int f_is_row,
                         int M, cudaStream_t stream, const float *act_x, int act_dtype) {
  const int nb = cu ? M : B;
  int fpad = ((F + 31) / 32) * 32;
  if (fpad > 1024) return LA_ERR_UNSUPPORTED;
  // two CTAs of 512 threads per SM: split the features while the (sequence, head) pairs alone would
  // leave room in one wave of 296
  int fsplit = 1;
  while (fpad % (2 * 32) == 0 && (int64_t)H * nb * fsplit * 2 <= 296 && fsplit < 8) { fpad /= 2; fsplit *= 2; }
  while (fpad > 512) { fpad = ((fpad / 2 + 31) / 32) * 32; fsplit *= 2; }  // wide features: more CTAs
  dim3 grid(H, nb, fsplit);
  const int lanes = 512 / fpad;
  const size_t smem = sizeof(float) * (2 * (size_t)lanes + 1) * fpad;
  revcumsum_vec_kernel<<<grid, lanes * fpad, smem, stream>>>(buf, final_state, dfinal_state, cu, N, H, F, fpad,
                                                             D, E, f_is_row, act_x, act_dtype);
  return launch_status();
}

// --------------------------------------------------------------------------------------------
// decode: one token, state streamed through once
// --------------------------------------------------------------------------------------------
namespace {

// One CTA (256 threads) per (b,h).  A thread owns one float4 of columns (e) and walks the rows
// (d) with stride 256/(E/4): every warp-wide access covers whole 128-byte lines of the state.
// HBM traffic per (b,h): D*E*4 bytes in, D*E*4 bytes out -- the algorithmic minimum.
template <typename T, int UNROLL>
__global__ void __launch_bounds__(256) decode_kernel(const T *__restrict__ q, const T *__restrict__ k,
                                                     const T *__restrict__ v, const float *ld,
                                                     int64_t ld_sb, int64_t ld_sh, const float *ldk,
                                                     const float *ldv, const float *state_in,
                                                     float *state_out, T *__restrict__ o, int H,
                                                     int D, int E) {
  extern __shared__ __align__(16) float sm[];
  const int tid = threadIdx.x;
  const int bh = blockIdx.x;
  const int b = bh / H, h = bh - b * H;
  const int ncol4 = E >> 2;
  const int col4 = tid % ncol4;
  const int r0 = tid / ncol4;
  const int rstep = 256 / ncol4;
  float *red = sm;                // [rstep][E], first so that it stays 16-byte aligned
  float *q_s = red + rstep * E;   // [D]
  float *k_s = q_s + D;           // [D]
  float *dk_s = k_s + D;          // [D] row decay factor (includes the scalar decay)

  float lam = 1.f;
  if (ld != nullptr) lam = (float)exp((double)ld[b * ld_sb + h * ld_sh]);
  for (int d = tid; d < D; d += 256) {
    q_s[d] = Cvt<T>::to_f(q[(int64_t)bh * D + d]);
    k_s[d] = Cvt<T>::to_f(k[(int64_t)bh * D + d]);
    dk_s[d] = lam * (ldk != nullptr ? expf(ldk[(int64_t)bh * D + d]) : 1.f);
  }
  float4 vv, dv = make_float4(1.f, 1.f, 1.f, 1.f);
  {
    const T *vp = v + (int64_t)bh * E + col4 * 4;
    vv = make_float4(Cvt<T>::to_f(vp[0]), Cvt<T>::to_f(vp[1]), Cvt<T>::to_f(vp[2]), Cvt<T>::to_f(vp[3]));
    if (ldv != nullptr) {
      const float4 l = ld4(ldv + (int64_t)bh * E + col4 * 4);
      dv = make_float4(expf(l.x), expf(l.y), expf(l.z), expf(l.w));
    }
  }
  __syncthreads();

  const float4 *sin4 = reinterpret_cast<const float4 *>(state_in + (int64_t)bh * D * E);
  float4 *sout4 = reinterpret_cast<float4 *>(state_out + (int64_t)bh * D * E);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int d0 = r0; d0 < D; d0 += rstep * UNROLL) {
    float4 s[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int d = d0 + u * rstep;
      if (d < D) s[u] = __ldcs(sin4 + (int64_t)d * ncol4 + col4);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int d = d0 + u * rstep;
      if (d < D) {
        const float f = dk_s[d], kd = k_s[d], qd = q_s[d];
        float4 n;
        n.x = fmaf(s[u].x, f * dv.x, kd * vv.x);
        n.y = fmaf(s[u].y, f * dv.y, kd * vv.y);
        n.z = fmaf(s[u].z, f * dv.z, kd * vv.z);
        n.w = fmaf(s[u].w, f * dv.w, kd * vv.w);
        __stcs(sout4 + (int64_t)d * ncol4 + col4, n);
        acc.x = fmaf(qd, n.x, acc.x);
        acc.y = fmaf(qd, n.y, acc.y);
        acc.z = fmaf(qd, n.z, acc.z);
        acc.w = fmaf(qd, n.w, acc.w);
      }
    }
  }
  reinterpret_cast<float4 *>(red)[r0 * ncol4 + col4] = acc;
  __syncthreads();
  for (int e = tid; e < E; e += 256) {
    float s = 0.f;
    for (int r = 0; r < rstep; ++r) s += red[r * E + e];
    o[(int64_t)bh * E + e] = Cvt<T>::from_f(s);
  }
}

template <typename T>
int launch_decode_t(const void *q, const void *k, const void *v, const float *ld, int64_t ld_sb,
                    int64_t ld_sh, const float *ldk, const float *ldv, const float *state_in,
                    float *state_out, void *o, int B, int H, int D, int E, cudaStream_t stream) {
  const int ncol4 = E / 4;
  const int rstep = 256 / ncol4;
  const size_t smem = sizeof(float) * (3 * (size_t)D + (size_t)rstep * E);
  decode_kernel<T, 8><<<B * H, 256, smem, stream>>>(
      static_cast<const T *>(q), static_cast<const T *>(k), static_cast<const T *>(v), ld, ld_sb,
      ld_sh, ldk, ldv, state_in, state_out, static_cast<T *>(o), H, D, E);
  return launch_status();
}

}  // namespace

int launch_decode(const void *q, const void *k, const void *v, const float *ld, int64_t ld_sb,
                  int64_t ld_sh, const float *ldk, const float *ldv, const float *state_in,
                  float *state_out, void *o, int B, int H, int D, int E, int dtype,
                  cudaStream_t stream) {
  // vectorised layout needs E = 4 * 2^m with 256 % (E/4) == 0, and 16-byte aligned state rows
  const int ncol4 = E / 4;
  if (E % 4 != 0 || ncol4 < 1 || ncol4 > 256 || (256 % ncol4) != 0) return LA_ERR_UNSUPPORTED;
  if (D > 4096) return LA_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(state_in) | reinterpret_cast<uintptr_t>(state_out) |
       reinterpret_cast<uintptr_t>(ldv)) & 15u)
    return LA_ERR_MISALIGNED;
  switch (dtype) {
    case LA_F32: return launch_decode_t<float>(q, k, v, ld, ld_sb, ld_sh, ldk, ldv, state_in, state_out, o, B, H, D, E, stream);
    case LA_BF16: return launch_decode_t<__nv_bfloat16>(q, k, v, ld, ld_sb, ld_sh, ldk, ldv, state_in, state_out, o, B, H, D, E, stream);
    case LA_F16: return launch_decode_t<__half>(q, k, v, ld, ld_sb, ld_sh, ldk, ldv, state_in, state_out, o, B, H, D, E, stream);
  }
  return LA_ERR_UNSUPPORTED;
}

}  // namespace la
