// Fused normalisation + gate: the op that follows lightning attention in a model block
// (xopes/ops/normalize/normalize/normalize_torch.py:9-111, the gate branch):
//
//   a  = act(gate)                                   act in {none, relu, sigmoid, silu}
//   z  = x (.) a   (gate_pos = pre)   or   x         per group of e features (a head):
//   zc = z - mean(z)  (use_mean)      or   z
//   y  = c zc / sqrt(sum zc^2 + eps) (.) weight + bias
//   o  = y            (gate_pos = pre, or no gate)   or   y (.) a   (gate_pos = post)
//
// One pass over x and gate in, o out (forward), and one pass over x, gate, do in, dx, dgate out
// (backward), all arithmetic in fp32: pure HBM streaming, 3 x 2e bytes per group forward.  One warp
// owns one (row, group) at a time, a lane owns e / 32 elements as packs of 4; a warp walks rows of
// ONE group, so the weight / bias gradients accumulate in registers and leave with one atomicAdd
// per lane and element at the end.
#include "common.cuh"

namespace la {
namespace {

constexpr int kMaxPerLane = 16;  // e <= 512

enum { kActNone = 0, kActRelu = 1, kActSigmoid = 2, kActSilu = 3 };

__device__ __forceinline__ float act_f(float g, int act) {
  switch (act) {
    case kActRelu: return fmaxf(g, 0.f);
    case kActSigmoid: return 1.f / (1.f + __expf(-g));
    case kActSilu: return g / (1.f + __expf(-g));
  }
  return g;
}
// derivative of the activation at g
__device__ __forceinline__ float act_grad(float g, int act) {
  switch (act) {
    case kActRelu: return g >= 0.f ? 1.f : 0.f;
    case kActSigmoid: {
      const float s = 1.f / (1.f + __expf(-g));
      return s * (1.f - s);
    }
    case kActSilu: {
      const float s = 1.f / (1.f + __expf(-g));
      return s * (1.f + g * (1.f - s));
    }
  }
  return 1.f;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

struct NormArgs {
  const void *x, *gate;
  const float *weight, *bias;  // (G * e) fp32 or null
  void *out;
  const void *d_out;
  void *dx, *dgate;
  float *dweight, *dbias;      // (G * e) fp32 accumulators (zeroed by the caller) or null
  long long rows;
  int G, e, act, post, use_mean;
  float c, eps;
};

// Loads this lane's elements of one group: element j of the lane is feature lane * 4 + (j / 4) * 128 + j % 4.
template <typename T, int N>
__device__ __forceinline__ void load_lane(const T *p, int e, int lane, float (&v)[N]) {
#pragma unroll
  for (int j = 0; j < N; j += 4) {
    {
      const int f = lane * 4 + (j >> 2) * 128;
      if (f < e) {
        if (sizeof(T) == 2) {
          const uint2 u = *reinterpret_cast<const uint2 *>(p + f);
          const T *h = reinterpret_cast<const T *>(&u);
          v[j] = Cvt<T>::to_f(h[0]); v[j + 1] = Cvt<T>::to_f(h[1]); v[j + 2] = Cvt<T>::to_f(h[2]); v[j + 3] = Cvt<T>::to_f(h[3]);
        } else {
          const float4 u = *reinterpret_cast<const float4 *>(p + f);
          v[j] = u.x; v[j + 1] = u.y; v[j + 2] = u.z; v[j + 3] = u.w;
        }
      } else {
        v[j] = v[j + 1] = v[j + 2] = v[j + 3] = 0.f;
      }
    }
  }
}
template <typename T, int N>
__device__ __forceinline__ void store_lane(T *p, int e, int lane, const float (&v)[N]) {
#pragma unroll
  for (int j = 0; j < N; j += 4) {
    {
      const int f = lane * 4 + (j >> 2) * 128;
      if (f < e) {
        if (sizeof(T) == 2) {
          T h[4] = {Cvt<T>::from_f(v[j]), Cvt<T>::from_f(v[j + 1]), Cvt<T>::from_f(v[j + 2]), Cvt<T>::from_f(v[j + 3])};
          *reinterpret_cast<uint2 *>(p + f) = *reinterpret_cast<const uint2 *>(h);
        } else {
          *reinterpret_cast<float4 *>(p + f) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        }
      }
    }
  }
}

// grid (blocks over rows, G); a warp takes rows blockIdx.x * warps + warp, then strides.
// N = elements per lane = 4 * ceil(e / 128).
template <typename T, bool BWD, int N>
__global__ void __launch_bounds__(256) norm_gate_kernel(const NormArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int g = blockIdx.y, e = a.e;
  const long long stride = (long long)a.G * e;
  const bool has_gate = a.gate != nullptr;
  float w[N], b[N], dw[N], db[N];
#pragma unroll
  for (int j = 0; j < N; ++j) { w[j] = 1.f; b[j] = 0.f; dw[j] = 0.f; db[j] = 0.f; }
  if (a.weight != nullptr) load_lane<float, N>(a.weight + (long long)g * e, e, lane, w);
  if (a.bias != nullptr) load_lane<float, N>(a.bias + (long long)g * e, e, lane, b);
  const float inv_e = 1.f / (float)e;

  for (long long r = (long long)blockIdx.x * warps + warp; r < a.rows; r += (long long)gridDim.x * warps) {
    const long long off = r * stride + (long long)g * e;
    float x[N], gt[N], act[N], z[N];
    load_lane<T, N>(static_cast<const T *>(a.x) + off, e, lane, x);
    if (has_gate) load_lane<T, N>(static_cast<const T *>(a.gate) + off, e, lane, gt);
    float s1 = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) {
      {
        act[j] = has_gate ? act_f(gt[j], a.act) : 1.f;
        z[j] = (has_gate && !a.post) ? x[j] * act[j] : x[j];
        s1 += z[j];
      }
    }
    float mean = 0.f;
    if (a.use_mean) mean = warp_sum(s1) * inv_e;
    float s2 = 0.f;
#pragma unroll
    for (int j = 0; j < N; ++j) {
      {
        const int f = lane * 4 + (j >> 2) * 128 + (j & 3);
        z[j] = f < e ? z[j] - mean : 0.f;  // zc
        s2 += z[j] * z[j];
      }
    }
    const float rsig = rsqrtf(warp_sum(s2) + a.eps);
    if (!BWD) {
      float o[N];
#pragma unroll
      for (int j = 0; j < N; ++j) {
        {
          const float y = a.c * z[j] * rsig * w[j] + b[j];
          o[j] = (has_gate && a.post) ? y * act[j] : y;
        }
      }
      store_lane<T, N>(static_cast<T *>(a.out) + off, e, lane, o);
    } else {
      float d_o[N], dxh[N], dga[N];
      load_lane<T, N>(static_cast<const T *>(a.d_out) + off, e, lane, d_o);
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < N; ++j) {
        {
          const float xh = z[j] * rsig;                    // normalised value
          const float y = a.c * xh * w[j] + b[j];
          const float dy = (has_gate && a.post) ? d_o[j] * act[j] : d_o[j];
          dga[j] = (has_gate && a.post) ? d_o[j] * y : 0.f;  // d loss / d act(gate), post-gate part
          dw[j] += dy * a.c * xh;
          db[j] += dy;
          dxh[j] = dy * w[j] * a.c;
          dot += dxh[j] * xh;
        }
      }
      dot = warp_sum(dot);
      float s3 = 0.f;
#pragma unroll
      for (int j = 0; j < N; ++j) {
        {
          const int f = lane * 4 + (j >> 2) * 128 + (j & 3);
          const float xh = z[j] * rsig;
          dxh[j] = f < e ? (dxh[j] - xh * dot) * rsig : 0.f;  // d loss / d zc
          s3 += dxh[j];
        }
      }
      float dmean = 0.f;
      if (a.use_mean) dmean = warp_sum(s3) * inv_e;
      float gx[N], gg[N];
#pragma unroll
      for (int j = 0; j < N; ++j) {
        {
          const float dz = dxh[j] - dmean;                 // d loss / d z
          if (has_gate && !a.post) {
            gx[j] = dz * act[j];
            dga[j] = dz * x[j];
          } else {
            gx[j] = dz;
          }
          gg[j] = has_gate ? dga[j] * act_grad(gt[j], a.act) : 0.f;
        }
      }
      store_lane<T, N>(static_cast<T *>(a.dx) + off, e, lane, gx);
      if (has_gate) store_lane<T, N>(static_cast<T *>(a.dgate) + off, e, lane, gg);
    }
  }
  if (BWD) {
#pragma unroll
    for (int j = 0; j < N; ++j) {
      {
        const int f = lane * 4 + (j >> 2) * 128 + (j & 3);
        if (f < e) {
          if (a.dweight != nullptr) atomicAdd(a.dweight + (long long)g * e + f, dw[j]);
          if (a.dbias != nullptr) atomicAdd(a.dbias + (long long)g * e + f, db[j]);
        }
      }
    }
  }
}

template <typename T>
int launch_t(const NormArgs &a, bool bwd, cudaStream_t st) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return LA_ERR_CUDA;
  const int warps = 8;
  long long blocks = (a.rows + warps - 1) / warps;
  // enough CTAs to fill the GPU several times over, few enough that the per-warp gradient
  // accumulators are flushed rarely
  const long long cap = (long long)sms * 8 / (a.G > 0 ? (a.G < 8 ? a.G : 8) : 1) + 1;
  if (blocks > cap) blocks = cap;
  dim3 grid((unsigned)blocks, (unsigned)a.G);
  const int n = ((a.e + 127) / 128) * 4;
#define LA_NORM_LAUNCH(NN)                                                            \
  do {                                                                                \
    if (bwd) norm_gate_kernel<T, true, NN><<<grid, warps * 32, 0, st>>>(a);           \
    else norm_gate_kernel<T, false, NN><<<grid, warps * 32, 0, st>>>(a);              \
  } while (0)
  if (n <= 4) LA_NORM_LAUNCH(4);
  else if (n <= 8) LA_NORM_LAUNCH(8);
  else LA_NORM_LAUNCH(16);
#undef LA_NORM_LAUNCH
  return launch_status();
}

int dispatch(const NormArgs &a, int dtype, bool bwd, cudaStream_t st) {
  switch (dtype) {
    case LA_F32: return launch_t<float>(a, bwd, st);
    case LA_BF16: return launch_t<__nv_bfloat16>(a, bwd, st);
    case LA_F16: return launch_t<__half>(a, bwd, st);
  }
  return LA_ERR_UNSUPPORTED;
}

int check(const void *x, int64_t rows, int64_t G, int64_t e, int dtype, int act, int gate_pos) {
  cudaGetLastError();
  if (x == nullptr) return LA_ERR_NULL_POINTER;
  if (rows <= 0 || G <= 0 || e <= 0) return LA_ERR_BAD_SHAPE;
  if (e % 4 != 0 || e > 32 * kMaxPerLane || G > 65535) return LA_ERR_UNSUPPORTED;
  if (act < 0 || act > 3 || gate_pos < 0 || gate_pos > 1) return LA_ERR_UNSUPPORTED;
  if (!(dtype == LA_F32 || dtype == LA_BF16 || dtype == LA_F16)) return LA_ERR_UNSUPPORTED;
  return LA_OK;
}

}  // namespace
}  // namespace la

using namespace la;

extern "C" {

int la_normalize_gate_fwd(const void *x, const void *gate, const float *weight, const float *bias, void *out,
                          int64_t rows, int64_t G, int64_t e, int dtype, int act, int gate_pos, float c, float eps,
                          int use_mean, void *stream) {
  const int rc = check(x, rows, G, e, dtype, act, gate_pos);
  if (rc != LA_OK) return rc;
  if (out == nullptr) return LA_ERR_NULL_POINTER;
  NormArgs a = {};
  a.x = x; a.gate = gate; a.weight = weight; a.bias = bias; a.out = out;
  a.rows = rows; a.G = (int)G; a.e = (int)e; a.act = act; a.post = gate_pos; a.use_mean = use_mean;
  a.c = c; a.eps = eps;
  return dispatch(a, dtype, false, static_cast<cudaStream_t>(stream));
}

int la_normalize_gate_bwd(const void *x, const void *gate, const float *weight, const float *bias, const void *d_out,
                          void *dx, void *dgate, float *dweight, float *dbias, int64_t rows, int64_t G, int64_t e,
                          int dtype, int act, int gate_pos, float c, float eps, int use_mean, void *stream) {
  const int rc = check(x, rows, G, e, dtype, act, gate_pos);
  if (rc != LA_OK) return rc;
  if (d_out == nullptr || dx == nullptr || (gate != nullptr && dgate == nullptr)) return LA_ERR_NULL_POINTER;
  NormArgs a = {};
  a.x = x; a.gate = gate; a.weight = weight; a.bias = bias; a.d_out = d_out; a.dx = dx; a.dgate = dgate;
  a.dweight = dweight; a.dbias = dbias;
  a.rows = rows; a.G = (int)G; a.e = (int)e; a.act = act; a.post = gate_pos; a.use_mean = use_mean;
  a.c = c; a.eps = eps;
  return dispatch(a, dtype, true, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
