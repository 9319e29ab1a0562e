// Max-pooling of a channels-last activation, forward and backward.
//
// The reference's leaves (python/gtl/compiler/passes/pass_decomposition.py:109-132,
// max_pool2d_with_indices_channel_last / ..._backward_channel_last) permute to NCHW and call the
// library, which keeps one int64 index per output element -- at the ResNet stem (128 x 56 x 56 x 64
// outputs) that is 205 MB written in the forward pass and read in the backward pass, more than the
// activation itself.  Here the position of the maximum inside its window is one byte (r * k + t), a
// thread owns 8 channels of one position (16-byte accesses), and the backward pass gathers: every input
// position sums the gradients of the (at most ceil(k/s)^2) windows that cover it and chose it.  Ties go
// to the first maximum in window scan order and a NaN wins, as in the library's kernel, so outputs and
// chosen positions are the same.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <string>

#include "../../include/evt_b200.h"
#include "evtb_internal.h"
#include "epilogue_ops.cuh"

namespace evtb {

constexpr int kPoolThreads = 256;

struct PoolGeom {
  int N, H, W, C, P, Q, k, s, pad, kv;
};

// Window size and stride as template arguments for the common cases (0 = read from the geometry): the
// window loops unroll and the backward pass divides by a constant.  Index arithmetic avoids divisions by
// run-time values (3-D grid: x over the vectors of one row, y = row, z = image; channel vectors per pixel
// are split off with a shift when their count is a power of two): with them the backward pass executed
// 430 instructions per 16-byte result and ran at 15 % of the HBM rate.
template <int K, int S>
struct PoolKS {
  const int k, s;
  __device__ __forceinline__ explicit PoolKS(const PoolGeom& g) : k(K ? K : g.k), s(S ? S : g.s) {}
};

__device__ __forceinline__ void pool_split(const PoolGeom& g, int i, int& pixel, int& cv) {
  if ((g.kv & (g.kv - 1)) == 0) {
    cv = i & (g.kv - 1);
    pixel = i >> (31 - __clz(g.kv));
  } else {
    cv = i % g.kv;
    pixel = i / g.kv;
  }
}

// grid: x over Q * kv vectors of one output row, y = ph, z = n
template <typename T, int K, int S>
__global__ void __launch_bounds__(kPoolThreads)
maxpool_forward_kernel(const T* __restrict__ x, T* __restrict__ y, uint8_t* __restrict__ code, PoolGeom g) {
  const PoolKS<K, S> ks(g);
  const int i = blockIdx.x * kPoolThreads + threadIdx.x;
  if (i >= g.Q * g.kv) return;
  int cv, pw;
  pool_split(g, i, pw, cv);
  const int ph = blockIdx.y, n = blockIdx.z;
  const int h0 = ph * ks.s - g.pad, w0 = pw * ks.s - g.pad;
  float m[8];
  int best[8];
  const int r_first = h0 < 0 ? -h0 : 0, t_first = w0 < 0 ? -w0 : 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    m[j] = -INFINITY;
    best[j] = r_first * ks.k + t_first;
  }
  const T* base = x + ((static_cast<long long>(n) * g.H) * g.W) * g.C + cv * 8;
#pragma unroll
  for (int r = 0; r < (K ? K : 15); ++r) {
    if (r >= ks.k) break;
    const int h = h0 + r;
    if (h < 0 || h >= g.H) continue;
    const T* row = base + static_cast<long long>(h) * g.W * g.C;
#pragma unroll
    for (int t = 0; t < (K ? K : 15); ++t) {
      if (t >= ks.k) break;
      const int w = w0 + t;
      if (w < 0 || w >= g.W) continue;
      float v[8];
      Vec8<T>::load(row + static_cast<long long>(w) * g.C, true, v);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (v[j] > m[j] || v[j] != v[j]) {
          m[j] = v[j];
          best[j] = r * ks.k + t;
        }
    }
  }
  const long long o = (((static_cast<long long>(n) * g.P + ph) * g.Q + pw) * g.kv + cv) * 8;
  Vec8<T>::store(y + o, true, m);
  uint2 packed;
  uint8_t* b = reinterpret_cast<uint8_t*>(&packed);
#pragma unroll
  for (int j = 0; j < 8; ++j) b[j] = static_cast<uint8_t>(best[j]);
  *reinterpret_cast<uint2*>(code + o) = packed;
}

// grid: x over W * kv vectors of one input row, y = h, z = n
template <typename T, int K, int S>
__global__ void __launch_bounds__(kPoolThreads)
maxpool_backward_kernel(const T* __restrict__ dy, const uint8_t* __restrict__ code, T* __restrict__ dx, PoolGeom g) {
  const PoolKS<K, S> ks(g);
  const int i = blockIdx.x * kPoolThreads + threadIdx.x;
  if (i >= g.W * g.kv) return;
  int cv, w;
  pool_split(g, i, w, cv);
  const int h = blockIdx.y, n = blockIdx.z;
  // windows ph with ph * s - pad <= h <= ph * s - pad + k - 1
  const int hp = h + g.pad, wp = w + g.pad;
  int ph0 = hp - ks.k + 1;
  ph0 = ph0 > 0 ? (ph0 + ks.s - 1) / ks.s : 0;
  int ph1 = hp / ks.s;
  if (ph1 > g.P - 1) ph1 = g.P - 1;
  int pw0 = wp - ks.k + 1;
  pw0 = pw0 > 0 ? (pw0 + ks.s - 1) / ks.s : 0;
  int pw1 = wp / ks.s;
  if (pw1 > g.Q - 1) pw1 = g.Q - 1;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  for (int ph = ph0; ph <= ph1; ++ph) {
    const int r = hp - ph * ks.s;
    for (int pw = pw0; pw <= pw1; ++pw) {
      const int mine = r * ks.k + (wp - pw * ks.s);
      const long long o = (((static_cast<long long>(n) * g.P + ph) * g.Q + pw) * g.kv + cv) * 8;
      const uint2 packed = __ldg(reinterpret_cast<const uint2*>(code + o));
      // the eight one-byte places against this position's place, four at a time (0xff per equal byte);
      // most windows chose another position: their gradients are not even loaded
      const unsigned want = static_cast<unsigned>(mine) * 0x01010101u;
      const unsigned eq_lo = __vcmpeq4(packed.x, want), eq_hi = __vcmpeq4(packed.y, want);
      if ((eq_lo | eq_hi) == 0u) continue;
      float v[8];
      Vec8<T>::load(dy + o, true, v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if ((eq_lo >> (8 * j)) & 1u) acc[j] += v[j];          // fp32 sums, as the library's kernel
        if ((eq_hi >> (8 * j)) & 1u) acc[4 + j] += v[4 + j];
      }
    }
  }
  Vec8<T>::store(dx + (((static_cast<long long>(n) * g.H + h) * g.W + w) * g.kv + cv) * 8, true, acc);
}

static int pool_geom(const char* who, int32_t dtype, int64_t N, int64_t H, int64_t W, int64_t C, int32_t k, int32_t stride,
                     int32_t pad, PoolGeom* g) {
  if (dtype != EVTB_F16 && dtype != EVTB_BF16) {
    set_last_error(std::string(who) + ": activations must be fp16 or bf16");
    return EVTB_EINVAL;
  }
  if (N <= 0 || H <= 0 || W <= 0 || C <= 0 || C % 8 != 0 || k < 1 || k > 15 || stride < 1 || pad < 0 || 2 * pad > k ||
      W * C > 0x7fffffffLL || N > 65535 || H > 65535) {
    set_last_error(std::string(who) + ": needs C % 8 == 0, 1 <= kernel <= 15, stride >= 1, 0 <= 2 * padding <= kernel");
    return EVTB_EINVAL;
  }
  g->N = static_cast<int>(N); g->H = static_cast<int>(H); g->W = static_cast<int>(W); g->C = static_cast<int>(C);
  g->k = k; g->s = stride; g->pad = pad; g->kv = g->C / 8;
  g->P = (g->H + 2 * pad - k) / stride + 1;
  g->Q = (g->W + 2 * pad - k) / stride + 1;
  if (g->P < 1 || g->Q < 1) {
    set_last_error(std::string(who) + ": the window does not fit the padded image");
    return EVTB_EINVAL;
  }
  return EVTB_OK;
}

}  // namespace evtb

extern "C" {

int evtb_maxpool_forward(const void* x, int32_t dtype, int64_t N, int64_t H, int64_t W, int64_t C, int32_t kernel,
                         int32_t stride, int32_t padding, void* y, uint8_t* code, evtb_stream stream) {
  evtb::PoolGeom g;
  if (const int st = evtb::pool_geom("evtb_maxpool_forward", dtype, N, H, W, C, kernel, stride, padding, &g)) return st;
  if (x == nullptr || y == nullptr || code == nullptr || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(code) & 7u) != 0) {
    evtb::set_last_error("evtb_maxpool_forward: null pointer, or x / y not 16-byte (code not 8-byte) aligned");
    return EVTB_EINVAL;
  }
  if (g.P > 65535 || g.N > 65535) return EVTB_ETOOLARGE;
  const dim3 grid((g.Q * g.kv + evtb::kPoolThreads - 1) / evtb::kPoolThreads, static_cast<unsigned>(g.P), static_cast<unsigned>(g.N));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define EVTB_POOL_FWD(T, K, S) evtb::maxpool_forward_kernel<T, K, S><<<grid, evtb::kPoolThreads, 0, s>>>( \
      static_cast<const T*>(x), static_cast<T*>(y), code, g)
#define EVTB_POOL_FWD_KS(T)                                   \
  if (kernel == 3 && stride == 2) EVTB_POOL_FWD(T, 3, 2);     \
  else if (kernel == 3 && stride == 1) EVTB_POOL_FWD(T, 3, 1); \
  else if (kernel == 2 && stride == 2) EVTB_POOL_FWD(T, 2, 2); \
  else EVTB_POOL_FWD(T, 0, 0)
  if (dtype == EVTB_F16) { EVTB_POOL_FWD_KS(__half); } else { EVTB_POOL_FWD_KS(__nv_bfloat16); }
#undef EVTB_POOL_FWD_KS
#undef EVTB_POOL_FWD
  return cudaGetLastError() == cudaSuccess ? EVTB_OK : EVTB_ECUDA;
}

int evtb_maxpool_backward(const void* dy, const uint8_t* code, int32_t dtype, int64_t N, int64_t H, int64_t W, int64_t C,
                          int32_t kernel, int32_t stride, int32_t padding, void* dx, evtb_stream stream) {
  evtb::PoolGeom g;
  if (const int st = evtb::pool_geom("evtb_maxpool_backward", dtype, N, H, W, C, kernel, stride, padding, &g)) return st;
  if (dy == nullptr || dx == nullptr || code == nullptr || ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(code) & 7u) != 0) {
    evtb::set_last_error("evtb_maxpool_backward: null pointer, or dy / dx not 16-byte (code not 8-byte) aligned");
    return EVTB_EINVAL;
  }
  if (g.H > 65535 || g.N > 65535) return EVTB_ETOOLARGE;
  const dim3 grid((g.W * g.kv + evtb::kPoolThreads - 1) / evtb::kPoolThreads, static_cast<unsigned>(g.H), static_cast<unsigned>(g.N));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define EVTB_POOL_BWD(T, K, S) evtb::maxpool_backward_kernel<T, K, S><<<grid, evtb::kPoolThreads, 0, s>>>( \
      static_cast<const T*>(dy), code, static_cast<T*>(dx), g)
#define EVTB_POOL_BWD_KS(T)                                   \
  if (kernel == 3 && stride == 2) EVTB_POOL_BWD(T, 3, 2);     \
  else if (kernel == 3 && stride == 1) EVTB_POOL_BWD(T, 3, 1); \
  else if (kernel == 2 && stride == 2) EVTB_POOL_BWD(T, 2, 2); \
  else EVTB_POOL_BWD(T, 0, 0)
  if (dtype == EVTB_F16) { EVTB_POOL_BWD_KS(__half); } else { EVTB_POOL_BWD_KS(__nv_bfloat16); }
#undef EVTB_POOL_BWD_KS
#undef EVTB_POOL_BWD
  return cudaGetLastError() == cudaSuccess ? EVTB_OK : EVTB_ECUDA;
}

}  // extern "C"
