// Batch-norm passes of a channels-last training step that are not part of a convolution epilogue.
//
// The reference splits training-mode batch norm into four leaves
// (python/gtl/compiler/passes/pass_decomposition.py:135-189): batch_norm_stat (fused into the
// producing convolution's epilogue, evt_fuser.py:1272-1284), batch_norm_elemt,
// batch_norm_backward_stat and batch_norm_backward_elemt.  The last three are one pass each over a
// [rows, channels] activation (rows = N*H*W): HBM-bound, 16-byte accesses, every per-channel
// quantity folded into two or three coefficients that a CTA keeps in shared memory.  The ReLU that
// follows a batch norm, the residual addition of a bottleneck block and the ReLU mask / gradient
// addition in front of the backward statistics ride along in the same pass.
//
//  evtb_bn_apply            z = act(y * scale + shift [+ residual]),
//                           scale = gamma * rstd, shift = beta - mean * scale,
//                           rstd = rsqrt(E[y^2] - E[y]^2 + eps)
//  evtb_bn_backward_reduce  g' = (g [+ g2]) [* (act > 0)];  sums[c] += sum_r g',
//                           sums[C + c] += sum_r g' * (y - mean) * rstd        (fp32 atomics)
//  evtb_bn_backward_apply   dy = (g - mean_g - x_hat * mean_gx) * gamma * rstd
//                              = a * g + c1 * y + c0   with a = gamma * rstd,
//                                c1 = -a * rstd * mean_gx, c0 = -a * mean_g - c1 * mean
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "../../include/evt_b200.h"
#include "evtb_internal.h"
#include "epilogue_ops.cuh"
#include "sm100_ptx.cuh"

namespace evtb {

constexpr int kBnThreads = 256;
constexpr int kBnMaxChannels = 4096;     // 3 floats per channel in shared memory = 48 KB
constexpr int kBnUnroll = 4;             // independent 16-byte loads in flight per thread and operand

template <typename T> __device__ __forceinline__ float round_through(float v);
template <> __device__ __forceinline__ float round_through<__half>(float v) { return __half2float(__float2half_rn(v)); }
template <> __device__ __forceinline__ float round_through<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// --------------------------------------------------------------------------------------------
// forward apply
template <typename T, bool RELU, bool RES>
__global__ void __launch_bounds__(kBnThreads)
bn_apply_kernel(const T* __restrict__ y, const float* __restrict__ mean_in, const float* __restrict__ meansq_in,
                const T* __restrict__ gamma, const T* __restrict__ beta, float eps, const T* __restrict__ res,
                T* __restrict__ z, float* __restrict__ saved_mean, float* __restrict__ saved_rstd, long long nvec, int kv) {
  // (scale, shift) of channel c at [c % 8][c / 8]: the lanes of a warp work on consecutive 8-channel
  // vectors, so for each of a vector's 8 channels they read consecutive words (no bank conflicts;
  // channel-major order would put all lanes on two banks)
  extern __shared__ float2 bn_ss[];
  const int C = kv * 8;
  for (int c = threadIdx.x; c < C; c += kBnThreads) {
    const float m = mean_in[c];
    const float r = rsqrtf(fmaxf(meansq_in[c] - m * m, 0.f) + eps);
    const float sc = Vec8<T>::load1(gamma + c) * r;
    bn_ss[(c & 7) * kv + (c >> 3)] = make_float2(sc, Vec8<T>::load1(beta + c) - m * sc);
    if (blockIdx.x == 0) {
      if (saved_mean != nullptr) saved_mean[c] = m;
      if (saved_rstd != nullptr) saved_rstd[c] = r;
    }
  }
  __syncthreads();
  const long long stride = static_cast<long long>(gridDim.x) * kBnThreads;
  const long long first = static_cast<long long>(blockIdx.x) * kBnThreads + threadIdx.x;
  const int sv = static_cast<int>(stride % kv);        // channel-vector step between this thread's items
  int cv0 = static_cast<int>(first % kv);
  for (long long i0 = first; i0 < nvec; i0 += stride * kBnUnroll, cv0 = (cv0 + kBnUnroll * sv) % kv) {
    float v[kBnUnroll][8], r[kBnUnroll][8];
#pragma unroll
    for (int u = 0; u < kBnUnroll; ++u) {
      const long long i = i0 + u * stride;
      Vec8<T>::load(y + i * 8, i < nvec, v[u]);
      if (RES) Vec8<T>::load(res + i * 8, i < nvec, r[u]);
    }
#pragma unroll
    for (int u = 0; u < kBnUnroll; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) break;
      const float2* ss = bn_ss + (cv0 + u * sv) % kv;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 c = ss[j * kv];
        float o = fmaf(v[u][j], c.x, c.y);
        if (RES) o += r[u][j];
        if (RELU) o = fmaxf(o, 0.f);
        v[u][j] = o;
      }
      Vec8<T>::store(z + i * 8, true, v[u]);
    }
  }
}

// --------------------------------------------------------------------------------------------
// backward statistics: thread = (row lane, 8 channels); a CTA walks its chunk of rows
template <typename T, bool MASK, bool ADD, bool STORE>
__global__ void __launch_bounds__(kBnThreads)
bn_backward_reduce_kernel(const T* __restrict__ g, const T* __restrict__ g2, const T* __restrict__ act,
                          const T* __restrict__ y, const float* __restrict__ mean, const float* __restrict__ rstd,
                          T* __restrict__ gout, float* __restrict__ sums, int rows, int kv, int kvb, int rows_per_chunk) {
  __shared__ float red[kBnThreads][17];
  const int rpp = kBnThreads / kvb;                     // rows per pass
  const int lane_r = threadIdx.x / kvb;
  const int cv = blockIdx.y * kvb + threadIdx.x % kvb;   // channel vector of this thread
  const bool active = lane_r < rpp && cv < kv;
  const int C = kv * 8;
  float m[8], rs[8], s[8], sx[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    m[j] = active ? mean[cv * 8 + j] : 0.f;
    rs[j] = active ? rstd[cv * 8 + j] : 0.f;
    s[j] = 0.f;
    sx[j] = 0.f;
  }
  const int r0 = blockIdx.x * rows_per_chunk;
  const int r1 = min(rows, r0 + rows_per_chunk);
  if (active) {
    for (int rb = r0 + lane_r; rb < r1; rb += rpp * kBnUnroll) {
      float vg[kBnUnroll][8], vy[kBnUnroll][8], va[kBnUnroll][8], v2[kBnUnroll][8];
#pragma unroll
      for (int u = 0; u < kBnUnroll; ++u) {
        const int r = rb + u * rpp;
        const long long off = (static_cast<long long>(r) * kv + cv) * 8;
        const bool ok = r < r1;
        Vec8<T>::load(g + off, ok, vg[u]);
        Vec8<T>::load(y + off, ok, vy[u]);
        if (MASK) Vec8<T>::load(act + off, ok, va[u]);
        if (ADD) Vec8<T>::load(g2 + off, ok, v2[u]);
      }
#pragma unroll
      for (int u = 0; u < kBnUnroll; ++u) {
        const int r = rb + u * rpp;
        if (r >= r1) break;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float gv = vg[u][j];
          if (ADD) gv += v2[u][j];
          if (MASK) gv = va[u][j] > 0.f ? gv : 0.f;
          vg[u][j] = gv;
        }
        if (STORE) {
          Vec8<T>::store(gout + (static_cast<long long>(r) * kv + cv) * 8, true, vg[u]);
          // the consumer reads the rounded gradient: the sums are taken over what was stored
#pragma unroll
          for (int j = 0; j < 8; ++j) vg[u][j] = round_through<T>(vg[u][j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s[j] += vg[u][j];
          sx[j] = fmaf(vg[u][j], (vy[u][j] - m[j]) * rs[j], sx[j]);
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    red[threadIdx.x][j] = s[j];
    red[threadIdx.x][8 + j] = sx[j];
  }
  __syncthreads();
  // one thread per (channel vector, one of 16 values) adds the row lanes in a fixed order
  for (int t = threadIdx.x; t < kvb * 16; t += kBnThreads) {
    const int cvl = t / 16, q = t % 16;
    const int cvg = blockIdx.y * kvb + cvl;
    if (cvg >= kv) continue;
    float a = 0.f;
    for (int l = 0; l < rpp; ++l) a += red[l * kvb + cvl][q];
    red_add_f32(sums + (q < 8 ? 0 : C) + cvg * 8 + (q & 7), a);
  }
}

// --------------------------------------------------------------------------------------------
// backward apply
template <typename T>
__global__ void __launch_bounds__(kBnThreads)
bn_backward_apply_kernel(const T* __restrict__ g, const T* __restrict__ y, const float* __restrict__ mean,
                         const float* __restrict__ rstd, const T* __restrict__ gamma, const float* __restrict__ sums,
                         float rf, T* __restrict__ dy, T* __restrict__ dgamma, T* __restrict__ dbeta, long long nvec, int kv) {
  extern __shared__ float bn_c[];        // a, c1, c0: three arrays of C, channel c at [c % 8][c / 8]
  const int C = kv * 8;
  for (int c = threadIdx.x; c < C; c += kBnThreads) {
    const float sg = sums[c], sgx = sums[C + c];
    const float r = rstd[c];
    const float a = Vec8<T>::load1(gamma + c) * r;
    const float c1 = -a * r * (sgx * rf);
    const int at = (c & 7) * kv + (c >> 3);
    bn_c[at] = a;
    bn_c[C + at] = c1;
    bn_c[2 * C + at] = -a * (sg * rf) - c1 * mean[c];
    if (blockIdx.x == 0) {
      if (dgamma != nullptr) Vec8<T>::store1(dgamma + c, sgx);
      if (dbeta != nullptr) Vec8<T>::store1(dbeta + c, sg);
    }
  }
  __syncthreads();
  const long long stride = static_cast<long long>(gridDim.x) * kBnThreads;
  const long long first = static_cast<long long>(blockIdx.x) * kBnThreads + threadIdx.x;
  const int sv = static_cast<int>(stride % kv);
  int cv0 = static_cast<int>(first % kv);
  for (long long i0 = first; i0 < nvec; i0 += stride * kBnUnroll, cv0 = (cv0 + kBnUnroll * sv) % kv) {
    float vg[kBnUnroll][8], vy[kBnUnroll][8];
#pragma unroll
    for (int u = 0; u < kBnUnroll; ++u) {
      const long long i = i0 + u * stride;
      Vec8<T>::load(g + i * 8, i < nvec, vg[u]);
      Vec8<T>::load(y + i * 8, i < nvec, vy[u]);
    }
#pragma unroll
    for (int u = 0; u < kBnUnroll; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) break;
      const float* cc = bn_c + (cv0 + u * sv) % kv;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        vg[u][j] = fmaf(cc[j * kv], vg[u][j], fmaf(cc[C + j * kv], vy[u][j], cc[2 * C + j * kv]));
      Vec8<T>::store(dy + i * 8, true, vg[u]);
    }
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int bn_check(const char* who, int64_t rows, int64_t channels, int32_t dtype) {
  if (dtype != EVTB_F16 && dtype != EVTB_BF16) {
    set_last_error(std::string(who) + ": activations must be fp16 or bf16");
    return EVTB_EINVAL;
  }
  if (rows <= 0 || channels <= 0 || channels % 8 != 0 || rows > 0x7fffffffLL) {
    set_last_error(std::string(who) + ": rows must be positive and channels a positive multiple of 8");
    return EVTB_EINVAL;
  }
  if (channels > kBnMaxChannels) {
    set_last_error(std::string(who) + ": at most 4096 channels (per-channel coefficients live in 48 KB of shared memory)");
    return EVTB_ETOOLARGE;
  }
  return EVTB_OK;
}

static int flat_grid(long long nvec) {
  int sms = current_device_sm_count();
  if (sms <= 0) sms = 148;
  const long long want = (nvec + static_cast<long long>(kBnThreads) * kBnUnroll - 1) / (static_cast<long long>(kBnThreads) * kBnUnroll);
  const long long cap = static_cast<long long>(sms) * 8;       // 8 CTAs of 256 threads per SM
  return static_cast<int>(want < cap ? (want < 1 ? 1 : want) : cap);
}

template <typename T>
static int bn_apply_launch(const void* y, int64_t rows, int64_t channels, const float* mean, const float* mean_sq,
                           const void* gamma, const void* beta, float eps, const void* residual, int relu, void* z,
                           float* saved_mean, float* saved_rstd, cudaStream_t s) {
  const int kv = static_cast<int>(channels / 8);
  const long long nvec = rows * kv;
  const int grid = flat_grid(nvec);
  const size_t smem = sizeof(float2) * channels;
#define EVTB_BN_APPLY(RELU, RES)                                                                                       \
  bn_apply_kernel<T, RELU, RES><<<grid, kBnThreads, smem, s>>>(static_cast<const T*>(y), mean, mean_sq,               \
      static_cast<const T*>(gamma), static_cast<const T*>(beta), eps, static_cast<const T*>(residual),                 \
      static_cast<T*>(z), saved_mean, saved_rstd, nvec, kv)
  if (relu && residual) EVTB_BN_APPLY(true, true);
  else if (relu) EVTB_BN_APPLY(true, false);
  else if (residual) EVTB_BN_APPLY(false, true);
  else EVTB_BN_APPLY(false, false);
#undef EVTB_BN_APPLY
  return cudaGetLastError() == cudaSuccess ? EVTB_OK : EVTB_ECUDA;
}

template <typename T>
static int bn_backward_reduce_launch(const void* g, const void* g2, const void* act, const void* y, int64_t rows,
                                     int64_t channels, const float* mean, const float* rstd, void* gout, float* sums,
                                     cudaStream_t s) {
  const int kv = static_cast<int>(channels / 8);
  const int kvb = kv < kBnThreads ? kv : kBnThreads;
  const int col_blocks = (kv + kvb - 1) / kvb;
  const int rpp = kBnThreads / kvb;
  int sms = current_device_sm_count();
  if (sms <= 0) sms = 148;
  // about 8 CTAs per SM, at least one full unrolled pass of rows each
  long long chunks = static_cast<long long>(sms) * 8 / col_blocks;
  const long long max_chunks = (rows + static_cast<long long>(rpp) * kBnUnroll - 1) / (static_cast<long long>(rpp) * kBnUnroll);
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks < 1) chunks = 1;
  long long rpc = (rows + chunks - 1) / chunks;
  rpc = (rpc + rpp - 1) / rpp * rpp;
  chunks = (rows + rpc - 1) / rpc;
  const dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(col_blocks));
#define EVTB_BN_RED(MASK, ADD, STORE)                                                                                  \
  bn_backward_reduce_kernel<T, MASK, ADD, STORE><<<grid, kBnThreads, 0, s>>>(static_cast<const T*>(g),                 \
      static_cast<const T*>(g2), static_cast<const T*>(act), static_cast<const T*>(y), mean, rstd,                      \
      static_cast<T*>(gout), sums, static_cast<int>(rows), kv, kvb, static_cast<int>(rpc))
  const bool m = act != nullptr, a = g2 != nullptr, st = gout != nullptr;
  if (m && a && st) EVTB_BN_RED(true, true, true);
  else if (m && !a && st) EVTB_BN_RED(true, false, true);
  else if (!m && a && st) EVTB_BN_RED(false, true, true);
  else if (!m && !a && !st) EVTB_BN_RED(false, false, false);
  else if (!m && !a && st) EVTB_BN_RED(false, false, true);
  else {
    set_last_error("evtb_bn_backward_reduce: a mask or a second gradient changes the gradient, so grad_out is required");
    return EVTB_EINVAL;
  }
#undef EVTB_BN_RED
  return cudaGetLastError() == cudaSuccess ? EVTB_OK : EVTB_ECUDA;
}

template <typename T>
static int bn_backward_apply_launch(const void* g, const void* y, int64_t rows, int64_t channels, const float* mean,
                                    const float* rstd, const void* gamma, const float* sums, float rf, void* dy,
                                    void* dgamma, void* dbeta, cudaStream_t s) {
  const int kv = static_cast<int>(channels / 8);
  const long long nvec = rows * kv;
  bn_backward_apply_kernel<T><<<flat_grid(nvec), kBnThreads, sizeof(float) * 3 * channels, s>>>(
      static_cast<const T*>(g), static_cast<const T*>(y), mean, rstd, static_cast<const T*>(gamma), sums, rf,
      static_cast<T*>(dy), static_cast<T*>(dgamma), static_cast<T*>(dbeta), nvec, kv);
  return cudaGetLastError() == cudaSuccess ? EVTB_OK : EVTB_ECUDA;
}

}  // namespace evtb

extern "C" {

int evtb_bn_apply(const void* y, int32_t dtype, int64_t rows, int64_t channels, const float* mean, const float* mean_sq,
                  const void* gamma, const void* beta, float eps, const void* residual, int32_t relu, void* z,
                  float* saved_mean, float* saved_rstd, evtb_stream stream) {
  if (const int st = evtb::bn_check("evtb_bn_apply", rows, channels, dtype)) return st;
  if (y == nullptr || z == nullptr || mean == nullptr || mean_sq == nullptr || gamma == nullptr || beta == nullptr ||
      !evtb::aligned16(y) || !evtb::aligned16(z) || !evtb::aligned16(residual)) {
    evtb::set_last_error("evtb_bn_apply: null operand, or an activation pointer that is not 16-byte aligned");
    return EVTB_EINVAL;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == EVTB_F16
             ? evtb::bn_apply_launch<__half>(y, rows, channels, mean, mean_sq, gamma, beta, eps, residual, relu, z, saved_mean, saved_rstd, s)
             : evtb::bn_apply_launch<__nv_bfloat16>(y, rows, channels, mean, mean_sq, gamma, beta, eps, residual, relu, z, saved_mean, saved_rstd, s);
}

int evtb_bn_backward_reduce(const void* grad, const void* grad2, const void* act, const void* y, int32_t dtype,
                            int64_t rows, int64_t channels, const float* mean, const float* rstd, void* grad_out,
                            float* sums, evtb_stream stream) {
  if (const int st = evtb::bn_check("evtb_bn_backward_reduce", rows, channels, dtype)) return st;
  if (grad == nullptr || y == nullptr || mean == nullptr || rstd == nullptr || sums == nullptr || !evtb::aligned16(grad) ||
      !evtb::aligned16(grad2) || !evtb::aligned16(act) || !evtb::aligned16(y) || !evtb::aligned16(grad_out)) {
    evtb::set_last_error("evtb_bn_backward_reduce: null operand, or an activation pointer that is not 16-byte aligned");
    return EVTB_EINVAL;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == EVTB_F16
             ? evtb::bn_backward_reduce_launch<__half>(grad, grad2, act, y, rows, channels, mean, rstd, grad_out, sums, s)
             : evtb::bn_backward_reduce_launch<__nv_bfloat16>(grad, grad2, act, y, rows, channels, mean, rstd, grad_out, sums, s);
}

int evtb_bn_backward_apply(const void* grad, const void* y, int32_t dtype, int64_t rows, int64_t channels,
                           const float* mean, const float* rstd, const void* gamma, const float* sums,
                           float reduction_factor, void* dy, void* dgamma, void* dbeta, evtb_stream stream) {
  if (const int st = evtb::bn_check("evtb_bn_backward_apply", rows, channels, dtype)) return st;
  if (grad == nullptr || y == nullptr || dy == nullptr || mean == nullptr || rstd == nullptr || gamma == nullptr ||
      sums == nullptr || !evtb::aligned16(grad) || !evtb::aligned16(y) || !evtb::aligned16(dy)) {
    evtb::set_last_error("evtb_bn_backward_apply: null operand, or an activation pointer that is not 16-byte aligned");
    return EVTB_EINVAL;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == EVTB_F16
             ? evtb::bn_backward_apply_launch<__half>(grad, y, rows, channels, mean, rstd, gamma, sums, reduction_factor, dy, dgamma, dbeta, s)
             : evtb::bn_backward_apply_launch<__nv_bfloat16>(grad, y, rows, channels, mean, rstd, gamma, sums, reduction_factor, dy, dgamma, dbeta, s);
}

}  // extern "C"
