// Device-side vocabulary of the generated epilogues: vector loads / stores with
// conversion to fp32, the elementwise functors, warp-level reductions and a
// counter-based RNG.  Counterpart of the reference's visitor node types in
// src/cuda/epilogue/threadblock/visitor_load.hpp (loads, RNG),
// visitor_compute.hpp (elementwise) and visitor_store.hpp (stores, reductions);
// all math is fp32 with round-to-nearest conversion on store, as there
// (visitor_compute.hpp:47-88).
#pragma once
#include "sm100_ptx.cuh"

namespace evtb {

// ---------------------------------------------------------------------------
// 8-wide loads: 8 consecutive elements -> fp32.  `ok == false` yields zeros and
// touches no memory.
// ---------------------------------------------------------------------------
template <typename T>
struct Vec8;

template <>
struct Vec8<__half> {
  static __device__ __forceinline__ void load(const void* p, bool ok, float (&v)[8]) {
    uint4 r = make_uint4(0, 0, 0, 0);
    if (ok) r = __ldg(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(void* p, bool ok, const float (&v)[8]) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    if (ok) *reinterpret_cast<uint4*>(p) = r;
  }
  static __device__ __forceinline__ float load1(const void* p) { return __half2float(*reinterpret_cast<const __half*>(p)); }
  static __device__ __forceinline__ void store1(void* p, float v) { *reinterpret_cast<__half*>(p) = __float2half_rn(v); }
};

template <>
struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const void* p, bool ok, float (&v)[8]) {
    uint4 r = make_uint4(0, 0, 0, 0);
    if (ok) r = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store(void* p, bool ok, const float (&v)[8]) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    if (ok) *reinterpret_cast<uint4*>(p) = r;
  }
  static __device__ __forceinline__ float load1(const void* p) { return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p)); }
  static __device__ __forceinline__ void store1(void* p, float v) { *reinterpret_cast<__nv_bfloat16*>(p) = __float2bfloat16_rn(v); }
};

template <>
struct Vec8<float> {
  static __device__ __forceinline__ void load(const void* p, bool ok, float (&v)[8]) {
    float4 a = make_float4(0, 0, 0, 0), b = a;
    if (ok) {
      a = __ldg(reinterpret_cast<const float4*>(p));
      b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    }
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(void* p, bool ok, const float (&v)[8]) {
    if (ok) {
      reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
      reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
  static __device__ __forceinline__ float load1(const void* p) { return *reinterpret_cast<const float*>(p); }
  static __device__ __forceinline__ void store1(void* p, float v) { *reinterpret_cast<float*>(p) = v; }
};

// torch.bool / uint8: one byte per element, non-zero = true
template <>
struct Vec8<uint8_t> {
  static __device__ __forceinline__ void load(const void* p, bool ok, float (&v)[8]) {
    uint2 r = make_uint2(0, 0);
    if (ok) r = __ldg(reinterpret_cast<const uint2*>(p));
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&r);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = b[i] ? 1.f : 0.f;
  }
  static __device__ __forceinline__ void store(void* p, bool ok, const float (&v)[8]) {
    uint2 r;
    uint8_t* b = reinterpret_cast<uint8_t*>(&r);
#pragma unroll
    for (int i = 0; i < 8; ++i) b[i] = v[i] != 0.f ? 1 : 0;
    if (ok) *reinterpret_cast<uint2*>(p) = r;
  }
  static __device__ __forceinline__ float load1(const void* p) { return *reinterpret_cast<const uint8_t*>(p) ? 1.f : 0.f; }
  static __device__ __forceinline__ void store1(void* p, float v) { *reinterpret_cast<uint8_t*>(p) = v != 0.f ? 1 : 0; }
};

// int64 class indices (one_hot operand): scalar access only
template <>
struct Vec8<long long> {
  static __device__ __forceinline__ float load1(const void* p) { return static_cast<float>(*reinterpret_cast<const long long*>(p)); }
  static __device__ __forceinline__ void store1(void* p, float v) { *reinterpret_cast<long long*>(p) = static_cast<long long>(v); }
};

template <>
struct Vec8<int> {
  static __device__ __forceinline__ float load1(const void* p) { return static_cast<float>(*reinterpret_cast<const int*>(p)); }
  static __device__ __forceinline__ void store1(void* p, float v) { *reinterpret_cast<int*>(p) = static_cast<int>(v); }
};

// ---------------------------------------------------------------------------
// Warp staging tile for the GEMM epilogue: 32 rows x 64 bytes (32 columns of a 16-bit
// type) in shared memory, 16-byte slots XOR-swizzled so that both access patterns are
// free of bank conflicts:
//   thread-per-row   lane = row, fixed slot            (what tcgen05.ld hands out)
//   row-segment      lane = (row % 8, slot), 4 rounds  (coalesced global access: every
//                    instruction moves 8 rows x 64 contiguous bytes)
// Full tensors are moved global <-> staging tile in the second pattern and consumed /
// produced by the math in the first, instead of 32 scattered 16-byte accesses per
// instruction.
// ---------------------------------------------------------------------------
constexpr int kStageTileBytes = 32 * 64;

__device__ __forceinline__ uint32_t stage_slot(int row, int seg) {
  return static_cast<uint32_t>(row * 64 + (((seg ^ (row >> 1)) & 3) << 4));
}
__device__ __forceinline__ void stage_write16(char* tile, int row, int seg, uint4 v) {
  *reinterpret_cast<uint4*>(tile + stage_slot(row, seg)) = v;
}
__device__ __forceinline__ uint4 stage_read16(const char* tile, int row, int seg) {
  return *reinterpret_cast<const uint4*>(tile + stage_slot(row, seg));
}

template <typename T>
struct Pack8;
template <>
struct Pack8<__half> {
  static __device__ __forceinline__ uint4 pack(const float (&v)[8]) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    return r;
  }
  static __device__ __forceinline__ void unpack(uint4 r, float (&v)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};
template <>
struct Pack8<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 pack(const float (&v)[8]) {
    uint4 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return r;
  }
  static __device__ __forceinline__ void unpack(uint4 r, float (&v)[8]) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

// ---------------------------------------------------------------------------
// Elementwise functors
// ---------------------------------------------------------------------------
__device__ __forceinline__ float op_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float op_tanh_precise(float x) { return tanhf(x); }
__device__ __forceinline__ float op_sigmoid(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float op_relu(float x) { return fmaxf(x, 0.f); }
__device__ __forceinline__ float op_tanh_backward(float g, float y) { return g * (1.f - y * y); }

// erf by Abramowitz & Stegun 7.1.26 (|error| <= 1.5e-7, below fp32 rounding of 1 + erf):
// one reciprocal, one exp2 and seven FMAs instead of erff's branchy polynomial pair.
__device__ __forceinline__ float fast_erf(float x) {
  const float ax = fabsf(x);
  const float t = __fdividef(1.0f, fmaf(0.3275911f, ax, 1.0f));
  float y = fmaf(t, 1.061405429f, -1.453152027f);
  y = fmaf(t, y, 1.421413741f);
  y = fmaf(t, y, -0.284496736f);
  y = fmaf(t, y, 0.254829592f);
  y *= t;
  const float e = __expf(-ax * ax);
  const float r = fmaf(-y, e, 1.0f);
  return copysignf(r, x);
}

__device__ __forceinline__ float op_gelu_tanh(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + op_tanh(u));   // tanh.approx: relative error ~2^-11
}
__device__ __forceinline__ float op_gelu_erf(float x) {
  return 0.5f * x * (1.f + fast_erf(x * 0.7071067811865476f));
}
__device__ __forceinline__ float op_gelu_backward_tanh(float g, float x) {
  const float x2 = x * x;
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x2);
  const float t = op_tanh(u);
  const float du = 0.7978845608028654f * (1.f + 0.134145f * x2);
  return g * (0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du);
}
// d/dx [x Phi(x)] = Phi(x) + x phi(x).  The exponential of the Abramowitz & Stegun form of
// erf(x / sqrt 2) is exp(-x^2 / 2), the same one the density needs: one exp2 and one reciprocal per
// element (the special-function unit, 16 results per clock and SM, is what a GELU epilogue on a short-K
// GEMM runs out of first).
__device__ __forceinline__ float op_gelu_backward_erf(float g, float x) {
  const float ax = fabsf(x) * 0.7071067811865476f;
  const float t = __fdividef(1.0f, fmaf(0.3275911f, ax, 1.0f));
  float y = fmaf(t, 1.061405429f, -1.453152027f);
  y = fmaf(t, y, 1.421413741f);
  y = fmaf(t, y, -0.284496736f);
  y = fmaf(t, y, 0.254829592f);
  y *= t;
  const float e = __expf(-0.5f * x * x);
  const float erf_abs = fmaf(-y, e, 1.0f);
  const float cdf = fmaf(0.5f, copysignf(erf_abs, x), 0.5f);
  return g * fmaf(x * 0.3989422804014327f, e, cdf);
}

// ---------------------------------------------------------------------------
// Warp transpose-reduce: every lane holds 32 values (one per column); on return
// lane j holds the reduction over all 32 lanes of column j.  31 shuffles.
// ---------------------------------------------------------------------------
struct SumOp {
  static __device__ __forceinline__ float apply(float a, float b) { return a + b; }
  static __device__ __forceinline__ float identity() { return 0.f; }
};
struct MaxOp {
  static __device__ __forceinline__ float apply(float a, float b) { return fmaxf(a, b); }
  static __device__ __forceinline__ float identity() { return -INFINITY; }
};

template <class Op, int W>
struct TransposeReduce {
  // v holds 2*W live values; halves them across lanes `W` apart
  static __device__ __forceinline__ void step(float (&v)[32], int lane) {
    const bool upper = (lane & W) != 0;
#pragma unroll
    for (int i = 0; i < W; ++i) {
      const float send = upper ? v[i] : v[i + W];
      const float keep = upper ? v[i + W] : v[i];
      v[i] = Op::apply(keep, __shfl_xor_sync(0xffffffffu, send, W));
    }
    if constexpr (W > 1) TransposeReduce<Op, W / 2>::step(v, lane);
  }
};

template <class Op>
__device__ __forceinline__ float warp_transpose_reduce32(float (&v)[32], int lane) {
  TransposeReduce<Op, 16>::step(v, lane);
  return v[0];
}

template <class Op>
__device__ __forceinline__ float warp_allreduce(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---------------------------------------------------------------------------
// Philox4x32-10 (Salmon et al., SC'11): counter = element index / 4, key = seed.
// Gives the uniform numbers of fused dropout (the reference draws them with
// cuRAND's Philox in visitor_load.hpp:79-151; bitwise equality with it is not a
// goal, the mask is an output and is checked by reuse).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]);
  const uint32_t lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]);
  const uint32_t lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0;
  const uint32_t n2 = hi0 ^ c[3] ^ k1;
  c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
}

__device__ __forceinline__ void philox4x32_10(unsigned long long seed, unsigned long long ctr,
                                              uint32_t (&out)[4]) {
  uint32_t c[4] = {static_cast<uint32_t>(ctr), static_cast<uint32_t>(ctr >> 32), 0u, 0u};
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = c[i];
}

// 8 uniforms in [0,1) for 8 consecutive elements starting at linear index `idx` (idx % 8 == 0)
__device__ __forceinline__ void rand8(unsigned long long seed, unsigned long long offset,
                                      unsigned long long idx, float (&v)[8]) {
  uint32_t r[4];
  philox4x32_10(seed, offset + idx / 4, r);
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = (r[i] >> 8) * (1.0f / 16777216.0f);
  philox4x32_10(seed, offset + idx / 4 + 1, r);
#pragma unroll
  for (int i = 0; i < 4; ++i) v[4 + i] = (r[i] >> 8) * (1.0f / 16777216.0f);
}

}  // namespace evtb
