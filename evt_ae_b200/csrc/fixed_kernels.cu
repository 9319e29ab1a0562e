// Kernels that need no code generation.
//
//  evtb_colsum   y[c] = sum_r x[r, c]   (fp32 accumulate, deterministic two-step reduction
//                inside one launch).  Bias gradients whose producer is a row kernel, not a
//                GEMM, land here; the reference leaves such `aten.sum` nodes to
//                eager / TorchScript (python/gtl/compiler/passes/evt_fuser.py:1096-1100,
//                nv_fuser.py:134-141).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_select.cuh>

#include "../../include/evt_b200.h"
#include "evtb_internal.h"
#include "epilogue_ops.cuh"
#include "spmm.cuh"

namespace evtb {

constexpr int kColsumThreads = 128;      // each thread owns 8 adjacent columns
constexpr int kColsumColsPerCta = kColsumThreads * 8;
constexpr int kColsumMaxChunks = 1024;   // row chunks (second grid dim)

// workspace layout: float partial[chunks][cols_padded] followed by uint32 counter[col_blocks]
// y[c] += sum over this CTA's rows of x[r, c]: one pass, no partial buffer and no serial tail; the
// chunks of rows meet in y through fp32 atomics, so y must hold the value to add to (zero for a
// plain sum) and the order of the additions is not fixed.
template <typename TIn>
__global__ void __launch_bounds__(kColsumThreads)
colsum_accumulate_kernel(const TIn* __restrict__ x, float* __restrict__ y, int rows, int cols, int rows_per_chunk) {
  const int c0 = blockIdx.x * kColsumColsPerCta + threadIdx.x * 8;
  if (c0 >= cols) return;
  const bool vec = (cols % 8 == 0);
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  const int r0 = blockIdx.y * rows_per_chunk;
  const int r1 = min(rows, r0 + rows_per_chunk);
  int r = r0;
  if (vec) {
    for (; r + 4 <= r1; r += 4) {       // four independent row loads in flight per thread
      float v[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) Vec8<TIn>::load(x + static_cast<long long>(r + u) * cols + c0, true, v[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += v[u][j];
    }
  }
  for (; r < r1; ++r) {
    float v[8];
    const TIn* p = x + static_cast<long long>(r) * cols + c0;
    if (vec) {
      Vec8<TIn>::load(p, true, v);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (c0 + j < cols) ? Vec8<TIn>::load1(p + j) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += v[j];
  }
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (c0 + j < cols) red_add_f32(y + c0 + j, acc[j]);
}

// The same sum for column counts that are multiples of 8: 256 threads = `ct` column threads (8 columns
// each) x 256 / ct row lanes; the row lanes' sums meet in shared memory and the CTA sends ONE atomic
// per column.  With one atomic per thread (the kernel above) 586 CTAs put 586 additions on each of
// 1024 words and the launch took 57 us on 16384 x 1024 bf16 from cold caches; this form takes 12 us
// (33.6 MB: 5 us at the measured copy rate).
constexpr int kColsumWideThreads = 256;
template <typename TIn>
__global__ void __launch_bounds__(kColsumWideThreads)
colsum_accumulate_wide_kernel(const TIn* __restrict__ x, float* __restrict__ y, int rows, int cols, int rows_per_chunk,
                              int ct) {
  __shared__ float part[kColsumWideThreads][9];
  const int rl = kColsumWideThreads / ct;
  const int lane_r = threadIdx.x / ct;
  const int c0 = (blockIdx.x * ct + threadIdx.x % ct) * 8;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  const int r0 = blockIdx.y * rows_per_chunk;
  const int r1 = min(rows, r0 + rows_per_chunk);
  if (c0 < cols) {
    for (int rb = r0 + lane_r; rb < r1; rb += rl * 4) {     // four independent row loads in flight per thread
      float v[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = rb + u * rl;
        Vec8<TIn>::load(x + static_cast<long long>(r) * cols + c0, r < r1, v[u]);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += v[u][j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) part[threadIdx.x][j] = acc[j];
  __syncthreads();
  for (int t = threadIdx.x; t < ct * 8; t += kColsumWideThreads) {
    const int cv = t >> 3, j = t & 7;
    const int c = (blockIdx.x * ct + cv) * 8 + j;
    if (c >= cols) continue;
    float a = 0.f;
    for (int l = 0; l < rl; ++l) a += part[l * ct + cv][j];
    red_add_f32(y + c, a);
  }
}

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(kColsumThreads)
colsum_kernel(const TIn* __restrict__ x, TOut* __restrict__ y, int rows, int cols, int rows_per_chunk,
              float* __restrict__ partial, unsigned int* __restrict__ counters, int cols_padded) {
  const int cb = blockIdx.x;
  const int chunk = blockIdx.y;
  const int chunks = gridDim.y;
  const int c0 = cb * kColsumColsPerCta + threadIdx.x * 8;
  const bool vec = (cols % 8 == 0);
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  const int r0 = chunk * rows_per_chunk;
  const int r1 = min(rows, r0 + rows_per_chunk);
  if (c0 < cols) {
    int r = r0;
    if (vec) {
      // four independent row loads in flight per thread
      for (; r + 4 <= r1; r += 4) {
        float v[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) Vec8<TIn>::load(x + static_cast<long long>(r + u) * cols + c0, true, v[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += v[u][j];
      }
    }
    for (; r < r1; ++r) {
      float v[8];
      const TIn* p = x + static_cast<long long>(r) * cols + c0;
      if (vec) {
        Vec8<TIn>::load(p, true, v);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (c0 + j < cols) ? Vec8<TIn>::load1(p + j) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
    float* dst = partial + static_cast<long long>(chunk) * cols_padded + c0;
    reinterpret_cast<float4*>(dst)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    reinterpret_cast<float4*>(dst)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  // the last CTA of this column block to finish adds the partials up (fixed order)
  __shared__ bool last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(&counters[cb], 1u);
    last = (prev == static_cast<unsigned int>(chunks - 1));
    if (last) counters[cb] = 0u;   // leave the counter clean for the next launch
  }
  __syncthreads();
  if (!last || c0 >= cols) return;
  __threadfence();
  float tot[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) tot[j] = 0.f;
#pragma unroll 8
  for (int k = 0; k < chunks; ++k) {   // fixed order: the result does not depend on arrival order
    const float* src = partial + static_cast<long long>(k) * cols_padded + c0;
    const float4 a = __ldcg(reinterpret_cast<const float4*>(src));
    const float4 b = __ldcg(reinterpret_cast<const float4*>(src) + 1);
    tot[0] += a.x; tot[1] += a.y; tot[2] += a.z; tot[3] += a.w;
    tot[4] += b.x; tot[5] += b.y; tot[6] += b.z; tot[7] += b.w;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (c0 + j < cols) Vec8<TOut>::store1(y + c0 + j, tot[j]);
}

struct ColsumPlan {
  int col_blocks, chunks, rows_per_chunk, cols_padded;
  size_t bytes;
};

// The chunk count depends only on the shape (a workspace size is asked for without a device):
// sized for 148 SMs x 16 resident CTAs of 128 threads, which also fills smaller parts.
constexpr int kColsumTargetCtas = 148 * 16;

inline ColsumPlan colsum_plan(long long rows, long long cols, long long max_partial_floats = (1ll << 40)) {
  ColsumPlan p;
  p.col_blocks = static_cast<int>((cols + kColsumColsPerCta - 1) / kColsumColsPerCta);
  p.cols_padded = p.col_blocks * kColsumColsPerCta;
  // enough CTAs to fill the GPU a few times over, at least 32 rows per chunk, within the scratch
  // the caller has
  long long want = (kColsumTargetCtas + p.col_blocks - 1) / p.col_blocks;
  long long max_by_rows = (rows + 31) / 32;
  long long chunks = want < max_by_rows ? want : max_by_rows;
  if (chunks > kColsumMaxChunks) chunks = kColsumMaxChunks;
  if (chunks * p.cols_padded > max_partial_floats) chunks = max_partial_floats / p.cols_padded;
  if (chunks < 1) chunks = 1;
  p.chunks = static_cast<int>(chunks);
  p.rows_per_chunk = static_cast<int>((rows + chunks - 1) / chunks);
  p.bytes = sizeof(float) * static_cast<size_t>(p.chunks) * p.cols_padded + sizeof(unsigned int) * p.col_blocks;
  return p;
}

template <typename TIn>
int colsum_dispatch_out(const void* x, void* y, int out_dtype, int rows, int cols, const ColsumPlan& pl,
                        float* partial, unsigned int* counters, cudaStream_t s) {
  dim3 grid(pl.col_blocks, pl.chunks);
  const TIn* xi = static_cast<const TIn*>(x);
  switch (out_dtype) {
    case EVTB_F16:
      colsum_kernel<TIn, __half><<<grid, kColsumThreads, 0, s>>>(xi, static_cast<__half*>(y), rows, cols, pl.rows_per_chunk, partial, counters, pl.cols_padded);
      break;
    case EVTB_BF16:
      colsum_kernel<TIn, __nv_bfloat16><<<grid, kColsumThreads, 0, s>>>(xi, static_cast<__nv_bfloat16*>(y), rows, cols, pl.rows_per_chunk, partial, counters, pl.cols_padded);
      break;
    case EVTB_F32:
      colsum_kernel<TIn, float><<<grid, kColsumThreads, 0, s>>>(xi, static_cast<float*>(y), rows, cols, pl.rows_per_chunk, partial, counters, pl.cols_padded);
      break;
    default:
      return EVTB_EINVAL;
  }
  return cudaGetLastError() == cudaSuccess ? EVTB_OK : EVTB_ECUDA;
}

// ---------------------------------------------------------------------------------------
// SDDMM over a CSR pattern: out[p] = <U[i, :], V[col[p], :]> for every nonzero p of row i
// (edge gradients of a GCN layer; the reference has no SDDMM -- its GCN backward is a second
// SpMM, python/model_zoo/gcn/gcn_modeling.py:107-120).  Same merge-path shares as the SpMM:
// a warp whose share starts inside a hub row simply reloads that row of U.
// ---------------------------------------------------------------------------------------
constexpr int kSddmmThreads = 256;
constexpr int kSddmmItemsPerWarp = 64;

__global__ void __launch_bounds__(kSddmmThreads)
sddmm_kernel(const int* __restrict__ crow, const int* __restrict__ col, const float* __restrict__ u,
             const float* __restrict__ v, float* __restrict__ out, int rows, int nnz, int F, int total_warps) {
  const int lane = threadIdx.x & 31;
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (w >= total_warps) return;
  const int items = rows + nnz;
  const long long d0l = static_cast<long long>(w) * kSddmmItemsPerWarp;
  const int d0 = d0l < items ? static_cast<int>(d0l) : items;
  const int d1 = d0 + kSddmmItemsPerWarp < items ? d0 + kSddmmItemsPerWarp : items;
  if (d0 >= d1) return;
  int x0, y0, x1, y1;
  merge_path_search(crow, rows, nnz, d0, x0, y0);
  merge_path_search(crow, rows, nnz, d1, x1, y1);
  const int F4 = F >> 2;                       // F % 4 == 0 (checked on the host)
  int nz = y0;
  for (int row = x0; row <= x1 && row < rows; ++row) {
    const int end = row < x1 ? __ldg(crow + row + 1) : y1;
    if (end <= nz) continue;
    const float4* ur = reinterpret_cast<const float4*>(u + static_cast<long long>(row) * F);
    for (int q = nz; q < end; ++q) {
      const float4* vr = reinterpret_cast<const float4*>(v + static_cast<long long>(__ldg(col + q)) * F);
      float s = 0.f;
      for (int k = lane; k < F4; k += 32) {
        const float4 a = __ldg(ur + k), b = __ldg(vr + k);
        s += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
      }
      s = warp_allreduce<SumOp>(s);
      if (lane == 0) out[q] = s;
    }
    nz = end;
  }
}

// ---------------------------------------------------------------------------------------
// COO -> CSR with int32 indices: sort the (row, col) pairs, drop duplicates, find the row
// starts.  Bit-exact against sort + unique + searchsorted on the host.
// ---------------------------------------------------------------------------------------
__global__ void csr_pack_keys(const int* __restrict__ r, const int* __restrict__ c, unsigned long long* keys, long long n) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i < n) keys[i] = (static_cast<unsigned long long>(static_cast<unsigned int>(r[i])) << 32) | static_cast<unsigned int>(c[i]);
}

__global__ void csr_finish(const unsigned long long* __restrict__ keys, const int* __restrict__ n_unique, int rows,
                           int* __restrict__ crow, int* __restrict__ col, long long capacity) {
  const int nu = *n_unique;
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i < nu) col[i] = static_cast<int>(keys[i] & 0xffffffffull);
  if (i <= rows) {
    // first key whose row is >= i
    const unsigned long long target = static_cast<unsigned long long>(i) << 32;
    int lo = 0, hi = nu;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (keys[mid] < target) lo = mid + 1; else hi = mid;
    }
    crow[i] = lo;
  }
}

// ---------------------------------------------------------------------------------------
// Column sum without any caller- or library-side allocation.
//
// Some hosts of this library cannot hand it scratch memory: a serving process that gave its
// whole device-memory budget to its own arena at start-up, or a plugin slot where a
// cudaMalloc (which synchronises the whole device) would stall the other streams of the
// process.  For them the partial sums live in one fixed array that is part of the library
// image.  The price: the array is sized for a stated maximum, every GPU that loads the
// library carries it until the process exits, and all calls share it.
// ---------------------------------------------------------------------------------------
constexpr size_t kStaticCounterBytes = 256;                                  // 64 column blocks
constexpr size_t kStaticPartialBytes = sizeof(float) * 64 * 8192;   // 2 MiB: up to 8192 columns
constexpr size_t kStaticScratchBytes = kStaticCounterBytes + kStaticPartialBytes;

static __device__ __align__(256) unsigned char g_colsum_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_scratch_addr[kMaxDevices];      // device address of the array, per device
static bool g_scratch_ready[kMaxDevices];
static std::mutex g_scratch_mutex;

// The array's name is only a host-side handle here; the kernel needs its device address,
// looked up once per device with that device current.
static int static_scratch_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) {
    (void)cudaGetLastError();
    set_last_error("evtb_colsum_static: no current CUDA device");
    return EVTB_ECUDA;
  }
  if (dev >= kMaxDevices) {
    set_last_error("evtb_colsum_static: device ordinals above 63 are not supported");
    return EVTB_EINVAL;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ready[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_colsum_scratch);
    if (e != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      set_last_error(std::string("evtb_colsum_static: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
      return EVTB_ECUDA;
    }
    g_scratch_addr[dev] = p;
    g_scratch_ready[dev] = true;
  }
  *out = g_scratch_addr[dev];
  return EVTB_OK;
}

}  // namespace evtb

extern "C" {

int evtb_colsum_workspace_bytes(int64_t rows, int64_t cols, size_t* bytes) {
  if (bytes == nullptr || rows <= 0 || cols <= 0) return EVTB_EINVAL;
  *bytes = evtb::colsum_plan(rows, cols).bytes;
  return EVTB_OK;
}

int evtb_colsum_accumulate(const void* x, int32_t in_dtype, int64_t rows, int64_t cols, float* y, evtb_stream stream) {
  if (x == nullptr || y == nullptr || rows <= 0 || cols <= 0 || rows > 0x7fffffffLL || cols > 0x7fffffffLL)
    return EVTB_EINVAL;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0) return EVTB_EINVAL;
  const int r = static_cast<int>(rows), c = static_cast<int>(cols);
  int sms = evtb::current_device_sm_count();
  if (sms <= 0) sms = 148;
  if (c % 8 == 0) {
    // column threads per CTA: a power of two up to 64; about four CTAs per SM in total
    int ct = 8;
    while (ct < 64 && ct * 8 < c) ct *= 2;
    const int rl = evtb::kColsumWideThreads / ct;
    const int col_blocks = (c / 8 + ct - 1) / ct;
    int chunks = (sms * 4 + col_blocks - 1) / col_blocks;
    if (chunks > (r + rl - 1) / rl) chunks = (r + rl - 1) / rl;
    if (chunks < 1) chunks = 1;
    int rows_per_chunk = (r + chunks - 1) / chunks;
    rows_per_chunk = (rows_per_chunk + rl - 1) / rl * rl;
    chunks = (r + rows_per_chunk - 1) / rows_per_chunk;
    const dim3 grid(col_blocks, chunks);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (in_dtype) {
      case EVTB_F16: evtb::colsum_accumulate_wide_kernel<__half><<<grid, evtb::kColsumWideThreads, 0, s>>>(static_cast<const __half*>(x), y, r, c, rows_per_chunk, ct); break;
      case EVTB_BF16: evtb::colsum_accumulate_wide_kernel<__nv_bfloat16><<<grid, evtb::kColsumWideThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), y, r, c, rows_per_chunk, ct); break;
      case EVTB_F32: evtb::colsum_accumulate_wide_kernel<float><<<grid, evtb::kColsumWideThreads, 0, s>>>(static_cast<const float*>(x), y, r, c, rows_per_chunk, ct); break;
      default: return EVTB_EINVAL;
    }
    return cudaGetLastError() == cudaSuccess ? EVTB_OK : EVTB_ECUDA;
  }
  const int col_blocks = (c + evtb::kColsumColsPerCta - 1) / evtb::kColsumColsPerCta;
  // ragged column counts: about four CTAs per SM in total, one atomic per column and thread
  int chunks = (sms * 4 + col_blocks - 1) / col_blocks;
  if (chunks > r) chunks = r;
  if (chunks < 1) chunks = 1;
  const int rows_per_chunk = (r + chunks - 1) / chunks;
  chunks = (r + rows_per_chunk - 1) / rows_per_chunk;
  const dim3 grid(col_blocks, chunks);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (in_dtype) {
    case EVTB_F16: evtb::colsum_accumulate_kernel<__half><<<grid, evtb::kColsumThreads, 0, s>>>(static_cast<const __half*>(x), y, r, c, rows_per_chunk); break;
    case EVTB_BF16: evtb::colsum_accumulate_kernel<__nv_bfloat16><<<grid, evtb::kColsumThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), y, r, c, rows_per_chunk); break;
    case EVTB_F32: evtb::colsum_accumulate_kernel<float><<<grid, evtb::kColsumThreads, 0, s>>>(static_cast<const float*>(x), y, r, c, rows_per_chunk); break;
    default: return EVTB_EINVAL;
  }
  return cudaGetLastError() == cudaSuccess ? EVTB_OK : EVTB_ECUDA;
}

int evtb_colsum(const void* x, int32_t in_dtype, int64_t rows, int64_t cols, void* y, int32_t out_dtype,
                void* workspace, size_t workspace_bytes, evtb_stream stream) {
  if (x == nullptr || y == nullptr || workspace == nullptr || rows <= 0 || cols <= 0 ||
      rows > 0x7fffffffLL || cols > 0x7fffffffLL)
    return EVTB_EINVAL;
  const evtb::ColsumPlan pl = evtb::colsum_plan(rows, cols);
  if (workspace_bytes < pl.bytes) return EVTB_EINVAL;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0 || (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0)
    return EVTB_EINVAL;
  float* partial = static_cast<float*>(workspace);
  unsigned int* counters = reinterpret_cast<unsigned int*>(partial + static_cast<size_t>(pl.chunks) * pl.cols_padded);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int r = static_cast<int>(rows), c = static_cast<int>(cols);
  switch (in_dtype) {
    case EVTB_F16: return evtb::colsum_dispatch_out<__half>(x, y, out_dtype, r, c, pl, partial, counters, s);
    case EVTB_BF16: return evtb::colsum_dispatch_out<__nv_bfloat16>(x, y, out_dtype, r, c, pl, partial, counters, s);
    case EVTB_F32: return evtb::colsum_dispatch_out<float>(x, y, out_dtype, r, c, pl, partial, counters, s);
    default: return EVTB_EINVAL;
  }
}

int evtb_sddmm(const int32_t* crow, const int32_t* col, const float* u, const float* v, int64_t rows, int64_t nnz,
               int64_t F, float* out, evtb_stream stream) {
  if (crow == nullptr || col == nullptr || u == nullptr || v == nullptr || out == nullptr || rows <= 0 || nnz < 0 ||
      F <= 0 || F % 4 != 0 || rows + nnz > 0x7fffff00LL)
    return EVTB_EINVAL;
  if (((reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(v)) & 15u) != 0) return EVTB_EINVAL;
  if (nnz == 0) return EVTB_OK;
  const long long items = rows + nnz;
  const int total_warps = static_cast<int>((items + evtb::kSddmmItemsPerWarp - 1) / evtb::kSddmmItemsPerWarp);
  const int wpc = evtb::kSddmmThreads / 32;
  evtb::sddmm_kernel<<<(total_warps + wpc - 1) / wpc, evtb::kSddmmThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      crow, col, u, v, out, static_cast<int>(rows), static_cast<int>(nnz), static_cast<int>(F), total_warps);
  return cudaGetLastError() == cudaSuccess ? EVTB_OK : EVTB_ECUDA;
}

static size_t csr_align(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

int evtb_csr_build_workspace_bytes(int64_t n_edges, size_t* bytes) {
  if (bytes == nullptr || n_edges <= 0 || n_edges > 0x7fffff00LL) return EVTB_EINVAL;
  size_t sort_tmp = 0, sel_tmp = 0;
  unsigned long long* k = nullptr;
  int* cnt = nullptr;
  cub::DeviceRadixSort::SortKeys(nullptr, sort_tmp, k, k, static_cast<int>(n_edges));
  cub::DeviceSelect::Unique(nullptr, sel_tmp, k, k, cnt, static_cast<int>(n_edges));
  const size_t tmp = sort_tmp > sel_tmp ? sort_tmp : sel_tmp;
  *bytes = 3 * csr_align(sizeof(unsigned long long) * n_edges) + csr_align(tmp) + 256;
  return EVTB_OK;
}

int evtb_csr_build(const int32_t* coo_row, const int32_t* coo_col, int64_t n_edges, int64_t rows, void* workspace,
                   size_t workspace_bytes, int32_t* crow, int32_t* col, int32_t* nnz_out, evtb_stream stream) {
  if (coo_row == nullptr || coo_col == nullptr || workspace == nullptr || crow == nullptr || col == nullptr ||
      nnz_out == nullptr || n_edges <= 0 || rows <= 0 || n_edges > 0x7fffff00LL || rows > 0x7fffff00LL)
    return EVTB_EINVAL;
  size_t need = 0;
  if (evtb_csr_build_workspace_bytes(n_edges, &need) != EVTB_OK || workspace_bytes < need ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return EVTB_EINVAL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int n = static_cast<int>(n_edges);
  char* base = static_cast<char*>(workspace);
  const size_t kb = csr_align(sizeof(unsigned long long) * n_edges);
  unsigned long long* k0 = reinterpret_cast<unsigned long long*>(base);
  unsigned long long* k1 = reinterpret_cast<unsigned long long*>(base + kb);
  unsigned long long* k2 = reinterpret_cast<unsigned long long*>(base + 2 * kb);
  void* tmp = base + 3 * kb;
  size_t tmp_bytes = workspace_bytes - 3 * kb - 256;
  evtb::csr_pack_keys<<<(n + 255) / 256, 256, 0, s>>>(coo_row, coo_col, k0, n_edges);
  size_t t = tmp_bytes;
  if (cub::DeviceRadixSort::SortKeys(tmp, t, k0, k1, n, 0, 64, s) != cudaSuccess) return EVTB_ECUDA;
  t = tmp_bytes;
  if (cub::DeviceSelect::Unique(tmp, t, k1, k2, nnz_out, n, s) != cudaSuccess) return EVTB_ECUDA;
  const long long work = n_edges > rows + 1 ? n_edges : rows + 1;
  evtb::csr_finish<<<static_cast<unsigned int>((work + 255) / 256), 256, 0, s>>>(k2, nnz_out, static_cast<int>(rows), crow, col, n_edges);
  return cudaGetLastError() == cudaSuccess ? EVTB_OK : EVTB_ECUDA;
}

int evtb_colsum_static_max_cols(void) { return 8192; }

int evtb_colsum_static(const void* x, int32_t in_dtype, int64_t rows, int64_t cols, void* y, int32_t out_dtype,
                       evtb_stream stream) {
  if (x == nullptr || y == nullptr || rows <= 0 || cols <= 0 || rows > 0x7fffffffLL) return EVTB_EINVAL;
  if (cols > evtb_colsum_static_max_cols()) return EVTB_ETOOLARGE;   // beyond the built-in scratch
  const evtb::ColsumPlan pl = evtb::colsum_plan(rows, cols, static_cast<long long>(evtb::kStaticPartialBytes / sizeof(float)));
  if (pl.chunks < 1 || sizeof(float) * static_cast<size_t>(pl.chunks) * pl.cols_padded > evtb::kStaticPartialBytes ||
      sizeof(unsigned int) * pl.col_blocks > evtb::kStaticCounterBytes)
    return EVTB_ETOOLARGE;
  // rows are read with 16-byte loads only when every row starts on a 16-byte boundary
  if (cols % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) != 0) {
    evtb::set_last_error("evtb_colsum_static: x must be 16-byte aligned when cols is a multiple of 8");
    return EVTB_EINVAL;
  }
  // the scratch array used is the CURRENT device's copy: the buffers (and the stream) must belong
  // to that device, or the partial sums would be written through another GPU's memory
  {
    cudaPointerAttributes attr;
    int dev = -1;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaPointerGetAttributes(&attr, x) == cudaSuccess &&
        attr.type == cudaMemoryTypeDevice && attr.device != dev) {
      evtb::set_last_error("evtb_colsum_static: x lives on another device than the current one");
      return EVTB_EINVAL;
    }
    (void)cudaGetLastError();
  }
  void* base = nullptr;
  const int rc = evtb::static_scratch_address(&base);   // first call on a device: symbol look-up
  if (rc != EVTB_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned int* counters = static_cast<unsigned int*>(base);
  float* partial = reinterpret_cast<float*>(static_cast<unsigned char*>(base) + evtb::kStaticCounterBytes);
  // the array keeps whatever the previous call (possibly of another shape, possibly
  // interrupted) left behind: the arrival counters must start at zero
  if (cudaMemsetAsync(counters, 0, evtb::kStaticCounterBytes, s) != cudaSuccess) return EVTB_ECUDA;
  const int r = static_cast<int>(rows), c = static_cast<int>(cols);
  switch (in_dtype) {
    case EVTB_F16: return evtb::colsum_dispatch_out<__half>(x, y, out_dtype, r, c, pl, partial, counters, s);
    case EVTB_BF16: return evtb::colsum_dispatch_out<__nv_bfloat16>(x, y, out_dtype, r, c, pl, partial, counters, s);
    case EVTB_F32: return evtb::colsum_dispatch_out<float>(x, y, out_dtype, r, c, pl, partial, counters, s);
    default: return EVTB_EINVAL;
  }
}

}  // extern "C"
