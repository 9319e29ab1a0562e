// Host side of the C-ABI declared in include/evt_b200.h: plan objects, TMA
// descriptor encoding, loading of generated kernel images and launches.
// Uses the CUDA runtime (statically linked) and reaches the few driver entry
// points it needs through cudaGetDriverEntryPoint, so the library loads in a
// process without a driver (symbols resolve; calls return EVTB_ENODRIVER).
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/evt_b200.h"
#include "evtb_internal.h"
#include "conv_sm100.cuh"
#include "gemm_sm100.cuh"
#include "reduce_apply.cuh"
#include "spmm.cuh"

namespace {

thread_local std::string g_last_error;

void set_error(const std::string& s) { g_last_error = s; }

// ---------------------------------------------------------------------------
// driver entry points
// ---------------------------------------------------------------------------
struct Driver {
  bool ok = false;
  std::string why;
  CUresult (*TensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
  CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*ModuleUnload)(CUmodule) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                           unsigned, CUstream, void**, void**) = nullptr;
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*OccupancyMaxActiveClusters)(int*, CUfunction, const CUlaunchConfig*) = nullptr;
  CUresult (*OccupancyMaxActiveBlocksPerMultiprocessor)(int*, CUfunction, int, size_t) = nullptr;
};

template <typename F>
bool load_entry(const char* name, F& fn, std::string& why) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || p == nullptr || q != cudaDriverEntryPointSuccess) {
    why = std::string("driver entry point ") + name + " unavailable: " + cudaGetErrorString(e);
    (void)cudaGetLastError();
    return false;
  }
  fn = reinterpret_cast<F>(p);
  return true;
}

Driver& driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0) {
      d.why = std::string("no CUDA device: ") + cudaGetErrorString(e);
      (void)cudaGetLastError();
      return;
    }
    (void)cudaFree(nullptr);  // make sure the primary context exists and is current
    bool ok = true;
    ok = ok && load_entry("cuTensorMapEncodeTiled", d.TensorMapEncodeTiled, d.why);
    ok = ok && load_entry("cuModuleLoadData", d.ModuleLoadData, d.why);
    ok = ok && load_entry("cuModuleUnload", d.ModuleUnload, d.why);
    ok = ok && load_entry("cuModuleGetFunction", d.ModuleGetFunction, d.why);
    ok = ok && load_entry("cuFuncSetAttribute", d.FuncSetAttribute, d.why);
    ok = ok && load_entry("cuLaunchKernel", d.LaunchKernel, d.why);
    ok = ok && load_entry("cuGetErrorString", d.GetErrorString, d.why);
    ok = ok && load_entry("cuOccupancyMaxActiveClusters", d.OccupancyMaxActiveClusters, d.why);
    ok = ok && load_entry("cuOccupancyMaxActiveBlocksPerMultiprocessor", d.OccupancyMaxActiveBlocksPerMultiprocessor, d.why);
    d.ok = ok;
  });
  return d;
}

int cu_fail(const char* what, CUresult r) {
  const char* s = nullptr;
  if (driver().GetErrorString) driver().GetErrorString(r, &s);
  set_error(std::string(what) + ": " + (s ? s : "unknown CUDA driver error"));
  return EVTB_ECUDA;
}

// ---------------------------------------------------------------------------
// TMA descriptors for the GEMM operands
// ---------------------------------------------------------------------------
// inner: contiguous logical dim; outer: the other matrix dim; batch last.
int encode_operand_map(CUtensorMap* map, const void* base, int64_t inner, int64_t outer,
                       int64_t batch, int64_t stride_outer, int64_t stride_batch, uint32_t box_inner,
                       uint32_t box_outer) {
  Driver& d = driver();
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) {
    set_error("GEMM operand base address is not 16-byte aligned");
    return EVTB_EINVAL;
  }
  if (stride_outer < inner && outer > 1) {
    // rows may not overlap; (outer == 1 leaves the stride free)
    set_error("GEMM operand stride smaller than its contiguous extent");
    return EVTB_EINVAL;
  }
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer),
                        static_cast<cuuint64_t>(batch)};
  int64_t so = stride_outer, sb = stride_batch;
  if (outer == 1 && (so * 2) % 16 != 0) so = ((inner + 7) / 8) * 8;
  if (batch == 1) sb = so * outer;
  if ((so * 2) % 16 != 0 || (sb * 2) % 16 != 0 || so <= 0 || sb <= 0) {
    set_error("GEMM operand strides must be positive multiples of 8 elements (16 bytes)");
    return EVTB_EINVAL;
  }
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(so) * 2, static_cast<cuuint64_t>(sb) * 2};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = d.TensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base),
                                      dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cu_fail("cuTensorMapEncodeTiled", r);
  return EVTB_OK;
}

// Activation tensor of a convolution, channels-last [n, h, w, c]: a 4-D map (c, w, h, n) whose
// box is 64 channels x bq x bp x bn positions, traversed with the convolution stride.  To load
// bq elements at stride s the box extent must be bq * s.
int encode_activation_map(CUtensorMap* map, const void* base, int c, int w, int h, int n, int bq, int bp, int bn,
                          int sw, int sh, long long xs_w = 0, long long xs_h = 0, long long xs_n = 0) {
  Driver& d = driver();
  if (xs_w == 0 && xs_h == 0 && xs_n == 0) {      // contiguous
    xs_w = c;
    xs_h = 1ll * c * w;
    xs_n = 1ll * c * w * h;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) {
    set_error("convolution operand base address is not 16-byte aligned");
    return EVTB_EINVAL;
  }
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(c), static_cast<cuuint64_t>(w), static_cast<cuuint64_t>(h),
                        static_cast<cuuint64_t>(n)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(xs_w) * 2, static_cast<cuuint64_t>(xs_h) * 2,
                           static_cast<cuuint64_t>(xs_n) * 2};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(bq * sw), static_cast<cuuint32_t>(bp * sh),
                       static_cast<cuuint32_t>(bn)};
  cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(sw), static_cast<cuuint32_t>(sh), 1};
  CUresult r = d.TensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(base), dims, strides,
                                      box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cu_fail("cuTensorMapEncodeTiled(activation)", r);
  return EVTB_OK;
}

// Result tensor written by the epilogue warps' bulk stores: dims (columns, rows, batch), box
// 32 x 32 x 1 of 16-bit elements, 64-byte swizzle = the layout of a warp's staging tile.
int encode_store_map(CUtensorMap* map, void* base, int64_t cols, int64_t rows, int64_t batch, int64_t stride_row,
                     int64_t stride_batch) {
  Driver& d = driver();
  if (base == nullptr || (reinterpret_cast<uintptr_t>(base) & 15u) != 0) {
    set_error("TMA-stored result is null or not 16-byte aligned");
    return EVTB_EINVAL;
  }
  int64_t sr = rows > 1 ? stride_row : ((cols + 7) / 8) * 8;
  int64_t sb = batch > 1 ? stride_batch : sr * rows;
  if (sb % 8 != 0) sb = ((sb + 7) / 8) * 8;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(sr) * 2, static_cast<cuuint64_t>(sb) * 2};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = d.TensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, base, dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                                      CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cu_fail("cuTensorMapEncodeTiled(result)", r);
  return EVTB_OK;
}

int ceil_div(int a, int b) { return (a + b - 1) / b; }

constexpr long long kIntMax = 0x7fffffffLL;

// One launch of a tensor-core kernel.  (Programmatic dependent launch between consecutive kernels was
// tried here -- griddepcontrol.launch_dependents / wait after the kernels' set-up, launches with
// programmatic stream serialisation -- and taken out again: the BERT-large and ResNet-50 steps changed by
// less than 0.5 % either way; the sum of the kernels' own times is the step time.)
CUresult launch_tensor_kernel(CUfunction fn, int grid, int threads, int smem, CUstream stream, void** args) {
  return driver().LaunchKernel(fn, grid, 1, 1, threads, 1, 1, smem, stream, args, nullptr);
}

// x as a strided view: all three strides or none, positive multiples of 8 elements
const char* check_x_strides(const evtb_conv& g, bool allowed) {
  if (g.x_stride_w == 0 && g.x_stride_h == 0 && g.x_stride_n == 0) return nullptr;
  if (!allowed) return "x strides apply to the forward convolution and the weight gradient only";
  if (g.x_stride_w <= 0 || g.x_stride_h <= 0 || g.x_stride_n <= 0 || g.x_stride_w % 8 != 0 || g.x_stride_h % 8 != 0 ||
      g.x_stride_n % 8 != 0)
    return "x strides must all be given, positive and multiples of 8 elements";
  return nullptr;
}

// Fills plan->conv: parity classes, taps, the 128-position box and the tile counts.
int plan_convolution(const evtb_desc& d, evtb::ConvParams& cp, int* grid, int sm_count) {
  const evtb_conv& g = d.conv;
  const bool dgrad = d.kind == EVTB_CONV_DGRAD;
  if (g.N <= 0 || g.H <= 0 || g.W <= 0 || g.C <= 0 || g.K <= 0 || g.R <= 0 || g.S <= 0 || g.P <= 0 || g.Q <= 0 ||
      g.stride_h <= 0 || g.stride_w <= 0 || g.dil_h <= 0 || g.dil_w <= 0 || g.pad_h < 0 || g.pad_w < 0) {
    set_error("convolution plan: non-positive geometry");
    return EVTB_EINVAL;
  }
  if (g.P != (g.H + 2 * g.pad_h - g.dil_h * (g.R - 1) - 1) / g.stride_h + 1 ||
      g.Q != (g.W + 2 * g.pad_w - g.dil_w * (g.S - 1) - 1) / g.stride_w + 1) {
    set_error("convolution plan: P, Q do not match H, W, filter, padding and stride");
    return EVTB_EINVAL;
  }
  if (const char* why = check_x_strides(g, !dgrad)) {
    set_error(std::string("convolution plan: ") + why);
    return EVTB_EINVAL;
  }
  if (g.C % 64 != 0 || g.K % 64 != 0) {
    set_error("convolution plan: channel counts must be multiples of 64");
    return EVTB_EINVAL;
  }
  if (d.tile_n != 64 && d.tile_n != 128 && d.tile_n != 256) {
    set_error("convolution plan: tile_n must be 64, 128 or 256");
    return EVTB_EINVAL;
  }
  if (dgrad && (g.dil_h != 1 || g.dil_w != 1)) {
    set_error("convolution data gradient: dilation must be 1");
    return EVTB_EINVAL;
  }
  if (dgrad && g.stride_h * g.stride_w > evtb::kConvMaxClasses) {
    set_error("convolution data gradient: stride_h * stride_w must be at most 4");
    return EVTB_EINVAL;
  }
  if (g.stride_h > 127 || g.stride_w > 127 || g.R * g.S > 255) {
    set_error("convolution plan: stride or filter too large");
    return EVTB_EINVAL;
  }
  std::memset(&cp, 0, sizeof(cp));
  cp.On = g.N;
  cp.w_c = g.C;
  if (!dgrad) {
    cp.Oh = g.P; cp.Ow = g.Q; cp.NT = g.K; cp.red = g.C;
    cp.a_sh = g.stride_h; cp.a_sw = g.stride_w; cp.o_sh = 1; cp.o_sw = 1;
    cp.nclasses = 1;
    evtb::ConvClass& k = cp.cls[0];
    k.th = g.P; k.tw = g.Q;
    if (g.R * g.S > evtb::kConvMaxTaps) {
      set_error("convolution forward: more than 16 filter taps (use an explicit patch matrix and the GEMM)");
      return EVTB_EINVAL;
    }
    for (int r = 0; r < g.R; ++r)
      for (int s2 = 0; s2 < g.S; ++s2) {
        const int dh = r * g.dil_h - g.pad_h, dw = s2 * g.dil_w - g.pad_w;
        if (dh < -128 || dh > 127 || dw < -128 || dw > 127) {
          set_error("convolution forward: tap offset out of range");
          return EVTB_EINVAL;
        }
        k.dh[k.ntaps] = static_cast<signed char>(dh);
        k.dw[k.ntaps] = static_cast<signed char>(dw);
        k.rs[k.ntaps] = static_cast<unsigned char>(r * g.S + s2);
        ++k.ntaps;
      }
  } else {
    cp.Oh = g.H; cp.Ow = g.W; cp.NT = g.C; cp.red = g.K;
    cp.a_sh = 1; cp.a_sw = 1; cp.o_sh = g.stride_h; cp.o_sw = g.stride_w;
    cp.nclasses = 0;
    for (int a = 0; a < g.stride_h; ++a)
      for (int b = 0; b < g.stride_w; ++b) {
        if (a >= g.H || b >= g.W) continue;
        evtb::ConvClass& k = cp.cls[cp.nclasses++];
        k.o_oh = a; k.o_ow = b;
        k.th = ceil_div(g.H - a, g.stride_h);
        k.tw = ceil_div(g.W - b, g.stride_w);
        for (int r = 0; r < g.R; ++r) {
          if ((a + g.pad_h - r) % g.stride_h != 0) continue;
          for (int s2 = 0; s2 < g.S; ++s2) {
            if ((b + g.pad_w - s2) % g.stride_w != 0) continue;
            if (k.ntaps >= evtb::kConvMaxTaps) {
              set_error("convolution data gradient: more than 16 filter taps per output position");
              return EVTB_EINVAL;
            }
            // floor division is exact here: the remainders were checked above
            k.dh[k.ntaps] = static_cast<signed char>((a + g.pad_h - r) / g.stride_h);
            k.dw[k.ntaps] = static_cast<signed char>((b + g.pad_w - s2) / g.stride_w);
            k.rs[k.ntaps] = static_cast<unsigned char>(r * g.S + s2);
            ++k.ntaps;
          }
        }
      }
  }
  cp.M = cp.On * cp.Oh * cp.Ow;
  // the box of 128 positions that covers the tile grids with the fewest boxes (ties: widest rows)
  long long best = -1;
  for (int bq = 128; bq >= 1; bq /= 2)
    for (int bp = 128 / bq; bp >= 1; bp /= 2) {
      const int bn = 128 / (bq * bp);
      if (bq * cp.a_sw > 256 || bp * cp.a_sh > 256) continue;
      long long boxes = 0;
      for (int c = 0; c < cp.nclasses; ++c)
        boxes += 1ll * ceil_div(cp.cls[c].tw, bq) * ceil_div(cp.cls[c].th, bp) * ceil_div(cp.On, bn);
      if (best < 0 || boxes < best) {
        best = boxes;
        cp.bq = bq; cp.bp = bp; cp.bn = bn;
      }
    }
  cp.boxes_n = ceil_div(cp.On, cp.bn);
  cp.tiles_n = ceil_div(cp.NT, d.tile_n);
  int first = 0;
  for (int c = 0; c < cp.nclasses; ++c) {
    evtb::ConvClass& k = cp.cls[c];
    k.boxes_w = ceil_div(k.tw, cp.bq);
    k.boxes_h = ceil_div(k.th, cp.bp);
    k.first_tile = first;
    first += k.boxes_w * k.boxes_h * cp.boxes_n * cp.tiles_n;
  }
  cp.num_tiles = first;
  *grid = first < sm_count ? first : sm_count;
  return EVTB_OK;
}

}  // namespace

namespace evtb {

void set_last_error(const std::string& text) { set_error(text); }

int current_device_sm_count() {
  static int cached[64] = {0};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) {
    (void)cudaGetLastError();
    return 0;
  }
  if (dev < 64 && cached[dev] > 0) return cached[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  if (dev < 64) cached[dev] = n;
  return n;
}

}  // namespace evtb

// ---------------------------------------------------------------------------
// plan
// ---------------------------------------------------------------------------
struct evtb_plan {
  evtb_desc d{};
  std::string image_path, entry;
  CUmodule module = nullptr;
  CUfunction fn = nullptr;
  int sm_count = 0;
  int grid = 0;
  int main_operands = 0;
  size_t workspace = 0;
  // GEMM
  int tiles_m = 0, tiles_n = 0;
  int splits = 1, kb_per_split = 0;
  size_t partial_bytes = 0;
  void* profile_buffer = nullptr;
  // convolution: everything of ConvParams that does not depend on the operand addresses
  evtb::ConvParams conv{};
  // convolution weight gradient
  evtb::WgradGeom wg{};
  // SpMM
  CUfunction prep_fn = nullptr;
  int t_long = 0, task_len = 0, max_tasks = 0, long_ctas = 0, prep_grid = 0;
  size_t spmm_tasks_off = 0, spmm_scratch_off = 0;
};

extern "C" {

int evtb_version(void) { return 2; }

const char* evtb_status_string(int status) {
  switch (status) {
    case EVTB_OK: return "ok";
    case EVTB_EINVAL: return "invalid plan descriptor or argument";
    case EVTB_ECUDA: return "CUDA call failed";
    case EVTB_ENOTFOUND: return "kernel image or entry point not found";
    case EVTB_ENODRIVER: return "no CUDA driver or device available";
    case EVTB_EDEVICE_TIMEOUT: return "a bounded device-side wait ran out";
    case EVTB_ETOOLARGE: return "problem exceeds the fixed size limit of this entry point";
    default: return "unknown status";
  }
}

const char* evtb_last_error(void) { return g_last_error.c_str(); }

int evtb_plan_create(const evtb_desc* desc, evtb_plan** out) {
  if (desc == nullptr || out == nullptr) {
    set_error("null argument");
    return EVTB_EINVAL;
  }
  *out = nullptr;
  const evtb_desc& d = *desc;
  if (d.kind < EVTB_GEMM || d.kind > EVTB_CONV_WGRAD) {
    set_error("unknown plan kind");
    return EVTB_EINVAL;
  }
  if (d.M <= 0 || d.N <= 0 || d.image_path == nullptr || d.entry == nullptr) {
    set_error("plan needs positive sizes, an image path and an entry name");
    return EVTB_EINVAL;
  }
  if (d.n_epilogue_ptrs < 0 || d.n_epilogue_ptrs > evtb::kMaxEpiPtrs) {
    set_error("too many epilogue pointer slots");
    return EVTB_EINVAL;
  }
  // the kernels index with 32-bit integers: sizes, strides and the number of work units must fit
  {
    const long long k = d.K > 0 ? d.K : 1, l = d.L > 0 ? d.L : 1;
    const long long strides[4] = {d.a.stride_outer, d.a.stride_batch, d.b.stride_outer, d.b.stride_batch};
    bool fits = d.M <= kIntMax && d.N <= kIntMax && k <= kIntMax && l <= kIntMax;
    if (d.kind == EVTB_GEMM || d.kind == EVTB_BGEMM)
      for (long long s : strides) fits = fits && s >= 0;
    if (fits && (d.kind == EVTB_GEMM || d.kind == EVTB_BGEMM) && d.tile_n > 0) {
      const long long tm = (d.M + 127) / 128, tn = (d.N + d.tile_n - 1) / d.tile_n;
      const long long splits = d.split_k > 1 ? d.split_k : 1;
      // tm * tn * l * splits without overflowing 64 bits
      fits = tm <= kIntMax / tn && tm * tn <= kIntMax / l && tm * tn * l <= kIntMax / splits;
    }
    if (!fits) {
      set_error("plan: a size, a stride or the number of work units does not fit 32-bit indexing");
      return EVTB_EINVAL;
    }
  }
  if (d.kind == EVTB_GEMM || d.kind == EVTB_BGEMM) {
    if (d.K <= 0 || d.L <= 0 || (d.kind == EVTB_GEMM && d.L != 1)) {
      set_error("GEMM needs K > 0 and L == 1 (L >= 1 for batched)");
      return EVTB_EINVAL;
    }
    if (d.dtype != EVTB_F16 && d.dtype != EVTB_BF16) {
      set_error("GEMM operands must be f16 or bf16");
      return EVTB_EINVAL;
    }
    if (d.row_resident != 0) {
      if (d.tile_n != 512 || d.N > 512 || d.split_k > 1 || d.cta_pair != 0 || d.stages < 2 || d.stages > 8) {
        set_error("a row-resident GEMM needs tile_n = 512, N <= 512, no split-K, no CTA pair");
        return EVTB_EINVAL;
      }
    } else if (d.tile_n < 32 || d.tile_n > 256 || d.tile_n % 32 != 0 || d.stages < 2 || d.stages > 8) {
      set_error("GEMM tile_n must be a multiple of 32 in [32,256] and 2 <= stages <= 8");
      return EVTB_EINVAL;
    }
    if (d.b.major == EVTB_MAJOR_MN && d.tile_n % 64 != 0) {
      set_error("an MN-major B operand needs tile_n % 64 == 0");
      return EVTB_EINVAL;
    }
    if (d.n_tma_stores < 0 || d.n_tma_stores > evtb::kMaxTmaStores) {
      set_error("GEMM plan: at most 4 results can leave through TMA stores");
      return EVTB_EINVAL;
    }
    for (int i = 0; i < d.n_tma_stores; ++i) {
      const evtb_tma_store& ts = d.tma_stores[i];
      if (ts.slot < 0 || ts.slot >= d.n_epilogue_ptrs || ts.stride_row % 8 != 0 || ts.stride_batch % 8 != 0 ||
          (d.M > 1 && ts.stride_row < d.N) || (d.L > 1 && ts.stride_batch <= 0)) {
        set_error("GEMM plan: bad TMA store description (slot or strides)");
        return EVTB_EINVAL;
      }
    }
    if (d.cta_pair != 0 && d.tile_n != 128 && d.tile_n != 256) {
      set_error("a CTA-pair GEMM needs tile_n 128 or 256");
      return EVTB_EINVAL;
    }
  }
  if (d.smem_bytes < 0 || d.smem_bytes > 227 * 1024 || d.threads <= 0 || d.threads > 1024) {
    set_error("bad shared-memory size or CTA size");
    return EVTB_EINVAL;
  }
  Driver& drv = driver();
  if (!drv.ok) {
    set_error(drv.why);
    return EVTB_ENODRIVER;
  }
  evtb_plan* p = new evtb_plan();
  p->d = d;
  p->image_path = d.image_path;
  p->entry = d.entry;
  p->d.image_path = p->image_path.c_str();
  p->d.entry = p->entry.c_str();

  std::ifstream f(p->image_path, std::ios::binary);
  if (!f) {
    set_error("cannot open kernel image " + p->image_path);
    delete p;
    return EVTB_ENOTFOUND;
  }
  std::vector<char> image((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  image.push_back('\0');
  CUresult r = drv.ModuleLoadData(&p->module, image.data());
  if (r != CUDA_SUCCESS) {
    int rc = cu_fail("cuModuleLoadData", r);
    delete p;
    return rc;
  }
  r = drv.ModuleGetFunction(&p->fn, p->module, p->entry.c_str());
  if (r != CUDA_SUCCESS) {
    cu_fail("cuModuleGetFunction", r);
    drv.ModuleUnload(p->module);
    delete p;
    return EVTB_ENOTFOUND;
  }
  if (d.smem_bytes > 48 * 1024) {
    r = drv.FuncSetAttribute(p->fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, d.smem_bytes);
    if (r != CUDA_SUCCESS) {
      int rc = cu_fail("cuFuncSetAttribute(max dynamic shared memory)", r);
      drv.ModuleUnload(p->module);
      delete p;
      return rc;
    }
  }
  p->sm_count = d.sm_count;
  if (p->sm_count <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&p->sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  if ((d.kind == EVTB_GEMM || d.kind == EVTB_BGEMM) && d.cta_pair != 0) {
    // pair tiles are 256 rows; the grid is two CTAs for every cluster the device holds at once
    p->tiles_m = static_cast<int>((d.M + 2 * evtb::kBM - 1) / (2 * evtb::kBM));
    p->tiles_n = static_cast<int>((d.N + d.tile_n - 1) / d.tile_n);
    const long long tiles = 1ll * p->tiles_m * p->tiles_n * d.L;
    const int num_k = static_cast<int>((d.K + evtb::kBK - 1) / evtb::kBK);
    p->splits = d.split_k > 1 ? d.split_k : 1;
    if (p->splits > num_k) p->splits = num_k;
    p->kb_per_split = (num_k + p->splits - 1) / p->splits;
    p->splits = (num_k + p->kb_per_split - 1) / p->kb_per_split;   // no empty unit
    if (p->splits > 1) {
      // every CTA of a pair parks its own 128 x tile_n half: 2 * tiles half tiles
      p->partial_bytes = sizeof(float) * static_cast<size_t>(2 * tiles) * evtb::kBM * d.tile_n;
      p->workspace = p->partial_bytes + sizeof(unsigned int) * static_cast<size_t>(2 * tiles);
    }
    p->main_operands = 2;
    CUlaunchAttribute attr;
    std::memset(&attr, 0, sizeof(attr));
    attr.id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
    attr.value.clusterDim.x = 2;
    attr.value.clusterDim.y = 1;
    attr.value.clusterDim.z = 1;
    CUlaunchConfig cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDimX = static_cast<unsigned>(p->sm_count / 2 * 2);
    cfg.gridDimY = cfg.gridDimZ = 1;
    cfg.blockDimX = static_cast<unsigned>(d.threads);
    cfg.blockDimY = cfg.blockDimZ = 1;
    cfg.sharedMemBytes = static_cast<unsigned>(d.smem_bytes);
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    r = drv.OccupancyMaxActiveClusters(&clusters, p->fn, &cfg);
    if (r != CUDA_SUCCESS || clusters <= 0) {
      int rc = r != CUDA_SUCCESS ? cu_fail("cuOccupancyMaxActiveClusters", r) : EVTB_ECUDA;
      if (r == CUDA_SUCCESS) set_error("the device cannot hold a single CTA pair of this kernel");
      drv.ModuleUnload(p->module);
      delete p;
      return rc;
    }
    if (clusters > p->sm_count / 2) clusters = p->sm_count / 2;
    const long long units = tiles * p->splits;
    p->grid = 2 * static_cast<int>(units < clusters ? units : clusters);
  } else if (d.kind == EVTB_GEMM || d.kind == EVTB_BGEMM) {
    p->tiles_m = static_cast<int>((d.M + evtb::kBM - 1) / evtb::kBM);
    p->tiles_n = static_cast<int>((d.N + d.tile_n - 1) / d.tile_n);
    const long long tiles = 1ll * p->tiles_m * p->tiles_n * d.L;
    const int num_k = static_cast<int>((d.K + evtb::kBK - 1) / evtb::kBK);
    p->splits = d.split_k > 1 ? d.split_k : 1;
    if (p->splits > num_k) p->splits = num_k;
    p->kb_per_split = (num_k + p->splits - 1) / p->splits;
    p->splits = (num_k + p->kb_per_split - 1) / p->kb_per_split;   // no empty unit
    const long long units = tiles * p->splits;
    p->grid = static_cast<int>(units < p->sm_count ? units : p->sm_count);
    p->main_operands = 2;
    if (p->splits > 1) {
      p->partial_bytes = sizeof(float) * static_cast<size_t>(tiles) * evtb::kBM * d.tile_n;
      p->workspace = p->partial_bytes + sizeof(unsigned int) * static_cast<size_t>(tiles);
    }
  } else if (d.kind == EVTB_CONV_WGRAD) {
    p->main_operands = 2;
    const evtb_conv& g = d.conv;
    const char* bad = nullptr;
    if (d.dtype != EVTB_F16 && d.dtype != EVTB_BF16) bad = "weight gradient: operands must be f16 or bf16";
    else if (g.N <= 0 || g.H <= 0 || g.W <= 0 || g.C <= 0 || g.K <= 0 || g.R <= 0 || g.S <= 0 || g.P <= 0 || g.Q <= 0 ||
             g.stride_h <= 0 || g.stride_w <= 0 || g.dil_h <= 0 || g.dil_w <= 0 || g.pad_h < 0 || g.pad_w < 0)
      bad = "weight gradient: non-positive geometry";
    else if (g.P != (g.H + 2 * g.pad_h - g.dil_h * (g.R - 1) - 1) / g.stride_h + 1 ||
             g.Q != (g.W + 2 * g.pad_w - g.dil_w * (g.S - 1) - 1) / g.stride_w + 1)
      bad = "weight gradient: P, Q do not match H, W, filter, padding and stride";
    else if (check_x_strides(g, true) != nullptr) bad = "weight gradient: x strides must all be given, positive and multiples of 8 elements";
    else if (g.C % 64 != 0 || g.K % 8 != 0) bad = "weight gradient: C must be a multiple of 64 and K of 8";
    else if ((d.tile_n != 64 && d.tile_n != 128 && d.tile_n != 256) || g.C % d.tile_n != 0)
      bad = "weight gradient: tile_n must be 64, 128 or 256 and divide C";
    else if (d.M != g.K || d.N != 1ll * g.R * g.S * g.C) bad = "weight gradient: M must be K and N must be R*S*C";
    else if (d.stages < 2 || d.stages > 8) bad = "weight gradient: 2 <= stages <= 8";
    else if (d.n_tma_stores < 0 || d.n_tma_stores > evtb::kMaxTmaStores) bad = "weight gradient: at most 4 TMA-stored results";
    if (bad != nullptr) {
      set_error(bad);
      drv.ModuleUnload(p->module);
      delete p;
      return EVTB_EINVAL;
    }
    evtb::WgradGeom& w = p->wg;
    w.S = g.S; w.C = g.C;
    w.stride_h = g.stride_h; w.stride_w = g.stride_w; w.pad_h = g.pad_h; w.pad_w = g.pad_w;
    w.dil_h = g.dil_h; w.dil_w = g.dil_w;
    // the box of 64 output positions that covers N x P x Q with the fewest boxes (ties: widest rows)
    long long best = -1;
    for (int bq = 64; bq >= 1; bq /= 2)
      for (int bp = 64 / bq; bp >= 1; bp /= 2) {
        const int bn = 64 / (bq * bp);
        if (bq * g.stride_w > 256 || bp * g.stride_h > 256) continue;
        const long long boxes = 1ll * ceil_div(g.Q, bq) * ceil_div(g.P, bp) * ceil_div(g.N, bn);
        if (best < 0 || boxes < best) {
          best = boxes;
          w.bq = bq; w.bp = bp; w.bn = bn;
        }
      }
    w.boxes_w = ceil_div(g.Q, w.bq);
    w.boxes_h = ceil_div(g.P, w.bp);
    w.boxes_n = ceil_div(g.N, w.bn);
    p->tiles_m = static_cast<int>((d.M + evtb::kBM - 1) / evtb::kBM);
    p->tiles_n = static_cast<int>(d.N / d.tile_n);
    const long long tiles = 1ll * p->tiles_m * p->tiles_n;
    const int num_k = static_cast<int>(best);
    p->splits = d.split_k > 1 ? d.split_k : 1;
    if (p->splits > num_k) p->splits = num_k;
    p->kb_per_split = (num_k + p->splits - 1) / p->splits;
    p->splits = (num_k + p->kb_per_split - 1) / p->kb_per_split;
    const long long units = tiles * p->splits;
    p->grid = static_cast<int>(units < p->sm_count ? units : p->sm_count);
    if (p->splits > 1) {
      p->partial_bytes = sizeof(float) * static_cast<size_t>(tiles) * evtb::kBM * d.tile_n;
      p->workspace = p->partial_bytes + sizeof(unsigned int) * static_cast<size_t>(tiles);
    }
  } else if (d.kind == EVTB_CONV_FPROP || d.kind == EVTB_CONV_DGRAD) {
    p->main_operands = 2;
    int rc = (d.dtype == EVTB_F16 || d.dtype == EVTB_BF16) ? plan_convolution(d, p->conv, &p->grid, p->sm_count)
                                                           : EVTB_EINVAL;
    if (rc != EVTB_OK) {
      if (d.dtype != EVTB_F16 && d.dtype != EVTB_BF16) set_error("convolution operands must be f16 or bf16");
      drv.ModuleUnload(p->module);
      delete p;
      return rc;
    }
  } else if (d.kind == EVTB_SPMM) {
    // operands [crow(int32), col(int32), val(fp32)|0, dinv(fp32)|0, X]; M = rows, N = F, K = nnz;
    // rows_per_cta = work items (rows + nonzeros) per warp; tile_n = padded feature width
    p->main_operands = 5;
    if (d.K < 0 || d.rows_per_cta < 0 || d.stages < 0 || d.tile_n < d.N || d.tile_n % 8 != 0 ||
        d.M + d.K > 0x7fffff00LL || d.threads % 32 != 0) {
      set_error("SpMM plan: bad nnz, row-length threshold, task length or padded width");
      drv.ModuleUnload(p->module);
      delete p;
      return EVTB_EINVAL;
    }
    r = drv.ModuleGetFunction(&p->prep_fn, p->module, "evtb_spmm_prep_kernel");
    if (r != CUDA_SUCCESS) {
      cu_fail("cuModuleGetFunction(evtb_spmm_prep_kernel)", r);
      drv.ModuleUnload(p->module);
      delete p;
      return EVTB_ENOTFOUND;
    }
    p->t_long = d.rows_per_cta > 0 ? d.rows_per_cta : 64;
    p->task_len = d.stages > 0 ? d.stages : 1024;
    // rows longer than t_long: fewer than nnz / t_long of them; every one adds at most one
    // partly filled task to the nnz / task_len full ones
    const long long max_tasks = d.K / (p->t_long + 1) + d.K / p->task_len + 2;
    p->max_tasks = static_cast<int>(max_tasks);
    auto up256 = [](size_t x) { return (x + 255) & ~static_cast<size_t>(255); };
    p->spmm_tasks_off = up256(sizeof(unsigned int) * (1 + static_cast<size_t>(max_tasks)));
    p->spmm_scratch_off = p->spmm_tasks_off + up256(sizeof(evtb::SpmmTask) * static_cast<size_t>(max_tasks));
    p->workspace = p->spmm_scratch_off + sizeof(float) * static_cast<size_t>(max_tasks) * d.tile_n;
    const int wpc = d.threads / 32;
    const int g = d.tile_n / 8 < 32 ? d.tile_n / 8 : 32;            // lanes per row (power of two by construction)
    const int rows_per_cta = wpc * (32 / (g > 0 ? g : 1));
    const long long short_needed = (d.M + rows_per_cta - 1) / rows_per_cta;
    const long long short_cap = 8ll * p->sm_count;
    const int short_ctas = static_cast<int>(short_needed < short_cap ? short_needed : short_cap);
    p->long_ctas = static_cast<int>(max_tasks < 2ll * p->sm_count ? max_tasks : 2ll * p->sm_count);
    p->grid = p->long_ctas + (short_ctas > 0 ? short_ctas : 1);
    p->prep_grid = static_cast<int>((d.M + 255) / 256);
  } else {
    // reduce-apply: persistent CTAs stride over row blocks
    //   SOFTMAX [x, rowmax_out|0, rowsum_out|0]   SOFTMAX_BWD [grad, y]   LAYERNORM [x, mean_out, invstd_out]
    //   LAYERNORM_BWD [grad, x, mean, invstd, gamma]   (reference order, evt_fuser.py:917-924)
    p->main_operands = (d.kind == EVTB_SOFTMAX_BWD) ? 2
                       : (d.kind == EVTB_SOFTMAX || d.kind == EVTB_LAYERNORM) ? 3 : 5;
    const int rpc = d.rows_per_cta > 0 ? d.rows_per_cta : 1;
    const long long blocks = (d.M + rpc - 1) / rpc;
    // CTAs that are resident together (registers decide, not only the thread count); when the row
    // blocks do not fit, every CTA gets the same number of them (3.46 blocks per CTA would make all
    // wait for the quarter that has 4)
    int per_sm = 0;
    if (drv.OccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, p->fn, d.threads, static_cast<size_t>(d.smem_bytes)) != CUDA_SUCCESS ||
        per_sm < 1)
      per_sm = 2048 / d.threads > 0 ? 2048 / d.threads : 1;
    const long long cap = 1ll * p->sm_count * per_sm;
    if (blocks <= cap) {
      p->grid = static_cast<int>(blocks);
    } else {
      const long long iters = (blocks + cap - 1) / cap;
      p->grid = static_cast<int>((blocks + iters - 1) / iters);
    }
  }
  *out = p;
  return EVTB_OK;
}

int evtb_plan_destroy(evtb_plan* plan) {
  if (plan == nullptr) return EVTB_OK;
  if (plan->module != nullptr && driver().ok) driver().ModuleUnload(plan->module);
  delete plan;
  return EVTB_OK;
}

int evtb_plan_workspace_bytes(const evtb_plan* plan, size_t* bytes) {
  if (plan == nullptr || bytes == nullptr) return EVTB_EINVAL;
  *bytes = plan->workspace;
  return EVTB_OK;
}

int evtb_plan_num_main_operands(const evtb_plan* plan, int* n) {
  if (plan == nullptr || n == nullptr) return EVTB_EINVAL;
  *n = plan->main_operands;
  return EVTB_OK;
}

int evtb_plan_set_profile_buffer(evtb_plan* plan, void* device_buffer) {
  if (plan == nullptr) return EVTB_EINVAL;
  plan->profile_buffer = device_buffer;
  return EVTB_OK;
}

int evtb_plan_grid(const evtb_plan* plan, int* ctas) {
  if (plan == nullptr || ctas == nullptr) return EVTB_EINVAL;
  *ctas = plan->grid;
  return EVTB_OK;
}

int evtb_launch_ex(evtb_plan* plan, const void* const* ptrs, int n, void* workspace,
                   void* status_word, evtb_stream stream, const evtb_scalars* scalars) {
  if (plan == nullptr || ptrs == nullptr) {
    set_error("null plan or operand list");
    return EVTB_EINVAL;
  }
  const evtb_desc& d = plan->d;
  if (n != plan->main_operands + d.n_epilogue_ptrs) {
    set_error("operand count does not match the plan");
    return EVTB_EINVAL;
  }
  Driver& drv = driver();
  if (!drv.ok) {
    set_error(drv.why);
    return EVTB_ENODRIVER;
  }
  evtb::EpiParams epi;
  std::memset(&epi, 0, sizeof(epi));
  for (int i = 0; i < d.n_epilogue_ptrs; ++i)
    epi.ptr[i] = const_cast<void*>(ptrs[plan->main_operands + i]);
  if (scalars != nullptr) {
    std::memcpy(epi.scalar, scalars->scalar, sizeof(epi.scalar));
    epi.seed = scalars->seed;
    epi.rng_offset = scalars->rng_offset;
  }

  if (d.kind == EVTB_GEMM || d.kind == EVTB_BGEMM) {
    evtb::GemmParams p;
    std::memset(&p, 0, sizeof(p));
    int rc;
    if (d.a.major == EVTB_MAJOR_K)
      rc = encode_operand_map(&p.tma_a, ptrs[0], d.K, d.M, d.L, d.a.stride_outer, d.a.stride_batch, 64, 128);
    else
      rc = encode_operand_map(&p.tma_a, ptrs[0], d.M, d.K, d.L, d.a.stride_outer, d.a.stride_batch, 64, 64);
    if (rc != EVTB_OK) return rc;
    if (d.b.major == EVTB_MAJOR_K)
      rc = encode_operand_map(&p.tma_b, ptrs[1], d.K, d.N, d.L, d.b.stride_outer, d.b.stride_batch, 64,
                              static_cast<uint32_t>(d.row_resident != 0 ? 256 : d.cta_pair != 0 ? d.tile_n / 2 : d.tile_n));
    else
      rc = encode_operand_map(&p.tma_b, ptrs[1], d.N, d.K, d.L, d.b.stride_outer, d.b.stride_batch, 64, 64);
    if (rc != EVTB_OK) return rc;
    p.M = static_cast<int>(d.M);
    p.N = static_cast<int>(d.N);
    p.K = static_cast<int>(d.K);
    p.L = static_cast<int>(d.L);
    p.tiles_m = plan->tiles_m;
    p.tiles_n = plan->tiles_n;
    p.num_tiles = static_cast<int>(1ll * plan->tiles_m * plan->tiles_n * d.L);
    p.status = static_cast<int*>(status_word);
    p.prof = static_cast<long long*>(plan->profile_buffer);
    for (int i = 0; i < d.n_tma_stores; ++i) {
      const evtb_tma_store& ts = d.tma_stores[i];
      rc = encode_store_map(&epi.tmap[i], epi.ptr[ts.slot], d.N, d.M, d.L, ts.stride_row, ts.stride_batch);
      if (rc != EVTB_OK) return rc;
    }
    p.epi = epi;
    p.splits = plan->splits;
    p.kb_per_split = plan->kb_per_split;
    if (plan->splits > 1) {
      if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) {
        set_error("split-K plan needs a 16-byte aligned workspace of evtb_plan_workspace_bytes() bytes");
        return EVTB_EINVAL;
      }
      p.partial = static_cast<float*>(workspace);
      p.tile_counters = reinterpret_cast<unsigned int*>(static_cast<char*>(workspace) + plan->partial_bytes);
    }
    void* args[1] = {&p};
    CUresult r = launch_tensor_kernel(plan->fn, plan->grid, d.threads, d.smem_bytes, static_cast<CUstream>(stream), args);
    if (r != CUDA_SUCCESS) return cu_fail("cuLaunchKernel(gemm)", r);
    return EVTB_OK;
  }

  if (d.kind == EVTB_CONV_WGRAD) {
    const evtb_conv& g = d.conv;
    evtb::GemmParams p;
    std::memset(&p, 0, sizeof(p));
    p.wg = plan->wg;
    int rc = encode_activation_map(&p.tma_a, ptrs[0], g.K, g.Q, g.P, g.N, p.wg.bq, p.wg.bp, p.wg.bn, 1, 1);
    if (rc != EVTB_OK) return rc;
    rc = encode_activation_map(&p.tma_b, ptrs[1], g.C, g.W, g.H, g.N, p.wg.bq, p.wg.bp, p.wg.bn, g.stride_w, g.stride_h,
                               g.x_stride_w, g.x_stride_h, g.x_stride_n);
    if (rc != EVTB_OK) return rc;
    p.M = static_cast<int>(d.M);
    p.N = static_cast<int>(d.N);
    p.K = g.N * g.P * g.Q;
    p.L = 1;
    p.tiles_m = plan->tiles_m;
    p.tiles_n = plan->tiles_n;
    p.num_tiles = plan->tiles_m * plan->tiles_n;
    p.status = static_cast<int*>(status_word);
    p.prof = nullptr;
    for (int i = 0; i < d.n_tma_stores; ++i) {
      const evtb_tma_store& ts = d.tma_stores[i];
      rc = encode_store_map(&epi.tmap[i], epi.ptr[ts.slot], d.N, d.M, 1, ts.stride_row, ts.stride_batch);
      if (rc != EVTB_OK) return rc;
    }
    p.epi = epi;
    p.splits = plan->splits;
    p.kb_per_split = plan->kb_per_split;
    if (plan->splits > 1) {
      if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) {
        set_error("split weight-gradient plan needs a 16-byte aligned workspace of evtb_plan_workspace_bytes() bytes");
        return EVTB_EINVAL;
      }
      p.partial = static_cast<float*>(workspace);
      p.tile_counters = reinterpret_cast<unsigned int*>(static_cast<char*>(workspace) + plan->partial_bytes);
    }
    void* args[1] = {&p};
    CUresult r = launch_tensor_kernel(plan->fn, plan->grid, d.threads, d.smem_bytes, static_cast<CUstream>(stream), args);
    if (r != CUDA_SUCCESS) return cu_fail("cuLaunchKernel(convolution weight gradient)", r);
    return EVTB_OK;
  }

  if (d.kind == EVTB_CONV_FPROP || d.kind == EVTB_CONV_DGRAD) {
    const evtb_conv& g = d.conv;
    const bool dgrad = d.kind == EVTB_CONV_DGRAD;
    evtb::ConvParams cp = plan->conv;
    int rc = dgrad ? encode_activation_map(&cp.tma_a, ptrs[0], g.K, g.Q, g.P, g.N, cp.bq, cp.bp, cp.bn, 1, 1)
                   : encode_activation_map(&cp.tma_a, ptrs[0], g.C, g.W, g.H, g.N, cp.bq, cp.bp, cp.bn, g.stride_w,
                                           g.stride_h, g.x_stride_w, g.x_stride_h, g.x_stride_n);
    if (rc != EVTB_OK) return rc;
    const int64_t rsc = 1ll * g.R * g.S * g.C;
    rc = encode_operand_map(&cp.tma_b, ptrs[1], rsc, g.K, 1, rsc, rsc * g.K, 64,
                            dgrad ? 64u : static_cast<uint32_t>(d.tile_n));
    if (rc != EVTB_OK) return rc;
    cp.status = static_cast<int*>(status_word);
    cp.prof = nullptr;
    cp.epi = epi;
    void* cargs[1] = {&cp};
    CUresult r = launch_tensor_kernel(plan->fn, plan->grid, d.threads, d.smem_bytes, static_cast<CUstream>(stream), cargs);
    if (r != CUDA_SUCCESS) return cu_fail("cuLaunchKernel(convolution)", r);
    return EVTB_OK;
  }

  if (d.kind == EVTB_SPMM) {
    if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) {
      set_error("SpMM plan needs a 16-byte aligned, once-zeroed workspace of evtb_plan_workspace_bytes() bytes");
      return EVTB_EINVAL;
    }
    if (d.dtype == EVTB_F32 && (reinterpret_cast<uintptr_t>(ptrs[4]) & 31u) != 0) {
      set_error("SpMM: fp32 features must be 32-byte aligned (they are gathered with 256-bit loads)");
      return EVTB_EINVAL;
    }
    evtb::SpmmParams sp;
    std::memset(&sp, 0, sizeof(sp));
    sp.crow = static_cast<const int*>(ptrs[0]);
    sp.col = static_cast<const int*>(ptrs[1]);
    sp.val = static_cast<const float*>(ptrs[2]);
    sp.dinv = static_cast<const float*>(ptrs[3]);
    sp.x = ptrs[4];
    if (sp.crow == nullptr || sp.col == nullptr || sp.x == nullptr || (sp.val == nullptr) == (sp.dinv == nullptr)) {
      set_error("SpMM needs crow, col, X and exactly one of val / dinv");
      return EVTB_EINVAL;
    }
    char* ws = static_cast<char*>(workspace);
    sp.counters = reinterpret_cast<unsigned int*>(ws);
    sp.tasks = reinterpret_cast<evtb::SpmmTask*>(ws + plan->spmm_tasks_off);
    sp.scratch = reinterpret_cast<float*>(ws + plan->spmm_scratch_off);
    sp.rows = static_cast<int>(d.M);
    sp.nnz = static_cast<int>(d.K);
    sp.F = static_cast<int>(d.N);
    sp.t_long = plan->t_long;
    sp.task_len = plan->task_len;
    sp.long_ctas = plan->long_ctas;
    sp.max_tasks = plan->max_tasks;
    sp.status = static_cast<int*>(status_word);
    sp.epi = epi;
    void* sargs[1] = {&sp};
    // task count back to zero, task list of the long rows, then the main launch
    if (cudaMemsetAsync(sp.counters, 0, sizeof(unsigned int), static_cast<cudaStream_t>(stream)) != cudaSuccess) {
      set_error("cudaMemsetAsync(spmm task count) failed");
      (void)cudaGetLastError();
      return EVTB_ECUDA;
    }
    CUresult sr = drv.LaunchKernel(plan->prep_fn, plan->prep_grid, 1, 1, 256, 1, 1, 0, static_cast<CUstream>(stream), sargs, nullptr);
    if (sr != CUDA_SUCCESS) return cu_fail("cuLaunchKernel(spmm preparation)", sr);
    sr = drv.LaunchKernel(plan->fn, plan->grid, 1, 1, d.threads, 1, 1, 0, static_cast<CUstream>(stream), sargs, nullptr);
    if (sr != CUDA_SUCCESS) return cu_fail("cuLaunchKernel(spmm)", sr);
    return EVTB_OK;
  }

  // the reduce-apply family shares one parameter block
  evtb::RowParams p;
  std::memset(&p, 0, sizeof(p));
  if (d.kind == EVTB_LAYERNORM || d.kind == EVTB_SOFTMAX) {
    p.in[0] = ptrs[0];
    p.aux_out[0] = const_cast<void*>(ptrs[1]);
    p.aux_out[1] = const_cast<void*>(ptrs[2]);
  } else {
    for (int i = 0; i < plan->main_operands && i < 5; ++i) p.in[i] = ptrs[i];
  }
  p.rows = static_cast<int>(d.M);
  p.cols = static_cast<int>(d.N);
  p.status = static_cast<int*>(status_word);
  p.epi = epi;
  void* args[1] = {&p};
  CUresult r = drv.LaunchKernel(plan->fn, plan->grid, 1, 1, d.threads, 1, 1, d.smem_bytes,
                                static_cast<CUstream>(stream), args, nullptr);
  if (r != CUDA_SUCCESS) return cu_fail("cuLaunchKernel(row kernel)", r);
  return EVTB_OK;
}

int evtb_launch(evtb_plan* plan, const void* const* ptrs, int n, void* workspace, void* status_word,
                evtb_stream stream) {
  return evtb_launch_ex(plan, ptrs, n, workspace, status_word, stream, nullptr);
}

}  // extern "C"
