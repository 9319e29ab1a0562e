// CSR SpMM with a generated epilogue.
//
//   Y[i, :] = epilogue( sum_{p in row i} w(i, p) * X[col[p], :] )
//   w = val[p]                      (stored edge weights), or
//   w = dinv[i] * dinv[col[p]]      (symmetric normalisation fused: no value array at all)
//
// The reference's kernel (src/cuda/spmm/threadblock/spmm_reduction.h:98-150, launched by
// src/cuda/spmm/kernel/spmm_csr_with_callbacks.h:49-81) gives every row to one sub-warp that
// walks its nonzeros serially, so a hub row of a power-law graph sets the run time.  Here rows
// are split by length:
//
//   short rows (at most t_long nonzeros, almost all rows of a power-law graph): a lane group
//     of G lanes per row, 32 / G rows side by side in a warp, up to U nonzeros of a row in
//     flight; every lane owns 8-column slices and keeps their sums in registers, so the row
//     ends with the epilogue and one store, no cross-lane traffic at all.  The column indices
//     of the next step and the row pointers of the row after next are fetched while the
//     feature rows of this step are in flight.
//   long rows: cut into tasks of task_len nonzeros by a small preparation launch (one thread
//     per row, task list in the workspace).  A CTA takes a task, its warps split the nonzeros,
//     load their column indices 32 at a time (coalesced) and gather with all lanes; the warps'
//     sums meet in shared memory in warp order.  A row of several tasks parks one fp32 partial
//     per task; the last task to arrive adds them in task order and runs the epilogue.
//
// No atomics touch the data: every sum is formed in a fixed order, results are bit-identical
// from run to run.  Feature rows are gathered with 256-bit loads (fp32) / 128-bit loads (16-bit
// types), 8 columns per lane.
#pragma once
#include "reduce_apply.cuh"

namespace evtb {

struct SpmmTask {
  int row, p0, p1;   // nonzeros [p0, p1) of this row
  int k, nk;         // task k of nk of the row
  int base;          // index of the row's first task = its first scratch slot and its counter
};

struct alignas(16) SpmmParams {
  const int* crow;      // [rows + 1]
  const int* col;       // [nnz]
  const float* val;     // [nnz] or null (normalisation fused)
  const float* dinv;    // [rows] (normalisation fused) or null
  const void* x;        // dense features [*, F]
  float* scratch;       // [max_tasks][F_pad] partial sums of multi-task rows
  SpmmTask* tasks;      // [max_tasks]
  unsigned int* counters;   // [0]: number of tasks (zeroed, then written by the preparation launch);
                            // [1 + base]: arrivals per multi-task row, zero on entry and on exit
  int rows, nnz, F;
  int t_long, task_len, long_ctas, max_tasks;
  int* status;
  EpiParams epi;
};

constexpr int DEV_SPMM_TASK_OVERFLOW = 120;

// 8 consecutive feature columns of row `row` as fp32; fp32 features come as one 256-bit load
template <typename T>
__device__ __forceinline__ void gather8(const void* x, long long row, int F, int n, float (&v)[8]) {
  const char* p = reinterpret_cast<const char*>(x) + (row * F + n) * (long long)sizeof(T);
  if constexpr (sizeof(T) == 4) {
    asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
                 : "l"(p));
  } else {
    Vec8<T>::load(p, true, v);
  }
}

template <int VPT, class Epi>
__device__ __forceinline__ void spmm_finish_row(const SpmmParams& p, Epi& epi, int row, int gl, int G,
                                                float (&v)[VPT][8]) {
  EpiCtx c;
  c.ep = &p.epi;
  c.M = p.rows;
  c.N = p.F;
  c.L = 1;
  c.l = 0;
  c.m = row;
  c.m_warp = row;
  c.n0 = 0;
  c.row_ok = true;
  c.lane = gl;
  c.quad = 0;
  c.status = p.status;
  c.stage = nullptr;
  epi.tile_begin(c);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int n = (i * G + gl) * 8;
    if (n < p.F) epi.template visit8<0>(c, n, v[i]);
  }
  epi.tile_end(c);
}

// ---------------------------------------------------------------------------------------
// preparation: one lane per row; a warp writes the tasks of each of its long rows together
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void spmm_prep_body(const SpmmParams& p) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  const int lane = threadIdx.x & 31;
  int b = 0, e = 0;
  if (row < p.rows) {
    b = __ldg(p.crow + row);
    e = __ldg(p.crow + row + 1);
  }
  const int deg = e - b;
  int nk = 0, base = 0;
  if (deg > p.t_long) {
    nk = (deg + p.task_len - 1) / p.task_len;
    base = static_cast<int>(atomicAdd(p.counters, static_cast<unsigned int>(nk)));
    if (base + nk > p.max_tasks) {      // cannot happen with the workspace the plan asks for
      report_status(p.status, DEV_SPMM_TASK_OVERFLOW);
      nk = 0;
    }
  }
  unsigned int todo = __ballot_sync(0xffffffffu, nk > 0);
  while (todo != 0u) {
    const int src = __ffs(todo) - 1;
    todo &= todo - 1;
    const int r_row = __shfl_sync(0xffffffffu, row, src), r_b = __shfl_sync(0xffffffffu, b, src);
    const int r_e = __shfl_sync(0xffffffffu, e, src), r_nk = __shfl_sync(0xffffffffu, nk, src);
    const int r_base = __shfl_sync(0xffffffffu, base, src);
    for (int k = lane; k < r_nk; k += 32) {
      SpmmTask t;
      t.row = r_row;
      t.p0 = r_b + k * p.task_len;
      t.p1 = min(r_e, t.p0 + p.task_len);
      t.k = k;
      t.nk = r_nk;
      t.base = r_base;
      p.tasks[r_base + k] = t;
    }
  }
}

// ---------------------------------------------------------------------------------------
// short rows
// ---------------------------------------------------------------------------------------
template <typename T, int G, int VPT, bool NORM, int U, class Epi>
__device__ __forceinline__ void spmm_short_body(const SpmmParams& p, int gw, int nw) {
  constexpr int RPW = 32 / G;
  const int lane = threadIdx.x & 31, sub = lane / G, gl = lane % G;
  const int stride = nw * RPW;
  int row = gw * RPW + sub;
  if (row >= p.rows) return;
  Epi epi;
  int b = __ldg(p.crow + row), e = __ldg(p.crow + row + 1);
  bool is_long = e - b > p.t_long;
  if (is_long) e = b;
  int nb = 0, ne = 0;
  if (row + stride < p.rows) {
    nb = __ldg(p.crow + row + stride);
    ne = __ldg(p.crow + row + stride + 1);
  }
  int c[U];
  float wv[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    c[u] = (b + u < e) ? __ldg(p.col + b + u) : -1;
    wv[u] = (!NORM && b + u < e) ? __ldg(p.val + b + u) : 0.f;
  }
  int pos = b;
  float acc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  while (row < p.rows) {
    // this step's feature rows (and weights) in flight
    float v[U][VPT][8];
    float w[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (c[u] >= 0) {
        w[u] = NORM ? __ldg(p.dinv + c[u]) : wv[u];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int n = (i * G + gl) * 8;
          if (n < p.F) {
            gather8<T>(p.x, c[u], p.F, n, v[u][i]);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[u][i][j] = 0.f;
          }
        }
      } else {
        w[u] = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) v[u][i][j] = 0.f;
      }
    }
    // next step: the same row's next nonzeros, or the next row of this lane group
    const bool row_done = pos + U >= e;
    int nrow = row, nbb = b, nee = e, npos = pos + U;
    bool nlong = is_long;
    if (row_done) {
      nrow = row + stride;
      nbb = nb;
      nee = ne;
      nlong = nee - nbb > p.t_long;
      if (nlong) nee = nbb;
      npos = nbb;
      const int r2 = nrow + stride;
      if (r2 < p.rows) {
        nb = __ldg(p.crow + r2);
        ne = __ldg(p.crow + r2 + 1);
      } else {
        nb = 0;
        ne = 0;
      }
    }
    int nc[U];
    float nwv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool live = npos + u < nee && nrow < p.rows;
      nc[u] = live ? __ldg(p.col + npos + u) : -1;
      nwv[u] = (!NORM && live) ? __ldg(p.val + npos + u) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(w[u], v[u][i][j], acc[i][j]);
    if (row_done) {
      if (!is_long) {
        if (NORM) {
          const float di = __ldg(p.dinv + row);
#pragma unroll
          for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] *= di;
        }
        spmm_finish_row<VPT>(p, epi, row, gl, G, acc);
      }
#pragma unroll
      for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    }
    row = nrow;
    b = nbb;
    e = nee;
    pos = npos;
    is_long = nlong;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      c[u] = nc[u];
      wv[u] = nwv[u];
    }
  }
}

// ---------------------------------------------------------------------------------------
// long rows: a CTA per task
// ---------------------------------------------------------------------------------------
template <typename T, int G, int VPT, bool NORM, int U, int WPC, class Epi>
__device__ __forceinline__ void spmm_long_body(const SpmmParams& p, float* part /* [WPC][G * VPT * 8] */) {
  constexpr int P = 32 / G;            // nonzeros side by side in a warp
  constexpr int FP = G * VPT * 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / G, gl = lane % G;
  const int ntasks = static_cast<int>(__ldcg(p.counters));
  Epi epi;
  for (int ti = blockIdx.x; ti < ntasks && ti < p.max_tasks; ti += p.long_ctas) {
    const SpmmTask t = p.tasks[ti];
    // this warp's run of the task's nonzeros, in multiples of 32
    const int len = t.p1 - t.p0;
    const int per = ((len + WPC - 1) / WPC + 31) & ~31;
    const int q0 = t.p0 + warp * per;
    const int q1 = min(t.p1, q0 + per);
    float v[VPT][8];
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
    for (int base = q0; base < q1; base += 32) {
      const int q = base + lane;
      int c_l = 0;
      float w_l = 0.f;
      if (q < q1) {
        c_l = __ldg(p.col + q);
        w_l = NORM ? __ldg(p.dinv + c_l) : __ldg(p.val + q);
      }
      const int cnt = min(32, q1 - base);
      for (int k0 = 0; k0 < cnt; k0 += U * P) {
        float xv[U][VPT][8];
        float w[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int src = k0 + u * P + sub;
          const int cc = __shfl_sync(0xffffffffu, c_l, src & 31);
          w[u] = __shfl_sync(0xffffffffu, w_l, src & 31);
          if (src >= cnt) w[u] = 0.f;
#pragma unroll
          for (int i = 0; i < VPT; ++i) {
            const int n = (i * G + gl) * 8;
            if (src < cnt && n < p.F) {
              gather8<T>(p.x, cc, p.F, n, xv[u][i]);
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) xv[u][i][j] = 0.f;
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] = fmaf(w[u], xv[u][i][j], v[i][j]);
      }
    }
    // lane groups -> group 0 (fixed order), warps -> warp 0 through shared memory (warp order)
#pragma unroll
    for (int o = G; o < 32; o <<= 1)
#pragma unroll
      for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += __shfl_xor_sync(0xffffffffu, v[i][j], o);
    if (lane < G) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        float4* dst = reinterpret_cast<float4*>(part + warp * FP + (i * G + gl) * 8);
        dst[0] = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
        dst[1] = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
      }
    }
    __syncthreads();
    if (warp == 0) {
      if (lane < G) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
          for (int w2 = 0; w2 < WPC; ++w2) {
            const float4* src = reinterpret_cast<const float4*>(part + w2 * FP + (i * G + gl) * 8);
            const float4 a = src[0], b2 = src[1];
            v[i][0] += a.x; v[i][1] += a.y; v[i][2] += a.z; v[i][3] += a.w;
            v[i][4] += b2.x; v[i][5] += b2.y; v[i][6] += b2.z; v[i][7] += b2.w;
          }
        }
      }
      bool finish = t.nk == 1;
      if (t.nk > 1) {
        // park this task's partial; the last task of the row to arrive adds them in task order
        if (lane < G) {
#pragma unroll
          for (int i = 0; i < VPT; ++i) {
            float4* dst = reinterpret_cast<float4*>(p.scratch + static_cast<long long>(t.base + t.k) * FP + (i * G + gl) * 8);
            __stcg(dst, make_float4(v[i][0], v[i][1], v[i][2], v[i][3]));
            __stcg(dst + 1, make_float4(v[i][4], v[i][5], v[i][6], v[i][7]));
          }
        }
        __threadfence();
        __syncwarp();
        unsigned int prev = 0;
        if (lane == 0) prev = atomicAdd(p.counters + 1 + t.base, 1u);
        prev = __shfl_sync(0xffffffffu, prev, 0);
        if (prev == static_cast<unsigned int>(t.nk - 1)) {
          __threadfence();
          finish = true;
          if (lane == 0) p.counters[1 + t.base] = 0u;     // clean for the next launch
          if (lane < G) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
#pragma unroll
              for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
              for (int k = 0; k < t.nk; ++k) {
                const float4* src = reinterpret_cast<const float4*>(p.scratch + static_cast<long long>(t.base + k) * FP + (i * G + gl) * 8);
                const float4 a = __ldcg(src), b2 = __ldcg(src + 1);
                v[i][0] += a.x; v[i][1] += a.y; v[i][2] += a.z; v[i][3] += a.w;
                v[i][4] += b2.x; v[i][5] += b2.y; v[i][6] += b2.z; v[i][7] += b2.w;
              }
            }
          }
        }
      }
      if (finish && lane < G) {
        if (NORM) {
          const float di = __ldg(p.dinv + t.row);
#pragma unroll
          for (int i = 0; i < VPT; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i][j] *= di;
        }
        spmm_finish_row<VPT>(p, epi, t.row, gl, G, v);
      }
    }
    __syncthreads();     // `part` is free for the next task
  }
}

// main launch: the first long_ctas CTAs take the tasks of the long rows (the longest pieces of
// work start first), the others the short rows
template <typename T, int G, int VPT, bool NORM, int US, int UL, int WPC, class Epi>
__device__ __forceinline__ void spmm_body(const SpmmParams& p) {
  __shared__ __align__(16) float part[WPC * G * VPT * 8];
  if (static_cast<int>(blockIdx.x) < p.long_ctas) {
    spmm_long_body<T, G, VPT, NORM, UL, WPC, Epi>(p, part);
  } else {
    const int bi = blockIdx.x - p.long_ctas, nb = gridDim.x - p.long_ctas;
    spmm_short_body<T, G, VPT, NORM, US, Epi>(p, (bi * blockDim.x + threadIdx.x) >> 5, (nb * blockDim.x) >> 5);
  }
}

// merge-path split of (rows + nonzeros) used by the SDDMM kernel
__device__ __forceinline__ void merge_path_search(const int* __restrict__ crow, int rows, int nnz, int d,
                                                  int& x, int& y) {
  int lo = d - nnz > 0 ? d - nnz : 0;
  int hi = d < rows ? d : rows;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(crow + mid + 1) <= d - mid - 1) lo = mid + 1; else hi = mid;
  }
  x = lo < rows ? lo : rows;
  y = d - lo;
}

}  // namespace evtb
