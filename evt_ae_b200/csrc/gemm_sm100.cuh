// Persistent, warp-specialised GEMM / batched-GEMM main loop for sm_100a:
//   TMA (tile mode) -> multi-stage shared-memory ring -> tcgen05.mma (one issuing
//   thread) -> fp32 accumulators in tensor memory (two stages) -> tcgen05.ld ->
//   a generated epilogue functor that owns every load, store and reduction.
//
// This replaces the CUTLASS `mma.sync` GEMM the reference instantiates in
// python/gtl/compiler/passes/evt_fuser.py:481-546 (FusedGEMM) and :605-680
// (FusedBMM).  The epilogue protocol (tile_begin / visit / tile_end per thread,
// one accumulator row per thread) plays the role of the visitor callbacks in
// src/cuda/epilogue/threadblock/visitor.hpp:37-89.
//
// Warp roles (64 + 32*EPI_WARPS threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
// owner, warps 2.. = epilogue (warp w reads TMEM lanes 32*(w%4) .. +31; warps that
// share a lane quadrant split the tile's 32-column chunks between them).
#pragma once
#include "sm100_ptx.cuh"

namespace evtb {

constexpr int kBM = 128;      // accumulator rows per tile = TMEM lanes
constexpr int kBK = 64;       // 64 halfs = one 128-byte swizzle row
constexpr int kUmmaK = 16;    // K per tcgen05.mma for 16-bit inputs
constexpr int kMaxEpiPtrs = 24;

// Operands of the generated epilogue.  Slot numbers are fixed at code generation.
constexpr int kMaxTmaStores = 4;
struct alignas(64) EpiParams {
  // results that leave through TMA bulk stores: 3-D maps (columns, rows, batch), box 32 x 32 x 1,
  // 64-byte swizzle (the layout of the epilogue warps' staging tiles)
  CUtensorMap tmap[kMaxTmaStores];
  void* ptr[kMaxEpiPtrs];
  float scalar[8];
  unsigned long long seed;
  unsigned long long rng_offset;
};

// Convolution weight gradient run as a GEMM: dW[k, (r, s, c)] = sum over output positions of
// dy[position, k] * x[position shifted by tap (r, s), c].  Rows are output channels, columns the
// R*S*C filter entries of an output channel, the reduction runs over boxes of 64 output positions
// (bq x bp x bn) that TMA fetches from the two 4-D channels-last tensors: dy at the box itself, x at
// the box moved by the column tile's tap, strided by the convolution stride, zero-filled in the
// padding.  Both operand tiles arrive MN-major (channels contiguous).
struct WgradGeom {
  int bq, bp, bn;                  // box of 64 output positions
  int boxes_w, boxes_h, boxes_n;   // boxes along q, p, n: their product is the reduction length in k-blocks
  int S, C;                        // filter width; channels per tap (a column tile lies inside one tap)
  int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
};

struct alignas(64) GemmParams {
  CUtensorMap tma_a;  // K-major: dims (K, M, L), box (64, 128, 1); MN-major: dims (M, K, L), box (64, 64, 1)
  CUtensorMap tma_b;  // K-major: dims (K, N, L), box (64, BN, 1); MN-major: dims (N, K, L), box (64, 64, 1)
                      // weight gradient: a = dy dims (K, Q, P, N), b = x dims (C, W, H, N), boxes of 64 channels x 64 positions
  int M, N, K, L;
  int tiles_m, tiles_n, num_tiles;
  // split-K: a tile's K range is cut into `splits` units of `kb_per_split` k-blocks; every
  // unit leaves an fp32 partial tile in `partial`, the last one to arrive (counted in
  // `tile_counters`, which start at zero and are left at zero) adds them up in a fixed order
  // and runs the epilogue.  splits == 1: none of this is touched.
  int splits, kb_per_split;
  float* partial;                 // [num_tiles][splits][128][BN]
  unsigned int* tile_counters;    // [num_tiles]
  int* status;
  // -DEVTB_PROFILE builds only: per CTA 8 counters (clock64 ticks): [0] kernel, [1] producer
  // waiting for a free slot, [2] MMA issuer waiting for data, [3] MMA issuer waiting for a
  // free accumulator, [4] epilogue (warp 2) waiting for an accumulator, [5] epilogue working
  long long* prof;
  WgradGeom wg;       // weight-gradient kernels only
  EpiParams epi;
};

#ifdef EVTB_PROFILE
#define EVTB_PROF_T0() const long long prof_t0 = clock64()
#define EVTB_PROF_ADD(var) var += clock64() - prof_t0
#else
#define EVTB_PROF_T0()
#define EVTB_PROF_ADD(var)
#endif

// Convolution kernels (conv_sm100.cuh) walk boxes of output positions instead of row ranges.
struct ConvParams;
struct ConvTile {
  int cls;             // output parity class (strided data gradient), else 0
  int tq0, tp0, tn0;   // first tile-grid position of the box (w, h, image)
  int n0;              // first output channel
};

// What the generated epilogue sees for one accumulator row of one tile.
struct EpiCtx {
  const EpiParams* ep;
  int M, N, L;
  int l;        // batch index
  int m;        // global row of this thread
  int n0;       // first column of the tile
  bool row_ok;  // m < M
  int lane;     // lane in warp
  int quad;     // TMEM lane quadrant of this warp (0..3)
  int* status;  // device status word (may be null)
  char* stage;  // this warp's shared-memory staging tiles (GEMM epilogue only)
  int m_warp;   // first global row of this warp's 32 rows (convolutions: first tile row)
  const ConvParams* conv;   // convolution kernels only
  ConvTile conv_tile;
  int m_rows[4];            // convolution kernels: canonical rows of the four tile rows (i * 8 + lane / 4) this
                            // lane moves in the staged (coalesced) accesses, computed once per tile
};

// Canonical row of the `row`-th of this warp's 32 rows, for the staged (coalesced) accesses of
// the generated epilogues.  Convolution kernels define it through their box geometry.
#ifndef EVTB_ROW_M
#define EVTB_ROW_M(c, row) ((c).m_warp + (row))
#endif

// Debug builds of the generated epilogues (-DEVTB_BOUNDS_CHECK) route every global access
// through this: an access outside [0, numel) is recorded as status 1000 + slot and skipped.
#ifdef EVTB_BOUNDS_CHECK
__device__ __forceinline__ bool epi_in_bounds(const EpiCtx& c, long long off, int width, long long numel, int slot) {
  if (off >= 0 && off + width <= numel) return true;
  report_status(c.status, 1000 + slot);
  return false;
}
#define EVTB_CHK(c, off, width, numel, slot) epi_in_bounds(c, off, width, numel, slot)
#else
#define EVTB_CHK(c, off, width, numel, slot) true
#endif

template <int BN_, int STAGES_, bool A_MN_, bool B_MN_, bool BF16_, int EPI_WARPS_ = 8, int EPI_STAGE_BYTES_ = 0,
          bool SPLIT_K_ = false, bool K_ROTATE_ = false, bool WGRAD_ = false>
struct GemmConfig {
  static constexpr bool WGRAD = WGRAD_;      // operands are boxes of two 4-D convolution tensors (needs A_MN and B_MN)
  static_assert(!WGRAD_ || (A_MN_ && B_MN_ && BN_ % 64 == 0), "weight gradient: both operands MN-major, BN % 64 == 0");
  static_assert(!WGRAD_ || !K_ROTATE_, "weight gradient: k-blocks run in order (the producer steps box counters)");
  static constexpr bool SPLIT_K = SPLIT_K_;
  static constexpr bool K_ROTATE = K_ROTATE_;
  // bytes of shared-memory staging tiles each epilogue warp owns (a multiple of 2048)
  static constexpr int EPI_STAGE_BYTES = EPI_STAGE_BYTES_;
  static constexpr int BN = BN_;
  // epilogue warps: a multiple of 4 (one per TMEM lane quadrant); warps that share a
  // quadrant take alternating 32-column chunks of the tile
  static constexpr int EPI_WARPS = EPI_WARPS_;
  static constexpr int EPI_THREADS = EPI_WARPS_ * 32;
  static constexpr int THREADS = 64 + EPI_WARPS_ * 32;
  static constexpr int COL_GROUPS = EPI_WARPS_ / 4;
  static_assert(EPI_WARPS_ % 4 == 0 && EPI_WARPS_ >= 4 && EPI_WARPS_ <= 16, "epilogue warps: 4, 8, 12 or 16");
  static constexpr int STAGES = STAGES_;
  static constexpr bool A_MN = A_MN_;
  static constexpr bool B_MN = B_MN_;
  static constexpr bool BF16 = BF16_;
  static constexpr int A_BYTES = kBM * kBK * 2;
  static constexpr int B_BYTES = BN * kBK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
  // barriers + tmem pointer + abort flag live in the first 1024 bytes
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + EPI_WARPS_ * EPI_STAGE_BYTES_;
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "BN must be a multiple of 32 in [32,256]");
  static_assert(!B_MN_ || BN % 64 == 0, "MN-major B needs BN % 64 == 0");
};

struct GemmSmemHeader {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  // written by tcgen05.alloc only (asynchronously, not through the thread's own store path): no
  // thread ever stores to this 16-byte slot, so nothing can land on top of the allocator's write
  alignas(16) uint32_t tmem_base;
  uint32_t tmem_base_pad[3];
  volatile int abort_flag;
  volatile int is_last;   // split-K: this CTA holds the last unit of its tile
  volatile int epi_abort; // split-K: an epilogue warp gave up; all leave after the same unit
  volatile int quad_abort[4];  // row-resident kernel: per lane quadrant, same purpose
};

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x3fu) == 0u) {
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > EVTB_WAIT_LIMIT_NS) return false;
    }
  }
}

// Tile order: m fastest, then n, then batch, so that CTAs running side by side
// share one B column strip in L2.
__device__ __forceinline__ void decode_tile(const GemmParams& p, int t, int& l, int& tm, int& tn) {
  tm = t % p.tiles_m;
  int r = t / p.tiles_m;
  tn = r % p.tiles_n;
  l = r / p.tiles_n;
}

// split-K work units: unit u = tile * splits + split (the splits of one tile run side by side)
template <class Cfg>
__device__ __forceinline__ void decode_unit(const GemmParams& p, int u, int& t, int& kb0, int& kb1, int num_k) {
  if constexpr (Cfg::SPLIT_K) {
    t = u / p.splits;
    const int sp = u - t * p.splits;
    kb0 = sp * p.kb_per_split;
    kb1 = kb0 + p.kb_per_split < num_k ? kb0 + p.kb_per_split : num_k;
  } else {
    t = u;
    kb0 = 0;
    kb1 = num_k;
  }
}

// CTAs that work on the same operand slabs would otherwise walk K in lockstep and hammer one
// narrow band of addresses (a few L2 slices) at a time: each CTA starts its K loop at a
// different k-block and wraps around.  Producer and MMA issuer use the same order; fp32
// accumulation makes the result independent of it up to rounding.
__device__ __forceinline__ int rotated_kb(int i, int kb0, int kb1, int rot) {
  const int n = kb1 - kb0;
  int j = i + rot;
  if (j >= n) j -= n;
  return kb0 + j;
}

__device__ __forceinline__ void tma_load_4d_box(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                                int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0),
        "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void epi_bar_sync(int nthreads) {
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

// One accumulator tile through the generated epilogue, 32-column chunks, software-pipelined:
// the tensor-memory load of the next chunk and the global loads of this chunk (chunk_begin) are
// in flight while the previous values are being worked on.  `taddr` = this warp's lane quadrant
// at the first column of the accumulator stage.
template <class Cfg, class Epilogue>
__device__ __forceinline__ void epilogue_tile(Epilogue& epi, const EpiCtx& c, uint32_t taddr, int col_group, int N,
                                              bool zero = false) {
  constexpr int NCH = Cfg::BN / 32;
  constexpr int CG = Cfg::COL_GROUPS;
  float acc[32];
  if (zero) {
    // a tile nothing was accumulated into (a strided data gradient's empty parity class)
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
#pragma unroll 1
    for (int ch = col_group; ch < NCH; ch += CG) {
      const int n = c.n0 + ch * 32;
      if (n < N) epi.visit(c, n, acc);
    }
    return;
  }
  uint32_t ra[32], rb[32];
  int ch = col_group;
  if (ch < NCH) tmem_ld_32x32_issue(taddr + ch * 32, ra);
#pragma unroll 1
  while (ch < NCH) {
    {
      const int n = c.n0 + ch * 32;
      const bool live = n < N;
      if (live) epi.chunk_begin(c, n);
      tmem_ld_wait(ra);
      if (ch + CG < NCH) tmem_ld_32x32_issue(taddr + (ch + CG) * 32, rb);
      if (live) {
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = __uint_as_float(ra[i]);
        epi.body(c, n, acc);
        epi.chunk_end(c, n);
      }
    }
    ch += CG;
    if (ch >= NCH) break;
    {
      const int n = c.n0 + ch * 32;
      const bool live = n < N;
      if (live) epi.chunk_begin(c, n);
      tmem_ld_wait(rb);
      if (ch + CG < NCH) tmem_ld_32x32_issue(taddr + (ch + CG) * 32, ra);
      if (live) {
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = __uint_as_float(rb[i]);
        epi.body(c, n, acc);
        epi.chunk_end(c, n);
      }
    }
    ch += CG;
  }
}

template <class Cfg, class Epilogue>
__device__ __forceinline__ void gemm_kernel_body(const GemmParams& p) {
  extern __shared__ uint8_t smem_raw[];
  GemmSmemHeader* hdr = reinterpret_cast<GemmSmemHeader*>(smem_raw);
  // tiles start at the next 1024-byte boundary after the header (swizzle atoms need it)
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_off = ((raw_addr + 1024u + 1023u) & ~1023u) - raw_addr;
  uint8_t* tiles = smem_raw + tiles_off;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_k = Cfg::WGRAD ? p.wg.boxes_w * p.wg.boxes_h * p.wg.boxes_n : (p.K + kBK - 1) / kBK;
  const int num_units = Cfg::SPLIT_K ? p.num_tiles * p.splits : p.num_tiles;
#ifdef EVTB_PROFILE
  const long long prof_start = clock64();
  long long prof_a = 0, prof_b = 0;
#endif

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&hdr->full[s], 1);
      mbar_init(&hdr->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&hdr->tmem_full[s], 1);
      mbar_init(&hdr->tmem_empty[s], Cfg::EPI_THREADS);
    }
    hdr->abort_flag = 0;
    hdr->is_last = 0;
    hdr->epi_abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    // The allocator writes the address asynchronously; no thread stores to that word, ever.  (A
    // store issued just before the allocation by the same warp is not ordered with the
    // allocator's write: when CTAs of other kernels shared the SM it landed afterwards and every
    // tensor-memory access of the CTA then used the stale value.)
    tmem_alloc(&hdr->tmem_base, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = hdr->tmem_base;
  const bool tmem_ok = tmem_addr_valid(tmem_base, Cfg::TMEM_COLS);   // same value in every thread

  if (!tmem_ok) {
    if (threadIdx.x == 0) report_status(p.status, DEV_TMEM_ALLOC);
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&p.tma_a);
      tma_prefetch_desc(&p.tma_b);
      int it = 0;  // global k-block counter across tiles
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        int t, kb0, kb1, l, tm, tn;
        decode_unit<Cfg>(p, u, t, kb0, kb1, num_k);
        decode_tile(p, t, l, tm, tn);
        const int m0 = tm * kBM, n0 = tn * Cfg::BN;
        const int rot = Cfg::K_ROTATE ? static_cast<int>((blockIdx.x * 5u) % static_cast<unsigned>(kb1 - kb0)) : 0;
        // weight gradient: box coordinates of the unit's first k-block and the column tile's filter tap;
        // the loop then steps the box counters (one thread feeds the whole ring: three divisions per
        // k-block were more than a narrow tile's MMA time)
        int wq = 0, wp = 0, wi = 0, w_dh = 0, w_dw = 0, w_c0 = 0;
        if constexpr (Cfg::WGRAD) {
          const WgradGeom& g = p.wg;
          wq = kb0 % g.boxes_w;
          wp = (kb0 / g.boxes_w) % g.boxes_h;
          wi = kb0 / (g.boxes_w * g.boxes_h);
          const int tap = n0 / g.C;
          w_c0 = n0 - tap * g.C;
          w_dh = (tap / g.S) * g.dil_h - g.pad_h;
          w_dw = (tap % g.S) * g.dil_w - g.pad_w;
        }
        for (int ki = 0; ki < kb1 - kb0; ++ki, ++it) {
          const int kb = rotated_kb(ki, kb0, kb1, rot);
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (it / Cfg::STAGES) & 1;
          if (it >= Cfg::STAGES) {
            EVTB_PROF_T0();
            const bool got_slot = wait_or_abort(&hdr->empty[s], ph ^ 1, &hdr->abort_flag);
            EVTB_PROF_ADD(prof_a);
            if (!got_slot) {
              report_status(p.status, DEV_TIMEOUT_PRODUCER);
              hdr->abort_flag = 1;
              ok = false;
              break;
            }
          }
          uint8_t* sa = tiles + s * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_arrive_expect_tx(&hdr->full[s], Cfg::STAGE_BYTES);
          const int k0 = kb * kBK;
          if constexpr (Cfg::WGRAD) {
            // k-block = box of 64 output positions; the column tile picks the filter tap
            const WgradGeom& g = p.wg;
            const int q0 = wq * g.bq, p0 = wp * g.bp, i0 = wi * g.bn;
#pragma unroll
            for (int c = 0; c < kBM / 64; ++c)
              tma_load_4d_box(sa + c * (kBK * 128), &p.tma_a, &hdr->full[s], m0 + c * 64, q0, p0, i0);
#pragma unroll
            for (int c = 0; c < Cfg::BN / 64; ++c)
              tma_load_4d_box(sb + c * (kBK * 128), &p.tma_b, &hdr->full[s], w_c0 + c * 64, q0 * g.stride_w + w_dw,
                              p0 * g.stride_h + w_dh, i0);
            if (++wq == g.boxes_w) {          // next box (k-blocks of a weight gradient run in order)
              wq = 0;
              if (++wp == g.boxes_h) {
                wp = 0;
                ++wi;
              }
            }
          } else if constexpr (!Cfg::A_MN) {
            tma_load_3d(sa, &p.tma_a, &hdr->full[s], k0, m0, l);
          } else {
#pragma unroll
            for (int c = 0; c < kBM / 64; ++c)
              tma_load_3d(sa + c * (kBK * 128), &p.tma_a, &hdr->full[s], m0 + c * 64, k0, l);
          }
          if constexpr (Cfg::WGRAD) {
            // both operands were fetched above
          } else if constexpr (!Cfg::B_MN) {
            tma_load_3d(sb, &p.tma_b, &hdr->full[s], k0, n0, l);
          } else {
#pragma unroll
            for (int c = 0; c < Cfg::BN / 64; ++c)
              tma_load_3d(sb + c * (kBK * 128), &p.tma_b, &hdr->full[s], n0 + c * 64, k0, l);
          }
        }
      }
      if (!ok) {
        // Abort path: wait (bounded) for the loads this thread still has in flight.
        const int first = it > Cfg::STAGES ? it - Cfg::STAGES : 0;
        for (int j = first; j < it; ++j) {
          if (!mbar_wait(&hdr->full[j % Cfg::STAGES], (j / Cfg::STAGES) & 1, 200000000ull))
            report_status(p.status, DEV_TIMEOUT_DRAIN);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kBM, Cfg::BN, Cfg::BF16, Cfg::A_MN, Cfg::B_MN);
      int it = 0;
      int tile_iter = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++tile_iter) {
        int t, kb0, kb1;
        decode_unit<Cfg>(p, u, t, kb0, kb1, num_k);
        const int as = tile_iter & 1;
        const uint32_t aph = (tile_iter >> 1) & 1;
        if (tile_iter >= 2) {
          EVTB_PROF_T0();
          const bool got_acc = wait_or_abort(&hdr->tmem_empty[as], aph ^ 1, &hdr->abort_flag);
          EVTB_PROF_ADD(prof_b);
          if (!got_acc) {
            report_status(p.status, DEV_TIMEOUT_MMA_TMEM);
            hdr->abort_flag = 1;
            ok = false;
            break;
          }
        }
        tcgen05_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(as * Cfg::BN);
        for (int ki = 0; ki < kb1 - kb0; ++ki, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (it / Cfg::STAGES) & 1;
          EVTB_PROF_T0();
          const bool got_data = wait_or_abort(&hdr->full[s], ph, &hdr->abort_flag);
          EVTB_PROF_ADD(prof_a);
          if (!got_data) {
            report_status(p.status, DEV_TIMEOUT_MMA_FULL);
            hdr->abort_flag = 1;
            ok = false;
            break;
          }
          tcgen05_fence_after_sync();
          const uint32_t sa = smem_u32(tiles + s * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // K-major: step 32 bytes inside the 128-byte swizzle row.
            // MN-major: step 16 k-rows of 128 bytes.
            const uint64_t da = Cfg::A_MN ? make_smem_desc(sa + k * (kUmmaK * 128), kBK * 128, 1024)
                                          : make_smem_desc(sa + k * (kUmmaK * 2), 16, 1024);
            const uint64_t db = Cfg::B_MN ? make_smem_desc(sb + k * (kUmmaK * 128), kBK * 128, 1024)
                                          : make_smem_desc(sb + k * (kUmmaK * 2), 16, 1024);
            umma_f16(tmem_d, da, db, idesc, (ki | k) != 0 ? 1u : 0u);
          }
          umma_commit(&hdr->empty[s]);  // slot is free once these MMAs retire
        }
        if (ok) umma_commit(&hdr->tmem_full[as]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;
    const int col_group = (warp - 2) >> 2;
    Epilogue epi;
    EpiCtx c;
    c.ep = &p.epi;
    c.M = p.M;
    c.N = p.N;
    c.L = p.L;
    c.lane = lane;
    c.quad = quad;
    c.status = p.status;
    c.stage = reinterpret_cast<char*>(tiles) + Cfg::STAGES * Cfg::STAGE_BYTES + (warp - 2) * Cfg::EPI_STAGE_BYTES;
    int tile_iter = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++tile_iter) {
      int t, kb0, kb1, l, tm, tn;
      decode_unit<Cfg>(p, u, t, kb0, kb1, num_k);
      decode_tile(p, t, l, tm, tn);
      const int as = tile_iter & 1;
      const uint32_t aph = (tile_iter >> 1) & 1;
      c.l = l;
      c.m_warp = tm * kBM + quad * 32;
      c.m = c.m_warp + lane;
      c.n0 = tn * Cfg::BN;
      c.row_ok = c.m < p.M;
      EVTB_PROF_T0();
      const bool got = wait_or_abort(&hdr->tmem_full[as], aph, &hdr->abort_flag);
      EVTB_PROF_ADD(prof_a);
      if (!got) {
        report_status(p.status, DEV_TIMEOUT_EPILOGUE);
        hdr->abort_flag = 1;
        ok = false;
        if constexpr (!Cfg::SPLIT_K) break;
        hdr->epi_abort = 1;   // the other epilogue warps still meet this one at the barriers below
      }
      tcgen05_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                             static_cast<uint32_t>(as * Cfg::BN);
      if constexpr (!Cfg::SPLIT_K) {
        epi.tile_begin(c);
        epilogue_tile<Cfg>(epi, c, taddr, col_group, p.N);
        // accumulator stage can be overwritten by the MMA warp from here on
        tcgen05_fence_before_sync();
        mbar_arrive(&hdr->tmem_empty[as]);
        epi.tile_end(c);
      } else {
        // 1. add this unit's partial accumulator to the tile's fp32 sum in the workspace (16-byte
        //    reductions at the L2; the sum starts at zero and its reader leaves it at zero).  The sum is
        //    laid out [BN/4][128 rows] of float4: the 32 rows of a warp touch 512 contiguous bytes.
        //    One sum per tile, whatever the number of cuts: the unit that arrives last reads one tile,
        //    not one per cut (with 64 cuts that serial read was most of a weight gradient's time).
        float4* mine = reinterpret_cast<float4*>(p.partial + static_cast<long long>(t) * kBM * Cfg::BN) + quad * 32 + lane;
#pragma unroll 1
        for (int ch = col_group; got && ch < Cfg::BN / 32; ch += Cfg::COL_GROUPS) {
          float acc[32];
          tmem_ld_32x32(taddr + ch * 32, acc);
          float4* dst = mine + ch * 8 * kBM;
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4)
            red_add_f32x4(dst + q4 * kBM, acc[4 * q4], acc[4 * q4 + 1], acc[4 * q4 + 2], acc[4 * q4 + 3]);
        }
        tcgen05_fence_before_sync();
        mbar_arrive(&hdr->tmem_empty[as]);
        // 2. count arrivals; the last unit of the tile reduces and runs the epilogue
        __threadfence();
        epi_bar_sync(Cfg::EPI_THREADS);
        const bool leave = hdr->epi_abort != 0;   // written before the barrier above, if at all
        if (threadIdx.x == 64) {
          const unsigned int prev = atomicAdd(&p.tile_counters[t], 1u);
          const bool last = prev == static_cast<unsigned int>(p.splits - 1);
          if (last) p.tile_counters[t] = 0u;
          hdr->is_last = last ? 1 : 0;
        }
        epi_bar_sync(Cfg::EPI_THREADS);
        if (leave) {
          ok = false;
          break;
        }
        if (hdr->is_last) {
          __threadfence();
          epi.tile_begin(c);
          float4* base = reinterpret_cast<float4*>(p.partial + static_cast<long long>(t) * kBM * Cfg::BN) + quad * 32 + lane;
#pragma unroll 1
          for (int ch = col_group; ch < Cfg::BN / 32; ch += Cfg::COL_GROUPS) {
            float acc[32];
            float4* src = base + ch * 8 * kBM;
            float4 v[8];
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) v[q4] = __ldcg(src + q4 * kBM);
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) {
              __stcg(src + q4 * kBM, make_float4(0.f, 0.f, 0.f, 0.f));     // ready for the next launch
              acc[4 * q4] = v[q4].x; acc[4 * q4 + 1] = v[q4].y; acc[4 * q4 + 2] = v[q4].z; acc[4 * q4 + 3] = v[q4].w;
            }
            if (c.n0 + ch * 32 < p.N) epi.visit(c, c.n0 + ch * 32, acc);
          }
          epi.tile_end(c);
        }
      }
    }
    epi.finish(c);
  }

#ifdef EVTB_PROFILE
  if (p.prof != nullptr && lane == 0) {
    long long* o = p.prof + blockIdx.x * 8;
    const long long total = clock64() - prof_start;
    if (warp == 0) { o[1] = prof_a; o[6] = total; }
    if (warp == 1) { o[2] = prof_a; o[3] = prof_b; }
    if (warp == 2) { o[0] = total; o[4] = prof_a; o[5] = total - prof_a; o[7] = static_cast<long long>(global_timer_ns()); }
  }
#endif
  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after_sync();
    if (tmem_ok) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace evtb
