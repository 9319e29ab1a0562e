// Row-resident GEMM / batched GEMM for sm_100a: one CTA owns whole rows of the result, so a
// row-wise reduce-apply step (softmax, softmax backward) runs inside the GEMM epilogue and the
// intermediate never goes to memory.
//
// The accumulator tile is 128 x 512 fp32 = all 512 tensor-memory columns of the SM (two
// tcgen05.mma of N = 256 per k-step), so N <= 512 and there is one accumulator stage: the
// epilogue reads it twice -- a statistics pass (row maximum and sum of exponentials, or the row
// sum of grad * y) and an apply pass that recomputes the element from the accumulator, finishes
// the row-wise step and runs the rest of the generated epilogue -- and only then hands tensor
// memory back to the MMA issuer, while the TMA producer already fetches the next tile's operands.
// The 16 (or 8) epilogue warps split a row's columns four (two) ways; their partial statistics
// meet in shared memory under one named barrier per lane quadrant.
//
// In the reference the attention scores and their softmax are two kernels with the S x S tensor
// written and read in between (FusedBMM, evt_fuser.py:561-697; FusedSoftmax, :700-762); this
// variant is the fusion BASELINE's north_star asks for on top of that.
#pragma once
#include "gemm_sm100.cuh"

namespace evtb {

constexpr int kRowsBN = 512;

template <int STAGES_, bool A_MN_, bool B_MN_, bool BF16_, int EPI_WARPS_ = 16, int EPI_STAGE_BYTES_ = 0>
struct GemmRowsConfig {
  static constexpr int EPI_STAGE_BYTES = EPI_STAGE_BYTES_;
  static constexpr int BN = kRowsBN;
  static constexpr int EPI_WARPS = EPI_WARPS_;
  static constexpr int EPI_THREADS = EPI_WARPS_ * 32;
  static constexpr int THREADS = 64 + EPI_WARPS_ * 32;
  static constexpr int COL_GROUPS = EPI_WARPS_ / 4;
  static_assert(EPI_WARPS_ == 8 || EPI_WARPS_ == 16, "8 or 16 epilogue warps");
  static constexpr int STAGES = STAGES_;
  static constexpr bool A_MN = A_MN_;
  static constexpr bool B_MN = B_MN_;
  static constexpr bool BF16 = BF16_;
  static constexpr int A_BYTES = kBM * kBK * 2;
  static constexpr int B_BYTES = BN * kBK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 512;
  static constexpr int XCHG_BYTES = 2 * 4 * COL_GROUPS * 32 * 8;  // (a, b) per row and column group, two passes
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 1024 + EPI_WARPS_ * EPI_STAGE_BYTES_ + XCHG_BYTES;
  static_assert(STAGES_ >= 2 && STAGES_ <= 8, "2..8 ring stages");
};

__device__ __forceinline__ void quad_bar_sync(int quad, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(2 + quad), "r"(nthreads) : "memory");
}

// p.tiles_n == 1; p.num_tiles = tiles_m * L.
template <class Cfg, class Epilogue>
__device__ __forceinline__ void gemm_rows_kernel_body(const GemmParams& p) {
  extern __shared__ uint8_t smem_raw[];
  GemmSmemHeader* hdr = reinterpret_cast<GemmSmemHeader*>(smem_raw);
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_off = ((raw_addr + 1024u + 1023u) & ~1023u) - raw_addr;
  uint8_t* tiles = smem_raw + tiles_off;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_k = (p.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&hdr->full[s], 1);
      mbar_init(&hdr->empty[s], 1);
    }
    mbar_init(&hdr->tmem_full[0], 1);
    mbar_init(&hdr->tmem_empty[0], Cfg::EPI_WARPS);
    hdr->abort_flag = 0;
    hdr->is_last = 0;
    hdr->epi_abort = 0;
    for (int q = 0; q < 4; ++q) hdr->quad_abort[q] = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    // the allocator writes the address asynchronously; no thread stores to that word
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
      int it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.num_tiles && ok; u += gridDim.x) {
        int l, tm, tn;
        decode_tile(p, u, l, tm, tn);
        const int m0 = tm * kBM;
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (it / Cfg::STAGES) & 1;
          if (it >= Cfg::STAGES) {
            if (!wait_or_abort(&hdr->empty[s], ph ^ 1, &hdr->abort_flag)) {
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
          if constexpr (!Cfg::A_MN) {
            tma_load_3d(sa, &p.tma_a, &hdr->full[s], k0, m0, l);
          } else {
#pragma unroll
            for (int c = 0; c < kBM / 64; ++c)
              tma_load_3d(sa + c * (kBK * 128), &p.tma_a, &hdr->full[s], m0 + c * 64, k0, l);
          }
          if constexpr (!Cfg::B_MN) {
#pragma unroll
            for (int h = 0; h < 2; ++h)     // box rows are limited to 256
              tma_load_3d(sb + h * (256 * 128), &p.tma_b, &hdr->full[s], k0, h * 256, l);
          } else {
#pragma unroll
            for (int c = 0; c < Cfg::BN / 64; ++c)
              tma_load_3d(sb + c * (kBK * 128), &p.tma_b, &hdr->full[s], c * 64, k0, l);
          }
        }
      }
      if (!ok) {
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
      constexpr uint32_t idesc = make_idesc_f16(kBM, 256, Cfg::BF16, Cfg::A_MN, Cfg::B_MN);
      int it = 0;
      int tile_iter = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.num_tiles && ok; u += gridDim.x, ++tile_iter) {
        if (tile_iter >= 1) {
          if (!wait_or_abort(&hdr->tmem_empty[0], (tile_iter - 1) & 1, &hdr->abort_flag)) {
            report_status(p.status, DEV_TIMEOUT_MMA_TMEM);
            hdr->abort_flag = 1;
            ok = false;
            break;
          }
        }
        tcgen05_fence_after_sync();
        for (int kb = 0; kb < num_k; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (it / Cfg::STAGES) & 1;
          if (!wait_or_abort(&hdr->full[s], ph, &hdr->abort_flag)) {
            report_status(p.status, DEV_TIMEOUT_MMA_FULL);
            hdr->abort_flag = 1;
            ok = false;
            break;
          }
          tcgen05_fence_after_sync();
          const uint32_t sa = smem_u32(tiles + s * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            // columns h*256 .. +255: K-major rows of 128 bytes, or four 64-column MN-major chunks
            const uint32_t sbh = sb + h * (256 * 128);
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              const uint64_t da = Cfg::A_MN ? make_smem_desc(sa + k * (kUmmaK * 128), kBK * 128, 1024)
                                            : make_smem_desc(sa + k * (kUmmaK * 2), 16, 1024);
              const uint64_t db = Cfg::B_MN ? make_smem_desc(sbh + k * (kUmmaK * 128), kBK * 128, 1024)
                                            : make_smem_desc(sbh + k * (kUmmaK * 2), 16, 1024);
              umma_f16(tmem_base + static_cast<uint32_t>(h * 256), da, db, idesc, (kb | k) != 0 ? 1u : 0u);
            }
          }
          umma_commit(&hdr->empty[s]);
        }
        if (ok) umma_commit(&hdr->tmem_full[0]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;
    const int col_group = (warp - 2) >> 2;
    constexpr int NCH = Cfg::BN / 32;
    constexpr int CG = Cfg::COL_GROUPS;
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
    float2* xchg = reinterpret_cast<float2*>(reinterpret_cast<char*>(tiles) + Cfg::STAGES * Cfg::STAGE_BYTES +
                                             Cfg::EPI_WARPS * Cfg::EPI_STAGE_BYTES);
    int tile_iter = 0;
    for (int u = blockIdx.x; u < p.num_tiles; u += gridDim.x, ++tile_iter) {
      int l, tm, tn;
      decode_tile(p, u, l, tm, tn);
      c.l = l;
      c.m_warp = tm * kBM + quad * 32;
      c.m = c.m_warp + lane;
      c.n0 = 0;
      c.row_ok = c.m < p.M;
      bool got = wait_or_abort(&hdr->tmem_full[0], tile_iter & 1, &hdr->abort_flag);
      if (!got) {
        report_status(p.status, DEV_TIMEOUT_EPILOGUE);
        hdr->abort_flag = 1;
        hdr->quad_abort[quad] = 1;     // the warps of this quadrant still meet at the barrier below
      }
      tcgen05_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
      epi.tile_begin(c);
      // statistics pass(es) over this warp's columns; the partials of the warps that share a row
      // meet in shared memory.  A second pass may rewrite the accumulator in place (softmax: the
      // exponentials, so that each is computed once).
#pragma unroll 1
      for (int ch = col_group; got && ch < NCH; ch += CG) {
        const int n = ch * 32;
        if (n >= p.N) break;
        float acc[32];
        epi.chunk_begin(c, n);
        tmem_ld_32x32(taddr + ch * 32, acc);
        epi.stat_body0(c, n, acc);
        __syncwarp();            // staging tiles of this chunk may be overwritten by the next
      }
      xchg[(quad * CG + col_group) * 32 + lane] = make_float2(epi.stat_a0(), epi.stat_b0());
      quad_bar_sync(quad, 32 * CG);
      if (hdr->quad_abort[quad] != 0) break;   // written before the barrier, if at all: the quadrant leaves together
      {
        float pa[CG], pb[CG];
#pragma unroll
        for (int g = 0; g < CG; ++g) {
          const float2 v = xchg[(quad * CG + g) * 32 + lane];
          pa[g] = v.x;
          pb[g] = v.y;
        }
        epi.merge0(pa, pb, CG);
      }
      if constexpr (Epilogue::kStatPasses == 2) {
        float2* xchg1 = xchg + 4 * CG * 32;
#pragma unroll 1
        for (int ch = col_group; ch < NCH; ch += CG) {
          const int n = ch * 32;
          if (n >= p.N) break;
          float acc[32];
          epi.chunk_begin(c, n);
          tmem_ld_32x32(taddr + ch * 32, acc);
          epi.stat_body1(c, n, acc);
          if constexpr (Epilogue::kWriteBack) tmem_st_32x32(taddr + ch * 32, acc);
          __syncwarp();
        }
        if constexpr (Epilogue::kWriteBack) tmem_st_wait();
        xchg1[(quad * CG + col_group) * 32 + lane] = make_float2(epi.stat_a1(), epi.stat_b1());
        quad_bar_sync(quad, 32 * CG);
        float pa[CG], pb[CG];
#pragma unroll
        for (int g = 0; g < CG; ++g) {
          const float2 v = xchg1[(quad * CG + g) * 32 + lane];
          pa[g] = v.x;
          pb[g] = v.y;
        }
        epi.merge1(pa, pb, CG);
      }
      // pass 2: recompute, apply, rest of the epilogue, stores
#pragma unroll 1
      for (int ch = col_group; ch < NCH; ch += CG) {
        const int n = ch * 32;
        if (n >= p.N) break;
        float acc[32];
        tmem_ld_32x32(taddr + ch * 32, acc);
        epi.visit(c, n, acc);
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&hdr->tmem_empty[0]);
      epi.tile_end(c);
    }
    epi.finish(c);
  }

  tcgen05_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after_sync();
    if (tmem_ok) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace evtb
