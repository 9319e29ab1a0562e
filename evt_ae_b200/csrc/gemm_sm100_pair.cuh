// GEMM / batched-GEMM main loop on CTA pairs (tcgen05 cta_group::2) for sm_100a.
//
// Two CTAs of a cluster work on one 256 x BN output tile.  Each stages its own 128 rows of A and
// its own BN/2 columns of B per k-block (32 KB instead of the 48 KB a lone CTA needs for a
// 128 x 256 tile), the leader's MMA thread issues tcgen05.mma.cta_group::2 over both CTAs'
// shared memory, and each CTA's tensor memory receives the 128 x BN accumulator of its own rows.
// Per flop the pair reads a third less from L2 than two independent CTAs, which is what bounds
// the single-CTA kernel on long-K shapes.  Roles, epilogue protocol and bounded waits are those
// of gemm_sm100.cuh; this variant has no split-K.
//
// Barriers: the leader's full[s] counts the bytes of both CTAs' loads (each CTA's TMA names the
// leader's barrier); empty[s] and tmem_full[a] are signalled in both CTAs by a commit that
// arrives at the same shared-memory offset in each; the leader's tmem_empty[a] collects one
// arrival per epilogue warp of both CTAs.
#pragma once
#include "gemm_sm100.cuh"

namespace evtb {

template <int BN_, int STAGES_, bool A_MN_, bool B_MN_, bool BF16_, int EPI_WARPS_ = 8, int EPI_STAGE_BYTES_ = 0,
          bool SPLIT_K_ = false>
struct GemmPairConfig {
  // split-K: a pair tile's K range is cut into p.splits units that run on different pairs; each
  // CTA parks the fp32 partial of its own 128 x BN half, and per half the last arriver adds the
  // partials in a fixed order and runs the epilogue (same scheme as the single-CTA kernel, with
  // half-tile index 2 * tile + rank).
  static constexpr bool SPLIT_K = SPLIT_K_;
  static constexpr int EPI_STAGE_BYTES = EPI_STAGE_BYTES_;
  static constexpr int BN = BN_;
  static constexpr int BN_HALF = BN_ / 2;      // B columns staged by each CTA
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
  static constexpr int B_BYTES = BN_HALF * kBK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;     // two accumulator stages of BN fp32 columns
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 1024 + EPI_WARPS_ * EPI_STAGE_BYTES_;
  static_assert(BN_ == 128 || BN_ == 256, "pair tiles are 256 x 128 or 256 x 256");
  static_assert(STAGES_ >= 2 && STAGES_ <= 8, "2..8 ring stages");
};

__device__ __forceinline__ bool wait_or_abort_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((++spins & 0x3fu) == 0u) {
      if (*abort_flag != 0) return false;
      if (global_timer_ns() - t0 > EVTB_WAIT_LIMIT_NS) return false;
    }
  }
}

// p.tiles_m counts 256-row pair tiles; p.num_tiles = tiles_m * tiles_n * L pair tiles; with
// split-K the work units are (tile, split) pairs, unit = tile * splits + split.
template <class Cfg, class Epilogue>
__device__ __forceinline__ void gemm_pair_kernel_body(const GemmParams& p) {
  extern __shared__ uint8_t smem_raw[];
  GemmSmemHeader* hdr = reinterpret_cast<GemmSmemHeader*>(smem_raw);
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_off = ((raw_addr + 1024u + 1023u) & ~1023u) - raw_addr;
  uint8_t* tiles = smem_raw + tiles_off;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_k = (p.K + kBK - 1) / kBK;
  const int rank = static_cast<int>(cluster_ctarank());   // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
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
      mbar_init(&hdr->tmem_empty[s], 2 * Cfg::EPI_WARPS);   // used in the leader only
    }
    hdr->abort_flag = 0;
    hdr->is_last = 0;
    hdr->epi_abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    // the allocator writes the address asynchronously; no thread stores to that word
    tmem_alloc_pair(&hdr->tmem_base, Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_sync_all();          // the peer's barriers are initialised before anything arrives on them
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = hdr->tmem_base;
  const bool tmem_ok = tmem_addr_valid(tmem_base, Cfg::TMEM_COLS);   // same value in every thread

  if (!tmem_ok) {
    // the peer's bounded waits run out and it meets this CTA at the cluster barrier below
    if (threadIdx.x == 0) report_status(p.status, DEV_TMEM_ALLOC);
    hdr->abort_flag = 1;
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&p.tma_a);
      tma_prefetch_desc(&p.tma_b);
      const uint32_t leader_full = mapa_shared(smem_u32(&hdr->full[0]), 0);
      int it = 0;
      bool ok = true;
      for (int u = pair_id; u < num_units && ok; u += num_pairs) {
        int t, kb0, kb1, l, tm, tn;
        decode_unit<Cfg>(p, u, t, kb0, kb1, num_k);
        decode_tile(p, t, l, tm, tn);
        const int m0 = tm * (2 * kBM) + rank * kBM;
        const int n0 = tn * Cfg::BN + rank * Cfg::BN_HALF;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (it / Cfg::STAGES) & 1;
          if (it >= Cfg::STAGES) {
            EVTB_PROF_T0();
            const bool got_slot = wait_or_abort_cluster(&hdr->empty[s], ph ^ 1, &hdr->abort_flag);
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
          const uint32_t bar = leader_full + static_cast<uint32_t>(s) * 8u;
          if (rank == 0) mbar_arrive_expect_tx(&hdr->full[s], 2 * Cfg::STAGE_BYTES);
          const int k0 = kb * kBK;
          if constexpr (!Cfg::A_MN) {
            tma_load_3d_pair(sa, &p.tma_a, bar, k0, m0, l);
          } else {
#pragma unroll
            for (int c = 0; c < kBM / 64; ++c)
              tma_load_3d_pair(sa + c * (kBK * 128), &p.tma_a, bar, m0 + c * 64, k0, l);
          }
          if constexpr (!Cfg::B_MN) {
            tma_load_3d_pair(sb, &p.tma_b, bar, k0, n0, l);
          } else {
#pragma unroll
            for (int c = 0; c < Cfg::BN_HALF / 64; ++c)
              tma_load_3d_pair(sb + c * (kBK * 128), &p.tma_b, bar, n0 + c * 64, k0, l);
          }
        }
      }
      // This CTA's loads are accounted on the leader's barriers; the MMA issuer consumes every
      // stage that was filled, or gives up after its own bounded wait, before the final cluster
      // barrier lets either CTA leave.
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_f16(2 * kBM, Cfg::BN, Cfg::BF16, Cfg::A_MN, Cfg::B_MN);
      int it = 0;
      int tile_iter = 0;
      bool ok = true;
      for (int u = pair_id; u < num_units && ok; u += num_pairs, ++tile_iter) {
        int t, kb0, kb1;
        decode_unit<Cfg>(p, u, t, kb0, kb1, num_k);
        const int as = tile_iter & 1;
        const uint32_t aph = (tile_iter >> 1) & 1;
        if (tile_iter >= 2) {
          EVTB_PROF_T0();
          const bool got_acc = wait_or_abort_cluster(&hdr->tmem_empty[as], aph ^ 1, &hdr->abort_flag);
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
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (it / Cfg::STAGES) & 1;
          EVTB_PROF_T0();
          const bool got_data = wait_or_abort_cluster(&hdr->full[s], ph, &hdr->abort_flag);
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
            const uint64_t da = Cfg::A_MN ? make_smem_desc(sa + k * (kUmmaK * 128), kBK * 128, 1024)
                                          : make_smem_desc(sa + k * (kUmmaK * 2), 16, 1024);
            const uint64_t db = Cfg::B_MN ? make_smem_desc(sb + k * (kUmmaK * 128), kBK * 128, 1024)
                                          : make_smem_desc(sb + k * (kUmmaK * 2), 16, 1024);
            umma_f16_pair(tmem_d, da, db, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&hdr->empty[s], 3);   // both CTAs' slot s is free once these MMAs retire
        }
        if (ok) umma_commit_pair(&hdr->tmem_full[as], 3);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
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
    const uint32_t leader_tmem_empty = mapa_shared(smem_u32(&hdr->tmem_empty[0]), 0);
    int tile_iter = 0;
    bool ok = true;
    for (int u = pair_id; u < num_units && ok; u += num_pairs, ++tile_iter) {
      int t, kb0, kb1, l, tm, tn;
      decode_unit<Cfg>(p, u, t, kb0, kb1, num_k);
      decode_tile(p, t, l, tm, tn);
      const int as = tile_iter & 1;
      const uint32_t aph = (tile_iter >> 1) & 1;
      c.l = l;
      c.m_warp = tm * (2 * kBM) + rank * kBM + quad * 32;
      c.m = c.m_warp + lane;
      c.n0 = tn * Cfg::BN;
      c.row_ok = c.m < p.M;
      EVTB_PROF_T0();
      const bool got = wait_or_abort_cluster(&hdr->tmem_full[as], aph, &hdr->abort_flag);
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
        // this warp is done with the accumulator stage: one arrival per warp on the leader's barrier
        tcgen05_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_tmem_empty + static_cast<uint32_t>(as) * 8u);
        epi.tile_end(c);
      } else {
        // 1. add this CTA's half of the unit's partial accumulator to the half tile's fp32 sum in the
        //    workspace ([BN/4][128 rows] of float4, 16-byte reductions at the L2; see gemm_sm100.cuh)
        const long long half = 2ll * t + rank;
        float4* mine = reinterpret_cast<float4*>(p.partial + half * kBM * Cfg::BN) + quad * 32 + lane;
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
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_tmem_empty + static_cast<uint32_t>(as) * 8u);
        // 2. count arrivals per half tile; the last unit reduces and runs the epilogue
        __threadfence();
        epi_bar_sync(Cfg::EPI_THREADS);
        const bool leave = hdr->epi_abort != 0;   // written before the barrier above, if at all
        if (threadIdx.x == 64) {
          const unsigned int prev = atomicAdd(&p.tile_counters[half], 1u);
          const bool last = prev == static_cast<unsigned int>(p.splits - 1);
          if (last) p.tile_counters[half] = 0u;
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
          float4* base = reinterpret_cast<float4*>(p.partial + half * kBM * Cfg::BN) + quad * 32 + lane;
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
  // Abort path only: loads of this CTA that are still in flight complete on the leader's barrier,
  // so they cannot be waited for here; give them a bounded moment to land before leaving.
  if (hdr->abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 1000000ull) __nanosleep(1000);
  }
  // Neither CTA may leave while the other can still read its shared memory, arrive on its
  // barriers or write its tensor memory.
  tcgen05_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after_sync();
    if (tmem_ok) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace evtb
