// Implicit-GEMM 2-D convolution (NHWC, fp16/bf16, fp32 accumulate) for sm_100a: forward
// (activations x filters) and data gradient (output gradients x filters), with the same
// generated epilogue protocol as the GEMM.
//
// This replaces the CUTLASS implicit-GEMM kernels the reference instantiates in
// python/gtl/compiler/passes/evt_fuser.py:282-362 (FusedConvFprop) and :365-450
// (FusedConvDgrad); as there, the result is the (N*P*Q, K) matrix in channels-last order
// (evt_fuser.py:1083-1094) and the epilogue sees canonical rows m = (n*OH + oh)*OW + ow.
//
// No im2col buffer exists anywhere: an accumulator tile covers a box of bq x bp x bn output
// positions (bq*bp*bn = 128), and for every filter tap (r, s) and 64-channel block the TMA
// engine fetches the matching box of the activation tensor straight out of its 4-D tensor map
// (C, W, H, N) -- shifted by the tap, strided by the convolution stride, zero-filled where the
// tap falls into the padding -- into the 128-row K-major operand tile the tensor core reads.
// The filter tile comes from the [K, R*S*C] view of the channels-last filter: K-major for the
// forward pass, MN-major (channels contiguous) for the data gradient.
//
// Strided data gradients are split by output parity class ((oh % sh, ow % sw)): within a class
// every output position receives the same subset of taps at unit stride in the gradient tensor,
// so a class is a dense convolution over the sub-grid; a class without taps (1x1 stride-2
// filters reach only one position in four) stores the epilogue of a zero accumulator.
#pragma once
#include "gemm_sm100.cuh"

namespace evtb {

constexpr int kConvMaxTaps = 16;
constexpr int kConvMaxClasses = 4;

struct ConvClass {
  int ntaps;
  int o_oh, o_ow;          // output position = tile-grid position * o_s{h,w} + o_o{h,w}
  int th, tw;              // tile-grid extent of this class
  int boxes_w, boxes_h;    // boxes along w and h (boxes along n = ConvParams::boxes_n)
  int first_tile;          // index of the class's first (m, n) tile
  signed char dh[kConvMaxTaps];   // activation row = tile-grid row * a_sh + dh[tap]
  signed char dw[kConvMaxTaps];
  unsigned char rs[kConvMaxTaps]; // r * S + s of the tap
};

struct alignas(64) ConvParams {
  CUtensorMap tma_a;   // dims (Ca, Aw, Ah, An), box (64, bq, bp, bn), element strides (1, a_sw, a_sh, 1)
  CUtensorMap tma_b;   // forward: dims (R*S*C, K), box (64, BN); data gradient: box (64, 64)
  int On, Oh, Ow;      // output positions
  int NT;              // output channels of this pass (K forward, C data gradient)
  int red;             // reduction channels per tap (C forward, K data gradient)
  int a_sh, a_sw;      // tile-grid -> activation coordinate multiplier (stride forward, 1 data gradient)
  int o_sh, o_sw;      // tile-grid -> output position multiplier (1, or the stride for a strided data gradient)
  int w_c;             // channels per tap in the filter's [K, R*S*C] view (C)
  int bq, bp, bn;      // box of one accumulator tile, bq * bp * bn == 128
  int boxes_n;
  int tiles_n;         // tiles along the output-channel axis
  int num_tiles;
  int nclasses;
  int M;               // On * Oh * Ow
  ConvClass cls[kConvMaxClasses];
  int* status;
  long long* prof;
  EpiParams epi;
};

template <int BN_, int STAGES_, bool DGRAD_, bool BF16_, int EPI_WARPS_ = 8, int EPI_STAGE_BYTES_ = 0>
struct ConvConfig {
  static constexpr int EPI_STAGE_BYTES = EPI_STAGE_BYTES_;
  static constexpr int BN = BN_;
  static constexpr int EPI_WARPS = EPI_WARPS_;
  static constexpr int EPI_THREADS = EPI_WARPS_ * 32;
  static constexpr int THREADS = 64 + EPI_WARPS_ * 32;
  static constexpr int COL_GROUPS = EPI_WARPS_ / 4;
  static_assert(EPI_WARPS_ % 4 == 0 && EPI_WARPS_ >= 4 && EPI_WARPS_ <= 16, "epilogue warps: 4, 8, 12 or 16");
  static constexpr int STAGES = STAGES_;
  static constexpr bool DGRAD = DGRAD_;    // filter operand MN-major (channels contiguous)
  static constexpr bool BF16 = BF16_;
  static constexpr int A_BYTES = kBM * kBK * 2;
  static constexpr int B_BYTES = BN * kBK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 1024 + EPI_WARPS_ * EPI_STAGE_BYTES_;
  static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "BN must be 64, 128, 192 or 256");
  static_assert(STAGES_ >= 2 && STAGES_ <= 8, "2..8 ring stages");
};

__device__ __forceinline__ ConvTile conv_decode_tile(const ConvParams& p, int t, int bn_cols) {
  ConvTile r;
  int c = 0;
#pragma unroll
  for (int i = 1; i < kConvMaxClasses; ++i)
    if (i < p.nclasses && t >= p.cls[i].first_tile) c = i;
  r.cls = c;
  const ConvClass& k = p.cls[c];
  int u = t - k.first_tile;
  const int boxes = k.boxes_w * k.boxes_h * p.boxes_n;
  const int tm = u % boxes;      // position boxes fastest: CTAs side by side share a filter strip
  const int tn = u / boxes;
  r.tq0 = (tm % k.boxes_w) * p.bq;
  r.tp0 = ((tm / k.boxes_w) % k.boxes_h) * p.bp;
  r.tn0 = (tm / (k.boxes_w * k.boxes_h)) * p.bn;
  r.n0 = tn * bn_cols;
  return r;
}

// canonical row of tile row `row` (0..127), or p.M when the row lies outside the output
__device__ __forceinline__ int conv_row_to_m(const ConvParams& p, const ConvTile& t, int row) {
  const ConvClass& k = p.cls[t.cls];
  // bq * bp * bn = 128: each is a power of two, so the split of a tile row is shifts and masks (this
  // runs for every stored row of every 32-column chunk; with divisions it was most of the epilogue)
  const int lq = 31 - __clz(p.bq), lp = 31 - __clz(p.bp);
  const int qi = row & (p.bq - 1);
  const int pi = (row >> lq) & (p.bp - 1);
  const int ni = row >> (lq + lp);
  const int tq = t.tq0 + qi, tp = t.tp0 + pi, tn = t.tn0 + ni;
  if (tq >= k.tw || tp >= k.th || tn >= p.On) return p.M;
  const int oh = tp * p.o_sh + k.o_oh, ow = tq * p.o_sw + k.o_ow;
  return (tn * p.Oh + oh) * p.Ow + ow;
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0),
        "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

template <class Cfg, class Epilogue>
__device__ __forceinline__ void conv_kernel_body(const ConvParams& p) {
  extern __shared__ uint8_t smem_raw[];
  GemmSmemHeader* hdr = reinterpret_cast<GemmSmemHeader*>(smem_raw);
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_off = ((raw_addr + 1024u + 1023u) & ~1023u) - raw_addr;
  uint8_t* tiles = smem_raw + tiles_off;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int red_blocks = (p.red + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&hdr->full[s], 1);
      mbar_init(&hdr->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&hdr->tmem_full[s], 1);
      mbar_init(&hdr->tmem_empty[s], Cfg::EPI_WARPS);
    }
    hdr->abort_flag = 0;
    hdr->is_last = 0;
    hdr->epi_abort = 0;
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
        const ConvTile t = conv_decode_tile(p, u, Cfg::BN);
        const ConvClass& k = p.cls[t.cls];
        for (int tap = 0; tap < k.ntaps && ok; ++tap) {
          const int aw = t.tq0 * p.a_sw + k.dw[tap];
          const int ah = t.tp0 * p.a_sh + k.dh[tap];
          const int w_inner = static_cast<int>(k.rs[tap]) * p.w_c;
          for (int rb = 0; rb < red_blocks; ++rb, ++it) {
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
            tma_load_4d(sa, &p.tma_a, &hdr->full[s], rb * kBK, aw, ah, t.tn0);
            if constexpr (!Cfg::DGRAD) {
              tma_load_3d(sb, &p.tma_b, &hdr->full[s], w_inner + rb * kBK, t.n0, 0);
            } else {
#pragma unroll
              for (int c = 0; c < Cfg::BN / 64; ++c)
                tma_load_3d(sb + c * (kBK * 128), &p.tma_b, &hdr->full[s], w_inner + t.n0 + c * 64, rb * kBK, 0);
            }
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
      constexpr uint32_t idesc = make_idesc_f16(kBM, Cfg::BN, Cfg::BF16, false, Cfg::DGRAD);
      int it = 0;
      int tile_iter = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.num_tiles && ok; u += gridDim.x, ++tile_iter) {
        const ConvTile t = conv_decode_tile(p, u, Cfg::BN);
        const int iters = p.cls[t.cls].ntaps * red_blocks;
        const int as = tile_iter & 1;
        const uint32_t aph = (tile_iter >> 1) & 1;
        if (tile_iter >= 2) {
          if (!wait_or_abort(&hdr->tmem_empty[as], aph ^ 1, &hdr->abort_flag)) {
            report_status(p.status, DEV_TIMEOUT_MMA_TMEM);
            hdr->abort_flag = 1;
            ok = false;
            break;
          }
        }
        tcgen05_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(as * Cfg::BN);
        for (int ki = 0; ki < iters; ++ki, ++it) {
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
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint64_t da = make_smem_desc(sa + k * (kUmmaK * 2), 16, 1024);
            const uint64_t db = Cfg::DGRAD ? make_smem_desc(sb + k * (kUmmaK * 128), kBK * 128, 1024)
                                           : make_smem_desc(sb + k * (kUmmaK * 2), 16, 1024);
            umma_f16(tmem_d, da, db, idesc, (ki | k) != 0 ? 1u : 0u);
          }
          umma_commit(&hdr->empty[s]);
        }
        if (ok) umma_commit(&hdr->tmem_full[as]);   // with no taps this arrives at once
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
    c.N = p.NT;
    c.L = 1;
    c.l = 0;
    c.lane = lane;
    c.quad = quad;
    c.status = p.status;
    c.stage = reinterpret_cast<char*>(tiles) + Cfg::STAGES * Cfg::STAGE_BYTES + (warp - 2) * Cfg::EPI_STAGE_BYTES;
    c.conv = &p;
    int tile_iter = 0;
    for (int u = blockIdx.x; u < p.num_tiles; u += gridDim.x, ++tile_iter) {
      const ConvTile t = conv_decode_tile(p, u, Cfg::BN);
      const int as = tile_iter & 1;
      const uint32_t aph = (tile_iter >> 1) & 1;
      c.conv_tile = t;
      c.m_warp = quad * 32;                       // tile row of this warp's first row (see EVTB_ROW_M)
#pragma unroll
      for (int i = 0; i < 4; ++i) c.m_rows[i] = conv_row_to_m(p, t, quad * 32 + i * 8 + (lane >> 2));
      c.m = conv_row_to_m(p, t, quad * 32 + lane);
      c.n0 = t.n0;
      c.row_ok = c.m < p.M;
      if (!wait_or_abort(&hdr->tmem_full[as], aph, &hdr->abort_flag)) {
        report_status(p.status, DEV_TIMEOUT_EPILOGUE);
        hdr->abort_flag = 1;
        break;
      }
      tcgen05_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                             static_cast<uint32_t>(as * Cfg::BN);
      epi.tile_begin(c);
      epilogue_tile<Cfg>(epi, c, taddr, col_group, p.NT, p.cls[t.cls].ntaps == 0);
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&hdr->tmem_empty[as]);
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
