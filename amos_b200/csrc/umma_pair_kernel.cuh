// CTA-pair variant of the persistent tcgen05 kernel: a cluster of two CTAs (two SMs) computes one
// 256 (M) x BN (N) tile with tcgen05.mma.cta_group::2.  Modes: GEMM, NCHW convolution on the
// re-laid-out operands (16-bit elements), NHWC and HWNC convolution in place; kinds f16 / bf16,
// int8 and tf32 (the latter two: GEMM and the in-place convolutions).
//
// Each CTA of the pair owns 128 rows of the tile: it loads its own 128-row A tile and HALF of the
// B tile (BN/2 columns), and holds the 128 x BN accumulator of its rows in its own TMEM.  The MMA
// is issued by one thread of the even ("leader") CTA and reads A and B from the shared memory of
// both CTAs, so every byte of B is fetched from L2 once per pair instead of once per CTA: per
// k-step a CTA moves 16 KB (A) + BN/2 x 128 B (B) for 128 x BN x 64 MACs, against 16 KB + BN x 128 B
// in the single-CTA kernel.
//
// Synchronisation (all mbarriers; every wait bounded):
//   full[s]        leader only, count 1: leader's producer arms it with the bytes of BOTH CTAs;
//                  both CTAs' TMA loads credit it (cp.async.bulk.tensor.cta_group::2).
//   empty[s]       in both CTAs, count 1: tcgen05.commit of the leader arrives on both.
//   tmem_full[a]   in both CTAs, count 1: same commit form, accumulator `a` is complete.
//   tmem_empty[a]  leader only, count 8: the four epilogue warps of each CTA arrive on it.
// No load in this file has more than one destination CTA.
#pragma once
#include "umma_kernel.cuh"

namespace amosb {

template <int BN, bool EPI_TMA>
struct PairConfig {
  static constexpr int kBTileBytes = (BN / 2) * 128;  // this CTA's half of B
  static constexpr int kStageBytes = kATileBytes + kBTileBytes;
  static constexpr int kStages = (BN == 256) ? 6 : 8;  // 192 KB of stages either way
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kEpiRegion = EPI_TMA ? kEpiBytes : 0;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiRegion + kBarrierBytes + 1024;
};

template <int KIND, int BN, bool B_MN_MAJOR, int MODE, typename OutT, bool EPI_TMA>
__global__ void __launch_bounds__(kNumThreads, 1)
umma_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const UmmaParams p) {
  using Cfg = PairConfig<BN, EPI_TMA>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kElemsPer128B = (KIND == 0) ? 64 : (KIND == 1) ? 128 : 32;
  constexpr int kUmmaKRows = (KIND == 0) ? 16 : (KIND == 1) ? 32 : 8;
  static_assert(KIND != 2 || MODE == kModeGemm || MODE == kModeConvNhwc || MODE == kModeConvHwnc,
                "float32 (tf32) pairs: GEMM and NHWC / HWNC convolution");
  static_assert(MODE != kModeConvHwnc || B_MN_MAJOR, "HWNC conv reads the RSCK filter MN-major");
  constexpr int kMmaPerStage = 4;
  constexpr uint32_t kBChunkBytes = kElemsPer128B * 128;
  constexpr int kBChunksPerCta = (BN / 2) / kElemsPer128B;  // MN-major chunks this CTA loads
  constexpr int kPairM = 2 * kBlockM;
  static_assert(BN == 256 || BN == 128, "pair tiles are 256 or 128 columns wide");
  static_assert(!B_MN_MAJOR || ((BN / 2) % kElemsPer128B == 0), "half of B must be whole chunks");
  static_assert(MODE != kModeConv || !B_MN_MAJOR, "NCHW conv consumes a K-major prepacked filter");
  static_assert(MODE != kModeConvNhwc || B_MN_MAJOR, "NHWC conv reads the RSCK filter MN-major");
  static_assert(!EPI_TMA || MODE != kModeConv, "the TMA-store epilogue writes row-major C");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t epi_base = smem_base + kStages * Cfg::kStageBytes;
  uint8_t* bar_region = smem_aligned + kStages * Cfg::kStageBytes + Cfg::kEpiRegion;
  const uint32_t bar_base = epi_base + Cfg::kEpiRegion;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
  auto tmem_empty_bar = [&](int s) { return bar_base + 8u * (2 * kStages + 2 + s); };
  volatile uint32_t* tmem_base_slot =
      reinterpret_cast<volatile uint32_t*>(bar_region + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_region + 8 * (2 * kStages + 4) + 8);

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const uint32_t rank = cluster_cta_rank();  // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  // ------------------------------------------------------------------ set-up
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    if constexpr (EPI_TMA) prefetch_tensormap(&tmC);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tmem_full_bar(s), 1);
      mbar_init(tmem_empty_bar(s), 8);  // four epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc_2cta(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), Cfg::kTmemCols);
    tmem_relinquish_2cta();
  }
  tc_fence_before_sync();
  __syncthreads();
  // the peer's barriers must exist before anything is signalled across the pair
  cluster_arrive();
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  const int tiles_per_batch = p.tiles_m * p.tiles_n;  // tiles_m counts 256-row tiles here
  auto decode_tile = [&](int tile, int& b, int& m_blk, int& n_blk) {
    b = tile / tiles_per_batch;
    const int t = tile - b * tiles_per_batch;
    const int group_sz = p.group_m * p.tiles_n;
    const int g = t / group_sz;
    const int first_m = g * p.group_m;
    const int gm = min(p.tiles_m - first_m, p.group_m);
    const int r = t - g * group_sz;
    m_blk = first_m + r % gm;
    n_blk = r / gm;
  };

  // A pair's work units are whole 256 x BN tiles, or k-block ranges of them where the schedule
  // shares out a short last round (see SegmentIter).  (Cutting tiles into column slices was tried:
  // a pair MMA of half the width costs its issuing thread the same, so it did not pay.)
  constexpr int n_off = 0;
  constexpr int width = BN;

  if (warp == 0 || warp >= 6) {
    // ================================================================ TMA producer (both CTAs)
    // Up to three issuing threads (lane 0 of warps 0, 6, 7).  The pair's k-blocks form one stream
    // across its units; thread pi owns k-blocks pi, pi + P, pi + 2P, ... of that stream.  The
    // loop only adds and compares (no integer division per k-block): positions advance by P steps.
    const int pi = warp == 0 ? 0 : warp - 5;
    const int P = min(p.producers, kStages);  // stage = pi + j * P below needs P <= kStages
    if (lane == 0 && pi < P && !p.diag_no_loads) {
      // the kernel may have been started while its predecessor in the stream was still running
      // (for the NCHW conv that is the re-layout kernel that writes both operands): nothing is
      // read from global memory before that kernel has completed
      grid_dependency_wait();
      int stage = pi;
      uint32_t phase = 0;
      bool ok = true;
      int kb = pi;  // this thread's next k-block inside the current unit
#ifdef AMOSB_ROLE_CYCLES
      long long rc_wait = 0;
      const long long rc_begin = clock64();
#endif
      SegmentIter it(p, pair_id, num_pairs);
      Segment sg;
      while (ok && it.next(p, sg)) {
        // `kb` counts inside the segment; the k-block it names is sg.kb_begin + kb
        const int seg_len = sg.kb_end - sg.kb_begin;
        if (kb >= seg_len) {  // fewer k-blocks in the segment than issuing threads
          kb -= seg_len;
          continue;
        }
        int b, m_blk, n_blk;
        decode_tile(sg.tile, b, m_blk, n_blk);
        const int m0 = m_blk * kPairM + static_cast<int>(rank) * kBlockM;  // first row of this CTA
        const int half = width >> 1;                                       // B columns of this CTA
        const int n_half0 = n_blk * BN + n_off + static_cast<int>(rank) * half;
        const uint32_t stage_tx = 2u * (kATileBytes + static_cast<uint32_t>(half) * 128u);
        int cw = 0, ch = 0, cn = 0;
        int cc = 0, fs = 0, fr = 0;  // channel chunk and filter tap of k-block kb
        if constexpr (MODE != kModeGemm) {
          int op, oq;
          if constexpr (MODE == kModeConvHwnc) {
            // this CTA's 128 rows: 128 images of one output pixel, or (few images) a group of
            // consecutive pixels of an output row x the images -- as in the single-CTA kernel
            if (p.hw_group > 1) {
              const int t = m0 / kBlockM;
              op = t / p.hw_qgroups;
              oq = (t - op * p.hw_qgroups) * p.hw_group;
              cn = 0;
            } else {
              const int pq = m0 / p.conv_N;
              cn = m0 - pq * p.conv_N;
              op = pq / p.Q;
              oq = pq - op * p.Q;
            }
          } else {
            cn = m0 / p.PQ;
            const int pq = m0 - cn * p.PQ;
            op = pq / p.Q;
            oq = pq - op * p.Q;
          }
          cw = oq * p.stride_w - p.pad_w;
          ch = op * p.stride_h - p.pad_h;
          const int rs = (sg.kb_begin + kb) / p.c_chunks;
          cc = (sg.kb_begin + kb) - rs * p.c_chunks;
          fr = rs / p.S;
          fs = rs - fr * p.S;
        }
        for (; kb < seg_len; kb += P) {
          const int kabs = sg.kb_begin + kb;
#ifdef AMOSB_ROLE_CYCLES
          const long long rc_t0 = clock64();
#endif
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status,
                         kStatusTimeoutProducer, p.wait_budget_ns)) {
            ok = false;
            break;
          }
#ifdef AMOSB_ROLE_CYCLES
          rc_wait += clock64() - rc_t0;
#endif
          const uint32_t sA = smem_base + stage * Cfg::kStageBytes;
          const uint32_t sB = sA + kATileBytes;
          const uint32_t fb = full_bar(stage);  // credited on the leader's copy of this barrier
          if (rank == 0) mbar_arrive_expect_tx(fb, stage_tx);
          if constexpr (MODE == kModeGemm) {
            tma_load_3d_pair(sA, &tmA, fb, kabs * kElemsPer128B, m0, p.a_bcast ? 0 : b);
            if constexpr (B_MN_MAJOR) {
              for (int j = 0; j * kElemsPer128B < half; ++j) {
                tma_load_3d_pair(sB + j * kBChunkBytes, &tmB, fb, n_half0 + j * kElemsPer128B,
                                 kabs * kElemsPer128B, b);
              }
            } else {
              // K-major B arrives in boxes of 64 rows
              for (int j = 0; j * 64 < half; ++j) {
                tma_load_3d_pair(sB + j * 64 * 128, &tmB, fb, kabs * kElemsPer128B, n_half0 + j * 64, b);
              }
            }
          } else {
            if constexpr (MODE == kModeConvHwnc) {
              // {channels, images, w, h}: padding and rows past the last pixel are out-of-range
              // coordinates -> zeros
              tma_load_4d_pair(sA, &tmA, fb, cc * kElemsPer128B, cn, cw + fs * p.dil_w,
                               ch + fr * p.dil_h);
            } else {
              tma_load_im2col_4d_pair(sA, &tmA, fb, cc * kElemsPer128B, cw, ch, cn,
                                      static_cast<uint16_t>(fs * p.dil_w),
                                      static_cast<uint16_t>(fr * p.dil_h));
            }
            if constexpr (MODE == kModeConv) {
              for (int j = 0; j * 64 < half; ++j) {
                tma_load_2d_pair(sB + j * 64 * 128, &tmB, fb, kabs * kElemsPer128B, n_half0 + j * 64);
              }
            } else {
              const int brow = (fr * p.S + fs) * p.conv_C + cc * kElemsPer128B;
              for (int j = 0; j * kElemsPer128B < half; ++j) {
                tma_load_3d_pair(sB + j * kBChunkBytes, &tmB, fb, n_half0 + j * kElemsPer128B,
                                 brow, 0);
              }
            }
            cc += P;
            while (cc >= p.c_chunks) {
              cc -= p.c_chunks;
              if (++fs == p.S) {
                fs = 0;
                ++fr;
              }
            }
          }
          stage += P;
          if (stage >= kStages) {
            stage -= kStages;
            phase ^= 1u;
          }
        }
        kb -= seg_len;
      }
#ifdef AMOSB_ROLE_CYCLES
      if (pi == 0) {
        atomicAdd(&p.role_cycles[rank == 0 ? 0 : 8], (unsigned long long)rc_wait);
        atomicAdd(&p.role_cycles[rank == 0 ? 1 : 9], (unsigned long long)(clock64() - rc_begin));
      }
#endif
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
#ifdef AMOSB_ROLE_CYCLES
      long long rc_full = 0, rc_tmem = 0, rc_issue = 0, rc_commit = 0;
      const long long rc_begin = clock64();
#endif
      SegmentIter it(p, pair_id, num_pairs);
      Segment sg;
      while (ok && it.next(p, sg)) {
        const uint32_t idesc = make_idesc<KIND>(kPairM, width, B_MN_MAJOR) | p.idesc_formats;
#ifdef AMOSB_ROLE_CYCLES
        const long long rc_t1 = clock64();
#endif
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag, p.status,
                       kStatusTimeoutMmaTmem, p.wait_budget_ns)) {
          ok = false;
          break;
        }
#ifdef AMOSB_ROLE_CYCLES
        rc_tmem += clock64() - rc_t1;
#endif
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = sg.kb_begin; kb < sg.kb_end; ++kb) {
#ifdef AMOSB_ROLE_CYCLES
          const long long rc_t0 = clock64();
#endif
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, kStatusTimeoutMmaFull, p.wait_budget_ns)) {
            ok = false;
            break;
          }
#ifdef AMOSB_ROLE_CYCLES
          rc_full += clock64() - rc_t0;
#endif
          tc_fence_after_sync();
          const uint32_t sA = smem_base + stage * Cfg::kStageBytes;
          const uint32_t sB = sA + kATileBytes;
#ifdef AMOSB_ROLE_CYCLES
          const long long rc_t2 = clock64();
#endif
          constexpr int kAStep = 32 >> 4;
          constexpr int kBStep = B_MN_MAJOR ? (kUmmaKRows * 128) >> 4 : 32 >> 4;
          // MN-major operands of 32-bit elements lie in the 128-byte swizzle with 32-byte units
          constexpr uint32_t kHiMn =
              KIND == 2 ? smem_desc_hi_sw128_base32(512) : smem_desc_hi_sw128(1024);
          umma_kblock4<KIND, true, kAStep, kBStep>(tmem_d, smem_desc_lo(sA, 16),
                                                   smem_desc_lo(sB, B_MN_MAJOR ? kBChunkBytes : 16),
                                                   smem_desc_hi_sw128(1024),
                                                   B_MN_MAJOR ? kHiMn : smem_desc_hi_sw128(1024), idesc,
                                                   kb != sg.kb_begin ? 1u : 0u);
#ifdef AMOSB_ROLE_CYCLES
          const long long rc_t3 = clock64();
          rc_issue += rc_t3 - rc_t2;
#endif
          umma_commit_2cta(empty_bar(stage));  // frees this stage in both CTAs
#ifdef AMOSB_ROLE_CYCLES
          rc_commit += clock64() - rc_t3;
#endif
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_2cta(tmem_full_bar(acc));  // accumulator complete, in both CTAs
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
#ifdef AMOSB_ROLE_CYCLES
      atomicAdd(&p.role_cycles[2], (unsigned long long)rc_full);
      atomicAdd(&p.role_cycles[3], (unsigned long long)rc_tmem);
      atomicAdd(&p.role_cycles[4], (unsigned long long)(clock64() - rc_begin));
      atomicAdd(&p.role_cycles[7], 1ull);
      atomicAdd(&p.role_cycles[10], (unsigned long long)rc_issue);
      atomicAdd(&p.role_cycles[11], (unsigned long long)rc_commit);
#endif
    }
  } else {
    // ================================================================ epilogue (both CTAs)
    // The next kernel in the stream, if it was launched as a programmatic dependent, may take this
    // CTA's SM as soon as the CTA exits and set itself up while the rest of this grid finishes.
    // Issued from an epilogue thread, which has nothing to do yet: the instruction holds its thread
    // for about a microsecond, which the threads that start the pipeline cannot spare.
    if (warp == 2 && lane == 0) grid_launch_dependents();
    // addend reads and output stores, too, come after the predecessor kernel has completed
    grid_dependency_wait();
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    int epi_buf = 0;
    OutT* const out = reinterpret_cast<OutT*>(p.out);
#ifdef AMOSB_ROLE_CYCLES
    long long rc_wait = 0;
    const long long rc_begin = clock64();
#endif
    constexpr size_t kPartialElems = static_cast<size_t>(kBlockM) * BN;  // per CTA slot
    const int my_slot = blockIdx.x;  // a pair's two CTAs keep the sums of their own 128 rows
    SegmentIter it(p, pair_id, num_pairs);
    Segment sg;
    while (ok && it.next(p, sg)) {
      int b, m_blk, n_blk;
      decode_tile(sg.tile, b, m_blk, n_blk);
#ifdef AMOSB_ROLE_CYCLES
      const long long rc_t0 = clock64();
#endif
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag, p.status, kStatusTimeoutEpilogue, 2 * p.wait_budget_ns)) {
        ok = false;
        break;
      }
#ifdef AMOSB_ROLE_CYCLES
      rc_wait += clock64() - rc_t0;
#endif
      tc_fence_after_sync();
      // shared-out tile: see the single-CTA kernel; the workers are pairs, and the CTA of rank r
      // exchanges sums with the CTAs of rank r of the other pairs
      const bool sk_contrib = sg.kb_begin > 0;
      int fix_first = 0, fix_last = -1;
      if (!sk_contrib && sg.kb_end < p.num_kb) {
        fix_first = pair_id + 1;
        fix_last = sk_worker_of(
            p, static_cast<long long>(sg.tile - p.sk_first) * p.num_kb + p.num_kb - 1);
        bool got = true;
        if (lane == 0) {
          for (int cw = fix_first; got && cw <= fix_last; ++cw)
            got = gflag_wait(p.sk_flags + (2 * cw + static_cast<int>(rank)) * 4 + quarter,
                             abort_flag, p.status, 2 * p.wait_budget_ns);
        }
        if (__shfl_sync(0xffffffffu, got ? 1 : 0, 0) == 0) {
          ok = false;
          break;
        }
      }
      if (sk_contrib || fix_last >= fix_first) {
        const uint32_t taddr_q =
            tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
        const size_t part_lane = static_cast<size_t>(quarter * 32) + lane;
        if (sk_contrib) {
          sk_dump_partials<BN>(taddr_q,
                               p.sk_partials + static_cast<size_t>(my_slot) * kPartialElems + part_lane);
          __threadfence();  // the partial sums are in L2 before the flag says so
          __syncwarp();
          if (lane == 0) {
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.sk_flags + my_slot * 4 + quarter),
                         "r"(1u)
                         : "memory");
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_leader(tmem_empty_bar(acc));
          if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1u;
          }
          continue;
        }
        // slot of pair cw's CTA of this rank: 2 * cw + rank
        sk_add_partials<KIND, BN>(taddr_q,
                                  p.sk_partials + static_cast<size_t>(rank) * kPartialElems + part_lane,
                                  fix_first, fix_last, 2 * kPartialElems);
        __syncwarp();  // every lane has read its partial sums: the flags can be reused
        if (lane == 0) {
          for (int cw = fix_first; cw <= fix_last; ++cw)
            p.sk_flags[(2 * cw + static_cast<int>(rank)) * 4 + quarter] = 0u;
        }
      }
      const int row0 = m_blk * kPairM + static_cast<int>(rank) * kBlockM + quarter * 32;
      const int row = row0 + static_cast<int>(lane);
      // row of the output matrix this thread holds and whether it exists; HWNC: a GEMM row is
      // (pixel, image), laid out as in the single-CTA kernel (see there)
      int orow = row;
      bool row_ok = row < p.M;
      int st_row = row0, st_batch = b, st_q = 0;  // where this warp's TMA-store box starts
      if constexpr (MODE == kModeConvHwnc) {
        if (p.hw_group > 1) {
          const int t = row0 / kBlockM;
          const int op = t / p.hw_qgroups;
          const int q0 = (t - op * p.hw_qgroups) * p.hw_group;
          const int r = quarter * 32 + static_cast<int>(lane);
          const int g = r / p.hw_nbox, img = r - g * p.hw_nbox;
          orow = (op * p.Q + q0 + g) * p.conv_N_real + img;
          row_ok = row_ok && q0 + g < p.Q && img < p.conv_N_real;
          st_batch = op;
          st_q = q0 + (quarter * 32) / p.hw_nbox;
          st_row = (quarter * 32) % p.hw_nbox;
          if (st_q >= p.Q) st_row = p.conv_N_real;  // nothing of this warp exists
        } else {
          const int pix = row / p.conv_N;
          const int img = row - pix * p.conv_N;
          orow = pix * p.conv_N_real + img;
          row_ok = row_ok && img < p.conv_N_real;
          const int spix = row0 / p.conv_N;
          st_row = row0 - spix * p.conv_N;
          st_batch = spix / p.Q;
          st_q = spix - st_batch * p.Q;
        }
      }
      (void)st_q;
      const uint32_t taddr_row =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
      auto run_chunks = [&](int nch, auto&& process) { for_each_chunk(taddr_row, nch, process); };
      // chunks of this unit that hold columns < N (warp-uniform); none when all rows are >= M
      const int cols_left = p.N - (n_blk * BN + n_off);
      int valid_chunks = row0 < p.M ? min(width >> 5, (cols_left + 31) >> 5) : 0;
      if constexpr (MODE == kModeConvHwnc) {
        // all 32 rows of this warp are padding images, or pixels past the end of the output row
        if (st_row >= p.conv_N_real) valid_chunks = 0;
      }
      if constexpr (EPI_TMA) {
        constexpr int kColsPerStore = 128 / static_cast<int>(sizeof(OutT));
        constexpr int kLoadsPerStore = kColsPerStore / 32;
        const uint32_t my_epi = epi_base + static_cast<uint32_t>((warp - 2) * kEpiBytesPerWarp);
        const uint32_t swz = (lane & 7u) << 4;
        // whole stores only: a chunk past N inside the last store is clipped by the store engine
        const int nch = (valid_chunks + kLoadsPerStore - 1) / kLoadsPerStore * kLoadsPerStore;
        run_chunks(nch, [&](uint32_t(&r)[32], int c) {
          const int st = c / kLoadsPerStore;
          const int h = c - st * kLoadsPerStore;
          const int col0 = n_blk * BN + n_off + st * kColsPerStore;
          if (h == 0) {
            if (lane == 0) tma_store_wait_read<kEpiBufs - 1>();  // the oldest buffer is free again
            __syncwarp();
          }
          const uint32_t buf = my_epi + static_cast<uint32_t>(epi_buf * kEpiBufBytes);
          const uint32_t row_addr = buf + lane * 128u;
          {
            const int c0h = col0 + h * 32;
            const long long off =
                (p.epi_flags & kEpiAddRowVec)
                    ? static_cast<long long>(row)
                    : static_cast<long long>(b) * p.c_batch_stride +
                          static_cast<long long>(orow) * p.ldc + c0h;
            const void* fp = addend_ptr(p, off);
            apply_trailing_ops<KIND>(r, p, c0h, p.N - c0h, row_ok, fp, 1);
          }
          stage_chunk<OutT>(row_addr, swz, h, r);
          if (h == kLoadsPerStore - 1) {
            fence_proxy_async_smem();  // generic-proxy smem writes -> visible to the TMA engine
            __syncwarp();
            if (lane == 0) {
              if constexpr (MODE == kModeConvHwnc) {
                tma_store_4d(&tmC, buf, col0, st_row, st_q, st_batch);
              } else {
                tma_store_3d(&tmC, buf, col0, row0, b);
              }
              tma_store_commit();
            }
            epi_buf = epi_buf + 1 == kEpiBufs ? 0 : epi_buf + 1;
          }
        });
      } else {
        OutT* row_ptr = nullptr;
        OutT* quad_ptr = nullptr;  // NCHW in 4-pixel units: this lane's channel and 4-row group
        bool quad_ok = false;
        if constexpr (MODE != kModeConv) {
          row_ptr = out + static_cast<long long>(b) * p.c_batch_stride +
                    static_cast<long long>(orow) * p.ldc;
        } else {
          const int n_img = row / p.PQ;
          const int pq = row - n_img * p.PQ;
          row_ptr = out + (static_cast<long long>(n_img) * p.N) * p.PQ + pq;
          if (p.nchw_quads) {
            const int qrow = row0 + static_cast<int>(lane & ~3u);
            const int q_img = qrow / p.PQ;
            quad_ok = qrow < p.M;
            quad_ptr = out + (static_cast<long long>(q_img) * p.N + (lane & 3u)) * p.PQ +
                       (qrow - q_img * p.PQ);
          }
        }
        run_chunks(valid_chunks, [&](uint32_t(&r)[32], int c) {
          const int col0 = n_blk * BN + n_off + c * 32;
          const int ncols_valid = p.N - col0;
          if (p.epi_flags != 0) {
            long long off, stride;
            if constexpr (MODE != kModeConv) {
              off = (p.epi_flags & kEpiAddRowVec)
                        ? static_cast<long long>(row)
                        : static_cast<long long>(b) * p.c_batch_stride +
                              static_cast<long long>(orow) * p.ldc + col0;
              stride = 1;
            } else {
              const int ni = row / p.PQ;
              off = (static_cast<long long>(ni) * p.N + col0) * p.PQ + (row - ni * p.PQ);
              stride = p.PQ;
            }
            const void* fp = addend_ptr(p, off);
            apply_trailing_ops<KIND>(r, p, col0, ncols_valid, row_ok, fp, stride);
          }
          if constexpr (MODE == kModeConv) {
            if (p.nchw_quads) {  // warp-uniform
              store_nchw_quads<OutT>(quad_ptr + static_cast<long long>(col0) * p.PQ, p.PQ, r,
                                     ncols_valid, lane, quad_ok);
              return;
            }
          }
          if (row_ok) {
            if constexpr (MODE != kModeConv) {
              store_row_chunk<OutT>(row_ptr + col0, r, ncols_valid);
            } else {
              // NCHW: lanes of a warp are consecutive pixels of one channel plane -> coalesced.
              // The epilogue of these kernels is bound by the instructions it issues, so the usual
              // case of 32 channels that all exist carries no per-element test.
              OutT* dst = row_ptr + static_cast<long long>(col0) * p.PQ;
              if (ncols_valid >= 32) {
#pragma unroll
                for (int j = 0; j < 32; ++j) dst[static_cast<long long>(j) * p.PQ] = convert_acc<OutT>(r[j]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  if (j < ncols_valid) dst[static_cast<long long>(j) * p.PQ] = convert_acc<OutT>(r[j]);
                }
              }
            }
          }
        });
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(tmem_empty_bar(acc));  // the MMA issuer lives in the leader
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if constexpr (EPI_TMA) {
      if (lane == 0) tma_store_wait_all<0>();
    }
#ifdef AMOSB_ROLE_CYCLES
    if (warp == 2 && lane == 0 && rank == 0) {
      atomicAdd(&p.role_cycles[5], (unsigned long long)rc_wait);
      atomicAdd(&p.role_cycles[6], (unsigned long long)(clock64() - rc_begin));
    }
#endif
    (void)epi_buf;
    (void)out;
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 50; ++i) __nanosleep(20000);
  }
  tc_fence_before_sync();
  __syncthreads();
  // neither CTA may leave while the other can still read its shared memory or signal its barriers
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_2cta(tmem_base, Cfg::kTmemCols);
  }
}

}  // namespace amosb
