// Persistent, warp-specialised tcgen05 kernel shared by GEMM, batched GEMM and conv2d (implicit
// GEMM).  One CTA per SM, 256 threads:
//   warps 0, 6, 7  TMA producers (one lane each issues cp.async.bulk.tensor into a ring of smem
//                                 stages; the k-blocks are dealt round-robin)
//   warp 1         MMA issuer    (one lane issues tcgen05.mma into one of two TMEM accumulators;
//                                 the warp also owns TMEM alloc/dealloc).  Tall tiles (MT = 2) make
//                                 warp 7 a second issuer, one per accumulator tile.
//   warps 2..5     epilogue      (tcgen05.ld -> registers -> cast -> stores; overlaps with the main
//                                 loop of the next tile through the second accumulator)
//
// Tile: 128 (M) x BN (N) x 128 bytes of K per stage (64 fp16 or 128 int8).
// A is always K-major (rows of K contiguous).  B is either K-major ([N,K], used for the prepacked
// conv filter and the transposed-B GEMM) or MN-major ([K,N] row-major, the `te` GEMM layout), in
// which case the operand is consumed in place with no transpose pass.
#pragma once
#include "ptx.cuh"
#include <cuda_fp16.h>

namespace amosb {

constexpr int kBlockM = 128;
constexpr int kStageKBytes = 128;           // bytes of K per stage row (one 128B swizzle span)
constexpr int kATileBytes = kBlockM * 128;  // 16 KB
constexpr int kNumThreads = 256;  // 8 warps: 0 producer, 1 MMA, 2-5 epilogue, 6-7 extra producers
constexpr int kPwCopyWarps = 4;   // kModeConvPw: warps 8..11 copy the activation
constexpr int kNumThreadsPw = kNumThreads + 32 * kPwCopyWarps;
constexpr int umma_threads(int mode) { return mode == 4 ? kNumThreadsPw : kNumThreads; }

// kModeConv: NCHW activation re-laid-out to NHWC scratch + prepacked K-major filter, NCHW output.
// kModeConvNhwc: NHWC activation and RSCK filter consumed in place (im2col A, MN-major B), NHWC
// output = row-major [pixels][K] like a GEMM.
// kModeConvHwnc: activation [H,W,N,C] and RSCK filter consumed in place, output [P,Q,N,K].  GEMM
// rows are (p, q, n) with n fastest and N padded to a multiple of 128 (images past N load as zeros
// and are not stored), so a 128-row tile is one output pixel
// times 128 consecutive images: its A operand for a filter tap is a plain tiled box
// {64 channels, 128 images} of the input pixel (p*st + r*dil - pad, q*st + s*dil - pad), and a
// pixel outside the image is an out-of-range coordinate that the load fills with zeros.  With at
// most 64 images and stride 1 along W the images are padded to 8, 16, 32 or 64 instead and a
// 128-row tile is that many images x 128 / that many consecutive pixels of an output row (box
// {64 channels, images, pixels, 1}; UmmaParams::hw_group / hw_nbox / hw_qgroups).
// kModeConvPw: 1x1, stride-1, unpadded NCHW convolution consumed in place when the channel planes
// are not 16-byte multiples (so that no tensor map can describe them): GEMM rows are the pixels
// (n, p, q) flattened, the activation [C][P*Q] of an image is an MN-major A operand that four extra
// warps copy into the stages with 8-byte cp.async (four pixels each, written straight into the
// 128-byte-swizzled layout the copy engine would have produced), the KCRS filter is the K-major B
// operand through TMA, the output is NCHW as in kModeConv.  No re-layout pass, no scratch.
enum : int { kModeGemm = 0, kModeConv = 1, kModeConvNhwc = 2, kModeConvHwnc = 3, kModeConvPw = 4 };
enum : int { kEpiAddVec = 1, kEpiAddFull = 2, kEpiRelu = 4, kEpiAddRowVec = 8 };

struct UmmaParams {
#ifdef AMOSB_ROLE_CYCLES
  unsigned long long* role_cycles;  // diagnostic build only: cycles per role, summed over CTAs
  int dbg_skip;  // diagnostic build only: 1 = issue no A loads, 2 = no B loads (results are garbage)
#endif
  // GEMM view of the problem (per batch). conv: M = N_img*P*Q, N = K_out, K = R*S*C_pad.
  int M, N, K;
  int batch;
  int tiles_m, tiles_n;  // per batch
  int mt;                // accumulator tiles (128 rows each) per CTA tile: 1, or 2 for tall tiles
  // operand-format bits OR-ed into the instruction descriptor: 0 for fp16 / int8 (the kernel's
  // KIND fixes those), A and B format = 1 (bits 7 and 10) for bfloat16 inputs of KIND 0
  uint32_t idesc_formats;
  int group_m;           // raster group height in tiles
  int num_kb;            // K blocks per tile
  int num_tiles;         // batch * tiles_m * tiles_n
  long long ldc;             // GEMM: output row stride in elements
  long long c_batch_stride;  // GEMM: output batch stride in elements
  void* out;
  int* status;
  int a_bcast;  // GEMM family: 1 if every batch uses the same A (batch coordinate 0)
  // fused trailing element-wise stages, applied to the accumulator before the final cast:
  // out = cast(relu?(acc + addend?)).  The addend is either a vector indexed by the N column
  // (GEMM: j, conv: output channel) or a tensor of the output's shape.
  int nchw_quads;       // NCHW output planes are whole 4-pixel groups and aligned: store 4 pixels at a time
  int epi_flags;        // kEpiAddVec | kEpiAddFull | kEpiRelu | kEpiAddRowVec (vector indexed by the row)
  int addend_f16;       // addend stored as fp16 (cast to the accumulator type before the add)
  const void* addend;
  // conv geometry
  int P, Q, PQ;
  int c_chunks;  // 128-byte channel chunks per filter tap
  int S;         // filter width
  int conv_C;    // NHWC / HWNC modes: channels (row pitch of the RSCK filter viewed as [R*S*C][K])
  int conv_N;    // HWNC mode: images per output pixel in the GEMM row index, padded to 128
  int conv_N_real;  // HWNC mode: images that exist (rows past them are computed on zeros, not stored)
  // HWNC mode with fewer than 128 images: a 128-row tile is hw_group consecutive pixels of one
  // output row x hw_nbox images (hw_group * hw_nbox = 128; hw_group = 1: the tile is 128 images
  // of one pixel); hw_qgroups such tiles cover an output row
  int hw_group, hw_nbox, hw_qgroups;
  int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  int producers;   // 1..3 threads (in warps 0, 6, 7) issuing the TMA loads, k-blocks dealt round-robin
  const void* act;  // kModeConvPw: the NCHW activation (16-bit elements)
  // Shared-out tail.  Whole tiles are dealt round-robin to the CTAs (CTA pairs); when the tile
  // count does not fill the last round, the k-blocks of the last `sk_tiles` tiles, taken as one
  // sequence, are cut into equal shares instead, one per worker: worker w gets
  // sk_q + (w < sk_r) k-blocks starting at w * sk_q + min(w, sk_r).  A share that starts inside a
  // tile yields partial sums, which its CTA leaves in `sk_partials` (one accumulator tile per
  // CTA, 32-bit) and announces in `sk_flags` ([CTA][4], one per epilogue warp); the CTA whose
  // share holds the tile's first k-block adds them to its own and stores the tile.
  int sk_tiles;   // 0: every tile is computed whole by one worker
  int sk_first;   // first shared tile (= num_tiles - sk_tiles)
  int sk_q, sk_r;
  uint32_t* sk_partials;
  unsigned int* sk_flags;
  // Nanoseconds after which a wait on an mbarrier is given up (the CTA then raises its abort flag,
  // records a status code and leaves).  An epilogue wait spans the whole k-loop of a tile, each of
  // whose own waits has this budget, so it gets twice as much.
  unsigned long long wait_budget_ns;
  // Diagnostic: the copy-issuing threads issue no loads and arm no barrier, so that the MMA
  // thread's first wait runs out with nothing in flight.  The way the give-up path is exercised.
  int diag_no_loads;
};

// One piece of a worker's schedule: k-blocks [kb_begin, kb_end) of `tile`.
struct Segment {
  int tile, kb_begin, kb_end;
};
// The schedule of worker `w` of `nw`: first its share of the shared-out tail (so that partial
// sums are ready long before the CTA that adds them up asks), then its whole tiles.  Every role
// of a CTA walks the same sequence.
struct SegmentIter {
  long long u, u_end;  // next and end unit (k-block of the shared tiles' sequence) of the share
  int dp_tile, nw;
  __device__ __forceinline__ SegmentIter(const UmmaParams& p, int w, int workers) {
    nw = workers;
    dp_tile = w;
    if (p.sk_tiles > 0) {
      u = static_cast<long long>(w) * p.sk_q + min(w, p.sk_r);
      u_end = u + p.sk_q + (w < p.sk_r ? 1 : 0);
    } else {
      u = u_end = 0;
    }
  }
  __device__ __forceinline__ bool next(const UmmaParams& p, Segment& s) {
    if (u < u_end) {
      const int t = static_cast<int>(u / p.num_kb);
      const int kb = static_cast<int>(u - static_cast<long long>(t) * p.num_kb);
      const int len = static_cast<int>(min(static_cast<long long>(p.num_kb - kb), u_end - u));
      s.tile = p.sk_first + t;
      s.kb_begin = kb;
      s.kb_end = kb + len;
      u += len;
      return true;
    }
    if (dp_tile < p.sk_first) {
      s.tile = dp_tile;
      s.kb_begin = 0;
      s.kb_end = p.num_kb;
      dp_tile += nw;
      return true;
    }
    return false;
  }
};
// Worker whose share holds unit `u` of the shared tiles' sequence.
__device__ __forceinline__ int sk_worker_of(const UmmaParams& p, long long u) {
  const long long big = static_cast<long long>(p.sk_r) * (p.sk_q + 1);
  if (u < big) return static_cast<int>(u / (p.sk_q + 1));
  return p.sk_r + static_cast<int>((u - big) / p.sk_q);
}
constexpr int kStatusTimeoutPartials = 106;  // an epilogue warp waited for another CTA's partial sums

// Bounded wait for a flag in global memory that another CTA of this grid sets (all CTAs of the
// grid are resident: the grid never exceeds one CTA per SM).
__device__ __forceinline__ bool gflag_wait(const unsigned int* flag, volatile int* abort_flag,
                                           int* status, uint64_t budget_ns) {
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (true) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v != 0) return true;
    if ((++spins & 0x3Fu) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > budget_ns) {
        *abort_flag = 1;
        atomicCAS(status, 0, kStatusTimeoutPartials);
        return false;
      }
    }
  }
}

// The two halves of the exchange of partial sums, kept out of line: they run for a handful of
// tiles per launch, and inlined into the epilogue's chunk loop they cost every kernel 70 registers
// and a third of its speed on short shapes.  `taddr_row` = this warp's lane quarter, first column
// of the accumulator; COLS = accumulator columns of the CTA's tile (MT * BN).  A partial tile is
// laid out [column][128 rows], so a warp moves 128 contiguous bytes per register.
//
// Contributor: the raw accumulator words go to this CTA's slot (`dst` = slot + this thread's row).
template <int COLS>
__device__ __noinline__ void sk_dump_partials(uint32_t taddr_row, uint32_t* dst) {
  uint32_t r[32];
#pragma unroll 1
  for (int c = 0; c < COLS / 32; ++c) {
    tmem_ld_32x32b_x32(taddr_row + static_cast<uint32_t>(c * 32), r);
    tmem_ld_wait_regs(r);
#pragma unroll
    for (int j = 0; j < 32; ++j) __stcg(dst + (static_cast<size_t>(c) * 32 + j) * kBlockM, r[j]);
  }
}
// Finisher: the partial sums that workers first..last left in their slots (`src` = slot 0 + this
// thread's row; slots `slot_stride` words apart) are added into the accumulator in TMEM, in worker
// order; the ordinary epilogue then runs on the completed sums.
template <int KIND, int COLS>
__device__ __noinline__ void sk_add_partials(uint32_t taddr_row, const uint32_t* src, int first,
                                             int last, size_t slot_stride) {
  uint32_t r[32];
#pragma unroll 1
  for (int c = 0; c < COLS / 32; ++c) {
    tmem_ld_32x32b_x32(taddr_row + static_cast<uint32_t>(c * 32), r);
    tmem_ld_wait_regs(r);
    for (int cw = first; cw <= last; ++cw) {
      const uint32_t* s = src + static_cast<size_t>(cw) * slot_stride +
                          (static_cast<size_t>(c) * 32) * kBlockM;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const uint32_t v = __ldcg(s + j * kBlockM);
        if constexpr (KIND == 1) {
          r[j] += v;  // int32 sums: exact in any order
        } else {
          r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(v));
        }
      }
    }
    tmem_st_32x32b_x32(taddr_row + static_cast<uint32_t>(c * 32), r);
  }
  tmem_st_wait();
}

// Output staging of the TMA-store epilogue: per epilogue warp kEpiBufs buffers of 32 rows x 128
// bytes, used in rotation; a buffer is rewritten once the store issued kEpiBufs stores ago has
// read it.
#ifndef AMOSB_EPI_BUFS
#define AMOSB_EPI_BUFS 2
#endif
constexpr int kEpiBufs = AMOSB_EPI_BUFS;
constexpr int kEpiBufBytes = 32 * 128;
constexpr int kEpiBytesPerWarp = kEpiBufs * kEpiBufBytes;
constexpr int kEpiBytes = 4 * kEpiBytesPerWarp;

// MT = accumulator tiles of 128 rows per CTA tile.  MT = 2 ("tall" tiles, 256 x BN) lets two MMAs
// share every B stage: for outputs no wider than 128 columns this halves the B bytes pulled from
// L2 per flop, which is what bounds the 128-wide tile.
template <int BN, bool EPI_TMA = false, int MT = 1>
struct UmmaConfig {
  static_assert(MT == 1 || (MT == 2 && BN <= 128), "tall tiles need 2 * MT * BN <= 512 TMEM columns");
  static constexpr int kBTileBytes = BN * 128;
  static constexpr int kStageBytes = MT * kATileBytes + kBTileBytes;
#ifdef AMOSB_EXP_STAGES
  static constexpr int kStages = AMOSB_EXP_STAGES;
#else
  static constexpr int kStages = MT == 2 ? 4 : ((BN == 256) ? 4 : (BN == 128 ? 6 : 8));
#endif
  static constexpr int kAccCols = MT * BN;  // TMEM columns of one accumulator buffer
  static constexpr int kTmemCols = (2 * kAccCols < 32) ? 32 : 2 * kAccCols;  // power of two
  static constexpr int kBarrierBytes = 256;
  static constexpr int kEpiRegion = EPI_TMA ? kEpiBytes : 0;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiRegion + kBarrierBytes + 1024;
};


__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}
__device__ __forceinline__ void st_shared_v2(uint32_t addr, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
// 8-byte read of data that is used once: no L1 allocation (the L1 beside ~200 KB of stages is
// small, and lines allocated for in-flight loads would cap how many can be outstanding).
__device__ __forceinline__ uint2 ldg_stream_v2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];"
               : "=r"(v.x), "=r"(v.y)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t pack_half2(uint32_t lo_f32_bits, uint32_t hi_f32_bits) {
  __half2 h = __floats2half2_rn(__uint_as_float(lo_f32_bits), __uint_as_float(hi_f32_bits));
  return *reinterpret_cast<uint32_t*>(&h);
}

template <typename OutT>
__device__ __forceinline__ OutT convert_acc(uint32_t bits);
template <>
__device__ __forceinline__ float convert_acc<float>(uint32_t bits) {
  return __uint_as_float(bits);
}
template <>
__device__ __forceinline__ __half convert_acc<__half>(uint32_t bits) {
  return __float2half_rn(__uint_as_float(bits));
}
template <>
__device__ __forceinline__ int32_t convert_acc<int32_t>(uint32_t bits) {
  return static_cast<int32_t>(bits);
}

// Fused trailing stages on the 32 accumulator columns a thread holds (raw 32-bit patterns of f32
// or s32).  `full_ptr` points at the addend element of (this row, column col0) for a full-shape
// addend, consecutive columns `full_stride` elements apart; unused for the vector form.
template <int KIND>
__device__ __forceinline__ void apply_trailing_ops(uint32_t (&r)[32], const UmmaParams& p,
                                                   int col0, int ncols_valid, bool row_valid,
                                                   const void* full_ptr, long long full_stride) {
  if (p.epi_flags == 0) return;
  if (p.epi_flags & kEpiAddRowVec) {
    // one addend per row (1x1 convolutions run as GEMMs whose rows are the output channels)
    if (row_valid) {
      if constexpr (KIND != 1) {
        const float add = p.addend_f16 ? __half2float(__ldg(static_cast<const __half*>(full_ptr)))
                                       : __ldg(static_cast<const float*>(full_ptr));
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + add);
      } else {
        const int add = __ldg(static_cast<const int*>(full_ptr));
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = static_cast<uint32_t>(static_cast<int>(r[j]) + add);
      }
    }
  }
  if (p.epi_flags & (kEpiAddVec | kEpiAddFull)) {
    const bool vec = (p.epi_flags & kEpiAddVec) != 0;
    if (vec || row_valid) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < ncols_valid) {
          if constexpr (KIND != 1) {
            float add;
            if (vec) {
              add = p.addend_f16 ? __half2float(__ldg(static_cast<const __half*>(p.addend) + col0 + j))
                                 : __ldg(static_cast<const float*>(p.addend) + col0 + j);
            } else {
              add = p.addend_f16
                        ? __half2float(__ldg(static_cast<const __half*>(full_ptr) + j * full_stride))
                        : __ldg(static_cast<const float*>(full_ptr) + j * full_stride);
            }
            r[j] = __float_as_uint(__uint_as_float(r[j]) + add);
          } else {
            const int add = vec ? __ldg(static_cast<const int*>(p.addend) + col0 + j)
                                : __ldg(static_cast<const int*>(full_ptr) + j * full_stride);
            r[j] = static_cast<uint32_t>(static_cast<int>(r[j]) + add);
          }
        }
      }
    }
  }
  if (p.epi_flags & kEpiRelu) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if constexpr (KIND != 1) {
        r[j] = __float_as_uint(fmaxf(__uint_as_float(r[j]), 0.f));
      } else {
        r[j] = static_cast<uint32_t>(max(static_cast<int>(r[j]), 0));
      }
    }
  }
}

// Row-major store of 32 consecutive columns held by one thread.
template <typename OutT>
__device__ __forceinline__ void store_row_chunk(OutT* __restrict__ dst, const uint32_t (&r)[32],
                                                int ncols_valid) {
  constexpr int kPerVec = 16 / sizeof(OutT);
  const bool aligned = (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
  if (ncols_valid >= 32 && aligned) {
#pragma unroll
    for (int v = 0; v < 32 / kPerVec; ++v) {
      if constexpr (sizeof(OutT) == 4) {
        // f32 and s32 accumulators are stored as their raw 32-bit patterns.
        const uint4 pk = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
        *reinterpret_cast<uint4*>(dst + v * 4) = pk;
      } else {
        __half2 h0 = __floats2half2_rn(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
        __half2 h1 = __floats2half2_rn(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
        __half2 h2 = __floats2half2_rn(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
        __half2 h3 = __floats2half2_rn(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
        uint4 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&h0);
        pk.y = *reinterpret_cast<uint32_t*>(&h1);
        pk.z = *reinterpret_cast<uint32_t*>(&h2);
        pk.w = *reinterpret_cast<uint32_t*>(&h3);
        *reinterpret_cast<uint4*>(dst + v * 8) = pk;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < ncols_valid) dst[j] = convert_acc<OutT>(r[j]);
    }
  }
}

// NCHW store of a 32-column chunk when every image plane is a whole number of 4-pixel groups.
// A thread holds one pixel (row) of 32 channels; groups of 4 lanes transpose 4 x 4 blocks among
// themselves with shuffles, after which a lane holds 4 consecutive pixels of one channel and stores
// them as one 16-byte (float32, int32) or 8-byte (float16) unit: a quarter of the store instructions
// of the element-wise form, each of which the memory pipe takes as long to accept.
// `quad_dst` points at the lane's own channel (chunk column lane & 3) and the first pixel of the
// lane's 4-row group; `plane` is the distance between channel planes in elements.  All 32 lanes
// must call; lanes whose group lies past the last row pass quad_ok = false.
template <typename OutT>
__device__ __forceinline__ void store_nchw_quads(OutT* __restrict__ quad_dst, long long plane,
                                                 const uint32_t (&r)[32], int ncols_valid,
                                                 uint32_t lane, bool quad_ok) {
  const bool hi2 = (lane & 2u) != 0, hi1 = (lane & 1u) != 0;
  const int my_col = static_cast<int>(lane & 3u);
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    const uint32_t a0 = r[4 * b], a1 = r[4 * b + 1], a2 = r[4 * b + 2], a3 = r[4 * b + 3];
    // 2 x 2 blocks change places between lanes i and i ^ 2 ...
    const uint32_t t0 = __shfl_xor_sync(0xffffffffu, hi2 ? a0 : a2, 2);
    const uint32_t t1 = __shfl_xor_sync(0xffffffffu, hi2 ? a1 : a3, 2);
    const uint32_t b0 = hi2 ? t0 : a0, b1 = hi2 ? t1 : a1, b2 = hi2 ? a2 : t0, b3 = hi2 ? a3 : t1;
    // ... then single elements between lanes i and i ^ 1
    const uint32_t v0 = __shfl_xor_sync(0xffffffffu, hi1 ? b0 : b1, 1);
    const uint32_t v1 = __shfl_xor_sync(0xffffffffu, hi1 ? b2 : b3, 1);
    const uint32_t c0 = hi1 ? v0 : b0, c1 = hi1 ? b1 : v0, c2 = hi1 ? v1 : b2, c3 = hi1 ? b3 : v1;
    if (quad_ok && 4 * b + my_col < ncols_valid) {
      OutT* dst = quad_dst + static_cast<long long>(4 * b) * plane;
      if constexpr (sizeof(OutT) == 4) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(c0, c1, c2, c3);
      } else {
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_half2(c0, c1), pack_half2(c2, c3));
      }
    }
  }
}

// ---- pieces of the epilogue shared by the single-CTA and the CTA-pair kernel -------------------
// The accumulator leaves TMEM in chunks of 32 columns.  Loads are double-buffered: the load of
// chunk c+1 is in flight while chunk c is converted and stored, so the TMEM read latency is paid
// once per tile instead of once per chunk.  `process(registers, c)` is called for c = 0..nch-1.
template <class F>
__device__ __forceinline__ void for_each_chunk(uint32_t taddr_row, int nch, F&& process) {
  uint32_t ra[32], rb[32];
  if (nch > 0) tmem_ld_32x32b_x32(taddr_row, ra);
#pragma unroll 1
  for (int c = 0; c < nch; c += 2) {
    tmem_ld_wait_regs(ra);
    if (c + 1 < nch) tmem_ld_32x32b_x32(taddr_row + static_cast<uint32_t>((c + 1) * 32), rb);
    process(ra, c);
    if (c + 1 < nch) {
      tmem_ld_wait_regs(rb);
      if (c + 2 < nch) tmem_ld_32x32b_x32(taddr_row + static_cast<uint32_t>((c + 2) * 32), ra);
      process(rb, c + 1);
    }
  }
}

// Element `off` of the fused addend (float32 or float16 in memory).
__device__ __forceinline__ const void* addend_ptr(const UmmaParams& p, long long off) {
  return p.addend_f16 ? static_cast<const void*>(static_cast<const __half*>(p.addend) + off)
                      : static_cast<const void*>(static_cast<const float*>(p.addend) + off);
}

// 32 columns of one output row into the row's 128 bytes of a 128B-swizzled staging buffer
// (`swz` = (row & 7) << 4).  32-bit outputs fill the row; 16-bit outputs fill half `h` of it.
template <typename OutT>
__device__ __forceinline__ void stage_chunk(uint32_t row_addr, uint32_t swz, int h,
                                            const uint32_t (&r)[32]) {
  if constexpr (sizeof(OutT) == 4) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      st_shared_v4(row_addr + ((static_cast<uint32_t>(j) << 4) ^ swz), r[4 * j], r[4 * j + 1],
                   r[4 * j + 2], r[4 * j + 3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      st_shared_v4(row_addr + ((static_cast<uint32_t>(h * 4 + j) << 4) ^ swz),
                   pack_half2(r[8 * j], r[8 * j + 1]), pack_half2(r[8 * j + 2], r[8 * j + 3]),
                   pack_half2(r[8 * j + 4], r[8 * j + 5]), pack_half2(r[8 * j + 6], r[8 * j + 7]));
    }
  }
}

// A_MN_MAJOR: A is given as [K][M] (the `te` text indexes it A[k, i]) and consumed in place as an
// MN-major operand, in chunks of 128 bytes of M like an MN-major B.  GEMM mode, MT = 1 only.
template <int KIND, int BN, bool B_MN_MAJOR, int MODE, typename OutT, bool EPI_TMA, int MT = 1,
          bool A_MN_MAJOR = false>
__global__ void __launch_bounds__(umma_threads(MODE), 1)
umma_persistent_kernel(const __grid_constant__ CUtensorMap tmA,
                       const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmC, const UmmaParams p) {
  using Cfg = UmmaConfig<BN, EPI_TMA, MT>;
  constexpr int kTileRows = kBlockM * MT;  // output rows of one CTA tile
  static_assert(!EPI_TMA || (MODE != kModeConv && MODE != kModeConvPw),
                "the TMA-store epilogue writes row-major C");
  constexpr bool kNchwOut = MODE == kModeConv || MODE == kModeConvPw;  // output stored as NCHW
  constexpr int kStages = Cfg::kStages;
  constexpr int kElemsPer128B = (KIND == 0) ? 64 : (KIND == 1) ? 128 : 32;  // K elements per stage; also MN chunk
  constexpr int kUmmaKRows = (KIND == 0) ? 16 : (KIND == 1) ? 32 : 8;       // K per MMA instruction
  constexpr int kMmaPerStage = 4;                        // 128 B / 32 B
  constexpr uint32_t kBChunkBytes = kElemsPer128B * 128;  // MN-major: one 128B-wide column chunk
  constexpr int kBChunks = BN / kElemsPer128B;            // MN-major chunks per stage
  static_assert(!B_MN_MAJOR || (BN % kElemsPer128B == 0), "BN must cover whole 128B chunks");
  static_assert(MODE != kModeConv || !B_MN_MAJOR, "NCHW conv consumes a K-major prepacked filter");
  static_assert(MODE != kModeConvNhwc || B_MN_MAJOR, "NHWC conv reads the RSCK filter MN-major");
  static_assert(MODE != kModeConvHwnc || B_MN_MAJOR, "HWNC conv reads the RSCK filter MN-major");
  static_assert(!A_MN_MAJOR || ((MODE == kModeGemm || MODE == kModeConvPw) && MT == 1),
                "MN-major A: 128-row tiles of the GEMM and of the in-place 1x1 convolution");
  static_assert(MODE != kModeConvPw || (A_MN_MAJOR && !B_MN_MAJOR && KIND == 0),
                "in-place 1x1 NCHW: 16-bit activation as MN-major A, KCRS filter as K-major B");
  constexpr int kAChunks = kBlockM / kElemsPer128B;  // MN-major A: 128-byte chunks of M per stage

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128B swizzle atom (8 rows x 128 B).
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t epi_base = smem_base + kStages * Cfg::kStageBytes;  // 1024-byte aligned
  uint8_t* bar_region = smem_aligned + kStages * Cfg::kStageBytes + Cfg::kEpiRegion;
  const uint32_t bar_base = epi_base + Cfg::kEpiRegion;
  // barrier layout (8 B each): full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
  auto tmem_empty_bar = [&](int s) { return bar_base + 8u * (2 * kStages + 2 + s); };
  volatile uint32_t* tmem_base_slot =
      reinterpret_cast<volatile uint32_t*>(bar_region + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_region + 8 * (2 * kStages + 4) + 8);

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();

  // ------------------------------------------------------------------ set-up
  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    if constexpr (EPI_TMA) prefetch_tensormap(&tmC);
    for (int s = 0; s < kStages; ++s) {
      // one arrival of the TMA-issuing thread (with the bytes it expects), plus one per copying
      // thread where the activation is brought in by cp.async
      mbar_init(full_bar(s), MODE == kModeConvPw ? 1 + 32 * kPwCopyWarps : 1);
      mbar_init(empty_bar(s), MT);  // one commit per MMA-issuing thread
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tmem_full_bar(s), MT);
      mbar_init(tmem_empty_bar(s), 4);  // one arrive per epilogue warp
    }
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_base_slot)), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  const int tiles_per_batch = p.tiles_m * p.tiles_n;

  // tile index -> (batch, m block, n block); grouped raster so that CTAs running at the same time
  // share operand rows/columns in L2.
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

  // Issuing one tcgen05.mma, TMA load or commit costs its thread ~50-90 cycles, so one thread
  // feeds the tensor pipe only as long as a k-block holds >= ~400 cycles of math (256-wide tiles).
  // Tall tiles therefore give each of their two accumulators its own issuing thread (warps 1 and
  // 7; the accumulators are independent, so no ordering between the two is needed) and keep two
  // TMA-issuing threads (warps 0 and 6).
  constexpr bool kSecondIssuer = MT == 2;
  const bool is_producer_warp = warp == 0 || warp == 6 || (warp == 7 && !kSecondIssuer);
  const bool is_mma_warp = warp == 1 || (warp == 7 && kSecondIssuer);
  if (MODE == kModeConvPw && warp >= 8) {
    // ================================================================ activation copier (1x1 NCHW)
    // A stage's A tile is 64 channels (k-rows) x 128 pixels, stored as the copy engine stores an
    // MN-major tile: two chunks of 64 pixels, each 64 rows of 128 bytes, the 16-byte units of a
    // row XOR-ed with the row number (128-byte swizzle).  Lane g of a warp owns the four pixels
    // 4g..4g+3 of the tile (8 bytes); a warp instruction therefore moves one whole channel row of
    // the tile, 256 contiguous bytes of global memory.  Warp w of the four moves channels
    // 16w..16w+15 of every k-block.  P*Q is a multiple of 4, so a pixel quad never straddles two
    // images and is 8-byte aligned.
    // One cp.async moves a lane's 8 bytes straight into the stage, and the stage's barrier is told
    // to count this thread's arrival once the copies it has issued so far have landed
    // (cp.async.mbarrier.arrive.noinc): nothing in this loop waits for data, so a CTA has all the
    // stages but the one being multiplied in flight.  (Waiting in line for an earlier group before
    // issuing the next one kept only two groups in flight and ran at half the rate: the loop's
    // period was half the memory latency.)
    if constexpr (MODE == kModeConvPw) {
      grid_dependency_wait();
      const int cwp = warp - 8;
      const uint32_t g = lane;
      const uint32_t dst_lane = (g >> 4) * kBChunkBytes + (g & 1u) * 8u;
      const uint32_t unit = (g & 15u) >> 1;
      const uint8_t* const act = static_cast<const uint8_t*>(p.act);
      const long long plane_bytes = static_cast<long long>(p.PQ) * 2;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = !p.diag_no_loads;
      SegmentIter it(p, blockIdx.x, gridDim.x);
      Segment sg;
      while (ok && it.next(p, sg)) {
        int b, m_blk, n_blk;
        decode_tile(sg.tile, b, m_blk, n_blk);
        const int m = m_blk * kBlockM + 4 * static_cast<int>(g);
        const bool row_ok = m < p.M;
        const int img = row_ok ? m / p.PQ : 0;
        const int pq = row_ok ? m - img * p.PQ : 0;
        const uint8_t* src_lane =
            act + (static_cast<long long>(img) * p.conv_C * p.PQ + pq) * 2;
        for (int kb = sg.kb_begin; kb < sg.kb_end; ++kb) {
          bool got = true;
          if (lane == 0)
            got = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status,
                            kStatusTimeoutProducer, p.wait_budget_ns);
          got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
          if (!got) {
            ok = false;
            break;
          }
          const uint32_t sA = smem_base + stage * Cfg::kStageBytes;
          const int c0 = cwp * 16;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int c = c0 + i;                        // k-row inside the stage
            const int chan = kb * kElemsPer128B + c;     // channel of the layer
            const bool live = row_ok && chan < p.conv_C;
            const uint8_t* src = live ? src_lane + chan * plane_bytes : act;
            const uint32_t dst = sA + dst_lane + static_cast<uint32_t>(c) * 128u +
                                 ((unit ^ (static_cast<uint32_t>(c) & 7u)) << 4);
            cp_async_8(dst, src, live ? 8u : 0u);
          }
          cp_async_arrive_noinc(full_bar(stage));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // nothing may be in flight when the CTA's shared memory is given up
      cp_async_wait_all();
    }
  } else if (is_producer_warp) {
    // ================================================================ TMA producer
    // Up to three issuing threads (lane 0 of warps 0, 6, 7).  The CTA's k-blocks form one stream
    // across its tiles; thread pi owns k-blocks pi, pi + P, pi + 2P, ... of that stream and arms
    // and fills their stages.  A lone thread runs dependent scalar code at a few cycles per
    // instruction and an integer division costs it over a hundred, so the loop below only adds
    // and compares: positions (stage, filter tap, channel chunk) advance by P steps at a time.
    const int pi = warp == 0 ? 0 : warp - 5;
    // stage = pi + j * P below needs P <= kStages
    const int P = MODE == kModeConvPw ? 1 : min(min(p.producers, kSecondIssuer ? 2 : 3), kStages);
    if (lane == 0 && pi < P && !p.diag_no_loads) {
      // the kernel may have been started while its predecessor in the stream was still running
      // (for the NCHW conv that is the re-layout kernel that writes both operands): nothing is
      // read from global memory before that kernel has completed
      grid_dependency_wait();
      int stage = pi;
      uint32_t phase = 0;
      bool ok = true;
      int kb = pi;  // this thread's next k-block inside the current tile
#ifdef AMOSB_ROLE_CYCLES
      long long rc_wait = 0;
      const long long rc_begin = clock64();
#endif
      SegmentIter it(p, blockIdx.x, gridDim.x);
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
        int cw[MT], ch[MT], cn[MT];  // im2col start of each 128-row sub-tile
        int cc = 0, fs = 0, fr = 0;  // channel chunk and filter tap of k-block kb
        if constexpr (MODE != kModeGemm && MODE != kModeConvPw) {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const int m0 = m_blk * kTileRows + mt * kBlockM;
            int pq, op, oq;
            if constexpr (MODE == kModeConvHwnc) {
              if (p.hw_group > 1) {
                const int t = m0 / kBlockM;  // this sub-tile among the pixel groups
                op = t / p.hw_qgroups;
                oq = (t - op * p.hw_qgroups) * p.hw_group;  // first pixel of the group
                cn[mt] = 0;
              } else {
                pq = m0 / p.conv_N;            // output pixel of this sub-tile
                cn[mt] = m0 - pq * p.conv_N;   // its first image
                op = pq / p.Q;
                oq = pq - op * p.Q;
              }
            } else {
              cn[mt] = m0 / p.PQ;
              pq = m0 - cn[mt] * p.PQ;
              op = pq / p.Q;
              oq = pq - op * p.Q;
            }
            cw[mt] = oq * p.stride_w - p.pad_w;
            ch[mt] = op * p.stride_h - p.pad_h;
          }
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
          const uint32_t sB = sA + MT * kATileBytes;
          const uint32_t fb = full_bar(stage);
#ifdef AMOSB_ROLE_CYCLES
          const bool dbg_no_a = (p.dbg_skip & 1) != 0, dbg_no_b = (p.dbg_skip & 2) != 0;
          mbar_arrive_expect_tx(fb, ((dbg_no_a || MODE == kModeConvPw) ? 0 : MT * kATileBytes) +
                                        (dbg_no_b ? 0 : Cfg::kBTileBytes));
#define AMOSB_DBG_A if (!dbg_no_a)
#define AMOSB_DBG_B if (!dbg_no_b)
#else
          mbar_arrive_expect_tx(fb, MODE == kModeConvPw ? Cfg::kBTileBytes : Cfg::kStageBytes);
#define AMOSB_DBG_A
#define AMOSB_DBG_B
#endif
          if constexpr (MODE == kModeConvPw) {
            // the filter [K_out][C] is the K-major B operand; channels past C load as zeros
            AMOSB_DBG_B tma_load_2d(sB, &tmB, fb, kabs * kElemsPer128B, n_blk * BN);
          } else if constexpr (MODE == kModeGemm) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              // rows past M are zero-filled by the load and still counted in the stage's bytes
              if constexpr (A_MN_MAJOR) {
#pragma unroll
                for (int j = 0; j < kAChunks; ++j) {
                  AMOSB_DBG_A tma_load_3d(sA + j * kBChunkBytes, &tmA, fb,
                                          m_blk * kBlockM + j * kElemsPer128B, kabs * kElemsPer128B,
                                          p.a_bcast ? 0 : b);
                }
              } else {
                AMOSB_DBG_A tma_load_3d(sA + mt * kATileBytes, &tmA, fb, kabs * kElemsPer128B,
                                        m_blk * kTileRows + mt * kBlockM, p.a_bcast ? 0 : b);
              }
            }
            if constexpr (B_MN_MAJOR) {
#pragma unroll
              for (int j = 0; j < kBChunks; ++j) {
                AMOSB_DBG_B tma_load_3d(sB + j * kBChunkBytes, &tmB, fb, n_blk * BN + j * kElemsPer128B,
                            kabs * kElemsPer128B, b);
              }
            } else {
              AMOSB_DBG_B tma_load_3d(sB, &tmB, fb, kabs * kElemsPer128B, n_blk * BN, b);
            }
          } else {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              if constexpr (MODE == kModeConvHwnc) {
                // {channels, images, w, h}: padding pixels and rows past the last output pixel are
                // out-of-range w / h coordinates -> zeros, counted in the stage's bytes
                AMOSB_DBG_A tma_load_4d(sA + mt * kATileBytes, &tmA, fb, cc * kElemsPer128B, cn[mt],
                                        cw[mt] + fs * p.dil_w, ch[mt] + fr * p.dil_h);
              } else {
                // pixels past the last image are zero-filled and counted like any other
                AMOSB_DBG_A tma_load_im2col_4d(sA + mt * kATileBytes, &tmA, fb, cc * kElemsPer128B, cw[mt],
                                               ch[mt], cn[mt], static_cast<uint16_t>(fs * p.dil_w),
                                               static_cast<uint16_t>(fr * p.dil_h));
              }
            }
            if constexpr (MODE == kModeConv) {
              AMOSB_DBG_B tma_load_2d(sB, &tmB, fb, kabs * kElemsPer128B, n_blk * BN);
            } else {
              // RSCK filter as [R*S*C][K]: rows of tap rs start at rs*C; channels past C multiply
              // activation columns that the im2col load zero-fills
              const int brow = (fr * p.S + fs) * p.conv_C + cc * kElemsPer128B;
#pragma unroll
              for (int j = 0; j < kBChunks; ++j) {
                AMOSB_DBG_B tma_load_3d(sB + j * kBChunkBytes, &tmB, fb, n_blk * BN + j * kElemsPer128B, brow,
                            0);
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
#undef AMOSB_DBG_A
#undef AMOSB_DBG_B
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
        atomicAdd(&p.role_cycles[0], (unsigned long long)rc_wait);
        atomicAdd(&p.role_cycles[1], (unsigned long long)(clock64() - rc_begin));
      }
#endif
    }
  } else if (is_mma_warp) {
    // ================================================================ MMA issuer(s)
    // accumulator tiles [mt_lo, mt_hi) of every CTA tile are this thread's
    const int mt_lo = (kSecondIssuer && warp == 7) ? 1 : 0;
    const int mt_hi = kSecondIssuer ? mt_lo + 1 : MT;
    if (lane == 0) {
      const uint32_t idesc = make_idesc<KIND>(kBlockM, BN, B_MN_MAJOR, A_MN_MAJOR) | p.idesc_formats;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
#ifdef AMOSB_ROLE_CYCLES
      long long rc_full = 0, rc_tmem = 0;
      const long long rc_begin = clock64();
#endif
      SegmentIter it(p, blockIdx.x, gridDim.x);
      Segment sg;
      while (ok && it.next(p, sg)) {
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
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * Cfg::kAccCols);
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
          // cp.async wrote the activation through the generic proxy; the MMA reads it through
          // the asynchronous one
          if constexpr (MODE == kModeConvPw) fence_proxy_async_smem();
          tc_fence_after_sync();
          const uint32_t sA = smem_base + stage * Cfg::kStageBytes;
          const uint32_t sB = sA + MT * kATileBytes;
          // K-major operands step 32 bytes inside the swizzle span per MMA; an MN-major B steps
          // whole k-rows (kUmmaKRows rows of 128 bytes).
          constexpr int kAStep = A_MN_MAJOR ? (kUmmaKRows * 128) >> 4 : 32 >> 4;
          constexpr int kBStep = B_MN_MAJOR ? (kUmmaKRows * 128) >> 4 : 32 >> 4;
          // MN-major operands of 32-bit elements lie in the 128-byte swizzle with 32-byte units
          // (groups of 4 k-rows, 512 bytes apart); all others in the plain 128-byte swizzle
          constexpr uint32_t kHiMn =
              KIND == 2 ? smem_desc_hi_sw128_base32(512) : smem_desc_hi_sw128(1024);
          const uint32_t b_lo = smem_desc_lo(sB, B_MN_MAJOR ? kBChunkBytes : 16);
          for (int mt = mt_lo; mt < mt_hi; ++mt) {
            umma_kblock4<KIND, false, kAStep, kBStep>(
                tmem_d + static_cast<uint32_t>(mt * BN),
                smem_desc_lo(sA + mt * kATileBytes, A_MN_MAJOR ? kBChunkBytes : 16), b_lo,
                A_MN_MAJOR ? kHiMn : smem_desc_hi_sw128(1024),
                B_MN_MAJOR ? kHiMn : smem_desc_hi_sw128(1024), idesc,
                kb != sg.kb_begin ? 1u : 0u);  // the segment's first MMA overwrites
          }
          umma_commit(empty_bar(stage));  // smem slot reusable once these MMAs have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(tmem_full_bar(acc));  // accumulator complete
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
#ifdef AMOSB_ROLE_CYCLES
      if (warp == 1) {
        atomicAdd(&p.role_cycles[2], (unsigned long long)rc_full);
        atomicAdd(&p.role_cycles[3], (unsigned long long)rc_tmem);
        atomicAdd(&p.role_cycles[4], (unsigned long long)(clock64() - rc_begin));
        atomicAdd(&p.role_cycles[7], 1ull);
      }
#endif
    }
  } else {
    // ================================================================ epilogue (warps 2..5)
    // The next kernel in the stream, if it was launched as a programmatic dependent, may take this
    // CTA's SM as soon as the CTA exits and set itself up while the rest of this grid finishes.
    // Issued from an epilogue thread, which has nothing to do yet: the instruction holds its thread
    // for about a microsecond, which the threads that start the pipeline cannot spare.
    if (warp == 2 && lane == 0) grid_launch_dependents();
    // addend reads and output stores, too, come after the predecessor kernel has completed
    grid_dependency_wait();
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    int epi_buf = 0;
    OutT* const out = reinterpret_cast<OutT*>(p.out);
#ifdef AMOSB_ROLE_CYCLES
    long long rc_wait = 0;
    const long long rc_begin = clock64();
#endif
    constexpr size_t kPartialElems = static_cast<size_t>(MT) * kBlockM * BN;  // per CTA slot
    const int worker = blockIdx.x;
    SegmentIter it(p, worker, gridDim.x);
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
      // Part of a shared-out tile?  A segment that does not start at the tile's first k-block
      // leaves its sums for the CTA that holds the first k-block; that CTA, if its segment stops
      // short of the last k-block, adds the sums of the workers after it (their shares follow
      // its own without a gap) before the usual epilogue.
      const bool sk_contrib = sg.kb_begin > 0;
      int fix_first = 0, fix_last = -1;
      if (!sk_contrib && sg.kb_end < p.num_kb) {
        fix_first = worker + 1;
        fix_last = sk_worker_of(
            p, static_cast<long long>(sg.tile - p.sk_first) * p.num_kb + p.num_kb - 1);
        bool got = true;
        if (lane == 0) {
          for (int cw = fix_first; got && cw <= fix_last; ++cw)
            got = gflag_wait(p.sk_flags + cw * 4 + quarter, abort_flag, p.status,
                             2 * p.wait_budget_ns);
        }
        if (__shfl_sync(0xffffffffu, got ? 1 : 0, 0) == 0) {
          ok = false;
          break;
        }
      }
      if (sk_contrib || fix_last >= fix_first) {
        const uint32_t taddr_q = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                 static_cast<uint32_t>(acc * Cfg::kAccCols);
        const size_t part_lane = static_cast<size_t>(quarter * 32) + lane;
        if (sk_contrib) {
          sk_dump_partials<Cfg::kAccCols>(
              taddr_q, p.sk_partials + static_cast<size_t>(worker) * kPartialElems + part_lane);
          __threadfence();  // the partial sums are in L2 before the flag says so
          __syncwarp();
          if (lane == 0) {
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.sk_flags + worker * 4 + quarter),
                         "r"(1u)
                         : "memory");
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(tmem_empty_bar(acc));
          if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1u;
          }
          continue;
        }
        sk_add_partials<KIND, Cfg::kAccCols>(taddr_q, p.sk_partials + part_lane, fix_first, fix_last,
                                             kPartialElems);
        __syncwarp();  // every lane has read its partial sums: the flags can be reused
        if (lane == 0) {
          for (int cw = fix_first; cw <= fix_last; ++cw) p.sk_flags[cw * 4 + quarter] = 0u;
        }
      }
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {  // the 128-row accumulator tiles of this CTA tile
      const int row = m_blk * kTileRows + mt * kBlockM + quarter * 32 + static_cast<int>(lane);
      // row of the output matrix this thread holds, and whether it exists: in HWNC mode a GEMM row
      // is (pixel, image) with the images padded to a multiple of 128 per pixel
      int orow = row;
      bool row_ok = row < p.M;
      int st_row = m_blk * kTileRows + mt * kBlockM + quarter * 32, st_batch = b;  // TMA-store box
      int st_q = 0;  // HWNC: the box starts at image st_row of output pixel (st_batch, st_q)
      if constexpr (MODE == kModeConvHwnc) {
        if (p.hw_group > 1) {
          const int t = st_row / kBlockM;  // pixel group of this 128-row accumulator tile
          const int op = t / p.hw_qgroups;
          const int q0 = (t - op * p.hw_qgroups) * p.hw_group;
          const int r = quarter * 32 + static_cast<int>(lane);
          const int g = r / p.hw_nbox, img = r - g * p.hw_nbox;
          orow = (op * p.Q + q0 + g) * p.conv_N_real + img;
          row_ok = row_ok && q0 + g < p.Q && img < p.conv_N_real;
          st_batch = op;
          st_q = q0 + (quarter * 32) / p.hw_nbox;
          st_row = (quarter * 32) % p.hw_nbox;
          if (st_q >= p.Q) st_row = p.conv_N_real;  // nothing of this warp exists (see below)
        } else {
          const int pix = row / p.conv_N;
          const int img = row - pix * p.conv_N;
          orow = pix * p.conv_N_real + img;
          row_ok = row_ok && img < p.conv_N_real;
          const int spix = st_row / p.conv_N;  // {K, images, Q, P} map: clipped at the last image
          st_row -= spix * p.conv_N;
          st_batch = spix / p.Q;
          st_q = spix - st_batch * p.Q;
        }
      }
      const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                 static_cast<uint32_t>(acc * Cfg::kAccCols + mt * BN);
      constexpr int kChunks = BN / 32;
      const int row0 = m_blk * kTileRows + mt * kBlockM + quarter * 32;  // first row of this warp
      auto run_chunks = [&](int nch, auto&& process) { for_each_chunk(taddr_row, nch, process); };
      // chunks that hold columns < N (warp-uniform); none when all of the warp's rows are >= M
      const int cols_left = p.N - n_blk * BN;
      int valid_chunks = row0 < p.M ? min(kChunks, (cols_left + 31) >> 5) : 0;
      if constexpr (MODE == kModeConvHwnc) {
        // all 32 rows of this warp are padding images, or pixels past the end of the output row
        if (st_row >= p.conv_N_real) valid_chunks = 0;
      }
      (void)st_q;
      if constexpr (EPI_TMA) {
        // registers -> 128B-swizzled staging rows -> one TMA store per 32 rows x 128 bytes.
        // The store engine clips rows >= M and columns >= N, and writes whole lines.
        constexpr int kColsPerStore = 128 / static_cast<int>(sizeof(OutT));
        constexpr int kLoadsPerStore = kColsPerStore / 32;
        const uint32_t my_epi = epi_base + static_cast<uint32_t>((warp - 2) * kEpiBytesPerWarp);
        const uint32_t swz = (lane & 7u) << 4;
        // whole stores only: a chunk past N inside the last store is clipped by the store engine
        const int nch = (valid_chunks + kLoadsPerStore - 1) / kLoadsPerStore * kLoadsPerStore;
        run_chunks(nch, [&](uint32_t(&r)[32], int c) {
          const int st = c / kLoadsPerStore;
          const int h = c - st * kLoadsPerStore;
          const int col0 = n_blk * BN + st * kColsPerStore;
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
                tma_store_3d(&tmC, buf, col0, st_row, st_batch);
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
        if constexpr (!kNchwOut) {
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
          const int col0 = n_blk * BN + c * 32;
          const int ncols_valid = p.N - col0;
          if (p.epi_flags != 0) {
            long long off, stride;
            if constexpr (!kNchwOut) {
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
          if constexpr (kNchwOut) {
            if (p.nchw_quads) {  // warp-uniform
              store_nchw_quads<OutT>(quad_ptr + static_cast<long long>(col0) * p.PQ, p.PQ, r,
                                     ncols_valid, lane, quad_ok);
              return;
            }
          }
          if (row_ok) {
            if constexpr (!kNchwOut) {
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
      }  // mt
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(acc));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if constexpr (EPI_TMA) {
      if (lane == 0) tma_store_wait_all<0>();  // all output stores of this warp have completed
    }
#ifdef AMOSB_ROLE_CYCLES
    if (warp == 2 && lane == 0) {
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
    // A wait was abandoned: give copies still in flight time to land before the CTA's shared
    // memory is handed to another CTA.
    for (int i = 0; i < 50; ++i) __nanosleep(20000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

}  // namespace amosb
