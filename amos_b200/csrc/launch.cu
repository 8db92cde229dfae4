// Host side of the device path: argument validation, tensor-map construction, tile choice and
// kernel launches behind the C ABI declared in include/amosb.h.
#include "../../include/amosb.h"
#include "host_common.h"
#include "umma_kernel.cuh"
#include "umma_pair_kernel.cuh"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <cstring>
#include <mutex>
#include <string>

namespace amosb {

// --------------------------------------------------------------------------------------------
// Driver entry points for tensor-map encoding, fetched through the runtime so that the library
// links against nothing but the (static) CUDA runtime and loads on machines without a driver.
// --------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                   cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

static EncodeTiledFn g_encode_tiled = nullptr;
static EncodeIm2colFn g_encode_im2col = nullptr;
static std::once_flag g_driver_once;
static int g_driver_rc = AMOSB_OK;

static int load_driver_entry_points() {
  std::call_once(g_driver_once, []() {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr) {
      g_driver_rc = AMOSB_ERR_CUDA;
      return;
    }
    g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    fn = nullptr;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr) {
      g_driver_rc = AMOSB_ERR_CUDA;
      return;
    }
    g_encode_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
  });
  if (g_driver_rc != AMOSB_OK) set_error("cannot resolve cuTensorMapEncode* from the CUDA driver");
  return g_driver_rc;
}

// --------------------------------------------------------------------------------------------
// Per-device state
// --------------------------------------------------------------------------------------------
__device__ int g_status_word = 0;
// Flags of the shared-out tail (one word per CTA and epilogue warp; see UmmaParams::sk_flags).
// They are zero when the library is loaded, and the kernels leave them zero (the CTA that reads a
// flag clears it).  A launch takes the next of kSkSlots blocks, so that kernels running side by
// side on different streams do not share a block unless 64 such launches are in flight at once.
constexpr int kSkSlots = 64;
constexpr int kSkCtasMax = 160;
__device__ unsigned int g_sk_flags[kSkSlots * kSkCtasMax * 4];
#ifdef AMOSB_ROLE_CYCLES
// Diagnostic build only (-DAMOSB_ROLE_CYCLES): cycles each role of the single-CTA kernel spent
// waiting and in total, summed over CTAs; read and cleared by amosb_debug_role_cycles().
__device__ unsigned long long g_role_cycles[16];
extern "C" int amosb_debug_role_cycles(unsigned long long* out16) {
  if (cudaMemcpyFromSymbol(out16, g_role_cycles, sizeof(unsigned long long) * 16) != cudaSuccess)
    return -3;
  unsigned long long zero[16] = {0};
  return cudaMemcpyToSymbol(g_role_cycles, zero, sizeof(zero)) == cudaSuccess ? 0 : -3;
}
#endif

struct DeviceState {
  bool init = false;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  int* status_ptr = nullptr;
  unsigned int* sk_flags = nullptr;
};
static std::atomic<unsigned int> g_sk_next[64];
static DeviceState g_dev[64];
static std::mutex g_dev_mutex;

static int get_device_state(int device, DeviceState** out) {
  if (device < 0 || device >= 64) {
    set_error("device id %d out of range", device);
    return AMOSB_ERR_ARG;
  }
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  DeviceState& st = g_dev[device];
  if (!st.init) {
    cudaDeviceProp prop;
    AMOSB_CUDA_CHECK(cudaGetDeviceProperties(&prop, device));
    st.sm_count = prop.multiProcessorCount;
    st.cc_major = prop.major;
    st.cc_minor = prop.minor;
    if (prop.major != 10) {
      set_error("device %d is sm_%d%d; this library only carries sm_100a code", device, prop.major,
                prop.minor);
      return AMOSB_ERR_UNSUPPORTED;
    }
    AMOSB_CUDA_CHECK(cudaSetDevice(device));
    void* p = nullptr;
    AMOSB_CUDA_CHECK(cudaGetSymbolAddress(&p, g_status_word));
    st.status_ptr = static_cast<int*>(p);
    p = nullptr;
    AMOSB_CUDA_CHECK(cudaGetSymbolAddress(&p, g_sk_flags));
    st.sk_flags = static_cast<unsigned int*>(p);
    st.init = true;
  }
  *out = &st;
  return AMOSB_OK;
}

// --------------------------------------------------------------------------------------------
// Tensor maps
// --------------------------------------------------------------------------------------------
static int encode_tiled_3d(CUtensorMap* tm, CUtensorMapDataType dt, int elem_bytes, void* base,
                           uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                           uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                           CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  (void)elem_bytes;
  CUresult r = g_encode_tiled(tm, dt, 3, base, dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled(3d) failed with %d (dims %llu,%llu,%llu strides %llu,%llu box "
              "%u,%u)",
              (int)r, (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2,
              (unsigned long long)stride1_bytes, (unsigned long long)stride2_bytes, b0, b1);
    return AMOSB_ERR_CUDA;
  }
  return AMOSB_OK;
}

// HWNC activation as {C, N, W, H}: boxes of 128 bytes of channels x 128 images of one input pixel.
// With fewer than 128 images a box is `nbox` images x `group` consecutive input pixels of a row.
static int encode_tiled_hwnc(CUtensorMap* tm, CUtensorMapDataType dt, uint64_t es, void* base,
                             uint64_t c, uint64_t n, uint64_t w, uint64_t h, uint32_t nbox = kBlockM,
                             uint32_t group = 1) {
  cuuint64_t dims[4] = {c, n, w, h};
  cuuint64_t strides[3] = {c * es, n * c * es, w * n * c * es};
  cuuint32_t box[4] = {(cuuint32_t)(128 / es), nbox, group, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = g_encode_tiled(tm, dt, 4, base, dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled(hwnc) failed with %d (C %llu N %llu W %llu H %llu)", (int)r,
              (unsigned long long)c, (unsigned long long)n, (unsigned long long)w,
              (unsigned long long)h);
    return AMOSB_ERR_CUDA;
  }
  return AMOSB_OK;
}

// HWNC output [P][Q][N][K] as {K, N, Q, P}: a store box is 128 bytes of K x 32 rows, the rows being
// `nbox` images x 32 / nbox consecutive pixels of an output row (32 images of one pixel when the
// image count is 32 or more).  Images past N and pixels past Q are dropped by the store engine.
static int encode_store_hwnc(CUtensorMap* tm, CUtensorMapDataType dt, uint64_t ob, void* base,
                             uint64_t k, uint64_t n, uint64_t q, uint64_t p, uint32_t nbox) {
  cuuint64_t dims[4] = {k, n, q, p};
  cuuint64_t strides[3] = {k * ob, n * k * ob, q * n * k * ob};
  const uint32_t imgs = nbox < 32 ? nbox : 32;
  cuuint32_t box[4] = {(cuuint32_t)(128 / ob), imgs, 32 / imgs, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = g_encode_tiled(tm, dt, 4, base, dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled(hwnc output) failed with %d (K %llu N %llu Q %llu P %llu)",
              (int)r, (unsigned long long)k, (unsigned long long)n, (unsigned long long)q,
              (unsigned long long)p);
    return AMOSB_ERR_CUDA;
  }
  return AMOSB_OK;
}

static int encode_tiled_2d(CUtensorMap* tm, CUtensorMapDataType dt, void* base, uint64_t d0,
                           uint64_t d1, uint64_t stride1_bytes, uint32_t b0, uint32_t b1) {
  cuuint64_t dims[2] = {d0, d1};
  cuuint64_t strides[1] = {stride1_bytes};
  cuuint32_t box[2] = {b0, b1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode_tiled(tm, dt, 2, base, dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled(2d) failed with %d", (int)r);
    return AMOSB_ERR_CUDA;
  }
  return AMOSB_OK;
}

// NHWC activation, im2col mode: one column = 128 output pixels x 128 bytes of channels.
static int encode_im2col_nhwc(CUtensorMap* tm, CUtensorMapDataType dt, void* base, int n, int h, int w, int c_pad,
                              int pad_h, int pad_w, int r, int s, int dil_h, int dil_w,
                              int stride_h, int stride_w, int pixels_per_column, int es = 2) {
  cuuint64_t dims[4] = {(cuuint64_t)c_pad, (cuuint64_t)w, (cuuint64_t)h, (cuuint64_t)n};
  cuuint64_t strides[3] = {(cuuint64_t)c_pad * es, (cuuint64_t)w * c_pad * es,
                           (cuuint64_t)h * w * c_pad * es};
  int lower[2] = {-pad_w, -pad_h};
  int upper[2] = {pad_w - (s - 1) * dil_w, pad_h - (r - 1) * dil_h};
  cuuint32_t estr[4] = {1, (cuuint32_t)stride_w, (cuuint32_t)stride_h, 1};
  CUresult res = g_encode_im2col(tm, dt, 4, base, dims, strides, lower,
                                 upper, (cuuint32_t)(128 / es), (cuuint32_t)pixels_per_column, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeIm2col failed with %d (N%d H%d W%d Cp%d lower %d,%d upper %d,%d)",
              (int)res, n, h, w, c_pad, lower[0], lower[1], upper[0], upper[1]);
    return AMOSB_ERR_CUDA;
  }
  return AMOSB_OK;
}

// --------------------------------------------------------------------------------------------
// Re-layout kernel of the conv path (one launch does both operands)
// --------------------------------------------------------------------------------------------
constexpr int kPackCT = 64;   // channels per activation block
constexpr int kPackPT = 64;   // pixels per activation block
constexpr int kPackLdW = 33;  // smem row pitch in 32-bit words (two pixels per word)
constexpr int kPackSmemHalves = kPackCT * kPackLdW * 2;

// Blocks [0, act_blocks): NCHW fp16 -> NHWC fp16, channels padded to `c_pad8` (zero filled).  A block
// transposes a 64 (channels) x 64 (pixels) tile of one image through shared memory.  Reads are
// contiguous along pixels, VEC elements per load (4 when the plane size is a multiple of 4, 2 when
// even, else 1); the tile is held as 32-bit words of two pixels; each thread then assembles, with
// byte permutes, the two 16-byte vectors (8 channels) of a pixel pair and writes them contiguous
// along channels.  Small tiles keep many blocks resident per SM, which hides the latency of the
// short rows of 7x7 / 14x14 planes.
// Blocks [act_blocks, ...): KCRS fp16 -> [K][R*S][c_pad64] fp16 (zero filled), the K-major B operand
// of the implicit GEMM with reduction index (r*S + s)*c_pad64 + c.  A block moves one filter's
// channel chunk: one contiguous read, then writes contiguous along channels for every tap.
template <int VEC>
__global__ void __launch_bounds__(256)
conv_prepack_kernel(const __half* __restrict__ act, __half* __restrict__ act_nhwc,
                    const __half* __restrict__ flt, __half* __restrict__ flt_krsc, int C, int HW,
                    int c_pad8, int act_blocks, int c_tiles, int p_tiles, int RS, int c_pad64,
                    int flt_chunk, int flt_chunks) {
  __shared__ __align__(16) uint32_t tile_w[kPackCT * kPackLdW];
  __half* tile = reinterpret_cast<__half*>(tile_w);
  const int tid = threadIdx.x;
  // the implicit-GEMM kernel may take SMs as this grid's last blocks drain
  if (threadIdx.x == 255) grid_launch_dependents();
  if (static_cast<int>(blockIdx.x) < act_blocks) {
    const int id = blockIdx.x;
    const int pt = id % p_tiles;
    const int ct = (id / p_tiles) % c_tiles;
    const int n = id / (p_tiles * c_tiles);
    const int p0 = pt * kPackPT;
    const int c0 = ct * kPackCT;
    const __half* s = act + (static_cast<long long>(n) * C) * HW;
    __half* d = act_nhwc + (static_cast<long long>(n) * HW) * c_pad8;
    if constexpr (VEC == 4) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = tid + 256 * i;
        const int cl = idx >> 4;
        const int px = (idx & 15) * 4;
        uint2 v = make_uint2(0u, 0u);
        if (c0 + cl < C && p0 + px < HW)
          v = *reinterpret_cast<const uint2*>(s + static_cast<long long>(c0 + cl) * HW + p0 + px);
        tile_w[cl * kPackLdW + (px >> 1)] = v.x;
        tile_w[cl * kPackLdW + (px >> 1) + 1] = v.y;
      }
    } else if constexpr (VEC == 2) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = tid + 256 * i;
        const int cl = idx >> 5;
        const int px = (idx & 31) * 2;
        uint32_t v = 0u;
        if (c0 + cl < C && p0 + px < HW)
          v = *reinterpret_cast<const uint32_t*>(s + static_cast<long long>(c0 + cl) * HW + p0 + px);
        tile_w[cl * kPackLdW + (px >> 1)] = v;
      }
    } else if constexpr (VEC == 0) {
      // whole plane fits one tile (HW <= 64) and C is a multiple of 8: the 64 channel planes of
      // this block are ONE contiguous, 16-byte aligned run of 64*HW elements -> 16-byte loads into
      // a flat copy, transposed on the way out with a row pitch of HW elements
      const int nch = min(kPackCT, C - c0);
      const int total16 = (nch * HW) >> 3;  // nch is a multiple of 8
      const uint4* src16 = reinterpret_cast<const uint4*>(s + static_cast<long long>(c0) * HW);
      uint4* dst16 = reinterpret_cast<uint4*>(tile_w);
      for (int i = tid; i < total16; i += 256) dst16[i] = src16[i];
      __syncthreads();
      for (int item = tid; item < HW * 8; item += 256) {
        const int pix = item >> 3;
        const int cv = (item & 7) * 8;
        if (c0 + cv < c_pad8) {
          __align__(16) __half v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            v[j] = (cv + j < nch) ? tile[(cv + j) * HW + pix] : __float2half(0.f);
          *reinterpret_cast<uint4*>(d + static_cast<long long>(pix) * c_pad8 + c0 + cv) =
              *reinterpret_cast<const uint4*>(v);
        }
      }
      return;
    } else {
      const int tx = tid & 63;
      const int ty = tid >> 6;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int cl = ty + 4 * i;
        __half v = __float2half(0.f);
        if (c0 + cl < C && p0 + tx < HW) v = s[static_cast<long long>(c0 + cl) * HW + p0 + tx];
        tile[cl * (2 * kPackLdW) + tx] = v;
      }
    }
    __syncthreads();
    // one pixel pair x 8 channels per thread: 8 words in, two 16-byte vectors out
    const int cg = tid & 7;
    const int pp = tid >> 3;
    const int pix = p0 + 2 * pp;
    const int c = c0 + cg * 8;
    if (c < c_pad8 && pix < HW) {
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) w[j] = tile_w[(cg * 8 + j) * kPackLdW + pp];
      uint4 lo, hi;
      lo.x = __byte_perm(w[0], w[1], 0x5410);
      lo.y = __byte_perm(w[2], w[3], 0x5410);
      lo.z = __byte_perm(w[4], w[5], 0x5410);
      lo.w = __byte_perm(w[6], w[7], 0x5410);
      hi.x = __byte_perm(w[0], w[1], 0x7632);
      hi.y = __byte_perm(w[2], w[3], 0x7632);
      hi.z = __byte_perm(w[4], w[5], 0x7632);
      hi.w = __byte_perm(w[6], w[7], 0x7632);
      *reinterpret_cast<uint4*>(d + static_cast<long long>(pix) * c_pad8 + c) = lo;
      if (pix + 1 < HW) *reinterpret_cast<uint4*>(d + static_cast<long long>(pix + 1) * c_pad8 + c) = hi;
    }
  } else {
    const int id = blockIdx.x - act_blocks;
    const int k = id / flt_chunks;
    const int cc = id - k * flt_chunks;
    const int cstart = cc * flt_chunk;
    const int c_in = max(0, min(flt_chunk, C - cstart));   // channels that exist in the source
    const bool last = cc == flt_chunks - 1;
    const int c_out = last ? (c_pad64 - cstart) : flt_chunk;  // channels written (zero padded)
    const __half* s = flt + (static_cast<long long>(k) * C + cstart) * RS;
    // flt_chunk is a multiple of 8, so with C % 8 == 0 the chunk starts 16-byte aligned
    if ((C & 7) == 0) {
      const int total16 = (c_in * RS) >> 3;
      const uint4* src16 = reinterpret_cast<const uint4*>(s);
      uint4* dst16 = reinterpret_cast<uint4*>(tile_w);
      for (int i = tid; i < total16; i += 256) dst16[i] = src16[i];
      for (int i = (total16 << 3) + tid; i < c_in * RS; i += 256) tile[i] = s[i];
    } else {
      for (int i = tid; i < c_in * RS; i += 256) tile[i] = s[i];
    }
    __syncthreads();
    __half* d = flt_krsc + static_cast<long long>(k) * RS * c_pad64 + cstart;
    // c_out is a multiple of 8: one 16-byte vector of 8 channels per item
    const int vec_per_rs = c_out >> 3;
    for (int i = tid; i < vec_per_rs * RS; i += 256) {
      const int rs = i / vec_per_rs;
      const int cv = (i - rs * vec_per_rs) * 8;
      __align__(16) __half v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        v[j] = (cv + j < c_in) ? tile[(cv + j) * RS + rs] : __float2half(0.f);
      *reinterpret_cast<uint4*>(d + static_cast<long long>(rs) * c_pad64 + cv) =
          *reinterpret_cast<const uint4*>(v);
    }
  }
}

// The same re-layout for 8-bit and 32-bit elements (int8 and float32 tensors), kept simple: a block
// transposes a 32 (channels) x 32 (pixels) tile of one image through shared memory, or moves one
// filter.  Blocks [0, act_blocks): NCHW -> NHWC with `c_pad_a` channels per pixel (zero filled);
// blocks [act_blocks, ...): filter k of KCRS -> [R*S][c_pad_f] (zero filled).
template <typename T>
__global__ void __launch_bounds__(256)
conv_prepack_generic_kernel(const T* __restrict__ act, T* __restrict__ act_nhwc,
                            const T* __restrict__ flt, T* __restrict__ flt_krsc, int C, int HW,
                            int c_pad_a, int act_blocks, int c_tiles, int p_tiles, int RS,
                            int c_pad_f) {
  __shared__ T tile[32][33];
  if (threadIdx.x == 255) grid_launch_dependents();
  const int tx = threadIdx.x & 31;
  const int ty = threadIdx.x >> 5;  // 0..7
  if (static_cast<int>(blockIdx.x) < act_blocks) {
    const int id = blockIdx.x;
    const int pt = id % p_tiles;
    const int ct = (id / p_tiles) % c_tiles;
    const int n = id / (p_tiles * c_tiles);
    const int p0 = pt * 32, c0 = ct * 32;
    const T* s = act + static_cast<long long>(n) * C * HW;
    T* d = act_nhwc + static_cast<long long>(n) * HW * c_pad_a;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int cl = ty + 8 * i;
      T v = T(0);
      if (c0 + cl < C && p0 + tx < HW) v = s[static_cast<long long>(c0 + cl) * HW + p0 + tx];
      tile[cl][tx] = v;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int pl = ty + 8 * i;
      if (p0 + pl < HW && c0 + tx < c_pad_a)
        d[static_cast<long long>(p0 + pl) * c_pad_a + c0 + tx] = tile[tx][pl];
    }
  } else {
    const int k = blockIdx.x - act_blocks;
    const T* s = flt + static_cast<long long>(k) * C * RS;
    T* d = flt_krsc + static_cast<long long>(k) * RS * c_pad_f;
    for (int i = threadIdx.x; i < RS * c_pad_f; i += 256) {
      const int rs = i / c_pad_f;
      const int c = i - rs * c_pad_f;
      d[i] = c < C ? s[static_cast<long long>(c) * RS + rs] : T(0);
    }
  }
}

// --------------------------------------------------------------------------------------------
// Kernel dispatch
// --------------------------------------------------------------------------------------------
static thread_local int g_launch_count = 0;

// Issuing threads for the TMA loads.  Measured on B200: three threads beat one by 5-8 % on the
// 3x3 convolutions and by ~1 % on the large GEMMs; never slower.
static bool dependent_launch_enabled() { return getenv("AMOSB_NO_PDL") == nullptr; }

// Budget of the kernels' bounded waits and the diagnostic that makes one run out; both are read at
// every launch so that a test can set them around a single call.
static void set_wait_params(UmmaParams* p) {
  p->wait_budget_ns = 2000000000ull;
  if (const char* e = getenv("AMOSB_WAIT_BUDGET_NS")) {
    const long long v = atoll(e);
    if (v > 0) p->wait_budget_ns = static_cast<unsigned long long>(v);
  }
  const char* d = getenv("AMOSB_DIAG_NO_LOADS");
  p->diag_no_loads = (d != nullptr && d[0] == '1') ? 1 : 0;
}

static int producer_threads() {
  int n = 3;
  if (const char* e = getenv("AMOSB_PRODUCERS")) n = atoi(e);
  return n < 1 ? 1 : (n > 3 ? 3 : n);
}

template <int KIND, int BN, bool B_MN, int MODE, typename OutT, bool EPI, int MT = 1,
          bool A_MN = false>
static int launch_umma(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                       const UmmaParams& p, int grid, cudaStream_t stream) {
  auto kernel = umma_persistent_kernel<KIND, BN, B_MN, MODE, OutT, EPI, MT, A_MN>;
  constexpr int smem = UmmaConfig<BN, EPI, MT>::kSmemBytes;
  // one bit per device; setting the attribute twice from racing threads is harmless
  static std::atomic<unsigned long long> attr_set{0};
  int dev = 0;
  AMOSB_CUDA_CHECK(cudaGetDevice(&dev));
  if (((attr_set.load(std::memory_order_acquire) >> dev) & 1ull) == 0) {
    AMOSB_CUDA_CHECK(
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set.fetch_or(1ull << dev, std::memory_order_release);
  }
#ifdef AMOSB_ROLE_CYCLES
  UmmaParams pd = p;
  void* rc_ptr = nullptr;
  AMOSB_CUDA_CHECK(cudaGetSymbolAddress(&rc_ptr, g_role_cycles));
  pd.role_cycles = static_cast<unsigned long long*>(rc_ptr);
  pd.dbg_skip = getenv("AMOSB_DBG_SKIP") ? atoi(getenv("AMOSB_DBG_SKIP")) : 0;
  kernel<<<grid, umma_threads(MODE), smem, stream>>>(tmA, tmB, tmC, pd);
#else
  {
    // programmatic dependent of whatever precedes it in the stream (the re-layout kernel of an NCHW
    // conv, the previous call's kernel): its set-up overlaps that kernel's tail, its first global
    // access waits for that kernel's completion
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(umma_threads(MODE), 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = dependent_launch_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    AMOSB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmC, p));
  }
#endif
  AMOSB_CUDA_CHECK(cudaGetLastError());
  ++g_launch_count;
  return AMOSB_OK;
}

template <int KIND, bool B_MN, int MODE, typename OutT, bool EPI, bool A_MN = false>
static int dispatch_bn(int bn, const CUtensorMap& tmA, const CUtensorMap& tmB,
                       const CUtensorMap& tmC, const UmmaParams& p, int grid,
                       cudaStream_t stream) {
  switch (bn) {
    case 256:
      return launch_umma<KIND, 256, B_MN, MODE, OutT, EPI, 1, A_MN>(tmA, tmB, tmC, p, grid,
                                                                    stream);
    case 128:
      if (p.mt == 2) {
        if constexpr (KIND == 0 && !A_MN) {  // tall tiles: fp16, K-major A only
          return launch_umma<KIND, 128, B_MN, MODE, OutT, EPI, 2>(tmA, tmB, tmC, p, grid, stream);
        } else {
          break;
        }
      }
      return launch_umma<KIND, 128, B_MN, MODE, OutT, EPI, 1, A_MN>(tmA, tmB, tmC, p, grid,
                                                                    stream);
    case 64:
      if constexpr (KIND == 1 && B_MN) {
        break;  // an int8 MN-major chunk is 128 columns wide
      } else {
        return launch_umma<KIND, 64, B_MN, MODE, OutT, EPI, 1, A_MN>(tmA, tmB, tmC, p, grid,
                                                                     stream);
      }
    default:
      break;
  }
  set_error("tile_n=%d is not available for this operand layout", bn);
  return AMOSB_ERR_UNSUPPORTED;
}

// GEMM-mode dispatch over output type, B layout and epilogue kind.
template <int KIND, typename OutT>
static int dispatch_gemm(bool trans_a, bool trans_b, bool epi_tma, int bn, const CUtensorMap& tmA,
                         const CUtensorMap& tmB, const CUtensorMap& tmC, const UmmaParams& p,
                         int grid, cudaStream_t stream) {
  if (trans_a) {  // A given as [K][M]: MN-major A operand
    if (trans_b) {
      if (epi_tma)
        return dispatch_bn<KIND, false, kModeGemm, OutT, true, true>(bn, tmA, tmB, tmC, p, grid,
                                                                     stream);
      return dispatch_bn<KIND, false, kModeGemm, OutT, false, true>(bn, tmA, tmB, tmC, p, grid,
                                                                    stream);
    }
    if (epi_tma)
      return dispatch_bn<KIND, true, kModeGemm, OutT, true, true>(bn, tmA, tmB, tmC, p, grid,
                                                                  stream);
    return dispatch_bn<KIND, true, kModeGemm, OutT, false, true>(bn, tmA, tmB, tmC, p, grid,
                                                                 stream);
  }
  if (trans_b) {
    if (epi_tma)
      return dispatch_bn<KIND, false, kModeGemm, OutT, true>(bn, tmA, tmB, tmC, p, grid, stream);
    return dispatch_bn<KIND, false, kModeGemm, OutT, false>(bn, tmA, tmB, tmC, p, grid, stream);
  }
  if (epi_tma)
    return dispatch_bn<KIND, true, kModeGemm, OutT, true>(bn, tmA, tmB, tmC, p, grid, stream);
  return dispatch_bn<KIND, true, kModeGemm, OutT, false>(bn, tmA, tmB, tmC, p, grid, stream);
}

// ---- CTA-pair kernels (cluster of two CTAs per 256-row tile)
template <int KIND, int BN, bool B_MN, int MODE, typename OutT, bool EPI>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                       const UmmaParams& p, int pairs, cudaStream_t stream) {
  auto kernel = umma_pair_kernel<KIND, BN, B_MN, MODE, OutT, EPI>;
  constexpr int smem = PairConfig<BN, EPI>::kSmemBytes;
  // one bit per device; setting the attribute twice from racing threads is harmless
  static std::atomic<unsigned long long> attr_set{0};
  int dev = 0;
  AMOSB_CUDA_CHECK(cudaGetDevice(&dev));
  if (((attr_set.load(std::memory_order_acquire) >> dev) & 1ull) == 0) {
    AMOSB_CUDA_CHECK(
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set.fetch_or(1ull << dev, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kNumThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (dependent_launch_enabled()) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
#ifdef AMOSB_ROLE_CYCLES
  UmmaParams pd = p;
  void* rc_ptr = nullptr;
  AMOSB_CUDA_CHECK(cudaGetSymbolAddress(&rc_ptr, g_role_cycles));
  pd.role_cycles = static_cast<unsigned long long*>(rc_ptr);
  AMOSB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmC, pd));
#else
  AMOSB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmC, p));
#endif
  ++g_launch_count;
  return AMOSB_OK;
}

template <int KIND, bool B_MN, int MODE, typename OutT, bool EPI>
static int dispatch_pair_bn(int bn, const CUtensorMap& tmA, const CUtensorMap& tmB,
                            const CUtensorMap& tmC, const UmmaParams& p, int pairs,
                            cudaStream_t stream) {
  if (bn == 256) return launch_pair<KIND, 256, B_MN, MODE, OutT, EPI>(tmA, tmB, tmC, p, pairs, stream);
  if (bn == 128) {
    if constexpr (KIND == 1 && B_MN) {
      // half of a 128-wide int8 MN-major tile is narrower than one 128-byte chunk
    } else {
      return launch_pair<KIND, 128, B_MN, MODE, OutT, EPI>(tmA, tmB, tmC, p, pairs, stream);
    }
  }
  set_error("tile_n=%d is not available for CTA pairs with this operand layout", bn);
  return AMOSB_ERR_UNSUPPORTED;
}

template <int KIND, typename OutT>
static int dispatch_pair_gemm(bool trans_b, bool epi_tma, int bn, const CUtensorMap& tmA,
                              const CUtensorMap& tmB, const CUtensorMap& tmC, const UmmaParams& p,
                              int pairs, cudaStream_t stream) {
  if (trans_b) {
    if (epi_tma)
      return dispatch_pair_bn<KIND, false, kModeGemm, OutT, true>(bn, tmA, tmB, tmC, p, pairs, stream);
    return dispatch_pair_bn<KIND, false, kModeGemm, OutT, false>(bn, tmA, tmB, tmC, p, pairs, stream);
  }
  if (epi_tma)
    return dispatch_pair_bn<KIND, true, kModeGemm, OutT, true>(bn, tmA, tmB, tmC, p, pairs, stream);
  return dispatch_pair_bn<KIND, true, kModeGemm, OutT, false>(bn, tmA, tmB, tmC, p, pairs, stream);
}

struct TailPlan {
  int sk_tiles = 0, q = 0, r = 0;
};
// `tiles` tiles of `num_kb` k-blocks on `workers` CTAs (CTA pairs); a k-block of this tile family
// takes about `kb_ns` nanoseconds.  Whole tiles cost ceil(tiles / workers) rounds of num_kb
// k-blocks; when the last round is short, its k-blocks can be shared out evenly instead, at the
// price of exchanging partial sums through L2.  The CTA that finishes a shared tile pulls each
// other part's 128 KB with 128 threads, 16 KB in flight at a time: ~6 us per part (measured), which
// only stays off the critical path when a round of whole tiles follows the shares (the exchange
// then runs under that round's main loop) and the tile is not store-bound already.  So the tail
// is shared out only where the gain is large and clear: a whole round follows, the shares save at
// least half a round and at least 16 us.  (Measured on B200: 7x7 C512->K512 3x3 batch 256, NHWC
// 53 -> 46 us; tf32 4096^3 214 -> 205 us.  The fp16 4096^3 GEMM, power-bound, and the 28x28 /
// 14x14 3x3 layers, store-bound or with little to save, lose 2-16 us and are left alone.)
// AMOSB_TAIL_SHARING=1 shares out whenever the last round is short (tests use it on small shapes),
// AMOSB_NO_TAIL_SHARING=1 never does.
static TailPlan plan_tail(long long tiles, int workers, int num_kb, double kb_ns) {
  TailPlan t;
  if (getenv("AMOSB_NO_TAIL_SHARING") != nullptr || workers <= 1 || num_kb < 2) return t;
  const long long rem = tiles % workers;
  if (rem == 0) return t;
  const long long units = rem * num_kb;
  const long long q = units / workers;
  const char* force = getenv("AMOSB_TAIL_SHARING");
  if (force != nullptr && force[0] == '1') {
    if (q < 1) return t;
  } else {
    const long long saved_kb = num_kb - (units + workers - 1) / workers;
    if (tiles < workers || q < 4 || saved_kb * 2 < num_kb || saved_kb * kb_ns < 16000.0) return t;
  }
  t.sk_tiles = static_cast<int>(rem);
  t.q = static_cast<int>(q);
  t.r = static_cast<int>(units % workers);
  return t;
}
// Nanoseconds per k-block of a tile family (the constants of choose_plan).
static double kb_cost_ns(int bn, int mt, bool pairs) {
  if (pairs) return bn == 256 ? 410.0 : 335.0;
  if (mt == 2) return 415.0;
  return bn == 256 ? 400.0 : bn == 128 ? 240.0 : 168.0;
}

// Tile width and kernel family for a problem, from a small cost model: time ~ waves x cost of one
// k-block of the tile.  The costs are nanoseconds per k-block and wave, fitted on B200 to GEMMs
// with M = 256..4096, N = K = 4096 and to the batch-256 3x3 convolution layers: CTA pair x256:
// 410, x128: 335; single CTA 128x256: 400, 128x128: 240, 128x64: 168.  A 256-wide tile runs at
// the rate of the tensor pipe; narrower tiles are bound by what one SM can pull from L2
// (~75 bytes per clock), so they are cheaper but not in proportion; a pair MMA with N = 128 runs
// at half rate, so that family only wins when its wave count does.  Convolutions cost ~12 % more
// in every family, which does not change the ranking.
// A single CTA can also run "tall" 256 x 128 tiles (two accumulators sharing each B stage): the
// MMA time of a 128 x 256 tile with half the B bytes per flop of a 128 x 128 one (415 per k-block
// measured, against 2 x 240 for the two 128 x 128 tiles it replaces); `tall_ok` says whether that
// family exists for the operands (fp16 only).
// `tile_n` / `pair_mode` (0 = free, 1 = single CTA, 2 = CTA pair, 3 = single CTA, tall tiles; 4,
// internal: any single-CTA family) pin either choice.
void choose_plan(bool i8_mn, bool tall_ok, long long batch, long long m, long long n,
                 long long kblocks, int tile_n, int pair_mode, int sm_count, int* bn_out,
                 bool* pairs_out, int* mt_out) {
  if (getenv("AMOSB_NO_PAIRS") != nullptr && pair_mode != 3) pair_mode = 1;
  struct Cand {
    int bn;
    bool pair;
    double cost;
    int mt;
  };
  constexpr int kCands = 6;
  const Cand cands[kCands] = {{256, true, 410.0, 1},  {128, true, 335.0, 1}, {256, false, 400.0, 1},
                              {128, false, 415.0, 2}, {128, false, 240.0, 1}, {64, false, 168.0, 1}};
  if (mt_out) *mt_out = 1;
  double best = 0.0;
  int best_i = -1;
  for (int i = 0; i < kCands; ++i) {
    const Cand& c = cands[i];
    if (tile_n != 0 && c.bn != tile_n) continue;
    if (c.mt == 2 && (!tall_ok || mt_out == nullptr || m <= kBlockM || pair_mode == 1 ||
                      pair_mode == 2))
      continue;
    if (c.mt == 1 && pair_mode == 3 && tall_ok && mt_out != nullptr && m > kBlockM &&
        (tile_n == 0 || tile_n == 128))
      continue;  // tall tiles were asked for and are possible
    if (c.pair && (pair_mode == 1 || pair_mode == 3 || pair_mode == 4 || sm_count < 2 || m <= kBlockM))
      continue;
    if (!c.pair && pair_mode == 2 && m > kBlockM && sm_count >= 2 &&
        !(i8_mn && tile_n == 128) && tile_n != 64)
      continue;  // pairs were asked for and are possible
    if (i8_mn && (c.bn == 64 || (c.pair && c.bn == 128))) continue;  // 128-byte chunk granularity
    const int narrowest = i8_mn ? 128 : 64;
    if (tile_n == 0 && c.bn > narrowest && n <= c.bn / 2) continue;  // half the tile would be padding
    const long long rows = (c.pair || c.mt == 2) ? 2 * kBlockM : kBlockM;
    const long long tiles = batch * ((m + rows - 1) / rows) * ((n + c.bn - 1) / c.bn);
    const long long slots = c.pair ? sm_count / 2 : sm_count;
    double waves = static_cast<double>((tiles + slots - 1) / slots);
    const long long rem = tiles % slots;
    // a short last round whose k-blocks are shared out among all workers costs its share of a
    // round plus the exchange of partial sums (see plan_tail)
    const bool shared_tail =
        plan_tail(tiles, static_cast<int>(slots), static_cast<int>(kblocks), c.cost).sk_tiles > 0;
    if (shared_tail)
      waves = static_cast<double>(tiles / slots) +
              static_cast<double>((rem * kblocks + slots - 1) / slots + 3) / static_cast<double>(kblocks);
    // a short last wave of a pair launch costs less than its tile time: the idle SMs leave their
    // share of the power budget to the busy ones (seen from the third wave on; with two waves the
    // 7x7 layers of 512 channels measured 8 % faster on 128-wide single-CTA tiles)
    if (!shared_tail && c.pair && c.bn == 256 && tiles > 2 * slots && rem > 0 && 2 * rem <= slots)
      waves -= 0.25;
    double cost = c.cost;
    // Over several waves a 256-wide pair tile is a little cheaper than the single-CTA tile (half
    // the B reads per SM leave more of the power budget to the tensor pipe); within one wave the
    // larger tile only adds latency.
    // With one or two k-blocks per tile the epilogue is all there is, and a pair only adds the
    // hand-shake between its CTAs.
    if (c.pair && c.bn == 256) cost = (tiles > slots && kblocks > 2) ? 395.0 : 430.0;
    const double t = waves * cost;
    if (best_i < 0 || t < best * 0.999) {
      best = t;
      best_i = i;
    }
  }
  if (best_i < 0) {  // nothing satisfied the pins: fall back to the request as a single-CTA tile
    *bn_out = tile_n != 0 ? tile_n : (i8_mn ? 128 : 64);
    *pairs_out = false;
    return;
  }
  *bn_out = cands[best_i].bn;
  *pairs_out = cands[best_i].pair;
  if (mt_out) *mt_out = cands[best_i].mt;
}

static void plan_for_desc(const AmosbOpDesc& d, int sm_count, int* bn, bool* pairs, int* mt) {
  const bool conv = d.kind == AMOSB_OP_CONV2D_NCHW || d.kind == AMOSB_OP_CONV2D_NHWC ||
                    d.kind == AMOSB_OP_CONV2D_HWNC;
  const bool tall_ok = d.in_dtype == AMOSB_F16 || d.in_dtype == AMOSB_BF16;
  if (d.kind == AMOSB_OP_CONV2D_NCHW && conv_is_pointwise_gemm(d)) {
    choose_plan(false, tall_ok, d.conv_n, d.conv_k, d.conv_p * d.conv_q, (d.conv_c + 63) / 64,
                d.tile_n, d.cta_pair, sm_count, bn, pairs, mt);
    return;
  }
  const long long n = conv ? d.conv_k : d.n;
  const long long m = conv ? d.conv_n * d.conv_p * d.conv_q : d.m;
  const long long batch = conv ? 1 : d.batch;
  // the RSCK filter of the in-place conv layouts is an MN-major operand as well
  const bool i8_mn = d.in_dtype == AMOSB_S8 &&
                     (conv ? d.kind != AMOSB_OP_CONV2D_NCHW : !d.trans_b);
  const long long kelems = d.in_dtype == AMOSB_S8 ? 128 : d.in_dtype == AMOSB_F32 ? 32 : 64;
  const long long kblocks = conv ? d.conv_r * d.conv_s * ((d.conv_c + kelems - 1) / kelems)
                                 : (d.k + kelems - 1) / kelems;
  // A indexed [k,i] runs on single-CTA 128-row tiles only, and so do float32 (tf32) and int8 NCHW
  // convolutions
  const bool single_only =
      (!conv && d.trans_a) ||
      (d.kind == AMOSB_OP_CONV2D_NCHW && (d.in_dtype == AMOSB_F32 || d.in_dtype == AMOSB_S8));
  const int pair_mode = single_only ? 1 : d.cta_pair;
  choose_plan(i8_mn, tall_ok, batch, m, n, kblocks, d.tile_n, pair_mode, sm_count, bn, pairs, mt);
}

int choose_tile_n(const AmosbOpDesc& d, int sm_count) {
  int bn = 0, mt = 1;
  bool pairs = false;
  plan_for_desc(d, sm_count, &bn, &pairs, &mt);
  return bn;
}

int choose_tile_rows(const AmosbOpDesc& d, int sm_count) {
  int bn = 0, mt = 1;
  bool pairs = false;
  plan_for_desc(d, sm_count, &bn, &pairs, &mt);
  return (pairs || mt == 2) ? 2 * kBlockM : kBlockM;
}

bool choose_cta_pairs(const AmosbOpDesc& d, int sm_count) {
  int bn = 0, mt = 1;
  bool pairs = false;
  plan_for_desc(d, sm_count, &bn, &pairs, &mt);
  return pairs;
}

// --------------------------------------------------------------------------------------------
// Schedule: whole tiles round-robin, plus a shared-out tail where the last round would be short
// --------------------------------------------------------------------------------------------
// Completes the schedule fields of `p` (num_tiles and num_kb are final) and returns the number of
// workers to launch.  The tail is shared out only if `ws` has room for one partial accumulator tile
// per CTA (`partial_elems` 32-bit words each, `ctas_per_worker` CTAs per worker).
static int setup_schedule(UmmaParams* p, DeviceState* st, int device, int workers_max,
                          int ctas_per_worker, size_t partial_elems, void* ws, long long ws_bytes) {
  // k-block time of the tile family, from the accumulator columns a CTA holds (a tall 256 x 128
  // tile counts as 256 columns: the same MMA time per k-block)
  const double kb_ns = kb_cost_ns(static_cast<int>(partial_elems / kBlockM), 1, ctas_per_worker == 2);
  p->sk_tiles = 0;
  p->sk_first = p->num_tiles;
  p->sk_q = p->sk_r = 0;
  p->sk_partials = nullptr;
  p->sk_flags = st->sk_flags;
  const TailPlan t = plan_tail(p->num_tiles, workers_max, p->num_kb, kb_ns);
  const long long need =
      static_cast<long long>(workers_max) * ctas_per_worker * partial_elems * 4;
  if (t.sk_tiles > 0 && ws != nullptr && ws_bytes >= need &&
      workers_max * ctas_per_worker <= kSkCtasMax &&
      (reinterpret_cast<uintptr_t>(ws) & 15u) == 0) {
    p->sk_tiles = t.sk_tiles;
    p->sk_first = p->num_tiles - t.sk_tiles;
    p->sk_q = t.q;
    p->sk_r = t.r;
    p->sk_partials = static_cast<uint32_t*>(ws);
    const unsigned int slot = g_sk_next[device].fetch_add(1u) % kSkSlots;
    p->sk_flags = st->sk_flags + static_cast<size_t>(slot) * kSkCtasMax * 4;
    return workers_max;  // every worker has a share
  }
  return p->num_tiles < workers_max ? p->num_tiles : workers_max;
}

// Scratch the shared-out tail wants for `tiles` tiles on a full B200 (148 SMs), 0 if the tail is
// not shared out.
static long long tail_scratch_bytes(long long tiles, int num_kb, bool pairs, int mt, int bn) {
  const int sms = 148;
  const int workers = pairs ? sms / 2 : sms;
  if (tiles > 0x7fffffffLL ||
      plan_tail(tiles, workers, num_kb, kb_cost_ns(pairs ? bn : mt * bn, 1, pairs)).sk_tiles == 0)
    return 0;
  const long long elems = static_cast<long long>(pairs ? 1 : mt) * kBlockM * bn;
  return static_cast<long long>(sms) * elems * 4;
}

// --------------------------------------------------------------------------------------------
// GEMM family
// --------------------------------------------------------------------------------------------
// Core of the GEMM family: C[b] (M x N) = A[b or shared] (M x K, K-major) * B[b] (K x N row-major,
// or N x K when trans_b).  Also used by 1x1 convolutions (A = filter shared by all images).
struct TrailingOps {
  int flags = 0;  // kEpi*
  int f16 = 0;
  const void* addend = nullptr;
};

// Kernel-side flags for the descriptor's fused stages; `rows_are_channels` = the N-axis vector of
// the operator indexes the rows of the GEMM that runs it (1x1 convolution as GEMM).
static int trailing_ops_for(const AmosbOpDesc& d, const void* addend, bool rows_are_channels,
                            TrailingOps* t) {
  t->flags = 0;
  t->addend = addend;
  t->f16 = d.addend_dtype == AMOSB_F16 ? 1 : 0;
  const int add_bits = d.epilogue & (AMOSB_EPI_ADD_VECTOR | AMOSB_EPI_ADD_FULL);
  if (add_bits == (AMOSB_EPI_ADD_VECTOR | AMOSB_EPI_ADD_FULL)) {
    set_error("only one addend can be fused");
    return AMOSB_ERR_UNSUPPORTED;
  }
  if (add_bits != 0) {
    if (addend == nullptr) {
      set_error("descriptor fuses an addend but none was passed");
      return AMOSB_ERR_ARG;
    }
    const bool ok_dtype = d.addend_dtype == d.acc_dtype ||
                          (d.acc_dtype == AMOSB_F32 && d.addend_dtype == AMOSB_F16);
    if (!ok_dtype) {
      set_error("addend dtype must be the accumulator dtype (or float16 for float32)");
      return AMOSB_ERR_UNSUPPORTED;
    }
    if (add_bits == AMOSB_EPI_ADD_VECTOR)
      t->flags |= rows_are_channels ? kEpiAddRowVec : kEpiAddVec;
    else
      t->flags |= kEpiAddFull;
  }
  if (d.epilogue & AMOSB_EPI_RELU) t->flags |= kEpiRelu;
  if (d.epilogue & ~(AMOSB_EPI_ADD_VECTOR | AMOSB_EPI_ADD_FULL | AMOSB_EPI_RELU)) {
    set_error("unknown epilogue bits 0x%x", d.epilogue);
    return AMOSB_ERR_ARG;
  }
  return AMOSB_OK;
}

// Operand-format bits of the instruction descriptor for a 16-bit input type.
static uint32_t idesc_formats_for(int in_dtype) {
  return in_dtype == AMOSB_BF16 ? ((1u << 7) | (1u << 10)) : 0u;
}
// float32 operands travel as TFLOAT32: the copy engine rounds every element to tf32 (nearest, ties to
// even) on its way into shared memory, so the MMA, which reads only the upper 19 bits, sees
// rounded rather than truncated values.
static CUtensorMapDataType tma_dtype_for(int in_dtype) {
  return in_dtype == AMOSB_S8     ? CU_TENSOR_MAP_DATA_TYPE_UINT8
         : in_dtype == AMOSB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
         : in_dtype == AMOSB_F32  ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32
                                  : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

static int run_gemm_core(DeviceState* st, int in_dtype, int out_dtype, bool trans_a, bool trans_b,
                         bool a_shared, long long batch, long long M, long long N, long long K,
                         int tile_n, int pair_mode, const TrailingOps& ops, const void* a,
                         const void* b, void* c, void* ws, long long ws_bytes, int device,
                         cudaStream_t stream) {
  const bool is_i8 = in_dtype == AMOSB_S8;
  const bool is_tf32 = in_dtype == AMOSB_F32;  // float32 operands, read by the MMA as tf32
  if (in_dtype == AMOSB_BF16 && out_dtype != AMOSB_F32) {
    set_error("bfloat16 inputs accumulate into and write float32");
    return AMOSB_ERR_UNSUPPORTED;
  }
  if (is_tf32) {
    if (out_dtype != AMOSB_F32) {
      set_error("float32 (tf32) inputs accumulate into and write float32");
      return AMOSB_ERR_UNSUPPORTED;
    }
    // single-CTA 128-row tiles and CTA pairs; no tall tiles
    if (pair_mode == 3) {
      set_error("cta_pair=%d is not available for float32 (tf32) inputs", pair_mode);
      return AMOSB_ERR_UNSUPPORTED;
    }
  }
  const int es = is_i8 ? 1 : is_tf32 ? 4 : 2;
  const int elems128 = 128 / es;
  if (trans_a) {
    // A[K,M] is an MN-major operand of the single-CTA 128-row tiles only
    if (pair_mode == 2 || pair_mode == 3) {
      set_error("cta_pair=%d is not available for A indexed [k,i]", pair_mode);
      return AMOSB_ERR_UNSUPPORTED;
    }
    pair_mode = 1;
    if ((M * es) % 16 != 0) {
      set_error("M=%lld: rows of A[K,M] must be a multiple of 16 bytes for TMA", M);
      return AMOSB_ERR_UNSUPPORTED;
    }
  }
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) {
    set_error("GEMM extents must be positive (batch=%lld m=%lld n=%lld k=%lld)", batch, M, N, K);
    return AMOSB_ERR_ARG;
  }
  if ((!trans_a || trans_b) && (K * es) % 16 != 0) {
    set_error("K=%lld: rows of A[M,K] / B[N,K] must be a multiple of 16 bytes for TMA", K);
    return AMOSB_ERR_UNSUPPORTED;
  }
  if (!trans_b && (N * es) % 16 != 0) {
    set_error("N=%lld: rows of B[K,N] must be a multiple of 16 bytes for TMA", N);
    return AMOSB_ERR_UNSUPPORTED;
  }
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) {
    set_error("extent beyond 2^31");
    return AMOSB_ERR_UNSUPPORTED;
  }
  int bn = 0, mt = 1;
  bool pairs = false;
  choose_plan(is_i8 && !trans_b, !is_i8 && !is_tf32, batch, M, N, (K + elems128 - 1) / elems128, tile_n,
              pair_mode, st->sm_count, &bn, &pairs, &mt);
  const long long tiles_pair = batch * ((M + 2 * kBlockM - 1) / (2 * kBlockM)) * ((N + bn - 1) / bn);
  const CUtensorMapDataType dt = tma_dtype_for(in_dtype);
  CUtensorMap tmA, tmB, tmC;
  memset(&tmC, 0, sizeof(tmC));
  // MN-major operands of 32-bit elements: the 128-byte swizzle with 32-byte units
  const CUtensorMapSwizzle sw_mn =
      is_tf32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
  int rc = trans_a ? encode_tiled_3d(&tmA, dt, es, const_cast<void*>(a), M, K, a_shared ? 1 : batch,
                                     M * es, K * M * es, elems128, elems128, sw_mn)
                   : encode_tiled_3d(&tmA, dt, es, const_cast<void*>(a), K, M, a_shared ? 1 : batch,
                                     K * es, M * K * es, elems128, kBlockM);
  if (rc != AMOSB_OK) return rc;
  if (trans_b) {
    rc = encode_tiled_3d(&tmB, dt, es, const_cast<void*>(b), K, N, batch, K * es, N * K * es,
                         elems128, pairs ? 64 : bn);
  } else {
    rc = encode_tiled_3d(&tmB, dt, es, const_cast<void*>(b), N, K, batch, N * es, K * N * es,
                         elems128, elems128, sw_mn);
  }
  if (rc != AMOSB_OK) return rc;
  // Output through TMA stores when the rows of C are 16-byte multiples; else plain stores.
  const int ob = (out_dtype == AMOSB_F16) ? 2 : 4;
  const bool epi_tma = (N * ob) % 16 == 0 && getenv("AMOSB_DIRECT_STORE") == nullptr;
  if (epi_tma) {
    CUtensorMapDataType odt = out_dtype == AMOSB_F16   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                              : out_dtype == AMOSB_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                       : CU_TENSOR_MAP_DATA_TYPE_INT32;
    rc = encode_tiled_3d(&tmC, odt, ob, c, N, M, batch, N * ob, M * N * ob, 128 / ob, 32);
    if (rc != AMOSB_OK) return rc;
  }

  UmmaParams p;
  memset(&p, 0, sizeof(p));
  set_wait_params(&p);
  p.M = (int)M;
  p.N = (int)N;
  p.K = (int)K;
  p.batch = (int)batch;
  p.mt = mt;
  p.idesc_formats = idesc_formats_for(in_dtype);
  p.tiles_m = (int)((M + mt * kBlockM - 1) / (mt * kBlockM));
  p.tiles_n = (int)((N + bn - 1) / bn);
  p.group_m = 16;
  p.num_kb = (int)((K + elems128 - 1) / elems128);
  const long long tiles = batch * p.tiles_m * p.tiles_n;
  if (tiles > 0x7fffffffLL) {
    set_error("too many tiles");
    return AMOSB_ERR_UNSUPPORTED;
  }
  p.num_tiles = (int)tiles;
  p.ldc = N;
  p.c_batch_stride = M * N;
  p.out = c;
  p.status = st->status_ptr;
  p.a_bcast = a_shared ? 1 : 0;
  p.producers = producer_threads();
  p.epi_flags = ops.flags;
  p.addend_f16 = ops.f16;
  p.addend = ops.addend;
  if (is_i8 && out_dtype != AMOSB_S32) {
    set_error("int8 GEMM writes int32");
    return AMOSB_ERR_UNSUPPORTED;
  }
  if (pairs) {
    p.tiles_m = (int)((M + 2 * kBlockM - 1) / (2 * kBlockM));
    p.num_tiles = (int)tiles_pair;
    const int npairs = setup_schedule(&p, st, device, st->sm_count / 2, 2,
                                      static_cast<size_t>(kBlockM) * bn, ws, ws_bytes);
    if (is_i8)
      return dispatch_pair_gemm<1, int32_t>(trans_b, epi_tma, bn, tmA, tmB, tmC, p, npairs, stream);
    if (is_tf32)
      return dispatch_pair_gemm<2, float>(trans_b, epi_tma, bn, tmA, tmB, tmC, p, npairs, stream);
    if (out_dtype == AMOSB_F32)
      return dispatch_pair_gemm<0, float>(trans_b, epi_tma, bn, tmA, tmB, tmC, p, npairs, stream);
    if (out_dtype == AMOSB_F16)
      return dispatch_pair_gemm<0, __half>(trans_b, epi_tma, bn, tmA, tmB, tmC, p, npairs, stream);
    set_error("fp16 GEMM writes float32 or float16");
    return AMOSB_ERR_UNSUPPORTED;
  }

  const int grid = setup_schedule(&p, st, device, st->sm_count, 1,
                                  static_cast<size_t>(mt) * kBlockM * bn, ws, ws_bytes);
  if (is_i8) {
    return dispatch_gemm<1, int32_t>(trans_a, trans_b, epi_tma, bn, tmA, tmB, tmC, p, grid, stream);
  }
  if (is_tf32) {
    return dispatch_gemm<2, float>(trans_a, trans_b, epi_tma, bn, tmA, tmB, tmC, p, grid, stream);
  }
  if (out_dtype == AMOSB_F32)
    return dispatch_gemm<0, float>(trans_a, trans_b, epi_tma, bn, tmA, tmB, tmC, p, grid, stream);
  if (out_dtype == AMOSB_F16)
    return dispatch_gemm<0, __half>(trans_a, trans_b, epi_tma, bn, tmA, tmB, tmC, p, grid, stream);
  set_error("fp16 GEMM writes float32 or float16");
  return AMOSB_ERR_UNSUPPORTED;
}

int run_gemm(const AmosbOpDesc& d, const void* a, const void* b, const void* addend, void* c,
             void* workspace, long long workspace_bytes, int device, cudaStream_t stream) {
  DeviceState* st = nullptr;
  int rc = get_device_state(device, &st);
  if (rc != AMOSB_OK) return rc;
  rc = load_driver_entry_points();
  if (rc != AMOSB_OK) return rc;
  TrailingOps ops;
  rc = trailing_ops_for(d, addend, false, &ops);
  if (rc != AMOSB_OK) return rc;
  return run_gemm_core(st, d.in_dtype, d.out_dtype, d.trans_a != 0, d.trans_b != 0, false,
                       d.batch, d.m, d.n, d.k, d.tile_n, d.cta_pair, ops, a, b, c, workspace,
                       workspace_bytes, device, stream);
}

// --------------------------------------------------------------------------------------------
// conv2d NCHW
// --------------------------------------------------------------------------------------------
static inline long long round_up(long long x, long long m) { return (x + m - 1) / m * m; }

static int conv_elem_bytes(const AmosbOpDesc& d) {
  return d.in_dtype == AMOSB_S8 ? 1 : d.in_dtype == AMOSB_F32 ? 4 : 2;
}

bool conv_is_pointwise_gemm(const AmosbOpDesc& d) {
  // 16-bit tensors only: an int8 plane would have to be cut in 128-pixel chunks
  return conv_elem_bytes(d) == 2 && d.conv_r == 1 && d.conv_s == 1 && d.stride_h == 1 &&
         d.stride_w == 1 && d.pad_h == 0 && d.pad_w == 0 && (d.conv_h * d.conv_w) % 8 == 0 &&
         d.conv_c % 8 == 0 && getenv("AMOSB_CONV_NO_POINTWISE") == nullptr;
}

// The other 1x1 / stride 1 / unpadded layers with 16-bit tensors whose planes are a multiple of 4
// pixels (8 bytes) but not of 8: no tensor map can describe the activation, so it is brought into
// shared memory by cp.async instead (kModeConvPw); the filter and the output need nothing special.
bool conv_is_pointwise_inplace(const AmosbOpDesc& d) {
  return d.kind == AMOSB_OP_CONV2D_NCHW && conv_elem_bytes(d) == 2 && d.conv_r == 1 &&
         d.conv_s == 1 && d.stride_h == 1 && d.stride_w == 1 && d.pad_h == 0 && d.pad_w == 0 &&
         (d.conv_h * d.conv_w) % 4 == 0 && d.conv_c % 8 == 0 && !conv_is_pointwise_gemm(d) &&
         d.cta_pair != 2 && d.cta_pair != 3 &&  // pinned pair / tall tiles: the re-layout path has them
         getenv("AMOSB_CONV_NO_POINTWISE") == nullptr;
}

void conv_workspace_layout(const AmosbOpDesc& d, long long* act_bytes, long long* flt_bytes,
                           int* c_pad8, int* c_pad64) {
  // channels per pixel padded to 16 bytes, channels per filter tap to whole 128-byte k-blocks
  const int es = conv_elem_bytes(d);
  *c_pad8 = (int)round_up(d.conv_c, 16 / es);
  *c_pad64 = (int)round_up(d.conv_c, 128 / es);
  if (conv_is_pointwise_gemm(d) || conv_is_pointwise_inplace(d)) {
    *act_bytes = 0;
    *flt_bytes = 0;
    return;
  }
  *act_bytes = round_up(d.conv_n * d.conv_h * d.conv_w * (long long)(*c_pad8) * es, 1024);
  *flt_bytes = round_up(d.conv_k * d.conv_r * d.conv_s * (long long)(*c_pad64) * es, 1024);
}

// Tile width of the in-place 1x1 kernel: the narrowest of 64 / 128 / 256 that covers K_out, so that
// the activation passes through the copying warps once (measured on the 14x14, C1024 -> K256 layer:
// 128-wide tiles copy it twice and take 1.6x as long).
int pointwise_inplace_tile_n(const AmosbOpDesc& d) {
  if (d.tile_n == 64 || d.tile_n == 128 || d.tile_n == 256) return d.tile_n;
  return d.conv_k > 128 ? 256 : d.conv_k > 64 ? 128 : 64;
}

// float16 NCHW outputs whose planes are whole 4-pixel groups, from an 8-byte aligned address, are
// stored 4 pixels (8 bytes) per lane after a transposition among lanes.  Measured on the 14x14
// 1x1 layer (C1024 -> K256, batch 256): 62 -> 51 us.  32-bit outputs gain nothing from it (a warp's
// element-wise store already fills a 128-byte line: 52 us either way, and 94 against 90 us on a
// layer that writes four times as much), so they keep the element-wise store.
// AMOSB_NCHW_QUADS=0 / 1 turns the transposed store off / on for every element size (tests).
static int nchw_quads_ok(long long pq, const void* out, int out_elem_bytes) {
  const char* force = getenv("AMOSB_NCHW_QUADS");
  if (force != nullptr && force[0] == '0') return 0;
  const bool wanted = out_elem_bytes == 2 || (force != nullptr && force[0] == '1');
  return wanted && pq % 4 == 0 && reinterpret_cast<uintptr_t>(out) % (4 * out_elem_bytes) == 0 ? 1 : 0;
}

static int run_conv2d_pointwise_inplace(DeviceState* st, const AmosbOpDesc& d, const void* act,
                                        const void* flt, const void* addend, void* out, void* ws,
                                        long long ws_bytes, int device, cudaStream_t stream) {
  const long long PQ = d.conv_p * d.conv_q, Mtot = d.conv_n * PQ, C = d.conv_c, Kout = d.conv_k;
  if (Mtot > 0x7fffffffLL || C * PQ * d.conv_n > (1LL << 40)) {
    set_error("conv2d problem too large");
    return AMOSB_ERR_UNSUPPORTED;
  }
  const int bn = pointwise_inplace_tile_n(d);
  CUtensorMap tmA, tmB, tmC;
  memset(&tmA, 0, sizeof(tmA));
  memset(&tmC, 0, sizeof(tmC));
  int rc = encode_tiled_2d(&tmB, tma_dtype_for(d.in_dtype), const_cast<void*>(flt), C, Kout, C * 2,
                           64, bn);
  if (rc != AMOSB_OK) return rc;
  UmmaParams p;
  memset(&p, 0, sizeof(p));
  set_wait_params(&p);
  p.M = (int)Mtot;
  p.N = (int)Kout;
  p.K = (int)C;
  p.batch = 1;
  p.mt = 1;
  p.idesc_formats = idesc_formats_for(d.in_dtype);
  p.tiles_m = (int)((Mtot + kBlockM - 1) / kBlockM);
  p.tiles_n = (int)((Kout + bn - 1) / bn);
  p.group_m = 16;
  p.num_kb = (int)((C + 63) / 64);
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.out = out;
  p.status = st->status_ptr;
  p.P = (int)d.conv_p;
  p.Q = (int)d.conv_q;
  p.PQ = (int)PQ;
  p.nchw_quads = nchw_quads_ok(PQ, out, d.out_dtype == AMOSB_F16 ? 2 : 4);
  p.conv_C = (int)C;
  p.producers = 1;
  p.act = act;
  TrailingOps ops;
  rc = trailing_ops_for(d, addend, false, &ops);
  if (rc != AMOSB_OK) return rc;
  p.epi_flags = ops.flags;
  p.addend_f16 = ops.f16;
  p.addend = ops.addend;
  const int grid = setup_schedule(&p, st, device, st->sm_count, 1,
                                  static_cast<size_t>(kBlockM) * bn, ws, ws_bytes);
  const bool f32 = d.out_dtype == AMOSB_F32;
  if (!f32 && d.out_dtype != AMOSB_F16) {
    set_error("conv2d writes float32 or float16");
    return AMOSB_ERR_UNSUPPORTED;
  }
  switch (bn) {
    case 256:
      return f32 ? launch_umma<0, 256, false, kModeConvPw, float, false, 1, true>(tmA, tmB, tmC, p, grid, stream)
                 : launch_umma<0, 256, false, kModeConvPw, __half, false, 1, true>(tmA, tmB, tmC, p, grid, stream);
    case 128:
      return f32 ? launch_umma<0, 128, false, kModeConvPw, float, false, 1, true>(tmA, tmB, tmC, p, grid, stream)
                 : launch_umma<0, 128, false, kModeConvPw, __half, false, 1, true>(tmA, tmB, tmC, p, grid, stream);
    default:
      return f32 ? launch_umma<0, 64, false, kModeConvPw, float, false, 1, true>(tmA, tmB, tmC, p, grid, stream)
                 : launch_umma<0, 64, false, kModeConvPw, __half, false, 1, true>(tmA, tmB, tmC, p, grid, stream);
  }
}

long long tail_workspace_bytes(const AmosbOpDesc& d) {
  const int sms = 148;
  const bool conv = d.kind == AMOSB_OP_CONV2D_NCHW || d.kind == AMOSB_OP_CONV2D_NHWC ||
                    d.kind == AMOSB_OP_CONV2D_HWNC;
  if (conv && (d.conv_n <= 0 || d.conv_c <= 0 || d.conv_k <= 0 || d.conv_p <= 0 || d.conv_q <= 0 ||
               d.conv_r <= 0 || d.conv_s <= 0))
    return 0;
  if (!conv && (d.m <= 0 || d.n <= 0 || d.k <= 0 || d.batch <= 0)) return 0;
  if (d.kind == AMOSB_OP_CONV2D_NCHW && conv_is_pointwise_inplace(d)) {
    const int bn = pointwise_inplace_tile_n(d);
    const long long m = d.conv_n * d.conv_p * d.conv_q;
    const long long tiles = ((m + kBlockM - 1) / kBlockM) * ((d.conv_k + bn - 1) / bn);
    return tail_scratch_bytes(tiles, (int)((d.conv_c + 63) / 64), false, 1, bn);
  }
  int bn = 0, mt = 1;
  bool pairs = false;
  plan_for_desc(d, sms, &bn, &pairs, &mt);
  const long long rows = (pairs || mt == 2) ? 2 * kBlockM : kBlockM;
  const long long kelems = d.in_dtype == AMOSB_S8 ? 128 : d.in_dtype == AMOSB_F32 ? 32 : 64;
  long long tiles, kb;
  if (d.kind == AMOSB_OP_CONV2D_NCHW && conv_is_pointwise_gemm(d)) {
    const long long pq = d.conv_p * d.conv_q;
    tiles = d.conv_n * ((d.conv_k + rows - 1) / rows) * ((pq + bn - 1) / bn);
    kb = (d.conv_c + kelems - 1) / kelems;
  } else if (conv) {
    long long nimg = d.conv_n;
    if (d.kind == AMOSB_OP_CONV2D_HWNC && nimg > 1) nimg = (nimg + kBlockM - 1) / kBlockM * kBlockM;
    long long m = nimg * d.conv_p * d.conv_q;
    if (d.kind == AMOSB_OP_CONV2D_HWNC && d.conv_n > 1 && d.conv_n <= 64 && d.stride_w == 1 &&
        getenv("AMOSB_HWNC_NO_PACKING") == nullptr) {
      // few images: a 128-row group is several pixels of an output row x the images
      int nbox = 8;
      while (nbox < d.conv_n) nbox *= 2;
      const long long group = kBlockM / nbox;
      m = d.conv_p * ((d.conv_q + group - 1) / group) * kBlockM;
    }
    tiles = ((m + rows - 1) / rows) * ((d.conv_k + bn - 1) / bn);
    kb = d.conv_r * d.conv_s * ((d.conv_c + kelems - 1) / kelems);
  } else {
    tiles = d.batch * ((d.m + rows - 1) / rows) * ((d.n + bn - 1) / bn);
    kb = (d.k + kelems - 1) / kelems;
  }
  if (kb > 0x7fffffffLL) return 0;
  return tail_scratch_bytes(tiles, (int)kb, pairs, mt, bn);
}

int run_conv2d(const AmosbOpDesc& d, const void* act, const void* flt, const void* addend, void* out,
               void* workspace, long long workspace_bytes, int device, cudaStream_t stream) {
  DeviceState* st = nullptr;
  int rc = get_device_state(device, &st);
  if (rc != AMOSB_OK) return rc;
  rc = load_driver_entry_points();
  if (rc != AMOSB_OK) return rc;
  const bool is_tf32 = d.in_dtype == AMOSB_F32, is_i8 = d.in_dtype == AMOSB_S8;
  if (d.in_dtype != AMOSB_F16 && d.in_dtype != AMOSB_BF16 && !is_tf32 && !is_i8) {
    set_error("conv2d supports float16, bfloat16, float32 (tf32) and int8 inputs");
    return AMOSB_ERR_UNSUPPORTED;
  }
  if ((d.in_dtype == AMOSB_BF16 || is_tf32) && d.out_dtype != AMOSB_F32) {
    set_error("bfloat16 and float32 inputs accumulate into and write float32");
    return AMOSB_ERR_UNSUPPORTED;
  }
  if (is_i8 && d.out_dtype != AMOSB_S32) {
    set_error("int8 conv2d writes int32");
    return AMOSB_ERR_UNSUPPORTED;
  }
  if ((is_tf32 || is_i8) && (d.cta_pair == 2 || d.cta_pair == 3)) {
    set_error("cta_pair=%d is not available for float32 (tf32) or int8 conv2d", d.cta_pair);
    return AMOSB_ERR_UNSUPPORTED;
  }
  const int es = conv_elem_bytes(d);
  const int e128 = 128 / es;
  const long long Nimg = d.conv_n, C = d.conv_c, H = d.conv_h, W = d.conv_w;
  const long long Kout = d.conv_k, R = d.conv_r, S = d.conv_s;
  if (Nimg <= 0 || C <= 0 || H <= 0 || W <= 0 || Kout <= 0 || R <= 0 || S <= 0 ||
      d.stride_h <= 0 || d.stride_w <= 0 || d.dil_h <= 0 || d.dil_w <= 0 || d.pad_h < 0 ||
      d.pad_w < 0) {
    set_error("conv2d extents must be positive");
    return AMOSB_ERR_ARG;
  }
  const long long P = (H + 2 * d.pad_h - d.dil_h * (R - 1) - 1) / d.stride_h + 1;
  const long long Q = (W + 2 * d.pad_w - d.dil_w * (S - 1) - 1) / d.stride_w + 1;
  if (P != d.conv_p || Q != d.conv_q || P <= 0 || Q <= 0) {
    set_error("conv2d output extent mismatch: expected %lldx%lld, descriptor says %lldx%lld", P, Q,
              (long long)d.conv_p, (long long)d.conv_q);
    return AMOSB_ERR_ARG;
  }
  // Limits of the im2col tensor map: corner offsets are 8-bit, traversal strides at most 8.
  const int upper_w = d.pad_w - (int)(S - 1) * d.dil_w, upper_h = d.pad_h - (int)(R - 1) * d.dil_h;
  if (d.pad_w > 128 || d.pad_h > 128 || upper_w < -128 || upper_h < -128 || upper_w > 127 ||
      upper_h > 127 || d.stride_w > 8 || d.stride_h > 8 || (S - 1) * d.dil_w > 255 ||
      (R - 1) * d.dil_h > 255) {
    set_error("conv2d geometry outside what an im2col tensor map can express");
    return AMOSB_ERR_UNSUPPORTED;
  }
  // A 1x1, stride-1, unpadded convolution is, per image, Out[n] (K x PQ) = W (K x C) * X[n] (C x PQ)
  // with every matrix already row-major in NCHW/KCRS: a batched GEMM whose A is shared by all
  // images and whose B is consumed MN-major in place.  No re-layout, no scratch.
  if (conv_is_pointwise_gemm(d)) {
    TrailingOps gops;
    rc = trailing_ops_for(d, addend, true, &gops);
    if (rc != AMOSB_OK) return rc;
    return run_gemm_core(st, d.in_dtype, d.out_dtype, false, false, true, Nimg, Kout, P * Q, C, d.tile_n,
                         d.cta_pair, gops, flt, act, out, workspace, workspace_bytes, device, stream);
  }
  if (conv_is_pointwise_inplace(d))
    return run_conv2d_pointwise_inplace(st, d, act, flt, addend, out, workspace, workspace_bytes,
                                        device, stream);
  long long act_bytes, flt_bytes;
  int c_pad8, c_pad64;
  conv_workspace_layout(d, &act_bytes, &flt_bytes, &c_pad8, &c_pad64);
  if (workspace == nullptr || workspace_bytes < act_bytes + flt_bytes) {
    set_error("conv2d needs %lld bytes of workspace, got %lld", act_bytes + flt_bytes,
              workspace_bytes);
    return AMOSB_ERR_ARG;
  }
  if ((reinterpret_cast<uintptr_t>(workspace) & 1023u) != 0) {
    set_error("workspace must be 1024-byte aligned");
    return AMOSB_ERR_ARG;
  }
  const long long Mtot = Nimg * P * Q;
  const long long Kd = R * S * c_pad64;
  if (Mtot > 0x7fffffffLL || Kd > 0x7fffffffLL || Nimg * Kout * P * Q > (1LL << 40)) {
    set_error("conv2d problem too large");
    return AMOSB_ERR_UNSUPPORTED;
  }
  __half* act_nhwc = static_cast<__half*>(workspace);
  __half* flt_krsc = reinterpret_cast<__half*>(static_cast<uint8_t*>(workspace) + act_bytes);

  // 1) re-layout both operands (one launch)
  if (es != 2) {
    const int HW = (int)(H * W);
    const int c_tiles = (c_pad8 + 31) / 32, p_tiles = (HW + 31) / 32;
    const long long act_blocks = Nimg * c_tiles * p_tiles;
    const long long blocks = act_blocks + Kout;
    if (blocks > 0x7fffffffLL) {
      set_error("conv2d problem too large for the re-layout kernel");
      return AMOSB_ERR_UNSUPPORTED;
    }
    if (es == 1) {
      conv_prepack_generic_kernel<int8_t><<<(unsigned)blocks, 256, 0, stream>>>(
          static_cast<const int8_t*>(act), reinterpret_cast<int8_t*>(act_nhwc),
          static_cast<const int8_t*>(flt), reinterpret_cast<int8_t*>(flt_krsc), (int)C, HW, c_pad8,
          (int)act_blocks, c_tiles, p_tiles, (int)(R * S), c_pad64);
    } else {
      conv_prepack_generic_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>(
          static_cast<const float*>(act), reinterpret_cast<float*>(act_nhwc),
          static_cast<const float*>(flt), reinterpret_cast<float*>(flt_krsc), (int)C, HW, c_pad8,
          (int)act_blocks, c_tiles, p_tiles, (int)(R * S), c_pad64);
    }
    AMOSB_CUDA_CHECK(cudaGetLastError());
    ++g_launch_count;
  } else {
    const int HW = (int)(H * W);
    const int RS = (int)(R * S);
    const int c_tiles = (c_pad8 + kPackCT - 1) / kPackCT;
    const int p_tiles = (HW + kPackPT - 1) / kPackPT;
    const long long act_blocks = Nimg * c_tiles * p_tiles;
    // channels of one filter handled per block: as many as fit the shared tile
    int flt_chunk = (kPackSmemHalves / RS) / 8 * 8;
    if (flt_chunk > 1024) flt_chunk = 1024;
    if (flt_chunk < 8) {
      set_error("filter window %lldx%lld is too large for the re-layout kernel", R, S);
      return AMOSB_ERR_UNSUPPORTED;
    }
    const int flt_chunks = (c_pad64 + flt_chunk - 1) / flt_chunk;
    const long long blocks = act_blocks + Kout * flt_chunks;
    if (blocks > 0x7fffffffLL) {
      set_error("conv2d problem too large for the re-layout kernel");
      return AMOSB_ERR_UNSUPPORTED;
    }
    auto pack = conv_prepack_kernel<1>;
    // vector width of the activation reads: every channel plane must start on that alignment
    if (HW % 4 == 0) {
      pack = conv_prepack_kernel<4>;
    } else if (HW % 2 == 0) {
      pack = conv_prepack_kernel<2>;
    } else if (HW <= kPackPT && C % 8 == 0) {
      pack = conv_prepack_kernel<0>;  // small odd planes (7x7): flat 16-byte copies
    }
    pack<<<(unsigned)blocks, 256, 0, stream>>>(
        static_cast<const __half*>(act), act_nhwc, static_cast<const __half*>(flt), flt_krsc, (int)C,
        HW, c_pad8, (int)act_blocks, c_tiles, p_tiles, RS, c_pad64, flt_chunk, flt_chunks);
    AMOSB_CUDA_CHECK(cudaGetLastError());
    ++g_launch_count;
  }

  // 2) implicit GEMM
  int bn = 0, mt = 1;
  bool pairs = false;
  plan_for_desc(d, st->sm_count, &bn, &pairs, &mt);
  CUtensorMap tmA, tmB;
  const int ppc = kBlockM;  // one im2col column of 128 pixels fills an A tile
  rc = encode_im2col_nhwc(&tmA, tma_dtype_for(d.in_dtype), act_nhwc, (int)Nimg, (int)H, (int)W, c_pad8, d.pad_h, d.pad_w,
                          (int)R, (int)S, d.dil_h, d.dil_w, d.stride_h, d.stride_w, ppc, es);
  if (rc != AMOSB_OK) return rc;
  const long long conv_tiles_pair =
      ((Mtot + 2 * kBlockM - 1) / (2 * kBlockM)) * ((Kout + bn - 1) / bn);
  rc = encode_tiled_2d(&tmB, tma_dtype_for(d.in_dtype), flt_krsc, Kd, Kout, Kd * es, e128,
                       pairs ? 64 : bn);
  if (rc != AMOSB_OK) return rc;

  UmmaParams p;
  memset(&p, 0, sizeof(p));
  set_wait_params(&p);
  p.M = (int)Mtot;
  p.N = (int)Kout;
  p.K = (int)Kd;
  p.batch = 1;
  p.mt = mt;
  p.idesc_formats = idesc_formats_for(d.in_dtype);
  p.tiles_m = (int)((Mtot + mt * kBlockM - 1) / (mt * kBlockM));
  p.tiles_n = (int)((Kout + bn - 1) / bn);
  p.group_m = 16;
  p.num_kb = (int)(Kd / e128);
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.out = out;
  p.status = st->status_ptr;
  p.P = (int)P;
  p.Q = (int)Q;
  p.PQ = (int)(P * Q);
  p.nchw_quads = nchw_quads_ok(P * Q, out, d.out_dtype == AMOSB_F16 ? 2 : 4);
  p.c_chunks = c_pad64 / e128;
  p.S = (int)S;
  p.stride_h = d.stride_h;
  p.stride_w = d.stride_w;
  p.pad_h = d.pad_h;
  p.pad_w = d.pad_w;
  p.dil_h = d.dil_h;
  p.dil_w = d.dil_w;
  p.producers = producer_threads();
  {
    TrailingOps cops;
    rc = trailing_ops_for(d, addend, false, &cops);
    if (rc != AMOSB_OK) return rc;
    p.epi_flags = cops.flags;
    p.addend_f16 = cops.f16;
    p.addend = cops.addend;
  }
  // scratch left behind the two re-laid-out operands: partial sums of a shared-out tail
  void* sk_ws = static_cast<uint8_t*>(workspace) + act_bytes + flt_bytes;
  const long long sk_ws_bytes = workspace_bytes - act_bytes - flt_bytes;
  CUtensorMap tmC;
  memset(&tmC, 0, sizeof(tmC));
  if (pairs) {
    p.tiles_m = (int)((Mtot + 2 * kBlockM - 1) / (2 * kBlockM));
    p.num_tiles = (int)conv_tiles_pair;
    const int npairs = setup_schedule(&p, st, device, st->sm_count / 2, 2,
                                      static_cast<size_t>(kBlockM) * bn, sk_ws, sk_ws_bytes);
    if (d.out_dtype == AMOSB_F32)
      return dispatch_pair_bn<0, false, kModeConv, float, false>(bn, tmA, tmB, tmC, p, npairs, stream);
    if (d.out_dtype == AMOSB_F16)
      return dispatch_pair_bn<0, false, kModeConv, __half, false>(bn, tmA, tmB, tmC, p, npairs, stream);
    set_error("conv2d writes float32 or float16");
    return AMOSB_ERR_UNSUPPORTED;
  }
  const int grid = setup_schedule(&p, st, device, st->sm_count, 1,
                                  static_cast<size_t>(mt) * kBlockM * bn, sk_ws, sk_ws_bytes);
  if (is_i8) return dispatch_bn<1, false, kModeConv, int32_t, false>(bn, tmA, tmB, tmC, p, grid, stream);
  if (is_tf32) return dispatch_bn<2, false, kModeConv, float, false>(bn, tmA, tmB, tmC, p, grid, stream);
  if (d.out_dtype == AMOSB_F32)
    return dispatch_bn<0, false, kModeConv, float, false>(bn, tmA, tmB, tmC, p, grid, stream);
  if (d.out_dtype == AMOSB_F16)
    return dispatch_bn<0, false, kModeConv, __half, false>(bn, tmA, tmB, tmC, p, grid, stream);
  set_error("conv2d writes float32 or float16");
  return AMOSB_ERR_UNSUPPORTED;
}

// --------------------------------------------------------------------------------------------
// conv2d NHWC / RSCK: everything is consumed in place.  A = im2col view of the activation, B = the
// filter viewed as a row-major [R*S*C][K] matrix (an MN-major operand), output [N*P*Q][K] row-major.
// --------------------------------------------------------------------------------------------
int run_conv2d_nhwc(const AmosbOpDesc& d, const void* act, const void* flt, const void* addend,
                    void* out, void* workspace, long long workspace_bytes, int device,
                    cudaStream_t stream) {
  // One image in HWNC is the same memory as one image in NHWC, for the activation and the output
  // alike (the reference's benchmark script runs its layers at batch 1 by default).
  if (d.kind == AMOSB_OP_CONV2D_HWNC && d.conv_n == 1) {
    AmosbOpDesc one = d;
    one.kind = AMOSB_OP_CONV2D_NHWC;
    return run_conv2d_nhwc(one, act, flt, addend, out, workspace, workspace_bytes, device, stream);
  }
  DeviceState* st = nullptr;
  int rc = get_device_state(device, &st);
  if (rc != AMOSB_OK) return rc;
  rc = load_driver_entry_points();
  if (rc != AMOSB_OK) return rc;
  const bool is_tf32 = d.in_dtype == AMOSB_F32;  // float32 tensors, multiplied as tf32
  const bool is_i8 = d.in_dtype == AMOSB_S8;
  if (d.in_dtype != AMOSB_F16 && d.in_dtype != AMOSB_BF16 && !is_tf32 && !is_i8) {
    set_error("conv2d supports float16, bfloat16, float32 (tf32) and int8 inputs");
    return AMOSB_ERR_UNSUPPORTED;
  }
  if ((d.in_dtype == AMOSB_BF16 || is_tf32) && d.out_dtype != AMOSB_F32) {
    set_error("bfloat16 and float32 inputs accumulate into and write float32");
    return AMOSB_ERR_UNSUPPORTED;
  }
  if (is_i8 && d.out_dtype != AMOSB_S32) {
    set_error("int8 conv2d writes int32");
    return AMOSB_ERR_UNSUPPORTED;
  }
  // CTA pairs: every element type in both layouts; tall tiles: float16 / bfloat16 only
  if ((is_tf32 || is_i8) && d.cta_pair == 3) {
    set_error("cta_pair=%d is not available for float32 (tf32) or int8 conv2d", d.cta_pair);
    return AMOSB_ERR_UNSUPPORTED;
  }
  const int es = is_tf32 ? 4 : is_i8 ? 1 : 2;
  const int e128 = 128 / es;  // elements per 128-byte k-block row
  const long long Nimg = d.conv_n, C = d.conv_c, H = d.conv_h, W = d.conv_w;
  const long long Kout = d.conv_k, R = d.conv_r, S = d.conv_s;
  if (Nimg <= 0 || C <= 0 || H <= 0 || W <= 0 || Kout <= 0 || R <= 0 || S <= 0 ||
      d.stride_h <= 0 || d.stride_w <= 0 || d.dil_h <= 0 || d.dil_w <= 0 || d.pad_h < 0 ||
      d.pad_w < 0) {
    set_error("conv2d extents must be positive");
    return AMOSB_ERR_ARG;
  }
  const long long P = (H + 2 * d.pad_h - d.dil_h * (R - 1) - 1) / d.stride_h + 1;
  const long long Q = (W + 2 * d.pad_w - d.dil_w * (S - 1) - 1) / d.stride_w + 1;
  if (P != d.conv_p || Q != d.conv_q || P <= 0 || Q <= 0) {
    set_error("conv2d output extent mismatch: expected %lldx%lld, descriptor says %lldx%lld", P, Q,
              (long long)d.conv_p, (long long)d.conv_q);
    return AMOSB_ERR_ARG;
  }
  const int upper_w = d.pad_w - (int)(S - 1) * d.dil_w, upper_h = d.pad_h - (int)(R - 1) * d.dil_h;
  if (d.pad_w > 128 || d.pad_h > 128 || upper_w < -128 || upper_h < -128 || upper_w > 127 ||
      upper_h > 127 || d.stride_w > 8 || d.stride_h > 8 || (S - 1) * d.dil_w > 255 ||
      (R - 1) * d.dil_h > 255) {
    set_error("conv2d geometry outside what an im2col tensor map can express");
    return AMOSB_ERR_UNSUPPORTED;
  }
  const bool hwnc = d.kind == AMOSB_OP_CONV2D_HWNC;
  // HWNC: a tile is one output pixel x 128 images; other image counts are padded per pixel (the
  // padding images load as zeros and are not stored)
  const long long Npad = hwnc ? round_up(Nimg, kBlockM) : Nimg;
  // ... unless there are at most 64 of them and the filter moves one pixel at a time along a row:
  // then a tile is `hw_group` consecutive pixels of an output row x `hw_nbox` images
  // (hw_nbox = 8, 16, 32 or 64, the smallest that holds the images)
  int hw_nbox = kBlockM, hw_group = 1;
  if (hwnc && Nimg <= 64 && d.stride_w == 1 && getenv("AMOSB_HWNC_NO_PACKING") == nullptr) {
    hw_nbox = 8;
    while (hw_nbox < Nimg) hw_nbox *= 2;
    hw_group = kBlockM / hw_nbox;
  }
  if (C % (16 / es) != 0 || Kout % (16 / es) != 0) {
    set_error("NHWC / HWNC conv2d needs C and K to be multiples of %d (16-byte rows for TMA); got "
              "C=%lld K=%lld", 16 / es, C, Kout);
    return AMOSB_ERR_UNSUPPORTED;
  }
  const long long hw_qgroups = (Q + hw_group - 1) / hw_group;
  const long long Mtot = hw_group > 1 ? P * hw_qgroups * kBlockM : Npad * P * Q;
  const long long Kd = R * S * C;
  if (Mtot > 0x7fffffffLL || Kd > 0x7fffffffLL) {
    set_error("conv2d problem too large");
    return AMOSB_ERR_UNSUPPORTED;
  }
  int bn = 0, mt = 1;
  bool pairs = false;
  plan_for_desc(d, st->sm_count, &bn, &pairs, &mt);
  CUtensorMap tmA, tmB, tmC;
  memset(&tmC, 0, sizeof(tmC));
  if (hwnc) {
    rc = encode_tiled_hwnc(&tmA, tma_dtype_for(d.in_dtype), es, const_cast<void*>(act), C, Nimg, W, H,
                           hw_nbox, hw_group);
  } else {
    rc = encode_im2col_nhwc(&tmA, tma_dtype_for(d.in_dtype), const_cast<void*>(act), (int)Nimg, (int)H, (int)W, (int)C, d.pad_h,
                            d.pad_w, (int)R, (int)S, d.dil_h, d.dil_w, d.stride_h, d.stride_w, kBlockM, es);
  }
  if (rc != AMOSB_OK) return rc;
  // the filter is an MN-major operand: 32-bit elements need the 128-byte swizzle with 32-byte units
  rc = encode_tiled_3d(&tmB, tma_dtype_for(d.in_dtype), es, const_cast<void*>(flt), Kout, Kd, 1,
                       Kout * es, Kd * Kout * es, e128, e128,
                       is_tf32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != AMOSB_OK) return rc;
  const int ob = d.out_dtype == AMOSB_F16 ? 2 : 4;
  const bool epi_tma = (Kout * ob) % 16 == 0 && getenv("AMOSB_DIRECT_STORE") == nullptr;
  if (epi_tma) {
    const CUtensorMapDataType odt = d.out_dtype == AMOSB_F16   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                    : d.out_dtype == AMOSB_S32 ? CU_TENSOR_MAP_DATA_TYPE_INT32
                                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    rc = hwnc ? encode_store_hwnc(&tmC, odt, ob, out, Kout, Nimg, Q, P, hw_nbox)
              : encode_tiled_3d(&tmC, odt, ob, out, Kout, Mtot, 1, Kout * ob, Mtot * Kout * ob,
                                128 / ob, 32);
    if (rc != AMOSB_OK) return rc;
  }
  UmmaParams p;
  memset(&p, 0, sizeof(p));
  set_wait_params(&p);
  p.M = (int)Mtot;
  p.N = (int)Kout;
  p.K = (int)Kd;
  p.batch = 1;
  p.mt = mt;
  p.idesc_formats = idesc_formats_for(d.in_dtype);
  p.tiles_m = (int)((Mtot + mt * kBlockM - 1) / (mt * kBlockM));
  p.tiles_n = (int)((Kout + bn - 1) / bn);
  p.group_m = 16;
  p.c_chunks = (int)((C + e128 - 1) / e128);
  p.num_kb = (int)(R * S) * p.c_chunks;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.ldc = Kout;
  p.c_batch_stride = Mtot * Kout;
  p.out = out;
  p.status = st->status_ptr;
  p.P = (int)P;
  p.Q = (int)Q;
  p.PQ = (int)(P * Q);
  p.S = (int)S;
  p.conv_C = (int)C;
  p.conv_N = (int)Npad;
  p.conv_N_real = (int)Nimg;
  p.hw_group = hw_group;
  p.hw_nbox = hw_nbox;
  p.hw_qgroups = (int)hw_qgroups;
  p.stride_h = d.stride_h;
  p.stride_w = d.stride_w;
  p.pad_h = d.pad_h;
  p.pad_w = d.pad_w;
  p.dil_h = d.dil_h;
  p.dil_w = d.dil_w;
  p.producers = producer_threads();
  {
    TrailingOps cops;
    rc = trailing_ops_for(d, addend, false, &cops);
    if (rc != AMOSB_OK) return rc;
    p.epi_flags = cops.flags;
    p.addend_f16 = cops.f16;
    p.addend = cops.addend;
  }
  if (!is_i8 && d.out_dtype != AMOSB_F32 && d.out_dtype != AMOSB_F16) {
    set_error("conv2d writes float32 or float16");
    return AMOSB_ERR_UNSUPPORTED;
  }
  const bool f32 = d.out_dtype == AMOSB_F32;
  if (is_i8 && pairs) {
    p.tiles_m = (int)((Mtot + 2 * kBlockM - 1) / (2 * kBlockM));
    p.num_tiles = (int)(((Mtot + 2 * kBlockM - 1) / (2 * kBlockM)) * ((Kout + bn - 1) / bn));
    const int npairs8 = setup_schedule(&p, st, device, st->sm_count / 2, 2,
                                       static_cast<size_t>(kBlockM) * bn, workspace, workspace_bytes);
    if (hwnc) {
      if (epi_tma) return dispatch_pair_bn<1, true, kModeConvHwnc, int32_t, true>(bn, tmA, tmB, tmC, p, npairs8, stream);
      return dispatch_pair_bn<1, true, kModeConvHwnc, int32_t, false>(bn, tmA, tmB, tmC, p, npairs8, stream);
    }
    if (epi_tma) return dispatch_pair_bn<1, true, kModeConvNhwc, int32_t, true>(bn, tmA, tmB, tmC, p, npairs8, stream);
    return dispatch_pair_bn<1, true, kModeConvNhwc, int32_t, false>(bn, tmA, tmB, tmC, p, npairs8, stream);
  }
  if (is_tf32 && pairs) {
    p.tiles_m = (int)((Mtot + 2 * kBlockM - 1) / (2 * kBlockM));
    p.num_tiles = (int)(((Mtot + 2 * kBlockM - 1) / (2 * kBlockM)) * ((Kout + bn - 1) / bn));
    const int npairs32 = setup_schedule(&p, st, device, st->sm_count / 2, 2,
                                        static_cast<size_t>(kBlockM) * bn, workspace, workspace_bytes);
    if (hwnc) {
      if (epi_tma) return dispatch_pair_bn<2, true, kModeConvHwnc, float, true>(bn, tmA, tmB, tmC, p, npairs32, stream);
      return dispatch_pair_bn<2, true, kModeConvHwnc, float, false>(bn, tmA, tmB, tmC, p, npairs32, stream);
    }
    if (epi_tma) return dispatch_pair_bn<2, true, kModeConvNhwc, float, true>(bn, tmA, tmB, tmC, p, npairs32, stream);
    return dispatch_pair_bn<2, true, kModeConvNhwc, float, false>(bn, tmA, tmB, tmC, p, npairs32, stream);
  }
  if (is_i8) {
    const int grid8 = setup_schedule(&p, st, device, st->sm_count, 1,
                                     static_cast<size_t>(mt) * kBlockM * bn, workspace,
                                     workspace_bytes);
    if (hwnc) {
      if (epi_tma) return dispatch_bn<1, true, kModeConvHwnc, int32_t, true>(bn, tmA, tmB, tmC, p, grid8, stream);
      return dispatch_bn<1, true, kModeConvHwnc, int32_t, false>(bn, tmA, tmB, tmC, p, grid8, stream);
    }
    if (epi_tma) return dispatch_bn<1, true, kModeConvNhwc, int32_t, true>(bn, tmA, tmB, tmC, p, grid8, stream);
    return dispatch_bn<1, true, kModeConvNhwc, int32_t, false>(bn, tmA, tmB, tmC, p, grid8, stream);
  }
  if (pairs) {
    const long long tiles_pair = ((Mtot + 2 * kBlockM - 1) / (2 * kBlockM)) * ((Kout + bn - 1) / bn);
    p.tiles_m = (int)((Mtot + 2 * kBlockM - 1) / (2 * kBlockM));
    p.num_tiles = (int)tiles_pair;
    const int npairs = setup_schedule(&p, st, device, st->sm_count / 2, 2,
                                      static_cast<size_t>(kBlockM) * bn, workspace, workspace_bytes);
    if (hwnc) {
      if (epi_tma) {
        if (f32) return dispatch_pair_bn<0, true, kModeConvHwnc, float, true>(bn, tmA, tmB, tmC, p, npairs, stream);
        return dispatch_pair_bn<0, true, kModeConvHwnc, __half, true>(bn, tmA, tmB, tmC, p, npairs, stream);
      }
      if (f32) return dispatch_pair_bn<0, true, kModeConvHwnc, float, false>(bn, tmA, tmB, tmC, p, npairs, stream);
      return dispatch_pair_bn<0, true, kModeConvHwnc, __half, false>(bn, tmA, tmB, tmC, p, npairs, stream);
    }
    if (epi_tma) {
      if (f32) return dispatch_pair_bn<0, true, kModeConvNhwc, float, true>(bn, tmA, tmB, tmC, p, npairs, stream);
      return dispatch_pair_bn<0, true, kModeConvNhwc, __half, true>(bn, tmA, tmB, tmC, p, npairs, stream);
    }
    if (f32) return dispatch_pair_bn<0, true, kModeConvNhwc, float, false>(bn, tmA, tmB, tmC, p, npairs, stream);
    return dispatch_pair_bn<0, true, kModeConvNhwc, __half, false>(bn, tmA, tmB, tmC, p, npairs, stream);
  }
  const int grid = setup_schedule(&p, st, device, st->sm_count, 1,
                                  static_cast<size_t>(mt) * kBlockM * bn, workspace, workspace_bytes);
  if (is_tf32) {
    if (hwnc) {
      if (epi_tma) return dispatch_bn<2, true, kModeConvHwnc, float, true>(bn, tmA, tmB, tmC, p, grid, stream);
      return dispatch_bn<2, true, kModeConvHwnc, float, false>(bn, tmA, tmB, tmC, p, grid, stream);
    }
    if (epi_tma) return dispatch_bn<2, true, kModeConvNhwc, float, true>(bn, tmA, tmB, tmC, p, grid, stream);
    return dispatch_bn<2, true, kModeConvNhwc, float, false>(bn, tmA, tmB, tmC, p, grid, stream);
  }
  if (hwnc) {
    if (epi_tma) {
      if (f32) return dispatch_bn<0, true, kModeConvHwnc, float, true>(bn, tmA, tmB, tmC, p, grid, stream);
      return dispatch_bn<0, true, kModeConvHwnc, __half, true>(bn, tmA, tmB, tmC, p, grid, stream);
    }
    if (f32) return dispatch_bn<0, true, kModeConvHwnc, float, false>(bn, tmA, tmB, tmC, p, grid, stream);
    return dispatch_bn<0, true, kModeConvHwnc, __half, false>(bn, tmA, tmB, tmC, p, grid, stream);
  }
  if (epi_tma) {
    if (f32) return dispatch_bn<0, true, kModeConvNhwc, float, true>(bn, tmA, tmB, tmC, p, grid, stream);
    return dispatch_bn<0, true, kModeConvNhwc, __half, true>(bn, tmA, tmB, tmC, p, grid, stream);
  }
  if (f32) return dispatch_bn<0, true, kModeConvNhwc, float, false>(bn, tmA, tmB, tmC, p, grid, stream);
  return dispatch_bn<0, true, kModeConvNhwc, __half, false>(bn, tmA, tmB, tmC, p, grid, stream);
}

int status_peek(int device, int clear) {
  DeviceState* st = nullptr;
  int rc = get_device_state(device, &st);
  if (rc != AMOSB_OK) return rc;
  AMOSB_CUDA_CHECK(cudaSetDevice(device));
  AMOSB_CUDA_CHECK(cudaDeviceSynchronize());
  int v = 0;
  AMOSB_CUDA_CHECK(cudaMemcpy(&v, st->status_ptr, sizeof(int), cudaMemcpyDeviceToHost));
  if (clear && v != 0) {
    int zero = 0;
    AMOSB_CUDA_CHECK(cudaMemcpy(st->status_ptr, &zero, sizeof(int), cudaMemcpyHostToDevice));
    // a kernel that gave up may have left flags of the shared-out tail set
    AMOSB_CUDA_CHECK(cudaMemset(st->sk_flags, 0, sizeof(unsigned int) * kSkSlots * kSkCtasMax * 4));
  }
  return v;
}

int* device_status_ptr(int device) {
  DeviceState* st = nullptr;
  if (get_device_state(device, &st) != AMOSB_OK) return nullptr;
  return st->status_ptr;
}

int device_sm_count(int device) {
  DeviceState* st = nullptr;
  if (get_device_state(device, &st) != AMOSB_OK) return -1;
  return st->sm_count;
}

void reset_launch_count() { g_launch_count = 0; }
int launch_count() { return g_launch_count; }
void set_launch_count(int n) { g_launch_count = n; }

}  // namespace amosb
