// Shared host-side helpers: thread-local error message, CUDA error check, internal entry points.
#pragma once
#include "../../include/amosb.h"

#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

namespace amosb {

// Host-side NVTX range around an entry point (a no-op costing a pointer test unless a tool such as
// Nsight Systems has attached itself to the process).
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

// printf-style; stores the message returned by amosb_last_error() on this thread.
void set_error(const char* fmt, ...) __attribute__((format(printf, 1, 2)));
const char* last_error();

#define AMOSB_CUDA_CHECK(expr)                                                              \
  do {                                                                                      \
    cudaError_t _e = (expr);                                                                \
    if (_e != cudaSuccess) {                                                                \
      ::amosb::set_error("CUDA error %d (%s) at %s:%d: %s", (int)_e, cudaGetErrorName(_e),  \
                         __FILE__, __LINE__, cudaGetErrorString(_e));                       \
      return AMOSB_ERR_CUDA;                                                                \
    }                                                                                       \
  } while (0)

// launch.cu
int run_gemm(const AmosbOpDesc& d, const void* a, const void* b, const void* addend, void* c,
             void* workspace, long long workspace_bytes, int device, cudaStream_t stream);
int run_conv2d(const AmosbOpDesc& d, const void* act, const void* flt, const void* addend, void* out,
               void* workspace, long long workspace_bytes, int device, cudaStream_t stream);
int run_conv2d_nhwc(const AmosbOpDesc& d, const void* act, const void* flt, const void* addend,
                    void* out, void* workspace, long long workspace_bytes, int device,
                    cudaStream_t stream);
// scratch the shared-out tail of `d`'s schedule wants on a full B200 (0: the tail is not shared out)
long long tail_workspace_bytes(const AmosbOpDesc& d);
void conv_workspace_layout(const AmosbOpDesc& d, long long* act_bytes, long long* flt_bytes,
                           int* c_pad8, int* c_pad64);
int choose_tile_n(const AmosbOpDesc& d, int sm_count);
int choose_tile_rows(const AmosbOpDesc& d, int sm_count);  // 128, or 256 for pairs and tall tiles
bool choose_cta_pairs(const AmosbOpDesc& d, int sm_count);
bool conv_is_pointwise_gemm(const AmosbOpDesc& d);
bool conv_is_pointwise_inplace(const AmosbOpDesc& d);
int pointwise_inplace_tile_n(const AmosbOpDesc& d);
int status_peek(int device, int clear);
int* device_status_ptr(int device);  // device address of the status word, or nullptr
int device_sm_count(int device);
void reset_launch_count();
int launch_count();
void set_launch_count(int n);

// recognize.cc
int recognize(const char* text, AmosbOpDesc* out);

}  // namespace amosb
