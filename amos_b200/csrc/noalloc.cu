// conv2d entry point for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to hand it scratch memory: an inference server that
// gave the whole device to its own arena at start-up and forbids further cudaMalloc calls, a
// plugin interface that passes tensors but no allocator, or a latency-critical loop in which the
// implicit device synchronisation of cudaMalloc/cudaFree is not acceptable.  For them the NHWC
// copy of the activation and the re-laid-out filter live in a fixed array that is part of the
// library image, so the call needs nothing but its inputs and its output.
#include "../../include/amosb.h"
#include "host_common.h"

#include <cuda_runtime.h>

#include <mutex>

namespace amosb {

// Room for 1024-byte alignment of the usable part on top of the advertised maximum.
constexpr long long kStaticScratchBytes = AMOSB_STATIC_SCRATCH_BYTES;
constexpr long long kStaticArrayBytes = kStaticScratchBytes + 1024;

// Every GPU whose context loads this library holds one copy of this array until the process
// exits.  In host code the identifier below is only a handle for the runtime's symbol table --
// it is NOT a device address and must never be passed to a kernel; the address that device code
// can use is obtained per device with cudaGetSymbolAddress (see static_scratch_for).
static __device__ __align__(256) unsigned char g_static_scratch[kStaticArrayBytes];

struct StaticScratch {
  bool ready = false;
  unsigned char* base = nullptr;  // device address, rounded up to 1024 bytes
};
static StaticScratch g_scratch[64];
static std::mutex g_scratch_mutex;

// Set-up, once per device: resolve the device address of the array with that device current.
static int static_scratch_for(int device, unsigned char** out) {
  if (device < 0 || device >= 64) {
    set_error("device id %d out of range", device);
    return AMOSB_ERR_ARG;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  StaticScratch& s = g_scratch[device];
  if (!s.ready) {
    AMOSB_CUDA_CHECK(cudaSetDevice(device));
    void* ptr = nullptr;
    AMOSB_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (ptr == nullptr) {
      set_error("cudaGetSymbolAddress returned a null address for the static scratch array");
      return AMOSB_ERR_CUDA;
    }
    const uintptr_t addr = reinterpret_cast<uintptr_t>(ptr);
    s.base = reinterpret_cast<unsigned char*>((addr + 1023u) & ~static_cast<uintptr_t>(1023u));
    s.ready = true;
  }
  *out = s.base;
  return AMOSB_OK;
}

}  // namespace amosb

using namespace amosb;

extern "C" int amosb_conv2d_nchw_static(const AmosbOpDesc* desc, const AmosbTensor* ins, int n_in,
                                        AmosbTensor* outs, int n_out, void* cuda_stream) {
  if (desc == nullptr || ins == nullptr || outs == nullptr) {
    set_error("NULL descriptor or tensor list");
    return AMOSB_ERR_ARG;
  }
  if (desc->kind != AMOSB_OP_CONV2D_NCHW) {
    set_error("amosb_conv2d_nchw_static runs conv2d descriptors only (kind %d given)", desc->kind);
    return AMOSB_ERR_ARG;
  }
  if (n_in < 2 || n_in > 3 || n_out != 1) {
    set_error("expected 2 or 3 inputs and 1 output, got %d inputs and %d outputs", n_in, n_out);
    return AMOSB_ERR_ARG;
  }
  // what the call cannot do without (the re-laid-out operands); if the array has room left for the
  // optional part of the scratch, amosb_run uses it
  const int64_t need = amosb_workspace_bytes_min(desc);
  if (need < 0) return static_cast<int>(need);
  if (need > kStaticScratchBytes) {
    set_error("this conv2d needs %lld bytes of scratch but the built-in scratch holds %lld "
              "(AMOSB_STATIC_SCRATCH_BYTES); use amosb_run with a caller-provided workspace",
              (long long)need, (long long)kStaticScratchBytes);
    return AMOSB_ERR_UNSUPPORTED;
  }
  // Same argument checks as amosb_run, done here so that nothing is launched on a bad call.
  if (desc->arg_a < 0 || desc->arg_a >= n_in) {
    set_error("descriptor operand order (arg_a=%d) is invalid", desc->arg_a);
    return AMOSB_ERR_ARG;
  }
  const int device = ins[desc->arg_a].device_id;
  unsigned char* scratch = nullptr;
  int rc = static_scratch_for(device, &scratch);
  if (rc != AMOSB_OK) return rc;
  // amosb_run validates shapes, dtypes, strides, alignment and devices, then launches with the
  // workspace it is given: here, the device address of the built-in array.
  return amosb_run(desc, ins, n_in, outs, n_out, scratch, kStaticScratchBytes, cuda_stream);
}
