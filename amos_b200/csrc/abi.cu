// extern "C" entry points of libamosb: argument checks in the manner of the host function that the
// reference generates around its kernels (reference: src/tir/transforms/make_packed_api.cc:107-198,
// src/tir/transforms/arg_binder.cc:150-299), then hand-off to the launchers.
#include "../../include/amosb.h"
#include "host_common.h"

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

namespace amosb {

static thread_local char g_error[1024] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_error; }

static const char* dtype_name(int dt) {
  switch (dt) {
    case AMOSB_F16:
      return "float16";
    case AMOSB_F32:
      return "float32";
    case AMOSB_S8:
      return "int8";
    case AMOSB_S32:
      return "int32";
    case AMOSB_BF16:
      return "bfloat16";
    default:
      return "?";
  }
}
static int dtype_bytes(int dt) {
  switch (dt) {
    case AMOSB_F16:
      return 2;
    case AMOSB_F32:
      return 4;
    case AMOSB_S8:
      return 1;
    case AMOSB_S32:
      return 4;
    case AMOSB_BF16:
      return 2;
    default:
      return 0;
  }
}

struct Expect {
  int ndim;
  int64_t shape[4];
  int dtype;
};

// Expected signature (inputs in argument order, then the output) for a descriptor.
static int expected_args(const AmosbOpDesc& d, Expect* a, Expect* b, Expect* c) {
  switch (d.kind) {
    case AMOSB_OP_GEMM:
      *a = {2, {d.m, d.k, 0, 0}, d.in_dtype};
      if (d.trans_a) *a = {2, {d.k, d.m, 0, 0}, d.in_dtype};
      *b = {2, {d.k, d.n, 0, 0}, d.in_dtype};
      if (d.trans_b) *b = {2, {d.n, d.k, 0, 0}, d.in_dtype};
      *c = {2, {d.m, d.n, 0, 0}, d.out_dtype};
      return AMOSB_OK;
    case AMOSB_OP_BATCHED_GEMM:
      *a = {3, {d.batch, d.m, d.k, 0}, d.in_dtype};
      if (d.trans_a) *a = {3, {d.batch, d.k, d.m, 0}, d.in_dtype};
      *b = {3, {d.batch, d.k, d.n, 0}, d.in_dtype};
      if (d.trans_b) *b = {3, {d.batch, d.n, d.k, 0}, d.in_dtype};
      *c = {3, {d.batch, d.m, d.n, 0}, d.out_dtype};
      return AMOSB_OK;
    case AMOSB_OP_CONV2D_NCHW:
      *a = {4, {d.conv_n, d.conv_c, d.conv_h, d.conv_w}, d.in_dtype};
      *b = {4, {d.conv_k, d.conv_c, d.conv_r, d.conv_s}, d.in_dtype};
      *c = {4, {d.conv_n, d.conv_k, d.conv_p, d.conv_q}, d.out_dtype};
      return AMOSB_OK;
    case AMOSB_OP_CONV2D_NHWC:
      *a = {4, {d.conv_n, d.conv_h, d.conv_w, d.conv_c}, d.in_dtype};
      *b = {4, {d.conv_r, d.conv_s, d.conv_c, d.conv_k}, d.in_dtype};
      *c = {4, {d.conv_n, d.conv_p, d.conv_q, d.conv_k}, d.out_dtype};
      return AMOSB_OK;
    case AMOSB_OP_CONV2D_HWNC:
      *a = {4, {d.conv_h, d.conv_w, d.conv_n, d.conv_c}, d.in_dtype};
      *b = {4, {d.conv_r, d.conv_s, d.conv_c, d.conv_k}, d.in_dtype};
      *c = {4, {d.conv_p, d.conv_q, d.conv_n, d.conv_k}, d.out_dtype};
      return AMOSB_OK;
    default:
      set_error("descriptor has no operator kind (%d)", d.kind);
      return AMOSB_ERR_ARG;
  }
}

static int check_tensor(const AmosbTensor& t, const Expect& e, const char* name, bool on_device) {
  if (t.data == nullptr) {
    set_error("Argument %s: data pointer is NULL", name);
    return AMOSB_ERR_ARG;
  }
  if (t.ndim != e.ndim) {
    set_error("%s.ndim is expected to equal %d, got %d", name, e.ndim, t.ndim);
    return AMOSB_ERR_ARG;
  }
  if (t.dtype != e.dtype) {
    set_error("%s.dtype is expected to be %s, got %s", name, dtype_name(e.dtype),
              dtype_name(t.dtype));
    return AMOSB_ERR_ARG;
  }
  if (t.shape == nullptr) {
    set_error("Argument %s: shape pointer is NULL", name);
    return AMOSB_ERR_ARG;
  }
  for (int i = 0; i < e.ndim; ++i) {
    if (t.shape[i] != e.shape[i]) {
      set_error("Argument %s.shape[%d] has an unsatisfied constraint: expected %lld, got %lld",
                name, i, (long long)e.shape[i], (long long)t.shape[i]);
      return AMOSB_ERR_ARG;
    }
  }
  if (t.strides != nullptr) {
    int64_t expect = 1;
    for (int i = e.ndim - 1; i >= 0; --i) {
      if (t.shape[i] != 1 && t.strides[i] != expect) {
        set_error("%s.strides: expected to be compact array", name);
        return AMOSB_ERR_ARG;
      }
      expect *= t.shape[i];
    }
  }
  if (on_device) {
    const uintptr_t addr = reinterpret_cast<uintptr_t>(t.data) + t.byte_offset;
    if (addr % 16 != 0) {
      set_error("Argument %s: data + byte_offset must be 16-byte aligned", name);
      return AMOSB_ERR_ARG;
    }
  }
  return AMOSB_OK;
}

// A tensor handed to amosb_run is encoded into a tensor map and read by the copy engine: a host
// pointer or a pointer into another GPU's memory would fault the context.  The reference's generated
// host function asserts device_type for the same reason (reference:
// src/tir/transforms/arg_binder.cc:285-286); AmosbTensor has no such field, so the runtime is asked.
static int check_residency(const AmosbTensor& t, const char* name) {
  cudaPointerAttributes attr;
  const void* p = static_cast<const uint8_t*>(t.data) + t.byte_offset;
  cudaError_t e = cudaPointerGetAttributes(&attr, p);
  if (e != cudaSuccess) {
    cudaGetLastError();  // not sticky: leave the runtime's error state clean
    set_error("CUDA error %d (%s): cannot query the memory of argument %s", (int)e,
              cudaGetErrorName(e), name);
    return AMOSB_ERR_CUDA;
  }
  const bool on_gpu = attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
  if (!on_gpu) {
    set_error("Argument %s.device_type is expected to be cuda: data is %s memory", name,
              attr.type == cudaMemoryTypeHost ? "pinned host" : "pageable host");
    return AMOSB_ERR_ARG;
  }
  if (attr.type == cudaMemoryTypeDevice && attr.device != t.device_id) {
    set_error("Argument %s: data lives on device %d, device_id says %d", name, attr.device,
              t.device_id);
    return AMOSB_ERR_ARG;
  }
  return AMOSB_OK;
}

static inline void* tensor_ptr(const AmosbTensor& t) {
  return static_cast<uint8_t*>(t.data) + t.byte_offset;
}

static int validate_call(const AmosbOpDesc* desc, const AmosbTensor* ins, int n_in,
                         AmosbTensor* outs, int n_out, bool on_device, const AmosbTensor** pa,
                         const AmosbTensor** pb, const AmosbTensor** pc = nullptr) {
  if (desc == nullptr || ins == nullptr || outs == nullptr) {
    set_error("NULL descriptor or tensor list");
    return AMOSB_ERR_ARG;
  }
  const bool has_addend =
      (desc->epilogue & (AMOSB_EPI_ADD_VECTOR | AMOSB_EPI_ADD_FULL)) != 0;
  const int want_in = has_addend ? 3 : 2;
  if (n_in != want_in || n_out != 1) {
    set_error("expected %d arguments (%d inputs, 1 output), got %d inputs and %d outputs",
              want_in + 1, want_in, n_in, n_out);
    return AMOSB_ERR_ARG;
  }
  bool order_ok = desc->arg_a >= 0 && desc->arg_a < want_in && desc->arg_b >= 0 &&
                  desc->arg_b < want_in && desc->arg_a != desc->arg_b;
  if (has_addend)
    order_ok = order_ok && desc->arg_c >= 0 && desc->arg_c < 3 && desc->arg_c != desc->arg_a &&
               desc->arg_c != desc->arg_b;
  if (!order_ok) {
    set_error("descriptor operand order (arg_a=%d, arg_b=%d, arg_c=%d) is invalid", desc->arg_a,
              desc->arg_b, desc->arg_c);
    return AMOSB_ERR_ARG;
  }
  Expect ea, eb, ec;
  int rc = expected_args(*desc, &ea, &eb, &ec);
  if (rc != AMOSB_OK) return rc;
  const AmosbTensor& A = ins[desc->arg_a];
  const AmosbTensor& B = ins[desc->arg_b];
  static const char* const names[4] = {"arg0", "arg1", "arg2", "arg3"};
  if ((rc = check_tensor(A, ea, names[desc->arg_a], on_device)) != AMOSB_OK) return rc;
  if ((rc = check_tensor(B, eb, names[desc->arg_b], on_device)) != AMOSB_OK) return rc;
  if ((rc = check_tensor(outs[0], ec, names[want_in], on_device)) != AMOSB_OK) return rc;
  if (on_device && (A.device_id != B.device_id || A.device_id != outs[0].device_id)) {
    set_error("Argument device_id mismatch: all tensors must be on one device (%d, %d, %d)",
              ins[0].device_id, ins[1].device_id, outs[0].device_id);
    return AMOSB_ERR_ARG;
  }
  if (on_device) {
    if ((rc = check_residency(A, names[desc->arg_a])) != AMOSB_OK) return rc;
    if ((rc = check_residency(B, names[desc->arg_b])) != AMOSB_OK) return rc;
    if ((rc = check_residency(outs[0], names[want_in])) != AMOSB_OK) return rc;
  }
  if (has_addend) {
    const AmosbTensor& D = ins[desc->arg_c];
    Expect ed = ec;
    ed.dtype = desc->addend_dtype;
    if (desc->epilogue & AMOSB_EPI_ADD_VECTOR) {
      const bool is_conv =
          desc->kind == AMOSB_OP_CONV2D_NCHW || desc->kind == AMOSB_OP_CONV2D_NHWC ||
          desc->kind == AMOSB_OP_CONV2D_HWNC;
      const int64_t n_axis = is_conv ? desc->conv_k : desc->n;
      ed = {1, {n_axis, 0, 0, 0}, desc->addend_dtype};
    }
    if ((rc = check_tensor(D, ed, names[desc->arg_c], on_device)) != AMOSB_OK) return rc;
    if (on_device && D.device_id != A.device_id) {
      set_error("Argument device_id mismatch: all tensors must be on one device");
      return AMOSB_ERR_ARG;
    }
    if (on_device && (rc = check_residency(D, names[desc->arg_c])) != AMOSB_OK) return rc;
    if (pc) *pc = &D;
  } else if (pc) {
    *pc = nullptr;
  }
  *pa = &A;
  *pb = &B;
  return AMOSB_OK;
}

static int64_t numel(const AmosbTensor& t) {
  int64_t n = 1;
  for (int i = 0; i < t.ndim; ++i) n *= t.shape[i];
  return n;
}

}  // namespace amosb

using namespace amosb;

extern "C" {

int amosb_version(void) { return 100; }

const char* amosb_last_error(void) { return last_error(); }

int amosb_recognize(const char* te_dag, AmosbOpDesc* out) {
  if (te_dag == nullptr || out == nullptr) {
    set_error("NULL argument");
    return AMOSB_ERR_ARG;
  }
  return recognize(te_dag, out);
}

int64_t amosb_workspace_bytes(const AmosbOpDesc* desc) {
  if (desc == nullptr) {
    set_error("NULL descriptor");
    return AMOSB_ERR_ARG;
  }
  if (desc->kind == AMOSB_OP_CONV2D_NCHW) {
    if (desc->conv_n <= 0 || desc->conv_c <= 0 || desc->conv_h <= 0 || desc->conv_w <= 0 ||
        desc->conv_k <= 0 || desc->conv_r <= 0 || desc->conv_s <= 0) {
      set_error("conv2d extents must be positive");
      return AMOSB_ERR_ARG;
    }
    long long act, flt;
    int c8, c64;
    conv_workspace_layout(*desc, &act, &flt, &c8, &c64);
    return act + flt + tail_workspace_bytes(*desc);
  }
  if (desc->kind == AMOSB_OP_GEMM || desc->kind == AMOSB_OP_BATCHED_GEMM ||
      desc->kind == AMOSB_OP_CONV2D_NHWC || desc->kind == AMOSB_OP_CONV2D_HWNC)
    return tail_workspace_bytes(*desc);
  set_error("descriptor has no operator kind (%d)", desc->kind);
  return AMOSB_ERR_ARG;
}

int64_t amosb_workspace_bytes_min(const AmosbOpDesc* desc) {
  if (desc == nullptr) {
    set_error("NULL descriptor");
    return AMOSB_ERR_ARG;
  }
  const int64_t all = amosb_workspace_bytes(desc);
  if (all < 0) return all;
  return all - tail_workspace_bytes(*desc);
}

int amosb_run(const AmosbOpDesc* desc, const AmosbTensor* ins, int n_in, AmosbTensor* outs,
              int n_out, void* workspace, int64_t workspace_bytes, void* cuda_stream) {
  NvtxRange range("amosb_run");
  const AmosbTensor *A = nullptr, *B = nullptr, *D = nullptr;
  int rc = validate_call(desc, ins, n_in, outs, n_out, true, &A, &B, &D);
  if (rc != AMOSB_OK) return rc;
  const void* addend = D ? tensor_ptr(*D) : nullptr;
  const int device = A->device_id;
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) {
    set_error("cudaSetDevice(%d) failed: %s", device, cudaGetErrorString(e));
    return AMOSB_ERR_CUDA;
  }
  reset_launch_count();
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (desc->kind == AMOSB_OP_CONV2D_NHWC || desc->kind == AMOSB_OP_CONV2D_HWNC) {
    return run_conv2d_nhwc(*desc, tensor_ptr(*A), tensor_ptr(*B), addend, tensor_ptr(outs[0]),
                           workspace, workspace_bytes, device, stream);
  }
  if (desc->kind == AMOSB_OP_CONV2D_NCHW) {
    return run_conv2d(*desc, tensor_ptr(*A), tensor_ptr(*B), addend, tensor_ptr(outs[0]),
                      workspace, workspace_bytes, device, stream);
  }
  return run_gemm(*desc, tensor_ptr(*A), tensor_ptr(*B), addend, tensor_ptr(outs[0]), workspace,
                  workspace_bytes, device, stream);
}

// Device buffers of the host-buffer path, kept per device and grown on demand so that repeated
// calls do not pay for cudaMalloc/cudaFree.
struct HostPathArena {
  // slots: inputs 0..2, output, workspace
  void* buf[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
  size_t cap[5] = {0, 0, 0, 0, 0};
};
static HostPathArena g_arena[64];
static std::mutex g_arena_mutex[64];  // one per device: calls on different GPUs do not serialise

static int arena_reserve(HostPathArena& ar, int slot, size_t bytes) {
  if (bytes == 0) bytes = 16;
  if (ar.cap[slot] >= bytes) return AMOSB_OK;
  if (ar.buf[slot]) cudaFree(ar.buf[slot]);
  ar.buf[slot] = nullptr;
  ar.cap[slot] = 0;
  cudaError_t e = cudaMalloc(&ar.buf[slot], bytes);
  if (e != cudaSuccess) {
    set_error("cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    return AMOSB_ERR_CUDA;
  }
  ar.cap[slot] = bytes;
  return AMOSB_OK;
}

// Streams and events of the pipelined host-buffer path, one set per device, made on first use.
struct HostPathStreams {
  static constexpr int kMaxChunks = 8;
  bool ready = false;
  cudaStream_t in = nullptr, compute = nullptr, out = nullptr;
  cudaEvent_t arrived[kMaxChunks], computed[kMaxChunks];
  int* status_host = nullptr;  // pinned landing place of the device's status word
};
static HostPathStreams g_host_streams[64];

static int host_streams(int device, HostPathStreams** out) {
  HostPathStreams& hs = g_host_streams[device];
  if (!hs.ready) {
    AMOSB_CUDA_CHECK(cudaStreamCreateWithFlags(&hs.in, cudaStreamNonBlocking));
    AMOSB_CUDA_CHECK(cudaStreamCreateWithFlags(&hs.compute, cudaStreamNonBlocking));
    AMOSB_CUDA_CHECK(cudaStreamCreateWithFlags(&hs.out, cudaStreamNonBlocking));
    for (int i = 0; i < HostPathStreams::kMaxChunks; ++i) {
      AMOSB_CUDA_CHECK(cudaEventCreateWithFlags(&hs.arrived[i], cudaEventDisableTiming));
      AMOSB_CUDA_CHECK(cudaEventCreateWithFlags(&hs.computed[i], cudaEventDisableTiming));
    }
    AMOSB_CUDA_CHECK(cudaHostAlloc(&hs.status_host, sizeof(int), cudaHostAllocDefault));
    *hs.status_host = 0;
    hs.ready = true;
  }
  *out = &hs;
  return AMOSB_OK;
}

// How many slices of the operator's independent axis (rows of M, batches, images -- dimension 0 of
// the sliced tensors) the host-buffer path works through: one per ~12 MB crossing the bus, so that
// the copy-in of slice i+1, the kernels of slice i and the copy-out of slice i-1 overlap.
static int host_chunks(const AmosbOpDesc& d, int64_t units, size_t sliced_bytes) {
  if (d.kind == AMOSB_OP_CONV2D_HWNC) return 1;           // images are not the outermost axis
  if (d.kind == AMOSB_OP_GEMM && d.trans_a) return 1;     // rows of M are columns of A[K,M]
  int n = (int)(sliced_bytes / (12u << 20));
  if (const char* e = getenv("AMOSB_HOST_CHUNKS")) n = atoi(e);
  if (n > HostPathStreams::kMaxChunks) n = HostPathStreams::kMaxChunks;
  if (n > units) n = (int)units;
  return n < 1 ? 1 : n;
}

int amosb_run_host(const AmosbOpDesc* desc, const AmosbTensor* ins, int n_in, AmosbTensor* outs,
                   int n_out, int device) {
  NvtxRange range("amosb_run_host");
  const AmosbTensor *A = nullptr, *B = nullptr, *D = nullptr;
  int rc = validate_call(desc, ins, n_in, outs, n_out, false, &A, &B, &D);
  if (rc != AMOSB_OK) return rc;
  if (device < 0 || device >= 64) {
    set_error("device id %d out of range", device);
    return AMOSB_ERR_ARG;
  }
  AMOSB_CUDA_CHECK(cudaSetDevice(device));
  const int64_t ws_bytes = amosb_workspace_bytes(desc);
  if (ws_bytes < 0) return (int)ws_bytes;
  std::lock_guard<std::mutex> lock(g_arena_mutex[device]);
  HostPathArena& ar = g_arena[device];
  size_t in_bytes[3] = {0, 0, 0};
  for (int i = 0; i < n_in; ++i) {
    in_bytes[i] = (size_t)numel(ins[i]) * dtype_bytes(ins[i].dtype);
    if ((rc = arena_reserve(ar, i, in_bytes[i])) != AMOSB_OK) return rc;
  }
  const size_t out_bytes = (size_t)numel(outs[0]) * dtype_bytes(outs[0].dtype);
  if ((rc = arena_reserve(ar, 3, out_bytes)) != AMOSB_OK) return rc;
  // the workspace must start on a 1024-byte boundary, which small allocations do not promise
  if (ws_bytes > 0 && (rc = arena_reserve(ar, 4, (size_t)ws_bytes + 1024)) != AMOSB_OK) return rc;
  void* ws_ptr = ws_bytes > 0 ? reinterpret_cast<void*>(
                                    (reinterpret_cast<uintptr_t>(ar.buf[4]) + 1023) & ~uintptr_t(1023))
                              : nullptr;

  // Tensors that are cut along dimension 0 with the operator's independent axis: A, the output,
  // both operands of a batched GEMM, a full-shape addend.  The rest (B, the filter, a vector
  // addend) goes in whole, first.
  bool sliced[3] = {false, false, false};
  for (int i = 0; i < n_in; ++i) {
    sliced[i] = (&ins[i] == A) || (&ins[i] == B && desc->kind == AMOSB_OP_BATCHED_GEMM) ||
                (&ins[i] == D && (desc->epilogue & AMOSB_EPI_ADD_FULL));
  }
  const int64_t units = outs[0].shape[0];
  size_t sliced_bytes = out_bytes;
  for (int i = 0; i < n_in; ++i)
    if (sliced[i]) sliced_bytes += in_bytes[i];
  const int chunks = host_chunks(*desc, units, sliced_bytes);
  HostPathStreams* hs = nullptr;
  if ((rc = host_streams(device, &hs)) != AMOSB_OK) return rc;
  // GEMM rows are cut at multiples of the tallest tile so that no slice ends in a ragged tile
  const int64_t align = desc->kind == AMOSB_OP_GEMM ? 256 : 1;
  int64_t per = (units + chunks - 1) / chunks;
  per = (per + align - 1) / align * align;
  // every slice must start on an aligned address in every sliced tensor; else one slice
  for (int i = 0; i < n_in; ++i)
    if (sliced[i] && ((size_t)per * (in_bytes[i] / (size_t)units)) % 256 != 0) per = units;
  if (((size_t)per * (out_bytes / (size_t)units)) % 256 != 0) per = units;
  const bool piped = per < units;

  for (int i = 0; i < n_in; ++i) {
    if (sliced[i] && piped) continue;
    AMOSB_CUDA_CHECK(cudaMemcpyAsync(ar.buf[i], tensor_ptr(ins[i]), in_bytes[i],
                                     cudaMemcpyHostToDevice, hs->in));
  }
  int launches = 0;
  int slice = 0;
  for (int64_t u0 = 0; u0 < units; u0 += per, ++slice) {
    const int64_t cnt = units - u0 < per ? units - u0 : per;
    AmosbOpDesc dd = *desc;
    if (!piped) {
      // one slice: the operator as given
    } else if (desc->kind == AMOSB_OP_GEMM) {
      dd.m = cnt;
    } else if (desc->kind == AMOSB_OP_BATCHED_GEMM) {
      dd.batch = cnt;
    } else {
      dd.conv_n = cnt;
    }
    int64_t shapes[4][8];
    AmosbTensor din[3];
    AmosbTensor dout[1] = {outs[0]};
    for (int i = 0; i < n_in; ++i) {
      din[i] = ins[i];
      din[i].byte_offset = 0;
      din[i].device_id = device;
      din[i].strides = nullptr;
      din[i].data = ar.buf[i];
      if (!sliced[i] || !piped) continue;
      const size_t unit_bytes = in_bytes[i] / (size_t)units;
      for (int k = 0; k < ins[i].ndim; ++k) shapes[i][k] = ins[i].shape[k];
      shapes[i][0] = cnt;
      din[i].shape = shapes[i];
      din[i].data = static_cast<uint8_t*>(ar.buf[i]) + (size_t)u0 * unit_bytes;
      AMOSB_CUDA_CHECK(cudaMemcpyAsync(
          din[i].data, static_cast<const uint8_t*>(tensor_ptr(ins[i])) + (size_t)u0 * unit_bytes,
          (size_t)cnt * unit_bytes, cudaMemcpyHostToDevice, hs->in));
    }
    const size_t out_unit = out_bytes / (size_t)units;
    for (int k = 0; k < outs[0].ndim; ++k) shapes[3][k] = outs[0].shape[k];
    if (piped) shapes[3][0] = cnt;
    dout[0].shape = shapes[3];
    dout[0].strides = nullptr;
    dout[0].byte_offset = 0;
    dout[0].device_id = device;
    dout[0].data = static_cast<uint8_t*>(ar.buf[3]) + (size_t)u0 * out_unit;
    AMOSB_CUDA_CHECK(cudaEventRecord(hs->arrived[slice], hs->in));
    AMOSB_CUDA_CHECK(cudaStreamWaitEvent(hs->compute, hs->arrived[slice], 0));
    // slices run one after another on one stream, so they can share the workspace
    rc = amosb_run(&dd, din, n_in, dout, 1, ws_ptr, ws_bytes, hs->compute);
    if (rc != AMOSB_OK) {
      cudaDeviceSynchronize();  // copies already queued still name the caller's buffers
      return rc;
    }
    launches += launch_count();
    AMOSB_CUDA_CHECK(cudaEventRecord(hs->computed[slice], hs->compute));
    AMOSB_CUDA_CHECK(cudaStreamWaitEvent(hs->out, hs->computed[slice], 0));
    AMOSB_CUDA_CHECK(cudaMemcpyAsync(static_cast<uint8_t*>(tensor_ptr(outs[0])) + (size_t)u0 * out_unit,
                                     dout[0].data, (size_t)cnt * out_unit, cudaMemcpyDeviceToHost,
                                     hs->out));
  }
  // the status word follows the last output copy, so the caller never gets numbers from a kernel
  // that gave up a wait together with a success code
  int* status_dev = device_status_ptr(device);
  if (status_dev != nullptr) {
    AMOSB_CUDA_CHECK(cudaMemcpyAsync(hs->status_host, status_dev, sizeof(int),
                                     cudaMemcpyDeviceToHost, hs->out));
  }
  AMOSB_CUDA_CHECK(cudaStreamSynchronize(hs->out));
  set_launch_count(launches);
  if (status_dev != nullptr && *hs->status_host != 0) {
    const int code = *hs->status_host;
    *hs->status_host = 0;
    status_peek(device, 1);  // clear the word for the next call
    set_error("a device-side wait ran out (status %d): the output is not valid", code);
    return AMOSB_ERR_DEVICE_TIMEOUT;
  }
  return AMOSB_OK;
}

int amosb_status_peek(int device, int clear) { return status_peek(device, clear); }

int amosb_sync_check(int device) {
  const int v = status_peek(device, 1);
  if (v < 0) return v;  // the peek itself failed; its message stands
  if (v != 0) {
    set_error("a device-side wait ran out (status %d: %s); results of kernels launched since the "
              "last check are not valid",
              v,
              v == 101   ? "a copy-issuing thread waited for a free stage"
              : v == 102 ? "the MMA thread waited for a filled stage"
              : v == 103 ? "the MMA thread waited for a drained accumulator"
              : v == 104 ? "an epilogue warp waited for a finished accumulator"
              : v == 105 ? "teardown waited for copies in flight"
                         : "unknown code");
    return AMOSB_ERR_DEVICE_TIMEOUT;
  }
  return AMOSB_OK;
}

// ---- the reference's calling convention -------------------------------------------------------
static thread_local void* g_packed_stream[64] = {nullptr};

int amosb_set_stream(int device, void* cuda_stream) {
  if (device < 0 || device >= 64) {
    set_error("device id %d out of range", device);
    return AMOSB_ERR_ARG;
  }
  g_packed_stream[device] = cuda_stream;
  return AMOSB_OK;
}

// Scratch of the packed entry point, per device, grown on demand (the reference's generated code
// gets it from TVMBackendAllocWorkspace and frees it before returning).
struct PackedScratch {
  void* buf = nullptr;
  size_t cap = 0;
};
static PackedScratch g_packed_scratch[64];
static std::mutex g_packed_mutex[64];

static int packed_fail(int code) {
  // the reference's convention is 0 / -1; the library's own code goes in front of the message
  char msg[1024];
  snprintf(msg, sizeof(msg), "[amosb %d] %s", code, last_error());
  set_error("%s", msg);
  return -1;
}

static int dl_dtype_code(const AmosbDLDataType& t) {
  if (t.lanes != 1) return -1;
  if (t.code == AMOSB_DL_FLOAT && t.bits == 16) return AMOSB_F16;
  if (t.code == AMOSB_DL_FLOAT && t.bits == 32) return AMOSB_F32;
  if (t.code == AMOSB_DL_INT && t.bits == 8) return AMOSB_S8;
  if (t.code == AMOSB_DL_INT && t.bits == 32) return AMOSB_S32;
  if (t.code == AMOSB_DL_BFLOAT && t.bits == 16) return AMOSB_BF16;
  return -1;
}

int amosb_packed_call(AmosbTVMValue* args, int* type_codes, int num_args,
                      AmosbTVMValue* out_ret_value, int* out_ret_tcode, void* resource_handle) {
  const AmosbOpDesc* desc = static_cast<const AmosbOpDesc*>(resource_handle);
  if (desc == nullptr || args == nullptr || type_codes == nullptr) {
    set_error("NULL descriptor (resource_handle), argument list or type codes");
    return packed_fail(AMOSB_ERR_ARG);
  }
  const bool has_addend = (desc->epilogue & (AMOSB_EPI_ADD_VECTOR | AMOSB_EPI_ADD_FULL)) != 0;
  const int want = has_addend ? 4 : 3;
  if (num_args != want) {
    set_error("__tvm_main__: num_args should be %d, got %d", want, num_args);
    return packed_fail(AMOSB_ERR_ARG);
  }
  AmosbTensor t[4];
  int device = -1;
  for (int i = 0; i < num_args; ++i) {
    if (type_codes[i] != AMOSB_TVM_DLTENSOR_HANDLE && type_codes[i] != AMOSB_TVM_NDARRAY_HANDLE) {
      set_error("__tvm_main__: Expect arg[%d] to be pointer (type code %d given)", i,
                type_codes[i]);
      return packed_fail(AMOSB_ERR_ARG);
    }
    const AmosbDLTensor* dl = static_cast<const AmosbDLTensor*>(args[i].v_handle);
    if (dl == nullptr) {
      set_error("__tvm_main__: arg[%d] is a NULL tensor handle", i);
      return packed_fail(AMOSB_ERR_ARG);
    }
    if (dl->ctx.device_type != AMOSB_DL_GPU) {
      set_error("Argument arg%d.device_type has an unsatisfied constraint: expected %d (gpu), got %d",
                i, AMOSB_DL_GPU, dl->ctx.device_type);
      return packed_fail(AMOSB_ERR_ARG);
    }
    if (device < 0) device = dl->ctx.device_id;
    if (dl->ctx.device_id != device) {
      set_error("Argument arg%d.device_id has an unsatisfied constraint: expected %d, got %d", i,
                device, dl->ctx.device_id);
      return packed_fail(AMOSB_ERR_ARG);
    }
    const int dt = dl_dtype_code(dl->dtype);
    if (dt < 0) {
      set_error("arg%d.dtype (code %d, bits %d, lanes %d) is not one this library computes in: "
                "float16, bfloat16, float32, int8, int32, one lane",
                i, (int)dl->dtype.code, (int)dl->dtype.bits, (int)dl->dtype.lanes);
      return packed_fail(AMOSB_ERR_ARG);
    }
    t[i].data = dl->data;
    t[i].device_id = dl->ctx.device_id;
    t[i].dtype = dt;
    t[i].ndim = dl->ndim;
    t[i].shape = dl->shape;
    t[i].strides = dl->strides;
    t[i].byte_offset = dl->byte_offset;
  }
  if (device < 0 || device >= 64) {
    set_error("device id %d out of range", device);
    return packed_fail(AMOSB_ERR_ARG);
  }
  const int64_t ws_bytes = amosb_workspace_bytes(desc);
  if (ws_bytes < 0) return packed_fail((int)ws_bytes);
  void* ws = nullptr;
  if (ws_bytes > 0) {
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) {
      set_error("cudaSetDevice(%d) failed: %s", device, cudaGetErrorString(e));
      return packed_fail(AMOSB_ERR_CUDA);
    }
    std::lock_guard<std::mutex> lock(g_packed_mutex[device]);
    PackedScratch& sc = g_packed_scratch[device];
    if (sc.cap < (size_t)ws_bytes + 1024) {
      if (sc.buf) {
        cudaDeviceSynchronize();  // kernels queued earlier may still use the smaller buffer
        cudaFree(sc.buf);
        sc.buf = nullptr;
        sc.cap = 0;
      }
      e = cudaMalloc(&sc.buf, (size_t)ws_bytes + 1024);
      if (e != cudaSuccess) {
        set_error("cudaMalloc(%lld) failed: %s", (long long)ws_bytes + 1024, cudaGetErrorString(e));
        return packed_fail(AMOSB_ERR_CUDA);
      }
      sc.cap = (size_t)ws_bytes + 1024;
    }
    ws = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(sc.buf) + 1023) & ~uintptr_t(1023));
  }
  const int rc = amosb_run(desc, t, num_args - 1, &t[num_args - 1], 1, ws, ws_bytes,
                           g_packed_stream[device]);
  if (rc != AMOSB_OK) return packed_fail(rc);
  if (out_ret_tcode != nullptr) *out_ret_tcode = AMOSB_TVM_NULLPTR;
  if (out_ret_value != nullptr) out_ret_value->v_handle = nullptr;
  return 0;
}

int amosb_last_launch_count(void) { return launch_count(); }

int amosb_describe_plan(const AmosbOpDesc* desc, int device, char* buf, int buf_len) {
  if (desc == nullptr || buf == nullptr || buf_len <= 0) {
    set_error("NULL argument");
    return AMOSB_ERR_ARG;
  }
  AmosbOpDesc as_run = *desc;  // a single HWNC image runs as the NHWC operator (same memory)
  if (as_run.kind == AMOSB_OP_CONV2D_HWNC && as_run.conv_n == 1) as_run.kind = AMOSB_OP_CONV2D_NHWC;
  desc = &as_run;
  int sms = device >= 0 ? device_sm_count(device) : -1;
  if (sms <= 0) sms = 148;  // planning without a device: assume a full B200
  const int bn = choose_tile_n(*desc, sms);
  const bool pair = choose_cta_pairs(*desc, sms);
  const int rows = choose_tile_rows(*desc, sms);
  const bool tall = !pair && rows == 256;
  const int stages =
      pair ? (bn == 256 ? 6 : 8) : (tall ? 4 : (bn == 256 ? 4 : (bn == 128 ? 6 : 8)));
  const char* fam = pair   ? "umma_pair (2 CTAs per tile, cta_group::2)"
                    : tall ? "umma_persistent (tall tiles: two accumulators share each B stage)"
                           : "umma_persistent";
  int n = 0;
  const long long slots = pair ? sms / 2 : sms;
  // MMA kind and k-block depth of the in-place conv kernels
  const char* ck = desc->in_dtype == AMOSB_F32    ? "tf32"
                   : desc->in_dtype == AMOSB_BF16 ? "bf16"
                   : desc->in_dtype == AMOSB_S8   ? "i8"
                                                  : "f16";
  const int cbk = desc->in_dtype == AMOSB_F32 ? 32 : desc->in_dtype == AMOSB_S8 ? 128 : 64;
  if (desc->kind == AMOSB_OP_CONV2D_NCHW && conv_is_pointwise_gemm(*desc)) {
    const long long pq = desc->conv_p * desc->conv_q;
    const long long tiles = desc->conv_n * ((desc->conv_k + rows - 1) / rows) * ((pq + bn - 1) / bn);
    n = snprintf(buf, buf_len,
                 "plan conv2d_nchw (1x1, stride 1, no padding) %s->%s as a batched GEMM over the "
                 "images with the filter as shared A and the NCHW activation as MN-major B, no "
                 "re-layout: [1] %s<f16,BN=%d,B MN-major> tile %dx%dx64, %d smem stages, TMA-store "
                 "epilogue, %lld tiles on %lld %s",
                 dtype_name(desc->in_dtype), dtype_name(desc->out_dtype), fam, bn, rows, bn, stages,
                 tiles, tiles < slots ? tiles : slots, pair ? "CTA pairs" : "CTAs");
  } else if (desc->kind == AMOSB_OP_CONV2D_NCHW && conv_is_pointwise_inplace(*desc)) {
    const long long m = desc->conv_n * desc->conv_p * desc->conv_q;
    const int pbn = pointwise_inplace_tile_n(*desc);
    const long long tiles = ((m + 127) / 128) * ((desc->conv_k + pbn - 1) / pbn);
    n = snprintf(buf, buf_len,
                 "plan conv2d_nchw (1x1, stride 1, no padding, planes of %lld pixels: not a 16-byte "
                 "multiple) %s->%s, operands in place (no re-layout, no workspace): [1] "
                 "umma_persistent<%s,BN=%d,conv-1x1-inplace> tile 128x%dx64, %d smem stages, "
                 "activation as MN-major A copied by four warps with 8-byte cp.async into the "
                 "swizzled stage layout, filter as K-major TMA B, NCHW stores, %lld tiles on %lld CTAs",
                 (long long)(desc->conv_p * desc->conv_q), dtype_name(desc->in_dtype),
                 dtype_name(desc->out_dtype), ck, pbn, pbn, pbn == 256 ? 4 : (pbn == 128 ? 6 : 8),
                 tiles, tiles < sms ? tiles : (long long)sms);
  } else if (desc->kind == AMOSB_OP_CONV2D_NCHW) {
    const long long m = desc->conv_n * desc->conv_p * desc->conv_q;
    const long long tiles = ((m + rows - 1) / rows) * ((desc->conv_k + bn - 1) / bn);
    n = snprintf(buf, buf_len,
                 "plan conv2d_nchw %s->%s: [1] conv_prepack (activation NCHW->NHWC and filter "
                 "KCRS->KRSC into the workspace), [2] %s<f16,BN=%d,conv> tile %dx%dx64, %d smem "
                 "stages, im2col TMA A + tiled TMA B, TMEM 2x%d cols, %lld tiles on %lld %s",
                 dtype_name(desc->in_dtype), dtype_name(desc->out_dtype), fam, bn, rows, bn, stages,
                 tall ? 2 * bn : bn, tiles, tiles < slots ? tiles : slots,
                 pair ? "CTA pairs" : "CTAs");
  } else if (desc->kind == AMOSB_OP_CONV2D_HWNC && desc->conv_n <= 64 && desc->stride_w == 1 &&
             getenv("AMOSB_HWNC_NO_PACKING") == nullptr) {
    int nbox = 8;
    while (nbox < desc->conv_n) nbox *= 2;
    const int group = 128 / nbox;
    const long long m = desc->conv_p * ((desc->conv_q + group - 1) / group) * 128;
    const long long tiles = ((m + rows - 1) / rows) * ((desc->conv_k + bn - 1) / bn);
    n = snprintf(buf, buf_len,
                 "plan conv2d_hwnc %s->%s, operands in place (no re-layout, no workspace): [1] "
                 "%s<%s,BN=%d,conv-hwnc> tile %dx%dx%d = %d consecutive pixels of an output row x %d "
                 "images per accumulator, %d smem stages, tiled TMA A {%d channels, %d images, %d "
                 "pixels} under each filter tap + MN-major TMA B (RSCK as [R*S*C][K]), TMA-store "
                 "epilogue, %lld tiles on %lld %s",
                 dtype_name(desc->in_dtype), dtype_name(desc->out_dtype), fam, ck, bn, rows, bn, cbk,
                 group, nbox, stages, cbk, nbox, group, tiles, tiles < slots ? tiles : slots,
                 pair ? "CTA pairs" : "CTAs");
  } else if (desc->kind == AMOSB_OP_CONV2D_HWNC) {
    const long long m = ((desc->conv_n + 127) / 128) * 128 * desc->conv_p * desc->conv_q;
    const long long tiles = ((m + rows - 1) / rows) * ((desc->conv_k + bn - 1) / bn);
    n = snprintf(buf, buf_len,
                 "plan conv2d_hwnc %s->%s, operands in place (no re-layout, no workspace): [1] "
                 "%s<%s,BN=%d,conv-hwnc> tile %dx%dx%d = one output pixel x 128 images per "
                 "128 rows, %d smem stages, tiled TMA A {%d channels, 128 images} of the input "
                 "pixel under each filter tap + MN-major TMA B (RSCK as [R*S*C][K]), TMA-store "
                 "epilogue, %lld tiles on %lld %s",
                 dtype_name(desc->in_dtype), dtype_name(desc->out_dtype), fam, ck, bn, rows, bn, cbk,
                 stages, cbk, tiles, tiles < slots ? tiles : slots, pair ? "CTA pairs" : "CTAs");
  } else if (desc->kind == AMOSB_OP_CONV2D_NHWC) {
    const long long m = desc->conv_n * desc->conv_p * desc->conv_q;
    const long long tiles = ((m + rows - 1) / rows) * ((desc->conv_k + bn - 1) / bn);
    n = snprintf(buf, buf_len,
                 "plan conv2d_nhwc %s->%s, operands in place (no re-layout, no workspace): [1] "
                 "%s<%s,BN=%d,conv-nhwc> tile %dx%dx%d, %d smem stages, im2col TMA A + MN-major "
                 "TMA B (RSCK as [R*S*C][K]), TMA-store epilogue, %lld tiles on %lld %s",
                 dtype_name(desc->in_dtype), dtype_name(desc->out_dtype), fam, ck, bn, rows, bn, cbk,
                 stages, tiles, tiles < slots ? tiles : slots, pair ? "CTA pairs" : "CTAs");
  } else if (desc->kind == AMOSB_OP_GEMM || desc->kind == AMOSB_OP_BATCHED_GEMM) {
    const long long tiles = desc->batch * ((desc->m + rows - 1) / rows) * ((desc->n + bn - 1) / bn);
    const int bk = desc->in_dtype == AMOSB_S8 ? 128 : desc->in_dtype == AMOSB_F32 ? 32 : 64;
    n = snprintf(buf, buf_len,
                 "plan %s %s->%s: [1] %s<%s,BN=%d,A %s,B %s> tile %dx%dx%d, %d smem stages, tiled "
                 "TMA A/B, TMEM 2x%d cols, %lld tiles on %lld %s",
                 desc->kind == AMOSB_OP_GEMM ? "gemm" : "batched_gemm", dtype_name(desc->in_dtype),
                 dtype_name(desc->out_dtype), fam,
                 desc->in_dtype == AMOSB_S8     ? "i8"
                 : desc->in_dtype == AMOSB_BF16 ? "bf16"
                 : desc->in_dtype == AMOSB_F32  ? "tf32"
                                                : "f16",
                 bn,
                 desc->trans_a ? "MN-major" : "K-major", desc->trans_b ? "K-major" : "MN-major", rows, bn, bk, stages, tall ? 2 * bn : bn,
                 tiles, tiles < slots ? tiles : slots, pair ? "CTA pairs" : "CTAs");
  } else {
    set_error("descriptor has no operator kind (%d)", desc->kind);
    return AMOSB_ERR_ARG;
  }
  return n < buf_len ? n : buf_len - 1;
}

}  // extern "C"
