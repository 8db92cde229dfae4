/*
 * amosb.h -- C ABI of the B200 (sm_100a) replacement for the kernels that AMOS generates for
 * tensor-core mapped operators: GEMM, batched GEMM, int8 GEMM and NCHW conv2d (implicit GEMM).
 *
 * The library is the drop-in for what a module built by `at.auto_tensorize` + `tvm.build(sch, args,
 * "cuda")` does when it is called: validate DLTensor-like arguments, then launch device kernels on
 * the caller's stream, writing the outputs in place.  Plain pointers and sizes only; the caller
 * owns every buffer, including the scratch ("workspace") that the conv path needs.
 *
 * Return codes (all entry points):  0 ok, -1 bad argument, -2 unsupported workload / unmatched
 * compute, -3 CUDA error, -4 a device-side wait ran out (see amosb_status_peek).  The message is
 * read with amosb_last_error() (thread local), mirroring TVMGetLastError
 * (reference: include/tvm/runtime/c_runtime_api.h:181-192).
 */
#ifndef AMOSB_H_
#define AMOSB_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AMOSB_OK 0
#define AMOSB_ERR_ARG -1
#define AMOSB_ERR_UNSUPPORTED -2
#define AMOSB_ERR_CUDA -3
#define AMOSB_ERR_DEVICE_TIMEOUT -4

/* Element types. */
typedef enum AmosbDType {
  AMOSB_F16 = 0,
  AMOSB_F32 = 1,
  AMOSB_S8 = 2,
  AMOSB_S32 = 3,
  AMOSB_BF16 = 4 /* inputs only: bfloat16 x bfloat16 -> float32 (reference: hw_abs_dag/cuda/wmma_bf16.py) */
} AmosbDType;

/* Operator kinds the recogniser can report. */
typedef enum AmosbOpKind {
  AMOSB_OP_NONE = 0,
  AMOSB_OP_GEMM = 1,         /* C[i,j]   = sum_k A[i,k]   * B[k,j]          */
  AMOSB_OP_BATCHED_GEMM = 2, /* C[b,i,j] = sum_k A[b,i,k] * B[b,k,j]        */
  AMOSB_OP_CONV2D_NCHW = 3,  /* Out[n,k,p,q] = sum_{c,r,s} Pad[n,c,..]*W[k,c,r,s] */
  AMOSB_OP_CONV2D_NHWC = 4,  /* Out[n,p,q,k] = sum_{r,s,c} Pad[n,..,c]*W[r,s,c,k] (reference:
                                benchmark/amos/mapping_conv2d_tensorcore.py:43-72) */
  AMOSB_OP_CONV2D_HWNC = 5   /* Out[p,q,n,k] = sum_{r,s,c} Pad[..,n,c]*W[r,s,c,k]: A[H,W,N,C]; a tile is one
                                output pixel x 128 images (reference: same file, :74-104) */
} AmosbOpKind;

/*
 * Tensor argument: the fields of a DLTensor that the generated host function of the reference
 * checks before launching (reference: src/tir/transforms/make_packed_api.cc:107-198,
 * src/tir/transforms/arg_binder.cc:150-299).  `strides` may be NULL (compact row-major) or must
 * describe a compact row-major tensor; `data + byte_offset` must be 16-byte aligned.  The struct has
 * no device_type field: amosb_run takes device memory only and verifies that with the CUDA runtime
 * (every pointer must be device or managed memory of `device_id`); amosb_packed_call below takes
 * real DLTensors and checks their device_type as the reference does.
 */
typedef struct AmosbTensor {
  void* data;
  int32_t device_id;
  int32_t dtype; /* AmosbDType */
  int32_t ndim;
  const int64_t* shape;
  const int64_t* strides; /* in elements, or NULL */
  uint64_t byte_offset;
} AmosbTensor;

/*
 * Operator descriptor: what the structural recogniser extracts from a `te` compute
 * (it replaces the result of the reference's intrinsic matching + mapping,
 * reference: src/auto_tensorize/matcher.cc:47-120, src/auto_tensorize/compute_transform.cc:500-628).
 */
typedef struct AmosbOpDesc {
  int32_t kind;      /* AmosbOpKind */
  int32_t in_dtype;  /* AMOSB_F16, AMOSB_BF16, AMOSB_S8, or AMOSB_F32 = float32 operands multiplied as tf32
                        (reference: hw_abs_dag/cuda/wmma_tf32.py).  Every operator kind takes every input type. */
  int32_t acc_dtype; /* AMOSB_F32 or AMOSB_S32 (the dtype of the reduction) */
  int32_t out_dtype; /* dtype of the last stage: acc_dtype, or AMOSB_F16 after a cast stage */
  int32_t trans_a;   /* GEMM family: 1 if A is indexed [k,i], i.e. stored [K,M] (single-CTA tiles) */
  int32_t trans_b;   /* GEMM family: 1 if B is indexed [j,k] ("ntn"), 0 for [k,j]                */
  int32_t tile_n;    /* 0 = let the launcher choose; else 64, 128 or 256                         */
  int32_t cta_pair;  /* 0 = let the launcher choose; 1 = one CTA per 128-row tile; 2 = CTA pairs
                        (256-row tiles); 3 = one CTA per 256 x 128 tile (fp16, tile_n 0 or 128)  */
  int64_t batch, m, n, k; /* GEMM family extents (batch = 1 for GEMM)                           */
  /* conv2d: NCHW / KCRS; NHWC / RSCK for AMOSB_OP_CONV2D_NHWC; HWNC / RSCK for AMOSB_OP_CONV2D_HWNC */
  int64_t conv_n, conv_c, conv_h, conv_w; /* input  [N,C,H,W]  ([N,H,W,C]) */
  int64_t conv_k, conv_r, conv_s;         /* filter [K,C,R,S]  ([R,S,C,K]) */
  int64_t conv_p, conv_q;                 /* output [N,K,P,Q]  ([N,P,Q,K]) */
  int32_t stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  /* operand order: index into the callable's input list of the "A"/"B" (activation/filter) */
  int32_t arg_a, arg_b;
  /* Trailing element-wise stages fused into the kernel's epilogue (the reference runs them as a
   * separate "last op" kernel, reference: python/tvm/auto_tensorize/tensorization_phases/
   * schedulers/cuda_v2.py:729-745; its bias DAG: hw_abs_dag/cuda/wmma_fp16_bias.py:11-60):
   *   out = cast(relu?(acc + addend?)), in that order.
   * epilogue: bit mask of AMOSB_EPI_*.  The addend is a third input (index arg_c): either a vector
   * indexed by the N axis (GEMM / batched GEMM: j, conv2d: output channel k) or a tensor of the
   * output's shape; dtype = acc_dtype, or float16 read through a cast. */
  int32_t epilogue;
  int32_t addend_dtype;
  int32_t arg_c;
  int32_t reserved1;
} AmosbOpDesc;

#define AMOSB_EPI_ADD_VECTOR 1 /* + addend[j]        */
#define AMOSB_EPI_ADD_FULL 2   /* + addend[same indices as the output] */
#define AMOSB_EPI_RELU 4       /* max(., 0)          */

/* Library version (major*10000 + minor*100 + patch). */
int amosb_version(void);

/* Message of the last failure on the calling thread (never NULL). */
const char* amosb_last_error(void);

/*
 * Structural recogniser.  `te_dag` is the textual serialisation of a `te` compute DAG produced by
 * the Python front end (one stage per line, see amos_b200/te.py: serialise_dag).  On a match fills
 * `*out` and returns 0; otherwise returns AMOSB_ERR_UNSUPPORTED with the reference's message
 * "This workload has no matched intrinsic for target" (reference:
 * python/tvm/auto_tensorize/auto_tensorize.py:76-78).  Replaces get_match_results / MatchIntrinsic
 * (reference: python/tvm/auto_tensorize/tensorization_phases/intrin_match.py:168-181,
 * src/auto_tensorize/matcher.cc:312-340).  Pure host code: needs no GPU.
 */
int amosb_recognize(const char* te_dag, AmosbOpDesc* out);

/*
 * Scratch memory (bytes, device global memory, 1024-byte aligned) that amosb_run needs for `desc`:
 * the NHWC copy of the activation and the re-laid-out filter of the NCHW conv path (nothing of the
 * kind for the GEMM family, for NHWC / HWNC convolutions and for 1x1 NCHW layers, which are consumed
 * in place), plus an optional part described under amosb_workspace_bytes_min.  Counterpart of the workspace the reference's generated host code obtains through
 * TVMBackendAllocWorkspace (reference: include/tvm/runtime/c_backend_api.h:49-91); here the caller
 * allocates it.  Returns a negative error code on a bad descriptor.
 */
int64_t amosb_workspace_bytes(const AmosbOpDesc* desc);

/*
 * The part of amosb_workspace_bytes(desc) that amosb_run cannot do without: the re-laid-out
 * operands of the NCHW conv path, 0 for everything else.  The rest is optional: room for the partial
 * sums that CTAs exchange when the tiles of the last, short round of a schedule are shared out
 * among all SMs (up to ~19 MB; where the tile count fills its last round it is 0).  With less than
 * the full amount -- or workspace == NULL for operators whose minimum is 0 -- amosb_run computes
 * the same numbers with every tile on one CTA, somewhat slower.  No counterpart in the reference.
 */
int64_t amosb_workspace_bytes_min(const AmosbOpDesc* desc);

/*
 * Run the operator: the counterpart of calling the built module, `func(A, B, C)`
 * (reference: python/tvm/runtime/module.py:108-112 -> TVMFuncCall, include/tvm/runtime/c_runtime_api.h:266;
 * kernel launch at src/runtime/cuda/cuda_module.cc:152-192).  `ins` are the inputs in the order
 * of the callable's argument list (two operands, plus the addend when desc->epilogue has an
 * AMOSB_EPI_ADD_* bit), `outs` the outputs (written in place).  All tensors must live
 * on one device, which becomes current.  Asynchronous: kernels are enqueued on `cuda_stream`
 * (a cudaStream_t; NULL = the default stream).  `workspace` must hold amosb_workspace_bytes(desc).
 */
int amosb_run(const AmosbOpDesc* desc, const AmosbTensor* ins, int n_in, AmosbTensor* outs,
              int n_out, void* workspace, int64_t workspace_bytes, void* cuda_stream);

/*
 * Host-buffer variant: every `data` pointer in `ins`/`outs` is HOST memory (device_id ignored).
 * Copies the inputs to `device`, runs, copies the outputs back and synchronises.  The device
 * buffers are kept per device between calls and grown on demand (calls on one device are
 * serialised).  For callers without device arrays, and for end-to-end measurement; pass pinned
 * host memory to get full copy bandwidth.  Has no counterpart in the reference, whose callers
 * copy with tvm.nd.array / asnumpy around the call.
 */
int amosb_run_host(const AmosbOpDesc* desc, const AmosbTensor* ins, int n_in, AmosbTensor* outs,
                   int n_out, int device);

/*
 * Device-side status word of `device`: 0 if no kernel gave up a bounded wait since the last
 * clear, else the code of the first wait that ran out (101..105).  Synchronises the device.
 * Replaces nothing in the reference (its kernels have no waits); it is how a device timeout is
 * reported without faulting the context.
 */
int amosb_status_peek(int device, int clear);

/* Number of kernels the last amosb_run on this thread enqueued (for launch accounting). */
int amosb_last_launch_count(void);

/* Human-readable description of the plan amosb_run would use for `desc` (tile shape, stages, grid,
 * kernels).  Counterpart of printing `tvm.lower(sch, args, simple_mode=True)`.  Returns the number
 * of bytes written (excluding the terminator) or a negative error code. */
int amosb_describe_plan(const AmosbOpDesc* desc, int device, char* buf, int buf_len);

/*
 * conv2d for callers that cannot allocate device memory (no counterpart in the reference, whose
 * generated host code always obtains its workspace from the runtime's allocator).  Meant for hosts
 * that gave the whole device to their own arena, plugin interfaces that pass tensors but no
 * allocator, and loops that cannot afford the device-wide synchronisation of cudaMalloc/cudaFree.
 * The scratch that amosb_run takes as `workspace` lives in an array built into the library
 * (AMOSB_STATIC_SCRATCH_BYTES usable bytes; every GPU that loads the library holds it until the
 * process exits).  The caller passes only inputs and output, exactly as for amosb_run; no
 * cudaMalloc, cudaFree or other allocating routine is called.
 *  - Descriptors whose amosb_workspace_bytes_min() exceeds AMOSB_STATIC_SCRATCH_BYTES are refused
 *    with AMOSB_ERR_UNSUPPORTED and a message naming both sizes.
 *  - The first call on a device resolves the array's device address (and does the library's
 *    one-time device set-up); make that first call before any stream capture begins.
 *  - All calls on a device share the array.  Every byte a call reads from it is written earlier in
 *    the same call, so stale contents of a previous call are never used and nothing needs
 *    clearing; but two calls that overlap on the GPU (different streams, or threads) race on it.
 */
#define AMOSB_STATIC_SCRATCH_BYTES (8ll * 1024 * 1024)
int amosb_conv2d_nchw_static(const AmosbOpDesc* desc, const AmosbTensor* ins, int n_in,
                             AmosbTensor* outs, int n_out, void* cuda_stream);


/*
 * Synchronise `device` and turn a device-side wait that ran out into an error code: returns 0 when
 * the status word is clear, else AMOSB_ERR_DEVICE_TIMEOUT (-4) with the wait's code (101..105) in
 * the message, and clears the word.  The kernels bound every wait (2 s by default; the environment
 * variable AMOSB_WAIT_BUDGET_NS overrides it for launches made afterwards) and give up instead of
 * hanging; this is where the host learns of it.  Counterpart of the per-candidate time-outs and
 * MeasureErrorNo codes of the reference's measurement loop
 * (reference: python/tvm/auto_tensorize/search/measure.py:529-554, 755-785).
 */
int amosb_sync_check(int device);

/*
 * Stream that amosb_packed_call launches on, per calling thread and device (NULL = the default
 * stream).  Counterpart of TVMSetStream (reference: include/tvm/runtime/c_runtime_api.h:476), which
 * sets the thread-local stream the reference's CUDA module launches on
 * (reference: src/runtime/cuda/cuda_module.cc:170).
 */
int amosb_set_stream(int device, void* cuda_stream);

/*
 * The reference's own calling convention.  A module built by the reference is entered through
 *   int f(TVMValue* args, int* type_codes, int num_args, TVMValue* out_ret_value,
 *         int* out_ret_tcode, void* resource_handle)
 * (TVMBackendPackedCFunc, reference: include/tvm/runtime/c_backend_api.h:49-51) with one DLTensor*
 * per argument.  The structs below restate the layout of the DLPack release the reference vendors
 * (DLContext{device_type, device_id}, DLDataType{code, bits, lanes}; reference:
 * include/tvm/runtime/c_runtime_api.h:79-135 for the type codes and the TVMValue union), under
 * names of their own so that this header can be included next to dlpack.h.
 */
typedef struct AmosbDLContext {
  int32_t device_type; /* AMOSB_DL_GPU is the only type accepted */
  int32_t device_id;
} AmosbDLContext;
typedef struct AmosbDLDataType {
  uint8_t code; /* AMOSB_DL_INT, AMOSB_DL_FLOAT, AMOSB_DL_BFLOAT */
  uint8_t bits;
  uint16_t lanes; /* must be 1 */
} AmosbDLDataType;
typedef struct AmosbDLTensor {
  void* data;
  AmosbDLContext ctx;
  int32_t ndim;
  AmosbDLDataType dtype;
  int64_t* shape;
  int64_t* strides; /* in elements, or NULL for compact row-major */
  uint64_t byte_offset;
} AmosbDLTensor;
typedef union AmosbTVMValue {
  int64_t v_int64;
  double v_float64;
  void* v_handle;
  const char* v_str;
  AmosbDLDataType v_type;
  AmosbDLContext v_ctx;
} AmosbTVMValue;

#define AMOSB_DL_GPU 2            /* kDLGPU */
#define AMOSB_DL_INT 0            /* kDLInt */
#define AMOSB_DL_FLOAT 2          /* kDLFloat */
#define AMOSB_DL_BFLOAT 4         /* kDLBfloat */
#define AMOSB_TVM_NULLPTR 4       /* kTVMNullptr */
#define AMOSB_TVM_DLTENSOR_HANDLE 7 /* kTVMDLTensorHandle */
#define AMOSB_TVM_NDARRAY_HANDLE 13 /* kTVMNDArrayHandle */

/*
 * Run the operator described by `resource_handle` (a `const AmosbOpDesc*`) on `num_args` tensors:
 * the inputs in the callable's order, then the output.  Performs the checks of the reference's
 * generated prologue before anything is launched (reference: src/tir/transforms/make_packed_api.cc:
 * 107-198, src/tir/transforms/arg_binder.cc:150-299): argument count, handle type codes, ndim,
 * dtype code / bits / lanes, every shape extent, compact (or NULL) strides, byte_offset alignment,
 * device_type == kDLGPU and one device_id for all tensors, which then becomes current.  Launches
 * on the stream set with amosb_set_stream; the conv scratch, which the reference obtains with
 * TVMBackendAllocWorkspace (reference: include/tvm/runtime/c_backend_api.h:87-100), comes from a
 * buffer the library keeps per device and grows on demand.  Returns 0, or -1 with the message (which
 * starts with this library's own code, "[amosb -2] ...") in amosb_last_error(), as the reference's
 * convention asks.
 */
int amosb_packed_call(AmosbTVMValue* args, int* type_codes, int num_args,
                      AmosbTVMValue* out_ret_value, int* out_ret_tcode, void* resource_handle);

#ifdef __cplusplus
}
#endif
#endif /* AMOSB_H_ */
