"""ctypes bindings of libamosb.so (declared in include/amosb.h).

The library is the only compute path: if it is missing or cannot be loaded the import fails
loudly -- there is no CPU or PyTorch fallback behind these calls.
"""
from __future__ import annotations

import ctypes
import os
from typing import Sequence

HERE = os.path.dirname(os.path.abspath(__file__))
# AMOSB_LIBRARY overrides the path (e.g. a diagnostic build of the same sources)
LIB_PATH = os.environ.get("AMOSB_LIBRARY") or os.path.join(HERE, "libamosb.so")

AMOSB_OK = 0
AMOSB_ERR_ARG = -1
AMOSB_ERR_UNSUPPORTED = -2
AMOSB_ERR_CUDA = -3
AMOSB_ERR_DEVICE_TIMEOUT = -4

AMOSB_F16, AMOSB_F32, AMOSB_S8, AMOSB_S32, AMOSB_BF16 = 0, 1, 2, 3, 4
DTYPE_NAMES = {AMOSB_F16: "float16", AMOSB_F32: "float32", AMOSB_S8: "int8", AMOSB_S32: "int32",
               AMOSB_BF16: "bfloat16"}
DTYPE_CODES = {v: k for k, v in DTYPE_NAMES.items()}
DTYPE_BYTES = {AMOSB_F16: 2, AMOSB_F32: 4, AMOSB_S8: 1, AMOSB_S32: 4, AMOSB_BF16: 2}

OP_NONE, OP_GEMM, OP_BATCHED_GEMM, OP_CONV2D_NCHW, OP_CONV2D_NHWC, OP_CONV2D_HWNC = 0, 1, 2, 3, 4, 5
CONV_KINDS = (OP_CONV2D_NCHW, OP_CONV2D_NHWC, OP_CONV2D_HWNC)
EPI_ADD_VECTOR, EPI_ADD_FULL, EPI_RELU = 1, 2, 4
OP_NAMES = {OP_GEMM: "gemm", OP_BATCHED_GEMM: "batched_gemm", OP_CONV2D_NCHW: "conv2d_nchw",
            OP_CONV2D_NHWC: "conv2d_nhwc", OP_CONV2D_HWNC: "conv2d_hwnc"}


class AmosbError(RuntimeError):
    """Raised for every non-zero return code of the C ABI (the TVMError of this library)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[amosb {code}] {message}")
        self.code = code
        self.message = message


class AmosbTensor(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("device_id", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
        ("ndim", ctypes.c_int32),
        ("shape", ctypes.POINTER(ctypes.c_int64)),
        ("strides", ctypes.POINTER(ctypes.c_int64)),
        ("byte_offset", ctypes.c_uint64),
    ]


class AmosbOpDesc(ctypes.Structure):
    _fields_ = [
        ("kind", ctypes.c_int32),
        ("in_dtype", ctypes.c_int32),
        ("acc_dtype", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32),
        ("trans_a", ctypes.c_int32),
        ("trans_b", ctypes.c_int32),
        ("tile_n", ctypes.c_int32),
        ("cta_pair", ctypes.c_int32),
        ("batch", ctypes.c_int64),
        ("m", ctypes.c_int64),
        ("n", ctypes.c_int64),
        ("k", ctypes.c_int64),
        ("conv_n", ctypes.c_int64),
        ("conv_c", ctypes.c_int64),
        ("conv_h", ctypes.c_int64),
        ("conv_w", ctypes.c_int64),
        ("conv_k", ctypes.c_int64),
        ("conv_r", ctypes.c_int64),
        ("conv_s", ctypes.c_int64),
        ("conv_p", ctypes.c_int64),
        ("conv_q", ctypes.c_int64),
        ("stride_h", ctypes.c_int32),
        ("stride_w", ctypes.c_int32),
        ("pad_h", ctypes.c_int32),
        ("pad_w", ctypes.c_int32),
        ("dil_h", ctypes.c_int32),
        ("dil_w", ctypes.c_int32),
        ("arg_a", ctypes.c_int32),
        ("arg_b", ctypes.c_int32),
        ("epilogue", ctypes.c_int32),
        ("addend_dtype", ctypes.c_int32),
        ("arg_c", ctypes.c_int32),
        ("reserved1", ctypes.c_int32),
    ]

    def copy(self) -> "AmosbOpDesc":
        other = AmosbOpDesc()
        ctypes.memmove(ctypes.byref(other), ctypes.byref(self), ctypes.sizeof(AmosbOpDesc))
        return other

    def as_dict(self) -> dict:
        return {name: getattr(self, name) for name, _ in self._fields_ if name != "reserved1"}

    @property
    def n_inputs(self) -> int:
        return 3 if self.epilogue & (EPI_ADD_VECTOR | EPI_ADD_FULL) else 2


# Every symbol include/amosb.h declares, with its ctypes signature.
_SIGNATURES = {
    "amosb_version": (ctypes.c_int, []),
    "amosb_last_error": (ctypes.c_char_p, []),
    "amosb_recognize": (ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(AmosbOpDesc)]),
    "amosb_workspace_bytes": (ctypes.c_int64, [ctypes.POINTER(AmosbOpDesc)]),
    "amosb_workspace_bytes_min": (ctypes.c_int64, [ctypes.POINTER(AmosbOpDesc)]),
    "amosb_run": (ctypes.c_int, [ctypes.POINTER(AmosbOpDesc), ctypes.POINTER(AmosbTensor),
                                 ctypes.c_int, ctypes.POINTER(AmosbTensor), ctypes.c_int,
                                 ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]),
    "amosb_run_host": (ctypes.c_int, [ctypes.POINTER(AmosbOpDesc), ctypes.POINTER(AmosbTensor),
                                      ctypes.c_int, ctypes.POINTER(AmosbTensor), ctypes.c_int,
                                      ctypes.c_int]),
    "amosb_status_peek": (ctypes.c_int, [ctypes.c_int, ctypes.c_int]),
    "amosb_last_launch_count": (ctypes.c_int, []),
    "amosb_describe_plan": (ctypes.c_int, [ctypes.POINTER(AmosbOpDesc), ctypes.c_int,
                                           ctypes.c_char_p, ctypes.c_int]),
    "amosb_conv2d_nchw_static": (ctypes.c_int, [ctypes.POINTER(AmosbOpDesc),
                                                ctypes.POINTER(AmosbTensor), ctypes.c_int,
                                                ctypes.POINTER(AmosbTensor), ctypes.c_int,
                                                ctypes.c_void_p]),
}



class AmosbDLContext(ctypes.Structure):
    _fields_ = [("device_type", ctypes.c_int32), ("device_id", ctypes.c_int32)]


class AmosbDLDataType(ctypes.Structure):
    _fields_ = [("code", ctypes.c_uint8), ("bits", ctypes.c_uint8), ("lanes", ctypes.c_uint16)]


class AmosbDLTensor(ctypes.Structure):
    """Layout of the DLTensor of the DLPack release the reference vendors (48 bytes)."""
    _fields_ = [("data", ctypes.c_void_p), ("ctx", AmosbDLContext), ("ndim", ctypes.c_int32),
                ("dtype", AmosbDLDataType), ("shape", ctypes.POINTER(ctypes.c_int64)),
                ("strides", ctypes.POINTER(ctypes.c_int64)), ("byte_offset", ctypes.c_uint64)]


class AmosbTVMValue(ctypes.Union):
    _fields_ = [("v_int64", ctypes.c_int64), ("v_float64", ctypes.c_double),
                ("v_handle", ctypes.c_void_p), ("v_str", ctypes.c_char_p),
                ("v_type", AmosbDLDataType), ("v_ctx", AmosbDLContext)]


DL_GPU, DL_INT, DL_FLOAT, DL_BFLOAT = 2, 0, 2, 4
TVM_NULLPTR, TVM_DLTENSOR_HANDLE, TVM_NDARRAY_HANDLE = 4, 7, 13
DL_DTYPES = {AMOSB_F16: (DL_FLOAT, 16), AMOSB_F32: (DL_FLOAT, 32), AMOSB_S8: (DL_INT, 8),
             AMOSB_S32: (DL_INT, 32), AMOSB_BF16: (DL_BFLOAT, 16)}

_SIGNATURES.update({
    "amosb_sync_check": (ctypes.c_int, [ctypes.c_int]),
    "amosb_set_stream": (ctypes.c_int, [ctypes.c_int, ctypes.c_void_p]),
    "amosb_packed_call": (ctypes.c_int, [ctypes.POINTER(AmosbTVMValue),
                                         ctypes.POINTER(ctypes.c_int), ctypes.c_int,
                                         ctypes.POINTER(AmosbTVMValue),
                                         ctypes.POINTER(ctypes.c_int), ctypes.c_void_p]),
})

STATIC_SCRATCH_BYTES = 8 * 1024 * 1024  # AMOSB_STATIC_SCRATCH_BYTES

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def load() -> ctypes.CDLL:
    """Load libamosb.so (built in-tree by ``python -m amos_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m amos_b200.build` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    msg = load().amosb_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int) -> int:
    if rc < 0:
        raise AmosbError(rc, last_error())
    return rc


def make_tensor(data_ptr: int, device_id: int, dtype: int, shape: Sequence[int],
                strides: Sequence[int] | None = None, byte_offset: int = 0):
    """Build an AmosbTensor; returns (struct, keepalive) -- hold on to keepalive during the call."""
    nd = len(shape)
    shp = (ctypes.c_int64 * max(nd, 1))(*shape)
    st = (ctypes.c_int64 * max(nd, 1))(*strides) if strides is not None else None
    t = AmosbTensor()
    t.data = data_ptr
    t.device_id = device_id
    t.dtype = dtype
    t.ndim = nd
    t.shape = ctypes.cast(shp, ctypes.POINTER(ctypes.c_int64))
    t.strides = ctypes.cast(st, ctypes.POINTER(ctypes.c_int64)) if st is not None else None
    t.byte_offset = byte_offset
    return t, (shp, st)


def make_dl_tensor(data_ptr: int, device_id: int, dtype: int, shape: Sequence[int],
                   strides: Sequence[int] | None = None, byte_offset: int = 0,
                   device_type: int = DL_GPU, lanes: int = 1):
    """Build an AmosbDLTensor (the reference's DLTensor layout); returns (struct, keepalive)."""
    nd = len(shape)
    shp = (ctypes.c_int64 * max(nd, 1))(*shape)
    st = (ctypes.c_int64 * max(nd, 1))(*strides) if strides is not None else None
    t = AmosbDLTensor()
    t.data = data_ptr
    t.ctx.device_type, t.ctx.device_id = device_type, device_id
    t.ndim = nd
    t.dtype.code, t.dtype.bits = DL_DTYPES[dtype]
    t.dtype.lanes = lanes
    t.shape = ctypes.cast(shp, ctypes.POINTER(ctypes.c_int64))
    t.strides = ctypes.cast(st, ctypes.POINTER(ctypes.c_int64)) if st is not None else None
    t.byte_offset = byte_offset
    return t, (shp, st)


def packed_call(desc: AmosbOpDesc, dl_tensors: Sequence[AmosbDLTensor],
                type_codes: Sequence[int] | None = None) -> int:
    """Enter the library the way a reference build enters its generated code: TVMValue array,
    type codes, the descriptor as resource handle.  Returns the raw return code (0 or -1)."""
    n = len(dl_tensors)
    vals = (AmosbTVMValue * max(n, 1))()
    for i, t in enumerate(dl_tensors):
        vals[i].v_handle = ctypes.addressof(t) if t is not None else None
    codes = (ctypes.c_int * max(n, 1))(*(type_codes or [TVM_DLTENSOR_HANDLE] * n))
    ret = AmosbTVMValue()
    ret_code = ctypes.c_int(-7)
    rc = load().amosb_packed_call(vals, codes, n, ctypes.byref(ret), ctypes.byref(ret_code),
                                  ctypes.cast(ctypes.byref(desc), ctypes.c_void_p))
    if rc == 0:
        assert ret_code.value == TVM_NULLPTR
    return rc


def recognize(te_dag_text: str) -> AmosbOpDesc:
    desc = AmosbOpDesc()
    check(load().amosb_recognize(te_dag_text.encode("utf-8"), ctypes.byref(desc)))
    return desc


def workspace_bytes(desc: AmosbOpDesc) -> int:
    return check(load().amosb_workspace_bytes(ctypes.byref(desc)))


def workspace_bytes_min(desc: AmosbOpDesc) -> int:
    """The part of `workspace_bytes` the call cannot do without (the rest only buys speed)."""
    return check(load().amosb_workspace_bytes_min(ctypes.byref(desc)))


def describe_plan(desc: AmosbOpDesc, device: int = -1) -> str:
    buf = ctypes.create_string_buffer(2048)
    check(load().amosb_describe_plan(ctypes.byref(desc), device, buf, len(buf)))
    return buf.value.decode("utf-8")


def gemm_desc(m: int, n: int, k: int, in_dtype: int = AMOSB_F16, out_dtype: int | None = None,
              batch: int = 1, trans_b: bool = False, batched: bool | None = None,
              tile_n: int = 0, cta_pair: int = 0, trans_a: bool = False) -> AmosbOpDesc:
    d = AmosbOpDesc()
    if batched is None:
        batched = batch != 1
    d.kind = OP_BATCHED_GEMM if batched else OP_GEMM
    d.in_dtype = in_dtype
    d.acc_dtype = AMOSB_S32 if in_dtype == AMOSB_S8 else AMOSB_F32
    d.out_dtype = d.acc_dtype if out_dtype is None else out_dtype
    d.trans_a = 1 if trans_a else 0
    d.trans_b = 1 if trans_b else 0
    d.batch, d.m, d.n, d.k = batch, m, n, k
    d.tile_n = tile_n
    d.cta_pair = cta_pair
    d.arg_a, d.arg_b = 0, 1
    return d


def conv2d_desc(n: int, c: int, h: int, w: int, k: int, r: int, s: int, stride: int = 1,
                pad: int = 0, dilation: int = 1, out_dtype: int = AMOSB_F32,
                tile_n: int = 0, cta_pair: int = 0) -> AmosbOpDesc:
    d = AmosbOpDesc()
    d.kind = OP_CONV2D_NCHW
    d.in_dtype = AMOSB_F16
    d.acc_dtype = AMOSB_F32
    d.out_dtype = out_dtype
    d.batch = 1
    d.conv_n, d.conv_c, d.conv_h, d.conv_w = n, c, h, w
    d.conv_k, d.conv_r, d.conv_s = k, r, s
    d.stride_h = d.stride_w = stride
    d.pad_h = d.pad_w = pad
    d.dil_h = d.dil_w = dilation
    d.conv_p = (h + 2 * pad - dilation * (r - 1) - 1) // stride + 1
    d.conv_q = (w + 2 * pad - dilation * (s - 1) - 1) // stride + 1
    d.tile_n = tile_n
    d.cta_pair = cta_pair
    d.arg_a, d.arg_b = 0, 1
    return d


def _set_conv_in_dtype(d: AmosbOpDesc, in_dtype: int) -> None:
    d.in_dtype = in_dtype
    if in_dtype == AMOSB_S8:
        d.acc_dtype = d.out_dtype = AMOSB_S32


def conv2d_nhwc_desc(n: int, h: int, w: int, c: int, k: int, r: int, s: int, stride: int = 1,
                     pad: int = 0, dilation: int = 1, out_dtype: int = AMOSB_F32,
                     tile_n: int = 0, cta_pair: int = 0, in_dtype: int = AMOSB_F16) -> AmosbOpDesc:
    """A[N,H,W,C] * B[R,S,C,K] -> Conv[N,P,Q,K]; both operands are consumed where they lie.
    `in_dtype` float16 (default), bfloat16, float32 (tf32 products) or int8 (int32 out)."""
    d = conv2d_desc(n, c, h, w, k, r, s, stride, pad, dilation, out_dtype, tile_n, cta_pair)
    d.kind = OP_CONV2D_NHWC
    _set_conv_in_dtype(d, in_dtype)
    return d


def conv2d_hwnc_desc(h: int, w: int, n: int, c: int, k: int, r: int, s: int, stride: int = 1,
                     pad: int = 0, dilation: int = 1, out_dtype: int = AMOSB_F32,
                     tile_n: int = 0, cta_pair: int = 0, in_dtype: int = AMOSB_F16) -> AmosbOpDesc:
    """A[H,W,N,C] * B[R,S,C,K] -> Conv[P,Q,N,K]; operands consumed where they lie (a tile is one
    output pixel x 128 images, or, for at most 64 images and stride 1 along W, several consecutive
    pixels of an output row x the images)."""
    d = conv2d_desc(n, c, h, w, k, r, s, stride, pad, dilation, out_dtype, tile_n, cta_pair)
    d.kind = OP_CONV2D_HWNC
    _set_conv_in_dtype(d, in_dtype)
    return d
