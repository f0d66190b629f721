"""ctypes binding of the C ABI in ``include/one_cuda.h``.

Loads ``lib/libone_b200.so`` (kernels + entry points) and the three drop-in operator libraries
``lib/<Op>/lib<Op>_cu.so`` whose ``eval`` symbol the reference host would dlsym
(host/op.h:58-76).  There is no fallback: a missing library raises, and every non-zero return
code raises ``OneCudaError`` with the library's error text.
"""
import ctypes as C
import os

from . import abi

_LIB_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")

ONE_OK = 0
ERR_NAMES = {-1: "ONE_ERR_BAD_ARG", -2: "ONE_ERR_BAD_SHAPE", -3: "ONE_ERR_UNSUPPORTED", -4: "ONE_ERR_CUDA",
             -5: "ONE_ERR_NOMEM", -6: "ONE_ERR_TIMEOUT", -7: "ONE_ERR_RANGE"}
PREC_TF32, PREC_BF16, PREC_F16 = 0x0, 0x1, 0x2
PRECISIONS = {"tf32": PREC_TF32, "bf16": PREC_BF16, "f16": PREC_F16}
LAYOUT_NHWC, OUT_F32, IN_S8, FUSE_ADD_RELU, FUSE_ADD, IN_NCHW_F32 = 0x10, 0x20, 0x40, 0x80, 0x100, 0x200
SLOT_RESIDUAL, SLOT_OUT_Q = 10, 1

# every symbol include/one_cuda.h declares
API_SYMBOLS = [
    "one_cuda_init", "one_cuda_release", "one_cuda_stream", "one_cuda_status", "one_cuda_last_error",
    "one_cuda_conv_eval", "one_cuda_gemm_eval", "one_cuda_matmul_eval", "one_cuda_set_eval_precision",
    "one_cuda_prepare", "one_cuda_eval_async", "one_cuda_packed_release", "one_cuda_packed_set_requant",
    "one_cuda_packed_work", "one_cuda_set_tile_n", "one_cuda_launch_count", "one_cuda_conv_eval_static", "one_cuda_selftest_wait_timeout",
    "one_cuda_matmul_async", "one_cuda_attention", "one_cuda_set_split_k", "one_cuda_set_launch_overlap", "one_cuda_packed_detail", "one_cuda_packed_set_split", "one_cuda_set_width_pairing", "one_cuda_set_cta_pairs", "one_cuda_set_half_tiles", "one_cuda_set_wide_epilogue", "one_cuda_set_epilogue_mode",
]


class OneCudaError(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"{ERR_NAMES.get(code, code)}: {text}")
        self.code = code


_lib = None
_shims = {}
_BIP = C.POINTER(abi.BUFFER_INFO_S)


def lib_path():
    return os.path.join(_LIB_DIR, "libone_b200.so")


def shim_path(op):
    return os.path.join(_LIB_DIR, op, f"lib{op}_cu.so")


def lib():
    """The core library; raises if it has not been built (``__graft_entry__.build()``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(lib_path()):
            raise OneCudaError(-4, f"{lib_path()} is missing: build the CUDA extension first (no CPU fallback exists)")
        L = C.CDLL(lib_path())
        L.one_cuda_last_error.restype = C.c_char_p
        L.one_cuda_launch_count.restype = C.c_ulonglong
        L.one_cuda_stream.restype = C.c_void_p
        L.one_cuda_stream.argtypes = [C.c_void_p]
        L.one_cuda_init.argtypes = [C.c_int, C.c_size_t, C.POINTER(C.c_void_p)]
        L.one_cuda_release.argtypes = [C.c_void_p]
        L.one_cuda_status.argtypes = [C.c_void_p]
        for n in ("one_cuda_conv_eval", "one_cuda_gemm_eval", "one_cuda_matmul_eval"):
            getattr(L, n).argtypes = [_BIP, _BIP, _BIP]
        L.one_cuda_conv_eval_static.argtypes = [_BIP, _BIP, _BIP, C.c_void_p]
        L.one_cuda_selftest_wait_timeout.argtypes = [C.c_void_p, C.c_ulonglong]
        L.one_cuda_prepare.argtypes = [C.c_void_p, C.c_char_p, _BIP, _BIP, C.c_int, C.POINTER(C.c_void_p)]
        L.one_cuda_eval_async.argtypes = [C.c_void_p, C.c_void_p, _BIP, _BIP, _BIP, C.c_void_p]
        L.one_cuda_packed_release.argtypes = [C.c_void_p]
        L.one_cuda_packed_set_requant.argtypes = [C.c_void_p, C.c_float]
        L.one_cuda_packed_work.argtypes = [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_double)]
        _lib = L
    return _lib


def check(rc):
    if rc != ONE_OK:
        raise OneCudaError(rc, lib().one_cuda_last_error().decode())


def shim_eval(op):
    """``eval`` of ``lib<Op>_cu.so`` -- the drop-in symbol."""
    if op not in _shims:
        lib()   # the shim links against the core library
        S = C.CDLL(shim_path(op))
        S.eval.restype = C.c_int
        S.eval.argtypes = [_BIP, _BIP, _BIP]
        _shims[op] = S
    return _shims[op].eval


class Context:
    """one_ctx: stream + workspace + status word of one device."""

    def __init__(self, device=0, workspace_bytes=0):
        self.handle = C.c_void_p()
        check(lib().one_cuda_init(device, workspace_bytes, C.byref(self.handle)))
        self.device = device

    @property
    def stream(self):
        return lib().one_cuda_stream(self.handle)

    def status(self):
        check(lib().one_cuda_status(self.handle))

    def close(self):
        if self.handle:
            lib().one_cuda_release(self.handle)
            self.handle = C.c_void_p()


class Packed:
    """one_packed: a prepared Conv / Gemm / MatMul."""

    def __init__(self, ctx, op_type, args, flags):
        self.ctx = ctx
        self.handle = C.c_void_p()
        check(lib().one_cuda_prepare(ctx.handle, op_type.encode(), args.params, args.inputs, flags, C.byref(self.handle)))

    def eval_async(self, args, stream=None):
        check(lib().one_cuda_eval_async(self.ctx.handle, self.handle, args.params, args.inputs, args.outputs, stream))

    def set_requant(self, scale):
        check(lib().one_cuda_packed_set_requant(self.handle, scale))

    def work(self):
        f, b = C.c_double(), C.c_double()
        check(lib().one_cuda_packed_work(self.handle, C.byref(f), C.byref(b)))
        return f.value, b.value

    def close(self):
        if self.handle:
            lib().one_cuda_packed_release(self.handle)
            self.handle = C.c_void_p()
