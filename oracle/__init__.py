"""CPU checkers for the Conv / Gemm / MatMul path.  TEST INFRASTRUCTURE ONLY.

Two checkers live here:

* ``port``      -- ``liboracle.so``, the plain-C restatement in ``oracle.c``;
* ``reference`` -- ``_ref/lib<Op>_x86.so``, the reference's own x86 operator sources compiled
  unmodified by ``oracle/Makefile`` and driven through their ``eval`` ABI exactly as the
  reference host does (host/op.h:109-185, host/ops/conv.h:133-157).

Only tests, the smoke test and the benchmark's CPU-baseline leg may import this package.  The
product package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

from onenew_b200 import abi

_DIR = os.path.dirname(os.path.abspath(__file__))
_REF_DIR = os.path.join(_DIR, "_ref")
_port = None
_ref_libs = {}
_scratch = None

f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")


def build(quiet=True):
    """Run the Makefile (restatement always; reference ops when the reference tree exists)."""
    subprocess.run(["make", "-C", _DIR], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def port():
    global _port
    if _port is None:
        path = os.path.join(_DIR, "liboracle.so")
        if not os.path.exists(path):
            build()
        _port = C.CDLL(path)
    return _port


def have_reference(op="Conv"):
    return os.path.exists(os.path.join(_REF_DIR, f"lib{op}_x86.so"))


def ref_eval(op):
    """``eval`` of the reference's compiled x86 operator library."""
    if op not in _ref_libs:
        lib = C.CDLL(os.path.join(_REF_DIR, f"lib{op}_x86.so"))
        fn = lib.eval
        fn.restype = C.c_int
        fn.argtypes = [C.POINTER(abi.BUFFER_INFO_S)] * 3
        _ref_libs[op] = (lib, fn)
    return _ref_libs[op][1]


def _public_buf(nbytes=1 << 29):
    """The reference's shared scratch buffer; 512 MiB is its converter default
    (tools/onnx2one/onnx2one.cpp:1331-1350)."""
    global _scratch
    if _scratch is None or _scratch.nbytes < nbytes:
        _scratch = _aligned((nbytes,), np.uint8)
    return _scratch


def _aligned(shape, dtype=np.float32, fill=None):
    """64-byte aligned array: the reference host hands its operators aligned_alloc'ed buffers
    (host/net.h:434-449) and the AVX2 SGEMM uses aligned loads on them."""
    n = int(np.prod(shape)) * np.dtype(dtype).itemsize
    raw = np.zeros(n + 64, np.uint8)
    off = (-raw.ctypes.data) % 64
    a = raw[off:off + n].view(dtype).reshape(shape)
    if fill is not None:
        a[...] = fill
    return a


def _addr(a):
    return a.ctypes.data if a is not None else 0


def conv_out_hw(H, W, KH, KW, strides, pads):
    """host/ops/conv.h:31-58; strides = (x, y), pads = (top, left, bottom, right)."""
    return ((H + pads[0] + pads[2] - KH) // strides[1] + 1, (W + pads[1] + pads[3] - KW) // strides[0] + 1)


def silu_lut():
    lut = np.empty(8192, np.float32)
    port().oracle_silu_lut(lut.ctypes.data_as(C.c_void_p))
    return lut


def gelu_lut():
    lut = np.empty(8192, np.float32)
    port().oracle_gelu_lut(lut.ctypes.data_as(C.c_void_p))
    return lut


# ----------------------------------------------------------------------------- port
def act(y, act_type, clip=(0.0, 6.0), leaky=0.01, hs=(1 / 6.0, 0.5), lut=None):
    y = np.ascontiguousarray(y, np.float32).copy()
    if act_type == abi.SILU and lut is None:
        lut = silu_lut()
    port().oracle_act(C.c_void_p(_addr(y)), C.c_int64(y.size), C.c_int(act_type), C.c_float(clip[0]),
                      C.c_float(clip[1]), C.c_float(leaky), C.c_float(hs[0]), C.c_float(hs[1]),
                      C.c_void_p(_addr(lut)))
    return y


def conv_f32(x, w, b, strides=(1, 1), pads=(0, 0, 0, 0), act_type=abi.NOT_ACT, **act_kw):
    """Restated fp32 Conv (+bias, +activation).  A bias-less conv gets no activation, as in
    the reference (device/x86/Conv/conv.c:18-27)."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    N, Cc, H, W = x.shape
    OC, _, KH, KW = w.shape
    OH, OW = conv_out_hw(H, W, KH, KW, strides, pads)
    y = np.empty((N, OC, OH, OW), np.float32)
    bb = None if b is None else np.ascontiguousarray(b, np.float32)
    port().oracle_conv_f32(C.c_void_p(_addr(x)), C.c_void_p(_addr(w)), C.c_void_p(_addr(bb)),
                           C.c_void_p(_addr(y)), N, Cc, H, W, OC, KH, KW, strides[0], strides[1],
                           pads[0], pads[1], pads[2], pads[3])
    if b is not None and act_type != abi.NOT_ACT:
        y = act(y, act_type, **act_kw)
    return y


def dwconv_f32(x, w, b, strides=(1, 1), pads=(0, 0, 0, 0), act_type=abi.NOT_ACT, **act_kw):
    """Restated depthwise fp32 Conv (weight [C][1][KH][KW])."""
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    N, Cc, H, W = x.shape
    _, _, KH, KW = w.shape
    OH, OW = conv_out_hw(H, W, KH, KW, strides, pads)
    y = np.empty((N, Cc, OH, OW), np.float32)
    bb = None if b is None else np.ascontiguousarray(b, np.float32)
    port().oracle_dwconv_f32(C.c_void_p(_addr(x)), C.c_void_p(_addr(w)), C.c_void_p(_addr(bb)), C.c_void_p(_addr(y)),
                             N, Cc, H, W, KH, KW, strides[0], strides[1], pads[0], pads[1], pads[2], pads[3])
    if b is not None and act_type != abi.NOT_ACT:
        y = act(y, act_type, **act_kw)
    return y


def dwconv_s8(x, w8, b32, aux, input_scale, strides=(1, 1), pad=0, act_type=abi.NOT_ACT, **act_kw):
    """Restated depthwise int8 Conv (weight int8 [C][1][KH][KW], bias int32)."""
    x = np.ascontiguousarray(x, np.float32)
    w8 = np.ascontiguousarray(w8, np.int8)
    N, Cc, H, W = x.shape
    _, _, KH, KW = w8.shape
    OH, OW = conv_out_hw(H, W, KH, KW, strides, (pad,) * 4)
    y = np.empty((N, Cc, OH, OW), np.float32)
    aux = np.ascontiguousarray(aux, np.float32)
    bb = None if b32 is None else np.ascontiguousarray(b32, np.int32)
    port().oracle_dwconv_s8(C.c_void_p(_addr(x)), C.c_void_p(_addr(w8)), C.c_void_p(_addr(bb)), C.c_void_p(_addr(y)),
                            N, Cc, H, W, KH, KW, strides[0], strides[1], pad, C.c_float(input_scale),
                            C.c_void_p(_addr(aux)))
    if b32 is not None and act_type != abi.NOT_ACT:
        y = act(y, act_type, **act_kw)
    return y


def quant_weight_bias(w, b):
    """Q1: per-OC truncating int8 weights, s32 bias, weight_aux (model_quant.hpp:6-29)."""
    w = np.ascontiguousarray(w, np.float32)
    OC = w.shape[0]
    inner = w.size // OC
    w8 = np.empty(w.shape, np.int8)
    b32 = np.empty(OC, np.int32)
    aux = np.empty(OC, np.float32)
    bb = None if b is None else np.ascontiguousarray(b, np.float32)
    port().oracle_quant_weight_bias(C.c_void_p(_addr(w)), C.c_void_p(_addr(bb)), OC, inner,
                                    C.c_void_p(_addr(w8)), C.c_void_p(_addr(b32)), C.c_void_p(_addr(aux)))
    return w8, (b32 if b is not None else None), aux


def quantize_s8(x, input_scale):
    x = np.ascontiguousarray(x, np.float32)
    q = np.empty(x.shape, np.int8)
    port().oracle_quantize_s8(C.c_void_p(_addr(x)), C.c_void_p(_addr(q)), C.c_int64(x.size),
                              C.c_float(input_scale))
    return q


def conv_s8(x, w8, b32, aux, input_scale, strides=(1, 1), pad=0, act_type=abi.NOT_ACT, **act_kw):
    """Restated int8 Conv.  Returns (y fp32, s32 accumulators, quantised input)."""
    x = np.ascontiguousarray(x, np.float32)
    w8 = np.ascontiguousarray(w8, np.int8)
    N, Cc, H, W = x.shape
    OC, _, KH, KW = w8.shape
    OH, OW = conv_out_hw(H, W, KH, KW, strides, (pad,) * 4)
    y = np.empty((N, OC, OH, OW), np.float32)
    acc = np.empty((N, OC, OH, OW), np.int32)
    q = np.empty(x.shape, np.int8)
    aux = np.ascontiguousarray(aux, np.float32)
    port().oracle_conv_s8(C.c_void_p(_addr(x)), C.c_void_p(_addr(w8)), C.c_void_p(_addr(b32)),
                          C.c_void_p(_addr(y)), C.c_void_p(_addr(acc)), C.c_void_p(_addr(q)),
                          N, Cc, H, W, OC, KH, KW, strides[0], strides[1], pad,
                          C.c_float(input_scale), C.c_void_p(_addr(aux)))
    if b32 is not None and act_type != abi.NOT_ACT:
        y = act(y, act_type, **act_kw)
    return y, acc, q


def mse_input_scale(samples):
    """Q2 + Q3 for one Conv input: ``samples`` is the list of that operand's fp32 values over the
    calibration images (the same images serve both passes; the reference's second pass keeps reading
    its image list where the first stopped, model_quant.hpp:541).  Returns input_scale."""
    L = port()
    L.oracle_abs_max.restype = C.c_float
    L.oracle_mse_threshold.restype = C.c_float
    mx = 0.0
    arrs = [np.ascontiguousarray(a, np.float32) for a in samples]
    for a in arrs:
        mx = L.oracle_abs_max(C.c_void_p(_addr(a)), C.c_int64(a.size), C.c_float(mx))
    hist = np.zeros(2048, np.float32)
    for a in arrs:
        L.oracle_hist_accumulate(C.c_void_p(_addr(a)), C.c_int64(a.size), C.c_float(mx), C.c_void_p(_addr(hist)))
    thr = L.oracle_mse_threshold(C.c_void_p(_addr(hist)), C.c_int32(arrs[0].size * len(arrs)), C.c_float(mx))
    return np.float32(np.float32(thr) / np.float32(127))


def _stats(samples):
    L = port()
    L.oracle_abs_max.restype = C.c_float
    arrs = [np.ascontiguousarray(a, np.float32) for a in samples]
    mx = 0.0
    for a in arrs:
        mx = L.oracle_abs_max(C.c_void_p(_addr(a)), C.c_int64(a.size), C.c_float(mx))
    hist = np.zeros(2048, np.float32)
    for a in arrs:
        L.oracle_hist_accumulate(C.c_void_p(_addr(a)), C.c_int64(a.size), C.c_float(mx), C.c_void_p(_addr(hist)))
    return arrs, mx, hist


def kl_input_scale(samples):
    """The KL method for one Conv input (tools/optimize/model_quant.hpp:197-435); ``samples`` as in
    mse_input_scale.  Returns input_scale."""
    arrs, mx, hist = _stats(samples)
    L = port()
    L.oracle_kl_threshold.restype = C.c_float
    thr = L.oracle_kl_threshold(C.c_void_p(_addr(hist)), C.c_int32(arrs[0].size * len(arrs)), C.c_float(mx))
    return np.float32(np.float32(thr) / np.float32(127))


def percent_input_scale(samples):
    """The percent method for one Conv input (tools/optimize/model_quant.hpp:83-185): per image the
    (int)(elem * (1 - 0.99998f) * 10) largest |x| are kept (full sort by falling |x|), the kept values
    of all images (in a zero-filled vector of (int)(n_img * elem * (1 - p) * 10) entries) are sorted
    again and entry (int)((1 - p) * n_img * elem) is the (signed) threshold."""
    f = np.float32
    pct = f(99.998 / 100)
    arrs = [np.ascontiguousarray(a, np.float32).ravel() for a in samples]
    elem, n_img = arrs[0].size, len(arrs)
    reserve = int(f(f(elem) * (f(1) - pct)) * f(10))
    total = int(f(f(n_img * elem) * (f(1) - pct)) * f(10))
    big = np.zeros(max(total, n_img * reserve), np.float32)
    for i, a in enumerate(arrs):
        big[i * reserve:(i + 1) * reserve] = a[np.argsort(-np.abs(a), kind="stable")][:reserve]
    big = big[np.argsort(-np.abs(big), kind="stable")]
    idx = int(f(f(f(1) - pct) * f(n_img)) * f(elem))
    return f(big[idx] / f(127))


def gemm(a, w, b):
    a = np.ascontiguousarray(a, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    M, K = a.shape[-2], a.shape[-1]
    N = w.shape[0]
    y = np.empty((M, N), np.float32)
    port().oracle_gemm(C.c_void_p(_addr(a)), C.c_void_p(_addr(w)), C.c_void_p(_addr(b)),
                       C.c_void_p(_addr(y)), M, N, K)
    return y


def matmul(a, b):
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    M, K = a.shape[-2], a.shape[-1]
    N = b.shape[-1]
    batch = int(np.prod(a.shape[:-2])) if a.ndim > 2 else 1
    y = np.empty(a.shape[:-1] + (N,), np.float32)
    port().oracle_matmul(C.c_void_p(_addr(a)), C.c_void_p(_addr(b)), C.c_void_p(_addr(y)),
                         batch, M, N, K, C.c_int64(b.size))
    return y


# ------------------------------------------------------------------------ reference
def ref_conv(x, w, b, strides=(1, 1), pads=(0, 0, 0, 0), act_type=abi.NOT_ACT, int8=None, **cfg_kw):
    """Reference ``eval`` of Conv on one or more images (one call per image: the reference
    forces N=1, host/ops/conv.h:43).  ``int8`` = (input_scale, weight_aux): then ``w`` is int8
    OIHW and ``b`` int32, laid out at the start of fp32-sized buffers as the reference's
    in-place quantiser leaves them (model_quant.hpp:6-29, host/ops/conv.h:60-131)."""
    x = _aligned(np.shape(x), np.float32, x)
    N, Cc, H, W = x.shape
    OC, _, KH, KW = w.shape
    OH, OW = conv_out_hw(H, W, KH, KW, strides, pads)
    y = _aligned((N, OC, OH, OW))
    wbuf = _aligned((w.size,))
    bbuf = _aligned((OC,))
    if int8 is not None:
        wbuf.view(np.int8)[:w.size] = np.ascontiguousarray(w, np.int8).ravel()
        if b is not None:
            bbuf.view(np.int32)[:] = b
        cfg = abi.conv_cfg((KH, KW), strides, pads, has_bias=b is not None, act=act_type,
                           int8_scale=int8[0], weight_aux=int8[1], **cfg_kw)
    else:
        wbuf[:] = np.ascontiguousarray(w, np.float32).ravel()
        if b is not None:
            bbuf[:] = b
        cfg = abi.conv_cfg((KH, KW), strides, pads, has_bias=b is not None, act=act_type, **cfg_kw)
    lut = silu_lut() if act_type == abi.SILU else None
    scratch = _public_buf()
    useful = abi.default_useful_info(scratch.ctypes.data, scratch.nbytes)
    fn = ref_eval("Conv")
    for n in range(N):
        args = abi.conv_eval_args(cfg, (1, Cc, H, W), w.shape, (1, OC, OH, OW), x[n].ctypes.data,
                                  wbuf.ctypes.data, bbuf.ctypes.data, y[n].ctypes.data, useful, _addr(lut))
        fn(args.params, args.inputs, args.outputs)
    return y


def ref_gemm(a, w, b):
    a = _aligned(np.shape(a), np.float32, a)
    w = _aligned(np.shape(w), np.float32, w)
    b = _aligned(np.shape(b), np.float32, b)
    M, K = a.shape[-2], a.shape[-1]
    N = w.shape[0]
    y = _aligned((M, N))
    args = abi.gemm_eval_args(a.shape, w.shape, y.shape, a.ctypes.data, w.ctypes.data, b.ctypes.data,
                              y.ctypes.data)
    ref_eval("Gemm")(args.params, args.inputs, args.outputs)
    return y


def ref_matmul(a, b):
    a = _aligned(np.shape(a), np.float32, a)
    b = _aligned(np.shape(b), np.float32, b)
    y = _aligned(a.shape[:-1] + (b.shape[-1],))
    args = abi.matmul_eval_args(a.shape, b.shape, y.shape, a.ctypes.data, b.ctypes.data, y.ctypes.data)
    ref_eval("MatMul")(args.params, args.inputs, args.outputs)
    return y


# ------------------------------------------------------------------ the reference's quantiser arithmetic
# _ref/libquant_ref.so holds fragments of tools/optimize/model_quant.hpp compiled from the reference tree
# (oracle/Makefile target quant_ref, wrapper oracle/quant_ref_wrap.cpp).  They pin the restated quantiser
# above and the product's; they are test infrastructure like everything else in this package.
_quant_ref = None


def have_quant_reference():
    return os.path.exists(os.path.join(_REF_DIR, "libquant_ref.so"))


def quant_ref():
    global _quant_ref
    if _quant_ref is None:
        L = C.CDLL(os.path.join(_REF_DIR, "libquant_ref.so"))
        L.ref_abs_max.restype = C.c_float
        L.ref_mse_threshold.restype = C.c_float
        L.ref_kl_threshold.restype = C.c_float
        L.ref_percent_threshold.restype = C.c_float
        _quant_ref = L
    return _quant_ref


def ref_quant_weight_bias(w, b):
    """quant_weight_bias of the reference (model_quant.hpp:6-29) on copies of w [OC][C][KH][KW] and b: it
    works in place, leaving int8 weights and int32 biases at the start of the float buffers."""
    w = np.ascontiguousarray(w, np.float32)
    OC = w.shape[0]
    wbuf = _aligned(w.shape, np.float32, w)
    bbuf = _aligned((OC,), np.float32, np.ascontiguousarray(b, np.float32))
    cfg = abi.CONV_CONFIG_S()
    shapes = (C.c_int32 * 8)(*([int(v) for v in w.shape] + [1] * (8 - w.ndim)))
    quant_ref().ref_quant_weight_bias(C.byref(cfg), C.c_void_p(_addr(wbuf)), C.c_void_p(_addr(bbuf)), shapes)
    w8 = wbuf.view(np.int8).ravel()[:w.size].reshape(w.shape).copy()
    b32 = bbuf.view(np.int32).copy()
    aux = np.array(cfg.weight_aux[:OC], np.float32)
    return w8, b32, aux


def ref_stats(samples):
    """Running max |x| (model_quant.hpp:526-533) and the 2048-bin histogram (:323-329) over the samples."""
    L = quant_ref()
    arrs = [np.ascontiguousarray(a, np.float32) for a in samples]
    mx = 0.0
    for a in arrs:
        mx = L.ref_abs_max(C.c_void_p(_addr(a)), C.c_int64(a.size), C.c_float(mx))
    hist = np.zeros(2048, np.float32)
    for a in arrs:
        L.ref_hist_accumulate(C.c_void_p(_addr(a)), C.c_int64(a.size), C.c_float(mx), C.c_void_p(_addr(hist)))
    return mx, hist


def ref_mse_threshold(hist, elem_count, max_abs):
    hist = np.ascontiguousarray(hist, np.float32)
    return np.float32(quant_ref().ref_mse_threshold(C.c_void_p(_addr(hist)), C.c_int32(elem_count), C.c_float(max_abs)))


def ref_kl_threshold(hist, elem_count, max_abs):
    hist = np.ascontiguousarray(hist, np.float32)
    return np.float32(quant_ref().ref_kl_threshold(C.c_void_p(_addr(hist)), C.c_int32(elem_count), C.c_float(max_abs)))


def ref_percent_threshold(samples):
    arrs = [np.ascontiguousarray(a, np.float32).ravel() for a in samples]
    ptrs = (C.c_void_p * len(arrs))(*[_addr(a) for a in arrs])
    return np.float32(quant_ref().ref_percent_threshold(ptrs, C.c_int32(len(arrs)), C.c_int32(arrs[0].size)))


def ref_silu_lut():
    """The SiLU table as the reference host builds it (host/ops/conv.h:180-188)."""
    lut = np.empty(8192, np.float32)
    quant_ref().ref_silu_lut(lut.ctypes.data_as(C.c_void_p))
    return lut


def ref_gelu_lut():
    """The Gelu table as the reference host builds it (host/ops/gelu.h:82-91)."""
    lut = np.empty(8192, np.float32)
    quant_ref().ref_gelu_lut(lut.ctypes.data_as(C.c_void_p))
    return lut
