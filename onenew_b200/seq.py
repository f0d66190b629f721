"""Thin wrappers of the token-sequence glue operators of ``include/one_glue.h`` (LayerNormalization,
Gelu, Softmax, Transpose, chunk copy, broadcasting arithmetic) for tests and scripts: numpy in,
numpy out, the work done by the CUDA kernels on the current device.  No CPU fallback exists."""
import ctypes as C

import numpy as np
import torch

from . import capi

_F = C.c_void_p


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ints(v):
    return (C.c_int * len(v))(*[int(i) for i in v])


def layernorm(x, w, b):
    xd, wd, bd = _dev(x), _dev(w), _dev(b)
    y = torch.empty_like(xd)
    D = x.shape[-1]
    capi.check(capi.lib().one_glue_layernorm(_F(xd.data_ptr()), _F(wd.data_ptr()), _F(bd.data_ptr()), _F(y.data_ptr()),
                                             C.c_longlong(xd.numel() // D), C.c_int(D), _stream()))
    return y.cpu().numpy()


def gelu(x, lut):
    xd, ld = _dev(x), _dev(lut)
    y = torch.empty_like(xd)
    capi.check(capi.lib().one_glue_gelu_lut(_F(xd.data_ptr()), _F(ld.data_ptr()), _F(y.data_ptr()), C.c_longlong(xd.numel()), _stream()))
    return y.cpu().numpy()


def softmax(x):
    xd = _dev(x)
    y = torch.empty_like(xd)
    D = x.shape[-1]
    capi.check(capi.lib().one_glue_softmax_rows(_F(xd.data_ptr()), _F(y.data_ptr()), C.c_longlong(xd.numel() // D), C.c_int(D), _stream()))
    return y.cpu().numpy()


def transpose(x, perm):
    xd = _dev(x)
    y = torch.empty([x.shape[p] for p in perm], dtype=torch.float32, device="cuda")
    capi.check(capi.lib().one_glue_transpose(_F(xd.data_ptr()), _F(y.data_ptr()), C.c_int(x.ndim), _ints(x.shape), _ints(perm), _stream()))
    return y.cpu().numpy()


def binary(op, a, b):
    """op: 0 add, 1 sub, 2 mul, 3 div, numpy broadcasting."""
    nd = max(a.ndim, b.ndim)
    sa = (1,) * (nd - a.ndim) + tuple(a.shape)
    sb = (1,) * (nd - b.ndim) + tuple(b.shape)
    ad, bd = _dev(a), _dev(b)
    y = torch.empty(np.broadcast_shapes(sa, sb), dtype=torch.float32, device="cuda")
    capi.check(capi.lib().one_glue_binary(C.c_int(op), _F(ad.data_ptr()), _F(bd.data_ptr()), _F(y.data_ptr()), C.c_int(nd),
                                          _ints(sa), _ints(sb), _stream()))
    return y.cpu().numpy()


def copy_chunks(x, out_elems, reps, chunk, x_reps, x_stride, y_stride, x_off=0, y_off=0, fill=0.0):
    xd = _dev(x)
    y = torch.full((out_elems,), fill, dtype=torch.float32, device="cuda")
    capi.check(capi.lib().one_glue_copy_chunks(_F(xd.data_ptr() + 4 * x_off), _F(y.data_ptr() + 4 * y_off), C.c_longlong(reps),
                                               C.c_longlong(chunk), C.c_longlong(x_reps), C.c_longlong(x_stride),
                                               C.c_longlong(y_stride), _stream()))
    return y.cpu().numpy()


def attention(qkv, heads, scale, ctx=None):
    """Fused self-attention on a [B, T, 3*D] tensor laid out q | k | v along the last axis."""
    own = ctx is None
    ctx = ctx or capi.Context()
    try:
        B, T, D3 = qkv.shape
        D = D3 // 3
        xd = _dev(qkv)
        y = torch.zeros((B, T, D), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        capi.check(capi.lib().one_cuda_attention(ctx.handle, _F(xd.data_ptr()), _F(y.data_ptr()), C.c_int(B), C.c_int(T),
                                                 C.c_int(heads), C.c_int(D // heads), C.c_int(D3), C.c_int(0), C.c_int(D),
                                                 C.c_int(2 * D), C.c_int(D), C.c_float(scale), _stream()))
        torch.cuda.synchronize()
        ctx.status()             # raises if a device-side wait ran out
        return y.cpu().numpy()
    finally:
        if own:
            ctx.close()
