"""Host-side mirror of the reference's Conv / Gemm / MatMul operator calls for device tensors.

Each function builds the ``params / inputs / outputs`` arrays the way the reference host does
(host/op.h:109-168, host/ops/conv.h:133-157) around torch CUDA tensors (used for device memory
only) and calls the ``eval`` symbol of the drop-in library ``lib<Op>_cu.so``.  Shapes and
layouts are the reference's: NCHW fp32 activations, OIHW weights, [N][K] Gemm weights.
"""
import numpy as np
import torch

from . import abi, capi


def _dev(a, dtype=torch.float32):
    if isinstance(a, torch.Tensor):
        return a.to("cuda", dtype).contiguous()
    return torch.from_numpy(np.ascontiguousarray(a)).to("cuda").to(dtype).contiguous()


def out_hw(H, W, KH, KW, strides, pads):
    return ((H + pads[0] + pads[2] - KH) // strides[1] + 1, (W + pads[1] + pads[3] - KW) // strides[0] + 1)


def conv(x, w, b, strides=(1, 1), pads=(0, 0, 0, 0), act=abi.NOT_ACT, int8=None, lut=None, **cfg_kw):
    """Conv through ``libConv_cu.so:eval``.  ``int8=(input_scale, weight_aux)``: ``w`` is the
    int8 OIHW weight and ``b`` the int32 bias, placed at the start of fp32-sized buffers as the
    reference's quantiser leaves them (tools/optimize/model_quant.hpp:6-29)."""
    xd = _dev(x)
    N, Cc, H, W = xd.shape
    OC, _, KH, KW = w.shape   # depthwise: pass group=C in cfg_kw, weight [C][1][KH][KW]
    OH, OW = out_hw(H, W, KH, KW, strides, pads)
    if int8 is not None:
        wd = torch.zeros(int(np.prod(w.shape)), dtype=torch.float32, device="cuda")
        wd.view(torch.int8)[: wd.numel()] = _dev(np.asarray(w, np.int8).ravel(), torch.int8)
        bd = None
        if b is not None:
            bd = _dev(np.asarray(b, np.int32), torch.int32)
        cfg = abi.conv_cfg((KH, KW), strides, pads, has_bias=b is not None, act=act, int8_scale=int8[0],
                           weight_aux=int8[1], **cfg_kw)
    else:
        wd = _dev(w)
        bd = _dev(b) if b is not None else None
        cfg = abi.conv_cfg((KH, KW), strides, pads, has_bias=b is not None, act=act, **cfg_kw)
    lutd = _dev(lut) if lut is not None else None
    y = torch.empty((N, OC, OH, OW), dtype=torch.float32, device="cuda")
    useful = abi.default_useful_info()
    args = abi.conv_eval_args(cfg, (N, Cc, H, W), tuple(w.shape), (N, OC, OH, OW), xd.data_ptr(), wd.data_ptr(),
                              bd.data_ptr() if bd is not None else 0, y.data_ptr(), useful,
                              lutd.data_ptr() if lutd is not None else 0)
    capi.check(capi.shim_eval("Conv")(args.params, args.inputs, args.outputs))
    return y


def gemm(a, w, b):
    ad, wd, bd = _dev(a), _dev(w), _dev(b)
    M, N = ad.shape[-2], wd.shape[0]
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    args = abi.gemm_eval_args(tuple(ad.shape), tuple(wd.shape), (M, N), ad.data_ptr(), wd.data_ptr(), bd.data_ptr(),
                              y.data_ptr())
    capi.check(capi.shim_eval("Gemm")(args.params, args.inputs, args.outputs))
    return y


def matmul(a, b):
    ad, bd = _dev(a), _dev(b)
    y = torch.empty(tuple(ad.shape[:-1]) + (bd.shape[-1],), dtype=torch.float32, device="cuda")
    args = abi.matmul_eval_args(tuple(ad.shape), tuple(bd.shape), tuple(y.shape), ad.data_ptr(), bd.data_ptr(),
                                y.data_ptr())
    capi.check(capi.shim_eval("MatMul")(args.params, args.inputs, args.outputs))
    return y
