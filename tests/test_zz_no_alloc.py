"""The allocation-free Conv entry point (one_cuda_conv_eval_static).

Some embedders cannot let this library allocate device memory: their memory budget went to an arena
of their own at start-up, a device allocation would break their latency budget, or the allocator is
simply not theirs to call.  For them the library carries a fixed scratch array in its own image and
this entry point computes the same Conv out of it.  The file is named so that pytest collects it
last; it passes when run alone in a fresh process and when run after the other GPU tests.

Checked here, through the C ABI: two calls in a row (the second on a smaller, different problem, so
leftovers of the first call in the shared array would show) give the same result as the regular
entry point one_cuda_conv_eval within the float tolerance of the suite; the int8 path stays bit
exact; a shape whose scratch exceeds the array is refused with ONE_ERR_NOMEM; and the amount of free
device memory does not move across a call (after the first, which may load the kernels).
"""
import numpy as np
import pytest

from common import assert_close
from onenew_b200 import abi, capi

pytestmark = pytest.mark.gpu


def _conv_both(x, w, b, strides, pads, act, int8=None, lut=None):
    """Run the regular drop-in and the static-scratch variant on the same device buffers."""
    import torch
    L = capi.lib()
    xd = torch.from_numpy(x).cuda()
    N, C, H, W = x.shape
    OC, _, KH, KW = w.shape
    OH = (H + pads[0] + pads[2] - KH) // strides[1] + 1
    OW = (W + pads[1] + pads[3] - KW) // strides[0] + 1
    if int8 is not None:
        wd = torch.zeros(w.size, dtype=torch.float32, device="cuda")
        wd.view(torch.int8)[:w.size] = torch.from_numpy(np.ascontiguousarray(w, np.int8).ravel()).cuda()
        bd = torch.from_numpy(np.asarray(b, np.int32)).cuda()
        cfg = abi.conv_cfg((KH, KW), strides, pads, act=act, int8_scale=int8[0], weight_aux=int8[1])
    else:
        wd = torch.from_numpy(w).cuda()
        bd = torch.from_numpy(b).cuda()
        cfg = abi.conv_cfg((KH, KW), strides, pads, act=act)
    lutd = torch.from_numpy(lut).cuda() if lut is not None else None
    outs = []
    for which in ("regular", "static"):
        y = torch.full((N, OC, OH, OW), float("nan"), dtype=torch.float32, device="cuda")
        a = abi.conv_eval_args(cfg, x.shape, w.shape, tuple(y.shape), xd.data_ptr(), wd.data_ptr(), bd.data_ptr(),
                               y.data_ptr(), abi.default_useful_info(), lutd.data_ptr() if lutd is not None else 0)
        torch.cuda.synchronize()
        if which == "regular":
            capi.check(L.one_cuda_conv_eval(a.params, a.inputs, a.outputs))
        else:
            capi.check(L.one_cuda_conv_eval_static(a.params, a.inputs, a.outputs, None))
        outs.append(y.cpu().numpy())
    return outs


def test_static_scratch_conv_matches_regular_entry_point_twice(oracle_mod):
    rng = np.random.default_rng(11)
    # call 1: the single-operator configuration at batch 2 (tensor-map im2col path)
    x = rng.uniform(-1, 1, (2, 64, 56, 56)).astype(np.float32)
    w = (rng.standard_normal((64, 64, 3, 3)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(64) * 0.01).astype(np.float32)
    reg, sta = _conv_both(x, w, b, (1, 1), (1, 1, 1, 1), abi.RELU)
    assert_close(sta, reg, "static vs regular, call 1")
    assert_close(sta, oracle_mod.conv_f32(x, w, b, (1, 1), (1, 1, 1, 1), abi.RELU), "static vs oracle, call 1")
    # call 2, straight after: a smaller stride-2 stem-like problem (space-to-depth path) that leaves most
    # of the first call's bytes in the shared array untouched
    x2 = rng.uniform(-1, 1, (1, 3, 32, 32)).astype(np.float32)
    w2 = (rng.standard_normal((16, 3, 7, 7)) * 0.05).astype(np.float32)
    b2 = (rng.standard_normal(16) * 0.01).astype(np.float32)
    reg2, sta2 = _conv_both(x2, w2, b2, (2, 2), (3, 3, 3, 3), abi.RELU)
    assert_close(sta2, reg2, "static vs regular, call 2")
    assert_close(sta2, oracle_mod.conv_f32(x2, w2, b2, (2, 2), (3, 3, 3, 3), abi.RELU), "static vs oracle, call 2")


def test_static_scratch_int8_bit_exact(oracle_mod):
    rng = np.random.default_rng(12)
    x = rng.uniform(0, 1, (1, 32, 40, 40)).astype(np.float32)
    w = (rng.standard_normal((64, 32, 3, 3)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(64) * 0.01).astype(np.float32)
    w8, b32, aux = oracle_mod.quant_weight_bias(w, b)
    scale = np.float32(0.9 / 127)
    ref, _, _ = oracle_mod.conv_s8(x, w8, b32, aux, scale, (2, 2), 1, abi.SILU)
    reg, sta = _conv_both(x, w8, b32, (2, 2), (1, 1, 1, 1), abi.SILU, int8=(float(scale), aux), lut=oracle_mod.silu_lut())
    assert np.array_equal(sta, reg) and np.array_equal(sta, ref)


def test_static_scratch_refuses_oversize():
    import torch
    L = capi.lib()
    # 64 x 64 x 112 x 112 in and out: ~400 MB of NHWC copies, far beyond the 32 MiB array
    x = torch.zeros((64, 64, 112, 112), device="cuda")
    w = torch.zeros((64, 64, 3, 3), device="cuda")
    b = torch.zeros(64, device="cuda")
    y = torch.zeros((64, 64, 112, 112), device="cuda")
    cfg = abi.conv_cfg((3, 3), (1, 1), (1, 1, 1, 1))
    a = abi.conv_eval_args(cfg, tuple(x.shape), tuple(w.shape), tuple(y.shape), x.data_ptr(), w.data_ptr(), b.data_ptr(),
                           y.data_ptr(), abi.default_useful_info())
    rc = L.one_cuda_conv_eval_static(a.params, a.inputs, a.outputs, None)
    assert rc == -5 and b"built-in array" in L.one_cuda_last_error()


def test_static_scratch_call_leaves_free_device_memory_unchanged():
    """What the entry point is for: once the kernels are loaded (first call), a call takes no device memory
    and gives none back.  The output tensor and the operands exist before the measurement starts."""
    import torch
    L = capi.lib()
    rng = np.random.default_rng(13)
    x = torch.from_numpy(rng.uniform(-1, 1, (2, 32, 28, 28)).astype(np.float32)).cuda()
    w = torch.from_numpy((rng.standard_normal((32, 32, 3, 3)) * 0.05).astype(np.float32)).cuda()
    b = torch.from_numpy((rng.standard_normal(32) * 0.01).astype(np.float32)).cuda()
    y = torch.zeros((2, 32, 28, 28), device="cuda")
    cfg = abi.conv_cfg((3, 3), (1, 1), (1, 1, 1, 1), act=abi.RELU)
    a = abi.conv_eval_args(cfg, tuple(x.shape), tuple(w.shape), tuple(y.shape), x.data_ptr(), w.data_ptr(), b.data_ptr(),
                           y.data_ptr(), abi.default_useful_info())
    capi.check(L.one_cuda_conv_eval_static(a.params, a.inputs, a.outputs, None))      # loads whatever is loaded lazily
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        capi.check(L.one_cuda_conv_eval_static(a.params, a.inputs, a.outputs, None))
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, (free0, free1)
