"""ABI layout and library-surface checks (CPU only)."""
import ctypes as C
import os
import re
import subprocess

import pytest

from onenew_b200 import abi, capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_static_asserts_compile_as_c_and_cxx(tmp_path):
    for comp, std, lang in (("gcc", "-std=c11", "c"), ("g++", "-std=c++17", "c++")):
        subprocess.run([comp, std, "-fsyntax-only", "-x", lang, os.path.join(ROOT, "include", "one_cuda.h")], check=True)


def test_ctypes_mirror_matches_reference_sizes():
    # sizes measured on the reference build (gcc 13, x86-64)
    assert C.sizeof(abi.CONV_CONFIG_S) == 29376
    assert C.sizeof(abi.OPERAND_S) == 312
    assert abi.OPERAND_S.shapes.offset == 276
    assert abi.BASE_CONFIG_S.in_operand_num.offset == 4608
    assert abi.CONV_CONFIG_S.strides.offset == 12920
    assert abi.CONV_CONFIG_S.input_scale.offset == 12980


def _declared_symbols(header="one_cuda.h", prefix="one_cuda_"):
    text = open(os.path.join(ROOT, "include", header)).read()
    return sorted(set(re.findall(r"ONE_API[^;(]*?\b(" + prefix + r"\w+)\s*\(", text)))


def test_binding_lists_every_declared_symbol():
    assert _declared_symbols() == sorted(capi.API_SYMBOLS)


def test_library_loads_and_exports_every_symbol():
    if not os.path.exists(capi.lib_path()):
        import __graft_entry__
        __graft_entry__.build()
    L = capi.lib()
    for s in (_declared_symbols() + _declared_symbols("one_glue.h", "one_glue_") + _declared_symbols("one_glue.h", "one_quant_") +
              _declared_symbols("one_net.h", "one_net_")):
        assert hasattr(L, s), s
    from onenew_b200 import net as onet
    assert sorted(onet.NET_SYMBOLS) == _declared_symbols("one_net.h", "one_net_")
    for op in ("Conv", "Gemm", "MatMul"):
        assert capi.shim_eval(op) is not None   # lib<Op>_cu.so exports `eval`


def test_no_gpu_fails_loudly_not_silently():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = capi.lib().one_cuda_init(0, 0, C.byref(h))
    assert rc == -4 and b"no CPU fallback" in capi.lib().one_cuda_last_error()
    args = abi.gemm_eval_args((1, 8), (8, 8), (1, 8), 16, 16, 16, 16)
    assert capi.shim_eval("Gemm")(args.params, args.inputs, args.outputs) == -4


def test_bad_descriptors_are_rejected_before_any_launch():
    L = capi.lib()
    # null arrays
    assert L.one_cuda_conv_eval(None, None, None) == -1
    # grouped conv -> UNSUPPORTED, wrong output shape -> BAD_SHAPE, int8 with unequal pads -> UNSUPPORTED
    u = abi.default_useful_info()
    cfg = abi.conv_cfg((3, 3), (1, 1), (1, 1, 1, 1), group=2)
    a = abi.conv_eval_args(cfg, (1, 8, 8, 8), (8, 8, 3, 3), (1, 8, 8, 8), 16, 16, 16, 16, u)
    assert L.one_cuda_conv_eval(a.params, a.inputs, a.outputs) == -3
    cfg = abi.conv_cfg((3, 3), (1, 1), (1, 1, 1, 1))
    a = abi.conv_eval_args(cfg, (1, 8, 8, 8), (8, 8, 3, 3), (1, 8, 7, 8), 16, 16, 16, 16, u)
    assert L.one_cuda_conv_eval(a.params, a.inputs, a.outputs) == -2
    a = abi.conv_eval_args(cfg, (1, 8, 8, 8), (8, 4, 3, 3), (1, 8, 8, 8), 16, 16, 16, 16, u)
    assert L.one_cuda_conv_eval(a.params, a.inputs, a.outputs) == -2
    cfg = abi.conv_cfg((3, 3), (1, 1), (1, 0, 1, 0), int8_scale=0.01, weight_aux=[1.0] * 8)
    a = abi.conv_eval_args(cfg, (1, 8, 8, 8), (8, 8, 3, 3), (1, 8, 8, 6), 16, 16, 16, 16, u)
    assert L.one_cuda_conv_eval(a.params, a.inputs, a.outputs) == -3
    # null tensor pointer
    cfg = abi.conv_cfg((3, 3), (1, 1), (1, 1, 1, 1))
    a = abi.conv_eval_args(cfg, (1, 8, 8, 8), (8, 8, 3, 3), (1, 8, 8, 8), 0, 16, 16, 16, u)
    assert L.one_cuda_conv_eval(a.params, a.inputs, a.outputs) == -1
    m = abi.matmul_eval_args((2, 4, 8), (3, 8, 5), (2, 4, 5), 16, 16, 16)
    assert L.one_cuda_matmul_eval(m.params, m.inputs, m.outputs) == -2
