"""GPU parity of the drop-in operators: lib<Op>_cu.so:eval against the CPU oracle and the golden
vectors made by the reference's own x86 operators.

Float path: cosine >= 0.9999 and max|a-b|/max|b| <= 1e-2 per tensor.  int8 path: bit exact
(fp32 outputs included, since the de-quantisation epilogue follows the reference's order)."""
import zlib

import numpy as np
import pytest

from common import assert_close, golden, golden_names
from onenew_b200 import abi, capi

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from onenew_b200 import ops as _ops
    return _ops


def _np(t):
    return t.cpu().numpy()


@pytest.mark.parametrize("name", [n for n in golden_names("conv") if not n.startswith("conv8")])
def test_conv_f32_golden(ops, oracle_mod, name):
    d = golden(name)
    m = d["meta"]
    s, pads, act, has_b = int(m[0]), tuple(int(v) for v in m[1:5]), int(m[5]), int(m[6])
    lut = oracle_mod.silu_lut() if act == abi.SILU else None
    y = _np(ops.conv(d["x"], d["w"], d["b"] if has_b else None, (s, s), pads, act, lut=lut))
    assert_close(y, d["y"], name)


@pytest.mark.parametrize("name", golden_names("conv8"))
def test_conv_int8_golden_bit_exact(ops, oracle_mod, name):
    d = golden(name)
    s, pad, act = (int(v) for v in d["meta"])
    y = _np(ops.conv(d["x"], d["w8"], d["b32"], (s, s), (pad,) * 4, act, int8=(float(d["scale"]), d["aux"]),
                     lut=oracle_mod.silu_lut()))
    assert np.array_equal(y, d["y"]), f"{name}: {(y != d['y']).sum()} of {y.size} outputs differ"


def test_gemm_matmul_golden(ops):
    d = golden("gemm")
    assert_close(_np(ops.gemm(d["a"], d["w"], d["b"])), d["y"], "gemm")
    for n in ("matmul_shared", "matmul_batched"):
        d = golden(n)
        assert_close(_np(ops.matmul(d["a"], d["b"])), d["y"], n)


# name, N, C, H, W, OC, k, stride, pads, act
CONV_CASES = [
    ("cfg1_64x56x56_3x3_relu", 1, 64, 56, 56, 64, 3, 1, (1, 1, 1, 1), abi.RELU),
    ("batch8_cfg1", 8, 64, 56, 56, 64, 3, 1, (1, 1, 1, 1), abi.RELU),
    ("1x1_256to64", 2, 256, 56, 56, 64, 1, 1, (0, 0, 0, 0), abi.RELU),
    ("1x1_s2_downsample", 2, 256, 56, 56, 512, 1, 2, (0, 0, 0, 0), abi.NOT_ACT),
    ("3x3_s2", 2, 128, 56, 56, 128, 3, 2, (1, 1, 1, 1), abi.RELU),
    ("3x3_512_7x7", 3, 512, 7, 7, 512, 3, 1, (1, 1, 1, 1), abi.RELU),
    ("stem_7x7_s2", 2, 3, 224, 224, 64, 7, 2, (3, 3, 3, 3), abi.RELU),
    ("vit_patch_16x16_s16", 2, 3, 224, 224, 192, 16, 16, (0, 0, 0, 0), abi.NOT_ACT),
    ("ragged_c24_oc40_asym", 1, 24, 19, 23, 40, 3, 1, (1, 0, 2, 1), abi.LEAKYRELU),
    ("c8_5x5", 1, 8, 20, 20, 16, 5, 1, (2, 2, 2, 2), abi.CLIP),
    ("c5_odd_channels", 1, 5, 11, 11, 7, 3, 1, (1, 1, 1, 1), abi.HARDSILU),
    ("one_pixel", 1, 32, 1, 1, 32, 1, 1, (0, 0, 0, 0), abi.RELU),
    ("kernel_equals_input", 1, 16, 3, 3, 8, 3, 1, (0, 0, 0, 0), abi.SILU),
    ("nobias_skips_act", 1, 32, 14, 14, 64, 3, 1, (1, 1, 1, 1), abi.RELU),
    # stride-1 multi-tap layers with 32..128 channels: ragged last rows, a non-square image, unequal pads,
    # a 128-wide output, SiLU, a 1x3 kernel without bias
    ("halo_128x28x28", 3, 128, 28, 28, 128, 3, 1, (1, 1, 1, 1), abi.RELU),
    ("halo_ragged_rows_64x14x14", 2, 64, 14, 14, 64, 3, 1, (1, 1, 1, 1), abi.RELU),
    ("halo_nonsquare_32x10x28", 2, 32, 10, 28, 96, 3, 1, (1, 1, 1, 1), abi.NOT_ACT),
    ("halo_asym_pads_64x20x30", 1, 64, 20, 30, 32, 3, 1, (2, 0, 0, 2), abi.SILU),
    ("halo_1x3_kernel_nobias", 1, 64, 12, 40, 64, (1, 3), 1, (0, 1, 0, 1), abi.RELU),
]


@pytest.mark.parametrize("prec", ["tf32", "bf16", "f16"])
@pytest.mark.parametrize("case", CONV_CASES, ids=[c[0] for c in CONV_CASES])
def test_conv_f32_vs_oracle(ops, oracle_mod, case, prec):
    name, N, C, H, W, OC, k, s, pads, act = case
    rng = np.random.default_rng(zlib.crc32(name.encode()))   # stable across processes (str hashes are salted)
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    kh, kw = k if isinstance(k, tuple) else (k, k)
    w = (rng.standard_normal((OC, C, kh, kw)) * 0.05).astype(np.float32)
    b = None if "nobias" in name else (rng.standard_normal(OC) * 0.01).astype(np.float32)
    lut = oracle_mod.silu_lut() if act == abi.SILU else None
    capi.check(capi.lib().one_cuda_set_eval_precision(capi.PRECISIONS[prec]))
    try:
        y = _np(ops.conv(x, w, b, (s, s), pads, act, lut=lut))
    finally:
        capi.lib().one_cuda_set_eval_precision(capi.PREC_TF32)
    assert_close(y, oracle_mod.conv_f32(x, w, b, (s, s), pads, act), name)


# few-channel stride-2 stems on 16-bit storage: eight image columns per space-to-depth position (one 128-byte
# row per filter row), odd sizes, 5- and 7-wide filters, 1 to 4 channels
WIDE_STEM_CASES = [
    ("wide_7x7_rgb_odd", 2, 3, 33, 47, 32, 7, 2, (3, 3, 3, 3)),
    ("wide_5x5_rgb", 1, 3, 40, 40, 64, 5, 2, (2, 2, 2, 2)),
    ("wide_7x7_gray", 3, 1, 30, 31, 40, 7, 2, (3, 3, 3, 3)),
    ("wide_7x7_rgba_pad2", 1, 4, 28, 36, 64, 7, 2, (2, 2, 2, 2)),
    ("wide_6x6_rgb_nopad_left", 1, 3, 32, 32, 32, 6, 2, (2, 2, 2, 2)),
]


@pytest.mark.parametrize("prec", ["f16", "bf16", "tf32"])
@pytest.mark.parametrize("case", WIDE_STEM_CASES, ids=[c[0] for c in WIDE_STEM_CASES])
def test_few_channel_stride2_stems_vs_oracle(ops, oracle_mod, case, prec):
    name, N, C, H, W, OC, k, s, pads = case
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((OC, C, k, k)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(OC) * 0.01).astype(np.float32)
    capi.check(capi.lib().one_cuda_set_eval_precision(capi.PRECISIONS[prec]))
    try:
        y = _np(ops.conv(x, w, b, (s, s), pads, abi.RELU))
    finally:
        capi.lib().one_cuda_set_eval_precision(capi.PREC_TF32)
    assert_close(y, oracle_mod.conv_f32(x, w, b, (s, s), pads, abi.RELU), f"{name} {prec}")


INT8_CASES = [
    ("yolo_stem_3to32_s2", 1, 3, 160, 160, 32, 3, 2, 1, abi.SILU),
    ("csp_32to64_s2", 1, 32, 80, 80, 64, 3, 2, 1, abi.SILU),
    ("csp_1x1_64", 2, 64, 40, 40, 64, 1, 1, 0, abi.SILU),
    ("csp_3x3_128", 1, 128, 20, 20, 128, 3, 1, 1, abi.SILU),
    ("wide_512", 1, 512, 10, 10, 512, 3, 1, 1, abi.RELU),
    ("c48_oc24_ragged", 1, 48, 9, 9, 24, 3, 1, 1, abi.NOT_ACT),
]


@pytest.mark.parametrize("case", INT8_CASES, ids=[c[0] for c in INT8_CASES])
def test_conv_int8_bit_exact_vs_oracle(ops, oracle_mod, case):
    name, N, C, H, W, OC, k, s, pad, act = case
    rng = np.random.default_rng(zlib.crc32(name.encode()))   # stable across processes (str hashes are salted)
    x = rng.uniform(0, 1, (N, C, H, W)).astype(np.float32)
    x.ravel()[:8] = [0.5 / 127 * 0.9, 1.5 / 127 * 0.9, 2.0, -3.0, 0.0, 0.9, 0.45, 1e-9]   # ties and clamps
    w = (rng.standard_normal((OC, C, k, k)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(OC) * 0.01).astype(np.float32)
    w8, b32, aux = oracle_mod.quant_weight_bias(w, b)
    scale = np.float32(0.9 / 127)
    ref, acc, q = oracle_mod.conv_s8(x, w8, b32, aux, scale, (s, s), pad, act)
    y = _np(ops.conv(x, w8, b32, (s, s), (pad,) * 4, act, int8=(float(scale), aux), lut=oracle_mod.silu_lut()))
    assert np.array_equal(y, ref), f"{name}: {(y != ref).sum()} of {y.size} outputs differ"


def test_conv_int8_negative_input_scale_follows_the_reference(ops, oracle_mod):
    """The reference's percent calibrator returns a signed threshold; with a negative input_scale its int8
    conv quantises x / s and multiplies the sum by s again.  Same here, bit for bit; zero is rejected."""
    rng = np.random.default_rng(5)
    x = rng.uniform(-1, 1, (1, 32, 12, 12)).astype(np.float32)
    w = (rng.standard_normal((32, 32, 3, 3)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(32) * 0.01).astype(np.float32)
    w8, b32, aux = oracle_mod.quant_weight_bias(w, b)
    scale = np.float32(-1.0 / 127)
    ref, _, _ = oracle_mod.conv_s8(x, w8, b32, aux, scale, (1, 1), 1, abi.RELU)
    y = _np(ops.conv(x, w8, b32, (1, 1), (1, 1, 1, 1), abi.RELU, int8=(float(scale), aux)))
    assert np.array_equal(y, ref)
    with pytest.raises(capi.OneCudaError):
        ops.conv(x, w8, b32, (1, 1), (1, 1, 1, 1), abi.RELU, int8=(0.0, aux))


@pytest.mark.parametrize("prec", ["tf32", "bf16", "f16"])
@pytest.mark.parametrize("shape", [(1, 2048, 1000), (256, 2048, 1000), (1, 192, 1000), (77, 100, 40), (130, 8, 8)])
def test_gemm_vs_oracle(ops, oracle_mod, shape, prec):
    M, K, N = shape
    rng = np.random.default_rng(M * 7 + K)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    capi.check(capi.lib().one_cuda_set_eval_precision(capi.PRECISIONS[prec]))
    try:
        y = _np(ops.gemm(a, w, b))
    finally:
        capi.lib().one_cuda_set_eval_precision(capi.PREC_TF32)
    assert_close(y, oracle_mod.gemm(a, w, b), f"gemm {shape}")


# ViT-Tiny shapes: shared initialiser B, and the two batched activation x activation products
@pytest.mark.parametrize("sa,sb", [((197, 192), (192, 576)), ((2, 197, 192), (192, 768)), ((2, 197, 768), (768, 192)),
                                    ((2, 3, 197, 64), (2, 3, 64, 197)), ((2, 3, 197, 197), (2, 3, 197, 64)),
                                    ((5, 3), (3, 2))])
def test_matmul_vs_oracle(ops, oracle_mod, sa, sb):
    rng = np.random.default_rng(sum(sa) + sum(sb))
    a = rng.standard_normal(sa).astype(np.float32)
    b = rng.standard_normal(sb).astype(np.float32)
    assert_close(_np(ops.matmul(a, b)), oracle_mod.matmul(a, b), f"matmul {sa} x {sb}")


def test_linearity_at_full_size(ops):
    """Size-independent property at the batch-sweep size: conv(x1 + x2) == conv(x1) + conv(x2)
    for a bias-less convolution (no activation is applied without a bias)."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(5)
    x1 = torch.rand((64, 64, 56, 56), device="cuda", generator=g) - 0.5
    x2 = torch.rand((64, 64, 56, 56), device="cuda", generator=g) - 0.5
    w = torch.randn((64, 64, 3, 3), device="cuda", generator=g) * 0.05
    f = lambda x: ops.conv(x, w, None, (1, 1), (1, 1, 1, 1), abi.NOT_ACT)
    ya, yb, yab = f(x1), f(x2), f(x1 + x2)
    err = ((ya + yb) - yab).abs().max().item() / yab.abs().max().item()
    assert err < 5e-3, err


@pytest.mark.parametrize("name", ["dw3x3_p1_relu", "dw3x3_s2_p1", "dw5x5_p2_silu"])
def test_depthwise_conv_golden_bit_exact(ops, oracle_mod, name):
    """group == C: the reference treats any group != 1 as depthwise; the CUDA-core kernel sums the taps
    in the reference's order, so the fp32 result is identical."""
    d = golden(name)
    s, pd, act = (int(v) for v in d["meta"])
    C = d["x"].shape[1]
    y = _np(ops.conv(d["x"], d["w"], d["b"], (s, s), (pd,) * 4, act, lut=oracle_mod.silu_lut(), group=C))
    if act == abi.SILU:
        assert_close(y, d["y"], name)      # table index can flip on a last-bit difference
    assert np.array_equal(y, d["y"]) or act == abi.SILU


@pytest.mark.parametrize("name", ["dw8_3x3_p1_relu", "dw8_3x3_s2_p1", "dw8_5x5_p2_leaky"])
def test_depthwise_int8_golden_bit_exact(ops, name):
    """int8 depthwise: quantise-on-read, int32 tap sums and the reference's three-step epilogue."""
    d = golden(name)
    s, pd, act = (int(v) for v in d["meta"])
    C = d["x"].shape[1]
    y = _np(ops.conv(d["x"], d["w8"], d["b32"], (s, s), (pd,) * 4, act, int8=(float(d["scale"]), d["aux"]), group=C))
    assert np.array_equal(y, d["y"])


def test_depthwise_int8_full_size_vs_oracle(ops, oracle_mod):
    rng = np.random.default_rng(78)
    x = rng.uniform(-1, 1, (4, 96, 56, 56)).astype(np.float32)
    w = (rng.standard_normal((96, 1, 3, 3)) * 0.2).astype(np.float32)
    b = (rng.standard_normal(96) * 0.05).astype(np.float32)
    w8, b32, aux = oracle_mod.quant_weight_bias(w, b)
    sc = float(np.float32(np.abs(x).max() / 127))
    y = _np(ops.conv(x, w8, b32, (2, 2), (1, 1, 1, 1), abi.RELU, int8=(sc, aux), group=96))
    assert np.array_equal(y, oracle_mod.dwconv_s8(x, w8, b32, aux, sc, (2, 2), 1, abi.RELU))


def test_depthwise_full_size_vs_oracle(ops, oracle_mod):
    rng = np.random.default_rng(77)
    x = rng.uniform(-1, 1, (4, 96, 56, 56)).astype(np.float32)
    w = (rng.standard_normal((96, 1, 3, 3)) * 0.2).astype(np.float32)
    b = (rng.standard_normal(96) * 0.05).astype(np.float32)
    y = _np(ops.conv(x, w, b, (2, 2), (1, 1, 1, 1), abi.RELU, group=96))
    assert np.array_equal(y, oracle_mod.dwconv_f32(x, w, b, (2, 2), (1, 1, 1, 1), abi.RELU))


# name, N, C, H, W, OC, k, stride, pad, act: launches with far fewer output tiles than SMs
SPLIT_CASES = [
    ("deep_3x3_512_7x7", 4, 512, 7, 7, 512, 3, 1, 1, abi.RELU),
    ("deep_1x1_2048to512_7x7", 2, 2048, 7, 7, 512, 1, 1, 0, abi.RELU),
    ("silu_3x3_256_14x14", 1, 256, 14, 14, 256, 3, 1, 1, abi.SILU),
    ("ragged_oc40_3x3_128", 1, 128, 9, 9, 40, 3, 1, 1, abi.LEAKYRELU),
    ("s2_3x3_256_14x14", 2, 256, 14, 14, 512, 3, 2, 1, abi.NOT_ACT),
]


@pytest.mark.parametrize("splits", [0, 2, 5, 64])
@pytest.mark.parametrize("case", SPLIT_CASES, ids=[c[0] for c in SPLIT_CASES])
def test_conv_split_k_vs_oracle_and_unsplit(ops, oracle_mod, case, splits):
    """Split-K (K cut into ranges, partial sums added in a fixed order by a second kernel): every forced
    split count, and the library's own choice, stay within the float tolerance of the oracle, agree with
    the unsplit launch to accumulation-order noise, and are deterministic."""
    name, N, C, H, W, OC, k, s, pad, act = case
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((OC, C, k, k)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(OC) * 0.01).astype(np.float32)
    lut = oracle_mod.silu_lut() if act == abi.SILU else None
    L = capi.lib()
    try:
        capi.check(L.one_cuda_set_split_k(1))
        y1 = _np(ops.conv(x, w, b, (s, s), (pad,) * 4, act, lut=lut))
        capi.check(L.one_cuda_set_split_k(splits))
        ys = _np(ops.conv(x, w, b, (s, s), (pad,) * 4, act, lut=lut))
        ys2 = _np(ops.conv(x, w, b, (s, s), (pad,) * 4, act, lut=lut))
    finally:
        L.one_cuda_set_split_k(0)
    ref = oracle_mod.conv_f32(x, w, b, (s, s), (pad,) * 4, act)
    assert_close(y1, ref, name + " unsplit")
    assert_close(ys, ref, f"{name} split {splits}")
    assert np.array_equal(ys, ys2)
    assert np.abs(ys - y1).max() <= 2e-3 * np.abs(ref).max()


@pytest.mark.parametrize("splits", [0, 4, 16])
@pytest.mark.parametrize("shape", [(32, 2048, 1000), (256, 2048, 1000), (8, 768, 192)])
def test_gemm_split_k_vs_oracle(ops, oracle_mod, shape, splits):
    M, K, N = shape
    rng = np.random.default_rng(M * 11 + K)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    L = capi.lib()
    try:
        capi.check(L.one_cuda_set_split_k(splits))
        y = _np(ops.gemm(a, w, b))
    finally:
        L.one_cuda_set_split_k(0)
    assert_close(y, oracle_mod.gemm(a, w, b), f"gemm {shape} split {splits}")
    assert L.one_cuda_set_split_k(65) == -1 and L.one_cuda_set_split_k(-1) == -1


def test_bias_pointer_that_is_only_float_aligned(oracle_mod):
    """The reference accepts any float-aligned bias (e.g. a pointer into a mapped .one image, whose payloads
    start 8 bytes past a 16-byte boundary).  Such a bias must not be read 16 bytes at a time."""
    import torch
    rng = np.random.default_rng(21)
    N, C, H, W, OC = 2, 64, 14, 14, 64
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((OC, C, 3, 3)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(OC) * 0.01).astype(np.float32)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    y = torch.empty((N, OC, H, W), device="cuda")
    for off in (1, 2, 3):                                        # 4, 8 and 12 bytes past a 16-byte boundary
        store = torch.zeros(OC + 8, device="cuda")
        assert store.data_ptr() % 16 == 0
        store[off:off + OC] = torch.from_numpy(b).cuda()
        cfg = abi.conv_cfg((3, 3), (1, 1), (1, 1, 1, 1), has_bias=True, act=abi.RELU)
        args = abi.conv_eval_args(cfg, (N, C, H, W), (OC, C, 3, 3), (N, OC, H, W), xd.data_ptr(), wd.data_ptr(),
                                  store.data_ptr() + 4 * off, y.data_ptr(), abi.default_useful_info(), 0)
        capi.check(capi.shim_eval("Conv")(args.params, args.inputs, args.outputs))
        assert_close(y.cpu().numpy(), oracle_mod.conv_f32(x, w, b, (1, 1), (1, 1, 1, 1), abi.RELU), f"bias + {4 * off} bytes")


# name, N, C, H, W, OC, k, stride, pad, act: launches as pairs of CTAs sharing 256-row tiles
PAIR_CASES = [
    ("pair_3x3_256_14x14", 8, 256, 14, 14, 256, 3, 1, 1, abi.RELU),          # M = 1568: 6 full pair tiles + a tail of 32 rows
    ("pair_1x1_512to1024_14x14", 4, 512, 14, 14, 1024, 1, 1, 0, abi.NOT_ACT),
    ("pair_3x3_s2_128_28x28", 3, 128, 28, 28, 128, 3, 2, 1, abi.RELU),       # M = 588
    ("pair_small_m_100_rows", 1, 64, 10, 10, 192, 3, 1, 1, abi.SILU),        # M = 100: the odd CTA's rows are all outside the tensor
    ("pair_ragged_oc40", 2, 32, 12, 12, 40, 3, 1, 1, abi.LEAKYRELU),         # transposing epilogue (N not a multiple of 32)
    ("pair_many_tiles_64x56x56", 4, 64, 56, 56, 128, 3, 1, 1, abi.RELU),     # M = 12544: more pair tiles than TPCs
]


@pytest.mark.parametrize("tile", [1128, 1192, 1256])
@pytest.mark.parametrize("case", PAIR_CASES, ids=[c[0] for c in PAIR_CASES])
def test_conv_cta_pairs_vs_oracle_and_single_cta(ops, oracle_mod, case, tile):
    """The contraction run as clusters of two CTAs (tcgen05 cta_group::2: 256-row tiles, each CTA loading
    half of the weight tile) against the oracle and against the single-CTA launch of the same width, which
    sums the same products in the same order: bit-identical."""
    name, N, C, H, W, OC, k, s, pad, act = case
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((OC, C, k, k)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(OC) * 0.01).astype(np.float32)
    lut = oracle_mod.silu_lut() if act == abi.SILU else None
    L = capi.lib()
    try:
        capi.check(L.one_cuda_set_split_k(1))
        capi.check(L.one_cuda_set_tile_n(tile - 1000))
        y1 = _np(ops.conv(x, w, b, (s, s), (pad,) * 4, act, lut=lut))
        capi.check(L.one_cuda_set_tile_n(tile))
        y2 = _np(ops.conv(x, w, b, (s, s), (pad,) * 4, act, lut=lut))
        y3 = _np(ops.conv(x, w, b, (s, s), (pad,) * 4, act, lut=lut))
    finally:
        L.one_cuda_set_tile_n(0)
        L.one_cuda_set_split_k(0)
    assert_close(y2, oracle_mod.conv_f32(x, w, b, (s, s), (pad,) * 4, act), f"{name} tile {tile}")
    assert np.array_equal(y2, y3)
    assert np.array_equal(y2, y1), f"{name}: {(y2 != y1).sum()} of {y2.size} differ from the single-CTA launch"


def test_int8_and_gemm_cta_pairs(ops, oracle_mod):
    """Pairs of CTAs on the int8 path (bit exact against the oracle) and on Gemm; a tile code the kernel
    does not have is refused."""
    rng = np.random.default_rng(77)
    x = rng.uniform(0, 1, (2, 128, 20, 20)).astype(np.float32)
    w = (rng.standard_normal((256, 128, 3, 3)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(256) * 0.01).astype(np.float32)
    w8, b32, aux = oracle_mod.quant_weight_bias(w, b)
    scale = np.float32(0.9 / 127)
    ref, _, _ = oracle_mod.conv_s8(x, w8, b32, aux, scale, (1, 1), 1, abi.SILU)
    a = rng.standard_normal((300, 2048)).astype(np.float32)
    wg = (rng.standard_normal((1000, 2048)) * 0.05).astype(np.float32)
    bg = rng.standard_normal(1000).astype(np.float32)
    L = capi.lib()
    try:
        capi.check(L.one_cuda_set_tile_n(1256))
        y = _np(ops.conv(x, w8, b32, (1, 1), (1, 1, 1, 1), abi.SILU, int8=(float(scale), aux), lut=oracle_mod.silu_lut()))
        yg = _np(ops.gemm(a, wg, bg))
    finally:
        L.one_cuda_set_tile_n(0)
    assert np.array_equal(y, ref)
    assert_close(yg, oracle_mod.gemm(a, wg, bg), "gemm as CTA pairs")
    assert L.one_cuda_set_tile_n(1064) == -1 and L.one_cuda_set_tile_n(2192) == -1 and L.one_cuda_set_tile_n(3128) == -1 and L.one_cuda_set_tile_n(4256) == -1


# name, N, C, H, W, OC, k, stride, pad, act: tiles of two 128-row halves per CTA
HALF_CASES = [
    ("half_stem_7x7_s2_3to64", 2, 3, 64, 64, 64, 7, 2, 3, abi.RELU),          # the few-channel path, M = 2048
    ("half_3x3_64_28x28", 3, 64, 28, 28, 64, 3, 1, 1, abi.RELU),              # M = 2352: 9 full tiles + 48 rows
    ("half_3x3_128_14x14", 5, 128, 14, 14, 128, 3, 1, 1, abi.SILU),           # M = 980: the last tile's second half is short
    ("half_1x1_256to128", 2, 256, 9, 9, 128, 1, 1, 0, abi.NOT_ACT),           # M = 162: second half all but 34 rows outside
    ("half_small_m_100_rows", 1, 64, 10, 10, 64, 3, 1, 1, abi.RELU),          # M = 100: the second half is all outside
    ("half_ragged_oc40", 2, 32, 12, 12, 40, 3, 1, 1, abi.LEAKYRELU),          # transposing epilogue (N not a multiple of 32)
    ("half_wide_oc320", 1, 64, 20, 20, 320, 3, 1, 1, abi.RELU),               # several tiles along N, the last one ragged
    ("half_many_tiles_64x112x112", 4, 64, 112, 112, 64, 3, 1, 1, abi.RELU),   # M = 50176: more tiles than SMs
]


@pytest.mark.parametrize("tile", [2064, 2128])
@pytest.mark.parametrize("case", HALF_CASES, ids=[c[0] for c in HALF_CASES])
def test_conv_two_half_tiles_vs_oracle_and_plain_tiles(ops, oracle_mod, case, tile):
    """Tiles of two 128-row halves per CTA (one tile of the weights per K block serves both halves) against
    the oracle and against the plain 128-row launch of the same width, which sums the same products in the
    same order: bit-identical."""
    name, N, C, H, W, OC, k, s, pad, act = case
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((OC, C, k, k)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(OC) * 0.01).astype(np.float32)
    lut = oracle_mod.silu_lut() if act == abi.SILU else None
    L = capi.lib()
    try:
        capi.check(L.one_cuda_set_split_k(1))
        capi.check(L.one_cuda_set_tile_n(tile - 2000))
        y1 = _np(ops.conv(x, w, b, (s, s), (pad,) * 4, act, lut=lut))
        capi.check(L.one_cuda_set_tile_n(tile))
        y2 = _np(ops.conv(x, w, b, (s, s), (pad,) * 4, act, lut=lut))
        y3 = _np(ops.conv(x, w, b, (s, s), (pad,) * 4, act, lut=lut))
    finally:
        L.one_cuda_set_tile_n(0)
        L.one_cuda_set_split_k(0)
    assert_close(y2, oracle_mod.conv_f32(x, w, b, (s, s), (pad,) * 4, act), f"{name} tile {tile}")
    assert np.array_equal(y2, y3)
    assert np.array_equal(y2, y1), f"{name}: {(y2 != y1).sum()} of {y2.size} differ from the 128-row launch"


@pytest.mark.parametrize("prec", ["tf32", "f16"])
@pytest.mark.parametrize("tile", [4064, 4128])
@pytest.mark.parametrize("case", HALF_CASES, ids=[c[0] for c in HALF_CASES])
def test_conv_twelve_epilogue_warps_vs_oracle_and_plain_tiles(ops, oracle_mod, case, tile, prec):
    """Twelve epilogue warps (three groups taking every third tile, or every third chunk of a CTA's only tile)
    behind a shallower operand ring: the same sums in the same order as the eight-warp launch of that width."""
    name, N, C, H, W, OC, k, s, pad, act = case
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((OC, C, k, k)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(OC) * 0.01).astype(np.float32)
    lut = oracle_mod.silu_lut() if act == abi.SILU else None
    L = capi.lib()
    try:
        capi.check(L.one_cuda_set_eval_precision(capi.PRECISIONS[prec]))
        capi.check(L.one_cuda_set_split_k(1))
        capi.check(L.one_cuda_set_tile_n(tile - 4000))
        y1 = _np(ops.conv(x, w, b, (s, s), (pad,) * 4, act, lut=lut))
        capi.check(L.one_cuda_set_tile_n(tile))
        y2 = _np(ops.conv(x, w, b, (s, s), (pad,) * 4, act, lut=lut))
        y3 = _np(ops.conv(x, w, b, (s, s), (pad,) * 4, act, lut=lut))
    finally:
        L.one_cuda_set_tile_n(0)
        L.one_cuda_set_split_k(0)
        L.one_cuda_set_eval_precision(capi.PREC_TF32)
    assert_close(y2, oracle_mod.conv_f32(x, w, b, (s, s), (pad,) * 4, act), f"{name} tile {tile} {prec}")
    assert np.array_equal(y2, y3)
    assert np.array_equal(y2, y1), f"{name}: {(y2 != y1).sum()} of {y2.size} differ from the eight-warp launch"


def test_int8_and_gemm_two_half_tiles(ops, oracle_mod):
    """Two-half tiles on the int8 path (bit exact against the oracle), on Gemm and on a batched MatMul."""
    rng = np.random.default_rng(78)
    x = rng.uniform(0, 1, (2, 64, 30, 30)).astype(np.float32)
    w = (rng.standard_normal((128, 64, 3, 3)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(128) * 0.01).astype(np.float32)
    w8, b32, aux = oracle_mod.quant_weight_bias(w, b)
    scale = np.float32(0.9 / 127)
    ref, _, _ = oracle_mod.conv_s8(x, w8, b32, aux, scale, (1, 1), 1, abi.SILU)
    a = rng.standard_normal((300, 512)).astype(np.float32)
    wg = (rng.standard_normal((200, 512)) * 0.05).astype(np.float32)
    bg = rng.standard_normal(200).astype(np.float32)
    L = capi.lib()
    for tile in (2064, 2128, 4064, 4128):
        try:
            capi.check(L.one_cuda_set_tile_n(tile))
            y = _np(ops.conv(x, w8, b32, (1, 1), (1, 1, 1, 1), abi.SILU, int8=(float(scale), aux), lut=oracle_mod.silu_lut()))
            yg = _np(ops.gemm(a, wg, bg))
        finally:
            L.one_cuda_set_tile_n(0)
        assert np.array_equal(y, ref), tile
        assert_close(yg, oracle_mod.gemm(a, wg, bg), f"gemm with two-half tiles {tile}")
