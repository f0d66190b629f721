"""Synthetic models in ``.one`` form for the benchmark configurations.

The reference's model zoo is an external download and its converter cannot be built here, so
the graphs are written directly with seeded random weights, in the shape the converter plus the
conv+activation fusion pass would produce (tools/optimize/op_fusion.hpp:47-192): BatchNorm
folded into the conv bias (the reference has no BatchNormalization operator), ReLU fused into
the convs except after a residual ``Add``, which stays ``Add`` + ``Relu`` as in the reference's
own trace (tools/perf_profiling/timeline_info/resnet50.csv:9-10).
"""
import numpy as np

from . import abi
from .one_file import OneBuilder

IMAGENET_MEAN = (0.485, 0.456, 0.406)   # configs/rt_cfgs/rt_resnet50.yml:17-18
IMAGENET_STD = (0.229, 0.224, 0.225)


def _he(rng, shape):
    fan_in = int(np.prod(shape[1:]))
    return (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)


def build_resnet50(seed=0, num_classes=1000, image=224, width=64, blocks=(3, 4, 6, 3)):
    """ResNet-50 v1 with the stride on the 3x3 conv, as in the reference's traced model
    (resnet50.csv:3-91: Conv_25 is a stride-1 1x1 at 56x56, Conv_27 the stride-2 3x3).
    Smaller ``image`` / ``width`` / ``blocks`` give test-sized variants of the same graph."""
    rng = np.random.default_rng(seed)
    b = OneBuilder()
    b.add_io("input", "input", (1, 3, image, image))
    idx = [0]

    def conv(x, cin, cout, k, s, p, act):
        i = idx[0]
        idx[0] += 1
        name = f"Conv_{i}"
        w = b.add_init(f"{name}.weight", _he(rng, (cout, cin, k, k)))
        bias = b.add_init(f"{name}.bias", (rng.standard_normal(cout) * 0.01).astype(np.float32))
        return b.conv(name, x, w, bias, f"{name}_out", (k, k), (s, s), (p, p, p, p), act=act)

    x = conv("input", 3, width, 7, 2, 3, abi.RELU)
    x = b.maxpool("MaxPool_0", x, "MaxPool_0_out", (3, 3), (2, 2), (1, 1, 1, 1))
    cin = width
    for stage, nblk in enumerate(blocks):
        mid = width * (2 ** stage)
        cout = mid * 4
        for blk in range(nblk):
            stride = 2 if (blk == 0 and stage > 0) else 1
            y = conv(x, cin, mid, 1, 1, 0, abi.RELU)
            y = conv(y, mid, mid, 3, stride, 1, abi.RELU)
            y = conv(y, mid, cout, 1, 1, 0, abi.NOT_ACT)
            sc = conv(x, cin, cout, 1, stride, 0, abi.NOT_ACT) if blk == 0 else x
            tag = f"{stage}_{blk}"
            s = b.simple("Add", f"Add_{tag}", [y, sc], f"Add_{tag}_out")
            x = b.simple("Relu", f"Relu_{tag}", [s], f"Relu_{tag}_out")
            cin = cout
    x = b.simple("GlobalAveragePool", "GlobalAveragePool_0", [x], "gap_out")
    x = b.flatten("Flatten_0", x, "flatten_out", axis=1)
    wfc = b.add_init("fc.weight", (rng.standard_normal((num_classes, cin)) * np.sqrt(1.0 / cin)).astype(np.float32))
    bfc = b.add_init("fc.bias", (rng.standard_normal(num_classes) * 0.01).astype(np.float32))
    b.gemm("Gemm_0", x, wfc, bfc, "output")
    b.add_io("output", "output", (1, num_classes))
    return b


def resnet50_input(n, seed=100, image=224):
    """uniform[0,1] images normalised with the ImageNet constants, one seed per image index."""
    out = np.empty((n, 3, image, image), np.float32)
    mean = np.array(IMAGENET_MEAN, np.float32).reshape(3, 1, 1)
    std = np.array(IMAGENET_STD, np.float32).reshape(3, 1, 1)
    for i in range(n):
        r = np.random.default_rng(seed + i)
        out[i] = (r.uniform(0, 1, (3, image, image)).astype(np.float32) - mean) / std
    return out


RESNET50_FLOPS_PER_IMAGE = 8.19e9   # the reference's own count: 8191.2 MFLOP (resnet50.csv:92)


# ------------------------------------------------------------------------------- int8 conv backbone
# YOLOv8s-shaped backbone as a plain conv stack: 3x3 stride-2 downsamples at CSP widths 32..512, a
# 1x1 and a 3x3 stride-1 conv inside each stage, SiLU (table) everywhere, every conv with a bias and
# symmetric pads (the int8 path pads every side by pads[0]).
YOLO_STACK = [  # cin, cout, kernel, stride, pad
    (3, 32, 3, 2, 1), (32, 64, 3, 2, 1), (64, 64, 1, 1, 0), (64, 64, 3, 1, 1),
    (64, 128, 3, 2, 1), (128, 128, 1, 1, 0), (128, 128, 3, 1, 1),
    (128, 256, 3, 2, 1), (256, 256, 1, 1, 0), (256, 256, 3, 1, 1),
    (256, 512, 3, 2, 1), (512, 512, 1, 1, 0), (512, 512, 3, 1, 1),
]


def yolo_backbone_weights(seed=0, stack=YOLO_STACK):
    rng = np.random.default_rng(seed)
    return [((rng.standard_normal((co, ci, k, k)) * 0.05).astype(np.float32),
             (rng.standard_normal(co) * 0.01).astype(np.float32)) for ci, co, k, s, p in stack]


def build_yolo_backbone(weights, image=640, stack=YOLO_STACK, quant=None):
    """fp32 model, or -- with ``quant`` = list of (w_s8, b_s32, weight_aux, input_scale) per conv --
    the image the reference's quantiser would leave: int8 weights / int32 bias at the start of the
    fp32-sized records, ``ifmap_quant2`` = INT8, ``input_scale`` and ``weight_aux`` in the config
    (tools/optimize/model_quant.hpp:6-29, :659-676)."""
    b = OneBuilder()
    b.add_io("input", "input", (1, 3, image, image))
    x, hw = "input", image
    for i, ((ci, co, k, s, p), (w, bias)) in enumerate(zip(stack, weights)):
        name = f"Conv_{i}"
        hw = (hw + 2 * p - k) // s + 1
        out = "output" if i == len(stack) - 1 else f"{name}_out"
        if quant is None:
            wn = b.add_init(f"{name}.weight", w)
            bn = b.add_init(f"{name}.bias", bias)
            b.conv(name, x, wn, bn, out, (k, k), (s, s), (p, p, p, p), act=abi.SILU)
        else:
            w8, b32, aux, scale = quant[i]
            wraw = bytearray(w.nbytes)
            wraw[:w8.size] = np.ascontiguousarray(w8, np.int8).tobytes()
            wn = b.add_init(f"{name}.weight", w, raw=bytes(wraw))
            bn = b.add_init(f"{name}.bias", bias, raw=np.ascontiguousarray(b32, np.int32).tobytes())
            b.conv(name, x, wn, bn, out, (k, k), (s, s), (p, p, p, p), act=abi.SILU, int8_scale=float(scale), weight_aux=aux)
        x = out
    b.add_io("output", "output", (1, stack[-1][1], hw, hw))
    return b


def yolo_input(n, seed=200, image=640):
    return np.stack([np.random.default_rng(seed + i).uniform(0, 1, (3, image, image)).astype(np.float32) for i in range(n)])
