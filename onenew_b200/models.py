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


# ------------------------------------------------------------------------------- ViT-Tiny/16
def _trunc_normal(rng, shape, std=0.02):
    """Truncated normal (|x| <= 2 std), the initialisation ViT weights are drawn from."""
    x = rng.standard_normal(shape)
    bad = np.abs(x) > 2
    while bad.any():
        x[bad] = rng.standard_normal(int(bad.sum()))
        bad = np.abs(x) > 2
    return (x * std).astype(np.float32)


def build_vit(seed=0, image=224, patch=16, dim=192, depth=12, heads=3, mlp=768, num_classes=1000):
    """ViT-Tiny/16 in the operator vocabulary the converter plus the LayerNorm / GELU fusion passes
    leave (tools/optimize/op_fusion.hpp:486-582): Conv patch embedding, Reshape / Transpose to a
    token sequence, Concat of the class token, Add of the position embedding, then per block
    LayerNormalization, a fused-qkv MatMul + Add(bias), Gather / Reshape / Transpose into heads,
    Mul by the scale, MatMul, Softmax, MatMul, projection, residual Adds, and the
    MatMul - Add - Gelu - MatMul - Add MLP; a final LayerNormalization, Gather of the class token and
    a Gemm head.  Every tensor keeps the batch as its leading dimension.  Smaller arguments give
    test-sized variants of the same graph."""
    rng = np.random.default_rng(seed)
    b = OneBuilder()
    grid = image // patch
    T = grid * grid + 1
    hd = dim // heads
    b.add_io("input", "input", (1, 3, image, image))

    def init(name, arr):
        return b.add_init(name, np.ascontiguousarray(arr, np.float32))

    def linear(tag, x, cin, cout):
        w = init(f"{tag}.weight", _trunc_normal(rng, (cin, cout)))
        bias = init(f"{tag}.bias", _trunc_normal(rng, (cout,)))
        y = b.matmul(f"{tag}/MatMul", x, w, f"{tag}/MatMul_out")
        return b.simple("Add", f"{tag}/Add", [y, bias], f"{tag}/Add_out")

    def norm(tag, x):
        w = init(f"{tag}.weight", 1.0 + _trunc_normal(rng, (dim,)))
        bias = init(f"{tag}.bias", _trunc_normal(rng, (dim,)))
        return b.layernorm(tag, x, w, bias, f"{tag}_out")

    w = init("patch_embed.weight", _trunc_normal(rng, (dim, 3, patch, patch)))
    bias = init("patch_embed.bias", _trunc_normal(rng, (dim,)))
    x = b.conv("patch_embed", "input", w, bias, "patch_embed_out", (patch, patch), (patch, patch), (0, 0, 0, 0))
    x = b.reshape("Reshape_tokens", x, "tokens_cf", (1, dim, grid * grid))
    x = b.transpose("Transpose_tokens", x, "tokens", (0, 2, 1))
    cls = init("cls_token", _trunc_normal(rng, (1, 1, dim)))
    x = b.concat("Concat_cls", [cls, x], "tokens_cls", axis=1)
    pos = init("pos_embed", _trunc_normal(rng, (1, T, dim)))
    x = b.simple("Add", "Add_pos", [x, pos], "embedded")
    scale = init("attn_scale", np.array([hd ** -0.5], np.float32))
    for i in range(depth):
        t = f"blocks.{i}"
        y = norm(f"{t}.norm1", x)
        qkv = linear(f"{t}.attn.qkv", y, dim, 3 * dim)
        qkv = b.reshape(f"{t}.attn/Reshape_qkv", qkv, f"{t}.qkv4", (1, T, 3, dim))
        parts = []
        for j, nm in enumerate("qkv"):
            p = b.gather(f"{t}.attn/Gather_{nm}", qkv, f"{t}.{nm}_flat", axis=2, index=j)
            p = b.reshape(f"{t}.attn/Reshape_{nm}", p, f"{t}.{nm}_heads", (1, T, heads, hd))
            perm = (0, 2, 3, 1) if nm == "k" else (0, 2, 1, 3)
            parts.append(b.transpose(f"{t}.attn/Transpose_{nm}", p, f"{t}.{nm}", perm))
        q, k, v = parts
        q = b.simple("Mul", f"{t}.attn/Mul", [q, scale], f"{t}.q_scaled")
        a = b.matmul(f"{t}.attn/MatMul_qk", q, k, f"{t}.scores")
        a = b.softmax(f"{t}.attn/Softmax", a, f"{t}.probs")
        y = b.matmul(f"{t}.attn/MatMul_av", a, v, f"{t}.ctx_heads")
        y = b.transpose(f"{t}.attn/Transpose_ctx", y, f"{t}.ctx_t", (0, 2, 1, 3))
        y = b.reshape(f"{t}.attn/Reshape_ctx", y, f"{t}.ctx", (1, T, dim))
        y = linear(f"{t}.attn.proj", y, dim, dim)
        x = b.simple("Add", f"{t}/Add_attn", [x, y], f"{t}.res1")
        y = norm(f"{t}.norm2", x)
        y = linear(f"{t}.mlp.fc1", y, dim, mlp)
        y = b.simple("Gelu", f"{t}.mlp/Gelu", [y], f"{t}.mlp_act")
        y = linear(f"{t}.mlp.fc2", y, mlp, dim)
        x = b.simple("Add", f"{t}/Add_mlp", [x, y], f"{t}.res2")
    x = norm("norm", x)
    x = b.gather("Gather_cls", x, "cls_out", axis=1, index=0)
    wfc = init("head.weight", _trunc_normal(rng, (num_classes, dim)))
    bfc = init("head.bias", _trunc_normal(rng, (num_classes,)))
    b.gemm("head", x, wfc, bfc, "output")
    b.add_io("output", "output", (1, num_classes))
    return b


def vit_input(n, seed=300, image=224):
    """uniform[0,1] images, one seed per image index."""
    return np.stack([np.random.default_rng(seed + i).uniform(0, 1, (3, image, image)).astype(np.float32) for i in range(n)])


VIT_TINY_FLOPS_PER_IMAGE = 2 * 1.26e9   # multiply-adds x 2 of the graph above at 224 x 224
