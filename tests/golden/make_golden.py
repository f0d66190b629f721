"""Generate tests/golden/*.npz by running the REFERENCE's own x86 operators.

Run in the build container (where the reference tree is mounted and ``make -C oracle`` has
compiled it unmodified into oracle/_ref/):

    python tests/golden/make_golden.py

Each file holds the seeded inputs and the reference's outputs for one case of the Conv / Gemm /
MatMul path, small enough to commit.  The GPU box has no reference tree; the tests there compare
against these files and against the C restatement (which test_oracle.py pins to the same files).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from onenew_b200 import abi  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))

# name, N, C, H, W, OC, K, stride, pads(t,l,b,r), act
CONV_F32 = [
    ("conv3x3_relu", 1, 16, 12, 12, 24, 3, 1, (1, 1, 1, 1), abi.RELU),
    ("conv3x3_s2_silu", 2, 8, 13, 13, 16, 3, 2, (1, 1, 1, 1), abi.SILU),
    ("conv1x1_clip", 1, 32, 7, 7, 40, 1, 1, (0, 0, 0, 0), abi.CLIP),
    ("conv7x7_s2_stem", 1, 3, 32, 32, 16, 7, 2, (3, 3, 3, 3), abi.RELU),
    ("conv5x5_asym_leaky", 1, 8, 10, 10, 8, 5, 1, (2, 1, 2, 3), abi.LEAKYRELU),
    ("conv3x3_hardsilu", 1, 8, 9, 9, 8, 3, 1, (1, 1, 1, 1), abi.HARDSILU),
    ("conv3x3_nobias", 1, 8, 9, 9, 8, 3, 1, (1, 1, 1, 1), abi.RELU),
]
CONV_S8 = [
    ("conv8_3x3_s2_silu", 1, 32, 16, 16, 32, 3, 2, 1, abi.SILU),
    ("conv8_1x1_relu", 2, 64, 6, 6, 16, 1, 1, 0, abi.RELU),
    ("conv8_stem_c3", 1, 3, 24, 24, 16, 3, 2, 1, abi.SILU),
]


VIT_SMALL = dict(seed=5, image=64, patch=16, dim=64, depth=2, heads=2, mlp=128, num_classes=10)
VIT_KEEP = ["tokens", "embedded", "blocks.0.norm1_out", "blocks.0.attn.qkv/Add_out", "blocks.0.k", "blocks.0.scores",
            "blocks.0.probs", "blocks.0.ctx", "blocks.0.res1", "blocks.0.mlp_act", "blocks.0.res2", "blocks.1.res2", "cls_out",
            "output"]


def quant_weight_bias(w, b):
    """Weights / bias / weight_aux from the reference's own quant_weight_bias (model_quant.hpp:6-29)."""
    assert oracle.have_quant_reference(), "oracle/_ref/libquant_ref.so is missing: run `make -C oracle` with the reference tree present"
    return oracle.ref_quant_weight_bias(w, b)


def main():
    assert oracle.have_reference(), "oracle/_ref is missing: run `make -C oracle` with the reference tree present"
    rng = np.random.default_rng(20240)
    for name, N, C, H, W, OC, K, s, pads, act in CONV_F32:
        x = rng.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
        w = (rng.standard_normal((OC, C, K, K)) * 0.05).astype(np.float32)
        b = None if "nobias" in name else (rng.standard_normal(OC) * 0.01).astype(np.float32)
        y = oracle.ref_conv(x, w, b, (s, s), pads, act)
        np.savez_compressed(os.path.join(OUT, name + ".npz"), x=x, w=w, b=b if b is not None else np.zeros(0, np.float32),
                            y=y, meta=np.array([s, *pads, act, int(b is not None)], np.int32))
    for name, N, C, H, W, OC, K, s, pad, act in CONV_S8:
        x = rng.uniform(0, 1, (N, C, H, W)).astype(np.float32)
        w = (rng.standard_normal((OC, C, K, K)) * 0.05).astype(np.float32)
        b = (rng.standard_normal(OC) * 0.01).astype(np.float32)
        w8, b32, aux = quant_weight_bias(w, b)
        scale = np.float32(x.max() / 127)
        y = oracle.ref_conv(x, w8, b32, (s, s), (pad,) * 4, act, int8=(scale, aux))
        np.savez_compressed(os.path.join(OUT, name + ".npz"), x=x, w=w, b=b, w8=w8, b32=b32, aux=aux, scale=scale, y=y,
                            meta=np.array([s, pad, act], np.int32))
    # depthwise (group == C): the reference's 3x3/pad-1 special case and its generic path
    for name, N, C, H, K, st, pd, act in [("dw3x3_p1_relu", 1, 16, 12, 3, 1, 1, abi.RELU), ("dw3x3_s2_p1", 2, 8, 14, 3, 2, 1, abi.NOT_ACT),
                                          ("dw5x5_p2_silu", 1, 8, 10, 5, 1, 2, abi.SILU)]:
        x = rng.uniform(-1, 1, (N, C, H, H)).astype(np.float32)
        w = (rng.standard_normal((C, 1, K, K)) * 0.2).astype(np.float32)
        b = (rng.standard_normal(C) * 0.05).astype(np.float32)
        y = oracle.ref_conv(x, w, b, (st, st), (pd,) * 4, act, group=C)
        np.savez_compressed(os.path.join(OUT, name + ".npz"), x=x, w=w, b=b, y=y, meta=np.array([st, pd, act], np.int32))
    # int8 depthwise: quantised by the reference's rule, run through the reference's W8A32 depthwise path
    rq = np.random.default_rng(4242)   # its own stream: the vectors above keep their values
    for name, N, C, H, K, st, pd, act in [("dw8_3x3_p1_relu", 1, 16, 12, 3, 1, 1, abi.RELU), ("dw8_3x3_s2_p1", 2, 8, 14, 3, 2, 1, abi.NOT_ACT),
                                          ("dw8_5x5_p2_leaky", 1, 12, 10, 5, 1, 2, abi.LEAKYRELU)]:
        x = rq.uniform(-1, 1, (N, C, H, H)).astype(np.float32)
        w = (rq.standard_normal((C, 1, K, K)) * 0.2).astype(np.float32)
        b = (rq.standard_normal(C) * 0.05).astype(np.float32)
        w8, b32, aux = quant_weight_bias(w, b)
        scale = np.float32(np.abs(x).max() / 127)
        y = oracle.ref_conv(x, w8, b32, (st, st), (pd,) * 4, act, int8=(scale, aux), group=C)
        np.savez_compressed(os.path.join(OUT, name + ".npz"), x=x, w8=w8, b32=b32, aux=aux, scale=scale, y=y,
                            meta=np.array([st, pd, act], np.int32))
    a = rng.standard_normal((5, 96)).astype(np.float32)
    w = (rng.standard_normal((50, 96)) * 0.1).astype(np.float32)
    b = rng.standard_normal(50).astype(np.float32)
    np.savez_compressed(os.path.join(OUT, "gemm.npz"), a=a, w=w, b=b, y=oracle.ref_gemm(a, w, b))
    a = rng.standard_normal((21, 48)).astype(np.float32)
    bm = rng.standard_normal((48, 36)).astype(np.float32)
    np.savez_compressed(os.path.join(OUT, "matmul_shared.npz"), a=a, b=bm, y=oracle.ref_matmul(a, bm))
    a = rng.standard_normal((2, 3, 13, 16)).astype(np.float32)
    bm = rng.standard_normal((2, 3, 16, 13)).astype(np.float32)
    np.savez_compressed(os.path.join(OUT, "matmul_batched.npz"), a=a, b=bm, y=oracle.ref_matmul(a, bm))
    # model level: a test-sized ResNet (same graph family as the benchmark model) run operator by
    # operator through the reference libraries; logits and a few intermediate operands are kept
    from onenew_b200 import models
    from oracle.model_ref import RefNet
    image = models.build_resnet50(seed=3, num_classes=10, image=32, width=16, blocks=(2, 1, 1, 1)).tobytes()
    x = models.resnet50_input(2, seed=500, image=32)
    ref = RefNet(image)
    keep = ["Conv_0_out", "MaxPool_0_out", "Relu_0_0_out", "Relu_0_1_out", "Relu_3_0_out", "gap_out", "output"]
    runs = [ref.run(x[i:i + 1], collect=keep) for i in range(2)]
    np.savez_compressed(os.path.join(OUT, "resnet_small.npz"), x=x,
                        **{k: np.concatenate([r[k] for r in runs]) for k in keep})
    # int8 conv backbone (YOLOv8s-shaped stack) at a test size: scales from the restated MSE calibration
    # over 8 seeded images, then the quantised image run through the reference's int8 Conv
    ws = models.yolo_backbone_weights()
    IM = 96
    cal = models.yolo_input(8, image=IM)
    fref = RefNet(models.build_yolo_backbone(ws, image=IM).tobytes())
    fruns = [fref.run(cal[i:i + 1], collect="*") for i in range(8)]
    scales, quant, xn = [], [], "input"
    for i, (w, b) in enumerate(ws):
        samples = [cal[j:j + 1] if xn == "input" else r[xn] for j, r in enumerate(fruns)]
        sc = oracle.mse_input_scale(samples)
        quant.append(quant_weight_bias(w, b) + (sc,))
        scales.append(sc)
        xn = f"Conv_{i}_out"
    qref = RefNet(models.build_yolo_backbone(ws, image=IM, quant=quant).tobytes())
    qo = qref.run(cal[0:1], collect="*")
    np.savez_compressed(os.path.join(OUT, "yolo_int8_small.npz"), x=cal[0:1], scales=np.array(scales, np.float32),
                        **{k: qo[k] for k in ("Conv_0_out", "Conv_3_out", "Conv_9_out", "output")})
    # test-sized ViT (same graph as ViT-Tiny/16): every operand of two images through the reference's operators
    vimg = models.build_vit(**VIT_SMALL).tobytes()
    vx = models.vit_input(2, image=VIT_SMALL["image"])
    vref = RefNet(vimg)
    vruns = [vref.run(vx[i:i + 1], collect=VIT_KEEP) for i in range(2)]
    np.savez_compressed(os.path.join(OUT, "vit_small.npz"), x=vx, **{k: np.concatenate([r[k] for r in vruns]) for k in VIT_KEEP})
    print("wrote", len(CONV_F32) + len(CONV_S8) + 5, "fixtures to", OUT)


if __name__ == "__main__":
    main()
