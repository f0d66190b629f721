"""Full-size parity against the reference's own compiled operators, run live.

oracle/_ref (the reference's unmodified x86 operators, compiled by oracle/Makefile where the reference
tree is present) travels with the built libraries, so these tests compare the GPU path with reference code
at the sizes the benchmark configurations name: the int8 backbone at 3x640x640 layer by layer and bit for
bit, ResNet-50 at 3x224x224 at every operand within the float tolerance, and the transformer glue
operators on the ViT-Tiny shapes.  Skipped when oracle/_ref is absent."""
import numpy as np
import pytest

import oracle
from common import BF16_INTERMEDIATE_REL_MAX, REL_MAX, assert_close
from onenew_b200 import abi, models, net as onet
from onenew_b200.one_file import OneBuilder

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not oracle.have_reference(), reason="oracle/_ref (the reference build) is not present")]


def test_int8_backbone_640_every_layer_bit_exact():
    """The quantised-backbone benchmark configuration at its full size: the YOLOv8s-shaped int8 stack at 1x3x640x640.  Every
    layer's fp32 output equals the reference's (device/x86/Conv/conv.c:901-1059) bit for bit, operator by
    operator and with the int8 chain fused; a batch of 2 equals two single images."""
    from oracle.model_ref import RefNet
    from onenew_b200 import quant
    ws = models.yolo_backbone_weights()
    fp32 = models.build_yolo_backbone(ws).tobytes()
    x = models.yolo_input(2, seed=640)
    scales = quant.calibrate_mse(fp32, x)                  # any positive scales do; these are the calibrated ones
    img = quant.quantize_model(fp32, scales)
    names = [f"Conv_{i}_out" for i in range(len(models.YOLO_STACK) - 1)]
    ref = RefNet(img).run(x[:1], collect=names)
    n = onet.Net(img, batch=1, fuse=False)                 # fp32 activations between the convolutions
    try:
        y = n(x[:1])
        assert np.array_equal(y, ref["output"]), f"output: {(y != ref['output']).sum()} of {y.size} differ"
        for k in names:
            got = n.fetch(k, ref[k].shape)
            assert np.array_equal(got, ref[k]), f"{k}: {(got != ref[k]).sum()} of {got.size} differ"
    finally:
        n.close()
    order = list(scales)                                   # conv names in file order: the reader of Conv_i_out is conv i + 1
    n = onet.Net(img, batch=2)                             # fused: each conv writes its reader's int8 input directly
    try:
        y2 = n(x)
        assert np.array_equal(y2[:1], ref["output"])
        for i, k in enumerate(names):
            q = n.fetch(k, (2,) + ref[k].shape[1:])[:1]
            want = oracle.quantize_s8(ref[k], scales[order[i + 1]]).astype(np.float32)
            assert np.array_equal(q, want), f"{k} (quantised for its reader): {(q != want).sum()} differ"
    finally:
        n.close()
    n1 = onet.Net(img, batch=1)
    try:
        assert np.array_equal(n1(x[1:2]), y2[1:2])         # batch 2 == 2 x batch 1
    finally:
        n1.close()


@pytest.mark.parametrize("precision,fuse", [("tf32", True), ("tf32", False), ("f16", True), ("f16", False), ("bf16", True)])
def test_resnet50_224_every_operand_within_tolerance(precision, fuse):
    """The ResNet-50 benchmark configuration at full size: every operand the runtime materialises -- each Conv output,
    the pooled tensors, the block outputs, the logits -- against the reference's value for the same image
    (cosine >= 0.9999, max |a - b| / max |b| <= 1e-2).  TF32 and fp16 storage (the same 10-bit mantissa, every
    activation in 16 bits) with and without operator folding, both held to the same bar.  The bf16
    mode (bf16 inside a block, the residual trunk in fp32) meets both criteria at the logits and the cosine
    criterion everywhere; the max-norm of its intermediate operands is held to 1.25e-2 (see tests/common.py)."""
    from oracle.model_ref import RefNet
    img = models.build_resnet50().tobytes()
    x = models.resnet50_input(1, seed=222)
    ref = RefNet(img).run(x, collect="*")
    n = onet.Net(img, batch=1, precision=precision, fuse=fuse)
    try:
        y = n(x)
        assert_close(y, ref["output"], "logits")
        have = [k for k in n.operands() if k in ref and "#" not in k]
        assert len(have) >= (80 if not fuse else 50), len(have)
        convs = [k for k in have if k.startswith("Conv_")]
        assert len(convs) >= 20
        rel_max = BF16_INTERMEDIATE_REL_MAX if precision == "bf16" else REL_MAX
        for k in have:
            assert_close(n.fetch(k, ref[k].shape), ref[k], k, rel_max=REL_MAX if k == "output" else rel_max)
    finally:
        n.close()


def _glue_zoo(T=197, D=192, heads=3):
    """One graph holding every transformer glue operator on the ViT-Tiny shapes."""
    rng = np.random.default_rng(31)
    b = OneBuilder()
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    b.add_io("input", "input", (1, T, D))
    b.layernorm("ln", "input", b.add_init("ln.w", 1 + 0.1 * f(D)), b.add_init("ln.b", 0.1 * f(D)), "ln_out")
    b.simple("Gelu", "gelu", ["input"], "gelu_out")                     # straight from the input: the table index is then the same on both sides
    b.softmax("softmax", "input", "softmax_out")
    b.simple("Mul", "mul_scalar", ["input", b.add_init("scale", np.array([0.125], np.float32))], "mul_out")
    b.simple("Div", "div_scalar", ["input", b.add_init("denom", np.array([1.4142], np.float32))], "div_out")
    b.simple("Add", "add_vector", ["input", b.add_init("bias", f(D))], "addv_out")
    b.simple("Add", "add_pos", ["input", b.add_init("pos", f(1, T, D))], "addp_out")
    b.simple("Add", "add_acts", ["ln_out", "softmax_out"], "adda_out")
    b.reshape("r4", "input", "x4", (1, T, heads, D // heads))
    b.transpose("t_q", "x4", "tq_out", (0, 2, 1, 3))
    b.transpose("t_k", "x4", "tk_out", (0, 2, 3, 1))
    b.gather("gather_h", "x4", "gather_out", axis=2, index=1)
    b.concat("concat_cls", [b.add_init("cls", f(1, 1, D)), "input"], "concat_out", axis=1)
    b.gather("gather_cls", "concat_out", "cls_out", axis=1, index=0)
    b.reshape("r3", "tq_out", "merge_in", (1, heads, T, D // heads))
    b.transpose("t_merge", "merge_in", "merged", (0, 2, 1, 3))
    b.matmul("scores", "tq_out", "tk_out", "scores_out")           # batched activation x activation, [1,3,197,64] x [1,3,64,197]
    b.softmax("probs", "scores_out", "probs_out")
    b.add_io("output", "adda_out", (1, T, D))
    return b.tobytes()


GLUE_OPERANDS = ["ln_out", "gelu_out", "softmax_out", "mul_out", "div_out", "addv_out", "addp_out", "adda_out", "tq_out", "tk_out",
                 "gather_out", "concat_out", "cls_out", "merged", "scores_out", "probs_out"]


@pytest.mark.parametrize("batch", [1, 3])
def test_transformer_glue_operators_against_the_reference_libraries(batch):
    """LayerNormalization, Gelu, Softmax, Mul, Div, Add (vector, full tensor and two activations),
    Transpose, Gather, Concat and the batched MatMul on the ViT-Tiny shapes (197 tokens x 192, 3 heads),
    each compared with the output of the reference's own lib<Op>_x86.so for the same input
    (device/x86/LayerNormalization/layer_normalization.c:59-98, Softmax/softmax.c:31-76, Gelu/gelu.c:22-38,
    Add/add.c:17-86, Transpose/transpose.c:27-75)."""
    from oracle.model_ref import RefNet
    img = _glue_zoo()
    rng = np.random.default_rng(batch)
    x = rng.uniform(-2, 2, (batch, 197, 192)).astype(np.float32)
    refnet = RefNet(img)
    refs = [refnet.run(x[i:i + 1], collect=GLUE_OPERANDS) for i in range(batch)]
    n = onet.Net(img, batch=batch, fuse=False)
    try:
        n(x)
        have = set(n.operands())
        for k in GLUE_OPERANDS:
            assert k in have, k
            want = np.concatenate([r[k] for r in refs])
            got = n.fetch(k, want.shape)
            if k in ("tq_out", "tk_out", "gather_out", "concat_out", "cls_out", "merged", "mul_out", "addv_out", "addp_out", "gelu_out"):
                assert np.array_equal(got, want), k          # copies, table look-ups and single exact operations
            else:
                assert_close(got, want, k)
                assert np.abs(got - want).max() <= (2e-3 if k in ("scores_out", "probs_out") else 1e-5) * max(np.abs(want).max(), 1.0), k
    finally:
        n.close()
