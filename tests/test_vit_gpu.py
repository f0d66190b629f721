"""Transformer-encoder path on the GPU: the glue operators one by one against numpy restatements of
the reference's arithmetic, and the ViT graph against operands computed by the reference's own x86
operators (tests/golden/vit_small.npz, made by tests/golden/make_golden.py)."""
import math

import numpy as np
import pytest

from common import assert_close, golden
from onenew_b200 import models, net as onet

pytestmark = pytest.mark.gpu
VIT_SMALL = dict(seed=5, image=64, patch=16, dim=64, depth=2, heads=2, mlp=128, num_classes=10)


@pytest.fixture(scope="module")
def seq():
    from onenew_b200 import seq as s
    return s


@pytest.mark.parametrize("rows,D", [(197, 192), (5, 7), (33, 1000), (3, 1500)])
def test_layernorm(seq, rows, D):
    rng = np.random.default_rng(rows + D)
    x = rng.standard_normal((rows, D)).astype(np.float32) * 3 + 1
    w = rng.standard_normal(D).astype(np.float32)
    b = rng.standard_normal(D).astype(np.float32)
    mean = x.mean(-1, keepdims=True, dtype=np.float64)
    var = (x.astype(np.float64) ** 2).mean(-1, keepdims=True) - mean ** 2      # one-pass form of layer_normalization.c:72-86
    ref = ((x - mean) / np.sqrt(var) * w + b).astype(np.float32)
    assert np.allclose(seq.layernorm(x, w, b), ref, rtol=1e-4, atol=1e-4)


def test_gelu_table_lookup_is_exact(seq, oracle_mod):
    lut = oracle_mod.gelu_lut()
    x = np.concatenate([np.array([-9, -8, -7.9999, -1 / 512, 0, 1 / 512, 7.998, 8, 9.5], np.float32),
                        np.random.default_rng(0).uniform(-10, 10, 4099).astype(np.float32)])
    ref = np.where(x < -8, 0, np.where(x >= 8, x, lut[np.clip(((x + np.float32(8)) * np.float32(512)).astype(np.int32), 0, 8191)]))
    assert np.array_equal(seq.gelu(x, lut), ref.astype(np.float32))
    assert abs(lut[4096 + 512] - 0.5 * (1 + math.erf(1 / 1.4142))) < 1e-6


@pytest.mark.parametrize("rows,D", [(3 * 197, 197), (7, 5), (4, 64), (9, 700), (2, 1300)])
def test_softmax(seq, rows, D):
    x = np.random.default_rng(D).standard_normal((rows, D)).astype(np.float32) * 4
    e = np.exp(x - x.max(-1, keepdims=True))
    got = seq.softmax(x)
    assert np.allclose(got, e / e.sum(-1, keepdims=True), rtol=1e-5, atol=1e-7)
    assert np.allclose(got.sum(-1), 1, atol=1e-5)


@pytest.mark.parametrize("shape,perm", [((2, 64, 16), (0, 2, 1)), ((2, 17, 2, 32), (0, 2, 1, 3)), ((2, 17, 2, 32), (0, 2, 3, 1)),
                                        ((3, 5, 7), (2, 0, 1)), ((2, 3, 4, 5, 6), (2, 0, 3, 1, 4)), ((2, 3, 2, 3, 4, 5), (5, 4, 3, 2, 1, 0)),
                                        ((1, 3, 197, 64), (0, 1, 3, 2))])
def test_transpose_bit_exact(seq, shape, perm):
    x = np.random.default_rng(len(shape)).standard_normal(shape).astype(np.float32)
    assert np.array_equal(seq.transpose(x, perm), np.transpose(x, perm))


@pytest.mark.parametrize("sa,sb", [((2, 197, 192), (2, 197, 192)), ((2, 197, 576), (576,)), ((4, 17, 64), (1, 17, 64)), ((3, 5, 7), (1,)),
                                   ((192,), (2, 5, 192)), ((2, 3, 1, 5), (1, 3, 4, 1)), ((2, 1, 6), (2, 5, 1)), ((3, 5), (5,))])
def test_broadcast_arithmetic(seq, sa, sb):
    rng = np.random.default_rng(len(sa) * 10 + len(sb))
    a = rng.standard_normal(sa).astype(np.float32)
    b = (rng.uniform(0.5, 2, sb) * rng.choice([-1, 1], sb)).astype(np.float32)
    assert np.array_equal(seq.binary(0, a, b), a + b)
    assert np.array_equal(seq.binary(1, a, b), a - b)
    assert np.array_equal(seq.binary(2, a, b), a * b)
    got = seq.binary(3, a, b)
    if b.size == 1 and a.size > 1:     # a scalar divisor is applied as its reciprocal (device/x86/Div/div.c:104-118)
        assert np.array_equal(got, a * (np.float32(1) / b.reshape(())))
    else:
        assert np.array_equal(got, a / b)


def test_chunk_copy_concat_and_gather(seq):
    rng = np.random.default_rng(3)
    cls = rng.standard_normal((1, 1, 8)).astype(np.float32)
    tok = rng.standard_normal((3, 4, 8)).astype(np.float32)
    # Concat(axis 1) of an initialiser repeated over the batch and a batch of token rows
    out = seq.copy_chunks(cls, 3 * 5 * 8, reps=3, chunk=8, x_reps=1, x_stride=8, y_stride=40)
    out2 = seq.copy_chunks(tok, 3 * 5 * 8, reps=3, chunk=32, x_reps=3, x_stride=32, y_stride=40, y_off=8)
    ref = np.concatenate([np.repeat(cls, 3, 0), tok], 1)
    assert np.array_equal((out + out2).reshape(3, 5, 8), ref)
    # Gather(axis 1, index 2) with an odd inner size (scalar path)
    x = rng.standard_normal((4, 5, 7)).astype(np.float32)
    g = seq.copy_chunks(x, 4 * 7, reps=4, chunk=7, x_reps=4, x_stride=35, y_stride=7, x_off=2 * 7)
    assert np.array_equal(g.reshape(4, 7), x[:, 2])


def _attention_ref(qkv, heads, scale):
    B, T, D3 = qkv.shape
    D = D3 // 3
    x = qkv.astype(np.float64).reshape(B, T, 3, heads, D // heads)
    q, k, v = (x[:, :, j].transpose(0, 2, 1, 3) for j in range(3))
    s = (q * scale) @ k.transpose(0, 1, 3, 2)
    e = np.exp(s - s.max(-1, keepdims=True))
    return ((e / e.sum(-1, keepdims=True)) @ v).transpose(0, 2, 1, 3).reshape(B, T, D).astype(np.float32)


@pytest.mark.parametrize("B,T,heads,hd", [(2, 197, 3, 64), (1, 17, 2, 32), (3, 128, 1, 64), (1, 256, 2, 64), (2, 50, 2, 64), (1, 129, 4, 32)])
def test_fused_attention_vs_numpy(seq, B, T, heads, hd):
    rng = np.random.default_rng(T)
    qkv = rng.standard_normal((B, T, 3 * heads * hd)).astype(np.float32)
    got = seq.attention(qkv, heads, hd ** -0.5)
    assert_close(got, _attention_ref(qkv, heads, hd ** -0.5), f"attention T={T} hd={hd}")


def test_fused_attention_rejects_what_it_cannot_tile(seq):
    """More than 256 tokens or a head wider than 64 do not fit the one-tile kernel: the call says so
    (the runtime then leaves such a block unfused)."""
    from onenew_b200 import capi
    for shape, heads in (((1, 257, 3 * 64), 1), ((1, 16, 3 * 128), 1)):
        with pytest.raises(capi.OneCudaError) as e:
            seq.attention(np.zeros(shape, np.float32), heads, 1.0)
        assert e.value.code == -3


@pytest.mark.parametrize("fuse", [False, True])
@pytest.mark.parametrize("graph", [False, True])
def test_small_vit_matches_reference_per_operand(graph, fuse):
    """fuse=False runs the graph operator by operator; fuse=True folds bias / Gelu / residual into the
    GEMM epilogues and each attention block into one kernel."""
    g = golden("vit_small")
    n = onet.Net(models.build_vit(**VIT_SMALL).tobytes(), batch=2, precision="tf32", graph=graph, fuse=fuse)
    try:
        y = n(g["x"])
        assert_close(y, g["output"], "logits")
        assert np.array_equal(y, n(g["x"]))
        have = set(n.operands())
        checked = 0
        for k in g.files:
            if k != "x" and k in have:
                assert_close(n.fetch(k, g[k].shape), g[k], k)
                checked += 1
        assert checked >= 8
        if fuse:     # 2 blocks x (2 LayerNorm + 4 GEMM + 1 attention) + patch embedding, class token, position, norm, head ...
            assert n.work()[2] <= 2 * 7 + 12, n.work()
            assert "blocks.0.scores" not in have and "blocks.0.probs" not in have
    finally:
        n.close()


def test_vit_tiny_batch_invariance_and_reference_sample(oracle_mod):
    """Full-size ViT-Tiny/16: image 0 of a batch of 4 equals the same image run alone, and -- when the
    reference build is present -- the logits match the reference's."""
    img = models.build_vit().tobytes()
    x = models.vit_input(4)
    n4 = onet.Net(img, batch=4)
    n1 = onet.Net(img, batch=1)
    try:
        y4 = n4(x)
        y1 = n1(x[:1])
        assert_close(y4[:1], y1, "batch 4 vs batch 1")
        if oracle_mod.have_reference():
            from oracle.model_ref import RefNet
            ref = RefNet(img).run(x[:1], collect=["blocks.5.res2", "blocks.11.res2"])
            assert_close(y1, ref["output"], "vit-tiny logits")
            for k in ("blocks.5.res2", "blocks.11.res2"):
                assert_close(n1.fetch(k, ref[k].shape), ref[k], k)
    finally:
        n1.close()
        n4.close()
