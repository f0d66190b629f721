"""Pins the quantiser to the reference's own code.  oracle/_ref/libquant_ref.so is compiled from lines of
tools/optimize/model_quant.hpp taken from the reference tree at build time (oracle/Makefile: quant_ref);
here the restated quantiser (oracle/oracle.c), the golden vectors and the product's host-side quantiser
arithmetic (csrc/quant.cu, no GPU involved) are all compared with it, bit for bit.  CPU only."""
import numpy as np
import pytest

import oracle
from common import golden, golden_names
from onenew_b200 import quant

pytestmark = pytest.mark.skipif(not oracle.have_quant_reference(), reason="oracle/_ref/libquant_ref.so not built (no reference tree at build time)")


def _weights(seed, shape, scale=0.05):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(shape) * scale).astype(np.float32)
    b = (rng.standard_normal(shape[0]) * 0.01).astype(np.float32)
    return w, b


@pytest.mark.parametrize("name", golden_names("conv8"))
def test_golden_int8_weights_are_the_references(name):
    """The w8 / b32 / aux stored in the int8 golden vectors are what the reference's quant_weight_bias
    (model_quant.hpp:6-29) makes of the stored fp32 weights."""
    d = golden(name)
    w8, b32, aux = oracle.ref_quant_weight_bias(d["w"], d["b"])
    assert np.array_equal(w8, d["w8"]) and np.array_equal(b32, d["b32"]) and np.array_equal(aux, d["aux"])


@pytest.mark.parametrize("shape", [(32, 3, 3, 3), (64, 32, 3, 3), (16, 1, 5, 5), (256, 128, 1, 1), (7, 5, 3, 3)])
def test_weight_quantiser_port_and_product_equal_the_reference(oracle_mod, shape):
    w, b = _weights(sum(shape), shape)
    w.ravel()[:4] = [0.0, -0.0, 1e-30, -3.0]                       # a zero, a denormal-scale value, a dominant one
    ref = oracle.ref_quant_weight_bias(w, b)
    for got in (oracle_mod.quant_weight_bias(w, b), quant.quantize_weights(w, b)):
        assert all(np.array_equal(g, r) for g, r in zip(got, ref))


def _histograms():
    rng = np.random.default_rng(99)
    out = []
    for kind in ("uniform", "relu_normal", "heavy_tail", "sparse"):
        imgs = []
        for _ in range(4):
            if kind == "uniform":
                a = rng.uniform(0, 1, 30000)
            elif kind == "relu_normal":
                a = np.maximum(rng.standard_normal(30000), 0)
            elif kind == "heavy_tail":
                a = rng.standard_normal(30000) * np.exp(rng.standard_normal(30000))
            else:
                a = rng.standard_normal(30000) * (rng.uniform(0, 1, 30000) < 0.05)
            imgs.append(a.astype(np.float32))
        out.append((kind, imgs))
    return out


@pytest.mark.parametrize("kind,imgs", _histograms(), ids=[k for k, _ in _histograms()])
def test_statistics_and_threshold_searches_equal_the_reference(oracle_mod, kind, imgs):
    """max |x| (model_quant.hpp:526-533), the 2048-bin histogram (:323-329), the MSE search (:586-619) and
    the KL search (:340-431): restatement and product against the reference's lines."""
    mx, hist = oracle.ref_stats(imgs)
    _, pmx, phist = oracle_mod._stats(imgs)
    assert np.float32(pmx) == np.float32(mx) and np.array_equal(phist, hist)
    n = imgs[0].size * len(imgs)
    ref_mse, ref_kl = oracle.ref_mse_threshold(hist, n, mx), oracle.ref_kl_threshold(hist, n, mx)
    assert oracle_mod.mse_input_scale(imgs) == np.float32(ref_mse / np.float32(127))
    assert oracle_mod.kl_input_scale(imgs) == np.float32(ref_kl / np.float32(127))
    # the product's host arithmetic takes the same histogram as integer counts
    assert quant.mse_threshold(hist.astype(np.uint32), n, mx) == ref_mse
    assert quant.kl_threshold(hist.astype(np.uint32), n, mx) == ref_kl


@pytest.mark.parametrize("kind,imgs", _histograms()[:3], ids=[k for k, _ in _histograms()[:3]])
def test_percent_threshold_equals_the_reference(oracle_mod, kind, imgs):
    """The percent method (model_quant.hpp:159-165, :173-179; 99.998 %): restatement and the product's
    host-side selection against the reference's sort-and-pick."""
    ref = oracle.ref_percent_threshold(imgs)
    assert oracle_mod.percent_input_scale(imgs) == np.float32(ref / np.float32(127))
    elem = imgs[0].size
    k = quant.percent_reserve(elem)
    kept = [a[np.argsort(-np.abs(a), kind="stable")][:k] for a in imgs]
    assert quant.percent_threshold(kept, elem, len(imgs)) == ref


def test_activation_tables_equal_the_reference_hosts(oracle_mod):
    """The SiLU and Gelu look-up tables are built on the host and handed to the operators (inputs[11]).
    Restatement and runtime against the reference host's own lines (host/ops/conv.h:180-188,
    host/ops/gelu.h:82-91), bit for bit."""
    from onenew_b200 import net as onet
    assert np.array_equal(oracle_mod.silu_lut(), oracle.ref_silu_lut())
    assert np.array_equal(oracle_mod.gelu_lut(), oracle.ref_gelu_lut())
    assert np.array_equal(onet.activation_table("silu"), oracle.ref_silu_lut())
    assert np.array_equal(onet.activation_table("gelu"), oracle.ref_gelu_lut())
