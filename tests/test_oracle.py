"""Pins the CPU restatement (oracle/oracle.c): against the golden vectors produced by the
reference's own compiled operators, and -- where oracle/_ref exists -- against those operators
run live on fresh seeded inputs.  CPU only."""
import numpy as np
import pytest

from common import golden, golden_names
from onenew_b200 import abi


def _conv_case(d):
    m = d["meta"]
    s, pads, act, has_b = int(m[0]), tuple(int(v) for v in m[1:5]), int(m[5]), int(m[6])
    return d["x"], d["w"], (d["b"] if has_b else None), (s, s), pads, act


@pytest.mark.parametrize("name", golden_names("conv") if golden_names("conv") else ["missing"])
def test_port_conv_matches_golden(oracle_mod, name):
    if name.startswith("conv8"):
        d = golden(name)
        s, pad, act = (int(v) for v in d["meta"])
        w8, b32, aux = oracle_mod.quant_weight_bias(d["w"], d["b"])
        assert np.array_equal(w8, d["w8"]) and np.array_equal(b32, d["b32"]) and np.array_equal(aux, d["aux"])
        y, acc, q = oracle_mod.conv_s8(d["x"], w8, b32, aux, d["scale"], (s, s), pad, act)
        assert np.array_equal(y, d["y"])          # int8 path: bit exact
    else:
        x, w, b, st, pads, act = _conv_case(golden(name))
        y = oracle_mod.conv_f32(x, w, b, st, pads, act)
        if b is None:
            # the bias-less entry is the one place the reference uses FMA (conv.c:498-522)
            assert np.allclose(y, golden(name)["y"], rtol=0, atol=1e-5)
        else:
            # the restatement sums k in the same order as the reference's SGEMM: bit exact
            assert np.array_equal(y, golden(name)["y"])


def test_port_gemm_matmul_match_golden(oracle_mod):
    d = golden("gemm")
    assert np.array_equal(oracle_mod.gemm(d["a"], d["w"], d["b"]), d["y"])
    for n in ("matmul_shared", "matmul_batched"):
        d = golden(n)
        assert np.allclose(oracle_mod.matmul(d["a"], d["b"]), d["y"], rtol=0, atol=1e-4)


def test_silu_lut_and_acts(oracle_mod):
    lut = oracle_mod.silu_lut()
    assert lut.shape == (8192,) and lut[4096] == 0.0 and abs(lut[8191] - 7.998046875 / (1 + np.exp(-7.998046875))) < 1e-5
    y = np.array([-9.0, -8.0, -0.001, 0.0, 3.3, 7.999, 8.0, 9.0], np.float32)
    out = oracle_mod.act(y, abi.SILU)
    assert out[0] == 0 and out[-1] == 9.0 and out[-2] == 8.0 and out[1] == lut[0]
    assert np.array_equal(oracle_mod.act(y, abi.RELU), np.maximum(y, 0))
    assert np.array_equal(oracle_mod.act(y, abi.RELU6), y)      # never handled by the reference: identity


def test_quantise_rounds_half_away_from_zero(oracle_mod):
    x = np.array([0.5, 1.5, 2.5, -0.5, -2.5, 126.5, 127.4, 300.0, -128.5, -400.0], np.float32)
    q = oracle_mod.quantize_s8(x, np.float32(1.0))
    assert q.tolist() == [1, 2, 3, -1, -3, 127, 127, 127, -128, -128]


@pytest.mark.parametrize("seed", [1, 2])
def test_port_matches_live_reference(oracle_mod, seed):
    if not oracle_mod.have_reference():
        pytest.skip("oracle/_ref not built (no reference tree on this machine)")
    rng = np.random.default_rng(seed)
    # config-1 shape: 64->64 3x3 s1 p1 + ReLU on 56x56
    x = rng.uniform(-1, 1, (1, 64, 56, 56)).astype(np.float32)
    w = (rng.standard_normal((64, 64, 3, 3)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(64) * 0.01).astype(np.float32)
    assert np.array_equal(oracle_mod.ref_conv(x, w, b, (1, 1), (1, 1, 1, 1), abi.RELU),
                          oracle_mod.conv_f32(x, w, b, (1, 1), (1, 1, 1, 1), abi.RELU))
    # 1x1 stride 1 goes through the reference's other entry (eval_1x1j1)
    w1 = (rng.standard_normal((32, 64, 1, 1)) * 0.05).astype(np.float32)
    assert np.allclose(oracle_mod.ref_conv(x, w1, b[:32], (1, 1), (0, 0, 0, 0), abi.RELU),
                       oracle_mod.conv_f32(x, w1, b[:32], (1, 1), (0, 0, 0, 0), abi.RELU), rtol=0, atol=1e-5)
    # int8, stride 2, SiLU: bit exact
    x8 = rng.uniform(0, 1, (1, 32, 24, 24)).astype(np.float32)
    w8, b32, aux = oracle_mod.quant_weight_bias((rng.standard_normal((48, 32, 3, 3)) * 0.05).astype(np.float32), b[:48])
    sc = np.float32(1 / 127)
    yr = oracle_mod.ref_conv(x8, w8, b32, (2, 2), (1, 1, 1, 1), abi.SILU, int8=(sc, aux))
    yp, _, _ = oracle_mod.conv_s8(x8, w8, b32, aux, sc, (2, 2), 1, abi.SILU)
    assert np.array_equal(yr, yp)
    a = rng.standard_normal((3, 197, 64)).astype(np.float32)
    bm = rng.standard_normal((3, 64, 197)).astype(np.float32)
    assert np.allclose(oracle_mod.ref_matmul(a, bm), oracle_mod.matmul(a, bm), rtol=0, atol=1e-4)


@pytest.mark.parametrize("name", ["dw3x3_p1_relu", "dw3x3_s2_p1", "dw5x5_p2_silu"])
def test_port_depthwise_matches_golden(oracle_mod, name):
    d = golden(name)
    s, pd, act = (int(v) for v in d["meta"])
    y = oracle_mod.dwconv_f32(d["x"], d["w"], d["b"], (s, s), (pd,) * 4, act)
    assert np.array_equal(y, d["y"])


@pytest.mark.parametrize("name", ["dw8_3x3_p1_relu", "dw8_3x3_s2_p1", "dw8_5x5_p2_leaky"])
def test_port_depthwise_int8_matches_golden(oracle_mod, name):
    d = golden(name)
    s, pd, act = (int(v) for v in d["meta"])
    y = oracle_mod.dwconv_s8(d["x"], d["w8"], d["b32"], d["aux"], float(d["scale"]), (s, s), pd, act)
    assert np.array_equal(y, d["y"])


def test_kl_and_percent_restatements_behave(oracle_mod):
    """No reference binary exists for the calibrators (they need its whole runtime), so the restatements
    are checked on properties: thresholds lie inside the data range, the percent threshold is the value at
    the documented rank, and clipping outliers moves the KL threshold below the maximum."""
    rng = np.random.default_rng(3)
    xs = [np.maximum(rng.standard_normal((8, 50, 50)) * 2, 0).astype(np.float32) for _ in range(4)]
    xs[0][0, 0, 0] = 40.0                                   # one outlier
    mx = max(float(x.max()) for x in xs)
    kl, pc, mse = oracle_mod.kl_input_scale(xs), oracle_mod.percent_input_scale(xs), oracle_mod.mse_input_scale(xs)
    for s in (kl, pc, mse):
        assert 0 < s <= np.float32(mx / 127) * np.float32(1.001)
    assert kl < np.float32(mx / 127) * 0.5 and pc < np.float32(mx / 127) * 0.5     # the outlier is clipped
    allv = np.sort(np.concatenate([x.ravel() for x in xs]))[::-1]
    idx = int(np.float32(np.float32(np.float32(1) - np.float32(99.998 / 100)) * np.float32(4)) * np.float32(xs[0].size))
    assert pc == np.float32(allv[idx] / np.float32(127))
