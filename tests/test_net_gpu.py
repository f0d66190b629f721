"""Model-level parity of the device-resident runtime against operands computed by the reference's
own x86 operators (tests/golden/resnet_small.npz, made by tests/golden/make_golden.py)."""
import numpy as np
import pytest

from common import assert_close, golden
from onenew_b200 import models, net as onet

pytestmark = pytest.mark.gpu
KEEP = ["Conv_0_out", "MaxPool_0_out", "Relu_0_0_out", "Relu_0_1_out", "Relu_3_0_out", "gap_out", "output"]


def _image():
    return models.build_resnet50(seed=3, num_classes=10, image=32, width=16, blocks=(2, 1, 1, 1)).tobytes()


@pytest.mark.parametrize("fuse", [False, True])
@pytest.mark.parametrize("graph", [False, True])
def test_small_resnet_tf32_matches_reference_per_layer(fuse, graph):
    g = golden("resnet_small")
    n = onet.Net(_image(), batch=2, precision="tf32", fuse=fuse, graph=graph)
    try:
        y = n(g["x"])
        assert_close(y, g["output"], "logits")
        y2 = n(g["x"])                      # second run (CUDA-graph replay when enabled) is deterministic
        assert np.array_equal(y, y2)
        have = set(n.operands())
        for k in KEEP:
            if k in have:
                assert_close(n.fetch(k, g[k].shape), g[k], k)
        flops, nbytes, launches = n.work()
        assert flops > 0 and nbytes > 0 and launches >= 10
    finally:
        n.close()


def test_small_resnet_bf16_mode_within_the_float_tolerance():
    """bf16 mode (bf16 activations inside a block, the residual trunk kept in fp32): logits and the kept
    intermediate operands meet the same criteria as TF32."""
    g = golden("resnet_small")
    n = onet.Net(_image(), batch=2, precision="bf16")
    try:
        y = n(g["x"])
        assert_close(y, g["output"], "logits (bf16 mode)")
        have = set(n.operands())
        for k in KEEP:
            if k in have:
                assert_close(n.fetch(k, g[k].shape), g[k], k + " (bf16 mode)")
    finally:
        n.close()


@pytest.mark.parametrize("fuse", [False, True])
def test_small_resnet_f16_mode_meets_the_float_tolerance_at_every_kept_operand(fuse):
    """fp16 storage (every activation and weight in 16 bits, the mantissa width of tf32, fp32 accumulate):
    the same criteria as TF32, at the logits and at every kept intermediate operand; nothing left the
    format's range."""
    g = golden("resnet_small")
    n = onet.Net(_image(), batch=2, precision="f16", fuse=fuse)
    try:
        y = n(g["x"])
        assert_close(y, g["output"], "logits (f16 mode)")
        assert np.array_equal(y, n(g["x"]))
        have = set(n.operands())
        assert sum(k in have for k in KEEP) >= 3
        for k in KEEP:
            if k in have:
                assert_close(n.fetch(k, g[k].shape), g[k], k + " (f16 mode)")
        assert any("dtype=f16" in line for line in onet.describe(_image(), batch=2, precision="f16"))
    finally:
        n.close()


def test_residual_added_by_the_tensor_core_matches_the_epilogue_add():
    """16-bit storage: a folded residual is added either by the epilogue (patches of the residual tensor) or by
    the tensor core (the residual as further operand stages times an identity tile).  Both meet the float
    tolerance against the reference, and they agree with each other to the rounding of one fp32 add."""
    from onenew_b200 import capi
    g = golden("resnet_small")
    L = capi.lib()
    ys = {}
    try:
        for mode in (7, 15):
            capi.check(L.one_cuda_set_epilogue_mode(mode))
            n = onet.Net(_image(), batch=2, precision="f16")
            try:
                ys[mode] = n(g["x"])
                assert_close(ys[mode], g["output"], f"logits, epilogue mode {mode}")
            finally:
                n.close()
    finally:
        L.one_cuda_set_epilogue_mode(15)
    assert np.abs(ys[7] - ys[15]).max() <= 2e-3 * np.abs(ys[7]).max()


def test_f16_mode_reports_a_value_outside_the_format(oracle_mod):
    """A conv whose output exceeds 65504 in fp16 storage: the run reports ONE_ERR_RANGE (nothing faults, the
    context stays usable), and the same model runs in TF32."""
    from onenew_b200 import abi, capi
    from onenew_b200.one_file import OneBuilder
    rng = np.random.default_rng(5)
    C = 32
    w = (rng.standard_normal((C, C, 3, 3))).astype(np.float32)
    b = np.zeros(C, np.float32)
    bld = OneBuilder()
    bld.add_io("input", "input", (1, C, 8, 8))
    bld.conv("Conv_0", "input", bld.add_init("w0", w), bld.add_init("b0", b), "c0", (3, 3), (1, 1), (1, 1, 1, 1), act=abi.RELU)
    bld.conv("Conv_1", "c0", bld.add_init("w1", w), bld.add_init("b1", b), "output", (3, 3), (1, 1), (1, 1, 1, 1))
    bld.add_io("output", "output", (1, C, 8, 8))
    img = bld.tobytes()
    small = rng.uniform(-1, 1, (1, C, 8, 8)).astype(np.float32)
    big = small * 4000.0                                    # Conv_0's outputs reach ~1e5
    ref = oracle_mod.conv_f32(np.maximum(oracle_mod.conv_f32(small, w, b, (1, 1), (1, 1, 1, 1), abi.RELU), 0), w, b, (1, 1), (1, 1, 1, 1), abi.NOT_ACT)
    n = onet.Net(img, batch=1, precision="f16")
    try:
        assert_close(n(small), ref, "in range")
        with pytest.raises(capi.OneCudaError, match="ONE_ERR_RANGE"):
            n(big)
        assert_close(n(small), ref, "after the report")      # the context is still usable
    finally:
        n.close()
    n = onet.Net(img, batch=1, precision="tf32")
    try:
        assert np.isfinite(n(big)).all()
    finally:
        n.close()


def _split_k(mode):
    from onenew_b200 import capi
    capi.check(capi.lib().one_cuda_set_split_k(mode))


def test_batch_is_per_image_independent():
    """Sharding property used by the multi-GPU path: running images separately or in one batch gives
    the same logits.  With every contraction summing K in one piece the results are bit-identical; with
    split-K (which a small batch turns on for more layers than a large one) they agree to summation-order
    noise, far inside the float tolerance."""
    g = golden("resnet_small")
    img = _image()
    for mode in (1, 0):                       # 1: never split, 0: the library's own choice
        _split_k(mode)
        try:
            n2 = onet.Net(img, batch=2)
            n1 = onet.Net(img, batch=1)
            try:
                y2 = n2(g["x"])
                y1 = np.concatenate([n1(g["x"][i:i + 1]) for i in range(2)])
                if mode == 1:
                    assert np.array_equal(y1, y2)
                else:
                    assert np.abs(y1 - y2).max() <= 5e-3 * np.abs(y2).max()
            finally:
                n1.close()
                n2.close()
        finally:
            _split_k(0)


def test_trace_csv_schema(tmp_path):
    """The runtime's tracing CSV: the reference's twelve columns (host/net.h:539-611), hardware and model
    fields on the first data row where its timeline tool reads them, bytes and detail appended."""
    n = onet.Net(_image(), batch=2)
    try:
        n(golden("resnet_small")["x"])
        p = tmp_path / "trace.csv"
        n.trace(p, runs=2, model_name="resnet_small")
        lines = p.read_text().strip().split("\n")
        assert lines[0] == ("op_name,op_type,op_st,op_ed,op_computation,,cpu,cpu_hw_info,gpu,gpu_hw_info,"
                            "hw_computing_power (GOPS),model name,op_bytes,op_detail")
        rows = [ln.split(",") for ln in lines[1:]]
        assert all(len(r) == 14 for r in rows)
        hw = rows[0][6:]                                   # as tools/perf_profiling/gen_timeline_json.py:41-42 slices it
        assert float(hw[4]) > 0 and "B200" in hw[2] and hw[5] == "resnet_small"
        convs = [r for r in rows if r[1] == "Conv"]
        assert convs and all(float(r[4]) > 0 and float(r[3]) > float(r[2]) and "tile=128x" in r[13] for r in convs)
        assert float(rows[-1][3]) >= float(rows[0][3])
    finally:
        n.close()


def test_full_resnet50_batch_invariance_and_reference_sample(oracle_mod):
    """Full-size model: image 0 of a batch of 8 equals the same image run alone (size-independent
    property: bit for bit when no contraction splits K, to summation-order noise with the library's own
    split choices), and -- when the reference build is present -- matches the reference's logits."""
    img = models.build_resnet50().tobytes()
    x = models.resnet50_input(8)
    for mode in (1, 0):
        _split_k(mode)
        try:
            n8 = onet.Net(img, batch=8)
            n1 = onet.Net(img, batch=1)
            try:
                y8 = n8(x)
                y1 = n1(x[:1])
                if mode == 1:
                    assert np.array_equal(y8[:1], y1)
                else:
                    assert np.abs(y8[:1] - y1).max() <= 5e-3 * np.abs(y1).max()
                if oracle_mod.have_reference():
                    from oracle.model_ref import RefNet
                    ref = RefNet(img).run(x[:1])["output"]
                    assert_close(y1, ref, "resnet50 logits")
            finally:
                n1.close()
                n8.close()
        finally:
            _split_k(0)


def test_pipelined_host_submission_equals_blocking_path():
    import torch
    g = golden("resnet_small")
    n = onet.Net(_image(), batch=2)
    try:
        ref = n(g["x"])
        xa = torch.from_numpy(g["x"]).pin_memory()
        xb = torch.from_numpy(g["x"][::-1].copy()).pin_memory()
        ya = torch.empty(ref.shape).pin_memory()
        yb = torch.empty(ref.shape).pin_memory()
        for _ in range(3):                   # back-to-back submissions overlap copy and compute
            n.submit_host(xa, ya)
            n.submit_host(xb, yb)
        n.sync()
        assert np.array_equal(ya.numpy(), ref) and np.array_equal(yb.numpy(), ref[::-1])
    finally:
        n.close()


def test_int8_backbone_chain_bit_exact():
    """YOLOv8s-shaped int8 conv stack through the runtime: every layer's fp32 output equals the
    reference's bit for bit (s32 accumulation exact, de-quantisation in the reference's order, next
    layer's quantisation therefore identical)."""
    import oracle
    g = golden("yolo_int8_small")
    ws = models.yolo_backbone_weights()
    quant = [oracle.quant_weight_bias(w, b) + (s,) for (w, b), s in zip(ws, g["scales"])]
    img = models.build_yolo_backbone(ws, image=96, quant=quant).tobytes()
    n = onet.Net(img, batch=1, fuse=False)      # operator by operator: fp32 activations between the convs
    try:
        y = n(g["x"])
        for k in ("Conv_0_out", "Conv_3_out", "Conv_9_out"):
            got = n.fetch(k, g[k].shape)
            assert np.array_equal(got, g[k]), f"{k}: {(got != g[k]).sum()} of {got.size} differ"
        assert np.array_equal(y, g["output"])
    finally:
        n.close()
    # fused chain: each conv's epilogue writes the activation already quantised for its reader (no fp32
    # copy); those integers equal the reference's quantisation of its own fp32 activation, and the
    # network output is still the reference's bit for bit
    n = onet.Net(img, batch=1)
    try:
        y = n(g["x"])
        assert np.array_equal(y, g["output"])
        for k, nxt in (("Conv_0_out", 1), ("Conv_3_out", 4), ("Conv_9_out", 10)):
            q = n.fetch(k, g[k].shape)
            assert np.array_equal(q, oracle.quantize_s8(g[k], g["scales"][nxt]).astype(np.float32)), k
        assert n.work()[2] == len(models.YOLO_STACK) + 2      # 13 convs + input pack + output re-layout: no separate quantise passes
    finally:
        n.close()
    # batch independence at batch 3
    n3 = onet.Net(img, batch=3)
    try:
        x3 = np.concatenate([g["x"], models.yolo_input(2, seed=300, image=96)])
        assert np.array_equal(n3(x3)[:1], g["output"])
    finally:
        n3.close()


def test_device_calibration_statistics_match_the_restated_quantiser(oracle_mod):
    """abs-max, the 2048-bin histogram and the MSE threshold taken on the device equal the C restatement
    of model_quant.hpp bit for bit on the same tensor; so does the weight quantiser."""
    import ctypes as C
    import torch
    from onenew_b200 import capi, quant
    rng = np.random.default_rng(11)
    x = np.maximum(rng.standard_normal((3, 40, 33, 7)) * 2.5, 0).astype(np.float32)     # post-ReLU-like, many zeros
    xd = torch.from_numpy(x).cuda()
    mx = torch.zeros(1, device="cuda")
    hist = torch.zeros(2048, dtype=torch.int32, device="cuda")
    L = capi.lib()
    capi.check(L.one_quant_abs_max(C.c_void_p(xd.data_ptr()), 0, C.c_longlong(x.size), C.c_void_p(mx.data_ptr()), None))
    torch.cuda.synchronize()
    m = float(mx.item())
    assert m == float(np.abs(x).max())
    capi.check(L.one_quant_abs_histogram(C.c_void_p(xd.data_ptr()), 0, C.c_longlong(x.size), C.c_float(m), C.c_void_p(hist.data_ptr()), None))
    torch.cuda.synchronize()
    ref_hist = np.zeros(2048, np.float32)
    P = oracle_mod.port()
    P.oracle_hist_accumulate(C.c_void_p(x.ctypes.data), C.c_int64(x.size), C.c_float(m), C.c_void_p(ref_hist.ctypes.data))
    assert np.array_equal(hist.cpu().numpy().astype(np.float32), ref_hist)
    thr = quant.mse_threshold(hist.cpu().numpy(), x.size, m)
    assert np.float32(thr / np.float32(127)) == oracle_mod.mse_input_scale([x])
    w = (rng.standard_normal((16, 8, 3, 3)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(16) * 0.01).astype(np.float32)
    for got, ref in zip(quant.quantize_weights(w, b), oracle_mod.quant_weight_bias(w, b)):
        assert np.array_equal(got, ref)


def test_calibrate_and_quantise_a_model_on_the_gpu():
    """End to end: fp32 conv stack -> MSE calibration on the device -> int8 image in the reference's
    format -> int8 inference close to the fp32 one."""
    from onenew_b200 import quant
    ws = models.yolo_backbone_weights()
    IM = 96
    fp32 = models.build_yolo_backbone(ws, image=IM).tobytes()
    cal = models.yolo_input(4, image=IM)
    scales = quant.calibrate_mse(fp32, cal)
    assert len(scales) == len(models.YOLO_STACK) and all(0 < s < 1 for s in scales.values())
    q = quant.quantize_model(fp32, scales)
    nf, nq = onet.Net(fp32, batch=1), onet.Net(q, batch=1)
    try:
        yf, yq = nf(cal[:1]), nq(cal[:1])
        a, b = yf.astype(np.float64).ravel(), yq.astype(np.float64).ravel()
        assert a @ b / (np.linalg.norm(a) * np.linalg.norm(b)) > 0.98
    finally:
        nf.close()
        nq.close()
    # calibration scales agree with the golden ones (made from the reference's fp32 activations) to within a bin or two
    g = golden("yolo_int8_small")
    cal8 = models.yolo_input(8, image=IM)
    s8 = quant.calibrate_mse(fp32, cal8)
    got = np.array([s8[f"Conv_{i}"] for i in range(len(models.YOLO_STACK))], np.float32)
    assert np.allclose(got, g["scales"], rtol=0.05)


def test_int8_depthwise_separable_stack_bit_exact(oracle_mod):
    """A MobileNet-shaped int8 stack (dense stem, depthwise 3x3, pointwise 1x1) quantised by this
    package's tool: every layer of the runtime equals the restated reference chained layer by layer."""
    from onenew_b200 import abi, quant
    from onenew_b200.one_file import OneBuilder
    rng = np.random.default_rng(31)
    IM = 48
    # cin, cout, k, stride, pad, group, act
    stack = [(3, 16, 3, 2, 1, 1, abi.RELU), (16, 16, 3, 1, 1, 16, abi.RELU), (16, 32, 1, 1, 0, 1, abi.RELU),
             (32, 32, 3, 2, 1, 32, abi.CLIP), (32, 64, 1, 1, 0, 1, abi.NOT_ACT)]
    b = OneBuilder()
    b.add_io("input", "input", (1, 3, IM, IM))
    x, hw, ws = "input", IM, []
    for i, (ci, co, k, s, p, grp, act) in enumerate(stack):
        w = (rng.standard_normal((co, ci // grp, k, k)) * np.sqrt(2.0 / (ci // grp * k * k))).astype(np.float32)
        bias = (rng.standard_normal(co) * 0.05).astype(np.float32)
        ws.append((w, bias))
        out = "output" if i == len(stack) - 1 else f"Conv_{i}_out"
        b.conv(f"Conv_{i}", x, b.add_init(f"Conv_{i}.weight", w), b.add_init(f"Conv_{i}.bias", bias), out, (k, k), (s, s),
               (p, p, p, p), act=act, group=grp)
        hw = (hw + 2 * p - k) // s + 1
        x = out
    b.add_io("output", "output", (1, stack[-1][1], hw, hw))
    fp32 = b.tobytes()
    scales = {f"Conv_{i}": np.float32(sc) for i, sc in enumerate([1 / 127, 0.02, 0.03, 0.03, 0.05])}
    img = quant.quantize_model(fp32, scales)
    xin = rng.uniform(0, 1, (2, 3, IM, IM)).astype(np.float32)
    # the restated reference, chained
    want, cur = {}, xin
    for i, ((ci, co, k, s, p, grp, act), (w, bias)) in enumerate(zip(stack, ws)):
        w8, b32, aux = oracle_mod.quant_weight_bias(w, bias)
        sc = float(scales[f"Conv_{i}"])
        if grp == 1:
            cur = oracle_mod.conv_s8(cur, w8, b32, aux, sc, (s, s), p, act)[0]
        else:
            cur = oracle_mod.dwconv_s8(cur, w8, b32, aux, sc, (s, s), p, act)
        want[f"Conv_{i}_out" if i < len(stack) - 1 else "output"] = cur
    for fuse in (False, True):
        n = onet.Net(img, batch=2, fuse=fuse)
        try:
            y = n(xin)
            assert np.array_equal(y, want["output"]), fuse
            if not fuse:
                for k_ in ("Conv_0_out", "Conv_1_out", "Conv_3_out"):
                    assert np.array_equal(n.fetch(k_, want[k_].shape), want[k_]), k_
        finally:
            n.close()


def test_tile_autotune_keeps_results_and_reports_every_contraction():
    """The tile search times each Conv / Gemm at every tile width and re-prepares it with the winner; the
    network's output does not depend on the choice, and a saved choice can be replayed per operator."""
    from onenew_b200 import capi
    g = golden("resnet_small")
    n = onet.Net(_image(), batch=2)
    try:
        y0 = n(g["x"])
        rep = n.autotune(runs=2)
        from onenew_b200.one_file import OneModel
        assert len(rep) == sum(t in ("Conv", "Gemm") for t, _ in OneModel(_image()).nodes)   # every contraction of the model
        assert all(bn in (0, 64, 128, 192, 256, 1128, 1192, 1256, 2064, 2128, 4064, 4128) and best <= heur * 1.0001 for _, heur, bn, best in rep.values())
        assert set(n.tuned_split) == set(rep) and all(0 <= v <= 64 for v in n.tuned_split.values())
        y1 = n(g["x"])
        assert_close(y1, y0, "after autotune")
        n.set_tile("Conv_3", 64)
        n.set_tile("Gemm_0", 128)
        assert_close(n(g["x"]), y0, "forced tiles")
        with pytest.raises(capi.OneCudaError):
            n.set_tile("Conv_3", 96)
        with pytest.raises(capi.OneCudaError):
            n.set_tile("MaxPool_0", 64)
    finally:
        n.close()


def test_two_half_tiles_on_every_conv_bit_identical_to_plain_tiles():
    """Two 128-row halves per CTA on every conv of a network (those with a folded residual included): the same
    sums in the same order as the plain tiles of that width.  A fresh network: a tile search would leave
    per-operator split-K choices behind, which only the plain tiles honour."""
    from onenew_b200 import capi
    from onenew_b200.one_file import OneModel
    g = golden("resnet_small")
    L = capi.lib()
    convs = [cfg.op_base_cfg.op_name.decode() for t, cfg in OneModel(_image()).nodes if t == "Conv"]
    try:
        capi.check(L.one_cuda_set_split_k(1))
        n = onet.Net(_image(), batch=2)
        try:
            y0 = n(g["x"])
            for width in (64, 128):
                for k in convs:
                    n.set_tile(k, width)
                ya = n(g["x"])
                for extra in (2000, 4000):   # two halves per CTA; twelve epilogue warps
                    for k in convs:
                        n.set_tile(k, extra + width)
                    yb = n(g["x"])
                    assert np.array_equal(ya, yb), (width, extra)
                    assert_close(yb, y0, f"tile code {extra + width}")
        finally:
            n.close()
    finally:
        L.one_cuda_set_split_k(0)


def test_kl_and_percent_calibrators_match_the_restated_quantiser(oracle_mod):
    """KL threshold search on the device histogram and the percent method's largest-|x| selection equal
    the C / numpy restatement of model_quant.hpp on the same tensors."""
    import ctypes as C
    import torch
    from onenew_b200 import capi, quant
    rng = np.random.default_rng(12)
    L = capi.lib()
    for signed in (False, True):
        imgs = [(rng.standard_normal((24, 61, 47)) * 1.7).astype(np.float32) for _ in range(3)]
        if not signed:
            imgs = [np.maximum(a, 0) for a in imgs]
        dev = [torch.from_numpy(a).cuda() for a in imgs]
        mx = torch.zeros(1, device="cuda")
        hist = torch.zeros(2048, dtype=torch.int32, device="cuda")
        for d in dev:
            capi.check(L.one_quant_abs_max(C.c_void_p(d.data_ptr()), 0, C.c_longlong(d.numel()), C.c_void_p(mx.data_ptr()), None))
        torch.cuda.synchronize()
        m = float(mx.item())
        for d in dev:
            capi.check(L.one_quant_abs_histogram(C.c_void_p(d.data_ptr()), 0, C.c_longlong(d.numel()), C.c_float(m), C.c_void_p(hist.data_ptr()), None))
        torch.cuda.synchronize()
        n_all = sum(a.size for a in imgs)
        thr = quant.kl_threshold(hist.cpu().numpy(), n_all, m)
        assert np.float32(thr / np.float32(127)) == oracle_mod.kl_input_scale(imgs)
        k = quant.percent_reserve(imgs[0].size)
        assert k > 10
        kept = [quant._largest_abs(L, torch, d.data_ptr(), d.numel(), 0, k, None, "cuda:0") for d in dev]
        for a, got in zip(imgs, kept):
            assert np.array_equal(np.abs(got), np.sort(np.abs(a).ravel())[::-1][:k])
        got_scale = np.float32(quant.percent_threshold(kept, imgs[0].size, len(imgs)) / np.float32(127))
        assert abs(got_scale) == abs(oracle_mod.percent_input_scale(imgs))     # sign of a tie at the cut is unspecified in both


@pytest.mark.parametrize("method", ["kl", "percent"])
def test_calibrate_other_methods_end_to_end(method):
    from onenew_b200 import quant
    ws = models.yolo_backbone_weights()
    IM = 96 if method == "kl" else 256      # the percent method keeps (1 - 0.99998) * 10 of each operand: it needs >= 5000 elements
    fp32 = models.build_yolo_backbone(ws, image=IM).tobytes()
    cal = models.yolo_input(4, image=IM)
    if method == "percent":
        with pytest.raises(ValueError):
            quant.calibrate(models.build_yolo_backbone(ws, image=96).tobytes(), models.yolo_input(2, image=96), method)
    scales = quant.calibrate(fp32, cal, method)
    # the percent threshold is signed in the reference (a negative SiLU value can sit at the cut); its sign cancels in the conv
    assert len(scales) == len(models.YOLO_STACK) and all(0 < abs(s) < 1 for s in scales.values()), scales
    q = quant.quantize_model(fp32, scales)
    nf, nq = onet.Net(fp32, batch=1), onet.Net(q, batch=1)
    try:
        yf, yq = nf(cal[:1]), nq(cal[:1])
        a, b = yf.astype(np.float64).ravel(), yq.astype(np.float64).ravel()
        assert a @ b / (np.linalg.norm(a) * np.linalg.norm(b)) > 0.97
    finally:
        nf.close()
        nq.close()


@pytest.mark.parametrize("shape", [(2, 13, 15, 8), (1, 12, 12, 16), (3, 7, 9, 4)])
@pytest.mark.parametrize("pad", [0, 1])
def test_maxpool_3x3_s2_odd_sizes_against_numpy(shape, pad):
    """The specialised 3x3 / stride-2 pool (two outputs per thread) on odd widths and both paddings:
    window max with the reference's padding value (device/x86/MaxPool/maxpool.c:40-90)."""
    import ctypes as C
    import torch
    from onenew_b200 import capi
    N, H, W, Cc = shape
    rng = np.random.default_rng(N * 100 + H)
    x = rng.standard_normal(shape).astype(np.float32)
    OH, OW = (H + 2 * pad - 3) // 2 + 1, (W + 2 * pad - 3) // 2 + 1
    xd = torch.from_numpy(x).cuda()
    yd = torch.empty((N, OH, OW, Cc), dtype=torch.float32, device="cuda")
    capi.check(capi.lib().one_glue_maxpool_nhwc(C.c_void_p(xd.data_ptr()), C.c_void_p(yd.data_ptr()), 0, N, H, W, Cc, 3, 3, 2, 2, pad, None))
    torch.cuda.synchronize()
    xp = np.full((N, H + 2 * pad, W + 2 * pad, Cc), -3276800.0, np.float32)
    xp[:, pad:pad + H, pad:pad + W] = x
    want = np.stack([[xp[:, 2 * i:2 * i + 3, 2 * j:2 * j + 3].max(axis=(1, 2)) for j in range(OW)] for i in range(OH)])   # [OH][OW][N][C]
    assert np.array_equal(yd.cpu().numpy(), want.transpose(2, 0, 1, 3))


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("shape", [(2, 13, 15, 8), (1, 12, 12, 16), (3, 7, 9, 24)])
@pytest.mark.parametrize("pad", [0, 1])
def test_maxpool_3x3_s2_16_bit_activations_bit_exact(shape, pad, dtype):
    """The 16-bit form of the specialised pool takes its maxima on the packed pairs as they lie in memory:
    bit-identical to the window maximum of the same 16-bit values, odd widths and both paddings."""
    import ctypes as C
    import torch
    from onenew_b200 import capi
    N, H, W, Cc = shape
    rng = np.random.default_rng(N * 100 + H + pad)
    tdt, code = (torch.float16, 3) if dtype == "f16" else (torch.bfloat16, 1)
    xd = torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).cuda().to(tdt)
    OH, OW = (H + 2 * pad - 3) // 2 + 1, (W + 2 * pad - 3) // 2 + 1
    yd = torch.empty((N, OH, OW, Cc), dtype=tdt, device="cuda")
    capi.check(capi.lib().one_glue_maxpool_nhwc(C.c_void_p(xd.data_ptr()), C.c_void_p(yd.data_ptr()), code, N, H, W, Cc, 3, 3, 2, 2, pad, None))
    torch.cuda.synchronize()
    want = torch.nn.functional.max_pool2d(xd.float().permute(0, 3, 1, 2), 3, 2, pad).permute(0, 2, 3, 1)
    assert torch.equal(yd.float().cpu(), want.cpu())


def test_nan_and_inf_survive_the_tf32_store():
    """Activations kept on the device are rounded to tf32 when they are stored.  A NaN or an infinity the
    convolution produces must come through that rounding as it is (the reference's fp32 arithmetic keeps
    both), not turn into a finite number."""
    from onenew_b200 import abi
    from onenew_b200.one_file import OneBuilder
    rng = np.random.default_rng(23)
    C, HW = 32, 10
    w = (rng.standard_normal((C, C, 3, 3)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(C) * 0.01).astype(np.float32)
    bld = OneBuilder()
    bld.add_io("input", "input", (1, C, HW, HW))
    bld.conv("Conv_0", "input", bld.add_init("w", w), bld.add_init("b", b), "output", (3, 3), (1, 1), (1, 1, 1, 1), act=abi.NOT_ACT)
    bld.add_io("output", "output", (1, C, HW, HW))
    x = rng.uniform(-1, 1, (3, C, HW, HW)).astype(np.float32)
    x[0, 1, 5, 5] = np.nan
    x[1, 0, 3, 3] = np.inf
    n = onet.Net(bld.tobytes(), batch=3)
    try:
        y = n(x)
        assert np.isnan(y[0, :, 4:7, 4:7]).all()                 # every output whose window holds the NaN
        assert np.isfinite(np.delete(y[0].reshape(C, -1), [44, 45, 46, 54, 55, 56, 64, 65, 66], axis=1)).all()
        assert np.isinf(y[1, :, 2:5, 2:5]).all()                 # inf * w = +-inf, summed with finite terms
        assert np.isfinite(y[2]).all()
    finally:
        n.close()


@pytest.mark.parametrize("precision", ["tf32", "bf16", "f16"])
def test_skip_connection_from_the_network_input(oracle_mod, precision):
    """Conv -> Add(network input) -> Relu: the folded Add's other operand is in the reference layout, not
    the conv's NHWC output form; the runtime converts it instead of refusing the model."""
    from onenew_b200 import abi
    from onenew_b200.one_file import OneBuilder
    rng = np.random.default_rng(17)
    C, HW = 32, 12
    w = (rng.standard_normal((C, C, 3, 3)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(C) * 0.01).astype(np.float32)
    bld = OneBuilder()
    bld.add_io("input", "input", (1, C, HW, HW))
    bld.conv("Conv_0", "input", bld.add_init("w", w), bld.add_init("b", b), "c0", (3, 3), (1, 1), (1, 1, 1, 1), act=abi.NOT_ACT)
    bld.simple("Add", "Add_0", ["c0", "input"], "a0")
    bld.simple("Relu", "Relu_0", ["a0"], "output")
    bld.add_io("output", "output", (1, C, HW, HW))
    x = rng.uniform(-1, 1, (3, C, HW, HW)).astype(np.float32)
    ref = np.maximum(oracle_mod.conv_f32(x, w, b, (1, 1), (1, 1, 1, 1), abi.NOT_ACT) + x, 0)
    for fuse in (True, False):
        n = onet.Net(bld.tobytes(), batch=3, precision=precision, fuse=fuse)
        try:
            y = n(x)
            if precision == "tf32":
                assert_close(y, ref, f"skip from input, fuse={fuse}")
            else:
                assert np.abs(y - ref).max() / np.abs(ref).max() < 3e-2
        finally:
            n.close()


@pytest.mark.parametrize("precision", ["tf32", "bf16", "f16"])
def test_width_pairing_of_narrow_convs_matches_unpaired_and_oracle(oracle_mod, precision):
    """A stride-1 3x3 convolution with 64 (32) output channels on device-resident activations is computed on
    pairs of adjacent output pixels (KH x (KW + 1) filter, stride 2 along w, twice the channels).  Same
    products, other grouping: the result agrees with the unpaired evaluation and with the oracle, with a
    residual, an odd height, unequal pads and a 5-wide filter in the mix."""
    from onenew_b200 import abi, capi
    from onenew_b200.one_file import OneBuilder
    rng = np.random.default_rng(41)
    f = lambda *s: (rng.standard_normal(s) * 0.05).astype(np.float32)
    w0, b0 = f(64, 16, 3, 3), f(64)
    w1, b1 = f(64, 64, 3, 3), f(64)          # paired, then Add(residual) + Relu folded into it
    w2, b2 = f(32, 64, 3, 5), f(32)          # 3 x 5 filter, pads (1, 2, 1, 2), 32 output channels: paired
    w3, b3 = f(64, 32, 1, 1), f(64)          # 1 x 1: never paired
    bld = OneBuilder()
    bld.add_io("input", "input", (1, 16, 13, 20))
    bld.conv("Conv_0", "input", bld.add_init("w0", w0), bld.add_init("b0", b0), "c0", (3, 3), (1, 1), (1, 1, 1, 1), act=abi.RELU)
    bld.conv("Conv_1", "c0", bld.add_init("w1", w1), bld.add_init("b1", b1), "c1", (3, 3), (1, 1), (1, 1, 1, 1), act=abi.NOT_ACT)
    bld.simple("Add", "Add_0", ["c1", "c0"], "a0")
    bld.simple("Relu", "Relu_0", ["a0"], "r0")
    bld.conv("Conv_2", "r0", bld.add_init("w2", w2), bld.add_init("b2", b2), "c2", (3, 5), (1, 1), (1, 2, 1, 2), act=abi.LEAKYRELU)
    bld.conv("Conv_3", "c2", bld.add_init("w3", w3), bld.add_init("b3", b3), "output", (1, 1), (1, 1), (0, 0, 0, 0), act=abi.NOT_ACT)
    bld.add_io("output", "output", (1, 64, 13, 20))
    x = rng.uniform(-1, 1, (3, 16, 13, 20)).astype(np.float32)
    c0 = oracle_mod.conv_f32(x, w0, b0, (1, 1), (1, 1, 1, 1), abi.RELU)
    r0 = np.maximum(oracle_mod.conv_f32(c0, w1, b1, (1, 1), (1, 1, 1, 1), abi.NOT_ACT) + c0, 0)
    c2 = oracle_mod.conv_f32(r0, w2, b2, (1, 1), (1, 2, 1, 2), abi.LEAKYRELU)
    ref = oracle_mod.conv_f32(c2, w3, b3, (1, 1), (0, 0, 0, 0), abi.NOT_ACT)
    outs, details = {}, {}
    for on in (1, 0):
        capi.check(capi.lib().one_cuda_set_width_pairing(on))
        try:
            n = onet.Net(bld.tobytes(), batch=3, precision=precision)
        finally:
            capi.lib().one_cuda_set_width_pairing(1)
        try:
            outs[on] = n(x)
            inter = {k: n.fetch(k, v.shape) for k, v in (("r0", r0), ("c2", c2))}
            p = n_trace_details(n)
            details[on] = p
            if precision == "tf32":
                assert_close(outs[on], ref, f"pairing={on} output")
                assert_close(inter["r0"], r0, f"pairing={on} r0")
                assert_close(inter["c2"], c2, f"pairing={on} c2")
        finally:
            n.close()
    assert "paired" in details[1]["Conv_1"] and "paired" in details[1]["Conv_2"]
    assert "paired" not in details[1]["Conv_0"] and "paired" not in details[1]["Conv_3"]
    assert not any("paired" in d for d in details[0].values())
    tol = 2e-3 if precision == "tf32" else 3e-2
    assert np.abs(outs[1] - outs[0]).max() <= tol * np.abs(ref).max()


def n_trace_details(n):
    """{operator name: detail string} from a tracing pass."""
    import tempfile, os
    with tempfile.TemporaryDirectory() as td:
        p = os.path.join(td, "t.csv")
        n.trace(p, runs=1)
        rows = [ln.split(",") for ln in open(p).read().strip().split("\n")[1:]]
    return {r[0]: r[13] for r in rows}
