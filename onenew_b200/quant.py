"""Post-training int8 quantisation of a ``.one`` model, the job of the reference's
``tools/optimize`` quantiser (model_quant.hpp) with the MSE calibrator (:437-623): the fp32 model is
run on the GPU over the calibration images, the statistics of every Conv input are taken on the
device where the activations live (``one_quant_abs_max`` / ``one_quant_abs_histogram``), the
thresholds are searched on the host in the reference's float order, and the image is rewritten the
way the reference leaves it (:6-29, :659-676): int8 weights / int32 bias at the start of the
fp32-sized initialiser payloads, ``ifmap_quant2 = INT8``, ``input_scale`` and ``weight_aux`` in
the Conv record.  No CPU fallback: calibration needs the CUDA library and a GPU."""
import ctypes as C

import numpy as np

from . import abi, capi
from . import net as onet
from .one_file import OneBuilder, OneModel


def quantize_weights(w, b=None):
    """Per-output-channel symmetric int8 weights (truncating), int32 bias, and max|w| per channel."""
    w = np.ascontiguousarray(w, np.float32)
    OC = w.shape[0]
    inner = w.size // OC
    w8 = np.empty(w.shape, np.int8)
    aux = np.empty(OC, np.float32)
    bb = None if b is None else np.ascontiguousarray(b, np.float32)
    b32 = None if b is None else np.empty(OC, np.int32)
    capi.check(capi.lib().one_quant_weights(C.c_void_p(w.ctypes.data), C.c_void_p(bb.ctypes.data if bb is not None else 0),
                                            OC, inner, C.c_void_p(w8.ctypes.data),
                                            C.c_void_p(b32.ctypes.data if b32 is not None else 0), C.c_void_p(aux.ctypes.data)))
    return w8, b32, aux


def mse_threshold(hist, elem_count, max_abs):
    hist = np.ascontiguousarray(hist, np.uint32)
    thr = C.c_float()
    capi.check(capi.lib().one_quant_mse_threshold(C.c_void_p(hist.ctypes.data), C.c_longlong(int(elem_count)),
                                                  C.c_float(float(max_abs)), C.byref(thr)))
    return np.float32(thr.value)


def _conv_inputs(model):
    """{conv name: name of its activation input}, in file order."""
    out = {}
    for t, cfg in model.nodes:
        if t == "Conv":
            ins, _ = OneModel.node_io(cfg)
            out[cfg.op_base_cfg.op_name.decode()] = ins[0]
    return out


def kl_threshold(hist, elem_count, max_abs):
    hist = np.ascontiguousarray(hist, np.uint32)
    thr = C.c_float()
    capi.check(capi.lib().one_quant_kl_threshold(C.c_void_p(hist.ctypes.data), C.c_longlong(int(elem_count)),
                                                 C.c_float(float(max_abs)), C.byref(thr)))
    return np.float32(thr.value)


PERCENT = np.float32(99.998 / 100)      # model_quant.hpp:98
AFFLUENCE = 10                          # model_quant.hpp:107


def percent_reserve(elem):
    """Values kept per image and operand: (int32)(elem * (1 - percent) * 10), float arithmetic (model_quant.hpp:157)."""
    return int(np.float32(np.float32(elem) * (np.float32(1) - PERCENT)) * np.float32(AFFLUENCE))


def percent_threshold(kept, elem, n_img):
    """Threshold of the percent method from the per-image largest values (model_quant.hpp:167-176): all kept
    values (zero padded to the reference's vector length) ordered by falling |v|, element
    (int)((1 - percent) * n_img * elem).  The value is signed, as in the reference."""
    total = int(np.float32(np.float32(n_img * elem) * (np.float32(1) - PERCENT)) * np.float32(AFFLUENCE))
    if percent_reserve(elem) == 0:
        raise ValueError(f"percent calibration keeps no value of a {elem}-element operand (it needs >= 5000 elements per image)")
    allv = np.zeros(max(total, sum(len(k) for k in kept)), np.float32)
    off = 0
    for k in kept:
        allv[off:off + len(k)] = k
        off += len(k)
    order = np.argsort(-np.abs(allv), kind="stable")
    idx = int(np.float32(np.float32(np.float32(1) - PERCENT) * np.float32(n_img)) * np.float32(elem))
    return np.float32(allv[order][idx])


def _largest_abs(L, torch, dev, n, dt, k, stream, device):
    """The k largest-|x| elements of a device tensor (ties at the cut in unspecified order), |x| descending:
    max and histogram on the device locate a bound below the k-th value, one more pass collects what lies
    above it, and only those few values are sorted (on the host)."""
    if k <= 0:
        return np.zeros(0, np.float32)
    mx = torch.zeros(1, dtype=torch.float32, device=device)
    hist = torch.zeros(2048, dtype=torch.int32, device=device)
    capi.check(L.one_quant_abs_max(C.c_void_p(dev), dt, C.c_longlong(n), C.c_void_p(mx.data_ptr()), stream))
    torch.cuda.synchronize()
    m = float(mx.item())
    thr, cap = 0.0, n
    if m > 0:
        capi.check(L.one_quant_abs_histogram(C.c_void_p(dev), dt, C.c_longlong(n), C.c_float(m), C.c_void_p(hist.data_ptr()), stream))
        torch.cuda.synchronize()
        h = hist.cpu().numpy().astype(np.int64)
        above = np.cumsum(h[::-1])[::-1]                 # elements in bins >= b
        ok = np.nonzero(above >= k)[0]
        if len(ok):
            b = max(int(ok[-1]) - 1, 0)                  # one bin of slack against rounding at the bin edge
            thr = b * m / 2048.0
            cap = int(above[b]) + 16 if b > 0 else n
    out = torch.empty(cap, dtype=torch.float32, device=device)
    cnt = torch.zeros(1, dtype=torch.int32, device=device)
    capi.check(L.one_quant_collect_abs_ge(C.c_void_p(dev), dt, C.c_longlong(n), C.c_float(thr), C.c_void_p(out.data_ptr()),
                                          C.c_uint(cap), C.c_void_p(cnt.data_ptr()), stream))
    torch.cuda.synchronize()
    got = int(cnt.item())
    if got > cap or got < k:
        raise capi.OneCudaError(-4, f"largest-|x| collection: {got} values for a bound expected to give {k}..{cap}")
    v = out[:got].cpu().numpy()
    return v[np.argsort(-np.abs(v), kind="stable")][:k]


def calibrate(image, calib_images, method="mse", device=0, precision="tf32"):
    """input_scale of every Conv of the fp32 model ``image`` (bytes) from the calibration images (array
    [n, C, H, W]) by the reference's ``mse``, ``kl`` or ``percent`` method (model_quant.hpp:437-623,
    :197-435, :83-185); the per-tensor statistics are taken on the device, where the activations are.
    mse / kl: two passes over the images (running max |x|, then the 2048-bin histogram against it);
    percent: one pass keeping each image's largest |x| values.  Returns {conv name: input_scale}."""
    import torch
    if method not in ("mse", "kl", "percent"):
        raise ValueError("method must be mse, kl or percent")
    model = OneModel(image)
    conv_in = _conv_inputs(model)
    operands = sorted(set(conv_in.values()))
    L = capi.lib()
    devname = f"cuda:{device}"
    net = onet.Net(image, device=device, batch=1, precision=precision, fuse=False, graph=False)
    try:
        have = set(net.operands())
        missing = [o for o in operands if o not in have]
        if missing:
            raise capi.OneCudaError(-3, f"operands {missing} are not materialised by the runtime")
        stream = C.c_void_p(net.stream)
        y = np.empty(net.outputs[0][1], np.float32)
        if method == "percent":
            kept = {o: [] for o in operands}
            elems = {}
            for img in calib_images:
                net.run_host(np.ascontiguousarray(img[None], np.float32), y)
                net.sync()
                for o in operands:
                    dev, n, dt, _ = net.operand_ptr(o)
                    elems[o] = n
                    kept[o].append(_largest_abs(L, torch, dev, n, dt, percent_reserve(n), stream, devname))
            thr_of = {o: percent_threshold(kept[o], elems[o], len(calib_images)) for o in operands}
        else:
            maxes = torch.zeros(len(operands), dtype=torch.float32, device=devname)
            hists = torch.zeros((len(operands), 2048), dtype=torch.int32, device=devname)
            torch.cuda.synchronize()
            counts = [0] * len(operands)
            for img in calib_images:                         # pass 1: max |x| per operand
                net.run_host(np.ascontiguousarray(img[None], np.float32), y)
                for i, o in enumerate(operands):
                    dev, n, dt, _ = net.operand_ptr(o)
                    capi.check(L.one_quant_abs_max(C.c_void_p(dev), dt, C.c_longlong(n), C.c_void_p(maxes[i:].data_ptr()), stream))
                net.sync()
            mx = maxes.cpu().numpy()
            for img in calib_images:                         # pass 2: histograms against those maxima
                net.run_host(np.ascontiguousarray(img[None], np.float32), y)
                for i, o in enumerate(operands):
                    dev, n, dt, _ = net.operand_ptr(o)
                    counts[i] += n
                    capi.check(L.one_quant_abs_histogram(C.c_void_p(dev), dt, C.c_longlong(n), C.c_float(float(mx[i])),
                                                         C.c_void_p(hists[i].data_ptr()), stream))
                net.sync()
            hs = hists.cpu().numpy().astype(np.uint32)
            search = mse_threshold if method == "mse" else kl_threshold
            thr_of = {o: search(hs[i], counts[i], mx[i]) for i, o in enumerate(operands)}
    finally:
        net.close()
    return {name: np.float32(thr_of[o] / np.float32(127)) for name, o in conv_in.items()}


def calibrate_mse(image, calib_images, device=0, precision="tf32"):
    return calibrate(image, calib_images, "mse", device, precision)


def quantize_model(image, scales):
    """The int8 image the reference's quantiser would write for the fp32 ``image`` (bytes) given
    {conv name: input_scale}: every listed Conv gets quantised weights / bias and its scales."""
    model = OneModel(image)
    b = OneBuilder()
    patched = {}
    for t, cfg in model.nodes:
        if t == "Conv" and cfg.op_base_cfg.op_name.decode() in scales:   # depthwise included, as in the reference (model_quant.hpp:40-68)
            ins, _ = OneModel.node_io(cfg)
            w = model.init_array(ins[1], np.float32)
            bias = model.init_array(ins[2], np.float32) if cfg.has_bias and len(ins) > 2 else None
            w8, b32, aux = quantize_weights(w, bias)
            raw = bytearray(w.nbytes)
            raw[:w8.size] = w8.tobytes()
            patched[ins[1]] = bytes(raw)
            if bias is not None:
                patched[ins[2]] = b32.tobytes()
            cfg.ifmap_quant2 = abi.TYPE_INT8
            cfg.input_scale = float(scales[cfg.op_base_cfg.op_name.decode()])
            for i, v in enumerate(aux):
                cfg.weight_aux[i] = float(v)
        cfg.op_base_cfg.producer_num = cfg.op_base_cfg.consumer_num = 0   # rebuilt when the image is written
        b.nodes.append(cfg)
    for name, (op, raw) in model.inits.items():
        b.inits.append((op, patched.get(name, raw)))
    b.ios = list(model.ios)
    return b.tobytes()
