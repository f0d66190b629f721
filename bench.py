#!/usr/bin/env python
"""Benchmark of the Conv / Gemm / MatMul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload resnet50|vit|yolo|conv] [--batch B] [--precision tf32|bf16|f16]

Workload `resnet50` (default): synthetic ResNet-50 v1 (.one model written by
onenew_b200.models, seeded He-init weights, BN folded, conv+ReLU fused), uniform[0,1]
ImageNet-normalised 3x224x224 images, global batch 256 cut into N contiguous shards of 256/N images
(`--scaling strong`, the default: one process per GPU, each with its own slice of the seeded global
batch, no collective on the data path; `--scaling weak` gives every GPU `--batch` images instead).
A step is one inference pass over the global batch.
`value` is img/s with the inputs resident in HBM (median of --repeats timed regions of --steps steps
each); `e2e` is the same through Net.submit_host with pinned host buffers, H2D and D2H copies inside
the timed region.
Workload `vit`: synthetic ViT-Tiny/16 (patch 16, width 192, 12 blocks, 3 heads, MLP 768, 197 tokens;
truncated-normal(0.02) weights), uniform[0,1] images, same batch rule.
Workload `yolo`: the int8 YOLOv8s-shaped conv backbone at 3x640x640 (CSP widths 32-512, SiLU table),
calibrated (MSE, 8 seeded images) and quantised on the spot with onenew_b200.quant; pass --batch (e.g. 64).
Workload `conv`: one 3x3 64->64 conv + ReLU on 56x56 (the single-operator configuration) at
batch B, used for kernel profiling.

`--impl reference` times the reference's own x86 operators (compiled unmodified into
oracle/_ref) on the host cores over the same model, a bounded sample of images per step.
"""
import os

# The reference's operators are OpenMP code built for 8 threads.  The thread count and binding have to
# be in the environment before any OpenMP runtime is loaded (torchrun exports OMP_NUM_THREADS=1 to its
# children), so this comes before every other import.
os.environ["OMP_NUM_THREADS"] = "8"
os.environ["OMP_PROC_BIND"] = "close"

import argparse
import json
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GLOBAL_BATCH = 256
# DRAM traffic of the contraction kernel relative to its algorithmic bytes: dram__bytes_read.sum +
# dram__bytes_write.sum over size(x) + size(W) + size(b) + size(y), pooled over ncu captures of six single
# layers of the model (3 launches each) at batches whose tensors exceed the L2.  The ratio is below 1 because
# the tail of a layer's output is still in the 126 MB L2 when its kernel ends and is written back under a
# later kernel; no operand is read from DRAM more than once.  `roofline.traffic` is this ratio times the
# algorithmic bytes of an average launch.
TRAFFIC_OVER_ALGORITHMIC = {"resnet50": {"tf32": 0.86, "f16": 0.77}}
REF_SAMPLE_IMAGES = 8   # "x86 at batch 8" = 8 back-to-back single-image inferences


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        pk = {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"],
              "source": "measured"}
    else:
        pk = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    # Only a bf16 GEMM peak is measured.  The tensor pipe runs tf32 at half and int8 at twice the bf16 rate,
    # so each kind is divided by a peak of its own kind derived from the measured (sustained) bf16 figure.
    pk["tensor_tflops"] = {"bf16": pk["bf16_tflops_sustained"], "f16": pk["bf16_tflops_sustained"], "tf32": 0.5 * pk["bf16_tflops_sustained"],
                           "s8": 2.0 * pk["bf16_tflops_sustained"]}
    pk["tensor_peak_note"] = f"derived from {pk['source']} bf16 (sustained): tf32 = 1/2 x, int8 = 2 x"
    return pk


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


METRIC = {"resnet50": "resnet50_img_per_s", "vit": "vit_tiny_img_per_s", "yolo": "yolo_int8_backbone_img_per_s",
          "conv": "conv_img_per_s"}
CONV_SHAPE = [64, 64, 3, 1, 1, 56]   # C, OC, kernel, stride, pad, H=W  (the single-operator configuration)


def build_model(workload):
    from onenew_b200 import abi, models
    from onenew_b200.one_file import OneBuilder
    import numpy as np
    if workload == "resnet50":
        return models.build_resnet50().tobytes(), (3, 224, 224), models.RESNET50_FLOPS_PER_IMAGE
    if workload == "vit":
        return models.build_vit().tobytes(), (3, 224, 224), models.VIT_TINY_FLOPS_PER_IMAGE
    if workload == "yolo":
        # fp32 stack -> MSE calibration over 8 seeded images on the GPU -> the int8 image the reference's
        # quantiser would write (onenew_b200/quant.py)
        from onenew_b200 import quant
        fp32 = models.build_yolo_backbone(models.yolo_backbone_weights()).tobytes()
        scales = quant.calibrate_mse(fp32, models.yolo_input(8))
        flops, hw = 0.0, 640
        for ci, co, k, s_, p_ in models.YOLO_STACK:
            hw = (hw + 2 * p_ - k) // s_ + 1
            flops += 2.0 * co * hw * hw * ci * k * k
        return quant.quantize_model(fp32, scales), (3, 640, 640), flops
    c, oc, k, s, pd, hw = CONV_SHAPE
    ohw = (hw + 2 * pd - k) // s + 1
    rng = np.random.default_rng(2)
    b = OneBuilder()
    b.add_io("input", "input", (1, c, hw, hw))
    w = b.add_init("w", (rng.standard_normal((oc, c, k, k)) * 0.05).astype(np.float32))
    bias = b.add_init("b", (rng.standard_normal(oc) * 0.01).astype(np.float32))
    b.conv("Conv_0", "input", w, bias, "output", (k, k), (s, s), (pd, pd, pd, pd), act=abi.RELU)
    b.add_io("output", "output", (1, oc, ohw, ohw))
    return b.tobytes(), (c, hw, hw), 2.0 * oc * ohw * ohw * c * k * k


def make_inputs(workload, n, seed):
    import numpy as np
    from onenew_b200 import models
    if workload == "resnet50":
        return models.resnet50_input(n, seed=seed)
    if workload == "vit":
        return models.vit_input(n, seed=seed)
    if workload == "yolo":
        return models.yolo_input(n, seed=seed)
    c, _, _, _, _, hw = CONV_SHAPE
    return np.random.default_rng(seed).uniform(-1, 1, (n, c, hw, hw)).astype(np.float32)


def time_reference(image, workload, steps, warmup):
    """Times the reference's x86 path: `warmup` untimed and `steps` timed passes, a pass being
    REF_SAMPLE_IMAGES single-image inferences back to back (the reference runs N = 1 only).  Returns
    (img/s from the median pass, img/s from the fastest pass, seconds per pass list)."""
    from oracle.model_ref import RefNet
    net = RefNet(image)
    x = make_inputs(workload, REF_SAMPLE_IMAGES, 100)
    per_pass = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        for i in range(REF_SAMPLE_IMAGES):
            net.run(x[i:i + 1])
        if it >= warmup:
            per_pass.append(time.perf_counter() - t0)
    return REF_SAMPLE_IMAGES / statistics.median(per_pass), REF_SAMPLE_IMAGES / min(per_pass), per_pass


def ref_threads():
    return min(8, os.cpu_count() or 8)


# The result is ONE JSON line on stdout.  Libraries print there too (NCCL's version banner under torchrun), so
# the process's stdout is pointed at stderr for the run and the line goes to the original descriptor.
_RESULT_OUT = None


def claim_stdout():
    global _RESULT_OUT
    if _RESULT_OUT is None:
        sys.stdout.flush()
        _RESULT_OUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(obj):
    claim_stdout()
    _RESULT_OUT.write(json.dumps(obj) + "\n")
    _RESULT_OUT.flush()


def run_reference(args, rank):
    """The reference's x86 operators on the host cores (rank 0 only)."""
    if rank != 0:
        return
    import oracle
    image, _, flops = build_model(args.workload)
    if not oracle.have_reference():
        emit({"impl": "reference", "unavailable": "oracle/_ref not built: the reference tree was not present at build time"})
        return
    steps = max(args.steps, 10)          # at least 10 timed passes, 3 warm-ups: median and minimum are reported
    v, vmax, per_pass = time_reference(image, args.workload, steps, max(args.warmup, 3))
    dt = sum(per_pass)
    cores = ref_threads()
    sample = (f"{REF_SAMPLE_IMAGES} sequential single-image inferences per step (the reference runs N=1 only), {steps} steps after "
              f"{max(args.warmup, 3)} warm-ups; value = median step, OMP_NUM_THREADS=8 OMP_PROC_BIND=close")
    emit({
        "impl": "reference", "metric": METRIC[args.workload],
        "value": v, "unit": "img/s", "n_gpus": args.gpus, "steps": steps, "warmup": max(args.warmup, 3),
        "ms_per_step": statistics.median(per_pass) * 1e3, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "global_batch": GLOBAL_BATCH, "reference_batch": REF_SAMPLE_IMAGES,
                   "host_cpus": os.cpu_count()},
        "value_best_step": vmax, "timed_s": dt,
        "cpu_baseline": {"value": v, "value_best": vmax, "unit": "img/s", "cores": cores, "kind": "reference", "sample": sample},
        "e2e": {"value": v, "unit": "img/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gflops": v * flops / 1e9,
    })


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="resnet50", choices=["resnet50", "vit", "yolo", "conv"])
    ap.add_argument("--batch", type=int, default=GLOBAL_BATCH, help="the global batch (strong scaling), or images per GPU with --scaling weak")
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="strong (default): --batch images are cut into N contiguous shards; weak: every GPU runs --batch images per step")
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps each; the median one is reported")
    ap.add_argument("--no-split-k", action="store_true", help="never cut the K range of a small contraction into pieces")
    ap.add_argument("--no-launch-overlap", action="store_true", help="launch the contraction kernels without programmatic stream serialisation")
    ap.add_argument("--no-pairing", action="store_true", help="do not evaluate narrow multi-tap convolutions on pixel pairs")
    ap.add_argument("--no-cta-pairs", action="store_true", help="keep pairs of CTAs (256-row tiles on two SMs) out of the tile search")
    ap.add_argument("--no-half-tiles", action="store_true", help="keep tiles of two 128-row halves per CTA out of the tile search")
    ap.add_argument("--no-wide-epilogue", action="store_true", help="keep the twelve-epilogue-warp tiles out of the tile search")
    ap.add_argument("--epilogue-mode", type=int, default=15, help="tuning switch of the contraction epilogue (bit 0: shared tile, bit 1: two patches, bit 2: early accumulator release, bit 3: 16-bit residual added by the tensor core)")
    ap.add_argument("--per-layer", default=None, help="write the per-operator table (markdown) of this run to this path")
    ap.add_argument("--precision", default="auto", choices=["auto", "tf32", "bf16", "f16"],
                    help="auto (default): f16 -- fp16 storage, the mantissa of tf32, held to the same parity bar -- for resnet50, with "
                         "tf32 taking over if a value leaves the fp16 range; tf32 for the other workloads")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-autotune", action="store_true", help="keep the library's tile heuristic (default: per-operator tile search at preparation time)")
    ap.add_argument("--conv-shape", default=None, help="workload conv: C,OC,kernel,stride,pad,HW (default 64,64,3,1,1,56)")
    args = ap.parse_args()
    claim_stdout()
    if args.conv_shape:
        CONV_SHAPE[:] = [int(v) for v in args.conv_shape.split(",")]
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from onenew_b200 import net as onet

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # keep the library's own lines (version banner) off stdout: one JSON line there
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from onenew_b200.sharding import shard_range
    from onenew_b200 import capi
    if args.no_split_k:
        capi.check(capi.lib().one_cuda_set_split_k(1))
    if args.no_launch_overlap:
        capi.check(capi.lib().one_cuda_set_launch_overlap(0))
    if args.no_pairing:
        capi.check(capi.lib().one_cuda_set_width_pairing(0))
    capi.check(capi.lib().one_cuda_set_epilogue_mode(args.epilogue_mode))
    if args.no_cta_pairs:
        capi.check(capi.lib().one_cuda_set_cta_pairs(0))
    if args.no_half_tiles:
        capi.check(capi.lib().one_cuda_set_half_tiles(0))
    if args.no_wide_epilogue:
        capi.check(capi.lib().one_cuda_set_wide_epilogue(0))
    # strong scaling (default): the global batch is `--batch` and is cut into N contiguous shards; weak:
    # each rank processes `--batch` images per step and the global batch is N times that.
    global_batch = args.batch * world if args.scaling == "weak" else args.batch
    lo, hi = shard_range(global_batch, world, rank)
    shard = hi - lo

    image, in_shape, flops_per_image = build_model(args.workload)
    requested = args.precision
    if args.precision == "auto":
        args.precision = "f16" if args.workload == "resnet50" else "tf32"

    def make_net(precision):
        return onet.Net(image, device=local_rank, batch=shard, precision=precision, graph=not args.no_graph,
                        workspace_bytes=(2 << 30) if args.workload == "conv" else (8 << 30))
    net = make_net(args.precision)
    out_shape = net.outputs[0][1]
    # this rank's contiguous shard of the seeded global batch, in pinned host memory
    x_host = torch.from_numpy(make_inputs(args.workload, shard, 100 + lo)).pin_memory()
    y_host = torch.empty(out_shape, dtype=torch.float32).pin_memory()
    stream = torch.cuda.ExternalStream(net.stream, device=torch.device("cuda", local_rank))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing -------------------------------------------------------------
    # The first inference fills the device input once.  With fp16 storage it is also the range check: a value
    # beyond the format is reported (ONE_ERR_RANGE) and, under `auto`, every rank then runs tf32 instead.
    precision_note = None
    out_of_range = 0
    try:
        net.run_host(x_host, y_host)
    except capi.OneCudaError as e:
        if "ONE_ERR_RANGE" not in str(e):
            raise
        out_of_range = 1
    if world > 1:
        t = torch.tensor([out_of_range], device="cuda", dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out_of_range = int(t.item())
    if out_of_range:
        if requested != "auto":
            raise SystemExit("a value left the fp16 range: run this workload with --precision tf32")
        net.close()
        args.precision = "tf32"
        precision_note = "f16 reported a value outside the fp16 range on this input; measured in tf32"
        net = make_net("tf32")
        stream = torch.cuda.ExternalStream(net.stream, device=torch.device("cuda", local_rank))
        net.run_host(x_host, y_host)
    tuned = 0
    if not args.no_autotune:                # preparation-time tile search on the model's own operators (outside every timed region)
        net.sync()
        tuned = sum(1 for v in net.autotune(runs=5).values() if v[2])
    for _ in range(args.warmup):
        net.run()
    net.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # The timed region (exactly --steps steps between a barrier + synchronise on both sides, events on the
    # net's stream, max over ranks) is taken --repeats times; the median region is the reported one.
    region_ms = []
    with ClockSampler(local_rank) as clk:
        for _ in range(max(args.repeats, 1)):
            barrier()
            with torch.cuda.stream(stream):
                e0.record(stream)
                for _ in range(args.steps):
                    net.run()
                e1.record(stream)
            net.sync()
            barrier()
            region_ms.append(max_over_ranks(e0.elapsed_time(e1)))
    ms_step = statistics.median(region_ms) / args.steps
    value = global_batch / (ms_step * 1e-3)
    flops, algo_bytes, launches = net.work()

    # ---- end to end: pinned host input -> device -> host output, every step ------------------
    x_alt = x_host.clone().pin_memory()
    for i in range(3):
        net.submit_host(x_host if i % 2 == 0 else x_alt, y_host)
    net.sync()
    e2e_region_ms = []
    for _ in range(max(args.repeats, 1)):
        barrier()
        with torch.cuda.stream(stream):
            e0.record(stream)
        # every step: H2D of that step's input from pinned memory (on the copy stream, overlapping the
        # previous step's inference), the inference, and the D2H read of its logits
        for i in range(args.steps):
            net.submit_host(x_host if i % 2 == 0 else x_alt, y_host)
        with torch.cuda.stream(stream):
            e1.record(stream)
        net.sync()
        barrier()
        e2e_region_ms.append(max_over_ranks(e0.elapsed_time(e1)))
    e2e_ms = statistics.median(e2e_region_ms) / args.steps
    e2e_value = global_batch / (e2e_ms * 1e-3)
    h2d = int(x_host.numel() * 4) * world
    d2h = int(y_host.numel() * 4) * world

    # ---- per-operator pass (after the timed region): time spent in the contraction kernel ----
    roof = None
    cpu_base = None
    kind = "s8" if args.workload == "yolo" else args.precision
    if rank == 0:
        pk = measured_peaks()
        with tempfile.TemporaryDirectory() as td:
            path = os.path.join(td, "trace.csv")
            net.trace(path, runs=10, model_name=args.workload, hw_gops=pk["tensor_tflops"][kind] * 1e3)
            rows = read_trace(path)
        hot = [r for r in rows if r["type"] in ("Conv", "Gemm", "MatMul")]
        hot_us = sum(r["us"] for r in hot)
        hot_flops = sum(r["flops"] for r in hot)
        hot_bytes = sum(r["bytes"] for r in hot)
        all_us = sum(r["us"] for r in rows)
        ach_gbs = hot_bytes / (hot_us * 1e-6) / 1e9
        ach_tf = hot_flops / (hot_us * 1e-6) / 1e12
        # The step's arithmetic intensity against the ridge of ITS operand kind decides the binding roofline.
        tensor_peak = pk["tensor_tflops"][kind]
        ridge = tensor_peak * 1e12 / (pk["hbm_gbs"] * 1e9)
        ai = hot_flops / hot_bytes
        bound = "tensor" if ai >= ridge else "hbm"
        ratio = TRAFFIC_OVER_ALGORITHMIC.get(args.workload, {}).get(args.precision)
        roof = {
            "kernel": "igemm_kernel (all Conv/Gemm/MatMul launches of one step)", "bound": bound,
            "achieved": ach_tf if bound == "tensor" else ach_gbs,
            "peak": tensor_peak if bound == "tensor" else pk["hbm_gbs"],
            "unit": "TFLOP/s" if bound == "tensor" else "GB/s",
            "frac": (ach_tf / tensor_peak) if bound == "tensor" else (ach_gbs / pk["hbm_gbs"]),
            "traffic": (ratio * hot_bytes / max(len(hot), 1)) if ratio else None,
            "traffic_note": "ncu DRAM bytes over algorithmic bytes of single-layer captures, times the algorithmic bytes of an average launch" if ratio else None,
            "peak_source": pk["source"], "tensor_peak_kind": kind, "tensor_peak_note": pk["tensor_peak_note"],
            "launches_per_step": len(hot), "avg_launch_us": hot_us / max(len(hot), 1),
            "algorithmic_bytes_per_launch": hot_bytes / max(len(hot), 1), "algorithmic_bytes_per_step": hot_bytes, "algorithmic_flops_per_step": hot_flops,
            "arithmetic_intensity": ai, "ridge": ridge,
            "tensor_tflops": ach_tf, "tensor_frac": ach_tf / tensor_peak, "tensor_frac_of_bf16_peak": ach_tf / pk["bf16_tflops_sustained"],
            "hbm_gbs": ach_gbs, "hbm_frac": ach_gbs / pk["hbm_gbs"], "hot_share_of_step": hot_us / all_us,
        }
        if args.per_layer:
            write_per_layer(args.per_layer, rows, pk, kind, args, shard, ms_step)
        if not args.no_cpu_baseline and world == 1:
            cpu_base = cpu_baseline(args, image)

    # The same step in tf32 (fp32 storage), measured beside the fp16-storage headline: same model, inputs, tile
    # search and timing rules, three regions instead of --repeats.
    also = None
    if world == 1 and requested == "auto" and args.precision == "f16":
        net.close()
        net = make_net("tf32")
        stream2 = torch.cuda.ExternalStream(net.stream, device=torch.device("cuda", local_rank))
        net.run_host(x_host, y_host)
        if not args.no_autotune:
            net.sync()
            net.autotune(runs=5)
        for _ in range(args.warmup):
            net.run()
        net.sync()
        regions = []
        for _ in range(3):
            torch.cuda.synchronize()
            with torch.cuda.stream(stream2):
                e0.record(stream2)
                for _ in range(args.steps):
                    net.run()
                e1.record(stream2)
            net.sync()
            regions.append(e0.elapsed_time(e1) / args.steps)
        ms2 = statistics.median(regions)
        also = {"tf32": {"value": global_batch / (ms2 * 1e-3), "unit": "img/s", "ms_per_step": ms2, "ms_per_step_regions": regions}}

    if rank == 0:
        emit({
            "metric": METRIC[args.workload],
            "value": value, "unit": "img/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": kind, "data": "synthetic",
            "config": {"workload": args.workload, "global_batch": global_batch, "per_gpu_batch": shard,
                       "input": list(in_shape), "layout": "row-major token sequence on device" if args.workload == "vit" else "NHWC on device, NCHW fp32 at the io boundary",
                       # no explicit flush: every step streams its whole working set (weights + every activation once)
                       # through the 126 MB L2, so nothing of step i is still cached when step i+1 reads it
                       "l2": "inputs_larger_than_l2" if x_host.numel() * 4 > 126e6 else "step_working_set_larger_than_l2",
                       "step_working_set_bytes_per_gpu": algo_bytes,
                       "parallelism": f"batch sharded over {world} GPU(s), no collective",
                       "precision": args.precision, "precision_requested": requested, "precision_note": precision_note,
                       "cuda_graph": not args.no_graph, "tile_autotune": not args.no_autotune, "operators_retiled": tuned,
                       "split_k": not args.no_split_k, "launch_overlap": not args.no_launch_overlap,
                       "width_pairing": not args.no_pairing, "cta_pairs": not args.no_cta_pairs, "half_tiles": not args.no_half_tiles, "wide_epilogue": not args.no_wide_epilogue, "epilogue_mode": args.epilogue_mode},
            "repeats": {"regions": len(region_ms), "ms_per_step": [m / args.steps for m in region_ms],
                        "spread": (max(region_ms) - min(region_ms)) / statistics.median(region_ms)},
            "e2e": {"value": e2e_value, "unit": "img/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "ms_per_step_regions": [m / args.steps for m in e2e_region_ms]},
            "gpu_launches": int(launches) * args.steps * world,
            "tflops": value * flops_per_image / 1e12,
            "clocks": clk.summary(),
            "roofline": roof, "cpu_baseline": cpu_base, "other_precisions": also,
        })
    net.close()
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(args, image):
    """The reference's x86 path on this box's host cores, a bounded sample (rank 0, N=1 only): the same
    procedure as `--impl reference` (3 warm-up and 10 timed passes of 8 single-image inferences, median)."""
    import oracle
    if not oracle.have_reference():
        return None
    v, vmax, per_pass = time_reference(image, args.workload, 10, 3)
    return {"value": v, "value_best": vmax, "unit": "img/s", "cores": ref_threads(), "kind": "reference",
            "sample": f"10 passes of {REF_SAMPLE_IMAGES} sequential single-image inferences (median pass; 3 warm-ups, {sum(per_pass):.1f} s) of the "
                      f"same model on {os.cpu_count()} host CPUs, OMP_NUM_THREADS=8 OMP_PROC_BIND=close"}


def read_trace(path):
    """Rows of the runtime's tracing CSV (the reference's twelve columns + op_bytes + op_detail)."""
    import csv
    rows = []
    with open(path) as f:
        rd = csv.reader(f)
        next(rd)
        for r in rd:
            if not r:
                continue
            rows.append({"name": r[0], "type": r[1], "us": float(r[3]) - float(r[2]), "flops": float(r[4]) * 1e6,
                         "bytes": float(r[12]) if len(r) > 12 and r[12] else 0.0, "detail": r[13] if len(r) > 13 else ""})
    return rows


def write_per_layer(path, rows, pk, kind, args, shard, ms_step):
    """Per-operator table of one traced pass: time, rates, the binding roofline and the fraction of it."""
    tensor_peak = pk["tensor_tflops"][kind]
    ridge = tensor_peak * 1e12 / (pk["hbm_gbs"] * 1e9)
    total = sum(r["us"] for r in rows)
    out = [f"# Per-operator table: {args.workload}, {kind}, {shard} images on one B200", "",
           f"Command: `python bench.py --workload {args.workload} --batch {shard} --precision {args.precision} --per-layer <this file>`"
           + (" (`--conv-shape " + args.conv_shape + "`)" if args.conv_shape else ""),
           f"One eager pass timed operator by operator with CUDA events after the timed region (sum {total:.0f} us; the replayed graph "
           f"takes {ms_step * 1e3:.0f} us per step).  Peaks: HBM {pk['hbm_gbs']:.0f} GB/s ({pk['source']}), tensor {tensor_peak:.0f} TFLOP/s "
           f"({pk['tensor_peak_note']}); ridge {ridge:.0f} FLOP/B.  Bytes are algorithmic: x + W + b + y once each, plus the other operand of a folded Add.", "",
           "| operator | type | GEMM view / tile | us | share | TFLOP/s | GB/s | bound | frac of bound |", "|---|---|---|---|---|---|---|---|---|"]
    for r in rows:
        us = max(r["us"], 1e-3)
        tf, gb = r["flops"] / us / 1e6, r["bytes"] / us / 1e3
        if r["flops"] > 0 and r["bytes"] > 0:
            bound = "tensor" if r["flops"] / r["bytes"] >= ridge else "hbm"
        else:
            bound = "hbm"
        frac = tf / tensor_peak if bound == "tensor" else gb / pk["hbm_gbs"]
        out.append(f"| {r['name']} | {r['type']} | {r['detail']} | {us:.1f} | {100 * us / total:.1f}% | {tf:.1f} | {gb:.0f} | {bound} | {frac:.2f} |")
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        f.write("\n".join(out) + "\n")


if __name__ == "__main__":
    main()
