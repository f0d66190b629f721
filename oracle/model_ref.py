"""Model-level CPU checker: runs a ``.one`` graph operator by operator through the REFERENCE's
compiled x86 libraries (oracle/_ref), one image at a time.  TEST INFRASTRUCTURE ONLY.

This restates graph plumbing only -- reading the records, ordering the operators, wiring the
``params / inputs / outputs`` arrays as host/op.h:109-168 and host/ops/*.h do, allocating one
fp32 buffer per operand as host/net.h:419-452 does.  Every arithmetic result comes from the
reference's own code.  The reference handles a single image per inference
(host/ops/conv.h:43), so a batch is a loop.
"""
import ctypes as C

import numpy as np

import oracle
from onenew_b200 import abi
from onenew_b200.one_file import OneModel


def _shape_of(op):
    return tuple(op.shapes[i] for i in range(abi.SHAPE_LEN))


class RefNet:
    def __init__(self, one_bytes):
        self.m = OneModel(one_bytes)
        self.order = self._toposort()
        self.scratch = oracle._public_buf()
        self.useful = abi.default_useful_info(self.scratch.ctypes.data, self.scratch.nbytes)
        # the tables the reference HOST builds and hands to the operators: its own lines where they were
        # compiled (oracle/_ref/libquant_ref.so), the restatement (pinned to those lines by the tests) otherwise
        pinned = oracle.have_quant_reference()
        self.lut = oracle.ref_silu_lut() if pinned else oracle.silu_lut()
        self.gelu_lut = oracle.ref_gelu_lut() if pinned else oracle.gelu_lut()
        self.per_op_seconds = {}

    def _toposort(self):
        """Ready-list order over producer -> consumer edges (host/net.h:275-319 does the same
        with an O(n^2) scan)."""
        ready = {io.operand.operand_name.decode() for io in self.m.ios if io.op_name == b"input"}
        ready |= set(self.m.inits)
        pending = list(self.m.nodes)
        order = []
        while pending:
            for i, (t, cfg) in enumerate(pending):
                ins, outs = OneModel.node_io(cfg)
                if all(n in ready for n in ins):
                    order.append((t, cfg))
                    ready |= set(outs)
                    pending.pop(i)
                    break
            else:
                raise ValueError("graph has a cycle or a dangling input")
        return order

    # shape inference, one operator type at a time (host/ops/<op>.h shape_infer)
    def _infer(self, t, cfg, ins, shapes):
        x = shapes[ins[0]]
        if t == "Conv":
            w = self.m.inits[ins[1]][0]
            oh, ow = oracle.conv_out_hw(x[2], x[3], w.shapes[2], w.shapes[3], (cfg.strides[0], cfg.strides[1]),
                                        tuple(cfg.pads))
            return (1, w.shapes[0], oh, ow), 4
        if t == "MaxPool":
            oh = (x[2] + cfg.pads[0] + cfg.pads[2] - cfg.kernel_shape[0]) // cfg.strides[0] + 1
            ow = (x[3] + cfg.pads[1] + cfg.pads[3] - cfg.kernel_shape[1]) // cfg.strides[1] + 1
            return (x[0], x[1], oh, ow), 4
        if t in ("Relu", "Gelu", "Softmax", "LayerNormalization"):
            return x, len(x)
        if t in ("Add", "Sub", "Mul", "Div"):          # numpy broadcasting (device/x86/Add/add.c:52-67)
            y = shapes[ins[1]]
            o = np.broadcast_shapes(tuple(x), tuple(y))
            return tuple(o), len(o)
        if t == "Transpose":                           # host/ops/transpose.h:32-48
            return tuple(x[cfg.perm[i]] for i in range(cfg.perm_num)), cfg.perm_num
        if t == "Reshape":                             # host/ops/reshape.h:30-68
            dst = [cfg.dst_shape[i] for i in range(cfg.dst_shape_num)]
            known = int(np.prod([d for d in dst if d != -1]))
            dst = [int(np.prod(x)) // known if d == -1 else d for d in dst]
            return tuple(dst), len(dst)
        if t == "Concat":                              # host/ops/concat.h:31-70
            ax = cfg.axis if cfg.axis >= 0 else len(shapes[ins[-1]]) + cfg.axis
            o = list(shapes[ins[-1]])
            o[ax] = sum(shapes[n][ax] for n in ins)
            return tuple(o), len(o)
        if t == "Gather":                              # host/ops/gather.h:63-77 (fixed index)
            o = list(x)
            del o[cfg.axis]
            return tuple(o), len(o)
        if t == "GlobalAveragePool":
            return (x[0], x[1], 1, 1), 4
        if t == "Flatten":
            ax = cfg.axis
            return tuple(x[:ax]) + (int(np.prod(x[ax:])),), ax + 1
        if t == "Gemm":
            n = self.m.inits[ins[2]][0].shapes[0]     # N comes from the bias length (host/ops/gemm.h:39)
            return tuple(x[:-1]) + (n,), len(x)
        if t == "MatMul":
            bshape = shapes[ins[1]] if ins[1] in shapes else None
            if bshape is None:
                op = self.m.inits[ins[1]][0]
                bshape = tuple(op.shapes[i] for i in range(op.dim_num_of_shapes))
            return tuple(x[:-1]) + (bshape[-1],), len(x)
        raise NotImplementedError(t)

    def run(self, image, collect=None, timing=False):
        """One image (leading dim 1) -> dict of output arrays.  ``collect``: operand names whose
        values to keep (``"*"`` keeps every operand)."""
        import time
        bufs, shapes = {}, {}
        inp = self.m.inputs()[0]
        name = inp.operand_name.decode()
        shapes[name] = tuple(inp.shapes[i] for i in range(inp.dim_num_of_shapes))
        bufs[name] = oracle._aligned(shapes[name], np.float32, image.reshape(shapes[name]))
        keep = {}
        for n, (op, raw) in self.m.inits.items():      # shapes of the initialisers, for broadcasting operators
            shapes[n] = tuple(op.shapes[i] for i in range(max(op.dim_num_of_shapes, 1)))
        for t, cfg in self.order:
            ins, outs = OneModel.node_io(cfg)
            oshape, ndim = self._infer(t, cfg, ins, shapes)
            shapes[outs[0]] = tuple(oshape)
            if t in ("Flatten", "Reshape"):    # zero copy (host/ops/flatten.h:33, reshape.h:33, host/op.h:149-155)
                bufs[outs[0]] = bufs[ins[0]].reshape(oshape)
                if collect == "*" or (collect and outs[0] in collect):
                    keep[outs[0]] = bufs[outs[0]].copy()
                continue
            y = oracle._aligned(oshape)
            a = abi.EvalArgs()
            a.set_param(0, cfg)
            hold = []
            # operand i of the record: descriptor at params[1 + i], pointer at inputs[i], whether it is
            # an activation or an initialiser (host/op.h:109-146, host/ops/conv.h:136-154,
            # gemm.h:108-126, mat_mul.h:109-121, mul.h:130-156)
            for i, n in enumerate(ins):
                if n in self.m.inits:
                    op, raw = self.m.inits[n]
                    arr = oracle._aligned((max(len(raw) // 4, 1),), np.float32)
                    arr.view(np.uint8)[:len(raw)] = np.frombuffer(raw, np.uint8)
                    hold.append(arr)
                    a.set_param(1 + i, op)
                    a.set_input(i, arr.ctypes.data)
                else:
                    a.set_param(1 + i, abi.make_operand(n, shapes[n]))
                    a.set_input(i, bufs[n].ctypes.data)
            a.set_param(1 + len(ins), abi.make_operand(outs[0], oshape))
            a.set_output(0, y.ctypes.data)
            if t == "Conv":
                a.set_input(abi.BUF_MAXNUM - 1, self.lut.ctypes.data)
            if t == "Gelu":                    # host/ops/gelu.h:80-100
                a.set_input(abi.BUF_MAXNUM - 1, self.gelu_lut.ctypes.data)
            if t in ("Conv", "MaxPool"):       # scratch descriptor (host/ops/conv.h:65-68, maxpool.h)
                a.set_param(abi.BUF_MAXNUM - 1, self.useful)
            t0 = time.perf_counter()
            oracle.ref_eval(t)(a.params, a.inputs, a.outputs)
            if timing:
                self.per_op_seconds[t] = self.per_op_seconds.get(t, 0.0) + time.perf_counter() - t0
            bufs[outs[0]] = y
            if collect == "*" or (collect and outs[0] in collect):
                keep[outs[0]] = y.copy()
        for o in self.m.outputs():
            n = o.operand_name.decode()
            keep[n] = np.array(bufs[n])
        return keep

    def run_batch(self, images, collect=None):
        outs = [self.run(images[i:i + 1], collect) for i in range(len(images))]
        return {k: np.concatenate([o[k].reshape((1,) + o[k].shape[1:]) if o[k].shape[0] == 1 else o[k][None] for o in outs])
                for k in outs[0]}
