"""Reader and writer of the ``.one`` model image.

Layout (tools/onnx2one/onnx2one.cpp:1294-1355): a 64-byte aligned ``ONE_MODEL_DESC_S`` header,
then the operator records (one ``*_CONFIG_S`` each, padded to 64 bytes), then the initialiser
records (``OPERAND_S`` + raw data, padded to 64 bytes; onnx2one.cpp:999-1104), then the io
records (``IO_CONFIG_S``, padded).  Offsets of the three sections are in the header.  The readers
this mirrors are host/net.h:138-221.

``OneBuilder`` emits what the converter followed by the fusion pass would: a Conv that was fused
with its activation carries ``act_type`` and three inputs (tools/optimize/op_fusion.hpp:47-192).
Nothing in this container can run the reference's converter (no protobuf), so synthetic models
are written directly in this format.
"""
import ctypes as C

import numpy as np

from . import abi


def _align(n):
    """align_buf_size, common/utils_c.h:4-7."""
    return (n + 63) & ~63


# cfg struct per operator type (what the reference registers with OP_REGISTER_GLOBAL)
CFG_TYPES = {
    "Conv": abi.CONV_CONFIG_S, "Gemm": abi.GEMM_CONFIG_S, "MatMul": abi.MATMUL_CONFIG_S,
    "MaxPool": abi.MAX_POOL_CONFIG_S, "Add": abi.SIMPLE_CONFIG_S, "Relu": abi.SIMPLE_CONFIG_S,
    "GlobalAveragePool": abi.SIMPLE_CONFIG_S, "Flatten": abi.FLATTEN_CONFIG_S,
    "Gelu": abi.SIMPLE_CONFIG_S, "Mul": abi.SIMPLE_CONFIG_S, "Div": abi.SIMPLE_CONFIG_S, "Sub": abi.SIMPLE_CONFIG_S,
    "Concat": abi.AXIS_CONFIG_S, "Gather": abi.GATHER_CONFIG_S, "LayerNormalization": abi.LAYERNORMALIZATION_CONFIG_S,
    "Reshape": abi.RESHAPE_CONFIG_S, "Softmax": abi.SOFTMAX_CONFIG_S, "Transpose": abi.TRANSPOSE_CONFIG_S,
}
_DTYPE_OF = {abi.TYPE_FP32: np.float32, abi.TYPE_INT8: np.int8, abi.TYPE_INT32: np.int32, 7: np.int64}


def register_cfg(op_type, struct):
    CFG_TYPES[op_type] = struct


class OneBuilder:
    """Accumulates operators, initialisers and io records and serialises them."""

    def __init__(self):
        self.nodes = []      # ctypes cfg structs
        self.inits = []      # (OPERAND_S, bytes)
        self.ios = []        # IO_CONFIG_S

    # -- records -------------------------------------------------------------------------
    def add_init(self, name, array, data_type=abi.TYPE_FP32, raw=None):
        """Initialiser record.  ``raw`` overrides the payload bytes (used for a quantised Conv,
        whose int8 weights / int32 bias sit at the start of the fp32-sized payload,
        tools/optimize/model_quant.hpp:6-29)."""
        array = np.ascontiguousarray(array)
        op = abi.make_operand(name, array.shape if array.ndim else (1,), data_type, is_fixed=True)
        self.inits.append((op, raw if raw is not None else array.tobytes()))
        return name

    def add_io(self, kind, name, shape):
        io = abi.IO_CONFIG_S()
        io.op_type = b"io"
        io.op_name = kind.encode()          # "input" | "output"
        io.operand = abi.make_operand(name, shape)
        self.ios.append(io)

    def _base(self, cfg, op_type, name, ins, outs):
        b = cfg.op_base_cfg
        b.op_type = op_type.encode()
        b.op_name = name.encode()
        for i, n in enumerate(ins):
            b.in_operand_name[i].value = n.encode()
        for i, n in enumerate(outs):
            b.out_operand_name[i].value = n.encode()
        b.in_operand_num = len(ins)
        b.out_operand_num = len(outs)
        self.nodes.append(cfg)
        return outs[0]

    def conv(self, name, x, w_name, b_name, y, kernel, strides, pads, act=abi.NOT_ACT, int8_scale=None,
             weight_aux=None, **kw):
        cfg = abi.conv_cfg(kernel, strides, pads, has_bias=b_name is not None, act=act, int8_scale=int8_scale,
                           weight_aux=weight_aux, name=name, **kw)
        ins = [x, w_name] + ([b_name] if b_name is not None else [])
        return self._base(cfg, "Conv", name, ins, [y])

    def gemm(self, name, x, w_name, b_name, y):
        cfg = abi.GEMM_CONFIG_S()
        cfg.has_bias = 1
        cfg.alpha = cfg.beta = 1.0
        cfg.transB = 1
        return self._base(cfg, "Gemm", name, [x, w_name, b_name], [y])

    def matmul(self, name, a, b, y):
        return self._base(abi.MATMUL_CONFIG_S(), "MatMul", name, [a, b], [y])

    def maxpool(self, name, x, y, kernel, strides, pads):
        cfg = abi.MAX_POOL_CONFIG_S()
        cfg.kernel_shape[0], cfg.kernel_shape[1] = kernel
        cfg.strides[0], cfg.strides[1] = strides
        for i in range(4):
            cfg.pads[i] = pads[i]
        return self._base(cfg, "MaxPool", name, [x], [y])

    def simple(self, op_type, name, ins, y):
        return self._base(CFG_TYPES[op_type](), op_type, name, ins, [y])

    def flatten(self, name, x, y, axis=1):
        cfg = abi.FLATTEN_CONFIG_S()
        cfg.axis = axis
        return self._base(cfg, "Flatten", name, [x], [y])

    def layernorm(self, name, x, w_name, b_name, y):
        cfg = abi.LAYERNORMALIZATION_CONFIG_S()
        cfg.axes[0], cfg.axes_num, cfg.keepdims = -1, 1, 1
        return self._base(cfg, "LayerNormalization", name, [x, w_name, b_name], [y])

    def softmax(self, name, x, y, axis=-1):
        cfg = abi.SOFTMAX_CONFIG_S()
        cfg.axis = axis
        return self._base(cfg, "Softmax", name, [x], [y])

    def transpose(self, name, x, y, perm):
        cfg = abi.TRANSPOSE_CONFIG_S()
        for i, p in enumerate(perm):
            cfg.perm[i] = p
        cfg.perm_num = len(perm)
        return self._base(cfg, "Transpose", name, [x], [y])

    def reshape(self, name, x, y, shape):
        cfg = abi.RESHAPE_CONFIG_S()
        for i, d in enumerate(shape):
            cfg.dst_shape[i] = d
        cfg.dst_shape_num = len(shape)
        return self._base(cfg, "Reshape", name, [x], [y])

    def concat(self, name, ins, y, axis):
        cfg = abi.AXIS_CONFIG_S()
        cfg.axis = axis
        return self._base(cfg, "Concat", name, list(ins), [y])

    def gather(self, name, x, y, axis, index):
        """Gather with a fixed index (the form the converter emits for ``x[:, i]``)."""
        cfg = abi.GATHER_CONFIG_S()
        cfg.axis, cfg.indices, cfg.indices_from_ifmap = axis, index, 0
        return self._base(cfg, "Gather", name, [x], [y])

    def node(self, op_type, cfg, name, ins, outs):
        """Generic record for operator types registered with ``register_cfg``."""
        return self._base(cfg, op_type, name, ins, outs)

    # -- serialise -----------------------------------------------------------------------
    def _fill_producer_consumer(self):
        """tools/onnx2one/onnx2one.cpp:1117-1227: who makes each input, who reads each output."""
        prod = {}
        for cfg in self.nodes:
            b = cfg.op_base_cfg
            for i in range(b.out_operand_num):
                prod[b.out_operand_name[i].value] = b
        for cfg in self.nodes:
            b = cfg.op_base_cfg
            for i in range(b.in_operand_num):
                p = prod.get(b.in_operand_name[i].value)
                if p is not None and b.producer_num < abi.OPERAND_MAXNUM and p.consumer_num < abi.OPERAND_MAXNUM:
                    b.producer[b.producer_num].op_type = p.op_type
                    b.producer[b.producer_num].op_name = p.op_name
                    b.producer_num += 1
                    p.consumer[p.consumer_num].op_type = b.op_type
                    p.consumer[p.consumer_num].op_name = b.op_name
                    p.consumer_num += 1

    def tobytes(self):
        self._fill_producer_consumer()
        head = _align(C.sizeof(abi.ONE_MODEL_DESC_S))
        cfg_bytes = sum(_align(C.sizeof(c)) for c in self.nodes)
        init_bytes = sum(_align(C.sizeof(abi.OPERAND_S) + len(raw)) for _, raw in self.inits)
        io_bytes = len(self.ios) * _align(C.sizeof(abi.IO_CONFIG_S))
        buf = bytearray(head + cfg_bytes + init_bytes + io_bytes)
        d = abi.ONE_MODEL_DESC_S()
        d.one_model_magic_num = abi.ONE_MAGIC_NUM
        d.version = 1
        d.node_cnt, d.node_cfg_offset = len(self.nodes), head
        d.init_cnt, d.init_info_offset = len(self.inits), head + cfg_bytes
        d.io_cfg_cnt, d.io_cfg_offset = len(self.ios), head + cfg_bytes + init_bytes
        d.useful_info = abi.default_useful_info(0, 512 * 1024 * 1024)
        buf[:C.sizeof(d)] = bytes(d)
        off = head
        for c in self.nodes:
            buf[off:off + C.sizeof(c)] = bytes(c)
            off += _align(C.sizeof(c))
        for op, raw in self.inits:
            buf[off:off + C.sizeof(op)] = bytes(op)
            buf[off + C.sizeof(op):off + C.sizeof(op) + len(raw)] = raw
            off += _align(C.sizeof(op) + len(raw))
        for io in self.ios:
            buf[off:off + C.sizeof(io)] = bytes(io)
            off += _align(C.sizeof(io))
        assert off == len(buf) < 2 ** 31, "a .one image is addressed with int32 (host/net.h:104)"
        return bytes(buf)

    def save(self, path):
        with open(path, "wb") as f:
            f.write(self.tobytes())


class OneModel:
    """Parsed view of a ``.one`` image (host/net.h:101-221)."""

    def __init__(self, data):
        self.data = bytes(data)
        d = abi.ONE_MODEL_DESC_S.from_buffer_copy(self.data[:C.sizeof(abi.ONE_MODEL_DESC_S)])
        if d.one_model_magic_num != abi.ONE_MAGIC_NUM:
            raise ValueError(f"not a .one image: magic {d.one_model_magic_num:#x}")
        self.desc = d
        self.nodes = []     # (op_type, cfg struct)
        off = d.node_cfg_offset
        for _ in range(d.node_cnt):
            op_type = self.data[off:off + 256].split(b"\0", 1)[0].decode()
            if op_type not in CFG_TYPES:
                raise ValueError(f"operator type {op_type!r} has no registered config struct")
            st = CFG_TYPES[op_type]
            self.nodes.append((op_type, st.from_buffer_copy(self.data[off:off + C.sizeof(st)])))
            off += _align(C.sizeof(st))
        self.inits = {}     # name -> (OPERAND_S, payload bytes)
        off = d.init_info_offset
        for _ in range(d.init_cnt):
            op = abi.OPERAND_S.from_buffer_copy(self.data[off:off + C.sizeof(abi.OPERAND_S)])
            n = int(np.prod(list(op.shapes))) * np.dtype(_DTYPE_OF.get(op.data_type, np.float32)).itemsize
            self.inits[op.operand_name.decode()] = (op, self.data[off + C.sizeof(op):off + C.sizeof(op) + n])
            off += _align(C.sizeof(op) + n)
        self.ios = []
        off = d.io_cfg_offset
        for _ in range(d.io_cfg_cnt):
            self.ios.append(abi.IO_CONFIG_S.from_buffer_copy(self.data[off:off + C.sizeof(abi.IO_CONFIG_S)]))
            off += _align(C.sizeof(abi.IO_CONFIG_S))

    @classmethod
    def load(cls, path):
        with open(path, "rb") as f:
            return cls(f.read())

    def init_array(self, name, dtype=None):
        op, raw = self.inits[name]
        dt = dtype or _DTYPE_OF.get(op.data_type, np.float32)
        shape = [op.shapes[i] for i in range(max(op.dim_num_of_shapes, 1))]
        return np.frombuffer(raw, dt, count=int(np.prod(shape))).reshape(shape)

    def inputs(self):
        return [io.operand for io in self.ios if io.op_name == b"input"]

    def outputs(self):
        return [io.operand for io in self.ios if io.op_name == b"output"]

    @staticmethod
    def node_io(cfg):
        b = cfg.op_base_cfg
        ins = [b.in_operand_name[i].value.decode() for i in range(b.in_operand_num)]
        outs = [b.out_operand_name[i].value.decode() for i in range(b.out_operand_num)]
        return ins, outs
