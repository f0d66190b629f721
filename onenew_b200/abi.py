"""ctypes mirror of ``include/one_abi.h``.

The structures here have the same field order and widths as the C header, which in
turn pins the reference layout (common/nn_common.h:28-243, :312-379).  They let
Python code build the ``params / inputs / outputs`` arrays an operator library's
``eval`` expects, exactly as the reference host does in host/op.h:109-168 and
host/ops/conv.h:133-157.
"""
import ctypes as C

BUF_MAXNUM = 12
OPERAND_MAXNUM = 8
SHAPE_LEN = 8
NAME_LEN = 256
ONE_MAGIC_NUM = 0x6F6E65

# ELEM_TYPE_E
TYPE_FP32, TYPE_INT8, TYPE_INT32 = 1, 3, 6
# ACT_TYPE_E
NOT_ACT, RELU, RELU6, SILU, CLIP, HARDSILU, LEAKYRELU = range(7)


class BLOCK_INFO_S(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "x86_gemm_single_threads_tile_m", "x86_gemm_single_threads_tile_n", "x86_gemm_single_threads_tile_k",
        "x86_gemm_multi_threads_tile_m", "x86_gemm_multi_threads_tile_n", "x86_gemm_multi_threads_tile_k",
        "cuda_gemm_tile_m", "cuda_gemm_tile_n", "cuda_gemm_tile_k")]


class PUBLIC_BUF_INFO_S(C.Structure):
    _fields_ = [("public_buf_size", C.c_int64), ("public_buf_ptr", C.c_int64)]


class KV_CACHE_INFO_S(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "kv_cache_buf_size", "kv_cache_buf_ptr", "prompts_amount", "max_token_supported", "cur_token_index")]


class USEFUL_INFO_S(C.Structure):
    _fields_ = [("useful_info_magic_num", C.c_int32), ("block_info", BLOCK_INFO_S),
                ("public_buf_info", PUBLIC_BUF_INFO_S), ("kv_cache_info", KV_CACHE_INFO_S)]


class ONE_MODEL_DESC_S(C.Structure):
    _fields_ = [("one_model_magic_num", C.c_int32), ("version", C.c_int32),
                ("node_cnt", C.c_int32), ("node_cfg_offset", C.c_int32),
                ("init_cnt", C.c_int32), ("init_info_offset", C.c_int32),
                ("io_cfg_cnt", C.c_int32), ("io_cfg_offset", C.c_int32),
                ("useful_info", USEFUL_INFO_S)]


class BUFFER_INFO_S(C.Structure):
    _fields_ = [("addr", C.c_int64), ("elem_size", C.c_int32), ("buf_size", C.c_int32)]


class NODE_INFO_S(C.Structure):
    _fields_ = [("op_type", C.c_char * NAME_LEN), ("op_name", C.c_char * NAME_LEN)]


class OPERAND_S(C.Structure):
    _fields_ = [("operand_name", C.c_char * NAME_LEN), ("is_fixed_val", C.c_int32),
                ("not_need_buf", C.c_int32), ("p_data", C.c_int64),
                ("dim_num_of_shapes", C.c_int32), ("shapes", C.c_int32 * SHAPE_LEN),
                ("data_type", C.c_int32)]


class IO_CONFIG_S(C.Structure):
    _fields_ = [("op_type", C.c_char * NAME_LEN), ("op_name", C.c_char * NAME_LEN), ("operand", OPERAND_S)]


class BASE_CONFIG_S(C.Structure):
    _fields_ = [("op_type", C.c_char * NAME_LEN), ("op_name", C.c_char * NAME_LEN),
                ("in_operand_name", (C.c_char * NAME_LEN) * OPERAND_MAXNUM),
                ("out_operand_name", (C.c_char * NAME_LEN) * OPERAND_MAXNUM),
                ("in_operand_num", C.c_int32), ("out_operand_num", C.c_int32),
                ("producer", NODE_INFO_S * OPERAND_MAXNUM), ("consumer", NODE_INFO_S * OPERAND_MAXNUM),
                ("producer_num", C.c_int32), ("consumer_num", C.c_int32),
                ("fusion_op_type", C.c_int32),
                ("fusion_op_cnt_in_entire_net", C.c_int64), ("cur_op_cnt_in_fusion_op", C.c_int64)]


class CONV_CONFIG_S(C.Structure):
    _fields_ = [("op_base_cfg", BASE_CONFIG_S), ("has_bias", C.c_int32),
                ("dilations", C.c_int64 * 2), ("group", C.c_int64), ("kernel_shape", C.c_int64 * 2),
                ("pads", C.c_int64 * 4), ("strides", C.c_int64 * 4),
                ("act_type", C.c_int32), ("clip_min", C.c_float), ("clip_max", C.c_float),
                ("leaky_relu_alpha", C.c_float), ("hard_sigmoid_alpha", C.c_float), ("hard_sigmoid_beta", C.c_float),
                ("ifmap_quant2", C.c_int32), ("input_scale", C.c_float), ("output_scale", C.c_float),
                ("weight_aux", C.c_float * 4096)]


class GEMM_CONFIG_S(C.Structure):
    _fields_ = [("op_base_cfg", BASE_CONFIG_S), ("has_bias", C.c_int32),
                ("alpha", C.c_float), ("beta", C.c_float), ("transB", C.c_int64)]


class MATMUL_CONFIG_S(C.Structure):
    _fields_ = [("op_base_cfg", BASE_CONFIG_S)]


class SIMPLE_CONFIG_S(C.Structure):
    """Add / Relu / GlobalAveragePool / Gelu ...: a bare BASE_CONFIG_S."""
    _fields_ = [("op_base_cfg", BASE_CONFIG_S)]


class FLATTEN_CONFIG_S(C.Structure):
    _fields_ = [("op_base_cfg", BASE_CONFIG_S), ("axis", C.c_int64)]


class MAX_POOL_CONFIG_S(C.Structure):
    _fields_ = [("op_base_cfg", BASE_CONFIG_S), ("ceil_mode", C.c_int64), ("kernel_shape", C.c_int64 * 2),
                ("pads", C.c_int64 * 4), ("strides", C.c_int64 * 2)]


class AXIS_CONFIG_S(C.Structure):
    """Concat: BASE_CONFIG_S + axis."""
    _fields_ = [("op_base_cfg", BASE_CONFIG_S), ("axis", C.c_int64)]


class GATHER_CONFIG_S(C.Structure):
    _fields_ = [("op_base_cfg", BASE_CONFIG_S), ("axis", C.c_int64), ("indices", C.c_int64),
                ("indices_from_ifmap", C.c_int32)]


class LAYERNORMALIZATION_CONFIG_S(C.Structure):
    _fields_ = [("op_base_cfg", BASE_CONFIG_S), ("axes", C.c_int32 * 8), ("axes_num", C.c_int32), ("keepdims", C.c_int32)]


class RESHAPE_CONFIG_S(C.Structure):
    _fields_ = [("op_base_cfg", BASE_CONFIG_S), ("allowzero", C.c_int64), ("dst_shape", C.c_int64 * 8),
                ("dst_shape_num", C.c_int64)]


class SOFTMAX_CONFIG_S(C.Structure):
    _fields_ = [("op_base_cfg", BASE_CONFIG_S), ("dims", C.c_int64), ("axis", C.c_int64)]


class TRANSPOSE_CONFIG_S(C.Structure):
    _fields_ = [("op_base_cfg", BASE_CONFIG_S), ("perm", C.c_int64 * 8), ("perm_num", C.c_int64)]


_SIZES = {AXIS_CONFIG_S: 12848, GATHER_CONFIG_S: 12864, LAYERNORMALIZATION_CONFIG_S: 12880, RESHAPE_CONFIG_S: 12920,
          SOFTMAX_CONFIG_S: 12856, TRANSPOSE_CONFIG_S: 12912, BUFFER_INFO_S: 16, OPERAND_S: 312, BASE_CONFIG_S: 12840, CONV_CONFIG_S: 29376,
          GEMM_CONFIG_S: 12864, MATMUL_CONFIG_S: 12840, ONE_MODEL_DESC_S: 128, USEFUL_INFO_S: 96,
          IO_CONFIG_S: 824, MAX_POOL_CONFIG_S: 12840 + 72, FLATTEN_CONFIG_S: 12848}
for _t, _s in _SIZES.items():
    assert C.sizeof(_t) == _s, (_t.__name__, C.sizeof(_t), _s)
assert CONV_CONFIG_S.weight_aux.offset == 12988 and CONV_CONFIG_S.pads.offset == 12888

EVAL_FN = C.CFUNCTYPE(C.c_int, C.POINTER(BUFFER_INFO_S), C.POINTER(BUFFER_INFO_S), C.POINTER(BUFFER_INFO_S))


def make_operand(name, shape, data_type=TYPE_FP32, is_fixed=False):
    """OPERAND_S with shapes[] padded by 1s the way the converter writes them."""
    o = OPERAND_S()
    o.operand_name = name.encode()
    o.is_fixed_val = int(is_fixed)
    o.dim_num_of_shapes = len(shape)
    for i in range(SHAPE_LEN):
        o.shapes[i] = int(shape[i]) if i < len(shape) else 1
    o.data_type = data_type
    return o


def default_useful_info(public_buf_ptr=0, public_buf_size=0):
    """Header defaults the converter writes: x86 tiles 32/1024/8, cuda tiles 16/16/16
    (tools/onnx2one/onnx2one.cpp:1331-1350)."""
    u = USEFUL_INFO_S()
    b = u.block_info
    b.x86_gemm_single_threads_tile_m, b.x86_gemm_single_threads_tile_n, b.x86_gemm_single_threads_tile_k = 32, 1024, 8
    b.x86_gemm_multi_threads_tile_m, b.x86_gemm_multi_threads_tile_n, b.x86_gemm_multi_threads_tile_k = 32, 1024, 8
    b.cuda_gemm_tile_m = b.cuda_gemm_tile_n = b.cuda_gemm_tile_k = 16
    u.public_buf_info.public_buf_ptr = public_buf_ptr
    u.public_buf_info.public_buf_size = public_buf_size
    return u


class EvalArgs:
    """The three BUF_MAXNUM-slot arrays of one ``eval`` call; keeps referents alive."""

    def __init__(self):
        self.params = (BUFFER_INFO_S * BUF_MAXNUM)()
        self.inputs = (BUFFER_INFO_S * BUF_MAXNUM)()
        self.outputs = (BUFFER_INFO_S * BUF_MAXNUM)()
        self._keep = []

    def set_param(self, idx, struct):
        self._keep.append(struct)
        self.params[idx].addr = C.addressof(struct)

    def set_input(self, idx, addr):
        self.inputs[idx].addr = int(addr)

    def set_output(self, idx, addr):
        self.outputs[idx].addr = int(addr)


def conv_cfg(kernel, strides, pads, has_bias=True, act=NOT_ACT, group=1, clip=(0.0, 6.0), leaky=0.01,
             hs=(1.0 / 6.0, 0.5), int8_scale=None, weight_aux=None, name="conv"):
    """CONV_CONFIG_S as the converter + fusion pass fill it
    (tools/onnx2one/onnx2one.cpp:314-378, tools/optimize/op_fusion.hpp:47-192)."""
    c = CONV_CONFIG_S()
    c.op_base_cfg.op_type = b"Conv"
    c.op_base_cfg.op_name = name.encode()
    c.op_base_cfg.in_operand_num = 3 if has_bias else 2
    c.op_base_cfg.out_operand_num = 1
    c.has_bias = int(has_bias)
    c.dilations[0] = c.dilations[1] = 1
    c.group = group
    c.kernel_shape[0], c.kernel_shape[1] = kernel
    for i in range(4):
        c.pads[i] = pads[i]
    c.strides[0] = strides[0]
    c.strides[1] = strides[1]
    c.act_type = act
    c.clip_min, c.clip_max = clip
    c.leaky_relu_alpha = leaky
    c.hard_sigmoid_alpha, c.hard_sigmoid_beta = hs
    if int8_scale is not None:
        c.ifmap_quant2 = TYPE_INT8
        c.input_scale = int8_scale
        for i, v in enumerate(weight_aux):
            c.weight_aux[i] = v
    else:
        c.ifmap_quant2 = TYPE_FP32
    return c


def conv_eval_args(cfg, x_shape, w_shape, y_shape, x_addr, w_addr, b_addr, y_addr, useful, lut_addr=0):
    """Slot layout of a Conv call: params [0]=cfg [1]=x [2]=W [3]=bias [4]=y (y at [3] without
    bias), [11]=USEFUL_INFO_S; inputs [0]=x [1]=W [2]=bias [11]=SiLU table
    (host/op.h:114-133, host/ops/conv.h:65-68, :136-154, :190-192)."""
    a = EvalArgs()
    a.set_param(0, cfg)
    a.set_param(1, make_operand("x", x_shape))
    a.set_param(2, make_operand("w", w_shape, is_fixed=True))
    if cfg.has_bias:
        a.set_param(3, make_operand("b", (w_shape[0],), is_fixed=True))
        a.set_param(4, make_operand("y", y_shape))
    else:
        a.set_param(3, make_operand("y", y_shape))
    a.set_param(BUF_MAXNUM - 1, useful)
    a.set_input(0, x_addr)
    a.set_input(1, w_addr)
    if cfg.has_bias:
        a.set_input(2, b_addr)
    a.set_input(BUF_MAXNUM - 1, lut_addr)
    a.set_output(0, y_addr)
    return a


def gemm_eval_args(x_shape, w_shape, y_shape, x_addr, w_addr, b_addr, y_addr):
    """Gemm: params [0]=cfg [1]=A [2]=W [3]=bias [4]=Y (device/x86/Gemm/gemm.c:13-23)."""
    cfg = GEMM_CONFIG_S()
    cfg.op_base_cfg.op_type = b"Gemm"
    cfg.op_base_cfg.in_operand_num = 3
    cfg.op_base_cfg.out_operand_num = 1
    cfg.has_bias = 1
    cfg.alpha = cfg.beta = 1.0
    cfg.transB = 1
    a = EvalArgs()
    a.set_param(0, cfg)
    a.set_param(1, make_operand("a", x_shape))
    a.set_param(2, make_operand("w", w_shape, is_fixed=True))
    a.set_param(3, make_operand("b", (w_shape[0],), is_fixed=True))
    a.set_param(4, make_operand("y", y_shape))
    a.set_input(0, x_addr)
    a.set_input(1, w_addr)
    a.set_input(2, b_addr)
    a.set_output(0, y_addr)
    return a


def matmul_eval_args(a_shape, b_shape, y_shape, a_addr, b_addr, y_addr, b_is_init=True):
    """MatMul: params [0]=cfg [1]=A [2]=B [3]=Y (device/x86/MatMul/mat_mul.c:14-22)."""
    cfg = MATMUL_CONFIG_S()
    cfg.op_base_cfg.op_type = b"MatMul"
    cfg.op_base_cfg.in_operand_num = 2
    cfg.op_base_cfg.out_operand_num = 1
    a = EvalArgs()
    a.set_param(0, cfg)
    a.set_param(1, make_operand("a", a_shape))
    a.set_param(2, make_operand("b", b_shape, is_fixed=b_is_init))
    a.set_param(3, make_operand("y", y_shape))
    a.set_input(0, a_addr)
    a.set_input(1, b_addr)
    a.set_output(0, y_addr)
    return a
