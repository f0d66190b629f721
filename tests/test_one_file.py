"""`.one` writer / reader round trip and the runtime's planning pass (CPU only)."""
import ctypes as C

import numpy as np

from onenew_b200 import abi, models, net as onet
from onenew_b200.one_file import OneBuilder, OneModel


def _small():
    return models.build_resnet50(seed=3, num_classes=10, image=32, width=16, blocks=(2, 1, 1, 1))


def test_layout_follows_the_converter():
    b = _small()
    data = b.tobytes()
    m = OneModel(data)
    d = m.desc
    assert d.one_model_magic_num == 0x6F6E65
    assert d.node_cfg_offset == 128 and d.node_cfg_offset % 64 == 0            # header padded to 64 bytes
    assert d.init_info_offset % 64 == 0 and d.io_cfg_offset % 64 == 0
    assert d.node_cnt == len(b.nodes) and d.init_cnt == len(b.inits) and d.io_cfg_cnt == 2
    assert d.useful_info.public_buf_info.public_buf_size == 512 * 1024 * 1024   # converter default
    assert d.useful_info.block_info.x86_gemm_multi_threads_tile_n == 1024
    assert len(data) == d.io_cfg_offset + 2 * ((C.sizeof(abi.IO_CONFIG_S) + 63) & ~63)


def test_round_trip_preserves_records():
    b = _small()
    m = OneModel(b.tobytes())
    t, cfg = m.nodes[0]
    assert t == "Conv" and cfg.act_type == abi.RELU and cfg.has_bias == 1
    assert tuple(cfg.kernel_shape) == (7, 7) and tuple(cfg.pads) == (3, 3, 3, 3) and cfg.strides[0] == 2
    ins, outs = OneModel.node_io(cfg)
    assert ins == ["input", "Conv_0.weight", "Conv_0.bias"] and outs == ["Conv_0_out"]
    w = m.init_array("Conv_0.weight")
    assert w.shape == (16, 3, 7, 7) and w.dtype == np.float32
    assert np.array_equal(w.ravel(), np.frombuffer(b.inits[0][1], np.float32))
    # producer / consumer lists as the converter fills them
    assert cfg.op_base_cfg.consumer_num == 1 and cfg.op_base_cfg.consumer[0].op_type == b"MaxPool"
    assert [o.operand_name for o in m.inputs()] == [b"input"] and [o.operand_name for o in m.outputs()] == [b"output"]


def test_bad_magic_rejected():
    data = bytearray(_small().tobytes())
    data[0] ^= 0xFF
    try:
        OneModel(bytes(data))
        assert False
    except ValueError:
        pass
    try:
        onet.describe(bytes(data))
        assert False
    except Exception as e:
        assert "magic" in str(e)


def test_plan_batch_rule_layouts_and_residual_fusion():
    image = _small().tobytes()
    plain = onet.describe(image, batch=4, fuse=False)
    fused = onet.describe(image, batch=4, fuse=True)
    # every activation gets the requested batch; convs produce NHWC; the classifier output is row major
    assert all(",".join(l.split("shape=")[1].split(",")[:1]) == "4" for l in fused if l.startswith("RUN"))
    assert "layout=NHWC" in fused[0] and fused[-1].startswith("RUN Gemm") and "layout=PLAIN dtype=f32" in fused[-1]
    n_add = sum(l.startswith("RUN Add") for l in plain)
    assert n_add == 5 and sum(l.startswith("RUN Relu") for l in plain) == 5
    assert not any(l.startswith(("RUN Add", "RUN Relu")) for l in fused)
    assert sum("residual=" in l and "relu=1" in l for l in fused) == n_add
    assert len(fused) == len(plain) - 2 * n_add
    # a fused conv runs after the operand it adds
    produced = {"input"}
    for l in fused:
        if l.startswith("RUN"):
            ins = l.split(" in=")[1].split(" ")[0].split(",")
            for i in ins:
                assert i in produced or "." in i, (i, l)          # "x.weight" style names are initialisers
            if "residual=" in l:
                assert l.split("residual=")[1].split(" ")[0] in produced
            produced.add(l.split(" out=")[1].split(" ")[0])
    # bf16 mode keeps activations in bf16
    assert "dtype=bf16" in onet.describe(image, batch=2, precision="bf16")[0]
    assert "dtype=f16" in onet.describe(image, batch=2, precision="f16")[0]
