"""The in-process multi-GPU runner (one_net_group): partition rule and argument checking on the CPU,
equivalence with a single-device Net and host-side failure reporting on one GPU."""
import ctypes as C

import numpy as np
import pytest

from onenew_b200 import capi, models, net as onet
from onenew_b200.sharding import shard_range


def _image():
    return models.build_resnet50(seed=3, num_classes=10, image=32, width=16, blocks=(2, 1, 1, 1)).tobytes()


def test_partition_rule_matches_the_sharding_helper():
    L = onet._lib()
    for batch, n in ((256, 1), (256, 2), (256, 4), (256, 8), (6, 3)):
        cuts = []
        for i in range(n):
            f, c = C.c_int(), C.c_int()
            assert L.one_net_group_partition(batch, n, i, C.byref(f), C.byref(c)) == 0
            cuts.append((f.value, f.value + c.value))
            assert cuts[-1] == shard_range(batch, n, i)
        assert cuts[0][0] == 0 and cuts[-1][1] == batch
    f, c = C.c_int(), C.c_int()
    assert L.one_net_group_partition(10, 4, 0, C.byref(f), C.byref(c)) == -1       # not divisible
    assert L.one_net_group_partition(8, 2, 2, C.byref(f), C.byref(c)) == -1        # no such shard
    assert L.one_net_group_partition(8, 0, 0, C.byref(f), C.byref(c)) == -1


def test_group_arguments_are_checked_before_anything_is_created():
    img = _image()
    with pytest.raises(capi.OneCudaError) as e:
        onet.NetGroup(img, devices=[0, 1, 2], batch=8)                             # 8 images do not divide by 3
    assert e.value.code == -1 and "divisible" in str(e.value)
    with pytest.raises(capi.OneCudaError) as e:
        onet.NetGroup(img, devices=[], batch=8)
    assert e.value.code == -1
    import torch
    if not torch.cuda.is_available():                                              # no GPU: loud failure, no fallback
        with pytest.raises(capi.OneCudaError) as e:
            onet.NetGroup(img, devices=[0], batch=2)
        assert e.value.code == -4


@pytest.mark.gpu
def test_group_of_one_equals_net_and_reports_host_side_failures():
    import torch
    img = _image()
    x = np.random.default_rng(4).uniform(0, 1, (4, 3, 32, 32)).astype(np.float32)
    n = onet.Net(img, batch=4)
    try:
        ref = n(x)
    finally:
        n.close()
    with pytest.raises(capi.OneCudaError) as e:
        onet.NetGroup(img, devices=[99], batch=4)
    assert e.value.code == -1 and "out of range" in str(e.value)
    with pytest.raises(capi.OneCudaError) as e:
        onet.NetGroup(img, devices=[0, 0], batch=4)
    assert e.value.code == -1 and "twice" in str(e.value)
    g = onet.NetGroup(img, devices=[0], batch=4)
    try:
        assert g.shards == [(0, 0, 4)]
        xin = torch.from_numpy(x).pin_memory()
        out = torch.zeros(ref.shape).pin_memory()
        for _ in range(3):
            g.submit_host(xin, out)
        g.sync()
        assert np.array_equal(out.numpy(), ref)
        # a shard whose host thread meets an error: sync returns it (nothing is injected on the device)
        before = capi.lib().one_cuda_launch_count()
        g.set_fault_hook(lambda device: -4)
        g.submit_host(xin, out)
        with pytest.raises(capi.OneCudaError) as e:
            g.sync()
        assert e.value.code == -4 and "device 0" in str(e.value)
        assert capi.lib().one_cuda_launch_count() == before                      # the failed shard launched nothing
        g.set_fault_hook(None)
        out.zero_()
        g.submit_host(xin, out)
        g.sync()                                                                   # the group is usable again
        assert np.array_equal(out.numpy(), ref)
    finally:
        g.close()


@pytest.mark.gpu
def test_group_over_every_visible_gpu_reassembles_the_batch():
    """With more than one GPU visible: the shards, run on different devices, reassemble to what one device
    computes for the whole batch (bit for bit: the replicas are identical and no contraction of this small
    model changes its summation order with the shard size)."""
    import torch
    ndev = torch.cuda.device_count()
    if ndev < 2:
        pytest.skip("one GPU visible")
    img = _image()
    x = np.random.default_rng(5).uniform(0, 1, (2 * ndev, 3, 32, 32)).astype(np.float32)
    capi.check(capi.lib().one_cuda_set_split_k(1))
    try:
        n = onet.Net(img, batch=2 * ndev)
        try:
            ref = n(x)
        finally:
            n.close()
        g = onet.NetGroup(img, devices=list(range(ndev)), batch=2 * ndev)
        try:
            assert [s[1:] for s in g.shards] == [(2 * i, 2) for i in range(ndev)]
            xin = torch.from_numpy(x).pin_memory()
            out = torch.zeros(ref.shape).pin_memory()
            g.submit_host(xin, out)
            g.sync()
            assert np.abs(out.numpy() - ref).max() <= 5e-3 * np.abs(ref).max()
        finally:
            g.close()
    finally:
        capi.lib().one_cuda_set_split_k(0)
