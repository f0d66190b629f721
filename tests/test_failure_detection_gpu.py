"""Failure detection without a GPU fault: a device-side wait that runs out is reported through the
status word as ONE_ERR_TIMEOUT, the kernel returns normally and the context keeps working."""
import numpy as np
import pytest

from onenew_b200 import abi, capi

pytestmark = pytest.mark.gpu


def test_bounded_wait_reports_timeout_and_context_survives(oracle_mod):
    ctx = capi.Context(0, 1 << 24)
    try:
        ctx.status()                                             # clean to begin with
        capi.check(capi.lib().one_cuda_selftest_wait_timeout(ctx.handle, 1 << 22))   # ~2 ms of clocks
        with pytest.raises(capi.OneCudaError) as e:
            ctx.status()
        assert e.value.code == -6 and "wait ran out" in str(e.value)
        ctx.status()                                             # the word was cleared
        # the device is still healthy: a normal operator call works and is correct
        from onenew_b200 import ops
        rng = np.random.default_rng(3)
        x = rng.uniform(-1, 1, (1, 32, 8, 8)).astype(np.float32)
        w = (rng.standard_normal((32, 32, 3, 3)) * 0.05).astype(np.float32)
        b = (rng.standard_normal(32) * 0.01).astype(np.float32)
        y = ops.conv(x, w, b, (1, 1), (1, 1, 1, 1), abi.RELU).cpu().numpy()
        ref = oracle_mod.conv_f32(x, w, b, (1, 1), (1, 1, 1, 1), abi.RELU)
        assert np.abs(y - ref).max() / np.abs(ref).max() < 1e-2
    finally:
        ctx.close()


def test_host_side_injection_is_rejected_before_launch():
    """Bad requests never reach the GPU: the launch counter does not move."""
    L = capi.lib()
    before = L.one_cuda_launch_count()
    u = abi.default_useful_info()
    cfg = abi.conv_cfg((3, 3), (1, 1), (1, 1, 1, 1), group=2)
    a = abi.conv_eval_args(cfg, (1, 8, 8, 8), (8, 8, 3, 3), (1, 8, 8, 8), 16, 16, 16, 16, u)
    assert L.one_cuda_conv_eval(a.params, a.inputs, a.outputs) == -3
    cfg = abi.conv_cfg((3, 3), (1, 1), (1, 1, 1, 1))
    a = abi.conv_eval_args(cfg, (1, 8, 8, 8), (8, 8, 3, 3), (1, 8, 9, 8), 16, 16, 16, 16, u)
    assert L.one_cuda_conv_eval(a.params, a.inputs, a.outputs) == -2
    assert L.one_cuda_launch_count() == before
