"""A bounded device-side wait that runs out: the kernel gives up after its limit, leaves a code in the status word, the host
raises, and the context stays usable.  The wait is made to run out without any fault: a flag barrier of a two-rank group
is launched in one process with both signal pads in local memory, so the flag of the second rank is simply never set;
the limit is 50 ms.  (This file sorts last on purpose: it runs after every other test.)"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_raises_on_the_host_and_leaves_the_context_usable():
    from fairscale_b200 import _native
    from fairscale_b200.ops import _bind
    from fairscale_b200.parallel import nvlink, symm
    from fairscale_b200.utils.failure import CommTimeoutError, check_device_status

    dev = torch.device("cuda", 0)
    nvlink._sigs()
    check_device_status(dev)  # clean before we start
    before_ms = nvlink.timeout_ms()
    poisoned_before = {k: getattr(ws, "poisoned", False) for k, ws in symm._WORKSPACES.items()}
    pads = [torch.zeros(64 * 8, dtype=torch.int32, device=dev) for _ in range(2)]  # ours, and a stand-in for the absent peer's
    try:
        nvlink.set_timeout(0.05)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        _bind.call("fsb_comm_barrier", 0, 2, 1, 40, nvlink._ptr_array([p.data_ptr() for p in pads]), _bind.status_ptr(dev),
                   _bind.stream_ptr(dev))
        stop.record()
        torch.cuda.synchronize()
        waited_ms = start.elapsed_time(stop)
        assert 40.0 <= waited_ms <= 1000.0, waited_ms  # it waited for its limit, not for ever
        # both arrivals of rank 0 were published; rank 1's never came
        assert int(pads[0][40 * 8 + 0]) == 1 and int(pads[1][40 * 8 + 0]) == 1 and int(pads[0][40 * 8 + 1]) == 0
        with pytest.raises(CommTimeoutError):
            check_device_status(dev)
        check_device_status(dev)  # reading the word cleared it
    finally:
        nvlink.set_timeout(before_ms / 1000.0)
        for k, ws in symm._WORKSPACES.items():
            ws.poisoned = poisoned_before.get(k, False)
    # the context is alive: PyTorch and native kernels still run and report nothing
    x = torch.randn(1024, 256, device=dev).bfloat16()
    from fairscale_b200.ops.reduce import column_sum

    torch.testing.assert_close(column_sum(x).float(), x.float().sum(0), atol=0.5, rtol=2e-2)
    assert _native.read_status(dev) == 0
