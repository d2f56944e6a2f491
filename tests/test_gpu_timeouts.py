"""A bounded device-side wait that runs out must come back to the host as VPQ_ERR_TIMEOUT with the
recorded site, leave the GPU usable, and clear (the analogue of Fence::wait_ok(&reason),
apple-silicon/metal-compute/command-stream.h:92-117). The waits are made to run out on the host's
terms: an mbarrier nobody arrives at, a rank that never publishes its flag, each with a poll limit
of about a millisecond. Nothing faults, traps or hangs."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

VPQ_ERR_TIMEOUT = 6


def _status(vpq):
    detail = C.c_uint32(0)
    rc = vpq.lib().vpq_device_status(torch.cuda.current_stream().cuda_stream, C.byref(detail))
    return rc, int(detail.value)


def test_mbarrier_wait_that_runs_out_reports_and_clears(vpq):
    torch.cuda.set_device(0)
    lib = vpq.lib()
    assert _status(vpq) == (0, 0)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.vpq_wait_probe(200, 1000, st) == 0          # 200 polls of <= 1 us
    rc, detail = _status(vpq)
    assert rc == VPQ_ERR_TIMEOUT and detail == 0x7f7f
    assert b"site 127" in lib.vpq_last_error()
    assert _status(vpq) == (0, 0)                            # cleared by the read
    # the device is still in working order
    a = torch.arange(1024, device="cuda:0")
    assert int(a.sum()) == 1023 * 512
    assert lib.vpq_wait_probe(0, 1000, st) != 0              # limits are enforced on the host
    assert lib.vpq_wait_probe(1 << 20, 1000, st) != 0


@pytest.mark.parametrize("world,absent", [(2, 1), (8, 5)])
def test_peer_barrier_gives_up_on_a_rank_that_never_arrives(vpq, world, absent):
    torch.cuda.set_device(0)
    lib = vpq.lib()
    assert _status(vpq) == (0, 0)
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    assert lib.vpq_peer_barrier_probe(ws.data_ptr(), world, absent, 10000, st) == 0   # ~1 ms
    rc, detail = _status(vpq)
    assert rc == VPQ_ERR_TIMEOUT and detail == (0x20000 | 0x7700 | absent)
    assert f"rank {absent}".encode() in lib.vpq_last_error()
    assert _status(vpq) == (0, 0)
    # and the next real call succeeds
    from vpipe_b200 import ops
    codes = torch.zeros((16, 8), dtype=torch.int32, device="cuda:0")
    s = torch.ones((16, 1), dtype=torch.bfloat16, device="cuda:0")
    x = torch.ones((1, 64), dtype=torch.bfloat16, device="cuda:0")
    y = ops.qmv(codes, s, s, x)
    torch.cuda.synchronize()
    assert torch.all(y == 64.0)
    assert lib.vpq_peer_barrier_probe(ws.data_ptr(), world, 0, 10000, st) != 0        # rank 0 is the caller
