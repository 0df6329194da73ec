"""Failure detection without GPU faults: a rank that stops is noticed through the heartbeat store; a device wait on a flag
that nothing sets runs out, reports a status code and leaves the context usable."""

import time

import pytest
import torch

from dist_utils import run_distributed


def _heartbeat_worker(rank, world):
    import torch.distributed as dist
    from yafsdp_b200.utils.failure import Heartbeat, RankFailure

    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval_s=0.1, timeout_s=1.0)
    hb.start()
    dist.barrier()
    hb.check()  # everybody alive
    if rank == world - 1:
        hb.stop()  # this rank "dies" between steps: no kernel or collective of it is in flight
        time.sleep(4.0)
        return
    deadline = time.monotonic() + 6.0
    with pytest.raises(RankFailure) as info:
        while time.monotonic() < deadline:
            hb.check()
            time.sleep(0.2)
    assert info.value.ranks == [world - 1]
    hb.stop()


@pytest.mark.timeout(120)
def test_heartbeat_reports_a_silent_rank():
    run_distributed(_heartbeat_worker, 3)


@pytest.mark.gpu
def test_device_wait_runs_out_and_reports_status():
    from yafsdp_b200 import _native
    from yafsdp_b200.ops import kernels

    kernels.status()  # clear
    flags = torch.zeros(8, device="cuda", dtype=torch.int64)
    rc = _native.lib().yf_flag_wait(flags.data_ptr(), 3, 1, 200, torch.cuda.current_stream().cuda_stream)  # nobody sets word 3
    assert rc == 0
    torch.cuda.synchronize()
    code, site = kernels.status()
    assert code == 2 and site == 400  # YF_ERR_FLAG_TIMEOUT at the flag-wait site
    # the context is intact: a satisfied wait and ordinary work still run
    _native.lib().yf_flag_set(flags.data_ptr(), 3, 1, torch.cuda.current_stream().cuda_stream)
    _native.lib().yf_flag_wait(flags.data_ptr(), 3, 1, 200, torch.cuda.current_stream().cuda_stream)
    x = torch.ones(1024, device="cuda").sum().item()
    assert x == 1024 and kernels.status() == (0, 0)
