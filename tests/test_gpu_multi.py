"""Multi-GPU checks (skipped with fewer than 2 GPUs): peer-memory collectives vs NCCL, and sharded training with
the peer-memory backend vs the NCCL backend."""

import os
import socket
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, errq):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        fn(rank, world)
        torch.cuda.synchronize()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _run(fn, world):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    if not errq.empty():
        rank, tb = errq.get()
        raise AssertionError(f"rank {rank} failed:\n{tb}")
    assert not alive, "timed out"
    assert all(p.exitcode == 0 for p in procs)


def _world():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    return 2 if n < 4 else (4 if n < 8 else 8)


def _collectives_worker(rank, world):
    import torch.distributed as dist
    from yafsdp_b200.comm.symm import SymmBackend
    from yafsdp_b200.ops import kernels

    dev = torch.device("cuda", rank)
    be = SymmBackend(dev, dist.group.WORLD)
    torch.manual_seed(rank)
    for shard in (1024, 8 * 1000 * 100 + 8 * 3):
        inp = be.alloc(shard, torch.bfloat16, dev, "gather_input")
        inp.copy_(torch.randn(shard, device=dev).bfloat16())
        out = torch.empty(shard * world, device=dev, dtype=torch.bfloat16)
        ref = torch.empty_like(out)
        dist.all_gather_into_tensor(ref, inp)
        be.step_barrier()
        be.all_gather(out, inp, dist.group.WORLD)
        torch.cuda.synchronize()
        assert torch.equal(out, ref)
        for wire in (torch.float32, torch.bfloat16):
            g = be.alloc(shard * world, wire, dev, "reduce_input")
            g.copy_(torch.randn(shard * world, device=dev).to(wire))
            want = torch.empty(shard, device=dev, dtype=torch.float32)
            dist.reduce_scatter_tensor(want, g.float(), op=dist.ReduceOp.SUM)
            dst = torch.ones(shard, device=dev, dtype=torch.float32)
            be.reduce_scatter(dst, g, dist.group.WORLD, scale=1.0 / world, accumulate=True)
            torch.cuda.synchronize()
            assert torch.allclose(dst, 1 + want / world, rtol=1e-5, atol=1e-5)
    kernels.check_status()


def test_symm_collectives_match_nccl():
    _run(_collectives_worker, _world())


def _train_worker(rank, world):
    from yafsdp_b200.models.llama import CONFIGS
    from yafsdp_b200.ops import kernels
    from yafsdp_b200.optim import ShardedAdamW
    from yafsdp_b200.train import TrainStep, build_llama

    dev = torch.device("cuda", rank)
    cfg = CONFIGS["tiny-gpu"]
    ids = torch.randint(0, cfg.vocab_size, (2, 256), generator=torch.Generator().manual_seed(1 + rank)).to(dev)
    losses = {}
    for backend in ("torch", "symm"):
        model = build_llama(cfg, dev, comm_backend=backend)
        opt = ShardedAdamW(model, lr=1e-3, max_grad_norm=1.0)
        step = TrainStep(model, opt, dev)
        losses[backend] = [step(ids).item() for _ in range(4)]
        kernels.check_status()
    for a, b in zip(losses["torch"], losses["symm"]):
        assert abs(a - b) < 2e-2 * abs(a), (losses["torch"], losses["symm"])
    assert losses["symm"][-1] < losses["symm"][0]


def test_training_symm_backend_matches_nccl_backend():
    _run(_train_worker, _world())
