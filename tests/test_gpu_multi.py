"""Multi-GPU checks (skipped with fewer than 2 GPUs): peer-memory collectives vs NCCL, and sharded training with
the peer-memory backend vs the NCCL backend."""

import datetime
import os
import socket
import time
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, errq, transport=None):
    import torch.distributed as dist

    if transport:
        os.environ["YAFSDP_SYMM_TRANSPORT"] = transport
    # a rank that fails must not leave its peers waiting for minutes: short limits on device-side waits and on NCCL
    os.environ.setdefault("YAFSDP_SYMM_TIMEOUT_MS", "20000")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                                timeout=datetime.timedelta(seconds=120))
        fn(rank, world)
        torch.cuda.synchronize()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        # leave with nothing of this rank in flight (every device-side wait is bounded), but without tearing the process
        # group down: that could wait for collectives that the peers will never join
        try:
            torch.cuda.synchronize()
        except Exception:
            pass
        os._exit(1)
    dist.destroy_process_group()


def _run(fn, world, transport=None):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, errq, transport)) for r in range(world)]
    for p in procs:
        p.start()
    deadline = time.monotonic() + 240  # for all ranks together: the tiny models below need well under a minute
    for p in procs:
        p.join(max(1.0, deadline - time.monotonic()))
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
    if os.environ.get("YAFSDP_SYMM_TRANSPORT") == "mc":
        if not be.has_multicast:
            return  # no NVSwitch multicast on this machine: the backend fell back (with a warning)
        assert be.ag_transport == "mc" and be.rs_transport == "mc"
    if os.environ.get("YAFSDP_SYMM_TRANSPORT") == "cp":
        assert be.ag_transport == "cp" and be.symmetric_gather_output  # the ranks write their shards into the peers' outputs
    torch.manual_seed(rank)
    for shard in (1024, 8 * 1000 * 100 + 8 * 3):
        inp = be.alloc(shard, torch.bfloat16, dev, "gather_input")
        inp.copy_(torch.randn(shard, device=dev).bfloat16())
        out = be.alloc(shard * world, torch.bfloat16, dev, "gather_output")
        out.zero_()
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
            tol = 1e-5 if (wire == torch.float32 or be.rs_transport != "mc") else 2e-2  # the switch returns bf16 sums
            assert torch.allclose(dst, 1 + want / world, rtol=tol, atol=tol)
            # gradient-norm fusion: the kernel also sums the squares of what it leaves in dst
            ss = torch.zeros(1, device=dev, dtype=torch.float32)
            assert be.reduce_scatter(dst, g, dist.group.WORLD, scale=1.0 / world, accumulate=False, sumsq=ss)
            torch.cuda.synchronize()
            assert torch.allclose(dst, want / world, rtol=tol, atol=tol)
            assert torch.allclose(ss, dst.double().pow(2).sum().float(), rtol=1e-4)
    kernels.check_status()


@pytest.mark.parametrize("transport", [None, "sm", "mc", "cp"])
def test_symm_collectives_match_nccl(transport):
    _run(_collectives_worker, _world(), transport)


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
        # with the multicast transports the reduce-scatter under test is the switch's (multimem.ld_reduce), so the gradients
        # are not pushed from the GEMM epilogues instead; otherwise the default of this world size runs
        fused_reduce = False if os.environ.get("YAFSDP_SYMM_TRANSPORT") == "mc" else None
        model = build_llama(cfg, dev, comm_backend=backend, fused_gather=True, fused_reduce=fused_reduce)
        opt = ShardedAdamW(model, lr=1e-3, max_grad_norm=1.0)
        step = TrainStep(model, opt, dev)
        losses[backend] = [step(ids).item() for _ in range(4)]
        kernels.check_status()
        if backend == "symm":
            # the first layer's forward all-gather ran inside its QKV GEMM (once per step), every other gather ahead of time
            g0 = model.model.layers[0]._get_fsdp_state()._param_group
            g1 = model.model.layers[1]._get_fsdp_state()._param_group
            assert g0.fused_gather and g0._gather_epoch == 4 and g1._gather_epoch == 0, (g0._gather_epoch, g1._gather_epoch)
    for a, b in zip(losses["torch"], losses["symm"]):
        assert abs(a - b) < 2e-2 * abs(a), (losses["torch"], losses["symm"])
    assert losses["symm"][-1] < losses["symm"][0]


@pytest.mark.parametrize("transport", [None, "mc", "cp"])
def test_training_symm_backend_matches_nccl_backend(transport):
    _run(_train_worker, _world(), transport)


def _fused_worker(rank, world):
    """All-gather -> GEMM and GEMM -> reduce-scatter fused kernels against NCCL + the plain GEMM."""
    import torch.distributed as dist
    from yafsdp_b200.comm.symm import SymmBackend
    from yafsdp_b200.ops import kernels

    dev = torch.device("cuda", rank)
    be = SymmBackend(dev, dist.group.WORLD)
    torch.manual_seed(100 + rank)
    # ---- a "layer": [pad 4096 | B: n x k | tail], sharded evenly; deliberately not aligned to rows or tiles
    n, k, m = 1280, 512, 384
    head, tail = 4096 + 8 * 7, 8 * 1001
    total = head + n * k + tail
    total = (total + world * 8 - 1) // (world * 8) * (world * 8)
    shard = total // world
    full = torch.randn(total, device=dev).bfloat16()
    dist.broadcast(full, 0)
    inp = be.alloc(shard, torch.bfloat16, dev, "gather_input")
    inp.copy_(full[rank * shard : (rank + 1) * shard])
    layer_buf = torch.zeros(total, device=dev, dtype=torch.bfloat16)
    counters = torch.zeros((n + 127) // 128, device=dev, dtype=torch.int64)
    a = torch.randn(m, k, device=dev).bfloat16()
    torch.cuda.synchronize()
    be.step_barrier()
    for epoch in (1, 2):
        layer_buf.zero_()
        out = kernels.gemm_gathered(a, n, k, peer_in=be._peers(inp), layer_buf=layer_buf, shard_bytes=shard * 2, b_byte_off=head * 2,
                                    rank=rank, world=world, counters=counters, epoch=epoch)
        torch.cuda.synchronize()
        assert torch.equal(layer_buf, full), "layer buffer is not the all-gather of the shards"
        ref = a.float() @ full[head : head + n * k].view(n, k).float().t()
        assert (out.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2
    kernels.check_status()
    # ---- GEMM -> reduce-scatter: dW = dy^T x of this rank's tokens, pushed to the owners, summed there
    t_tok, rows, cols = 256, 640, 384
    flat_off = 8 * 13
    ptotal = flat_off + rows * cols + 8 * 5
    ptotal = (ptotal + world * 8 - 1) // (world * 8) * (world * 8)
    pshard = ptotal // world
    dy = torch.randn(t_tok, rows, device=dev).bfloat16()
    x = torch.randn(t_tok, cols, device=dev).bfloat16()
    gbuf = be.alloc(ptotal, torch.float32, dev, "reduce_input")  # read as `world` slots of pshard floats
    gbuf.zero_()
    torch.cuda.synchronize()
    be.barrier(3)
    gbuf.fill_(float("nan"))  # whatever the pushes and the padding rule do not cover would poison the sums
    be.barrier(3)
    kernels.gemm_scatter(dy, x, a_mn_major=True, b_mn_major=True, peer_grad=be._peers(gbuf), c_flat_off=flat_off, shard_numel=pshard,
                         rank=rank, world=world)
    kernels.push_flat(None, flat_off, 0, be._peers(gbuf), pshard, rank, world)  # the range in front of the matrix: zeros
    tail0 = flat_off + rows * cols
    kernels.push_flat(torch.zeros(8 * 5, device=dev), 8 * 5, tail0, be._peers(gbuf), pshard, rank, world)
    got = torch.zeros(pshard, device=dev, dtype=torch.float32)
    be.reduce_pushed(got, gbuf, scale=1.0 / world, accumulate=False, valid_numel=tail0 + 8 * 5)  # waits for everybody's pushes
    local_dw = torch.zeros(ptotal, device=dev, dtype=torch.float32)
    local_dw[flat_off : flat_off + rows * cols] = (dy.float().t() @ x.float()).reshape(-1)
    want = torch.empty(pshard, device=dev, dtype=torch.float32)
    dist.reduce_scatter_tensor(want, local_dw, op=dist.ReduceOp.AVG)
    torch.cuda.synchronize()
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-1), (got - want).abs().max().item()
    kernels.check_status()
    # ---- the same as ONE grouped launch over three gradients of different shapes (owners' tiles dealt round-robin)
    shapes = [(640, 384), (256, 384), (512, 768)]  # (rows, cols) of the three weights; the last has another input width
    xs = {384: x, 768: torch.randn(t_tok, 768, device=dev).bfloat16()}
    dys = [torch.randn(t_tok, r, device=dev).bfloat16() for r, _ in shapes]
    offs, pos = [], 8 * 3
    for r, c in shapes:
        offs.append(pos)
        pos += r * c + 8 * 11  # a gap after every matrix (norm weights sit between the matrices of a real layer)
    gtotal = (pos + world * 8 - 1) // (world * 8) * (world * 8)
    gshard = gtotal // world
    gbuf2 = be.alloc(gtotal, torch.float32, dev, "reduce_input")
    torch.cuda.synchronize()
    be.barrier(3)
    gbuf2.zero_()  # the gaps are not pushed by anybody in this test
    be.barrier(3)
    kernels.gemm_scatter_grouped([(dy_i, xs[c], off) for dy_i, (_, c), off in zip(dys, shapes, offs)], peer_grad=be._peers(gbuf2),
                                 shard_numel=gshard, rank=rank, world=world)
    got2 = torch.zeros(gshard, device=dev, dtype=torch.float32)
    be.reduce_pushed(got2, gbuf2, scale=1.0 / world, accumulate=False)
    local2 = torch.zeros(gtotal, device=dev, dtype=torch.float32)
    for dy_i, (r, c), off in zip(dys, shapes, offs):
        local2[off : off + r * c] = (dy_i.float().t() @ xs[c].float()).reshape(-1)
    want2 = torch.empty(gshard, device=dev, dtype=torch.float32)
    dist.reduce_scatter_tensor(want2, local2, op=dist.ReduceOp.AVG)
    torch.cuda.synchronize()
    assert torch.allclose(got2, want2, rtol=2e-2, atol=2e-1), (got2 - want2).abs().max().item()
    kernels.check_status()


def test_fused_gather_gemm_and_gemm_scatter():
    _run(_fused_worker, _world())


def _unshard_after_step_worker(rank, world):
    """An explicit unshard() after an optimizer step (outside any forward) must gather the UPDATED weights of every
    rank: the peer-memory backend refreshes all gather inputs and lets the ranks meet before anybody pulls."""
    from yafsdp_b200.models.llama import CONFIGS
    from yafsdp_b200.ops import kernels
    from yafsdp_b200.train import build_llama

    dev = torch.device("cuda", rank)
    cfg = CONFIGS["tiny-gpu"]
    model = build_llama(cfg, dev, comm_backend="symm", fused_reduce=False)  # the plain reduce-scatter: this test is about gathers
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)  # a stock optimizer: the gather inputs go stale after its step
    ids = torch.randint(0, cfg.vocab_size, (2, 256), generator=torch.Generator().manual_seed(1 + rank)).to(dev)
    for _ in range(2):
        opt.zero_grad()
        model(ids, labels=ids).backward()
        opt.step()
        layer = model.model.layers[0]
        want = {n: p.full_tensor().to(torch.bfloat16) for n, p in layer.named_parameters()}
        layer.unshard()
        for n, p in layer.named_parameters():
            assert torch.equal(p.detach(), want[n]), f"{n}: gathered weights are not the updated ones"
        layer.reshard()
    torch.cuda.synchronize()
    kernels.check_status()


def test_unshard_after_optimizer_step_sees_updated_weights():
    _run(_unshard_after_step_worker, _world())


def _train_fused_reduce_worker(rank, world):
    """Training with the gradient reduce-scatter fused into the weight-gradient GEMMs (rows pushed from the epilogue to
    their owners) against the NCCL backend, including two micro-batches per step.  With YF_TEST_WIRE=bf16 the gradients
    travel as bf16 (reduce_dtype=bfloat16) and are summed in fp32 by their owners."""
    from yafsdp_b200 import MixedPrecisionPolicy
    from yafsdp_b200.models.llama import CONFIGS
    from yafsdp_b200.ops import kernels
    from yafsdp_b200.optim import ShardedAdamW
    from yafsdp_b200.train import build_llama

    dev = torch.device("cuda", rank)
    cfg = CONFIGS["tiny-gpu"]
    gen = torch.Generator().manual_seed(1 + rank)
    batches = [torch.randint(0, cfg.vocab_size, (2, 256), generator=gen).to(dev) for _ in range(2)]
    losses = {}
    bf16_wire = os.environ.get("YF_TEST_WIRE") == "bf16"
    policy = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16 if bf16_wire else torch.float32)
    for name, kw in (("torch", dict(comm_backend="torch")), ("fused", dict(comm_backend="symm", fused_reduce=True))):
        model = build_llama(cfg, dev, mp_policy=policy, **kw)
        opt = ShardedAdamW(model, lr=1e-3, max_grad_norm=1.0)
        out = []
        for _ in range(4):
            opt.zero_grad()
            for ids in batches:  # two micro-batches, each reduced and accumulated into the sharded gradient
                loss = model(ids, labels=ids)
                (loss / len(batches)).backward()
            opt.step()
            out.append((loss.item(), opt.last_grad_norm.item()))
        losses[name] = out
        kernels.check_status()
        if name == "fused":
            g = model.model.layers[0]._get_fsdp_state()._param_group
            assert g.fused_reduce and g._push_ptrs is not None, "the fused path was not active"
            assert g._grad_flat.dtype == (torch.bfloat16 if bf16_wire else torch.float32)
    for (a, na), (b, nb) in zip(losses["torch"], losses["fused"]):
        assert abs(a - b) < (4e-2 if bf16_wire else 2e-2) * abs(a), losses
        assert abs(na - nb) < (6e-2 if bf16_wire else 3e-2) * abs(na), losses
    assert losses["fused"][-1][0] < losses["fused"][0][0]


@pytest.mark.parametrize("wire", ["fp32", "bf16"])
def test_training_with_fused_gemm_reduce_scatter(wire):
    os.environ["YF_TEST_WIRE"] = wire
    try:
        _run(_train_fused_reduce_worker, _world())
    finally:
        os.environ.pop("YF_TEST_WIRE", None)


def _hpz_worker(rank, world):
    """Hierarchical partitioning on the peer-memory backend: the backward all-gather of the layers runs inside subgroups
    of half the ranks, from secondary shards in peer-mapped memory; losses must match the plain configuration."""
    import torch.distributed as dist
    from yafsdp_b200.models.llama import CONFIGS
    from yafsdp_b200.ops import kernels
    from yafsdp_b200.optim import ShardedAdamW
    from yafsdp_b200.train import TrainStep, build_llama

    dev = torch.device("cuda", rank)
    cfg = CONFIGS["tiny-gpu"]
    ids = torch.randint(0, cfg.vocab_size, (2, 256), generator=torch.Generator().manual_seed(1 + rank)).to(dev)
    n = max(1, world // 2)
    groups = [dist.new_group(list(range(s, s + n))) for s in range(0, world, n)]
    mine = groups[rank // n]
    losses = {}
    for hpz in (False, True):
        model = build_llama(cfg, dev, comm_backend="symm", fused_reduce=False)
        if hpz:
            for layer in model.model.layers:
                layer.set_secondary_shard_group(mine)
        opt = ShardedAdamW(model, lr=1e-3, max_grad_norm=1.0)
        step = TrainStep(model, opt, dev)
        losses[hpz] = [step(ids).item() for _ in range(3)]
        kernels.check_status()
        if hpz:
            g = model.model.layers[0]._get_fsdp_state()._param_group
            assert g._secondary_shard is not None and g._secondary_backend is model._get_fsdp_state()._comm_ctx.backend
    for a, b in zip(losses[False], losses[True]):
        assert abs(a - b) < 1e-3 * abs(a), losses


def test_hierarchical_partitioning_on_peer_memory_backend():
    _run(_hpz_worker, _world())
