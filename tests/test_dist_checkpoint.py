"""Checkpoint format, load planner and resharding across world sizes (gloo)."""

import os

import pytest
import torch

from dist_utils import run_distributed
from test_dist_features import _build, _data, _loss, _shard


def _save_worker(rank, world, path):
    from yafsdp_b200 import checkpoint

    model = _shard(_build())
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2, foreach=True)
    for _ in range(2):
        opt.zero_grad()
        _loss(model, _data(rank)).backward()
        opt.step()
    checkpoint.save(path, model)
    full = checkpoint.full_state_dict(model)
    if rank == 0:
        torch.save(full, os.path.join(path, "full_rank0.pt"))
        # on-disk metadata: every parameter is a flat tensor with one chunk per saving rank
        from torch.distributed.checkpoint import FileSystemReader

        md = FileSystemReader(path).read_metadata().state_dict_metadata
        entry = md["model.layers.0.a.weight"]
        assert tuple(entry.size) == (16 * 24,) and len(entry.chunks) == world
        assert sum(int(c.sizes[0]) for c in entry.chunks) == 16 * 24


def _load_worker(rank, world, path):
    from yafsdp_b200 import checkpoint

    want = torch.load(os.path.join(path, "full_rank0.pt"))
    model = _shard(_build(seed=123))  # different init: everything must come from the checkpoint
    checkpoint.load(path, model)
    for n, p in model.named_parameters():
        assert torch.equal(p.full_tensor(), want[n]), n
    # an unsharded model loads the same files through the flat-format planner
    if rank == 0:
        import torch.distributed.checkpoint as dcp

        plain = _build(seed=7)
        sd = {"model": plain.state_dict()}
        dcp.load(sd, checkpoint_id=path, planner=checkpoint.RaggedLoadPlanner(), no_dist=True)
        for n, p in plain.named_parameters():
            assert torch.equal(p.detach(), want[n]), n


@pytest.mark.timeout(300)
def test_save_world2_load_world3_and_unsharded(tmp_path):
    path = str(tmp_path / "ckpt")
    run_distributed(_save_worker, 2, path)
    run_distributed(_load_worker, 3, path)


def _optim_roundtrip_worker(rank, world, path):
    from yafsdp_b200 import checkpoint
    from yafsdp_b200.optim import ShardedAdamW

    model = _shard(_build())
    opt = ShardedAdamW(model, lr=1e-2)
    for _ in range(2):
        opt.zero_grad()
        _loss(model, _data(rank)).backward()
        opt.step()
    checkpoint.save(path, model, opt, extra={"step": 2})
    ref_m = [m.clone() for m in opt.exp_avg]
    model2 = _shard(_build(seed=5))
    opt2 = ShardedAdamW(model2, lr=1e-2)
    extra = checkpoint.load(path, model2, opt2, extra={"step": 0})
    assert extra["step"] == 2 and opt2.step_count == 2
    for a, b in zip(ref_m, opt2.exp_avg):
        assert torch.equal(a, b)
    # both continue identically
    for m, o in ((model, opt), (model2, opt2)):
        o.zero_grad()
        _loss(m, _data(rank)).backward()
        o.step()
    for (n, p), (_, q) in zip(model.named_parameters(), model2.named_parameters()):
        assert torch.equal(p._local_tensor, q._local_tensor), n


@pytest.mark.timeout(300)
def test_model_and_sharded_adamw_roundtrip(tmp_path):
    run_distributed(_optim_roundtrip_worker, 2, str(tmp_path / "ckpt2"))


# ------------------------------------------------------------------------------------------------ damaged checkpoints
def _load_damaged_worker(rank, world, path, kind):
    """A checkpoint with a missing shard file, or one written for a model of another size, must fail loudly on every rank
    instead of loading partial or shifted data."""
    from yafsdp_b200 import checkpoint

    if kind == "wrong_model":
        model = _shard(_build(seed=1, d=32))  # twice the width: the saved flat tensors have other sizes
    else:
        model = _shard(_build(seed=1))
    before = {n: p.full_tensor().clone() for n, p in model.named_parameters()}
    with pytest.raises(BaseException) as err:  # torch's CheckpointException derives from BaseException
        checkpoint.load(path, model)
    assert ("flat form" if kind == "wrong_model" else "No such file") in str(err.value)
    if kind == "wrong_model":
        # the planner refused before anything was read: the model is untouched
        for n, p in model.named_parameters():
            assert torch.equal(p.full_tensor(), before[n]), n


@pytest.mark.timeout(300)
@pytest.mark.parametrize("kind", ["missing_shard", "wrong_model"])
def test_damaged_checkpoint_fails_loudly(tmp_path, kind):
    path = str(tmp_path / "ckpt")
    run_distributed(_save_worker, 2, path)
    if kind == "missing_shard":
        shards = sorted(f for f in os.listdir(path) if f.endswith(".distcp"))
        assert len(shards) == 2
        os.remove(os.path.join(path, shards[1]))
    run_distributed(_load_damaged_worker, 1, path, kind)  # one loading rank: a failing load cannot leave peers waiting


# ------------------------------------------------------------------------------------------------ resume at another world size
def _adamw_reference(worlds_per_phase, steps_per_phase):
    """Unsharded AdamW over the same global batches: phase k uses the data of ``worlds_per_phase[k]`` ranks."""
    model = _build()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    for world, steps in zip(worlds_per_phase, steps_per_phase):
        for _ in range(steps):
            opt.zero_grad()
            for r in range(world):
                (_loss(model, _data(r)) / world).backward()
            opt.step()
    return {n: p.detach().clone() for n, p in model.named_parameters()}


def _resume_worker(rank, world, path, phase):
    from yafsdp_b200 import checkpoint
    from yafsdp_b200.optim import ShardedAdamW

    model = _shard(_build(seed=0 if phase == 0 else 99))
    opt = ShardedAdamW(model, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    if phase == 1:
        extra = checkpoint.load(path, model, opt, extra={"step": 0})
        assert extra["step"] == 2 and opt.step_count == 2
    for _ in range(2):
        opt.zero_grad()
        _loss(model, _data(rank)).backward()
        opt.step()
    if phase == 0:
        checkpoint.save(path, model, opt, extra={"step": 2})
    else:
        want = _adamw_reference([2, 3], [2, 2])
        for n, p in model.named_parameters():
            assert torch.allclose(p.full_tensor(), want[n], atol=1e-5), n


@pytest.mark.timeout(300)
def test_training_resumes_at_another_world_size_with_optimizer_state(tmp_path):
    path = str(tmp_path / "ckpt3")
    run_distributed(_resume_worker, 2, path, 0)
    run_distributed(_resume_worker, 3, path, 1)
