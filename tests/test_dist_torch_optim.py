"""Stock ``torch.optim`` machinery on sharded parameters (gloo, world 3): optimizers in single-tensor, foreach and fused
form, parameter groups with a learning-rate schedule, ``GradScaler``, and ``torch.save`` / ``torch.load`` of model and
optimizer state.  Every flow must reproduce the unsharded run."""

import io

import pytest
import torch

from dist_utils import run_distributed
from test_dist_randomized import _build, _config, _ids, _loss

OPTIMIZERS = {
    "sgd_nesterov": lambda ps: torch.optim.SGD(ps, lr=0.05, momentum=0.9, nesterov=True, weight_decay=0.01),
    "adamw_single_tensor": lambda ps: torch.optim.AdamW(ps, lr=0.01, foreach=False),
    "adamw_foreach_amsgrad": lambda ps: torch.optim.AdamW(ps, lr=0.01, foreach=True, amsgrad=True),
    "adamw_fused": lambda ps: torch.optim.AdamW(ps, lr=0.01, fused=True),
    "rmsprop_momentum": lambda ps: torch.optim.RMSprop(ps, lr=0.01, momentum=0.5, eps=1e-4),
    "adagrad": lambda ps: torch.optim.Adagrad(ps, lr=0.05),
}


def _models(seed=3):
    from yafsdp_b200 import fully_shard

    cfg = _config(seed)
    cfg.update(tie=False, freeze=False, micro=1)
    ref, model = _build(cfg, seed), _build(cfg, seed)
    fully_shard(model.emb)
    for l in model.layers:
        fully_shard(l)
    fully_shard([model.norm, model.head])
    fully_shard(model)
    return cfg, ref, model


def _backward_both(cfg, ref, model, rank, world, scale_ref=lambda x: x, scale=lambda x: x):
    for r in range(world):
        scale_ref(_loss(ref, _ids(cfg, r, 0)) / world).backward()
    scale(_loss(model, _ids(cfg, rank, 0))).backward()


def _check(model, ref, tag):
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p.full_tensor(), q.detach(), atol=3e-5), (tag, n, (p.full_tensor() - q).abs().max().item())


def _optimizer_worker(rank, world):
    for name in sorted(OPTIMIZERS):
        cfg, ref, model = _models()
        ref_opt, opt = OPTIMIZERS[name](list(ref.parameters())), OPTIMIZERS[name](list(model.parameters()))
        for _ in range(3):
            ref_opt.zero_grad()
            opt.zero_grad()
            _backward_both(cfg, ref, model, rank, world)
            ref_opt.step()
            opt.step()
        _check(model, ref, name)


@pytest.mark.timeout(300)
def test_torch_optimizers():
    run_distributed(_optimizer_worker, 3)


def _flows_worker(rank, world):
    # ---- parameter groups + learning-rate schedule
    cfg, ref, model = _models()

    def grouped(m):
        return [{"params": [p for p in m.parameters() if p.dim() > 1], "weight_decay": 0.1},
                {"params": [p for p in m.parameters() if p.dim() <= 1], "weight_decay": 0.0}]

    ref_opt, opt = torch.optim.AdamW(grouped(ref), lr=0.01), torch.optim.AdamW(grouped(model), lr=0.01)
    ref_sched = torch.optim.lr_scheduler.OneCycleLR(ref_opt, 0.05, total_steps=4)
    sched = torch.optim.lr_scheduler.OneCycleLR(opt, 0.05, total_steps=4)
    for _ in range(3):
        ref_opt.zero_grad()
        opt.zero_grad()
        _backward_both(cfg, ref, model, rank, world)
        ref_opt.step()
        opt.step()
        ref_sched.step()
        sched.step()
    _check(model, ref, "param groups + schedule")

    # ---- loss scaling: unscale, clip, step, update
    cfg, ref, model = _models()
    ref_opt, opt = torch.optim.SGD(ref.parameters(), lr=0.05), torch.optim.SGD(model.parameters(), lr=0.05)
    ref_scaler, scaler = torch.amp.GradScaler("cpu", init_scale=1024.0), torch.amp.GradScaler("cpu", init_scale=1024.0)
    for _ in range(3):
        ref_opt.zero_grad()
        opt.zero_grad()
        _backward_both(cfg, ref, model, rank, world, ref_scaler.scale, scaler.scale)
        ref_scaler.unscale_(ref_opt)
        scaler.unscale_(opt)
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        torch.nn.utils.clip_grad_norm_(model.parameters(), 0.5)
        ref_scaler.step(ref_opt)
        scaler.step(opt)
        ref_scaler.update()
        scaler.update()
    _check(model, ref, "GradScaler")

    # ---- torch.save / torch.load (weights_only) of the sharded model and optimizer state, then continue
    cfg, ref, model = _models()
    ref_opt, opt = torch.optim.AdamW(ref.parameters(), lr=0.01), torch.optim.AdamW(model.parameters(), lr=0.01)
    for _ in range(2):
        ref_opt.zero_grad()
        opt.zero_grad()
        _backward_both(cfg, ref, model, rank, world)
        ref_opt.step()
        opt.step()
    buf = io.BytesIO()
    torch.save({"model": model.state_dict(), "optim": opt.state_dict()}, buf)
    buf.seek(0)
    state = torch.load(buf, weights_only=True)
    _, _, model2 = _models(seed=3)
    with torch.no_grad():
        for p in model2.parameters():
            p.zero_()
    opt2 = torch.optim.AdamW(model2.parameters(), lr=0.01)
    model2.load_state_dict(state["model"])
    opt2.load_state_dict(state["optim"])
    ref_opt.zero_grad()
    opt2.zero_grad()
    _backward_both(cfg, ref, model2, rank, world)
    ref_opt.step()
    opt2.step()
    _check(model2, ref, "torch.save / torch.load")


@pytest.mark.timeout(240)
def test_param_groups_schedule_grad_scaler_and_torch_save():
    run_distributed(_flows_worker, 3)
