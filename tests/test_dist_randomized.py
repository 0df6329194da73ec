"""Randomised end-to-end check of the scheduler on CPU/gloo: random depth, widths, frozen parameters, tied embeddings,
resharding policy, micro-batch count and wrap granularity; sharded training must match the unsharded model."""

import random

import pytest
import torch
import torch.nn as nn

from dist_utils import run_distributed


class _Block(nn.Module):
    def __init__(self, d, h, norm):
        super().__init__()
        self.norm = nn.LayerNorm(d) if norm else nn.Identity()
        self.a = nn.Linear(d, h)
        self.b = nn.Linear(h, d, bias=False)

    def forward(self, x):
        return x + self.b(torch.tanh(self.a(self.norm(x))))


class _Net(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        d = cfg["d"]
        self.emb = nn.Embedding(cfg["vocab"], d)
        self.layers = nn.ModuleList([_Block(d, h, n) for h, n in zip(cfg["hidden"], cfg["norms"])])
        self.norm = nn.LayerNorm(d)
        self.head = nn.Linear(d, cfg["vocab"], bias=False)
        if cfg["tie"]:
            self.head.weight = self.emb.weight

    def forward(self, ids):
        x = self.emb(ids)
        for l in self.layers:
            x = l(x)
        return self.head(self.norm(x))


def _config(seed):
    rng = random.Random(seed)
    n = rng.randint(1, 4)
    return {
        "d": rng.choice([6, 10, 16]), "vocab": rng.choice([11, 32]), "hidden": [rng.choice([5, 12, 24]) for _ in range(n)],
        "norms": [rng.random() < 0.5 for _ in range(n)], "tie": rng.random() < 0.3, "micro": rng.randint(1, 2),
        "reshard": rng.choice([True, None]), "freeze": rng.random() < 0.5, "pair_layers": rng.random() < 0.3,
        "alignment": rng.choice([1, 8]), "eval_between": rng.random() < 0.4, "checkpoint": rng.random() < 0.4,
        "explicit_unshard": rng.random() < 0.3, "prefetch": rng.random() < 0.3, "adamw": rng.random() < 0.5,
        "wide_compute": rng.random() < 0.3, "nosync": rng.random() < 0.3, "state_dict_roundtrip": rng.random() < 0.3,
    }


def _build(cfg, seed):
    torch.manual_seed(seed)
    model = _Net(cfg)
    if cfg["freeze"]:
        rng = random.Random(seed + 1)
        for l in model.layers:
            if rng.random() < 0.5:
                l.a.bias.requires_grad_(False)
            if rng.random() < 0.3:
                l.b.weight.requires_grad_(False)
    return model


def _loss(model, ids):
    out = model(ids)
    return nn.functional.cross_entropy(out.view(-1, out.shape[-1]), ids.view(-1))


def _ids(cfg, rank, micro):
    return torch.randint(0, cfg["vocab"], (3, 5), generator=torch.Generator().manual_seed(1000 + 10 * rank + micro))


def _worker(rank, world, seed):
    from yafsdp_b200 import fully_shard

    cfg = _config(seed)
    ref = _build(cfg, seed)
    trainable = [p for p in ref.parameters() if p.requires_grad]
    ref_opt = (torch.optim.AdamW(trainable, lr=0.01, betas=(0.9, 0.95), weight_decay=0.1) if cfg["adamw"]
               else torch.optim.SGD(trainable, lr=0.05))
    for _ in range(2):
        ref_opt.zero_grad()
        for r in range(world):
            for m in range(cfg["micro"]):
                (_loss(ref, _ids(cfg, r, m)) / (world * cfg["micro"])).backward()
        if cfg["adamw"]:
            torch.nn.utils.clip_grad_norm_(trainable, 0.5)
        ref_opt.step()

    model = _build(cfg, seed)
    kw = dict(reshard_after_forward=cfg["reshard"], shard_alignment=cfg["alignment"])
    if cfg["wide_compute"]:
        # compute and reduce in float64: exercises the separate gather input, the casts and a reduce dtype that differs from
        # the parameters' while staying comparable with the fp32 reference
        from yafsdp_b200 import MixedPrecisionPolicy

        kw["mp_policy"] = MixedPrecisionPolicy(param_dtype=torch.float64, reduce_dtype=torch.float64, cast_forward_inputs=True)
    if cfg["tie"]:
        fully_shard([model.emb, model.norm, model.head], **{**kw, "reshard_after_forward": False})
        model.emb._get_fsdp_state()._param_group.dedicated_buffers = True
    else:
        fully_shard(model.emb, **kw)
    layers = list(model.layers)
    if cfg["pair_layers"] and len(layers) >= 2:
        fully_shard(layers[:2], **kw)
        layers = layers[2:]
    for l in layers:
        fully_shard(l, **kw)
    if not cfg["tie"]:
        fully_shard([model.norm, model.head], **kw)
    fully_shard(model, **kw)
    if cfg["checkpoint"]:
        from yafsdp_b200.utils.checkpointing import checkpoint_module

        for l in list(model.layers)[::2]:
            checkpoint_module(l)
    singles = [l for l in layers]
    if cfg["prefetch"] and len(singles) >= 2:
        singles[0].set_modules_to_forward_prefetch([singles[1]])
        singles[-1].set_modules_to_backward_prefetch([singles[-2]])
    nosync = cfg["nosync"] and cfg["micro"] > 1
    if nosync:
        model._get_fsdp_state()._lazy_init(allow_no_grad_reduce=True)
    if cfg["adamw"]:
        from yafsdp_b200.optim import ShardedAdamW

        opt = ShardedAdamW(model, lr=0.01, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=0.5)
    else:
        opt = torch.optim.SGD([p for p in model.parameters() if p.requires_grad], lr=0.05)
    for it in range(2):
        opt.zero_grad()
        if cfg["explicit_unshard"] and it == 1:
            handle = model.emb.unshard(async_op=True)  # the first group the forward needs: an early, explicit gather
            if handle is not None:
                handle.wait()
        for m in range(cfg["micro"]):
            if nosync:
                model.set_requires_gradient_sync(m == cfg["micro"] - 1)
            (_loss(model, _ids(cfg, rank, m)) / cfg["micro"]).backward()
        opt.step()
        if cfg["state_dict_roundtrip"] and it == 0:
            sd = {k: v.clone() for k, v in model.state_dict().items()}
            with torch.no_grad():
                for q in model.parameters():
                    q.zero_()
            model.load_state_dict(sd)
        if cfg["eval_between"]:
            with torch.no_grad():
                got = model(_ids(cfg, rank, 7))
            assert torch.isfinite(got).all()
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p.full_tensor(), q.detach(), atol=2e-5), (seed, cfg, n)


def _many(rank, world, worker, seeds):
    for seed in seeds:  # several configurations per spawned world: process start-up dominates a single case
        worker(rank, world, seed)


@pytest.mark.timeout(400)
@pytest.mark.parametrize("seeds", [(0, 1, 2, 3), (4, 5, 6, 7), (13, 16, 28, 38)])
def test_random_model_matches_unsharded(seeds):
    run_distributed(_many, 3, _worker, seeds, timeout=380.0)


# ------------------------------------------------------------------------------------------------ class-style wrapper
def _config_v1(seed):
    cfg = _config(seed)
    rng = random.Random(seed + 77)
    cfg.update(tie=False, freeze=False, zero=rng.choice([1, 2, 3]), gas=rng.randint(1, 2), use_norm_cls=rng.random() < 0.6,
               hpz=rng.random() < 0.4, clip=rng.random() < 0.5)
    return cfg


def _v1_worker(rank, world, seed):
    import torch.distributed as dist
    from yafsdp_b200.compat_v1 import YaFSDP

    cfg = _config_v1(seed)
    ref = _build(cfg, seed)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    for _ in range(2):
        ref_opt.zero_grad()
        for r in range(world):
            for m in range(cfg["gas"]):
                (_loss(ref, _ids(cfg, r, m)) / (world * cfg["gas"])).backward()
        if cfg["clip"]:
            torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.3)
        ref_opt.step()
    model = _build(cfg, seed)
    intra = None
    if cfg["hpz"] and world == 4 and cfg["zero"] == 3:
        for lo in (0, 2):
            g = dist.new_group([lo, lo + 1])
            if rank // 2 == lo // 2:
                intra = g
    wrapped = YaFSDP(
        model, zero_stage=cfg["zero"], param_dtype=torch.float32,
        modules_to_wrap_with_names=[(model.emb, "emb")] + [(l, f"layers.{i}") for i, l in enumerate(model.layers)] + [(model.head, "head")],
        layer_norm_module_cls=nn.LayerNorm if cfg["use_norm_cls"] else None, gradient_accumulation_steps=cfg["gas"],
        rogue_layer_norm_modules_with_names={model.norm: "norm"}, comm_backend="torch",
        hpz_first_layers_num=2 if intra is not None else 0, intra_node_data_parallel_process_group=intra,
    )
    opt = torch.optim.SGD(list(wrapped.parameters()), lr=0.05)
    for _ in range(2):
        wrapped.zero_grad()
        for m in range(cfg["gas"]):
            _loss(wrapped, _ids(cfg, rank, m)).backward()  # the wrapper divides by the accumulation steps itself
        if cfg["clip"]:
            wrapped.clip_grad_norm_(0.3)
        opt.step()
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        full = p.full_tensor() if hasattr(p, "full_tensor") else p.detach()
        assert torch.allclose(full, q.detach(), atol=2e-5), (seed, cfg, n)


@pytest.mark.timeout(400)
@pytest.mark.parametrize("seeds,world", [((0, 3, 9), 4), ((1, 2, 4), 2)])
def test_random_v1_wrapper_matches_unsharded(seeds, world):
    run_distributed(_many, world, _v1_worker, seeds, timeout=380.0)


# ------------------------------------------------------------------------------------------------ pipeline-style schedules
def _microbatch_schedule_worker(rank, world, seed):
    """Hooks that external pipeline schedules use: ``set_is_last_backward``, unreduced accumulation
    (``set_requires_gradient_sync``) and parameters kept gathered between micro-batches (``set_reshard_after_backward``)."""
    from yafsdp_b200 import fully_shard

    cfg = _config(seed)
    cfg.update(tie=False, freeze=False, micro=3)
    ref = _build(cfg, seed)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    for _ in range(2):
        ref_opt.zero_grad()
        for r in range(world):
            for m in range(3):
                (_loss(ref, _ids(cfg, r, m)) / (world * 3)).backward()
        ref_opt.step()
    for variant in ("plain", "nosync", "keep", "keep+nosync"):
        model = _build(cfg, seed)
        kw = dict(reshard_after_forward=False) if "keep" in variant else {}
        fully_shard(model.emb, **kw)
        for l in model.layers:
            fully_shard(l, **kw)
        fully_shard([model.norm, model.head], **kw)
        fully_shard(model, **kw)
        if "nosync" in variant:
            model._get_fsdp_state()._lazy_init(allow_no_grad_reduce=True)
        opt = torch.optim.SGD(model.parameters(), lr=0.05)
        for _ in range(2):
            opt.zero_grad()
            for m in range(3):
                last = m == 2
                model.set_is_last_backward(last)
                if "nosync" in variant:
                    model.set_requires_gradient_sync(last)
                if "keep" in variant:
                    model.set_reshard_after_backward(last)
                (_loss(model, _ids(cfg, rank, m)) / 3).backward()
            opt.step()
        for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
            assert torch.allclose(p.full_tensor(), q.detach(), atol=2e-5), (variant, n)


@pytest.mark.timeout(300)
def test_micro_batch_schedule_hooks():
    run_distributed(_microbatch_schedule_worker, 2, 1, timeout=280.0)
