"""Behavioural tests of the sharding API on CPU/gloo (world 2-3): accumulation modes, mixed precision, tied weights,
multi-module groups, ignored parameters, unshard/reshard, buffer sharing rules, gather counts, clipping, v1 wrapper."""

import pytest
import torch
import torch.nn as nn

from dist_utils import run_distributed


class Block(nn.Module):
    def __init__(self, d=16, h=24):
        super().__init__()
        self.a = nn.Linear(d, h)
        self.b = nn.Linear(h, d)

    def forward(self, x):
        return x + self.b(torch.relu(self.a(x)))


class Net(nn.Module):
    def __init__(self, n_layers=3, d=16, vocab=32, tie=False):
        super().__init__()
        self.emb = nn.Embedding(vocab, d)
        self.layers = nn.ModuleList([Block(d) for _ in range(n_layers)])
        self.norm = nn.LayerNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)
        if tie:
            self.head.weight = self.emb.weight

    def forward(self, ids):
        x = self.emb(ids)
        for l in self.layers:
            x = l(x)
        return self.head(self.norm(x))


def _build(seed=0, **kw):
    torch.manual_seed(seed)
    return Net(**kw)


def _shard(model, **kw):
    from yafsdp_b200 import fully_shard

    fully_shard(model.emb, **kw)
    for l in model.layers:
        fully_shard(l, **kw)
    fully_shard([model.norm, model.head], **kw)
    fully_shard(model, **kw)
    return model


def _data(rank, n=4, vocab=32):
    g = torch.Generator().manual_seed(100 + rank)
    return torch.randint(0, vocab, (n, 8), generator=g)


def _loss(model, ids):
    out = model(ids)
    return torch.nn.functional.cross_entropy(out.reshape(-1, out.shape[-1]).float(), ids.reshape(-1))


def _reference_params(world, steps, micro=1, lr=1e-2):
    model = _build()
    opt = torch.optim.SGD(model.parameters(), lr=lr)
    for _ in range(steps):
        opt.zero_grad()
        for r in range(world):
            for m in range(micro):
                (_loss(model, _data(r * 10 + m)) / (world * micro)).backward()
        opt.step()
    return {n: p.detach().clone() for n, p in model.named_parameters()}


def _check_params(model, want, atol=1e-5):
    for n, p in model.named_parameters():
        full = p.full_tensor() if hasattr(p, "full_tensor") else p.detach()
        assert torch.allclose(full, want[n], atol=atol), n


# ------------------------------------------------------------------------------------------------
def _accum_worker(rank, world, mode):
    model = _shard(_build())
    if mode == "nosync":
        model._get_fsdp_state()._lazy_init(allow_no_grad_reduce=True)
    opt = torch.optim.SGD(model.parameters(), lr=1e-2)
    micro = 3
    for _ in range(2):
        opt.zero_grad()
        for m in range(micro):
            if mode == "nosync":
                model.set_requires_gradient_sync(m == micro - 1)
            (_loss(model, _data(rank * 10 + m)) / micro).backward()
            if mode == "nosync" and m < micro - 1:
                assert all(p.grad is None for p in model.parameters())
        opt.step()
    _check_params(model, _reference_params(world, 2, micro))


@pytest.mark.timeout(180)
@pytest.mark.parametrize("mode", ["reduce_every_microbatch", "nosync"])
def test_gradient_accumulation(mode):
    run_distributed(_accum_worker, 2, mode)


def _nosync_default_raises_worker(rank, world):
    model = _shard(_build())
    model.set_requires_gradient_sync(False)
    with pytest.raises(AssertionError, match="share a grad buffer"):
        _loss(model, _data(rank))


@pytest.mark.timeout(120)
def test_nosync_needs_own_grad_buffers():
    run_distributed(_nosync_default_raises_worker, 2)


# ------------------------------------------------------------------------------------------------
def _mp_worker(rank, world):
    from yafsdp_b200 import MixedPrecisionPolicy, RaggedShardDTensor

    pol = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32, output_dtype=torch.float32, cast_forward_inputs=True)
    model = _shard(_build(), mp_policy=pol)
    out = model(_data(rank))
    assert out.dtype == torch.float32
    pass
    _loss(model, _data(rank)).backward()
    for p in model.parameters():
        assert isinstance(p, RaggedShardDTensor) and p.dtype == torch.float32
        assert isinstance(p.grad, RaggedShardDTensor) and p.grad.dtype == torch.float32 and p.grad.shape == p.shape
    g = model.layers[0]._get_fsdp_state()._param_group
    assert g.all_gather_dtype == torch.bfloat16 and g.reduce_scatter_dtype == torch.float32
    assert g.gather_input.dtype == torch.bfloat16


@pytest.mark.timeout(120)
def test_mixed_precision_dtypes():
    run_distributed(_mp_worker, 2)


# ------------------------------------------------------------------------------------------------
def _tied_ignored_worker(rank, world):
    from yafsdp_b200 import RaggedShardDTensor, fully_shard

    # tied weights inside one group + an ignored parameter that stays a plain replicated tensor
    model = _build(tie=True)
    ignored = {model.norm.bias}
    # the tied group is active from the first to the last module of the forward, so it must not rotate a buffer with the
    # layers: nobody reshards after forward -> every group gets its own data buffer
    fully_shard([model.emb, model.norm, model.head], ignored_params=ignored, reshard_after_forward=False)
    for l in model.layers:
        fully_shard(l, reshard_after_forward=False)
    fully_shard(model, reshard_after_forward=False)
    assert model.head.weight is model.emb.weight and isinstance(model.emb.weight, RaggedShardDTensor)
    assert not isinstance(model.norm.bias, RaggedShardDTensor)
    opt = torch.optim.SGD([p for p in model.parameters() if isinstance(p, RaggedShardDTensor)], lr=1e-2)
    _loss(model, _data(rank)).backward()
    assert model.emb.weight.grad is not None and model.norm.bias.grad is not None
    opt.step()
    # reference (tied, unsharded, averaged over ranks)
    ref = _build(tie=True)
    ropt = torch.optim.SGD([p for n, p in ref.named_parameters() if n != "norm.bias"], lr=1e-2)
    for r in range(world):
        (_loss(ref, _data(r)) / world).backward()
    ropt.step()
    assert torch.allclose(model.emb.weight.full_tensor(), ref.emb.weight, atol=1e-5)
    assert torch.allclose(model.layers[1].a.weight.full_tensor(), ref.layers[1].a.weight, atol=1e-5)


@pytest.mark.timeout(120)
def test_tied_weights_multi_module_group_and_ignored_params():
    run_distributed(_tied_ignored_worker, 2)


# ------------------------------------------------------------------------------------------------
def _unshard_api_worker(rank, world):
    from yafsdp_b200 import RaggedShardDTensor, UnshardHandle

    model = _shard(_build())
    ref = _build()
    layer = model.layers[1]
    assert isinstance(layer.a.weight, RaggedShardDTensor)
    assert layer.unshard() is None
    assert not isinstance(layer.a.weight, RaggedShardDTensor) and torch.allclose(layer.a.weight, ref.layers[1].a.weight)
    layer.reshard()
    assert isinstance(layer.a.weight, RaggedShardDTensor)
    h = model.layers[2].unshard(async_op=True)
    assert isinstance(h, UnshardHandle)
    h.wait()
    assert torch.allclose(model.layers[2].b.bias, ref.layers[2].b.bias)
    # layers 0 and 2 share a data buffer: gathering both at once must be refused
    with pytest.raises(RuntimeError, match="still owned"):
        model.layers[0].unshard()
    model.layers[2].reshard()
    with torch.no_grad():
        out = model(_data(rank))
    assert torch.allclose(out, ref(_data(rank)), atol=1e-5)
    assert all(isinstance(p, RaggedShardDTensor) for p in model.parameters())  # no-grad forward releases everything
    with pytest.raises(AssertionError):
        import copy

        copy.deepcopy(model)
    sd = model.state_dict()
    assert set(sd) == set(ref.state_dict()) and all(isinstance(v, RaggedShardDTensor) for v in sd.values())


@pytest.mark.timeout(120)
def test_unshard_reshard_api_state_dict_keys():
    run_distributed(_unshard_api_worker, 2)


# ------------------------------------------------------------------------------------------------
def _count_worker(rank, world, rarf, expect_gathers, expect_data_buffers):
    from yafsdp_b200.comm.backends import TorchBackend

    calls = []
    orig = TorchBackend.all_gather

    def counting(self, out, inp, group):
        calls.append(1)
        return orig(self, out, inp, group)

    TorchBackend.all_gather = counting
    try:
        model = _shard(_build(), reshard_after_forward=rarf)
        _loss(model, _data(rank)).backward()  # lazy init + first step
        calls.clear()
        _loss(model, _data(rank)).backward()
        state = model._get_fsdp_state()
        assert len(calls) == expect_gathers, len(calls)
        assert len(state._data_ctxs) == expect_data_buffers and len(state._grad_ctxs) == 1
    finally:
        TorchBackend.all_gather = orig


@pytest.mark.timeout(180)
@pytest.mark.parametrize("rarf,gathers,buffers", [(True, 8, 2), (False, 5, 5), (None, 10, 2)])
def test_all_gather_counts_and_buffer_counts(rarf, gathers, buffers):
    """5 groups (embedding, 3 layers, norm+head): default -> 5 forward + 3 backward gathers over 2 buffers (the last user of each
    buffer stays gathered); nobody reshards -> 5 gathers, one buffer each; auto mode off -> 10 gathers."""
    run_distributed(_count_worker, 2, rarf, gathers, buffers)


# ------------------------------------------------------------------------------------------------
def _clip_worker(rank, world):
    model = _shard(_build())
    _loss(model, _data(rank)).backward()
    ref = _build()
    for r in range(world):
        (_loss(ref, _data(r)) / world).backward()
    want = torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.05)
    got = torch.nn.utils.clip_grad_norm_(model.parameters(), 0.05, foreach=True)
    got = got.full_tensor() if hasattr(got, "full_tensor") else got
    assert torch.allclose(got, want, atol=1e-5), (got, want)
    assert torch.allclose(model.layers[0].a.weight.grad.full_tensor(), ref.layers[0].a.weight.grad, atol=1e-6)


@pytest.mark.timeout(120)
def test_torch_clip_grad_norm_on_sharded_grads():
    run_distributed(_clip_worker, 3)


# ------------------------------------------------------------------------------------------------
def _v1_worker(rank, world):
    from yafsdp_b200.compat_v1 import YaFSDP

    model = _build()
    wrapped = YaFSDP(
        model, zero_stage=3, param_dtype=torch.float32,
        modules_to_wrap_with_names=[(model.emb, "emb")] + [(l, f"layers.{i}") for i, l in enumerate(model.layers)] + [(model.head, "head")],
        layer_norm_module_cls=nn.LayerNorm, gradient_accumulation_steps=1,
        rogue_layer_norm_modules_with_names={model.norm: "norm"}, comm_backend="torch",
    )
    assert wrapped.layers is model.layers  # attribute passthrough
    params = list(wrapped.parameters())
    assert all(p.dim() == 1 for p in params) and len(params) == 6  # one flat parameter per group
    opt = torch.optim.SGD(params, lr=1e-2)
    with pytest.raises(ValueError):
        wrapped.zero_grad(set_to_none=True)
    for _ in range(2):
        wrapped.zero_grad()
        _loss(wrapped, _data(rank * 10)).backward()
        opt.step()
    _check_params(model, _reference_params(world, 2, 1))
    n = wrapped.clip_grad_norm_(1e-3)
    assert n.item() > 0
    local = wrapped.local_state_dict()
    assert "main_parameter" in local and "layernorm_parameter" in local and (("meta" in local) == (rank == 0))
    if rank == 0:
        assert "main_parameter_shard_bounaries" in local["meta"] and len(local["meta"]["main_shards_fqns"]) == 5
        assert local["meta"]["layernorm_fqns"] == [["norm.weight", "norm.bias"]]
    full = wrapped.state_dict()
    if rank == 0:
        assert set(full) == set(_build().state_dict()) and full["emb.weight"].shape == (32, 16)
    else:
        assert full == {}
    before = [p.detach().clone() for p in params]
    with torch.no_grad():
        for p in params:
            p.zero_()
    wrapped.load_state_dict(local)
    assert all(torch.equal(a, b) for a, b in zip(before, params))


@pytest.mark.timeout(180)
def test_v1_class_wrapper():
    run_distributed(_v1_worker, 2)


# ------------------------------------------------------------------------------------------------
def _mp_refresh_worker(rank, world):
    """Mixed precision with a stock torch optimizer: the bf16 gather input follows the fp32 master after every step."""
    from yafsdp_b200 import MixedPrecisionPolicy

    pol = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32, cast_forward_inputs=True)
    model = _shard(_build(), mp_policy=pol)
    opt = torch.optim.AdamW(model.parameters(), lr=5e-2, foreach=True)
    losses = []
    for _ in range(4):
        opt.zero_grad()
        loss = _loss(model, _data(rank))
        loss.backward()
        opt.step()
        losses.append(loss.item())
        for m in [model.emb, *model.layers]:
            g = m._get_fsdp_state()._param_group
            g.unshard(); g.wait_for_unshard(); g.reshard()  # a gather right after the step must see the new weights
            assert torch.equal(g.gather_input, g.master_flat.to(torch.bfloat16)), "stale compute-dtype copy after optimizer step"
    assert losses[-1] < losses[0]


@pytest.mark.timeout(120)
def test_mixed_precision_gather_input_follows_torch_optimizer():
    run_distributed(_mp_refresh_worker, 2)


# ------------------------------------------------------------------------------------------------
def _prefetch_api_worker(rank, world):
    """Explicit prefetch lists, post-optimizer event, divide factor, forced-sum reduction: same numbers as the defaults."""
    model = _shard(_build())
    layers = list(model.layers)
    for i, l in enumerate(layers[:-1]):
        l.set_modules_to_forward_prefetch([layers[i + 1]])
    for i, l in enumerate(layers[1:], start=1):
        l.set_modules_to_backward_prefetch([layers[i - 1]])
    with pytest.raises(ValueError):
        layers[0].set_modules_to_forward_prefetch([nn.Linear(2, 2)])
    model.set_force_sum_reduction_for_comms(True)
    model.set_post_optim_event(None)
    model.set_is_last_backward(True)
    opt = torch.optim.SGD(model.parameters(), lr=1e-2)
    for _ in range(2):
        opt.zero_grad()
        _loss(model, _data(rank * 10)).backward()
        opt.step()
    _check_params(model, _reference_params(world, 2, 1))
    # a custom divide factor rescales the reduced gradient
    model2 = _shard(_build())
    model2.set_gradient_divide_factor(float(world * 4))
    _loss(model2, _data(rank * 10)).backward()
    ref = _build()
    for r in range(world):
        (_loss(ref, _data(r * 10)) / (world * 4)).backward()
    assert torch.allclose(model2.layers[0].a.weight.grad.full_tensor(), ref.layers[0].a.weight.grad, atol=1e-6)


@pytest.mark.timeout(180)
def test_prefetch_lists_and_reduction_knobs():
    run_distributed(_prefetch_api_worker, 2)


# ------------------------------------------------------------------------------------------------
def _hpz_worker(rank, world):
    """Hierarchical partitioning: the first layers gather their weights for backward inside a 2-rank group."""
    import torch.distributed as dist
    from yafsdp_b200.comm import backends
    from yafsdp_b200.compat_v1 import YaFSDP

    intra = None
    for lo in range(0, world, 2):
        g = dist.new_group([lo, lo + 1])
        if rank // 2 == lo // 2:
            intra = g
    sizes = []
    orig = backends.TorchBackend.all_gather

    def spy(self, out, inp, group):
        sizes.append(1 if group is None else group.size())
        return orig(self, out, inp, group)

    backends.TorchBackend.all_gather = spy
    model = _build()
    wrapped = YaFSDP(
        model, zero_stage=3, param_dtype=torch.float32,
        modules_to_wrap_with_names=[(l, f"layers.{i}") for i, l in enumerate(model.layers)] + [(model.emb, "emb"), (model.head, "head")],
        gradient_accumulation_steps=1, rogue_layer_norm_modules_with_names={model.norm: "norm"}, comm_backend="torch",
        hpz_first_layers_num=2, intra_node_data_parallel_process_group=intra,
    )
    opt = torch.optim.SGD(list(wrapped.parameters()), lr=1e-2)
    for step in range(2):
        sizes.clear()
        wrapped.zero_grad()
        _loss(wrapped, _data(rank * 10)).backward()
        opt.step()
        # forward: 6 gathers over the whole group; backward: layers 0 and 1 inside the pair, the last-used groups stay gathered
        assert sizes.count(2) == 2, sizes
        assert sizes.count(world) >= 6, sizes
    _check_params(model, _reference_params(world, 2, 1))


@pytest.mark.timeout(240)
def test_hierarchical_partitioning_secondary_shards():
    run_distributed(_hpz_worker, 4)


# ------------------------------------------------------------------------------------------------
class NormBlock(nn.Module):
    def __init__(self, d=16, h=24):
        super().__init__()
        self.ln = nn.LayerNorm(d)
        self.a = nn.Linear(d, h)
        self.b = nn.Linear(h, d)

    def forward(self, x):
        return x + self.b(torch.relu(self.a(self.ln(x))))


class NormNet(Net):
    def __init__(self, n_layers=3, d=16, vocab=32):
        super().__init__(n_layers, d, vocab)
        self.layers = nn.ModuleList([NormBlock(d) for _ in range(n_layers)])


def _norm_net(seed=0):
    torch.manual_seed(seed)
    return NormNet()


def _v1_norm_group_worker(rank, world):
    """All norm weights form one group (gathered once per step, own buffers); inference mode keeps no gradient buffers."""
    from yafsdp_b200.comm import backends
    from yafsdp_b200.compat_v1 import YaFSDP
    from yafsdp_b200.optim import param_groups_of

    def wrap(model, **kw):
        return YaFSDP(
            model, zero_stage=3, param_dtype=torch.float32,
            modules_to_wrap_with_names=[(model.emb, "emb")] + [(l, f"layers.{i}") for i, l in enumerate(model.layers)] + [(model.head, "head")],
            layer_norm_module_cls=nn.LayerNorm, gradient_accumulation_steps=1,
            rogue_layer_norm_modules_with_names={model.norm: "norm"}, comm_backend="torch", **kw,
        )

    ref = _norm_net()
    ref_opt = torch.optim.SGD(ref.parameters(), lr=1e-2)
    for _ in range(2):
        ref_opt.zero_grad()
        for r in range(world):
            (_loss(ref, _data(r * 10)) / world).backward()
        ref_opt.step()

    model = _norm_net()
    wrapped = wrap(model)
    groups = param_groups_of(model)
    norm_groups = [g for g in groups if getattr(g, "is_norm_group", False)]
    assert len(norm_groups) == 1 and len(norm_groups[0].params) == 2 * 4 and len(groups) == 6
    gathers = []
    orig = backends.TorchBackend.all_gather

    def spy(self, out, inp, group):
        gathers.append(out.numel())
        return orig(self, out, inp, group)

    backends.TorchBackend.all_gather = spy
    params = list(wrapped.parameters())
    opt = torch.optim.SGD(params, lr=1e-2)
    for _ in range(2):
        gathers.clear()
        wrapped.zero_grad()
        _loss(wrapped, _data(rank * 10)).backward()
        opt.step()
        assert gathers.count(norm_groups[0].layout.padded_numel) == 1, gathers  # the norm group is gathered once per step
    backends.TorchBackend.all_gather = orig
    _check_params(model, {n: p.detach() for n, p in ref.named_parameters()})
    local = wrapped.local_state_dict()
    assert local["layernorm_parameter"].numel() == norm_groups[0].layout.shard_numel
    if rank == 0:
        assert local["meta"]["layernorm_fqns"][0][0] == "layers.0.ln.weight" and len(local["meta"]["main_shards_fqns"]) == 5
    before = [p.detach().clone() for p in params]
    with torch.no_grad():
        for p in params:
            p.zero_()
    wrapped.load_state_dict(local)
    assert all(torch.equal(a, b) for a, b in zip(before, params))

    # ---- inference mode
    frozen = _norm_net()
    want = frozen(_data(rank))
    inf = wrap(frozen, is_trainable=False)
    with torch.no_grad():
        got = inf(_data(rank))
    assert torch.allclose(got, want, atol=1e-6)
    state = frozen._get_fsdp_state()
    assert all(ctx.tensor is None for ctx in state._grad_ctxs)
    assert all(not p.requires_grad for p in inf.parameters())


@pytest.mark.timeout(240)
def test_v1_norm_group_and_inference_mode():
    run_distributed(_v1_norm_group_worker, 2)


# ------------------------------------------------------------------------------------------------
def _v1_model_parallel_worker(rank, world):
    """2 data-parallel x 2 model-parallel ranks: norm gradients are summed over the model-parallel group after the
    data-parallel reduction; the clipping norm is taken over both groups."""
    import torch.distributed as dist
    from yafsdp_b200.compat_v1 import YaFSDP
    from yafsdp_b200.optim import param_groups_of

    dp = mp = None
    for ranks in ([0, 1], [2, 3]):
        g = dist.new_group(ranks)
        if rank in ranks:
            dp = g
    for ranks in ([0, 2], [1, 3]):
        g = dist.new_group(ranks)
        if rank in ranks:
            mp = g
    model = _norm_net()
    wrapped = YaFSDP(
        model, zero_stage=3, param_dtype=torch.float32,
        modules_to_wrap_with_names=[(model.emb, "emb")] + [(l, f"layers.{i}") for i, l in enumerate(model.layers)] + [(model.head, "head")],
        layer_norm_module_cls=nn.LayerNorm, gradient_accumulation_steps=1, rogue_layer_norm_modules_with_names={model.norm: "norm"},
        data_parallel_process_group=dp, model_parallel_process_group=mp, all_reduce_grads_across_model_parallel_group=True,
        comm_backend="torch",
    )
    list(wrapped.parameters())
    wrapped.zero_grad()
    _loss(wrapped, _data(rank * 10)).backward()

    ref = _norm_net()
    grads = []
    for r in range(world):
        ref.zero_grad()
        _loss(ref, _data(r * 10)).backward()
        grads.append({n: p.grad.clone() for n, p in ref.named_parameters()})
    my_dp = [0, 1] if rank < 2 else [2, 3]
    for n, p in model.named_parameters():
        got = p.grad.full_tensor()
        if ".ln." in n or n.startswith("norm."):
            want = sum(grads[r][n] for r in range(world)) / 2  # mean over each data-parallel pair, summed over the pairs
        else:
            want = sum(grads[r][n] for r in my_dp) / 2
        assert torch.allclose(got, want, atol=1e-6), n
    local_sq = sum(g.sharded_grad_flat.double().pow(2).sum() for g in param_groups_of(model))
    tot = torch.tensor([float(local_sq)], dtype=torch.float64)
    dist.all_reduce(tot)
    norm = wrapped.clip_grad_norm_(1e9)
    assert abs(norm.item() - tot.sqrt().item()) < 1e-4 * tot.sqrt().item()


@pytest.mark.timeout(240)
def test_v1_norm_gradients_summed_over_model_parallel_group():
    run_distributed(_v1_model_parallel_worker, 4)


# ------------------------------------------------------------------------------------------------
def _clip_variants_worker(rank, world):
    """torch's gradient clipping on sharded gradients for the 1-, 2- and infinity-norm (ranks may hold no element of a
    parameter) and by value."""
    for norm_type in (1.0, 2.0, float("inf")):
        ref = _build()
        for r in range(world):
            (_loss(ref, _data(r)) / world).backward()
        want = torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.05, norm_type=norm_type)
        model = _shard(_build())
        _loss(model, _data(rank)).backward()
        got = torch.nn.utils.clip_grad_norm_(model.parameters(), 0.05, norm_type=norm_type)
        got = got.full_tensor() if hasattr(got, "full_tensor") else got
        assert torch.allclose(got, want, rtol=1e-5), (norm_type, got, want)
        for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
            assert torch.allclose(p.grad.full_tensor(), q.grad, atol=1e-6), (norm_type, n)
    ref = _build()
    for r in range(world):
        (_loss(ref, _data(r)) / world).backward()
    torch.nn.utils.clip_grad_value_(ref.parameters(), 0.002)
    model = _shard(_build())
    _loss(model, _data(rank)).backward()
    torch.nn.utils.clip_grad_value_(model.parameters(), 0.002)
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p.grad.full_tensor(), q.grad, atol=1e-7), n


@pytest.mark.timeout(180)
def test_torch_clipping_variants_on_sharded_grads():
    run_distributed(_clip_variants_worker, 3)


# ------------------------------------------------------------------------------------------------
def _apply_after_forward_worker(rank, world):
    """``module.to(dtype)`` / ``.float()`` / ``.double()`` after the first forward: the sharded storage keeps its dtype and
    takes over the transformed values (as the reference does), and training continues."""
    model = _shard(_build())
    opt = torch.optim.SGD(model.parameters(), lr=1e-2)
    _loss(model, _data(rank)).backward()
    opt.step()
    before = {n: p.full_tensor().clone() for n, p in model.named_parameters()}
    model.double()  # a no-op on the values; the parameters stay float32 RaggedShardDTensors bound to the same storage
    for n, p in model.named_parameters():
        assert p.dtype == torch.float32 and torch.equal(p.full_tensor(), before[n]), n
    model.to(torch.bfloat16)  # values go through bfloat16 and come back rounded
    for n, p in model.named_parameters():
        assert p.dtype == torch.float32
        assert torch.equal(p.full_tensor(), before[n].to(torch.bfloat16).float()), n
    # the optimizer still holds the registered parameters and the next gather uses the new values
    opt.zero_grad()
    _loss(model, _data(rank)).backward()
    opt.step()
    ref = _build()
    with torch.no_grad():
        for n, p in ref.named_parameters():
            p.copy_(before[n].to(torch.bfloat16).float())
    ropt = torch.optim.SGD(ref.parameters(), lr=1e-2)
    for r in range(world):
        (_loss(ref, _data(r)) / world).backward()
    ropt.step()
    _check_params(model, {n: p.detach() for n, p in ref.named_parameters()})


@pytest.mark.timeout(180)
def test_module_apply_after_first_forward():
    run_distributed(_apply_after_forward_worker, 2)


# ------------------------------------------------------------------------------------------------
def _clip_with_plain_param_worker(rank, world):
    """``clip_grad_norm_`` of this package with an ignored (replicated, unsharded) parameter beside sharded ones: the
    plain gradient is whole on every rank and must enter the total once, not once per rank."""
    from yafsdp_b200 import fully_shard
    from yafsdp_b200.optim import clip_grad_norm_

    ref = _build()
    for r in range(world):
        (_loss(ref, _data(r)) / world).backward()
    want = torch.nn.utils.clip_grad_norm_(ref.parameters(), 1e9)
    model = _build()
    ignored = {model.norm.weight, model.norm.bias}
    fully_shard(model.emb)
    for l in model.layers:
        fully_shard(l)
    fully_shard(model.head)
    fully_shard(model, ignored_params=ignored)  # the root itself manages nothing: the norm's parameters stay plain
    _loss(model, _data(rank)).backward()
    # data-parallel average of the replicated parameters' gradients is the user's job
    import torch.distributed as dist

    for p in ignored:
        dist.all_reduce(p.grad)
        p.grad /= world
    got = clip_grad_norm_(model, 1e9)
    assert torch.allclose(got, want, rtol=1e-5), (got, want)


@pytest.mark.timeout(180)
def test_clip_grad_norm_counts_plain_gradients_once():
    run_distributed(_clip_with_plain_param_worker, 2)
