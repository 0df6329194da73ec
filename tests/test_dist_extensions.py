"""All-gather tensor extensions: a parameter class that travels as int8 (quantised shard + scale metadata) and is
dequantised after the gather."""

import pytest
import torch
import torch.nn as nn

from dist_utils import run_distributed

SCALE = 1.0 / 64


class Int8Weight(torch.Tensor):
    """Plain-storage tensor subclass: fp32 master values, gathered as int8 with a fixed scale."""

    calls = {"pre": 0, "post": 0}

    def fsdp_pre_all_gather(self, mesh):
        Int8Weight.calls["pre"] += 1
        q = torch.clamp(torch.round(self.as_subclass(torch.Tensor) / SCALE), -127, 127).to(torch.int8)
        return (q,), {"scale": SCALE}

    def fsdp_post_all_gather(self, all_gather_outputs, metadata, param_dtype, *, out=None):
        Int8Weight.calls["post"] += 1
        (q,) = all_gather_outputs
        deq = q.to(param_dtype) * metadata["scale"]
        if out is not None:
            out.copy_(deq)
            return None
        return deq, (q,)


def _worker(rank, world):
    from yafsdp_b200 import MixedPrecisionPolicy, RaggedShardDTensor, fully_shard

    torch.manual_seed(0)
    lin = nn.Linear(24, 16, bias=False)
    full = lin.weight.detach().clone()
    lin.weight = nn.Parameter(lin.weight.data.as_subclass(Int8Weight))
    norm = nn.LayerNorm(24)
    model = nn.Sequential(norm, lin)
    policy = MixedPrecisionPolicy(all_gather_dtype_to_param_cls={torch.int8: Int8Weight})
    fully_shard(lin, mp_policy=policy)
    fully_shard(norm)
    fully_shard(model)
    g = lin._get_fsdp_state()._param_group
    assert g.all_gather_dtype == torch.int8 and isinstance(lin.weight, RaggedShardDTensor)
    x = torch.randn(4, 24, generator=torch.Generator().manual_seed(5 + rank))
    out = model(x)
    want_w = torch.clamp(torch.round(full / SCALE), -127, 127) * SCALE  # every rank computes with the dequantised weight
    ref = nn.functional.linear(nn.functional.layer_norm(x, (24,)), want_w)
    assert torch.allclose(out, ref, atol=1e-5)
    assert g.gather_input.dtype == torch.int8 and g.gather_input.numel() == g.layout.shard_numel
    out.sum().backward()
    assert isinstance(lin.weight.grad, RaggedShardDTensor) and lin.weight.grad.dtype == torch.float32
    # the master stays fp32 and trainable; a second step re-quantises the updated shard and refreshes in place
    with torch.no_grad():
        lin.weight._local_tensor.add_(0.5)
    pre, post = Int8Weight.calls["pre"], Int8Weight.calls["post"]
    out2 = model(x)
    assert Int8Weight.calls["pre"] == pre + 1 and Int8Weight.calls["post"] > post, (pre, post, Int8Weight.calls, g._is_unsharded, type(lin.weight))
    want_w2 = torch.clamp(torch.round((full + 0.5) / SCALE), -127, 127) * SCALE
    assert torch.allclose(out2, nn.functional.linear(nn.functional.layer_norm(x, (24,)), want_w2), atol=1e-5)


def _mixed_worker(rank, world):
    """Extension and ordinary parameters under ONE fully_shard call: one group per all-gather dtype, side by side in the
    shared buffers, trained like the unsharded (quantising) model."""
    from yafsdp_b200 import MixedPrecisionPolicy, fully_shard
    from yafsdp_b200.group import GroupSet
    from yafsdp_b200.optim import param_groups_of

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.norm = nn.LayerNorm(24)
            self.lin = nn.Linear(24, 24)

        def forward(self, x):
            return x + self.lin(self.norm(x))

    def build():
        torch.manual_seed(0)
        return nn.Sequential(Block(), Block(), nn.Linear(24, 8))

    policy = MixedPrecisionPolicy(all_gather_dtype_to_param_cls={torch.int8: Int8Weight})
    model = build()
    for blk in (model[0], model[1]):
        blk.lin.weight = nn.Parameter(blk.lin.weight.data.as_subclass(Int8Weight))
        fully_shard(blk, mp_policy=policy)
    fully_shard(model[2], mp_policy=policy)
    fully_shard(model, mp_policy=policy)
    gs = model[0]._get_fsdp_state()._param_group
    assert isinstance(gs, GroupSet) and [g.all_gather_dtype for g in gs.groups] == [torch.float32, torch.int8]
    assert len(gs.params) == 4 and len(param_groups_of(model)) == 5

    def quantise(w):
        return torch.clamp(torch.round(w / SCALE), -127, 127) * SCALE

    ref = build()
    x_all = [torch.randn(4, 24, generator=torch.Generator().manual_seed(5 + r)) for r in range(world)]
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.1)
    for _ in range(3):
        opt.zero_grad()
        model(x_all[rank]).pow(2).mean().backward()
        opt.step()
        # reference: forward with the quantised weights (straight-through: the gradient goes to the fp32 master)
        ref_opt.zero_grad()
        for r in range(world):
            h = x_all[r]
            for blk in (ref[0], ref[1]):
                w = blk.lin.weight + (quantise(blk.lin.weight) - blk.lin.weight).detach()
                h = h + nn.functional.linear(blk.norm(h), w, blk.lin.bias)
            (ref[2](h).pow(2).mean() / world).backward()
        ref_opt.step()
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p.full_tensor(), q.detach(), atol=1e-5), n
    # state dict keys and shapes are those of the plain model
    sd = model.state_dict()
    assert set(sd) == set(ref.state_dict()) and sd["0.lin.weight"].shape == (24, 24)


@pytest.mark.timeout(120)
def test_all_gather_extension_int8():
    run_distributed(_worker, 2)


@pytest.mark.timeout(180)
def test_extension_and_ordinary_parameters_in_one_module():
    run_distributed(_mixed_worker, 2)


class ScaledWeight(torch.Tensor):
    """Wrapper tensor subclass (inner tensors, ``__tensor_flatten__``): fp32 values in ``_data`` plus a per-tensor
    ``_scale``; travels as int8 like ``Int8Weight``.  Only what sharding needs is dispatched: detach, new_zeros, to."""

    @staticmethod
    def __new__(cls, data, scale):
        return torch.Tensor._make_wrapper_subclass(cls, data.shape, dtype=data.dtype, device=data.device, requires_grad=False)

    def __init__(self, data, scale):
        self._data = data
        self._scale = scale

    def __tensor_flatten__(self):
        return ["_data", "_scale"], None

    @staticmethod
    def __tensor_unflatten__(inner, meta, outer_size, outer_stride):
        return ScaledWeight(inner["_data"], inner["_scale"])

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        aten = torch.ops.aten
        self = args[0]
        if func in (aten.detach.default, aten.alias.default):
            return ScaledWeight(self._data.detach(), self._scale)
        if func is aten.new_zeros.default:
            return ScaledWeight(self._data.new_zeros(*args[1:], **kwargs), self._scale)
        if func in (aten._to_copy.default,):
            return ScaledWeight(func(self._data, *args[1:], **kwargs), self._scale)
        raise NotImplementedError(f"ScaledWeight: {func}")

    __torch_function__ = torch._C._disabled_torch_function_impl

    def fsdp_pre_all_gather(self, mesh):
        q = torch.clamp(torch.round(self._data / self._scale), -127, 127).to(torch.int8)
        return (q,), {"scale": self._scale}

    def fsdp_post_all_gather(self, all_gather_outputs, metadata, param_dtype, *, out=None):
        (q,) = all_gather_outputs
        deq = q.to(param_dtype) * metadata["scale"]
        if out is not None:
            out.copy_(deq)
            return None
        return deq, (q,)


def _wrapper_worker(rank, world):
    """A parameter whose tensor is a wrapper subclass with inner tensors: the hooks run on a local wrapper whose first
    inner tensor is the master shard, so optimizer updates of the shard reach the next gather."""
    from yafsdp_b200 import MixedPrecisionPolicy, RaggedShardDTensor, fully_shard

    torch.manual_seed(0)
    lin = nn.Linear(24, 16, bias=False)
    full = lin.weight.detach().clone()
    lin.weight = nn.Parameter(ScaledWeight(lin.weight.data.clone(), torch.tensor(SCALE)))
    norm = nn.LayerNorm(24)
    model = nn.Sequential(norm, lin)
    policy = MixedPrecisionPolicy(all_gather_dtype_to_param_cls={torch.int8: ScaledWeight})
    fully_shard(lin, mp_policy=policy)
    fully_shard(norm)
    fully_shard(model)
    g = lin._get_fsdp_state()._param_group
    assert g.all_gather_dtype == torch.int8 and isinstance(lin.weight, RaggedShardDTensor)
    x = torch.randn(4, 24, generator=torch.Generator().manual_seed(5 + rank))

    def quantise(w):
        return torch.clamp(torch.round(w / SCALE), -127, 127) * SCALE

    out = model(x)
    assert torch.allclose(out, nn.functional.linear(nn.functional.layer_norm(x, (24,)), quantise(full)), atol=1e-5)
    out.sum().backward()
    assert isinstance(lin.weight.grad, RaggedShardDTensor)
    with torch.no_grad():
        lin.weight._local_tensor.add_(0.25)  # what an optimizer does: the wrapper's inner tensor sees it
    out2 = model(x)
    assert torch.allclose(out2, nn.functional.linear(nn.functional.layer_norm(x, (24,)), quantise(full + 0.25)), atol=1e-5)


@pytest.mark.timeout(180)
def test_wrapper_subclass_extension_parameter():
    run_distributed(_wrapper_worker, 2)
