"""RaggedShardDTensor: dispatch rules, random-init parity, copy_, DCP items (single process)."""

import pytest
import torch

from yafsdp_b200.tensor import RaggedShard, RaggedShardDTensor


def _make(full: torch.Tensor, world: int, rank: int):
    n = full.numel()
    per = -(-n // world)
    lo, hi = min(rank * per, n), min((rank + 1) * per, n)
    counts = tuple(max(0, min((r + 1) * per, n) - min(r * per, n)) for r in range(world))
    pl = RaggedShard(hi - lo, lo if hi > lo else n, counts)
    return RaggedShardDTensor.from_local(full.reshape(-1)[lo:hi].clone(), full.shape, pl)


def test_shape_is_logical_and_local_is_flat():
    full = torch.arange(32 * 16, dtype=torch.float32).view(32, 16)
    t = _make(full, 2, 1)
    assert t.shape == (32, 16) and t._local_tensor.shape == (256,)
    assert t.placements[0].global_offset == 256
    assert torch.equal(t.to_local(), full.reshape(-1)[256:])


def test_pointwise_foreach_and_single_tensor_optimizer_ops():
    full = torch.randn(10, 7)
    a = _make(full, 3, 1)
    b = _make(full * 2, 3, 1)
    c = a + b
    assert isinstance(c, RaggedShardDTensor) and torch.allclose(c._local_tensor, 3 * a._local_tensor)
    a2 = a.clone()
    a2.mul_(2).add_(b, alpha=0.5)
    assert torch.allclose(a2._local_tensor, 3 * a._local_tensor)
    torch._foreach_add_([a2], [b])
    torch._foreach_mul_([a2], 0.5)
    assert torch.allclose(a2._local_tensor, 2.5 * a._local_tensor)
    # ops of the single-tensor Adam path that the reference does not support
    m = torch.zeros_like(a)
    m.lerp_(b, 0.1)
    v = torch.zeros_like(a).addcmul_(b, b, value=0.01)
    a2.addcdiv_(m, v.sqrt().add_(1e-8), value=-1e-3)
    assert isinstance(m, RaggedShardDTensor) and isinstance(v, RaggedShardDTensor)
    z = a.new_zeros(a.shape)
    assert isinstance(z, RaggedShardDTensor) and z._local_tensor.numel() == a._local_tensor.numel()
    assert a.to(torch.bfloat16).dtype == torch.bfloat16


@pytest.mark.parametrize("opt_kwargs", [dict(foreach=True), dict(foreach=False), dict()])
def test_torch_optimizers_run_on_sharded_parameters(opt_kwargs):
    torch.manual_seed(0)
    full = torch.randn(13, 5)
    grads = torch.randn(13, 5)
    ref = torch.nn.Parameter(full.clone())
    ref.grad = grads.clone()
    torch.optim.AdamW([ref], lr=1e-2).step()
    for rank in range(3):
        p = torch.nn.Parameter(_make(full, 3, rank))
        p.grad = _make(grads, 3, rank)
        torch.optim.AdamW([p], lr=1e-2, **opt_kwargs).step()
        want = _make(ref.detach(), 3, rank)._local_tensor
        assert torch.allclose(p.detach()._local_tensor, want, atol=1e-6)


def test_random_init_equals_unsharded_init():
    full = torch.empty(33, 9)
    torch.manual_seed(5)
    full.normal_(0, 0.02)
    for rank in range(4):
        t = _make(torch.zeros(33, 9), 4, rank)
        torch.manual_seed(5)
        t.normal_(0, 0.02)
        assert torch.equal(t._local_tensor, _make(full, 4, rank)._local_tensor)


def test_copy_from_full_tensor_and_unsupported_op_message():
    full = torch.randn(6, 6)
    t = _make(torch.zeros(6, 6), 4, 2)
    t.copy_(full)
    assert torch.equal(t._local_tensor, _make(full, 4, 2)._local_tensor)
    with pytest.raises(NotImplementedError, match="full_tensor"):
        t @ t


def test_norm_without_mesh_is_local_norm_and_clip_helper():
    from yafsdp_b200.optim import clip_grad_norm_

    full = torch.randn(20, 3)
    p = torch.nn.Parameter(_make(full, 1, 0))
    p.grad = _make(full * 3, 1, 0)
    (n,) = torch._foreach_norm([p.grad], 2)
    assert torch.allclose(n, (full * 3).norm())
    total = clip_grad_norm_([p], 1.0)
    assert torch.allclose(total, (full * 3).norm())
    assert torch.allclose(p.grad._local_tensor.norm(), torch.tensor(1.0), atol=1e-4)


def test_dcp_write_item_is_flat_chunk():
    full = torch.randn(32, 16)
    t = _make(full, 2, 1)
    (item,) = t.__create_write_items__("w", t)
    assert tuple(item.tensor_data.size) == (512,)
    assert tuple(item.tensor_data.chunk.offsets) == (256,) and tuple(item.tensor_data.chunk.sizes) == (256,)
    (chunk,) = t.__create_chunk_list__()
    assert tuple(chunk.offsets) == (256,)
    empty = RaggedShardDTensor.from_local(torch.empty(0), (4, 4), RaggedShard(0, 16, (16, 0)))
    (item,) = empty.__create_write_items__("e", empty)
    assert tuple(item.tensor_data.chunk.offsets) == (16,) and tuple(item.tensor_data.chunk.sizes) == (0,)
