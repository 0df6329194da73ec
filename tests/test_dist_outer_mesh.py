"""fully_shard composed with parameters that already are DTensors of an outer (expert-parallel style) mesh."""

import pytest
import torch
import torch.nn as nn

from dist_utils import run_distributed


class Experts(nn.Module):
    """E experts, each a [d, d] matrix; this rank applies the experts it holds to its own tokens."""

    def __init__(self, weight):
        super().__init__()
        self.weight = nn.Parameter(weight)

    def forward(self, x):
        from torch.distributed.tensor import DTensor

        w = self.weight
        if isinstance(w, DTensor):
            w = w.to_local()
        return sum(x @ w[e] for e in range(w.shape[0]))


def _worker(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import DTensor, Shard, distribute_tensor

    from yafsdp_b200 import RaggedShardDTensor, fully_shard

    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("ep", "fsdp"))
    ep_rank, fsdp_rank = mesh.get_local_rank("ep"), mesh.get_local_rank("fsdp")
    torch.manual_seed(0)
    full_w = torch.randn(4, 6, 6)  # 4 experts, 2 per ep rank
    model = Experts(distribute_tensor(full_w.clone(), mesh["ep"], [Shard(0)]))
    fully_shard(model, mesh=mesh["fsdp"])
    p = model.weight
    assert isinstance(p, RaggedShardDTensor) and tuple(p.shape) == (2, 6, 6)  # the piece this ep rank holds
    assert p._spec.outer_mesh is not None and p._spec.global_numel == 4 * 36
    assert torch.equal(p.full_tensor(), full_w)
    x = torch.randn(5, 6, generator=torch.Generator().manual_seed(10 + rank))
    out = model(x)
    out.sum().backward()
    g = model.weight.grad
    assert isinstance(g, RaggedShardDTensor) and tuple(g.shape) == (2, 6, 6)
    # expected: gradient of the local experts, averaged over the two fsdp ranks of this ep rank
    want_local = torch.zeros(2, 6, 6)
    for fr in range(2):
        r = ep_rank * 2 + fr
        xr = torch.randn(5, 6, generator=torch.Generator().manual_seed(10 + r))
        want_local += xr.sum(0)[:, None].expand(6, 6).unsqueeze(0).expand(2, 6, 6) / 2
    got_full = g.full_tensor()
    assert torch.allclose(got_full[ep_rank * 2 : ep_rank * 2 + 2], want_local, atol=1e-5)
    # DCP items address the full flat tensor: outer offset + ragged offset
    (item,) = model.weight.__create_write_items__("w", model.weight)
    assert tuple(item.tensor_data.size) == (144,)
    off = int(item.tensor_data.chunk.offsets[0])
    assert off == ep_rank * 72 + model.weight._spec.placement.global_offset


@pytest.mark.timeout(180)
def test_fully_shard_on_outer_mesh_dtensor_params():
    run_distributed(_worker, 4)
