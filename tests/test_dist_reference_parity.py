"""This package beside the unmodified reference (``ya_fsdp`` installed under ``baseline/_ref``) on gloo, world 2.

Same model, same data, same stock optimizer in both: the losses, the number of all-gathers per step for the three
``reshard_after_forward`` settings, the number of rotating buffers and the on-disk checkpoint metadata
(``ya_fsdp/_tensor.py:365-432``) must agree, and a checkpoint written by the reference must load here.

The reference needs one shim to run on gloo at all: gloo's all-gather bumps the autograd version counter of its output
(NCCL does not), and the reference's rotating gather buffers are saved for backward, so the call is wrapped in
``torch.autograd._unsafe_preserve_version_counter``.  Nothing else of the reference is touched.  Skipped when the
reference is not installed.
"""

import os
import sys

import pytest
import torch

from dist_utils import run_distributed
from test_dist_features import _build, _data, _loss, _shard

_REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(_REF, "ya_fsdp")), reason="reference package not installed under baseline/_ref")


def _import_reference():
    import torch.distributed as dist

    if _REF not in sys.path:
        sys.path.insert(0, _REF)
    import ya_fsdp

    counter = {"all_gather": 0}
    if not getattr(dist, "_yf_test_shimmed", False):
        plain = dist.all_gather_into_tensor

        def shimmed(output_tensor, input_tensor, *a, **k):
            counter["all_gather"] += 1
            with torch.autograd._unsafe_preserve_version_counter(output_tensor):
                return plain(output_tensor, input_tensor, *a, **k)

        dist.all_gather_into_tensor = shimmed
        dist._yf_test_shimmed = True
        dist._yf_test_counter = counter
    return ya_fsdp, dist._yf_test_counter


def _shard_reference(ya_fsdp, model, **kw):
    ya_fsdp.fully_shard(model.emb, **kw)
    for l in model.layers:
        ya_fsdp.fully_shard(l, **kw)
    ya_fsdp.fully_shard([model.norm, model.head], **kw)
    ya_fsdp.fully_shard(model, **kw)
    return model


def _train(model, rank, steps=3):
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2, foreach=True)
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = _loss(model, _data(rank))
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses


def _parity_worker(rank, world, tmp):
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import FileSystemReader

    from yafsdp_b200 import checkpoint
    from yafsdp_b200.comm import backends

    ya_fsdp, ref_counter = _import_reference()
    own_counter = {"all_gather": 0}
    plain_ag = backends.TorchBackend.all_gather

    def counting_ag(self, out, inp, group):
        own_counter["all_gather"] += 1
        return plain_ag(self, out, inp, group)

    backends.TorchBackend.all_gather = counting_ag

    # ---- all-gathers per step and rotating buffers for the three settings (5 groups: embedding, 3 layers, norm + head)
    for setting, want_gathers, want_data_buffers in ((True, 8, 2), (False, 5, 5), (None, 10, 2)):
        ref = _shard_reference(ya_fsdp, _build(), reshard_after_forward=setting)
        own = _shard(_build(), reshard_after_forward=setting)
        _loss(ref, _data(rank)).backward()  # first step: lazy init
        _loss(own, _data(rank)).backward()
        ref_counter["all_gather"] = 0
        _loss(ref, _data(rank)).backward()
        assert ref_counter["all_gather"] == want_gathers, (setting, ref_counter)
        own_counter["all_gather"] = 0  # (this package's gloo path calls the same torch function: count it at its own layer)
        _loss(own, _data(rank)).backward()
        assert own_counter["all_gather"] == want_gathers, (setting, own_counter)
        ref_state, own_state = ref._get_fsdp_state(), own._get_fsdp_state()
        ref_bufs = {id(s._fsdp_param_group.data_buffer_ctx) for s in ref_state._state_ctx.all_states if s._fsdp_param_group is not None}
        assert len(ref_bufs) == want_data_buffers == len(own_state._data_ctxs), (setting, len(ref_bufs), len(own_state._data_ctxs))
        assert len(own_state._grad_ctxs) == 1

    # ---- three optimizer steps: same losses
    ref = _shard_reference(ya_fsdp, _build())
    own = _shard(_build())
    ref_losses, own_losses = _train(ref, rank), _train(own, rank)
    for a, b in zip(ref_losses, own_losses):
        assert abs(a - b) <= 1e-5 * max(1.0, abs(a)), (ref_losses, own_losses)

    # ---- checkpoints: same keys, same flat sizes, same chunk offsets and sizes
    ref_dir, own_dir = os.path.join(tmp, "ref"), os.path.join(tmp, "own")
    dcp.save({"model": ref.state_dict()}, checkpoint_id=ref_dir)
    checkpoint.save(own_dir, own)
    if rank == 0:
        md_ref = FileSystemReader(ref_dir).read_metadata().state_dict_metadata
        md_own = FileSystemReader(own_dir).read_metadata().state_dict_metadata
        keys = sorted(k for k in md_ref if k.startswith("model."))
        assert keys == sorted(k for k in md_own if k.startswith("model.")), (keys, sorted(md_own))
        for k in keys:
            a, b = md_ref[k], md_own[k]
            assert tuple(a.size) == tuple(b.size), k
            ca = sorted((tuple(c.offsets), tuple(c.sizes)) for c in a.chunks if int(c.sizes[0]) > 0)
            cb = sorted((tuple(c.offsets), tuple(c.sizes)) for c in b.chunks if int(c.sizes[0]) > 0)
            assert ca == cb, (k, ca, cb)
    # ---- the reference's checkpoint loads into this package's model (fresh init) and reproduces the reference's weights
    fresh = _shard(_build(seed=9))
    checkpoint.load(ref_dir, fresh)
    ref_params = dict(ref.named_parameters())
    for n, p in fresh.named_parameters():
        assert torch.equal(p._local_tensor.reshape(-1), ref_params[n]._local_tensor.reshape(-1)), n
    backends.TorchBackend.all_gather = plain_ag


@pytest.mark.timeout(300)
def test_matches_reference_on_gloo(tmp_path):
    run_distributed(_parity_worker, 2, str(tmp_path))
