"""CPU/gloo plumbing run of the tiny Llama config: sharded training must reproduce an unsharded run."""

import pytest
import torch

from dist_utils import run_distributed


def _batch(rank: int, vocab: int = 1024):
    g = torch.Generator().manual_seed(1 + rank)
    ids = torch.randint(0, vocab, (2, 128), generator=g)
    return ids


def _unsharded_losses(world: int, steps: int):
    """Single process: average the per-rank losses / gradients exactly like data parallel does."""
    from yafsdp_b200.models.llama import CONFIGS, LlamaForCausalLM

    model = LlamaForCausalLM(CONFIGS["tiny"])
    model.init_weights(0)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, foreach=True)
    batches = [_batch(r) for r in range(world)]
    out = []
    for _ in range(steps):
        opt.zero_grad()
        losses = []
        for ids in batches:
            loss = model(ids, labels=ids)
            (loss / world).backward()
            losses.append(loss.item())
        opt.step()
        out.append(losses)
    return out


def _sharded_worker(rank, world, steps, expected, mode):
    from yafsdp_b200 import MixedPrecisionPolicy
    from yafsdp_b200.models.llama import CONFIGS, LlamaForCausalLM, shard_llama

    if mode == "meta":
        with torch.device("meta"):
            model = LlamaForCausalLM(CONFIGS["tiny"])
    else:
        model = LlamaForCausalLM(CONFIGS["tiny"])
        model.init_weights(0)
    shard_llama(model, mp_policy=MixedPrecisionPolicy(), comm_backend="torch", num_grad_buffers=1,
                checkpoint_layers=1 if mode == "ckpt" else 0)
    if mode == "meta":
        model.init_weights(0)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, foreach=(mode != "single_tensor_optim"))
    ids = _batch(rank)
    for step in range(steps):
        opt.zero_grad()
        loss = model(ids, labels=ids)
        loss.backward()
        opt.step()
        want = expected[step][rank]
        assert abs(loss.item() - want) < 2e-4 * max(1.0, abs(want)), f"step {step}: {loss.item()} vs {want}"


@pytest.mark.timeout(300)
@pytest.mark.parametrize("mode", ["plain", "meta", "ckpt", "single_tensor_optim"])
def test_tiny_llama_10_adamw_steps_match_unsharded(mode):
    steps = 10 if mode == "plain" else 4
    expected = _unsharded_losses(2, steps)
    run_distributed(_sharded_worker, 2, steps, expected, mode)
