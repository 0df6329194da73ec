"""Per-GPU memory plan of a sharded Llama-family training run, from the configuration alone.

Lets a user pick the world size and the number of checkpointed layers for the 180 GB of a B200 before anything is
allocated (the reference leaves this to trial and error with ``--fsdp_num_layers_to_checkpoint``,
``README.md:45-71``).  Components, all per GPU:

* sharded state: fp32 master, fp32 gradient shard, two fp32 AdamW moments and the bf16 all-gather input
  (18 bytes per parameter / world);
* communication buffers: two rotating bf16 layer buffers and ``num_grad_buffers`` fp32 layer gradient buffers of the
  largest group (none at world size 1, where the shards are the buffers);
* activations kept for backward by the fused layer (bf16 per token and layer: the layer input, both normalised
  inputs, q/k/v, the attention output, the attention-block output, gate/up and their product), or only the layer input
  for a checkpointed layer (plus one layer's worth while it is recomputed);
* the bf16 logits (written once, overwritten by their gradient).
"""

from __future__ import annotations

from typing import Any

__all__ = ["estimate_memory", "keep_gathered_fits", "B200_HBM_BYTES"]

B200_HBM_BYTES = 183_359 * 2**20  # what nvidia-smi reports for a B200


def estimate_memory(cfg: Any, world: int, seq_len: int, batch: int = 1, checkpoint_layers: int = 0,
                    num_grad_buffers: int = 1) -> dict[str, float]:
    """Bytes per GPU by component (keys ``state``, ``buffers``, ``activations``, ``logits``, ``total``) and ``fits``
    (total below 95 % of a B200's memory).  ``cfg`` is a ``LlamaConfig``."""
    d, f, v, n_layers = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.num_hidden_layers
    kv = cfg.num_key_value_heads * cfg.head_dim
    params = cfg.num_params()
    layer_params = 2 * d * d + 2 * d * kv + 3 * d * f + 2 * d
    largest_group = max(layer_params, v * d + d)
    state = 18.0 * params / world
    buffers = 0.0 if world == 1 else 2 * 2.0 * largest_group + num_grad_buffers * 4.0 * largest_group
    tokens = batch * seq_len
    per_layer = 2.0 * tokens * (6 * d + 2 * kv + 3 * f)
    ckpt = max(0, min(checkpoint_layers, n_layers))
    activations = (n_layers - ckpt) * per_layer + ckpt * 2.0 * tokens * d + (per_layer if ckpt else 0.0)
    activations += 2.0 * tokens * d * 3  # embedding output, final norm input and output
    logits = 2.0 * tokens * v
    total = state + buffers + activations + logits
    return {"state": state, "buffers": buffers, "activations": activations, "logits": logits, "total": total,
            "fits": float(total < 0.95 * B200_HBM_BYTES)}


def keep_gathered_fits(cfg: Any, world: int, seq_len: int, batch: int = 1, checkpoint_layers: int = 0, num_grad_buffers: int = 2,
                       budget_fraction: float = 0.6) -> bool:
    """Can every layer keep its gathered bf16 parameters from its forward to its backward pass (``reshard_after_forward=
    False``: one gather per layer and step instead of two) within ``budget_fraction`` of a B200's memory?  The whole
    compute-dtype model then sits on every GPU during a step (2 bytes per parameter) on top of the sharded plan."""
    if world <= 1:
        return False  # single rank: the shards are the parameters, nothing is gathered
    plan = estimate_memory(cfg, world, seq_len, batch, checkpoint_layers, num_grad_buffers)
    return plan["total"] + 2.0 * cfg.num_params() <= budget_fraction * B200_HBM_BYTES
