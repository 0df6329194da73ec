"""Llama-family decoder (Llama-2 MHA and Llama-3 GQA shapes) built on the native ops.

Parameter names follow the Hugging Face Llama layout (``model.embed_tokens.weight``,
``model.layers.N.self_attn.q_proj.weight`` ... ``lm_head.weight``), the model the reference's examples
train (``patches/transformers.diff:28-41``), so checkpoints map one to one.  The separate q/k/v and
gate/up projection weights sit back to back in a group's flat buffer, which lets the kernels use them
as one fused ``[rows, d]`` matrix without a copy.

``shard_llama`` applies ``fully_shard`` the way the reference recommends: embedding, every decoder
layer, ``[norm, lm_head]`` as one group, then a parameter-less root.
"""

from __future__ import annotations

import os

from dataclasses import dataclass
from typing import Any

import torch
import torch.nn as nn

from ..api import MixedPrecisionPolicy
from ..fully_shard import fully_shard
from ..ops import functional as Fn

__all__ = ["LlamaConfig", "LlamaForCausalLM", "LlamaDecoderLayer", "shard_llama", "CONFIGS"]


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_position_embeddings: int = 4096
    initializer_range: float = 0.02
    tie_word_embeddings: bool = False

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    def num_params(self) -> int:
        d, f, v = self.hidden_size, self.intermediate_size, self.vocab_size
        kv = self.num_key_value_heads * self.head_dim
        layer = 2 * d * d + 2 * d * kv + 3 * d * f + 2 * d
        return self.num_hidden_layers * layer + d + v * d * (1 if self.tie_word_embeddings else 2)

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token (forward + backward), causal attention counted at half."""
        d, f, v = self.hidden_size, self.intermediate_size, self.vocab_size
        kv = self.num_key_value_heads * self.head_dim
        dense = self.num_hidden_layers * (2 * d * d + 2 * d * kv + 3 * d * f) + v * d
        attn = self.num_hidden_layers * 2 * seq_len * d / 2
        return 6.0 * dense + 6.0 * attn


CONFIGS: dict[str, LlamaConfig] = {
    "tiny": LlamaConfig(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=4, max_position_embeddings=512),
    "tiny-gpu": LlamaConfig(vocab_size=1024, hidden_size=512, intermediate_size=1408, num_hidden_layers=2, num_attention_heads=4,
                            num_key_value_heads=2, max_position_embeddings=512),
    "llama2-7b": LlamaConfig(),
    "llama2-13b": LlamaConfig(hidden_size=5120, intermediate_size=13824, num_hidden_layers=40, num_attention_heads=40,
                              num_key_value_heads=40),
    "llama3-8b": LlamaConfig(vocab_size=128256, intermediate_size=14336, num_key_value_heads=8, rope_theta=500000.0,
                             max_position_embeddings=8192),
    "llama2-34b": LlamaConfig(hidden_size=8192, intermediate_size=22016, num_hidden_layers=48, num_attention_heads=64,
                              num_key_value_heads=8),
    "llama2-70b": LlamaConfig(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80, num_attention_heads=64,
                              num_key_value_heads=8),
    "llama3-70b": LlamaConfig(vocab_size=128256, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80,
                              num_attention_heads=64, num_key_value_heads=8, rope_theta=500000.0, max_position_embeddings=8192),
}


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, **kw: Any):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, **kw))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return Fn.rmsnorm_ref(x, self.weight, self.eps)


class _Proj(nn.Module):
    """Holder of one bias-free projection weight ``[out, in]`` (the math runs in the layer's fused op)."""

    def __init__(self, in_features: int, out_features: int, **kw: Any):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features, **kw))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.linear(x, self.weight)


class LlamaAttention(nn.Module):
    def __init__(self, cfg: LlamaConfig, **kw: Any):
        super().__init__()
        d, hd = cfg.hidden_size, cfg.head_dim
        self.q_proj = _Proj(d, cfg.num_attention_heads * hd, **kw)
        self.k_proj = _Proj(d, cfg.num_key_value_heads * hd, **kw)
        self.v_proj = _Proj(d, cfg.num_key_value_heads * hd, **kw)
        self.o_proj = _Proj(cfg.num_attention_heads * hd, d, **kw)


class LlamaMLP(nn.Module):
    def __init__(self, cfg: LlamaConfig, **kw: Any):
        super().__init__()
        self.gate_proj = _Proj(cfg.hidden_size, cfg.intermediate_size, **kw)
        self.up_proj = _Proj(cfg.hidden_size, cfg.intermediate_size, **kw)
        self.down_proj = _Proj(cfg.intermediate_size, cfg.hidden_size, **kw)


class LlamaDecoderLayer(nn.Module):
    def __init__(self, cfg: LlamaConfig, **kw: Any):
        super().__init__()
        self.cfg = cfg
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **kw)
        self.self_attn = LlamaAttention(cfg, **kw)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **kw)
        self.mlp = LlamaMLP(cfg, **kw)

    def forward(self, x: torch.Tensor, cos_sin: torch.Tensor, batch: int, seq: int) -> torch.Tensor:
        cfg = self.cfg
        dims = Fn.LayerDims(batch, seq, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
        a, m = self.self_attn, self.mlp
        return Fn.decoder_layer(
            x, self.input_layernorm.weight, a.q_proj.weight, a.k_proj.weight, a.v_proj.weight, a.o_proj.weight,
            self.post_attention_layernorm.weight, m.gate_proj.weight, m.up_proj.weight, m.down_proj.weight, cos_sin, dims,
        )


class LlamaEmbedding(nn.Module):
    def __init__(self, vocab: int, dim: int, **kw: Any):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab, dim, **kw))

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return Fn.embedding(ids, self.weight)


class LlamaModel(nn.Module):
    def __init__(self, cfg: LlamaConfig, **kw: Any):
        super().__init__()
        self.embed_tokens = LlamaEmbedding(cfg.vocab_size, cfg.hidden_size, **kw)
        self.layers = nn.ModuleList([LlamaDecoderLayer(cfg, **kw) for _ in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **kw)


class LMHead(nn.Module):
    def __init__(self, dim: int, vocab: int, **kw: Any):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(vocab, dim, **kw))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.linear(x, self.weight)


class LlamaForCausalLM(nn.Module):
    """``forward(input_ids [B,S], labels=None)`` returns the mean next-token loss when ``labels`` are given
    (shifted inside, like Hugging Face), else the logits ``[B,S,V]``."""

    def __init__(self, cfg: LlamaConfig, device: torch.device | str | None = None, dtype: torch.dtype | None = None):
        super().__init__()
        kw: dict[str, Any] = {}
        if device is not None:
            kw["device"] = device
        if dtype is not None:
            kw["dtype"] = dtype
        self.config = cfg
        self.model = LlamaModel(cfg, **kw)
        self.lm_head = LMHead(cfg.hidden_size, cfg.vocab_size, **kw)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self._rope: dict[tuple[int, str], torch.Tensor] = {}

    @torch.no_grad()
    def init_weights(self, seed: int | None = 0) -> None:
        """N(0, initializer_range) for every matrix, ones for the norms.  Works on sharded parameters too (every
        rank draws the full tensor from the same generator state and keeps its slice)."""
        if seed is not None:
            torch.manual_seed(seed)
        for name, p in self.named_parameters():
            if p.dim() == 1:
                p.fill_(1.0)
            else:
                p.normal_(0.0, self.config.initializer_range)

    def _rope_table(self, seq: int, device: torch.device) -> torch.Tensor:
        key = (seq, str(device))
        t = self._rope.get(key)
        if t is None:
            t = Fn.rope_table(seq, self.config.head_dim, self.config.rope_theta, device)
            self._rope[key] = t
        return t

    def head(self, h: torch.Tensor, labels: torch.Tensor | None) -> torch.Tensor:
        # runs inside the [norm, lm_head] fully_shard group: both modules' hooks fire around these calls
        return _run_head(self.model.norm, self.lm_head, h, labels, self.config.rms_norm_eps)

    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None, shift_labels: bool = True) -> torch.Tensor:
        b, s = input_ids.shape
        cos_sin = self._rope_table(s, input_ids.device)
        x = self.model.embed_tokens(input_ids).view(b * s, -1)
        for layer in self.model.layers:
            x = layer(x, cos_sin, b, s)
        if labels is not None:
            if shift_labels:
                labels = torch.cat([labels[:, 1:], labels.new_full((b, 1), -100)], dim=1)
            return self.head(x, labels.reshape(-1))
        return self.head(x, None).view(b, s, -1)


def _run_head(norm: RMSNorm, lm_head: LMHead, h: torch.Tensor, labels: torch.Tensor | None, eps: float) -> torch.Tensor:
    """Call order matters for the two-module group: the group's pre-forward fires on ``norm``'s forward
    hook and its post-forward on ``lm_head``'s, so each is invoked through ``__call__`` exactly once."""

    def norm_forward(x: torch.Tensor) -> torch.Tensor:
        return x

    def head_forward(x: torch.Tensor) -> torch.Tensor:
        if labels is not None:
            return Fn.head_loss(x, norm.weight, lm_head.weight, labels, eps)
        return Fn.head_logits(x, norm.weight, lm_head.weight, eps)

    # temporarily route the modules' forward through the fused op (norm passes h through, head does the math)
    norm.__dict__["forward"], lm_head.__dict__["forward"] = norm_forward, head_forward
    try:
        return lm_head(norm(h))
    finally:
        norm.__dict__.pop("forward", None)
        lm_head.__dict__.pop("forward", None)


def shard_llama(model: LlamaForCausalLM, *, mesh: Any = None, mp_policy: MixedPrecisionPolicy | None = None,
                reshard_after_forward: bool | None = True, comm_backend: Any = None,
                num_grad_buffers: int | None = 2, checkpoint_layers: int = 0, fused_reduce: bool | None = None,
                fused_gather: bool | None = None, **backend_options: Any) -> LlamaForCausalLM:
    """Wrap a Llama model: embedding, each decoder layer and ``[norm, lm_head]`` become groups, the model itself the
    parameter-less root.  ``checkpoint_layers`` wraps the first N layers' forward in activation checkpointing."""
    mp_policy = mp_policy or MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    kw = dict(mesh=mesh, mp_policy=mp_policy, reshard_after_forward=reshard_after_forward)
    if checkpoint_layers:
        from ..utils.checkpointing import checkpoint_module

        for layer in list(model.model.layers)[:checkpoint_layers]:
            checkpoint_module(layer)
    fully_shard(model.model.embed_tokens, **kw)
    for layer in model.model.layers:
        fully_shard(layer, **kw)
    if model.config.tie_word_embeddings:
        raise NotImplementedError("shard_llama: tied embeddings are not supported (wrap embed_tokens, norm and lm_head as one group yourself)")
    fully_shard([model.model.norm, model.lm_head], **kw)
    fully_shard(model, **kw)
    if fused_gather is None:
        fused_gather = os.environ.get("YAFSDP_FUSED_GATHER", "0") == "1"
    if fused_gather and len(model.model.layers) > 0:
        # the first layer's gather is the one nothing can hide (the step starts with it): its QKV GEMM pulls the layer itself;
        # every later layer's gather is issued ahead of time on the communication stream
        first = model.model.layers[0]
        first.set_fused_gather(True, prefix_params=[first.input_layernorm.weight])  # type: ignore[attr-defined]
    if fused_reduce is None:
        # measured (Llama-2-7B step): at two ranks the pushed gradients ride under the weight-gradient GEMMs (NVLink time
        # below GEMM time) and the step gets 1.5 % shorter; from four ranks on the push is link-bound and the overlapped
        # reduce-scatter wins.  YAFSDP_FUSED_REDUCE=0/1 overrides.
        env = os.environ.get("YAFSDP_FUSED_REDUCE")
        world = mesh.size() if mesh is not None else (torch.distributed.get_world_size() if torch.distributed.is_initialized() else 1)
        fused_reduce = (env == "1") if env is not None else world == 2
    if fused_reduce:
        # decoder layers and the head use every weight once per backward pass: their weight-gradient GEMMs push straight to
        # the owners (the embedding's gradient comes from a scatter-add kernel and stays on the unfused path)
        for layer in model.model.layers:
            layer.set_fused_gradient_reduce(True)  # type: ignore[attr-defined]
        model.lm_head.set_fused_gradient_reduce(True)  # type: ignore[attr-defined]
    if comm_backend is not None or num_grad_buffers is not None:
        model.set_comm_backend(comm_backend or "torch", num_grad_buffers=num_grad_buffers, **backend_options)  # type: ignore[attr-defined]
    return model
