"""Hugging Face integration on CPU/gloo (world 2): a tiny ``LlamaForCausalLM`` sharded through ``shard_causal_lm`` (both APIs,
tied and untied embeddings, activation checkpointing, weights only on rank 0) trains like the unsharded model; so do GPT-2, GPT-NeoX, Mistral, Qwen2, Mixtral (mixture of experts) and Gemma."""

import pytest
import torch

from dist_utils import run_distributed

transformers = pytest.importorskip("transformers")


def _tiny(tie=False, meta=False):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                      vocab_size=64, max_position_embeddings=64, tie_word_embeddings=tie, attn_implementation="eager")
    torch.manual_seed(0)
    if meta:
        with torch.device("meta"):
            return LlamaForCausalLM(cfg)
    return LlamaForCausalLM(cfg)


def _ids(rank):
    return torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(7 + rank))


def _reference(world, steps, tie):
    model = _tiny(tie)
    opt = torch.optim.SGD(model.parameters(), lr=5e-2)
    for _ in range(steps):
        opt.zero_grad()
        for r in range(world):
            ids = _ids(r)
            (model(input_ids=ids, labels=ids).loss / world).backward()
        opt.step()
    return {n: p.detach().clone() for n, p in model.named_parameters()}


def _worker(rank, world, api, tie):
    from yafsdp_b200 import MixedPrecisionPolicy
    from yafsdp_b200.integrations.hf import find_decoder_parts, shard_causal_lm, trainer_callbacks

    model = _tiny(tie, meta=rank != 0)  # weights exist on rank 0 only
    parts = find_decoder_parts(model)
    assert len(parts.layers) == 3 and parts.tied == tie and parts.name(parts.layers[1]) == "model.layers.1"
    wrapped = shard_causal_lm(model, mp_policy=MixedPrecisionPolicy(), num_layers_to_checkpoint=2, sync_from_rank0=True,
                              api=api, comm_backend="torch")
    params = list(wrapped.parameters())
    opt = torch.optim.SGD(params, lr=5e-2)
    for _ in range(2):
        if api == "v1":
            wrapped.zero_grad()
        else:
            opt.zero_grad()
        ids = _ids(rank)
        wrapped(input_ids=ids, labels=ids).loss.backward()
        opt.step()
    want = _reference(world, 2, tie)
    for n, p in model.named_parameters():
        full = p.full_tensor() if hasattr(p, "full_tensor") else p.detach()
        assert torch.allclose(full, want[n], atol=2e-5), n
    assert len(trainer_callbacks()) == 1 and len(trainer_callbacks(trace_path="t.json", memory_snapshot_path="m")) == 3


@pytest.mark.timeout(300)
@pytest.mark.parametrize("api,tie", [("fully_shard", False), ("fully_shard", True), ("v1", False)])
def test_hf_causal_lm(api, tie):
    run_distributed(_worker, 2, api, tie)


# ------------------------------------------------------------------------------------------------ other decoder layouts
def _tiny_other(kind):
    torch.manual_seed(0)
    if kind == "gpt2":  # tied embeddings, learned position embeddings outside the known parts, Conv1D projections
        from transformers import GPT2Config, GPT2LMHeadModel

        return GPT2LMHeadModel(GPT2Config(n_embd=32, n_layer=2, n_head=4, vocab_size=64, n_positions=32, resid_pdrop=0.0,
                                          embd_pdrop=0.0, attn_pdrop=0.0, attn_implementation="eager"))
    common = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, vocab_size=64,
                  max_position_embeddings=64, attention_dropout=0.0, attn_implementation="eager")
    if kind == "mistral":  # sliding-window attention configuration, grouped KV heads
        from transformers import MistralConfig, MistralForCausalLM

        return MistralForCausalLM(MistralConfig(sliding_window=8, **common))
    if kind == "qwen2":  # biases on the q/k/v projections: 1-D parameters inside every layer group
        from transformers import Qwen2Config, Qwen2ForCausalLM

        return Qwen2ForCausalLM(Qwen2Config(**common))
    if kind == "mixtral":  # mixture of experts: router + expert weights in every layer, all flat-sharded over the data ranks
        from transformers import MixtralConfig, MixtralForCausalLM

        return MixtralForCausalLM(MixtralConfig(num_local_experts=4, num_experts_per_tok=2, router_aux_loss_coef=0.0,
                                                output_router_logits=False, **common))
    if kind == "gemma":  # tied embeddings, (1 + weight) RMSNorm, explicit head_dim
        from transformers import GemmaConfig, GemmaForCausalLM

        return GemmaForCausalLM(GemmaConfig(head_dim=8, **common))
    from transformers import GPTNeoXConfig, GPTNeoXForCausalLM  # parallel residual, `gpt_neox.layers`, `embed_out`

    return GPTNeoXForCausalLM(GPTNeoXConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                                            vocab_size=64, max_position_embeddings=64, hidden_dropout=0.0, attention_dropout=0.0,
                                            attn_implementation="eager"))


def _other_worker(rank, world, kinds):
    from yafsdp_b200 import MixedPrecisionPolicy
    from yafsdp_b200.integrations.hf import shard_causal_lm

    for kind in kinds.split("+"):  # several families per launch: most of a launch is process start-up
        ref = _tiny_other(kind)
        ref_opt = torch.optim.SGD(ref.parameters(), lr=5e-2)
        for _ in range(2):
            ref_opt.zero_grad()
            for r in range(world):
                (ref(input_ids=_ids(r), labels=_ids(r)).loss / world).backward()
            ref_opt.step()
        model = shard_causal_lm(_tiny_other(kind), mp_policy=MixedPrecisionPolicy(), num_layers_to_checkpoint=1, comm_backend="torch")
        opt = torch.optim.SGD(model.parameters(), lr=5e-2)
        for _ in range(2):
            opt.zero_grad()
            model(input_ids=_ids(rank), labels=_ids(rank)).loss.backward()
            opt.step()
        for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
            assert torch.allclose(p.full_tensor(), q.detach(), atol=2e-5), (kind, n)


@pytest.mark.timeout(300)
@pytest.mark.parametrize("kinds", ["gpt2+neox", "mistral+qwen2+mixtral+gemma"])
def test_hf_other_decoder_layouts(kinds):
    run_distributed(_other_worker, 2, kinds)


# ------------------------------------------------------------------------------------------------ weights in and out
def _weights_worker(rank, world):
    """Hugging Face weights load into the package's sharded Llama by name (full tensors, every rank keeps its slices); the
    loss matches; the gathered full state dict loads back into a Hugging Face model."""
    from yafsdp_b200 import MixedPrecisionPolicy, checkpoint
    from yafsdp_b200.models.llama import LlamaConfig, LlamaForCausalLM, shard_llama

    hf = _tiny()
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=64, rms_norm_eps=hf.config.rms_norm_eps)
    with torch.device("meta"):
        model = LlamaForCausalLM(cfg)
    shard_llama(model, mp_policy=MixedPrecisionPolicy(), comm_backend="torch")  # fp32 compute: exact comparison
    model.init_weights(seed=11)  # something else than the Hugging Face weights
    result = model.load_state_dict(hf.state_dict(), strict=False)
    assert not result.unexpected_keys and not result.missing_keys, result
    ids = _ids(rank)
    loss = model(ids, labels=ids)
    want = hf(input_ids=ids, labels=ids).loss
    assert torch.allclose(loss, want, atol=1e-5), (loss.item(), want.item())
    full = checkpoint.full_state_dict(model)
    if rank == 0:
        back = _tiny()
        with torch.no_grad():
            for p in back.parameters():
                p.zero_()
        back.load_state_dict(full, strict=False)
        for (n, p), (_, q) in zip(back.named_parameters(), hf.named_parameters()):
            assert torch.equal(p, q), n


@pytest.mark.timeout(300)
def test_hugging_face_weights_load_into_sharded_llama_and_back():
    run_distributed(_weights_worker, 2)
