"""The package's Llama (CPU reference path of the fused layer functions) against ``transformers.LlamaForCausalLM`` with
the same weights: same parameter names, same loss, same gradients.  Covers MHA and GQA, tied embeddings and a RoPE base
other than the default."""

import pytest
import torch

transformers = pytest.importorskip("transformers")


@pytest.mark.parametrize("kv_heads,tie,theta", [(4, False, 10000.0), (2, False, 500000.0), (1, True, 10000.0)])
def test_loss_and_gradients_match_hugging_face_llama(kv_heads, tie, theta):
    from transformers import LlamaConfig as HFConfig
    from transformers import LlamaForCausalLM as HFLlama

    from yafsdp_b200.models.llama import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=kv_heads, rope_theta=theta, max_position_embeddings=64, tie_word_embeddings=tie)
    torch.manual_seed(0)
    ours = LlamaForCausalLM(cfg)
    ours.init_weights(seed=3)
    hf = HFLlama(HFConfig(vocab_size=96, hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4,
                          num_key_value_heads=kv_heads, rope_theta=theta, max_position_embeddings=64, tie_word_embeddings=tie,
                          rms_norm_eps=cfg.rms_norm_eps, attn_implementation="eager", attention_bias=False, mlp_bias=False))
    missing, unexpected = hf.load_state_dict(ours.state_dict(), strict=False)
    assert not unexpected and all("rotary" in k or "inv_freq" in k for k in missing), (missing, unexpected)
    ids = torch.randint(0, 96, (2, 24), generator=torch.Generator().manual_seed(1))
    loss = ours(ids, labels=ids)
    want = hf(input_ids=ids, labels=ids).loss
    assert torch.allclose(loss, want, atol=1e-5), (loss.item(), want.item())
    loss.backward()
    want.backward()
    theirs = dict(hf.named_parameters())
    for n, p in ours.named_parameters():
        assert torch.allclose(p.grad, theirs[n].grad, atol=2e-5), n
