"""The decode layer's fp32 oracle against an independent implementation: transformers' Qwen3DecoderLayer (eager
attention) with the same random weights, one new token per sequence over a filled KV cache. The GPU tests compare
the kernels with the oracle; this test pins the oracle itself to the published architecture (per-head QK RMSNorm,
half-rotation RoPE, grouped-query attention, SwiGLU MLP, pre-norm residuals). The reference validates against a
downloaded Qwen3 checkpoint (examples/validate_qwen3.py:28-120); there is no network here, so the weights are random."""
import pytest
import torch

mq = pytest.importorskip("transformers.models.qwen3.modeling_qwen3")


def test_decode_layer_oracle_matches_transformers_qwen3():
    from transformers import Qwen3Config
    from transformers.cache_utils import DynamicCache
    from maco_b200.models.qwen3_layer import Qwen3DecodeLayer
    torch.manual_seed(0)
    B, H, hq, hkv, D, F, kv_len = 4, 512, 8, 2, 128, 1024, 37
    layer = Qwen3DecodeLayer(hidden=H, q_heads=hq, kv_heads=hkv, head_dim=D, ffn=F, batch=B, kv_len=kv_len,
                             device=torch.device("cpu"), seed=3, weight_std=0.05)
    assert layer.program is None                                   # a CPU device plans only
    cfg = Qwen3Config(hidden_size=H, num_attention_heads=hq, num_key_value_heads=hkv, head_dim=D, intermediate_size=F,
                      rms_norm_eps=layer.eps, rope_theta=layer.theta, attention_bias=False, num_hidden_layers=1, vocab_size=32,
                      max_position_embeddings=4096)
    cfg._attn_implementation = "eager"
    hf = mq.Qwen3DecoderLayer(cfg, layer_idx=0).float().eval()
    with torch.no_grad():
        a = hf.self_attn
        a.q_proj.weight.copy_(layer.w_qkv[: hq * D].float())
        a.k_proj.weight.copy_(layer.w_qkv[hq * D:(hq + hkv) * D].float())
        a.v_proj.weight.copy_(layer.w_qkv[(hq + hkv) * D:].float())
        a.o_proj.weight.copy_(layer.w_o.float())
        a.q_norm.weight.copy_(layer.q_norm.float())
        a.k_norm.weight.copy_(layer.k_norm.float())
        hf.mlp.gate_proj.weight.copy_(layer.w_gate.float())
        hf.mlp.up_proj.weight.copy_(layer.w_up.float())
        hf.mlp.down_proj.weight.copy_(layer.w_down.float())
        hf.input_layernorm.weight.copy_(layer.w_in.float())
        hf.post_attention_layernorm.weight.copy_(layer.w_post.float())
    x = torch.randn(B, H).to(torch.bfloat16)
    ours = layer.reference(x)
    cache = DynamicCache(config=cfg)
    cache.update(layer.k_cache[:, :, :kv_len].float(), layer.v_cache[:, :, :kv_len].float(), 0)   # keys are stored rotated
    cs = layer.cos_sin.float()                                    # [B, D]: cosines | sines of the D/2 frequencies
    cos = torch.cat([cs[:, : D // 2], cs[:, : D // 2]], -1)[:, None, :]
    sin = torch.cat([cs[:, D // 2:], cs[:, D // 2:]], -1)[:, None, :]
    # the layer's own rotary table against transformers' (same frequencies, same position)
    rot = mq.Qwen3RotaryEmbedding(config=cfg)
    hf_cos, hf_sin = rot(x.float()[:, None, :], torch.full((B, 1), kv_len))
    assert torch.allclose(hf_cos, cos, atol=1e-2) and torch.allclose(hf_sin, sin, atol=1e-2)      # table is stored in bf16
    with torch.no_grad():
        out = hf(x.float()[:, None, :], attention_mask=None, position_ids=torch.full((B, 1), kv_len), past_key_values=cache,
                 use_cache=True, position_embeddings=(cos, sin))
    out = (out[0] if isinstance(out, tuple) else out)[:, 0]
    # the oracle rounds to bf16 where the kernels do (after every projection); transformers runs in fp32 throughout
    assert (out - ours).abs().max().item() < 2e-2 * ours.abs().max().item()
