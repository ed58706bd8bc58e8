"""The MoE layer's fp32 oracle against an independent implementation: transformers' Qwen3MoeSparseMoeBlock (softmax
router, top-k with renormalised weights, SwiGLU experts) with the same random weights. The GPU tests compare the
kernels with the oracle; this test pins the oracle's routing rule and expert arithmetic to the published block. The
reference simulates expert parallelism with equal splits and no router (examples/benchmark_all_to_all.py:31-127)."""
import pytest
import torch

mm = pytest.importorskip("transformers.models.qwen3_moe.modeling_qwen3_moe")


def test_moe_layer_oracle_matches_transformers_qwen3_moe_block():
    from maco_b200.models.moe_layer import MoEEPLayer
    from maco_b200.parallel.symm_heap import PlanningHeap
    torch.manual_seed(1)
    H, E, K, I, T = 256, 8, 2, 128, 256
    layer = MoEEPLayer(hidden=H, experts=E, top_k=K, inter=I, tokens=T, device=torch.device("cpu"), seed=5, weight_std=0.05,
                       router_std=0.5, capacity_factor=4.0, heap=PlanningHeap(0, 1, 1 << 26))
    assert layer.program is None                                   # a CPU device plans only
    cfg = mm.Qwen3MoeConfig(hidden_size=H, num_experts=E, num_experts_per_tok=K, moe_intermediate_size=I, norm_topk_prob=True,
                            hidden_act="silu", num_hidden_layers=1, vocab_size=32)
    blk = mm.Qwen3MoeSparseMoeBlock(cfg).float().eval()
    with torch.no_grad():
        blk.gate.weight.copy_(layer.w_router.float())
        for e in range(E):
            wg, wu, wd = layer.expert_weights(e)
            blk.experts.gate_up_proj[e].copy_(torch.cat([wg, wu], 0).float())
            blk.experts.down_proj[e].copy_(wd.float())
    x = torch.randn(T, H).to(torch.bfloat16)
    ours = layer.reference(x)
    with torch.no_grad():
        theirs = blk(x.float()[None])[0]
    # a token whose k-th and (k+1)-th logits tie after the bf16 rounding of the router output may pick another expert:
    # compare the tokens on whose routing both sides agree (all but a handful) closely, and require those to be most
    logits = (x.float() @ layer.w_router.float().t())
    top_ours = torch.sort(logits.to(torch.bfloat16).float(), dim=-1, descending=True, stable=True)[1][:, :K]
    top_theirs = torch.topk(torch.softmax(logits, -1), K, dim=-1)[1]
    same = (top_ours.sort(-1)[0] == top_theirs.sort(-1)[0]).all(-1)
    assert same.float().mean().item() > 0.95
    scale = ours.abs().max().item()
    assert (theirs[same] - ours[same]).abs().max().item() < 3e-2 * scale
