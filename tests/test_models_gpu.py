"""Single-GPU runs of the model-level programs against PyTorch autograd / fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_dp_backward_single_gpu_matches_autograd():
    from maco_b200 import _native
    from maco_b200.models.dp_mlp_stack import DPMLPStackBackward
    m = DPMLPStackBackward(layers=4, hidden=512, tokens=768, seed=2, weight_std=0.05)
    ref = m.reference_grads()
    for mode_iter in range(2):
        m.forward()
        g = m.backward()
        torch.cuda.synchronize()
        err = (g - ref).abs().max().item()
        assert err < 3e-2 * ref.abs().max().item() + 1e-7, (err, ref.abs().max().item())
    assert _native.status() == 0


@pytest.mark.parametrize("cta_pair", [True, False])
def test_tp_mlp_single_gpu(cta_pair):
    from maco_b200.models.tp_mlp import TPSwiGLUMLP
    layer = TPSwiGLUMLP(512, 512, 1024, seed=1, cta_pair=cta_pair)
    assert layer.program.cta_pair == cta_pair
    x = torch.randn(512, 512, device="cuda", dtype=torch.bfloat16)
    y = layer(x)
    torch.cuda.synchronize()
    ref = layer.reference(x)
    assert (y.float() - ref).abs().max().item() < 3e-2 * max(1.0, ref.abs().max().item())


def test_tp_mlp_two_input_slots():
    from maco_b200.models.tp_mlp import TPSwiGLUMLP
    layer = TPSwiGLUMLP(512, 512, 1024, seed=1, input_slots=2)
    xs = [torch.randn(512, 512, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    for it in range(4):
        y = layer(xs[it & 1], slot=it & 1)
        torch.cuda.synchronize()
        ref = layer.reference(xs[it & 1])
        assert (y.float() - ref).abs().max().item() < 3e-2 * max(1.0, ref.abs().max().item()), it


@pytest.mark.parametrize("mode,blocked", [("static", False), ("dynamic", False), ("static", True)])
def test_qwen3_decode_layer_single_gpu(mode, blocked):
    from maco_b200 import _native
    from maco_b200.models.qwen3_layer import Qwen3DecodeLayer
    # 1400 cached keys in 2 splits: 6 chunks of 128 keys per task, so the K/V ring wraps several times
    # (blocked: the four projections read tile-by-tile copies of their weights)
    layer = Qwen3DecodeLayer(hidden=1024, q_heads=16, kv_heads=2, ffn=2048, batch=8, kv_len=1400, seed=4, mode=mode, splits=2,
                             weight_std=0.05, blocked_weights=blocked)
    assert layer.blocked == blocked
    x = torch.randn(8, 1024, device="cuda", dtype=torch.bfloat16)
    ref = layer.reference(x)
    for _ in range(2):
        out = layer(x)
        torch.cuda.synchronize()
        err = (out.float() - ref).abs().max().item()
        assert err < 4e-2 * max(1.0, ref.abs().max().item()), err
    assert _native.status() == 0


def test_moe_layer_full_row_width():
    """hidden 2048: a token row is 256 16-byte vectors, more than one pass of a warp; every vector of the
    dispatched and of the returned rows has to arrive (checked against the fp32 reference, two launches)."""
    from maco_b200 import _native
    from maco_b200.models.moe_layer import MoEEPLayer
    layer = MoEEPLayer(hidden=2048, experts=16, top_k=4, inter=256, tokens=512, capacity_factor=4.0, seed=5,
                       weight_std=0.03, router_std=0.3)
    x = torch.randn(512, 2048, device="cuda", dtype=torch.bfloat16)
    ref = layer.reference(x)
    for _ in range(2):
        out = layer(x)
        torch.cuda.synchronize()
        assert layer.dropped() == 0
        err = (out.float() - ref).abs().max().item()
        assert err < 4e-2 * max(1.0, ref.abs().max().item()), err
    assert _native.status() == 0


@pytest.mark.parametrize("mode", ["static", "dynamic"])
def test_moe_layer_single_gpu(mode):
    from maco_b200 import _native
    from maco_b200.models.moe_layer import MoEEPLayer
    layer = MoEEPLayer(hidden=256, experts=8, top_k=2, inter=128, tokens=256, capacity_factor=4.0, seed=3, mode=mode,
                       weight_std=0.05, router_std=0.5)
    x = torch.randn(256, 256, device="cuda", dtype=torch.bfloat16)
    ref = layer.reference(x)
    for _ in range(2):
        out = layer(x)
        torch.cuda.synchronize()
        assert layer.dropped() == 0
        err = (out.float() - ref).abs().max().item()
        assert err < 4e-2 * max(1.0, ref.abs().max().item()), err
    assert _native.status() == 0


def test_moe_layer_reports_dropped_pairs_without_a_blocking_read():
    """Slabs too small for the routing skew: the step's dropped-pair count reaches the host behind the launch, the
    next forward() warns (or raises with on_drop="raise"), and dropped() agrees with a recount from the logits."""
    from maco_b200 import _native
    from maco_b200.models.moe_layer import MoEEPLayer
    layer = MoEEPLayer(hidden=256, experts=8, top_k=2, inter=128, tokens=1024, capacity_factor=0.5, seed=11,
                       weight_std=0.05, router_std=2.0, on_drop="ignore")
    assert layer.capacity == 128                                   # mean load is 256 rows per expert
    x = torch.randn(1024, 256, device="cuda", dtype=torch.bfloat16)
    layer(x)
    n = layer.dropped()                                            # waits for the counter's copy only
    logits = layer.logits.float()                                  # the router GEMM's own output
    idx = torch.sort(logits, dim=-1, descending=True, stable=True)[1][:, :2]
    load = torch.bincount(idx.flatten(), minlength=8)
    assert n == int((load - layer.capacity).clamp(min=0).sum())
    assert n > 0 and layer.total_dropped == n
    layer(x)
    torch.cuda.synchronize()
    layer.on_drop = "warn"
    with pytest.warns(RuntimeWarning, match="dropped"):
        layer(x)                                                   # learns about the previous step's drops
    torch.cuda.synchronize()
    layer.on_drop = "raise"
    with pytest.raises(RuntimeError, match="capacity_factor"):
        layer(x)
    assert _native.status() == 0
