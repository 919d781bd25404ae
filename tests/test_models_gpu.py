"""MoE layer forward/backward on one GPU (EP world of one rank) against a dense PyTorch oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dense_oracle(x, logits, w1, w2, topk, activation):
    from gpu_data_transfer_profile_b200.models.experts import activate
    from gpu_data_transfer_profile_b200.models.moe_layer import topk_softmax_router
    idx, probs = topk_softmax_router(logits, topk)
    out = torch.zeros_like(x, dtype=torch.float32)
    for k in range(topk):
        for e in range(w1.shape[0]):
            m = idx[:, k] == e
            if m.any():
                h = activate(x[m].float() @ w1[e].float().t(), activation) * probs[m, k][:, None]
                out[m] += h @ w2[e].float().t()
    return out


@pytest.mark.parametrize("mode", ["fused", "deepep"])
@pytest.mark.parametrize("activation", ["swiglu", "gelu"])
def test_moe_layer_forward_backward_matches_dense_oracle(mode, activation):
    from gpu_data_transfer_profile_b200.models import fused_a2a as A
    from gpu_data_transfer_profile_b200.models.moe_layer import MoELayer
    from gpu_data_transfer_profile_b200.parallel.symm import LocalWorld
    torch.manual_seed(0)
    T, H, F, E, K = 96, 256, 512, 4, 2
    world = LocalWorld.make(1)[0]
    A.configure_buffer(num_max_tokens_per_rank=128, num_topk=K, num_experts=E, group_by_expert=True)
    try:
        layer = MoELayer(H, F, E, K, None, dtype=torch.float32, activation=activation, expert_backend="torch",
                         dispatcher_mode=mode, world=world)
        x = torch.randn(T, H, device="cuda", requires_grad=True)
        logits = torch.randn(T, E, device="cuda", requires_grad=True)
        out = layer(x, logits)
        ref = _dense_oracle(x, logits, layer.experts.weight1, layer.experts.weight2, K, activation)
        torch.testing.assert_close(out, ref, atol=2e-4, rtol=2e-4)
        g = torch.randn_like(out)
        gx, gl, gw1 = torch.autograd.grad(out, [x, logits, layer.experts.weight1], g, retain_graph=False)
        rx, rl, rw1 = torch.autograd.grad(ref, [x, logits, layer.experts.weight1], g)
        torch.testing.assert_close(gx, rx, atol=2e-4, rtol=2e-4)
        torch.testing.assert_close(gl, rl, atol=2e-4, rtol=2e-3)
        torch.testing.assert_close(gw1, rw1, atol=2e-4, rtol=2e-3)
    finally:
        A.release_buffers()


def test_moe_layer_fused_combine_training_path_gradients():
    """fc2 epilogue performs the combine send in the TRAINING forward; gradients must equal the
    separate-combine path."""
    from gpu_data_transfer_profile_b200.models import fused_a2a as A
    from gpu_data_transfer_profile_b200.models.moe_layer import MoELayer
    from gpu_data_transfer_profile_b200.parallel.symm import LocalWorld
    torch.manual_seed(0)
    T, H, F, E, K = 200, 256, 512, 4, 2
    world = LocalWorld.make(1)[0]
    A.configure_buffer(num_max_tokens_per_rank=256, num_topk=K, num_experts=E, group_by_expert=True)
    try:
        layer = MoELayer(H, F, E, K, None, dtype=torch.bfloat16, expert_backend="tcgen05", world=world)
        x0 = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        logits = torch.randn(T, E, device="cuda")
        g = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        res = []
        for fuse in (True, False):
            layer.fuse_combine = fuse
            layer.zero_grad()
            x = x0.clone().requires_grad_(True)
            lg = logits.clone().requires_grad_(True)
            out = layer(x, lg)
            out.backward(g)
            res.append((out.detach().float(), x.grad.float(), lg.grad.float(), layer.experts.weight1.grad.float().clone(),
                        layer.experts.weight2.grad.float().clone()))
        for a, b in zip(*res):
            torch.testing.assert_close(a, b, atol=3e-2, rtol=3e-2)
    finally:
        A.release_buffers()


@pytest.mark.parametrize("fused", [False, True])
def test_moe_layer_tcgen05_experts_bf16(fused):
    """bf16 layer on the tcgen05 grouped GEMMs (separate combine with autograd, and the forward-only
    path whose fc2 epilogue performs the combine send) against the fp32 dense oracle."""
    from gpu_data_transfer_profile_b200.models import fused_a2a as A
    from gpu_data_transfer_profile_b200.models.moe_layer import MoELayer
    from gpu_data_transfer_profile_b200.parallel.symm import LocalWorld
    torch.manual_seed(0)
    T, H, F, E, K = 300, 512, 1024, 4, 2
    world = LocalWorld.make(1)[0]
    A.configure_buffer(num_max_tokens_per_rank=512, num_topk=K, num_experts=E, group_by_expert=True)
    try:
        layer = MoELayer(H, F, E, K, None, dtype=torch.bfloat16, activation="swiglu", expert_backend="tcgen05",
                         dispatcher_mode="fused", world=world)
        assert layer.expert_backend == "tcgen05_grouped_gemm"
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16).requires_grad_(not fused)
        logits = torch.randn(T, E, device="cuda")
        ref = _dense_oracle(x.detach().float(), logits, layer.experts.weight1.detach(), layer.experts.weight2.detach(),
                            K, "swiglu")
        if fused:
            with torch.no_grad():
                out = layer(x, logits)
        else:
            out = layer(x, logits)
            out.float().sum().backward()
            assert x.grad is not None and torch.isfinite(x.grad).all()
            assert layer.experts.weight1.grad is not None and torch.isfinite(layer.experts.weight1.grad).all()
        torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=5e-2)
    finally:
        A.release_buffers()


def test_moe_layer_fp8_inference_path_close_to_bf16():
    """fp8 dispatch (cast fused into the send kernel) feeding the block-scaled fp8 fc1 directly,
    against the same layer's bf16 path: the difference is the e4m3 rounding of rows and weights."""
    from gpu_data_transfer_profile_b200.models import fused_a2a as A
    from gpu_data_transfer_profile_b200.models.moe_layer import MoELayer
    from gpu_data_transfer_profile_b200.parallel.symm import LocalWorld
    torch.manual_seed(0)
    T, H, F, E, K = 300, 512, 1024, 4, 2
    world = LocalWorld.make(1)[0]
    A.configure_buffer(num_max_tokens_per_rank=512, num_topk=K, num_experts=E, group_by_expert=True)
    try:
        layer = MoELayer(H, F, E, K, None, dtype=torch.bfloat16, activation="swiglu", expert_backend="tcgen05",
                         dispatcher_mode="fused", world=world, use_fp8=True, fuse_combine=False)
        assert layer.use_fp8
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        logits = torch.randn(T, E, device="cuda")
        with torch.no_grad():
            out8 = layer(x, logits)
            layer.use_fp8 = False
            out16 = layer(x, logits)
        scale = float(out16.float().abs().max())
        torch.testing.assert_close(out8.float(), out16.float(), atol=0.06 * scale, rtol=0.1)
    finally:
        A.release_buffers()
