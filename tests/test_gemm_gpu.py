"""tcgen05 grouped GEMM against a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, w, counts):
    outs, r = [], 0
    for e, c in enumerate(counts):
        outs.append(a[r:r + c].float() @ w[e].float().t())
        r += c
    return torch.cat(outs) if outs else a.new_zeros((0, w.shape[1]), dtype=torch.float32)


# pair=True: the CTA-pair form (cluster of two SMs, 256-row tiles); False: one CTA per 128-row tile
@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("counts,N,K", [([128], 256, 64), ([256, 128], 512, 256), ([100, 0, 333, 7], 256, 320),
                                        ([513], 384, 1024), ([64, 64, 64, 64, 64, 64, 64, 64], 1024, 512),
                                        ([1000, 129, 2300], 768, 448)])
def test_grouped_gemm_plain(counts, N, K, pair):
    from gpu_data_transfer_profile_b200.ops import gemm as G
    torch.manual_seed(0)
    rows = sum(counts)
    a = torch.randn(rows + 5, K, device="cuda").to(torch.bfloat16)        # extra rows must stay untouched
    w = (torch.randn(len(counts), N, K, device="cuda") * 0.1).to(torch.bfloat16)
    off = G.offsets_from_counts(counts, "cuda")
    out = torch.full((rows + 5, N), 7.0, dtype=torch.bfloat16, device="cuda")
    G.grouped_gemm(a, w, off, out=out, pair=pair)
    torch.cuda.synchronize()
    ref = _ref(a[:rows], w, counts)
    torch.testing.assert_close(out[:rows].float(), ref, atol=0.05 * (K ** 0.5) * 0.1, rtol=2e-2)
    assert bool((out[rows:] == 7.0).all())


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("counts,N,K", [([128], 256, 64), ([100, 0, 333, 7], 320, 256), ([513, 31], 384, 1000),
                                        ([1000, 129, 2300], 768, 448)])
def test_grouped_gemm_weights_stored_k_by_n(counts, N, K, pair):
    """out[r] = a[r] @ w[e] with w stored [E, K, N]: the data-gradient form, weights read in place."""
    from gpu_data_transfer_profile_b200.ops import gemm as G
    torch.manual_seed(4)
    rows = sum(counts)
    a = torch.randn(rows, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(len(counts), K, N, device="cuda") * 0.1).to(torch.bfloat16)
    out = G.grouped_gemm(a, w, G.offsets_from_counts(counts, "cuda"), pair=pair, w_kn=True)
    torch.cuda.synchronize()
    ref = _ref(a, w.transpose(1, 2), counts)
    torch.testing.assert_close(out.float(), ref, atol=0.05 * (K ** 0.5) * 0.1, rtol=2e-2)


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("counts,F,K", [([128], 128, 128), ([200, 56], 256, 256), ([1, 300], 384, 192),
                                        ([700, 3, 257], 512, 512)])
def test_grouped_gemm_swiglu_prob(counts, F, K, pair):
    from gpu_data_transfer_profile_b200.ops import gemm as G
    torch.manual_seed(1)
    rows = sum(counts)
    a = torch.randn(rows, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(len(counts), 2 * F, K, device="cuda") * 0.1).to(torch.bfloat16)
    prob = torch.rand(rows, device="cuda")
    out = G.grouped_gemm_swiglu(a, w, G.offsets_from_counts(counts, "cuda"), prob, pair=pair)
    torch.cuda.synchronize()
    fc1 = _ref(a, w, counts)
    ref = torch.nn.functional.silu(fc1[:, :F]) * fc1[:, F:] * prob[:, None]
    torch.testing.assert_close(out.float(), ref, atol=0.06, rtol=3e-2)


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("counts,M,N", [([64], 256, 256), ([128, 192], 256, 512), ([100, 0, 333, 7], 256, 320),
                                        ([90, 40], 192, 256), ([70, 0, 130], 200, 136),
                                        ([1], 512, 64), ([513, 63, 65], 768, 264), ([0, 0, 40], 256, 128),
                                        ([1000, 129, 2300], 512, 1024)])
def test_grouped_wgrad(counts, M, N, pair):
    """dW[e] = g_e^T x_e with the reduction over each expert's (ragged) rows; rows after the last
    expert hold NaN and must not leak into any gradient."""
    from gpu_data_transfer_profile_b200.ops import gemm as G
    torch.manual_seed(3)
    rows = sum(counts)
    g = torch.randn(rows + 70, M, device="cuda").to(torch.bfloat16)
    x = torch.randn(rows + 70, N, device="cuda").to(torch.bfloat16)
    g[rows:] = float("nan")
    x[rows:] = float("nan")
    dw = G.grouped_wgrad(g, x, G.offsets_from_counts(counts, "cuda"), pair=pair)
    torch.cuda.synchronize()
    r = 0
    for e, c in enumerate(counts):
        ref = g[r:r + c].float().t() @ x[r:r + c].float()
        torch.testing.assert_close(dw[e].float(), ref, atol=0.05 * max(c, 1) ** 0.5, rtol=2e-2)
        r += c


@pytest.mark.parametrize("pair", [False, True])
def test_grouped_gemm_swiglu_also_stores_pre_activation(pair):
    from gpu_data_transfer_profile_b200.ops import gemm as G
    torch.manual_seed(6)
    counts, F, K = [300, 1, 0, 215], 384, 320
    rows = sum(counts)
    a = torch.randn(rows, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(len(counts), 2 * F, K, device="cuda") * 0.1).to(torch.bfloat16)
    prob = torch.rand(rows, device="cuda")
    pre = torch.full((rows + 3, 2 * F), 5.0, dtype=torch.bfloat16, device="cuda")
    out = G.grouped_gemm_swiglu(a, w, G.offsets_from_counts(counts, "cuda"), prob, pair=pair, pre_out=pre)
    torch.cuda.synchronize()
    fc1 = _ref(a, w, counts)
    torch.testing.assert_close(pre[:rows].float(), fc1, atol=0.06, rtol=2e-2)
    assert bool((pre[rows:] == 5.0).all())
    ref = torch.nn.functional.silu(fc1[:, :F]) * fc1[:, F:] * prob[:, None]
    torch.testing.assert_close(out.float(), ref, atol=0.06, rtol=3e-2)


def test_grouped_gemm_rejects_bad_shapes():
    from gpu_data_transfer_profile_b200.ops import gemm as G
    a = torch.zeros(8, 36, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(1, 64, 36, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        G.grouped_gemm(a, w, G.offsets_from_counts([8], "cuda"))


def test_swiglu_fwd_bwd_kernels_match_autograd():
    from gpu_data_transfer_profile_b200.ops import gemm as G
    torch.manual_seed(2)
    rows, F = 37, 264
    h = torch.randn(rows, 2 * F, device="cuda").to(torch.bfloat16)
    p = torch.rand(rows, device="cuda")
    dact = torch.randn(rows, F, device="cuda").to(torch.bfloat16)
    hf = h.float().requires_grad_(True)
    pf = p.clone().requires_grad_(True)
    ref = torch.nn.functional.silu(hf[:, :F]) * hf[:, F:] * pf[:, None]
    rdh, rdp = torch.autograd.grad(ref, [hf, pf], dact.float())
    act = G.swiglu_fwd(h, p)
    dh, dp = G.swiglu_bwd(h, p, dact)
    torch.testing.assert_close(act.float(), ref.detach(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(dh.float(), rdh, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(dp, rdp, atol=0.3, rtol=2e-2)


@pytest.mark.parametrize("kind", ["gelu", "silu", "relu"])
def test_ungated_activation_kernels_match_autograd(kind):
    from gpu_data_transfer_profile_b200.models.experts import activate
    from gpu_data_transfer_profile_b200.ops import gemm as G
    torch.manual_seed(2)
    rows, F = 77, 264
    h = (torch.randn(rows, F, device="cuda") * 2).to(torch.bfloat16)
    p = torch.rand(rows, device="cuda")
    d = torch.randn(rows, F, device="cuda").to(torch.bfloat16)
    act = G.act_fwd(h, p, kind)
    hf = h.float().requires_grad_(True)
    pf = p.clone().requires_grad_(True)
    ref = activate(hf, kind) * pf[:, None]
    torch.testing.assert_close(act.float(), ref.detach(), atol=2e-2, rtol=2e-2)
    ref.backward(d.float())
    dh, dp = G.act_bwd(h, p, d, kind)
    torch.testing.assert_close(dh.float(), hf.grad, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(dp, pf.grad, atol=5e-2, rtol=2e-2)


def test_tcgen05_experts_backward_matches_torch_experts():
    from gpu_data_transfer_profile_b200.models.experts import TorchGroupedExperts
    from gpu_data_transfer_profile_b200.models.experts_tcgen05 import Tcgen05GroupedExperts
    torch.manual_seed(3)
    E, H, F = 3, 256, 384
    counts = [70, 0, 131]
    rows = sum(counts)
    a = Tcgen05GroupedExperts(E, H, F, torch.bfloat16, "swiglu", init_std=0.05)
    b = TorchGroupedExperts(E, H, F, torch.float32, "swiglu")
    with torch.no_grad():
        b.weight1.copy_(a.weight1.float())
        b.weight2.copy_(a.weight2.float())
    x = torch.randn(rows, H, device="cuda")
    p = torch.rand(rows, device="cuda")
    xa, pa = x.to(torch.bfloat16).requires_grad_(True), p.clone().requires_grad_(True)
    xb, pb = x.to(torch.bfloat16).float().requires_grad_(True), p.clone().requires_grad_(True)
    g = torch.randn(rows, H, device="cuda")
    ya = a(xa, counts, pa)
    yb = b(xb, counts, pb)
    ya.backward(g.to(torch.bfloat16))
    yb.backward(g.to(torch.bfloat16).float())
    torch.testing.assert_close(ya.float(), yb, atol=5e-2, rtol=5e-2)
    torch.testing.assert_close(xa.grad.float(), xb.grad, atol=5e-2, rtol=5e-2)
    torch.testing.assert_close(pa.grad, pb.grad, atol=0.5, rtol=5e-2)
    torch.testing.assert_close(a.weight1.grad.float(), b.weight1.grad, atol=0.15, rtol=5e-2)
    torch.testing.assert_close(a.weight2.grad.float(), b.weight2.grad, atol=0.15, rtol=5e-2)


@pytest.mark.parametrize("activation", ["swiglu", "gelu", "silu", "relu"])
def test_tcgen05_expert_mlp_gradients_match_fp32_autograd(activation):
    """Training path of the expert MLP (tcgen05 forward, dgrads reading the weights in place,
    ragged-reduction wgrads, fused activation backward) against fp32 autograd of the same math,
    for every activation the reference's expert MLP offers."""
    from gpu_data_transfer_profile_b200.models.experts import activate
    from gpu_data_transfer_profile_b200.models.experts_tcgen05 import Tcgen05GroupedExperts
    torch.manual_seed(5)
    H, F, counts = 256, 384, [70, 0, 301, 129]
    rows = sum(counts)
    mod = Tcgen05GroupedExperts(len(counts), H, F, init_std=0.05, activation=activation)
    x = torch.randn(rows, H, device="cuda").to(torch.bfloat16).requires_grad_(True)
    p = torch.rand(rows, device="cuda").requires_grad_(True)
    gy = torch.randn(rows, H, device="cuda").to(torch.bfloat16)
    y = mod(x, counts, p)
    y.backward(gy)
    xf = x.detach().float().requires_grad_(True)
    pf = p.detach().clone().requires_grad_(True)
    w1 = mod.weight1.detach().float().requires_grad_(True)
    w2 = mod.weight2.detach().float().requires_grad_(True)
    outs, r = [], 0
    for e, c in enumerate(counts):
        h = xf[r:r + c] @ w1[e].t()
        a = activate(h, activation) * pf[r:r + c, None]
        outs.append(a @ w2[e].t())
        r += c
    yr = torch.cat(outs)
    yr.backward(gy.float())
    torch.testing.assert_close(y.float(), yr.detach(), atol=3e-2, rtol=5e-2)
    torch.testing.assert_close(x.grad.float(), xf.grad, atol=3e-2, rtol=5e-2)
    torch.testing.assert_close(p.grad, pf.grad, atol=5e-2, rtol=5e-2)
    torch.testing.assert_close(mod.weight1.grad.float(), w1.grad, atol=6e-2, rtol=5e-2)
    torch.testing.assert_close(mod.weight2.grad.float(), w2.grad, atol=6e-2, rtol=5e-2)


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("counts,N,K", [([128], 256, 128), ([200, 0, 57], 384, 512), ([1, 300, 129, 0], 256, 1024),
                                        ([513], 128, 7168)])
def test_grouped_gemm_fp8_block_scaled(counts, N, K, swiglu):
    """e4m3 rows with 1x128 scales times e4m3 weights with 128x128 scales, against the fp32 matmul
    of the DEQUANTISED operands (the kernel multiplies exactly those numbers, so only the
    accumulation order and the bf16 store differ). Ragged counts with an empty expert."""
    from gpu_data_transfer_profile_b200.ops import gemm as G
    torch.manual_seed(11)
    rows, E = sum(counts), len(counts)
    Nw = 2 * N if swiglu else N
    x = torch.randn(rows + 5, K, device="cuda") * (1 + torch.arange(K, device="cuda") % 7)     # uneven block scales
    w = torch.randn(E, Nw, K, device="cuda") * 0.05
    xq, xs = G.quantize_rows_1x128(x)
    wq, ws = G.quantize_weights_128x128(w)
    p = torch.rand(rows + 5, device="cuda")
    off = G.offsets_from_counts(counts, "cuda")
    out = torch.full((rows + 5, N), 7.0, dtype=torch.bfloat16, device="cuda")
    G.grouped_gemm_fp8(xq, xs, wq, ws, off, swiglu=swiglu, row_prob=p if swiglu else None, out=out)
    xd = (xq.float().view(rows + 5, K // 128, 128) * xs[..., None]).view(rows + 5, K)
    wd = G.dequantize_weights_128x128(wq, ws)
    r = 0
    for e, c in enumerate(counts):
        if c == 0:
            continue
        h = xd[r:r + c] @ wd[e].t()
        ref = torch.nn.functional.silu(h[:, :N]) * h[:, N:] * p[r:r + c, None] if swiglu else h
        torch.testing.assert_close(out[r:r + c].float(), ref, atol=2e-2 * float(ref.abs().max() + 1), rtol=2e-2)
        r += c
    assert bool((out[rows:] == 7.0).all())           # rows beyond the last expert are never written


def test_tcgen05_experts_consume_fp8_dispatch_rows():
    from gpu_data_transfer_profile_b200.models.experts_tcgen05 import Tcgen05GroupedExperts
    from gpu_data_transfer_profile_b200.ops import gemm as G
    torch.manual_seed(3)
    H, F, counts = 512, 256, [90, 0, 200, 33]
    rows = sum(counts)
    mod = Tcgen05GroupedExperts(len(counts), H, F, init_std=0.05, use_fp8=True)
    x = torch.randn(rows, H, device="cuda").to(torch.bfloat16)
    p = torch.rand(rows, device="cuda")
    xq, xs = G.quantize_rows_1x128(x)
    y = mod((xq, xs), counts, p)
    y_ref = mod(x, counts, p)                              # bf16 path on the unquantised rows
    torch.testing.assert_close(y.float(), y_ref.detach().float(), atol=0.08 * float(y_ref.detach().float().abs().max()), rtol=0.1)


def test_grouped_gemms_work_from_a_fresh_thread():
    """The launchers encode TMA descriptors through a driver entry point, which needs a context
    bound to the calling thread; a thread that has made no CUDA runtime call yet (autograd's
    backward workers, user threads) must get one bound by the launcher itself."""
    import threading
    from gpu_data_transfer_profile_b200.ops import gemm as G
    torch.manual_seed(0)
    counts = [70, 0, 130]
    rows, K, N = sum(counts), 256, 384
    off = G.offsets_from_counts(counts, "cuda")
    a = torch.randn(rows, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(len(counts), N, K, device="cuda") * 0.05).to(torch.bfloat16)
    g = torch.randn(rows, N, device="cuda").to(torch.bfloat16)
    out, dx, dw = (torch.empty(rows, N, dtype=torch.bfloat16, device="cuda"),
                   torch.empty(rows, K, dtype=torch.bfloat16, device="cuda"),
                   torch.empty(len(counts), N, K, dtype=torch.bfloat16, device="cuda"))
    torch.cuda.synchronize()
    err = []

    def work():                                    # first CUDA work of this thread
        try:
            G.grouped_gemm(a, w, off, out=out)
            G.grouped_gemm(g, w, off, out=dx, w_kn=True)
            G.grouped_wgrad(g, a, off, out=dw)
            torch.cuda.synchronize()
        except Exception as e:                     # noqa: BLE001
            err.append(e)

    t = threading.Thread(target=work)
    t.start()
    t.join()
    assert not err, err
    r = 0
    for e, c in enumerate(counts):
        if c:
            torch.testing.assert_close(out[r:r + c].float(), a[r:r + c].float() @ w[e].float().t(), atol=3e-2, rtol=3e-2)
            torch.testing.assert_close(dx[r:r + c].float(), g[r:r + c].float() @ w[e].float(), atol=3e-2, rtol=3e-2)
        r += c
