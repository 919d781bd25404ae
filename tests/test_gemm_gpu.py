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


@pytest.mark.parametrize("counts,N,K", [([128], 256, 64), ([256, 128], 512, 256), ([100, 0, 333, 7], 256, 320),
                                        ([513], 384, 1024), ([64, 64, 64, 64, 64, 64, 64, 64], 1024, 512)])
def test_grouped_gemm_plain(counts, N, K):
    from gpu_data_transfer_profile_b200.ops import gemm as G
    torch.manual_seed(0)
    rows = sum(counts)
    a = torch.randn(rows + 5, K, device="cuda").to(torch.bfloat16)        # extra rows must stay untouched
    w = (torch.randn(len(counts), N, K, device="cuda") * 0.1).to(torch.bfloat16)
    off = G.offsets_from_counts(counts, "cuda")
    out = torch.full((rows + 5, N), 7.0, dtype=torch.bfloat16, device="cuda")
    G.grouped_gemm(a, w, off, out=out)
    torch.cuda.synchronize()
    ref = _ref(a[:rows], w, counts)
    torch.testing.assert_close(out[:rows].float(), ref, atol=0.05 * (K ** 0.5) * 0.1, rtol=2e-2)
    assert bool((out[rows:] == 7.0).all())


@pytest.mark.parametrize("counts,F,K", [([128], 128, 128), ([200, 56], 256, 256), ([1, 300], 384, 192)])
def test_grouped_gemm_swiglu_prob(counts, F, K):
    from gpu_data_transfer_profile_b200.ops import gemm as G
    torch.manual_seed(1)
    rows = sum(counts)
    a = torch.randn(rows, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(len(counts), 2 * F, K, device="cuda") * 0.1).to(torch.bfloat16)
    prob = torch.rand(rows, device="cuda")
    out = G.grouped_gemm_swiglu(a, w, G.offsets_from_counts(counts, "cuda"), prob)
    torch.cuda.synchronize()
    fc1 = _ref(a, w, counts)
    ref = torch.nn.functional.silu(fc1[:, :F]) * fc1[:, F:] * prob[:, None]
    torch.testing.assert_close(out.float(), ref, atol=0.06, rtol=3e-2)


def test_grouped_gemm_rejects_bad_shapes():
    from gpu_data_transfer_profile_b200.ops import gemm as G
    a = torch.zeros(8, 36, device="cuda", dtype=torch.bfloat16)
    w = torch.zeros(1, 64, 36, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        G.grouped_gemm(a, w, G.offsets_from_counts([8], "cuda"))
