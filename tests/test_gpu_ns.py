"""tcgen05 Newton-Schulz kernels against fp32 torch matmuls."""
import pytest
import torch

from apexw_b200 import _native
from apexw_b200.ops import newton_schulz as NS

pytestmark = pytest.mark.gpu


def _nat():
    nat = _native.require()
    if not nat.ns_supported():
        pytest.skip("tcgen05 needs compute capability 10.x")
    return nat


@pytest.mark.parametrize("M,N,K,batch", [(128, 256, 64, 1), (256, 512, 192, 1), (384, 128, 1024, 2), (128, 320, 72, 3)])
@pytest.mark.parametrize("with_d", [False, True])
@pytest.mark.parametrize("tile_n", [0, 128, 256])
def test_tn_gemm_matches_fp32_reference(M, N, K, batch, with_d, tile_n):
    nat = _nat()
    torch.manual_seed(0)
    A = (torch.randn(batch, M, K, device="cuda") * 0.5).bfloat16()
    B = (torch.randn(batch, N, K, device="cuda") * 0.5).bfloat16()
    D = (torch.randn(batch, M, N, device="cuda")).bfloat16() if with_d else None
    alpha, beta = 0.75, (-1.25 if with_d else 0.0)
    out = nat.ns_gemm_tn(A, B, D, alpha, beta, False, False, tile_n)
    ref = alpha * torch.bmm(A.float(), B.float().transpose(1, 2)) + (beta * D.float() if with_d else 0.0)
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-2, err
    both = nat.ns_gemm_tn(A, B, D, alpha, beta, True, False, tile_n)
    C = both[0].view(batch, M, N)
    Ct = both[1].view(batch, N, M)
    assert torch.equal(C, out) and torch.equal(Ct, C.transpose(1, 2))


@pytest.mark.parametrize("shape", [(256, 256), (128, 512), (512, 128), (3, 256, 384)])
def test_newton_schulz_on_tensor_cores_matches_torch_path(shape, monkeypatch):
    _nat()
    torch.manual_seed(1)
    G = torch.randn(*shape, device="cuda")
    fn = NS.zeropower_via_newtonschulz5 if len(shape) == 2 else NS.zeropower_via_newtonschulz5_batched
    X = G.bfloat16()
    probe = X if len(shape) == 2 and shape[0] <= shape[1] else X.transpose(-2, -1)
    assert NS.ns_backend(probe.contiguous()) == "tcgen05"
    fast = fn(X, steps=5).float()
    monkeypatch.setenv("APEXW_B200_NS_BACKEND", "torch")
    slow = fn(X, steps=5).float()
    monkeypatch.delenv("APEXW_B200_NS_BACKEND")
    exact = fn(G, steps=5) if len(shape) == 2 else fn(G, steps=5)
    assert (fast - slow).abs().max() < 0.06                    # both are bf16 iterations of the same map
    s = torch.linalg.svdvals(fast.reshape(-1, fast.shape[-2], fast.shape[-1])[0])
    assert s.max() < 1.3 and torch.quantile(s, 0.1) > 0.45


@pytest.mark.parametrize("M,K,batch", [(128, 64, 1), (384, 128, 2), (1024, 256, 1), (2048, 192, 3), (640, 1024, 1)])
@pytest.mark.parametrize("with_d", [False, True])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_symmetric_product_skips_lower_tiles_and_mirrors_them(M, K, batch, with_d, tile_n):
    """A A^T (+ beta * symmetric D): only tiles touching the upper triangle are computed; the result must still be
    the full matrix, exactly symmetric, and equal to the non-symmetric launch.  (2048, 192, 3) has 264 tiles on
    148 persistent CTAs with 3 k-blocks each: the smem ring and both TMEM accumulators wrap several times."""
    nat = _nat()
    torch.manual_seed(2)
    A = (torch.randn(batch, M, K, device="cuda") * 0.5).bfloat16()
    D = None
    if with_d:
        D = torch.randn(batch, M, M, device="cuda")
        D = ((D + D.transpose(1, 2)) * 0.5).bfloat16()
    alpha, beta = 0.5, (1.5 if with_d else 0.0)
    full = nat.ns_gemm_tn(A, A, D, alpha, beta, False, False, tile_n)
    sym = nat.ns_gemm_tn(A, A, D, alpha, beta, False, True, tile_n)
    assert torch.equal(sym, sym.transpose(1, 2))
    assert torch.equal(torch.triu(sym), torch.triu(full))
    ref = alpha * torch.bmm(A.float(), A.float().transpose(1, 2)) + (beta * D.float() if with_d else 0.0)
    err = (sym.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-2, err


@pytest.mark.parametrize("M,N,K,batch,with_d,sym,want_t", [
    (256, 256, 64, 1, False, False, False), (256, 256, 128, 1, True, False, True), (512, 768, 192, 2, True, False, True),
    (512, 512, 256, 1, False, True, False), (2048, 2048, 192, 3, True, True, False), (256, 384, 72, 3, True, False, True),
    (1024, 4096, 1024, 2, True, False, True), (2048, 2048, 2048, 2, True, True, False)])
def test_cta_pair_kernel_matches_fp32_reference(M, N, K, batch, with_d, sym, want_t):
    """256 x 256 tiles on pairs of CTAs (cluster of two, ``tcgen05.mma.cta_group::2``, tile selector 512): plain and
    symmetric products, the beta operand, the transposed second output, partial column tiles (N = 384), ring and
    accumulator wrap-around ((2048, 2048, 192, 3): 108 tiles on at most 74 pairs, 3 k-blocks each)."""
    nat = _nat()
    torch.manual_seed(5)
    A = (torch.randn(batch, M, K, device="cuda") * 0.5).bfloat16()
    B = A if sym else (torch.randn(batch, N, K, device="cuda") * 0.5).bfloat16()
    D = None
    if with_d:
        D = torch.randn(batch, M, N, device="cuda")
        D = ((D + D.transpose(1, 2)) * 0.5 if sym else D).bfloat16()
    alpha, beta = 0.75, (-1.25 if with_d else 0.0)
    out = nat.ns_gemm_tn(A, B, D, alpha, beta, want_t, sym, 512)
    ref = alpha * torch.bmm(A.float(), B.float().transpose(1, 2)) + (beta * D.float() if with_d else 0.0)
    if want_t:
        C, Ct = out[0].view(batch, M, N), out[1].view(batch, N, M)
        assert torch.equal(Ct, C.transpose(1, 2))
        out = C
    if sym:
        assert torch.equal(out, out.transpose(1, 2))
    one_cta = nat.ns_gemm_tn(A, B, D, alpha, beta, False, sym, 256)
    assert torch.equal(out, one_cta)                      # same products, same accumulation order, same epilogue
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2


def test_many_tiles_per_cta_non_symmetric():
    nat = _nat()
    torch.manual_seed(3)
    A = (torch.randn(2, 2048, 320, device="cuda") * 0.3).bfloat16()
    B = (torch.randn(2, 2304, 320, device="cuda") * 0.3).bfloat16()
    D = torch.randn(2, 2048, 2304, device="cuda").bfloat16()
    both = nat.ns_gemm_tn(A, B, D, 1.0, 0.5, True)
    C = both[0].view(2, 2048, 2304)
    Ct = both[1].view(2, 2304, 2048)
    ref = torch.bmm(A.float(), B.float().transpose(1, 2)) + 0.5 * D.float()
    assert (C.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-2
    assert torch.equal(Ct, C.transpose(1, 2))


@pytest.mark.parametrize("shape", [(256, 384), (384, 256), (2, 128, 512), (3, 512, 128), (256, 256)])
def test_fused_orthogonalisation_matches_the_stepwise_path_and_writes_in_place(shape):
    """Norm + scale/transpose kernel + iteration + direct output against the same iteration driven step by step
    (torch norm and divide, explicit transposes, nat.ns_iterate)."""
    nat = _nat()
    torch.manual_seed(4)
    G = torch.randn(*shape, device="cuda").bfloat16()
    coeffs = [c for t in [NS.NS_COEFFS] * 5 for c in t]
    fused = nat.ns_orthogonalize(G.clone(), coeffs, 1e-7)
    X = G.float()
    X = (X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)).bfloat16()
    tall = X.shape[-2] > X.shape[-1]
    Y = nat.ns_iterate((X.transpose(-2, -1) if tall else X).contiguous(), coeffs)
    stepwise = Y.transpose(-2, -1) if tall else Y
    assert fused.shape == G.shape
    assert (fused.float() - stepwise.float()).abs().max() < 0.03       # same kernels; inputs differ by one bf16 rounding
    buf = G.clone()
    ret = NS.zeropower_via_newtonschulz5(buf, steps=5, out=buf) if len(shape) == 2 else \
        NS.zeropower_via_newtonschulz5_batched(buf, steps=5, out=buf)
    assert ret.data_ptr() == buf.data_ptr() and torch.equal(buf, fused)
    s = torch.linalg.svdvals(fused.float().reshape(-1, shape[-2], shape[-1])[0])
    assert s.max() < 1.3 and torch.quantile(s, 0.1) > 0.45
