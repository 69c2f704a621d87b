"""Fused sm_100a kernels against their fp32 torch oracle (engine_torch / model_ops CPU path)."""
import copy

import pytest
import torch
import torch.nn as nn

from apexw_b200 import ApexW, _native
from apexw_b200.ops import model_ops as M

pytestmark = pytest.mark.gpu


def _make(shapes, dtype, device, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [nn.Parameter((torch.randn(s, generator=g) * 0.05).to(dtype).to(device)) for s in shapes]


def _grads(ps, seed, scale=1e-3, dtype=None):
    g = torch.Generator().manual_seed(seed)
    for p in ps:
        p.grad = (torch.randn(p.shape, generator=g) * scale).to(dtype or p.dtype).to(p.device)


SHAPES = [(256, 128)] * 8 + [(128,), (64, 40), (3, 1000), (70,), (2048 * 3 + 8,), (16384 + 4,), (1,), (4096, 64)]


def _run_pair(prec, pdtype, steps=3, **kw):
    """Same parameters/gradients through the CUDA kernels and through the torch engine
    (plain torch fp32 ops on the same device: the numerical reference of these kernels)."""
    assert _native.available(), _native.load_error()
    pg = _make(SHAPES, pdtype, "cuda")
    pc = _make(SHAPES, pdtype, "cuda")
    og = ApexW(pg, lr=1e-2, precision=prec, weight_decay=0.1, seed=11, **kw)
    oc = ApexW(pc, lr=1e-2, precision=prec, weight_decay=0.1, seed=11, **kw)
    oc._native_ok = False
    for s in range(steps):
        _grads(pg, s)
        _grads(pc, s)
        og.step()
        oc.step()
    assert og._native_launches > 0 and oc._native_launches == 0
    return pg, pc, og, oc


def _close_params(a, b, frac=3e-3):
    """Kernel and reference use the same formula order and the same rounding bits; they differ only
    by the approximate sqrt/reciprocal in the update multiplier (relative error ~2^-21 on an update
    of about lr), which moves a bf16 result by one step in rare cases and an fp32 result in its
    last places."""
    af, bf = a.detach().float(), b.detach().float()
    diff = (af - bf).abs()
    if a.dtype == torch.bfloat16:
        ulp = bf.abs().clamp_min(1e-30) * 2.0 ** -7
        changed = (diff > 0).float().mean().item()
        assert changed <= frac, ("fraction of bf16 params that differ", tuple(a.shape), changed)
        # a one-step difference made in an early step persists (and can straddle a binade) in later ones
        assert (diff <= ulp * 4.5 + 1e-4).all(), ("bf16 diff beyond a few steps", tuple(a.shape), (diff / ulp).max().item())
    else:
        assert diff.max().item() <= 1e-7, ("fp32 param diff", tuple(a.shape), diff.max().item())


@pytest.mark.parametrize("pdtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("sr", [False, True])
@pytest.mark.parametrize("kw", [dict(), dict(nesterov=True), dict(maximize=True), dict(int4_m=False)])
def test_dense_kernel_matches_engine(pdtype, sr, kw):
    pg, pc, og, oc = _run_pair("compact", pdtype, stochastic_rounding=sr, force_compact_v=True, **kw)
    for a, b in zip(pg, pc):
        sa, sb = og.state[a], oc.state[b]
        # moments involve no approximate function: identical up to the rare double rounding of the
        # float64 fma emulation
        for k in ("exp_avg", "exp_avg_sq"):
            bad = (sa[k] != sb[k]).float().mean().item()
            assert bad < 1e-4, ("moment mismatch fraction", k, tuple(a.shape), bad, str(sa[k].dtype))
        _close_params(a, b)


@pytest.mark.parametrize("pdtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("sr", [False, True])
@pytest.mark.parametrize("kw", [dict(lion=True, betas=(0.9, 0.99)), dict(betas=(0.9, 0.999, 0.9999), alpha=5.0),
                                dict(amsgrad=True), dict(amsgrad=True, betas=(0.9, 0.999, 0.9999), nesterov=True)])
def test_lion_ademamix_amsgrad_run_on_the_dense_kernel(pdtype, sr, kw):
    """Sign updates, the slow first moment and the running maximum of the second moment are branches of the dense
    kernel's general path; every state tensor they keep must match the torch engine's."""
    pg, pc, og, oc = _run_pair("compact", pdtype, stochastic_rounding=sr, force_compact_v=True, **kw)
    assert og._native_launches >= 3
    keys = ["exp_avg"] if kw.get("lion") else ["exp_avg", "exp_avg_sq"]
    if len(kw.get("betas", ())) == 3:
        keys.append("exp_avg_slow")
    if kw.get("amsgrad"):
        keys.append("max_exp_avg_sq")
    for a, b in zip(pg, pc):
        sa, sb = og.state[a], oc.state[b]
        for k in keys:
            assert sa[k].dtype == sb[k].dtype and sa[k].shape == sb[k].shape
            bad = (sa[k] != sb[k]).float().mean().item()
            assert bad < 1e-4, ("state mismatch fraction", k, tuple(a.shape), bad, str(sa[k].dtype))
            if k in ("exp_avg_slow", "max_exp_avg_sq"):
                assert sa[k].float().abs().sum().item() > 0, (k, "was never written")
        _close_params(a, b)


@pytest.mark.parametrize("pdtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("sr", [False, True])
@pytest.mark.parametrize("kw", [dict(force_compact_v=True), dict(), dict(maximize=True, int4_m=False)])
def test_dense_cautious_runs_on_the_kernel(pdtype, sr, kw):
    """Cautious updates on dense state: a counting launch (what fraction of each tensor keeps its update) and the
    update launch; per-element and shared variances.  The moments do not depend on the mask and must be identical;
    the parameters see the mask and the kept fraction."""
    pg, pc, og, oc = _run_pair("compact", pdtype, stochastic_rounding=sr, cautious=True, **kw)
    assert og._native_launches >= 3 and oc._native_launches == 0
    for a, b in zip(pg, pc):
        sa, sb = og.state[a], oc.state[b]
        for k in ("exp_avg", "exp_avg_sq"):
            bad = (sa[k] != sb[k]).float().mean().item()
            assert bad < 1e-4, ("moment mismatch fraction", k, tuple(a.shape), bad, str(sa[k].dtype))
        _close_params(a, b)


def test_dense_cautious_differs_from_the_plain_update():
    """The mask is really applied: with and without `cautious` the kernel gives different parameters."""
    pa, _, oa, _ = _run_pair("compact", torch.float32, cautious=True)
    pb, _, ob, _ = _run_pair("compact", torch.float32)
    assert any((a - b).abs().max().item() > 1e-5 for a, b in zip(pa, pb))


@pytest.mark.parametrize("pdtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("sr", [False, True])
@pytest.mark.parametrize("kw", [dict(), dict(nesterov=True), dict(maximize=True), dict(betas=(0.9, 0.95))])
def test_ultra_layout_runs_on_the_kernel(pdtype, sr, kw):
    """precision="ultra": int8 first moment with one scale per block beside a 16/32-bit second moment per element."""
    pg, pc, og, oc = _run_pair("ultra", pdtype, stochastic_rounding=sr, **kw)
    n_ultra = 0
    for a, b in zip(pg, pc):
        sa, sb = og.state[a], oc.state[b]
        if sa.get("is_ultra", False):
            n_ultra += 1
            assert sa["exp_avg"].dtype == torch.int8
            # an approximate reciprocal never touches the moments: codes and scales are those of the torch engine,
            # up to the rare double rounding of the engine's float64 fma emulation (one code step)
            dm = (sa["exp_avg"].int() - sb["exp_avg"].int()).abs()
            assert dm.max().item() <= 1 and (dm > 0).float().mean().item() < 1e-3, tuple(a.shape)
            torch.testing.assert_close(sa["exp_avg_scales"], sb["exp_avg_scales"], rtol=1e-6, atol=0)
        bad = (sa["exp_avg_sq"] != sb["exp_avg_sq"]).float().mean().item()
        assert bad < 1e-4, ("second moment mismatch fraction", tuple(a.shape), bad, str(sa["exp_avg_sq"].dtype))
        _close_params(a, b)
    assert n_ultra >= 10 and og._native_launches >= 3


FACTORED_SHAPES = [(1024, 512), (512, 1024), (700, 1001), (130, 4099), (128,), (64, 40)]


@pytest.mark.parametrize("prec", ["compact", "8bit"])
@pytest.mark.parametrize("sr", [False, True])
@pytest.mark.parametrize("kw", [dict(), dict(nesterov=True), dict(maximize=True)])
def test_factored_second_moment_runs_on_the_kernels(prec, sr, kw):
    """factored_v=True: one statistic per row and per column.  A statistics launch (sums of g^2 through shared and
    global atomics), a finishing launch (moving averages, factor vectors) and the update launch; column counts that are
    no multiple of eight make a thread's eight elements straddle rows.  First moment bf16 (compact) or int8 (8bit)."""
    pg = _make(FACTORED_SHAPES, torch.bfloat16, "cuda")
    pc = _make(FACTORED_SHAPES, torch.bfloat16, "cuda")
    og = ApexW(pg, lr=1e-2, precision=prec, weight_decay=0.1, seed=11, factored_v=True, stochastic_rounding=sr, **kw)
    oc = ApexW(pc, lr=1e-2, precision=prec, weight_decay=0.1, seed=11, factored_v=True, stochastic_rounding=sr, **kw)
    oc._native_ok = False
    for s in range(3):
        _grads(pg, s)
        _grads(pc, s)
        for p in pg + pc:
            if p.dim() == 2:
                p.grad[1::2] *= 8      # neighbouring rows get very different statistics: a wrong row index would show
        og.step()
        oc.step()
    assert not og._execution_plans[id(og.param_groups[0])].fallback and oc._native_launches == 0
    n_fact = 0
    for a, b in zip(pg, pc):
        sa, sb = og.state[a], oc.state[b]
        if sa.get("is_factored_v", False):
            n_fact += 1
            # sums in a different order than torch's reductions: equal to rounding
            torch.testing.assert_close(sa["exp_avg_sq_row"], sb["exp_avg_sq_row"], rtol=2e-5, atol=1e-12)
            torch.testing.assert_close(sa["exp_avg_sq_col"], sb["exp_avg_sq_col"], rtol=2e-5, atol=1e-12)
            if sa["exp_avg"].dtype == torch.int8:
                dm = (sa["exp_avg"].int() - sb["exp_avg"].int()).abs()
                assert dm.max().item() <= 1 and (dm > 0).float().mean().item() < 1e-3, tuple(a.shape)
                torch.testing.assert_close(sa["exp_avg_scales"], sb["exp_avg_scales"], rtol=1e-6, atol=0)
            else:
                assert (sa["exp_avg"] != sb["exp_avg"]).float().mean().item() < 1e-4
        # The statistics are summed in another order than torch's reductions, so the denominators agree to ~1e-5 and a
        # parameter lands on the other side of a rounding boundary now and then.  Such a one-step difference is made at
        # the magnitude the parameter had then (up to 2^-10 for |p| < 0.25) and stays when the parameter later shrinks.
        diff = (a.detach().float() - b.detach().float()).abs()
        assert (diff > 0).float().mean().item() <= 5e-3, tuple(a.shape)
        assert (diff <= b.detach().float().abs() * 2.0 ** -7 * 4.5 + 1.1e-3).all(), (tuple(a.shape), diff.max().item())
    assert n_fact == 4


@pytest.mark.parametrize("prec", ["8bit", "ultra"])
@pytest.mark.parametrize("pdtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("sr", [False, True])
def test_lion_with_int8_momentum_runs_on_the_kernel(prec, pdtype, sr):
    """Lion keeps one moment; with precision 8bit / ultra it is int8 with a scale per block (64 to 2048 elements)."""
    pg, pc, og, oc = _run_pair(prec, pdtype, stochastic_rounding=sr, lion=True, betas=(0.9, 0.99))
    n_int8 = 0
    for a, b in zip(pg, pc):
        sa, sb = og.state[a], oc.state[b]
        assert "exp_avg_sq" not in sa
        if sa["exp_avg"].dtype == torch.int8:
            n_int8 += 1
            dm = (sa["exp_avg"].int() - sb["exp_avg"].int()).abs()
            assert dm.max().item() <= 1 and (dm > 0).float().mean().item() < 1e-3, tuple(a.shape)
            torch.testing.assert_close(sa["exp_avg_scales"], sb["exp_avg_scales"], rtol=1e-6, atol=0)
        _close_params(a, b)
    assert n_int8 >= 11 and og._native_launches >= 3
    assert not og._execution_plans[id(og.param_groups[0])].fallback


def test_full_precision_kernel_matches_adamw():
    pg, pc, og, oc = _run_pair("full", torch.float32, adamw_compat=True)
    pr = _make(SHAPES, torch.float32, "cuda")
    ref = torch.optim.AdamW(pr, lr=1e-2, weight_decay=0.1)
    for s in range(3):
        _grads(pr, s)
        ref.step()
    for a, b, r in zip(pg, pc, pr):
        assert (a - r).abs().max() < 5e-6 and (a - b).abs().max() < 5e-6


@pytest.mark.parametrize("pdtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("sr", [False, True])
@pytest.mark.parametrize("kw", [dict(), dict(cautious=True), dict(int4_m=False), dict(int4_m=True), dict(block_size=256), dict(nesterov=True)])
def test_quant_kernel_matches_engine(pdtype, sr, kw):
    pg, pc, og, oc = _run_pair("8bit", pdtype, stochastic_rounding=sr, **kw)
    for a, b in zip(pg, pc):
        sa, sb = og.state[a], oc.state[b]
        for k in ("is_8bit", "is_4bit_m", "is_quad_v"):
            assert sa.get(k) == sb.get(k), (k, sa.get(k), sb.get(k), tuple(a.shape))
        if not sa.get("is_8bit"):
            _close_params(a, b)
            continue
        # scales and first-moment codes: exact.  log-u8 codes: device log2f may differ from the
        # host's in the last place, which moves a code by one step in rare boundary cases.
        for k in ("exp_avg_scales", "exp_avg_sq_scales"):
            rel = ((sa[k] - sb[k]).abs() / sb[k].abs().clamp_min(1e-30)).max().item()
            assert rel < 1e-5, ("scale mismatch", k, tuple(a.shape), rel)
        m_bad = (sa["exp_avg"] != sb["exp_avg"]).float().mean().item()
        dv = (sa["exp_avg_sq"].int() - sb["exp_avg_sq"].int()).abs()
        assert m_bad < 2e-3, ("first-moment code mismatch", tuple(a.shape), m_bad)
        # log-u8 codes: the kernel's lg2.approx may differ from torch.log2 in the last place
        assert dv.max().item() <= 1 and (dv > 0).float().mean().item() < 5e-3, ("log-u8 codes", tuple(a.shape), dv.max().item(), (dv > 0).float().mean().item())
        diff = (a.detach().float() - b.detach().float()).abs()
        if a.dtype == torch.bfloat16:
            assert (diff > 0).float().mean().item() < 1e-2, ("bf16 params differ", tuple(a.shape), (diff > 0).float().mean().item())
        assert diff.max().item() < 1e-3, ("param diff", tuple(a.shape), diff.max().item())


def test_state_bytes_on_gpu_and_checkpoint_cross_device():
    pg, pc, og, oc = _run_pair("8bit", torch.bfloat16, stochastic_rounding=False)
    sd = og.state_dict()
    p2 = [nn.Parameter(p.detach().cpu().clone()) for p in pg]
    o2 = ApexW(p2, lr=1e-2, precision="8bit", weight_decay=0.1, seed=11, stochastic_rounding=False)
    o2.load_state_dict(sd)
    _grads(pg, 9)
    _grads(p2, 9)
    og.step()
    o2.step()
    bad = sum(((a.detach().cpu().float() - b.detach().float()).abs() > 1e-3).sum().item() for a, b in zip(pg, p2))
    assert bad == 0


def test_kernel_found_inf_and_grad_scale_on_device():
    pg = _make(SHAPES[:9], torch.bfloat16, "cuda")
    pr = _make(SHAPES[:9], torch.bfloat16, "cuda")
    og = ApexW(pg, lr=1e-2, precision="compact", seed=3)
    orf = ApexW(pr, lr=1e-2, precision="compact", seed=3)
    _grads(pg, 0, scale=1e-3 * 64.0)
    _grads(pr, 0, scale=1e-3)
    og.grad_scale = torch.tensor(64.0, device="cuda")
    og.step()
    orf.step()
    for a, b in zip(pg, pr):
        assert (a.float() - b.float()).abs().max() < 2e-3


def test_stochastic_rounding_statistics_on_device():
    """Mean of many SR steps approaches the fp32 trajectory (unbiasedness)."""
    torch.manual_seed(0)
    base = torch.full((16384,), 1.0, dtype=torch.bfloat16, device="cuda")
    ps = [nn.Parameter(base.clone()) for _ in range(8)]
    opt = ApexW(ps, lr=1e-4, precision="compact", weight_decay=0.0, betas=(0.0, 0.0), eps=1e-8, seed=5)
    for s in range(20):
        for p in ps:
            p.grad = torch.ones_like(p)
        opt.step()
    # each step wants to subtract 1e-4 (ulp of bf16 at 1.0 is 2^-7 below 1): expectation 1 - 20e-4
    mean = torch.stack([p.float().mean() for p in ps]).mean().item()
    assert abs(mean - (1.0 - 20e-4)) < 2e-4


# ---------------------------------------------------------------------------
# model-side ops
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("H", [128, 4096, 8192])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm_fwd_bwd(dtype, H, with_res):
    torch.manual_seed(0)
    x = torch.randn(37, H, device="cuda").to(dtype).requires_grad_(True)
    r = torch.randn(37, H, device="cuda").to(dtype).requires_grad_(True) if with_res else None
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(dtype).requires_grad_(True)
    y, h = M.rms_norm(x, w, 1e-5, r)
    dy, dh = torch.randn_like(y), torch.randn_like(y)
    (y * dy).sum().backward() if not with_res else ((y * dy).sum() + (h * dh).sum()).backward()
    xf = x.detach().float() + (r.detach().float() if with_res else 0)
    if with_res:
        xf = xf.to(dtype).float()
    xf.requires_grad_(True)
    wf = w.detach().float().requires_grad_(True)
    yf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    ((yf * dy.float()).sum() + ((xf * dh.float()).sum() if with_res else 0)).backward()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert (y.float() - yf).abs().max() < tol * max(1.0, yf.abs().max().item())
    assert (x.grad.float() - xf.grad).abs().max() < tol * max(1.0, xf.grad.abs().max().item())
    assert (w.grad.float() - wf.grad).abs().max() < tol * max(1.0, wf.grad.abs().max().item())
    if with_res:
        assert torch.equal(x.grad, r.grad)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_swiglu_rope_cross_entropy(dtype):
    torch.manual_seed(0)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    gu = torch.randn(50, 2 * 1024, device="cuda").to(dtype).requires_grad_(True)
    y = M.swiglu(gu)
    dy = torch.randn_like(y)
    (y * dy).sum().backward()
    gf = gu.detach().float().requires_grad_(True)
    a, b = gf.chunk(2, -1)
    yf = torch.nn.functional.silu(a) * b
    (yf * dy.float()).sum().backward()
    assert (y.float() - yf).abs().max() < tol * 4 and (gu.grad.float() - gf.grad).abs().max() < tol * 4

    B, S, Hq, Hkv, D = 2, 33, 8, 2, 128
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, device="cuda").to(dtype).requires_grad_(True)
    cos, sin = M.rope_tables(64, D, 10000.0, "cuda")
    out = M.rope_qkv(qkv, cos, sin, Hq + Hkv)
    ref = qkv.detach().clone()
    ref[:, :, :Hq + Hkv] = M._rope_torch(qkv.detach()[:, :, :Hq + Hkv], cos, sin, 1.0)
    assert (out.float() - ref.float()).abs().max() < tol
    assert torch.equal(out[:, :, Hq + Hkv:], qkv[:, :, Hq + Hkv:])
    d = torch.randn_like(out)
    (out * d).sum().backward()
    refg = d.clone()
    refg[:, :, :Hq + Hkv] = M._rope_torch(d[:, :, :Hq + Hkv], cos, sin, -1.0)
    assert (qkv.grad.float() - refg.float()).abs().max() < tol * 4

    T, V, Hd = 96, 1000 if dtype == torch.float32 else 1024, 64
    h = (torch.randn(T, Hd, device="cuda") * 0.5).to(dtype).requires_grad_(True)
    W = (torch.randn(V, Hd, device="cuda") * 0.2).to(dtype).requires_grad_(True)
    tgt = torch.randint(0, V, (T,), device="cuda")
    loss = M.linear_cross_entropy(h, W, tgt, chunk_rows=40)
    loss.backward()
    hf, Wf = h.detach().float().requires_grad_(True), W.detach().float().requires_grad_(True)
    lf = torch.nn.functional.cross_entropy(hf @ Wf.t(), tgt)
    lf.backward()
    assert abs(loss.item() - lf.item()) < tol
    assert (h.grad.float() - hf.grad).abs().max() < tol * 0.1 + 1e-5
    assert (W.grad.float() - Wf.grad).abs().max() < tol * 0.1 + 1e-5


def test_llama_tiny_gpu_matches_cpu_and_trains():
    from apexw_b200.models.llama import build_llama
    mc = build_llama("tiny", device="cpu", dtype=torch.float32)
    mg = build_llama("tiny", device="cuda", dtype=torch.float32)
    mg.load_state_dict(mc.state_dict())
    tok = torch.randint(0, 512, (2, 64))
    tgt = torch.randint(0, 512, (2, 64))
    lc = mc(tok, tgt)
    lg = mg(tok.cuda(), tgt.cuda())
    lc.backward()
    lg.backward()
    assert abs(lc.item() - lg.item()) < 1e-3
    for (n, a), (_, b) in zip(mc.named_parameters(), mg.named_parameters()):
        assert (a.grad - b.grad.cpu()).abs().max() < 1e-3 * max(1.0, a.grad.abs().max().item()), n
    mb = build_llama("tiny", device="cuda", dtype=torch.bfloat16)
    opt = ApexW(mb, lr=3e-3, precision="compact")
    first = None
    for _ in range(30):
        opt.zero_grad()
        loss = mb(tok.cuda(), tgt.cuda())
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < first * 0.7


EDGE_NUMELS = [1, 2, 3, 5, 7, 8, 9, 15, 16, 17, 31, 33, 255, 256, 257, 2047, 2048, 2049, 2055, 4095, 4097, 6143, 8191, 8192, 8195]


def _edge_params(dtype, device, seed):
    """Every size of EDGE_NUMELS at every start offset 0..7 elements inside one buffer (byte misalignment 0..14
    for bf16, 0..28 for fp32): tails, chunk and block boundaries, unaligned vector accesses."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for i, n in enumerate(EDGE_NUMELS):
        off = i % 8
        buf = (torch.randn(n + 8, generator=g) * 0.05).to(dtype).to(device)
        p = nn.Parameter(buf[off:off + n])
        assert p.data_ptr() == buf.data_ptr() + off * buf.element_size()
        out.append(p)
    return out


def _edge_grads(ps, seed):
    g = torch.Generator().manual_seed(seed)
    for i, p in enumerate(ps):
        off = (i * 3 + 1) % 8
        buf = (torch.randn(p.numel() + 8, generator=g) * 1e-3).to(p.dtype).to(p.device)
        p.grad = buf[off:off + p.numel()]


@pytest.mark.parametrize("prec", ["compact", "8bit"])
@pytest.mark.parametrize("pdtype", [torch.bfloat16, torch.float32])
def test_edge_sizes_and_misaligned_views(prec, pdtype):
    pg, pc = _edge_params(pdtype, "cuda", 5), _edge_params(pdtype, "cuda", 5)
    kw = dict(force_compact_v=True) if prec == "compact" else dict(block_size=256)
    og = ApexW(pg, lr=1e-2, precision=prec, weight_decay=0.1, seed=4, **kw)
    oc = ApexW(pc, lr=1e-2, precision=prec, weight_decay=0.1, seed=4, **kw)
    oc._native_ok = False
    for s in range(2):
        _edge_grads(pg, s)
        _edge_grads(pc, s)
        og.step()
        oc.step()
    assert og._native_launches > 0 and oc._native_launches == 0
    for a, b in zip(pg, pc):
        diff = (a.detach().float() - b.detach().float()).abs()
        assert diff.max().item() < 1e-3, (a.numel(), diff.max().item())
        if a.dtype == torch.bfloat16:
            assert (diff > 0).float().mean().item() <= 0.02 or a.numel() < 64, (a.numel(), (diff > 0).float().mean().item())
        sa, sb = og.state[a], oc.state[b]
        for k in ("exp_avg", "exp_avg_sq"):
            assert sa[k].shape == sb[k].shape and sa[k].dtype == sb[k].dtype
            if sa[k].dtype in (torch.uint8, torch.int8):
                # codes may move by one step where the approximate log2 / reciprocal lands on a boundary
                d = (sa[k].int() - sb[k].int()).abs()
                assert (d > 0).float().mean().item() <= 0.02 or a.numel() < 64, (k, a.numel())
            else:
                assert (sa[k] != sb[k]).float().mean().item() <= 1e-3 or a.numel() < 64, (k, a.numel())


def test_cached_plans_follow_parameters_that_were_re_homed():
    """``p.data`` moved to new storage after the first step (what ``model.to()``, ``flatten_parameters`` or a sharding
    wrapper does): the cached launch plan holds the old address and must be rebuilt, or the live parameters would
    silently stop training while the kernel keeps updating memory nobody reads."""
    pg, pc, og, oc = _run_pair("compact", torch.bfloat16, steps=2, stochastic_rounding=False)
    old = [p.data for p in pg]
    for p in pg:
        p.data = p.data.clone()
    frozen = [t.clone() for t in old]
    _grads(pg, 7)
    _grads(pc, 7)
    og.step()
    oc.step()
    for a, b, o, f in zip(pg, pc, old, frozen):
        assert torch.equal(o, f)                 # the abandoned storage is no longer written
        _close_params(a, b)


def test_a_parameter_that_sat_out_steps_keeps_its_own_bias_correction():
    """Unused parameters (gradient None on some steps) fall behind in step count.  When they come back, the same set
    of parameters is stepped as before, but one launch applies one step count: the plan has to be re-bucketed."""
    pg, pc, og, oc = _run_pair("compact", torch.bfloat16, steps=1, stochastic_rounding=False)
    for s in (1, 2):                             # two steps without the first two parameters
        _grads(pg, 20 + s)
        _grads(pc, 20 + s)
        for ps in (pg, pc):
            ps[0].grad = None
            ps[1].grad = None
        og.step()
        oc.step()
    _grads(pg, 30)
    _grads(pc, 30)
    og.step()
    oc.step()
    assert float(og.state[pg[0]]["step"]) == 2.0 and float(og.state[pg[2]]["step"]) == 4.0
    for a, b in zip(pg, pc):
        for k in ("exp_avg", "exp_avg_sq"):
            assert (og.state[a][k] != oc.state[b][k]).float().mean().item() < 1e-4
        _close_params(a, b)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_cross_entropy_ignores_targets_outside_the_vocabulary(dtype):
    """-100 (the usual ignore_index) and any other out-of-range target must be ignored rows - zero loss, zero
    gradient - and never an index into the logits row.  Oracle: torch's fp32 cross-entropy with ignore_index."""
    torch.manual_seed(1)
    T, V, Hd = 64, 1024, 64
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    h = (torch.randn(T, Hd, device="cuda") * 0.5).to(dtype).requires_grad_(True)
    W = (torch.randn(V, Hd, device="cuda") * 0.2).to(dtype).requires_grad_(True)
    tgt = torch.randint(0, V, (T,), device="cuda")
    tgt[::3] = -100
    tgt[5] = V + 7            # a stray value: ignored as well, not read out of bounds
    loss = M.linear_cross_entropy(h, W, tgt, chunk_rows=24, ignore_index=-100)
    loss.backward()
    hf, Wf = h.detach().float().requires_grad_(True), W.detach().float().requires_grad_(True)
    ref_t = tgt.clone()
    ref_t[5] = -100
    lf = torch.nn.functional.cross_entropy(hf @ Wf.t(), ref_t, ignore_index=-100)
    lf.backward()
    assert abs(loss.item() - lf.item()) < tol
    assert (h.grad.float() - hf.grad).abs().max() < tol * 0.1 + 1e-5
    assert (W.grad.float() - Wf.grad).abs().max() < tol * 0.1 + 1e-5
    assert float(h.grad[::3].abs().max()) == 0.0 and float(h.grad[5].abs().max()) == 0.0
    # the raw kernel, without ignore_index: ignored rows still give zero loss and gradient (mean over all rows)
    logits = (h.detach() @ W.detach().t()).contiguous()
    losses = _native.require().cross_entropy_fwd_bwd(logits, tgt, 1.0)
    assert float(losses[::3].abs().max()) == 0.0 and float(logits[::3].abs().max()) == 0.0
    assert float(losses[1]) > 0.0


@pytest.mark.parametrize("prec", ["compact", "8bit"])
def test_flat_parameter_decays_its_matrices_inside_the_kernel(prec):
    """A flat one-dimensional parameter that holds matrices and vectors (an FSDP flat shard, a flattened model): the
    matrices' ranges decay, the rest does not, decided per 2048-element chunk from a side table of the launch plan and,
    in chunks that a range boundary cuts (here at odd offsets, inside quantisation blocks), per element from a bit
    mask.  Kernel against the torch engine with the same element mask; and against the pieces stepped separately."""
    sizes = [(64, 300), (300,), (129, 77), (77,), (256, 256), (5,), (40, 1000)]          # matrix / vector alternate
    n = sum(int(torch.tensor(s).prod()) for s in sizes)
    ranges, off = [], 0
    for s in sizes:
        k = int(torch.tensor(s).prod())
        if len(s) == 2:
            ranges.append((off, off + k))
        off += k
    g0 = torch.Generator().manual_seed(21)
    init = (torch.randn(n, generator=g0) * 0.05).bfloat16()
    flats = []
    for _ in range(2):
        f = nn.Parameter(init.clone().cuda())
        f._apexw_decay_ranges = list(ranges)
        flats.append(f)
    kw = dict(lr=1e-2, precision=prec, weight_decay=0.1, seed=11, stochastic_rounding=False)
    og, oc = ApexW([flats[0]], **kw), ApexW([flats[1]], **kw)
    oc._native_ok = False
    for s in range(3):
        g = (torch.randn(n, generator=torch.Generator().manual_seed(50 + s)) * 1e-3).bfloat16().cuda()
        flats[0].grad, flats[1].grad = g.clone(), g.clone()
        og.step()
        oc.step()
    assert og._native_launches > 0 and oc._native_launches == 0
    plan = next(iter(og._execution_plans.values()))
    assert plan.classes[0][0].mixed_decay_chunks > 0                      # some chunks are cut by a range boundary
    for k in ("exp_avg", "exp_avg_sq"):
        assert (og.state[flats[0]][k] != oc.state[flats[1]][k]).float().mean().item() < 1e-4
    _close_params(flats[0], flats[1])
    # the decay really is partial: a run without weight decay differs on the matrices' ranges and nowhere else
    f2 = nn.Parameter(init.clone().cuda())
    o2 = ApexW([f2], **{**kw, "weight_decay": 0.0})
    for s in range(3):
        f2.grad = (torch.randn(n, generator=torch.Generator().manual_seed(50 + s)) * 1e-3).bfloat16().cuda()
        o2.step()
    mask = torch.zeros(n, dtype=torch.bool, device="cuda")
    for a, b in ranges:
        mask[a:b] = True
    differs = flats[0].data != f2.data
    assert not bool(differs[~mask].any())
    assert differs[mask].float().mean().item() > 0.2          # three steps of 0.1 % decay move some, not all, bf16 values


@pytest.mark.parametrize("sr", [False, True])
@pytest.mark.parametrize("kw", [dict(), dict(int4_m=False), dict(nesterov=True)])
def test_fp16_parameters_and_moments_run_on_the_kernel(sr, kw):
    """fp16 parameters, gradients and moments (second moment stored times its per-tensor scale 4^k): the kernel's
    general path against the torch engine.  Rounding goes through the conversion unit (cvt.rs.satfinite.f16x2.f32),
    whose rule the engine restates, so the moments agree and the parameters differ in rare last places only."""
    assert _native.available(), _native.load_error()
    pg, pc = _make(SHAPES, torch.float16, "cuda"), _make(SHAPES, torch.float16, "cuda")
    og = ApexW(pg, lr=1e-2, precision="compact", weight_decay=0.1, seed=11, stochastic_rounding=sr, **kw)
    oc = ApexW(pc, lr=1e-2, precision="compact", weight_decay=0.1, seed=11, stochastic_rounding=sr, **kw)
    oc._native_ok = False
    for s in range(3):
        _grads(pg, s)
        _grads(pc, s)
        og.step()
        oc.step()
    assert og._native_launches > 0 and oc._native_launches == 0
    assert all(og.state[p]["exp_avg"].dtype == torch.float16 for p in pg)
    assert any(float(og.state[p].get("scale_v", 1.0)) == 1024.0 for p in pg)            # scaled fp16 second moments were used
    for a, b in zip(pg, pc):
        for k in ("exp_avg", "exp_avg_sq"):
            bad = (og.state[a][k] != oc.state[b][k]).float().mean().item()
            assert bad < 2e-3, ("moment mismatch fraction", k, tuple(a.shape), bad)
        af, bf = a.detach().float(), b.detach().float()
        ulp = bf.abs().clamp_min(6.1e-5) * 2.0 ** -10
        # the approximate square root / reciprocal of the kernel moves an update by ~2^-21 of itself; fp16 keeps three
        # more mantissa bits than bf16, so that flips a last place (or a rounding draw) eight times as often
        assert ((af - bf).abs() > 0).float().mean().item() <= 2e-2
        # a one-step difference made while a value was large persists after an update has carried it close to zero
        assert ((af - bf).abs() <= ulp * 4.5 + 1e-4).all()


def test_fp16_hundred_steps_stay_finite_and_learn():
    """A hundred steps on fp16 parameters with fp16 state on the kernel, across one re-centring of the second-moment
    scale (step 100): no NaN or Inf anywhere, and the quadratic loss goes down."""
    torch.manual_seed(0)
    w = nn.Parameter((torch.randn(256, 64) * 0.5).half().cuda())
    target = (torch.randn(256, 64) * 0.5).half().cuda()
    opt = ApexW([w], lr=3e-3, precision="compact", weight_decay=0.0, seed=1)
    first = None
    for s in range(101):
        loss = ((w.float() - target.float()) ** 2).mean()
        first = first if first is not None else float(loss.detach())
        w.grad = ((w.float() - target.float()) * (2.0 / w.numel())).half() * 256.0     # a loss-scaled gradient ...
        opt.grad_scale = torch.tensor(256.0, device="cuda")                             # ... unscaled inside the kernel
        opt.step()
    assert opt._native_launches >= 100
    st = opt.state[w]
    assert torch.isfinite(w).all() and torch.isfinite(st["exp_avg"].float()).all() and torch.isfinite(st["exp_avg_sq"].float()).all()
    assert float(((w.float() - target.float()) ** 2).mean()) < 0.8 * first


@pytest.mark.parametrize("prec", ["compact", "8bit"])
def test_many_segments_and_many_chunks_per_thread_block(prec):
    """Three hundred tensors of assorted sizes, forty million elements: every persistent thread block walks dozens of
    chunks across many segments of the resident table (cursor seeks, prefetch, the rotating slots of the block maxima),
    which the small cases above do not reach.  Same oracle, same tolerances: moments identical up to the rare double
    rounding of the emulated fma, parameters within a bf16 step on a small fraction."""
    assert _native.available(), _native.load_error()
    g = torch.Generator().manual_seed(123)
    sizes = [int(x) for x in torch.randint(1, 300000, (300,), generator=g)]
    shapes = [(n,) if i % 3 else (max(1, n // 64), 64) for i, n in enumerate(sizes)]
    pg = [nn.Parameter((torch.randn(s, generator=g) * 0.05).bfloat16().cuda()) for s in shapes]
    pc = [nn.Parameter(p.detach().clone()) for p in pg]
    og = ApexW(pg, lr=1e-2, precision=prec, weight_decay=0.1, seed=11, stochastic_rounding=True)
    oc = ApexW(pc, lr=1e-2, precision=prec, weight_decay=0.1, seed=11, stochastic_rounding=True)
    oc._native_ok = False
    for s in range(2):
        gg = torch.Generator().manual_seed(900 + s)
        for a, b in zip(pg, pc):
            grad = (torch.randn(a.shape, generator=gg) * 1e-3).bfloat16().cuda()
            a.grad, b.grad = grad, grad.clone()
        og.step()
        oc.step()
    assert og._native_launches > 0 and oc._native_launches == 0
    total = sum(p.numel() for p in pg)
    bad_m = sum(int((og.state[a]["exp_avg"] != oc.state[b]["exp_avg"]).sum()) for a, b in zip(pg, pc))
    bad_v = sum(int((og.state[a]["exp_avg_sq"] != oc.state[b]["exp_avg_sq"]).sum()) for a, b in zip(pg, pc))
    limit = 1e-4 if prec == "compact" else 2e-3          # a 4-bit / log-8-bit code can flip where a last place differs
    assert bad_m <= limit * total and bad_v <= limit * total, (bad_m, bad_v, total)
    if prec == "compact":
        for a, b in zip(pg, pc):
            _close_params(a, b)
    else:
        diff = torch.cat([(a.detach().float() - b.detach().float()).abs().flatten() for a, b in zip(pg, pc)])
        assert float(diff.max()) < 1e-3 and float((diff > 0).float().mean()) < 5e-3


def _pair_with(kw_kernel, kw_ref, steps=3, prec="compact", pdtype=torch.bfloat16, before_step=None):
    """Kernel run with ``kw_kernel`` against a kernel run with ``kw_ref`` on the same gradients (no rounding noise)."""
    pa, pb = _make(SHAPES, pdtype, "cuda"), _make(SHAPES, pdtype, "cuda")
    oa = ApexW(pa, precision=prec, weight_decay=0.1, seed=11, stochastic_rounding=False, **kw_kernel)
    ob = ApexW(pb, precision=prec, weight_decay=0.1, seed=11, stochastic_rounding=False, **kw_ref)
    for s in range(steps):
        if before_step is not None:
            before_step(s, oa, ob)
        _grads(pa, s)
        _grads(pb, s)
        oa.step()
        ob.step()
    assert oa._native_launches > 0 and ob._native_launches > 0
    return pa, pb, oa, ob


@pytest.mark.parametrize("prec", ["compact", "8bit"])
def test_capturable_steps_run_on_the_kernel_with_the_counter_on_the_device(prec):
    """capturable=True keeps the step count on the device; a one-thread kernel derives the bias corrections there and
    the update kernel reads them, so nothing is read back.  Same result as the host-scalar launch (the corrections are
    computed in double precision on both sides and rounded to fp32 once)."""
    pa, pb, oa, ob = _pair_with(dict(lr=1e-2, capturable=True), dict(lr=1e-2), prec=prec)
    st = oa.state[pa[0]]
    assert st["step"].is_cuda and float(st["step"]) == 3.0
    assert not oa._execution_plans[id(oa.param_groups[0])].fallback
    for a, b in zip(pa, pb):
        _close_params(a, b)


def test_a_learning_rate_tensor_on_the_device_is_read_by_the_kernel():
    lr_t = torch.tensor(1e-2, device="cuda")
    sched = [1e-2, 5e-3, 2.5e-3]

    def before(s, oa, ob):
        lr_t.fill_(sched[s])                       # a scheduler that writes the tensor in place
        ob.param_groups[0]["lr"] = sched[s]

    pa, pb, oa, ob = _pair_with(dict(lr=lr_t), dict(lr=sched[0]), before_step=before)
    assert not oa._execution_plans[id(oa.param_groups[0])].fallback
    for a, b in zip(pa, pb):
        _close_params(a, b)


@pytest.mark.parametrize("prec", ["compact", "8bit"])
def test_the_step_is_captured_in_a_cuda_graph_and_replayed(prec):
    """Three eager warm-up steps, then ``step()`` is captured once and replayed three times with fresh gradients in
    the same buffers; the device-side counters advance with every replay.  Compared with six eager steps."""
    pa, pb = _make(SHAPES, torch.bfloat16, "cuda"), _make(SHAPES, torch.bfloat16, "cuda")
    oa = ApexW(pa, lr=1e-2, precision=prec, weight_decay=0.1, seed=11, stochastic_rounding=False, capturable=True)
    ob = ApexW(pb, lr=1e-2, precision=prec, weight_decay=0.1, seed=11, stochastic_rounding=False)
    for p in pa:
        p.grad = torch.zeros_like(p)               # static gradient buffers: the graph reads these addresses

    def load(step):
        g = torch.Generator().manual_seed(step)
        for p, q in zip(pa, pb):
            fresh = (torch.randn(p.shape, generator=g) * 1e-3).to(p.dtype).to(p.device)
            p.grad.copy_(fresh)
            q.grad = fresh.clone()

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for s in range(3):
            load(s)
            oa.step()
            ob.step()
    torch.cuda.current_stream().wait_stream(side)
    launches_before = oa._native_launches
    graph = torch.cuda.CUDAGraph()
    load(3)
    with torch.cuda.graph(graph):
        oa.step()
    assert oa._native_launches > launches_before          # the capture went through the kernels, not the torch engine
    graph.replay()                                         # (capturing does not execute: this is step 4)
    ob.step()
    for s in (4, 5):
        load(s)
        graph.replay()
        ob.step()
    torch.cuda.synchronize()
    assert float(oa.state[pa[0]]["step"]) == 6.0
    for a, b in zip(pa, pb):
        _close_params(a, b)


def test_options_switched_on_after_the_first_step_rebuild_the_plan():
    """AMSGrad and the slow moment of AdEMAMix may be enabled on a live optimizer; their buffers are created late and
    the cached launch plan (which did not know them) must not be reused."""
    pg, pc = _make(SHAPES, torch.bfloat16, "cuda"), _make(SHAPES, torch.bfloat16, "cuda")
    og = ApexW(pg, lr=1e-2, precision="compact", weight_decay=0.1, seed=11, force_compact_v=True, int4_m=False)
    oc = ApexW(pc, lr=1e-2, precision="compact", weight_decay=0.1, seed=11, force_compact_v=True, int4_m=False)
    oc._native_ok = False
    for s in range(4):
        if s == 2:
            for o in (og, oc):
                o.param_groups[0]["amsgrad"] = True
        _grads(pg, s)
        _grads(pc, s)
        og.step()
        oc.step()
    assert not og._execution_plans[id(og.param_groups[0])].fallback
    for a, b in zip(pg, pc):
        assert "max_exp_avg_sq" in og.state[a]
        assert (og.state[a]["max_exp_avg_sq"] != oc.state[b]["max_exp_avg_sq"]).float().mean().item() < 1e-4
        _close_params(a, b)
