"""Distributed Muon over peer memory: the gather / scatter kernels against the torch path on one GPU, the
bounded entry wait, and (with >= 2 GPUs) two ranks that hold different gradients."""
import datetime
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp
import torch.nn as nn

from apexw_b200 import _native
from apexw_b200.parallel.fsdp import DistMuon

pytestmark = pytest.mark.gpu

SHAPES = [(256, 128), (256, 128), (128, 384), (256,), (256, 128), (64, 40), (128, 128, 2)]


def _mk(dev, seed=0):
    g = torch.Generator().manual_seed(seed)
    # small initial values: a bf16 step of the parameters (<= 6e-5 below 1.6e-2) stays far below one update (lr * U ~ 1e-3)
    return [nn.Parameter((torch.randn(s, generator=g) * 0.002).bfloat16().to(dev)) for s in SHAPES]


def _grads(step):
    g = torch.Generator().manual_seed(200 + step)
    return [(torch.randn(s, generator=g) * 1e-2).bfloat16() for s in SHAPES]


def _close(a, b, lr):
    # both paths orthogonalise the same bf16 input with the same kernels; what differs is one fused rounding of
    # p*decay - lr*U here against two bf16 roundings in the torch path, i.e. a few bf16 steps of the parameter
    d = (a.float() - b.float()).abs()
    assert float(d.max()) <= 0.02 * lr, float(d.max())
    assert float(d.mean()) <= 0.002 * lr, float(d.mean())


@pytest.mark.parametrize("nesterov", [True, False])
def test_world1_fused_matches_torch_path(nesterov):
    dev = torch.device("cuda")
    pf, pt = _mk(dev), _mk(dev)
    lr = 2e-2
    of = DistMuon(pf, lr=lr, nesterov=nesterov, weight_decay=0.01)
    ot = DistMuon(pt, lr=lr, nesterov=nesterov, weight_decay=0.01, fused=False)
    assert of._fused and not ot._fused
    before = _native.launch_count()
    for s in range(3):
        for p, q, g in zip(pf, pt, _grads(s)):
            p.grad.copy_(g.to(dev))
            q.grad = g.to(dev)
        of.step()
        ot.step()
    of.check_status()
    assert _native.launch_count() > before
    for a, b in zip(pf, pt):
        _close(a.data, b.data, 3 * lr)
    # fp32 momentum of the fused path equals the torch path's (same averaging, world of 1)
    for p, q in zip(pf, pt):
        torch.testing.assert_close(of.state[p]["momentum"], ot.state[q]["momentum"], rtol=1e-5, atol=1e-7)
        assert of.state[p]["step"] == 3


def test_fresh_gradients_are_adopted_into_the_flat_buffer():
    dev = torch.device("cuda")
    ps = _mk(dev)
    opt = DistMuon(ps, lr=1e-2)
    for p in ps:
        p.grad = None                                 # what model.zero_grad(set_to_none=True) leaves behind
    (sum((p.float() ** 2).sum() for p in ps)).backward()
    stray = [p.grad.clone() for p in ps]
    before = [p.data.clone() for p in ps]
    opt.step()
    opt.check_status()
    base = opt._store.grad.data_ptr()
    for p, g, b in zip(ps, stray, before):
        assert base <= p.grad.data_ptr() < base + opt._store.grad.numel() * 2
        assert torch.equal(p.grad, g)
        assert not torch.equal(p.data, b)


def test_gather_entry_wait_runs_out_and_scatter_keeps_parameters():
    """World of 2 faked on one GPU with a second signal pad that nothing writes: the gather kernel reports
    status 1 without touching momentum or staging, and the scatter kernel then leaves the parameters alone."""
    nat = _native.require()
    dev = torch.device("cuda")
    from apexw_b200.parallel.symm import SymmetricBuffer
    n = 4096
    p = torch.randn(n, device=dev).bfloat16()
    g = torch.randn(n, device=dev).bfloat16()
    mom = torch.zeros(n, device=dev)
    staged = torch.zeros(n, device=dev, dtype=torch.bfloat16)
    pad0, pad1 = SymmetricBuffer(256, dev), SymmetricBuffer(256, dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    plan = nat.MuonPlan([mom], [staged], [0], [1.0], 0)
    before = p.clone()
    ptrs2 = [p.data_ptr(), p.data_ptr()]
    plan.gather([g.data_ptr(), g.data_ptr()], ptrs2, [pad0.local_ptr, pad1.local_ptr], 0, 1, 20.0, status, 0.95, 0.5, True)
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert float(mom.abs().sum()) == 0.0 and float(staged.float().abs().sum()) == 0.0
    plan.scatter([p.data_ptr()], [pad0.local_ptr], 0, 1, 20.0, status, 0.1, 0.9)
    torch.cuda.synchronize()
    assert torch.equal(p, before)
    # the context is healthy and a clean world-1 round works afterwards
    status.zero_()
    plan.gather([g.data_ptr()], [p.data_ptr()], [pad0.local_ptr], 0, 2, 20.0, status, 0.95, 1.0, False)
    plan.scatter([p.data_ptr()], [pad0.local_ptr], 0, 2, 20.0, status, 0.1, 1.0)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    omm = (torch.tensor(1.0) - torch.tensor(0.95)).item()           # 1 - momentum as the kernel forms it, in fp32
    assert torch.equal(mom, g.float() * omm)
    assert torch.equal(staged, (g.float() * omm).bfloat16())
    lr32 = torch.tensor(0.1, dtype=torch.float32).double().item()
    want = (before.double() - lr32 * staged.double()).float().bfloat16()   # one fused multiply-add, then round to bf16
    assert torch.equal(p, want)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=90))   # a failed rank must not stall the others for long
    try:
        ps = _mk(dev)
        opt = DistMuon(ps, lr=2e-2, weight_decay=0.01, peer_timeout_ms=20000)
        assert opt._fused, "fused peer path not selected"
        for s in range(3):
            for p, g in zip(ps, _grads(s)):
                # one rank carries world * g (exact in bf16 for a power-of-two world), the others zero, alternating
                # per step: the mean over ranks is exactly g and owners need their peers' memory
                p.grad.copy_((g.float() * (world if rank == s % world else 0.0)).to(dev))
            opt.step()
        opt.check_status()
        torch.cuda.synchronize()
        dist.barrier()
        owned = [i for i, p in enumerate(ps) if opt.state[p]]
        torch.save({"params": [p.data.cpu() for p in ps], "owned": owned, "state_mb": opt.get_state_memory_mb()},
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.multigpu
@pytest.mark.parametrize("world", [2, 4])
def test_multi_gpu_fused_dist_muon(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    ranks = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    r0 = ranks[0]
    for other in ranks[1:]:
        for a, b in zip(r0["params"], other["params"]):
            assert torch.equal(a, b)                      # the peer stores left identical parameters everywhere
    assert sorted(i for r in ranks for i in r["owned"]) == list(range(len(SHAPES)))   # exactly one owner per tensor
    assert all(r["owned"] for r in ranks)
    dev = torch.device("cuda")
    ps = _mk(dev)
    ref = DistMuon(ps, lr=2e-2, weight_decay=0.01, fused=False)
    for s in range(3):
        for p, g in zip(ps, _grads(s)):
            p.grad = g.to(dev)
        ref.step()
    for a, p in zip(r0["params"], ps):
        _close(a, p.data.cpu(), 3 * 2e-2)
    total = sum(p.numel() for p in ps) * 4 / 2 ** 20
    assert sum(r["state_mb"] for r in ranks) == pytest.approx(total, rel=1e-6)   # momentum lives on the owner only


def test_zero_wrapper_with_muon_and_fused_true_builds_the_peer_memory_hybrid():
    """``ApexWZeRO(model, use_muon=True, fused=True)``: hidden matrices go to the gather -> Newton-Schulz -> scatter
    kernels, everything else to the fused ZeRO step (with clipping inside it); no collective path is involved."""
    from apexw_b200 import _native
    from apexw_b200.models.llama import build_llama
    from apexw_b200.parallel.dist_hybrid import DistHybridApexW
    from apexw_b200.parallel.zero import ApexWZeRO
    dev = torch.device("cuda")
    model = build_llama("tiny", device=dev, dtype=torch.bfloat16, seed=0)
    opt = ApexWZeRO(model, lr=1e-3, use_muon=True, fused=True, clip_grad_norm=1.0, muon_lr=1e-2)
    assert isinstance(opt, DistHybridApexW) and opt._fused and opt.world_size == 1
    before = [p.detach().clone() for p in model.parameters()]
    launches = _native.launch_count()
    tok = torch.randint(0, 512, (2, 65), device=dev)
    for _ in range(2):
        opt.zero_grad()
        model(tok[:, :-1], tok[:, 1:]).backward()
        opt.step()
    opt.check_status()
    assert _native.launch_count() - launches >= 2 * 4            # gather, scatter, reduce + exchange + update per step
    assert all(torch.isfinite(p).all() for p in model.parameters())
    assert sum(int(not torch.equal(a, b)) for a, b in zip(before, model.parameters())) == len(before)
    plain = ApexWZeRO(build_llama("tiny", device=dev, dtype=torch.bfloat16, seed=0), lr=1e-3, use_muon=True)
    assert isinstance(plain, ApexWZeRO) and not plain._fused       # without fused=True: the reference's behaviour
