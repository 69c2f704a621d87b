"""Fused ZeRO kernel on real GPUs: single-GPU equivalence with the plain optimizer, the bounded-wait
status path, and (with >= 2 GPUs) child processes whose fused step must match a single-GPU run."""
import datetime
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp
import torch.nn as nn

from apexw_b200 import ApexW, _native
from apexw_b200.parallel.zero import ApexWZeRO

pytestmark = pytest.mark.gpu

SHAPES = [(512, 256)] * 8 + [(256,), (1000, 40), (70,), (4096, 64), (3, 5)]


def _mk(dev, dtype=torch.bfloat16, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [nn.Parameter((torch.randn(s, generator=g) * 0.05).to(dtype).to(dev)) for s in SHAPES]


def _grads(step, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(100 + step)
    return [(torch.randn(s, generator=g) * 1e-3).to(dtype) for s in SHAPES]


@pytest.mark.parametrize("prec", ["compact", "8bit"])
def test_world1_fused_zero_equals_plain_optimizer(prec):
    """World size 1: the peer kernel reads/writes only local memory and must reproduce ApexW bit for bit
    (same formats, same rounding bits, same arithmetic)."""
    dev = torch.device("cuda")
    pz, pp = _mk(dev), _mk(dev)
    oz = ApexWZeRO(pz, lr=1e-2, precision=prec, betas=(0.9, 0.99), seed=3)
    op = ApexW(pp, lr=1e-2, precision=prec, betas=(0.9, 0.99), seed=3)
    assert oz._fused
    for s in range(3):
        for p, q, g in zip(pz, pp, _grads(s)):
            p.grad.copy_(g.to(dev))
            q.grad = g.to(dev)
        oz.step()
        op.step()
    oz.check_status()
    for a, b in zip(pz, pp):
        assert torch.equal(a.data, b.data), a.shape
    n = sum(p.numel() for p in pz)
    assert oz.get_state_memory_mb() == pytest.approx(op.get_state_memory_mb(), rel=1e-6)


def test_entry_wait_runs_out_and_leaves_state_untouched():
    """A peer flag that nothing sets: the kernel gives up after its budget, reports status 1, and
    touches neither parameters nor moments.  (World of 2 faked on one GPU: both 'peers' are local.)"""
    nat = _native.require()
    dev = torch.device("cuda")
    from apexw_b200.parallel.symm import SymmetricBuffer
    n = 4096
    p = torch.randn(n, device=dev).bfloat16()
    g = torch.randn(n, device=dev).bfloat16()
    m = torch.zeros(n, device=dev, dtype=torch.bfloat16)
    v = torch.zeros(n, device=dev, dtype=torch.bfloat16)
    pad0, pad1 = SymmetricBuffer(256, dev), SymmetricBuffer(256, dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    plan = nat.StatePlan(0, [p], [m], [v], [], [], [0], [0], [0], [0], 0)
    before = p.clone()
    plan.step_zero([g.data_ptr(), g.data_ptr()], [p.data_ptr(), p.data_ptr()], [pad0.local_ptr, pad1.local_ptr], 0,
                   1, 20.0, status, 1, 1, 0.9, 0.99, 1e-2, 1e-8, 1e-8, 1e-8, 1e-8, 1.0, 0.5, 1.18, 0.68, 12345, 1)
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert torch.equal(p, before) and float(m.abs().sum()) == 0.0
    # the context is still healthy: an ordinary launch works afterwards
    status.zero_()
    plan.step_zero([g.data_ptr()], [p.data_ptr()], [pad0.local_ptr], 0, 2, 20.0, status, 1, 1,
                   0.9, 0.99, 1e-2, 1e-8, 1e-8, 1e-8, 1e-8, 1.0, 1.0, 1.18, 0.68, 12345, 1)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and not torch.equal(p, before)


def test_a_timed_out_step_raises_at_the_next_step_and_takes_its_step_count_back():
    """A user loop never calls ``check_status()``.  Here a second 'peer' whose flag nothing sets makes the entry wait
    of one step run out (20 ms budget; both 'peers' are buffers of this GPU).  The step itself returns normally; the
    NEXT ``step()`` raises, the parameters are untouched, and the step counters are back where they were."""
    from apexw_b200.parallel.status import PeerStepError
    from apexw_b200.parallel.symm import SymmetricBuffer
    dev = torch.device("cuda")
    ps = _mk(dev)
    opt = ApexWZeRO(ps, lr=1e-2, precision="compact", seed=3, peer_timeout_ms=20.0)
    for p, g in zip(ps, _grads(0)):
        p.grad.copy_(g.to(dev))
    opt.step()                                            # a healthy first step
    opt.check_status()
    steps_before = [float(st["step"]) for st in opt._local_opt.state.values()]
    before = [p.detach().clone() for p in ps]
    silent = SymmetricBuffer(256, dev)                    # the pad of a peer that never arrives
    real = opt._peer_pointers

    def with_a_silent_peer(store):
        g, p, s = real(store)
        return [g[0], g[0]], [p[0], p[0]], [s[0], silent.local_ptr]

    opt._peer_pointers = with_a_silent_peer
    opt.step()                                            # launches, times out on the device, returns
    torch.cuda.synchronize()
    opt._peer_pointers = real
    with pytest.raises(PeerStepError) as err:
        opt.step()
    assert "nothing was updated" in str(err.value)
    assert [float(st["step"]) for st in opt._local_opt.state.values()] == steps_before
    for p, b in zip(ps, before):
        assert torch.equal(p.data, b)
    opt.step()                                            # the words were cleared: the next step is healthy again
    opt.check_status()
    assert not torch.equal(ps[0].data, before[0])


def test_parameters_outlive_the_optimizer_that_flattened_them():
    """The flat buffers are reference-counted native allocations held by the storage of every tensor made over
    them.  Dropping the optimizer must neither free memory that the model's parameters still point into nor
    change their values; the allocations go when the parameters go."""
    import gc
    from apexw_b200.parallel.symm import live_allocations
    dev = torch.device("cuda")
    gc.collect()
    base = live_allocations()
    ps = _mk(dev)
    want = [p.detach().clone() for p in ps]
    opt = ApexWZeRO(ps, lr=1e-2, precision="compact", seed=3)
    assert opt._fused
    held = live_allocations()
    assert held >= base + 3                       # parameters, gradients, signal pad
    del opt
    gc.collect()
    torch.cuda.synchronize()
    assert live_allocations() >= base + 2         # parameters and gradients are still referenced by the model
    for p, w in zip(ps, want):
        assert torch.equal(p.data, w)
        p.data.add_(1.0)                          # still writable memory
        assert torch.equal(p.data, (w.float() + 1.0).to(w.dtype))
    opt2 = ApexWZeRO(ps, lr=1e-2, precision="compact", seed=3)      # a second optimizer re-homes them again
    for p, g in zip(ps, _grads(0)):
        p.grad.copy_(g.to(dev))
    opt2.step()
    opt2.check_status()
    del opt2, ps, p
    gc.collect()
    torch.cuda.synchronize()
    assert live_allocations() == base


@pytest.mark.parametrize("prec", ["compact", "8bit"])
def test_clipping_runs_inside_the_fused_step(prec):
    """``clip_grad_norm`` keeps the peer-memory path: a reduce-only kernel scales the shard's gradient in place and sums
    its squares, the partial sums are exchanged through the signal pad, and the update kernel applies the coefficient.
    World of one against the plain optimizer (which clips the bf16 gradients with torch ops first): same norm, same
    coefficient up to rounding, so the parameters agree to a bf16 step."""
    dev = torch.device("cuda")
    pz, pp = _mk(dev), _mk(dev)
    oz = ApexWZeRO(pz, lr=1e-2, precision=prec, betas=(0.9, 0.99), seed=3, clip_grad_norm=0.05, stochastic_rounding=False)
    op = ApexW(pp, lr=1e-2, precision=prec, betas=(0.9, 0.99), seed=3, clip_grad_norm=0.05, stochastic_rounding=False)
    assert oz._fused
    launches = _native.launch_count()
    for s in range(3):
        for p, q, g in zip(pz, pp, _grads(s)):
            p.grad.copy_((g * 50.0).to(dev))          # norm well above the limit: the coefficient matters
            q.grad = (g * 50.0).to(dev)
        oz.step()
        op.step()
    oz.check_status()
    assert _native.launch_count() - launches >= 3 * 3          # reduce + exchange + update per step at least
    total = float(oz._clip_total[0].sqrt())
    assert total > 0.05 * 5                                     # the exchanged norm is the (large) norm of the whole gradient
    # the torch path rounds the clipped gradient (and the coefficient) to bf16, the kernel scales in fp32: the moments
    # agree to a bf16 step, and an update that differs by that much flips the rounding of a parameter now and then
    for a, b in zip(pz, pp):
        diff = (a.data.float() - b.data.float()).abs()
        if prec == "compact":
            assert (diff <= b.data.float().abs() * 2.0 ** -7 * 3.5 + 4e-4).all(), (a.shape, diff.max())
            assert (diff > 0).float().mean() < 0.4
        else:       # 4-bit / log-8-bit codes turn a last-place difference of a moment into a code step now and then
            assert diff.max() <= 3 * 1e-2 and diff.mean() <= 1e-3, (a.shape, diff.max(), diff.mean())
    if prec == "compact":
        for la, b in zip(oz._local_params, pp):
            ma, mb = oz._local_opt.state[la]["exp_avg"].float(), op.state[b]["exp_avg"].float()
            assert ((ma - mb).abs().max() <= 0.02 * mb.abs().max())


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, prec, out_dir, nvls=False, clip=None):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=90))   # a failed rank must not stall the others for long
    try:
        ps = _mk(dev)
        opt = ApexWZeRO(ps, lr=1e-2, precision=prec, betas=(0.9, 0.99), seed=3, stochastic_rounding=False,
                        peer_timeout_ms=20000, nvls=nvls, clip_grad_norm=clip)
        assert opt._fused, "fused peer path not selected"
        multicast = all(st.multicast for st in opt._stores)
        boost = 50.0 if clip is not None else 1.0
        for s in range(3):
            for p, g in zip(ps, _grads(s)):
                # one rank carries world*g, the others zero, alternating per step: the mean over ranks is exactly g
                # (power-of-two scaling is exact in bf16), and every shard's update depends on a peer's memory
                carrier = s % world
                p.grad.copy_((g.float() * boost * (world if rank == carrier else 0.0)).to(dev))
            opt.step()
        opt.check_status()
        torch.cuda.synchronize()
        dist.barrier()
        torch.save({"params": [p.data.cpu() for p in ps], "state_mb": opt.get_state_memory_mb(), "multicast": multicast},
                   os.path.join(out_dir, f"rank{rank}.pt"))
        del opt, ps, p            # multicast-bound buffers go before the process group does, on every rank alike
        import gc
        gc.collect()
        torch.cuda.synchronize()
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.multigpu
@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("prec", ["compact", "8bit"])
@pytest.mark.parametrize("transport", ["peer", "nvls"])
def test_multi_gpu_fused_step_matches_single_gpu(tmp_path, prec, world, transport):
    """``transport="nvls"``: gradients come back from the switch already summed (``multimem.ld_reduce``) and parameters
    go out through ``multimem.st``.  The switch rounds the sum to bf16; in this test one rank carries the whole
    gradient and the others zeros, so that sum is exact and the result must still equal the single-GPU run bit for bit."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    mp.spawn(_worker, args=(world, _free_port(), prec, str(tmp_path), transport == "nvls"), nprocs=world, join=True)
    ranks = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    r0 = ranks[0]
    if transport == "nvls" and not r0["multicast"]:
        pytest.skip("no NVSwitch multicast address on this machine (the optimizer fell back to peer loads)")
    assert r0["multicast"] == (transport == "nvls")
    for other in ranks[1:]:
        for a, b in zip(r0["params"], other["params"]):
            assert torch.equal(a, b)                  # the in-kernel all-gather left identical parameters
    # single-GPU reference: same mean gradient, sharded the same way (world-size-2 slices on one device)
    dev = torch.device("cuda")
    import warnings
    merged = None
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        runs = []
        for r in range(world):
            ps = _mk(dev)
            o = ApexWZeRO(ps, lr=1e-2, precision=prec, betas=(0.9, 0.99), seed=3, stochastic_rounding=False,
                          world_size=world, rank=r, fused=False, reduce_gradients=False)
            for s in range(3):
                for p, g in zip(ps, _grads(s)):
                    p.grad.copy_(g.to(dev))
                o.step()
            runs.append((ps, o))
    for i in range(len(SHAPES)):
        full = torch.empty_like(runs[0][0][i].data)
        for r, (ps, o) in enumerate(runs):
            e = o._sharded_param_map[i]
            if e["type"] == "slice":
                full[e["start"]:e["end"]] = ps[i].data[e["start"]:e["end"]]
            elif e["owner_rank"] == r:
                full.copy_(ps[i].data)
        # same mean gradient, same shard layout, same arithmetic: the peer-memory step is bit-identical
        assert torch.equal(full.cpu(), r0["params"][i]), (SHAPES[i], (full.cpu().float() - r0["params"][i].float()).abs().max())
    assert sum(r["state_mb"] for r in ranks) == pytest.approx(sum(o.get_state_memory_mb() for _, o in runs), rel=1e-6)


@pytest.mark.multigpu
@pytest.mark.parametrize("world", [2, 8])
def test_multi_gpu_clipped_fused_step_is_close_to_the_unsharded_clip(tmp_path, world):
    """Global-norm clipping inside the fused step on real ranks: every rank ends with the same parameters, and they
    match a single-process run that clips the whole gradient with torch ops (bf16 rounding of the clipped gradient
    differs between the two, so to a bf16 step, not bit for bit)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    mp.spawn(_worker, args=(world, _free_port(), "compact", str(tmp_path), False, 0.05), nprocs=world, join=True)
    ranks = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    for other in ranks[1:]:
        for a, b in zip(ranks[0]["params"], other["params"]):
            assert torch.equal(a, b)
    dev = torch.device("cuda")
    ps = _mk(dev)
    ref = ApexW(ps, lr=1e-2, precision="compact", betas=(0.9, 0.99), seed=3, stochastic_rounding=False, clip_grad_norm=0.05)
    for s in range(3):
        for p, g in zip(ps, _grads(s)):
            p.grad = (g.float() * 50.0).to(torch.bfloat16).to(dev)
        ref.step()
    for a, b in zip(ranks[0]["params"], ps):
        diff = (a.float() - b.data.cpu().float()).abs()
        assert (diff <= b.data.cpu().float().abs() * 2.0 ** -7 * 3.5 + 4e-4).all(), (a.shape, diff.max())


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("prec", ["compact", "8bit"])
def test_rank0_of_an_emulated_world_on_one_gpu(prec, world, monkeypatch):
    """Rank 0 of a world of 2/4/8 whose peers' buffers all live on this GPU and whose peers' flags the host has
    set beforehand: one launch, nothing waits on another launch.  Exercises the world-size specialisations
    (unrolled peer loops) numerically: the result must be bit-identical to the plain
    optimizer stepping on the rank-ordered fp32 sum of the gradients with scale 1/world, and every peer's
    parameter buffer must receive the same bytes."""
    from apexw_b200.parallel.symm import SymmetricBuffer
    dev = torch.device("cuda")
    pz, pp = _mk(dev), _mk(dev)
    kw = dict(lr=1e-2, precision=prec, betas=(0.9, 0.99), seed=3)
    oz = ApexWZeRO(pz, **kw)
    op = ApexW(pp, **kw)
    assert oz._fused and len(oz._stores) == 1
    store = oz._stores[0]
    fake_g = [store.grad] + [torch.zeros_like(store.grad) for _ in range(world - 1)]
    fake_p = [store.param] + [torch.zeros_like(store.param) for _ in range(world - 1)]
    pads = [SymmetricBuffer(256, dev) for _ in range(world)]
    flags = pads[0].tensor(torch.int32, 64)
    flags[0:world] = 1 << 20            # entry flags of every peer: "arrived" for any epoch this test reaches
    flags[8:8 + world] = 1 << 20        # exit flags likewise
    monkeypatch.setattr(oz, "_peer_pointers", lambda st: ([g.data_ptr() for g in fake_g], [p.data_ptr() for p in fake_p],
                                                         [pad.local_ptr for pad in pads]))
    for s in range(2):
        gen = torch.Generator().manual_seed(500 + s)
        for i, (p, q) in enumerate(zip(pz, pp)):
            off, n = store.offsets[id(p)], p.numel()
            total = None
            for r in range(world):
                g = (torch.randn(p.shape, generator=gen) * 1e-3).bfloat16().to(dev)
                fake_g[r][off:off + n].copy_(g.reshape(-1))
                total = g.float() if total is None else total + g.float()      # rank order, fp32, as the kernel sums
            q.grad_dtype = None          # the reference run takes the fp32 sum as its gradient
            q.grad = total
        op.grad_scale = torch.tensor(float(world), device=dev)
        oz.step()
        op.step()
    oz.check_status()
    torch.cuda.synchronize()
    for p, q in zip(pz, pp):
        assert torch.equal(p.data, q.data), tuple(p.shape)
    for r in range(1, world):
        assert torch.equal(fake_p[r], store.param)


def test_debug_mode_guard_bands_survive_the_peer_kernel(monkeypatch):
    """APEXW_B200_DEBUG=1: symmetric buffers get guard bands with a pattern; after fused steps (whose stores go
    through the same peer-pointer arithmetic as on many GPUs) the bands must be untouched, and plan building runs
    the host-side disjoint-write-set check."""
    monkeypatch.setenv("APEXW_B200_DEBUG", "1")
    dev = torch.device("cuda")
    for prec in ("compact", "8bit"):
        ps = _mk(dev)
        opt = ApexWZeRO(ps, lr=1e-2, precision=prec, seed=3)
        assert opt._fused
        for s in range(2):
            for p, g in zip(ps, _grads(s)):
                p.grad.copy_(g.to(dev))
            opt.step()
        opt.check_status()
        torch.cuda.synchronize()
        for store in opt._stores:
            assert store.symm_param._guard > 0
            assert store.symm_param.check_canaries() and store.symm_grad.check_canaries()
        assert opt._signal.check_canaries()
    plain = ApexW(_mk(dev), lr=1e-2, precision="compact")
    for p, g in zip(plain.param_groups[0]["params"], _grads(0)):
        p.grad = g.to(dev)
    plain.step()                       # builds its plans under the disjointness check
    assert plain._native_launches > 0


@pytest.mark.parametrize("prec", ["compact", "8bit"])
def test_overlap_with_backward_gives_the_same_parameters(prec):
    """Buckets stepped on a side stream during the last micro-batch's backward (world of one) against the plain
    step after backward: same kernels on the same data, so the parameters must be bit-identical."""
    from apexw_b200.models.llama import build_llama
    from apexw_b200.train import TrainEngine
    dev = torch.device("cuda")
    results = []
    for overlap in (False, True):
        model = build_llama("tiny", device=dev, dtype=torch.bfloat16, seed=0)
        opt = ApexWZeRO(model, lr=1e-2, precision=prec, seed=5, fused_wgrad=True, overlap_backward=overlap,
                        overlap_buckets=3, overlap_ctas=8)
        assert opt._fused and opt.overlap_backward == overlap
        engine = TrainEngine(model, opt, 1, 2, 64, dev)
        g = torch.Generator().manual_seed(9)
        launched = []
        for s in range(3):
            tok = torch.randint(0, 512, (2, 65), generator=g).to(dev)
            engine.step_device(tok)
            launched.append(list(opt._launched))
        opt.check_status()
        torch.cuda.synchronize()
        results.append(([p.detach().clone() for p in model.parameters()], launched))
    (plain, _), (over, launched) = results
    assert all(len(l) == 3 for l in launched), launched             # every bucket went out during backward
    assert launched[0][0] == 2                                      # the last layers' bucket first
    for a, b in zip(plain, over):
        assert torch.equal(a, b)


def _worker_overlap(rank, world, port, out_dir):
    import torch.distributed as dist
    from apexw_b200.models.llama import build_llama
    from apexw_b200.train import TrainEngine
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=90))
    try:
        outs = []
        for overlap in (False, True):
            model = build_llama("tiny", device=dev, dtype=torch.bfloat16, seed=0)
            opt = ApexWZeRO(model, lr=1e-2, precision="compact", seed=5, fused_wgrad=True, overlap_backward=overlap,
                            overlap_buckets=3, overlap_ctas=8, peer_timeout_ms=20000)
            assert opt._fused and opt.overlap_backward == overlap
            engine = TrainEngine(model, opt, 1, 2, 64, dev)
            g = torch.Generator().manual_seed(20 + rank)          # every rank trains on its own tokens
            for s in range(3):
                engine.step_device(torch.randint(0, 512, (2, 65), generator=g).to(dev))
            opt.check_status()
            torch.cuda.synchronize()
            dist.barrier()
            outs.append([p.detach().cpu() for p in model.parameters()])
        torch.save({"plain": outs[0], "overlap": outs[1]}, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.multigpu
def test_two_gpu_overlap_with_backward_matches_the_plain_step(tmp_path):
    world = 2
    mp.spawn(_worker_overlap, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r0, r1 = torch.load(tmp_path / "rank0.pt"), torch.load(tmp_path / "rank1.pt")
    for a, b, c, d in zip(r0["plain"], r0["overlap"], r1["plain"], r1["overlap"]):
        assert torch.equal(a, b) and torch.equal(c, d)          # overlapped buckets = plain step, bit for bit
        assert torch.equal(a, c)                                # and the ranks hold the same parameters
