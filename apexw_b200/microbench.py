"""Kernel-level benchmarks with their roofline fractions.

    python -m apexw_b200.microbench optimizer --precision compact --layers 8
    python -m apexw_b200.microbench ns --batch 4 --m 2048 --n 2048 --steps 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m apexw_b200.microbench zero --precision compact --layers 32 [--impl reference]
    python -m torch.distributed.run ... -m apexw_b200.microbench muon --model llama-1.1b [--impl reference]

``optimizer``  one ApexW step over ``--layers`` Llama-3-8B layer sets (q/o 4096x4096, k/v 1024x4096, gate/up
               14336x4096, down 4096x14336, two RMSNorm 4096; bf16 parameters, gradients N(0, 1e-3^2)).
``zero``       the same tensors under ApexWZeRO on every rank of the job: the fused reduce-scatter + update +
               all-gather kernel here, gradient all-reduce + ``ApexWZeRO.step`` for ``--impl reference``.
``ns``         the Newton-Schulz iteration on the tcgen05 kernels against the same iteration on library GEMMs.
``muon``       DistMuon over the hidden matrices of a Llama-style model (gather -> Newton-Schulz -> scatter).

Every command prints one JSON line (rank 0).  Times are CUDA-event medians after warm-up, max over ranks.
Peak figures for the fractions come from ``MEASURED_PEAKS.json`` at the repository root when present
(copy bandwidth, library bf16 GEMM rate), else from the fallbacks 6650 GB/s and 1590 TFLOP/s.
``--small`` shrinks the problem to a few GB for captures under a profiler.
"""

from __future__ import annotations

import argparse
import datetime
import json
import os
import sys
from typing import Callable, Dict, List

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LAYER_SET = [(4096, 4096), (4096, 4096), (1024, 4096), (1024, 4096), (14336, 4096), (14336, 4096), (4096, 14336),
             (4096,), (4096,)]
# HBM bytes per parameter of one fused step: p read+write, g read, moments read+write (+ scales)
TRAFFIC = {"compact": 11.0, "8bit": 7.51}
# optimizer modes beside the default AdamW-style step (keyword arguments of ApexW)
VARIANTS = {"default": {}, "lion": dict(lion=True, betas=(0.9, 0.99)), "cautious": dict(cautious=True),
            "amsgrad": dict(amsgrad=True), "ademamix": dict(betas=(0.9, 0.999, 0.9999)), "nesterov": dict(nesterov=True),
            "factored": dict(factored_v=True), "capturable": dict(capturable=True)}
NVLINK_GBS = 770.0      # measured peer copy, per direction per GPU


def peaks() -> Dict[str, float]:
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            data = json.load(fh)
        for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if k in data:
                out[k] = float(data[k])
        out["source"] = "measured"
    except Exception:
        pass
    return out


def median_ms(fn: Callable[[], None], warmup: int, iters: int, device) -> float:
    from .utils.timing import max_over_ranks, barrier_sync
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        barrier_sync(device)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize(device)
        times.append(max_over_ranks(a.elapsed_time(b), device))
    times.sort()
    return times[len(times) // 2]


def init_dist():
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=300))
    return rank, local, world


def layer_params(layers: int, device, seed: int = 0) -> List[torch.nn.Parameter]:
    g = torch.Generator(device=device).manual_seed(seed)
    return [torch.nn.Parameter(torch.randn(s, device=device, dtype=torch.bfloat16, generator=g) * 0.02)
            for _ in range(layers) for s in LAYER_SET]


def fill_grads(params, device, seed: int) -> None:
    g = torch.Generator(device=device).manual_seed(seed)
    for p in params:
        grad = torch.randn(p.shape, device=device, dtype=torch.bfloat16, generator=g) * 1e-3
        if p.grad is None:
            p.grad = grad
        else:
            p.grad.copy_(grad)


def cmd_optimizer(args) -> Dict:
    dev = torch.device("cuda")
    layers = 1 if args.small else args.layers
    ps = layer_params(layers, dev)
    fill_grads(ps, dev, 1)
    n = sum(p.numel() for p in ps)
    if args.impl == "reference":
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "apexw")):
            return {"bench": "optimizer", "impl": "reference", "unavailable": "baseline/_ref is missing"}
        sys.path.insert(0, ref_dir)
        os.environ.setdefault("APEXW_B200_RUNTIME_HOOKS", "0")
        import apexw as ref
        opt = ref.ApexW(ps, lr=1e-4, precision=args.precision, **VARIANTS[args.variant])
        if hasattr(opt, "_disable_auto_8bit_hooks"):
            opt._disable_auto_8bit_hooks()     # time optimizer.step(), not the in-backward hooks
    else:
        from . import ApexW
        opt = ApexW(ps, lr=1e-4, precision=args.precision, **VARIANTS[args.variant])
    ms = median_ms(opt.step, args.warmup, 1 if args.small else args.iters, dev)
    pk = peaks()
    if args.variant == "default" and args.precision in TRAFFIC:
        per_param = TRAFFIC[args.precision]
    else:
        # p read + write, g read, every state byte read + written (a mode that reads g twice still needs it only once)
        per_param = 4.0 + 2.0 + 2.0 * opt.get_state_memory_mb() * 2 ** 20 / n
    gbs = n * per_param / ms / 1e6
    fused = getattr(opt, "_native_launches", None)
    return {"bench": "optimizer", "impl": args.impl, "precision": args.precision, "variant": args.variant,
            "algorithmic_bytes_per_param": per_param, "kernel_launches_so_far": fused, "params": n, "ms": ms, "algorithmic_gbs": gbs,
            "fraction_of_hbm_copy": gbs / pk["hbm_gbs"], "peaks": pk["source"],
            "state_bytes_per_param": opt.get_state_memory_mb() * 2 ** 20 / n,
            "l2": "inputs far above the 126 MB L2 (every step streams all tensors)"}


def cmd_zero(args) -> Dict:
    import torch.distributed as dist
    rank, local, world = init_dist()
    dev = torch.device("cuda", local)
    layers = 1 if args.small else args.layers
    ps = layer_params(layers, dev)
    n = sum(p.numel() for p in ps)
    pk = peaks()
    if args.impl == "reference":
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "apexw")):
            return {"bench": "zero", "impl": "reference", "unavailable": "baseline/_ref is missing"}
        sys.path.insert(0, ref_dir)
        import apexw as ref
        opt = ref.ApexWZeRO(ps, lr=1e-4, precision=args.precision)
        fill_grads(ps, dev, 1 + rank)
        flat = None

        def step():
            if world > 1:      # what DDP does before the optimizer: average the gradients over ranks
                for p in ps:
                    dist.all_reduce(p.grad, op=dist.ReduceOp.AVG)
            opt.step()
        fused = False
    else:
        from .parallel.zero import ApexWZeRO
        opt = ApexWZeRO(ps, lr=1e-4, precision=args.precision, nvls=bool(getattr(args, "nvls", False)) or None)
        fill_grads(ps, dev, 1 + rank)
        step = opt.step
        fused = bool(opt._fused)
    nvls = bool(getattr(opt, "_stores", None)) and any(getattr(st, "multicast", False) for st in opt._stores)
    ms = median_ms(step, args.warmup, 1 if args.small else args.iters, dev)
    if hasattr(opt, "check_status"):
        opt.check_status()
    state_bpp = opt.get_state_memory_mb() * 2 ** 20 / n
    # NVLink bytes per GPU and direction.  Inbound: the responses to this rank's gradient loads from W-1 peers
    # (2 B x n/W each) plus the W-1 peers' stores of their parameter shards into this rank's buffer; outbound
    # is the mirror image.  Both are 2 * (W-1)/W * 2 B * n.
    link_bytes_per_direction = 2.0 * (2.0 * n * (world - 1) / world)
    if nvls:
        # through the switch: every rank's gradients leave once (2 B x n, the requester's own share included) and the
        # reduced shard comes back (2 B x n/W); parameters mirror that.  2 B * n * (1 + 1/W) each way.
        link_bytes_per_direction = 2.0 * n * (1.0 + 1.0 / world)
    # local HBM: the shard's fused update, plus peers reading this rank's gradients and writing its parameters
    hbm_bytes = n * TRAFFIC[args.precision] / world + 4.0 * n * (world - 1) / world
    floor_ms = max(link_bytes_per_direction / (NVLINK_GBS * 1e6), hbm_bytes / (pk["hbm_gbs"] * 1e6))
    link_bytes = link_bytes_per_direction
    return {"bench": "zero", "impl": args.impl, "precision": args.precision, "n_gpus": world, "params": n, "ms": ms,
            "fused": fused, "transport": "nvls multimem" if nvls else "peer loads/stores", "link_gbs_per_direction": link_bytes / ms / 1e6 if world > 1 else 0.0,
            "state_bytes_per_param_per_gpu": state_bpp, "roofline_ms": floor_ms,
            "fraction_of_roofline": floor_ms / ms, "peaks": pk["source"]}


def ns_flops(batch: int, m: int, n: int, steps: int) -> float:
    return float(steps) * batch * (2.0 * m * m * n + 2.0 * m * m * m + 2.0 * m * m * n)


def cmd_ns(args) -> Dict:
    from . import _native
    from .ops import newton_schulz as NS
    nat = _native.require()
    dev = torch.device("cuda")
    b, m, n = (4, 2048, 2048) if args.small else (args.batch, args.m, args.n)
    X = torch.randn(b, m, n, device=dev)
    X = (X / X.norm(dim=(-2, -1), keepdim=True)).bfloat16()
    coeffs = [NS.NS_COEFFS] * args.steps
    flat = [c for t in coeffs for c in t]
    iters = 1 if args.small else args.iters
    t_ours = median_ms(lambda: nat.ns_iterate(X, flat), args.warmup, iters, dev)
    out = {"bench": "ns", "batch": b, "m": m, "n": n, "steps": args.steps, "tcgen05_ms": t_ours}
    flops = ns_flops(b, m, n, args.steps)
    pk = peaks()
    out["tcgen05_dense_equivalent_tflops"] = flops / t_ours / 1e9
    out["fraction_of_library_gemm_peak"] = out["tcgen05_dense_equivalent_tflops"] / pk["bf16_tflops"]
    if not args.small:
        os.environ["APEXW_B200_NS_BACKEND"] = "torch"
        try:
            t_lib = median_ms(lambda: NS._iterate(X, coeffs), args.warmup, iters, dev)
        finally:
            del os.environ["APEXW_B200_NS_BACKEND"]
        out["library_ms"] = t_lib
        out["library_tflops"] = flops / t_lib / 1e9
        out["speedup_vs_library"] = t_lib / t_ours
    out["peaks"] = pk["source"]
    out["note"] = "dense-equivalent FLOPs: the symmetric products skip their lower-triangle tiles"
    return out


def cmd_muon(args) -> Dict:
    import torch.distributed as dist
    from .models.llama import get_config
    rank, local, world = init_dist()
    dev = torch.device("cuda", local)
    cfg = get_config(args.model)
    layers = 2 if args.small else cfg.n_layers
    hd = cfg.d_model // cfg.n_heads
    shapes = [(cfg.d_model + 2 * cfg.n_kv_heads * hd, cfg.d_model), (cfg.d_model, cfg.d_model),
              (2 * cfg.d_ff, cfg.d_model), (cfg.d_model, cfg.d_ff)]
    if args.split_fused:
        shapes = [(cfg.d_model, cfg.d_model), (cfg.n_kv_heads * hd, cfg.d_model), (cfg.n_kv_heads * hd, cfg.d_model),
                  (cfg.d_model, cfg.d_model), (cfg.d_ff, cfg.d_model), (cfg.d_ff, cfg.d_model), (cfg.d_model, cfg.d_ff)]
    g = torch.Generator(device=dev).manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(s, device=dev, dtype=torch.bfloat16, generator=g) * 0.02)
          for _ in range(layers) for s in shapes]
    n = sum(p.numel() for p in ps)
    if args.impl == "reference":
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "apexw")):
            return {"bench": "muon", "impl": "reference", "unavailable": "baseline/_ref is missing"}
        sys.path.insert(0, ref_dir)
        from apexw.fsdp import DistMuon as RefDistMuon
        opt = RefDistMuon(ps, lr=2e-2, ns_steps=args.steps)
        fill_grads(ps, dev, 1 + rank)

        def step():
            if world > 1:
                for p in ps:
                    dist.all_reduce(p.grad, op=dist.ReduceOp.AVG)
            opt.step()
        fused = False
    else:
        from .parallel.fsdp import DistMuon
        opt = DistMuon(ps, lr=2e-2, ns_steps=args.steps, balance={"shape": "shape", "cost": True}.get(args.owners, "auto"))
        fill_grads(ps, dev, 1 + rank)
        step = opt.step
        fused = bool(opt._fused)
    ms = median_ms(step, args.warmup, 1 if args.small else args.iters, dev)
    if hasattr(opt, "check_status"):
        opt.check_status()
    phases = getattr(opt, "last_phase_ms", None)       # set when APEXW_B200_MUON_TIMING=1
    flops = 0.0
    for s in shapes:
        lo, hi = min(s), max(s)
        flops += layers * ns_flops(1, lo, hi, args.steps)
    pk = peaks()

    # per GPU and direction: an owner pulls its matrices' gradients from W-1 peers and pushes the updated matrices
    # to W-1 peers; over a balanced ownership that is 2 * (W-1)/W * 2 B * n each way, as for ZeRO
    link_bytes = 2.0 * (2.0 * n * (world - 1) / world)
    floor_ms = max(flops / world / (pk["bf16_tflops"] * 1e9), link_bytes / (NVLINK_GBS * 1e6))
    return {"bench": "muon", "impl": args.impl, "model": args.model, "n_gpus": world, "params": n, "ns_steps": args.steps,
            "ms": ms, "fused": fused, "owners": args.owners, "ns_tflop_per_step": flops / 1e12, "roofline_ms": floor_ms,
            "fraction_of_roofline": floor_ms / ms, "peaks": pk["source"],
            "state_bytes_per_param_per_gpu": opt.get_state_memory_mb() * 2 ** 20 / n,
            "rank0_gather_ns_scatter_ms": [[round(x, 3) for x in t] for t in phases] if phases else None}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(prog="python -m apexw_b200.microbench")
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("optimizer", "zero", "ns", "muon"):
        sp = sub.add_parser(name)
        sp.add_argument("--warmup", type=int, default=3)
        sp.add_argument("--iters", type=int, default=10)
        sp.add_argument("--small", action="store_true", help="a few GB at most, one timed iteration (profiler captures)")
        if name in ("optimizer", "zero"):
            sp.add_argument("--precision", default="compact", choices=["compact", "8bit"] + (["ultra", "full"] if name == "optimizer" else []))
            if name == "optimizer":
                sp.add_argument("--variant", default="default", choices=sorted(VARIANTS))
            sp.add_argument("--layers", type=int, default=8 if name == "optimizer" else 32)
        if name == "zero":
            sp.add_argument("--nvls", action="store_true",
                            help="move gradients and parameters with multimem loads / stores through the NVSwitch")
        if name in ("optimizer", "zero", "muon"):
            sp.add_argument("--impl", default="apexw_b200", choices=["apexw_b200", "reference"])
        if name == "ns":
            sp.add_argument("--batch", type=int, default=4)
            sp.add_argument("--m", type=int, default=2048)
            sp.add_argument("--n", type=int, default=2048)
        if name in ("ns", "muon"):
            sp.add_argument("--steps", type=int, default=5)
        if name == "muon":
            sp.add_argument("--model", default="llama-1.1b")
            sp.add_argument("--split-fused", action="store_true", help="separate q/k/v and gate/up matrices")
            sp.add_argument("--owners", default="auto", choices=["auto", "cost", "shape"],
                            help="owner map: balanced by cost, or equal shapes kept on one rank (fewer, larger batches)")
    args = ap.parse_args(argv)
    out = {"optimizer": cmd_optimizer, "zero": cmd_zero, "ns": cmd_ns, "muon": cmd_muon}[args.cmd](args)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(out), flush=True)
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
