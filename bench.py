"""Headline benchmark: Llama-3-8B pretraining step (bf16, seq 4096, micro-batch 1, global batch 64,
uniform-random tokens, random-init weights) with DDP-style data parallelism + ApexWZeRO compact state.

    python bench.py --gpus 1 --steps K --warmup W                 # this framework
    python bench.py --impl reference --gpus 1 --steps K --warmup W  # unmodified reference from baseline/_ref
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Prints ONE JSON line on rank 0.  ``value`` is whole-job tokens/s from a device-timed loop whose
inputs already sit on the GPU; ``e2e`` is the same metric through ``TrainEngine.step`` with the
per-step host->device copy of the tokens from pinned memory and the device->host read of the loss
inside the timed region.  The global batch is fixed at 64 sequences, so scaling is "strong".

Both arms start from the same weights: the ``transformers`` Llama of the reference arm is built with seed 0 and
this framework's model loads those very tensors (``--init own`` skips that and draws its own N(0, 0.02) weights).
``loss_curve`` is one contiguous record: warm-up steps, the device-timed steps, the end-to-end steps, in training
order.  ``optimizer_step_ms`` is the median over the device-timed steps of CUDA events around ``optimizer.step()``.
``optimizer_only_swap`` (this framework's arm) repeats a few steps with the reference arm's ``transformers`` model
and only the optimizer replaced by this framework's ``ApexWZeRO``: it tells how much of the headline ratio is the
optimizer and how much the model-side kernels.
"""

from __future__ import annotations

import argparse
import datetime
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MODEL = "llama3-8b"
SEQ = 4096
GLOBAL_BATCH = 64
MICRO_BATCH = 1
LR, WD = 3e-4, 0.1


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="apexw_b200", choices=["apexw_b200", "reference"])
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--seq", type=int, default=SEQ)
    ap.add_argument("--global-batch", type=int, default=GLOBAL_BATCH)
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (debug only; marks the result)")
    ap.add_argument("--precision", default="compact", choices=["compact", "8bit"])
    ap.add_argument("--optimizer", default="zero", choices=["zero", "hybrid"],
                    help="zero: ApexWZeRO (headline).  hybrid: Muon on the hidden matrices + AdamW on the rest "
                         "(pair it with --model llama-1.1b --seq 2048 --global-batch 256)")
    ap.add_argument("--overlap", dest="overlap", action="store_true", default=None,
                    help="step buckets of parameters on a side stream during the last micro-batch's backward "
                         "(default: on with 2 or more GPUs, where the fused step carries NVLink traffic worth hiding)")
    ap.add_argument("--no-overlap", dest="overlap", action="store_false")
    ap.add_argument("--nvls", action="store_true",
                    help="fused ZeRO step through NVSwitch multimem loads / stores instead of plain peer loads / stores")
    ap.add_argument("--init", default="hf-weights", choices=["hf-weights", "own"],
                    help="hf-weights: start from the tensors of a seed-0 transformers Llama, as the reference arm does; "
                         "own: this model's own N(0, 0.02) draw")
    ap.add_argument("--swap-steps", type=int, default=3,
                    help="timed steps of the extra measurement 'transformers model + this framework's optimizer' (0 = skip)")
    return ap.parse_args()


def init_dist(n_gpus: int):
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=300))
    return rank, local, world


def make_tokens(rank: int, rows: int, seq: int, vocab: int, steps: int):
    """One fresh batch of uniform-random tokens per step (nothing repeats, so nothing can be memorised: the loss
    moves from its initial value towards ln(vocab) and no further), in pinned host memory."""
    g = torch.Generator().manual_seed(1234 + rank)
    return [torch.randint(0, vocab, (rows, seq + 1), generator=g).pin_memory() for _ in range(max(1, min(steps, 96)))]


def build_hf_llama(c, seq: int, dev):
    """The reference arm's model: ``transformers.LlamaForCausalLM`` of the named architecture, seed 0, bf16."""
    from transformers import LlamaConfig, LlamaForCausalLM
    hf_cfg = LlamaConfig(vocab_size=c.vocab_size, hidden_size=c.d_model, intermediate_size=c.d_ff,
                         num_hidden_layers=c.n_layers, num_attention_heads=c.n_heads, num_key_value_heads=c.n_kv_heads,
                         max_position_embeddings=seq, rope_theta=c.rope_theta, rms_norm_eps=c.norm_eps,
                         tie_word_embeddings=False, attn_implementation="sdpa", use_cache=False)
    torch.manual_seed(0)
    with torch.device(dev):
        model = LlamaForCausalLM(hf_cfg).to(torch.bfloat16)
    model.train()
    return model


def hf_step_fns(net, opt, accum: int, world: int, dev, dev_buf, loss_host, opt_events=None):
    """One optimizer step of a ``transformers`` causal LM (``labels`` = the inputs: the model shifts them itself)."""
    def step_device(tok):
        opt.zero_grad(set_to_none=True)
        total = torch.zeros((), dtype=torch.float32, device=dev)
        for i in range(accum):
            mb = tok[i * MICRO_BATCH:(i + 1) * MICRO_BATCH]
            ctx = net.no_sync() if (hasattr(net, "no_sync") and world > 1 and i < accum - 1) else _null()
            with ctx:
                out = net(input_ids=mb[:, :-1], labels=mb[:, :-1])
                (out.loss / accum).backward()
            total += out.loss.detach() / accum
        if opt_events is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            opt.step()
            e1.record()
            opt_events.append((e0, e1))
        else:
            opt.step()
        return total

    def step_e2e(tok_pinned):
        dev_buf.copy_(tok_pinned, non_blocking=True)
        loss = step_device(dev_buf)
        loss_host.copy_(loss, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return float(loss_host)

    return step_device, step_e2e


def median_event_ms(events, dev) -> float:
    """Median of (start, end) CUDA event pairs, maximum over ranks; call after a synchronisation."""
    import statistics
    from apexw_b200.utils.timing import max_over_ranks
    ms = [a.elapsed_time(b) for a, b in events]
    return max_over_ranks(statistics.median(ms) if ms else float("nan"), dev)


def run_optimizer_only_swap(args, rank, local, world, cfg, tokens):
    """The reference arm's model (``transformers`` Llama, stock autograd) with this framework's ``ApexWZeRO`` in place
    of DDP + the reference's ``ApexWZeRO``: gradients are reduced inside the fused step, so no DDP wrapper."""
    from apexw_b200.parallel.zero import ApexWZeRO
    from apexw_b200.utils.timing import time_steps
    dev = torch.device("cuda", local)
    accum = args.global_batch // (world * MICRO_BATCH)
    model = build_hf_llama(cfg, args.seq, dev)
    opt = ApexWZeRO(model.parameters(), lr=LR, weight_decay=WD, betas=(0.9, 0.95), precision=args.precision)
    dev_buf = torch.empty(accum * MICRO_BATCH, args.seq + 1, dtype=torch.int64, device=dev)
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()
    events = []
    step_device, step_e2e = hf_step_fns(model, opt, accum, world, dev, dev_buf, loss_host, events)
    curve = [step_e2e(tokens[i % len(tokens)]) for i in range(2)]
    del events[:]
    ms = time_steps(lambda i: curve.append(step_e2e(tokens[(2 + i) % len(tokens)])), args.swap_steps, dev)
    opt.check_status()
    return {"what": "transformers LlamaForCausalLM + apexw_b200.ApexWZeRO (fused peer-memory step, no DDP wrapper), "
                    "end to end, 2 warm-up steps",
            "value": args.global_batch * args.seq / (ms / args.swap_steps / 1e3), "unit": "tokens/s",
            "steps": args.swap_steps, "ms_per_step": ms / args.swap_steps,
            "optimizer_step_ms": median_event_ms(events, dev), "fused_zero_kernel": bool(opt._fused),
            "loss_curve": [round(x, 4) for x in curve]}


def run_ours(args, rank, local, world):
    from apexw_b200 import _native
    from apexw_b200.models.llama import build_llama, get_config
    from apexw_b200.parallel.zero import ApexWZeRO
    from apexw_b200.train import TrainEngine
    from apexw_b200.utils.timing import ClockSampler, time_steps, max_over_ranks
    _native.require()
    dev = torch.device("cuda", local)
    overrides = {"n_layers": args.layers} if args.layers else {}
    cfg = get_config(args.model, **overrides)
    model = build_llama(cfg, device=dev, dtype=torch.bfloat16, seed=0, init="hf")
    init = "own N(0, 0.02) draw, seed 0"
    if args.init == "hf-weights":
        try:
            from apexw_b200.models.llama import load_hf_llama_weights
            hf = build_hf_llama(cfg, args.seq, dev)
            load_hf_llama_weights(model, hf.state_dict())
            del hf
            init = "tensors of the seed-0 transformers Llama (same start as the reference arm)"
        except ImportError:
            pass
        import gc
        gc.collect()
        torch.cuda.empty_cache()
    accum = args.global_batch // (world * MICRO_BATCH)
    assert accum * world * MICRO_BATCH == args.global_batch, "global batch must divide evenly"
    if args.overlap is None:
        # bit-identical to the plain step (tests/test_gpu_zero.py); measured on 8 GPUs: 183.4 k against 173.5 k tokens/s
        args.overlap = world >= 2 and args.optimizer == "zero"
    if args.optimizer == "hybrid":
        from apexw_b200.parallel.dist_hybrid import DistHybridApexW
        opt = DistHybridApexW(model, lr=LR, weight_decay=WD, betas=(0.9, 0.95), precision=args.precision, ns_steps=5,
                              muon_momentum=0.95, fused_wgrad=True)
    else:
        opt = ApexWZeRO(model, lr=LR, weight_decay=WD, betas=(0.9, 0.95), precision=args.precision, fused_wgrad=True,
                        overlap_backward=args.overlap, nvls=True if args.nvls else None)
    engine = TrainEngine(model, opt, MICRO_BATCH, accum, args.seq, dev)
    tokens = make_tokens(rank, accum * MICRO_BATCH, args.seq, cfg.vocab_size, 2 * args.steps + args.warmup)
    dev_tokens = [t.to(dev) for t in tokens]

    curve = []
    n = 0
    for i in range(args.warmup):
        curve.append(engine.step(tokens[n % len(tokens)]))
        n += 1
    opt.check_status()
    launches0 = _native.launch_count()
    torch.cuda.reset_peak_memory_stats(dev)

    sampler = ClockSampler(local)
    sampler.start()
    dev_losses = []
    engine.optimizer_events = []
    ms = time_steps(lambda i: dev_losses.append(engine.step_device(dev_tokens[(n + i) % len(dev_tokens)])), args.steps, dev)
    clocks = sampler.stop()
    launches = _native.launch_count() - launches0
    opt.check_status()
    opt_ms = median_event_ms(engine.optimizer_events, dev)      # optimizer step alone, in place, median over the timed steps
    engine.optimizer_events = None
    curve += [float(x) for x in dev_losses]
    n += args.steps

    losses = []
    e2e_ms = time_steps(lambda i: losses.append(engine.step(tokens[(n + i) % len(tokens)])), args.steps, dev)
    opt.check_status()
    tokens_per_step = args.global_batch * args.seq
    n_params = sum(p.numel() for p in model.parameters())
    peak = torch.cuda.max_memory_allocated(dev)
    stores = list(opt._stores) if args.optimizer == "zero" else list(opt.adamw_opt._stores) + [opt.muon_opt._store]
    symm = sum(2 * s.numel * torch.empty((), dtype=s.dtype).element_size() for s in stores if s is not None)
    fused_flag = bool(opt._fused) if args.optimizer == "zero" else bool(opt.adamw_opt._fused and opt.muon_opt._fused)
    transport = "nvls multimem" if any(getattr(s, "multicast", False) for s in stores if s is not None) else "peer loads/stores"
    res = dict(transport=transport, overlap=bool(args.overlap), ms=ms, e2e_ms=e2e_ms, clocks=clocks, launches=launches, opt_ms=opt_ms, loss=losses[-1], curve=curve + losses,
               tokens_per_step=tokens_per_step, n_params=n_params, h2d=engine.h2d_bytes_per_step,
               d2h=engine.d2h_bytes_per_step, peak_bytes=peak + symm,
               state_bpp=opt.get_state_memory_mb() * 2 ** 20 * world / n_params, init=init,
               fused=fused_flag, accum=accum, model=args.model if not args.layers else f"{args.model}[{args.layers} layers]")
    if args.swap_steps > 0 and args.optimizer == "zero":
        import gc
        del engine, opt, model, stores, dev_tokens, dev_losses
        gc.collect()
        torch.cuda.empty_cache()
        try:
            res["swap"] = run_optimizer_only_swap(args, rank, local, world, cfg, tokens)
        except ImportError as exc:
            res["swap"] = {"unavailable": f"transformers not importable: {exc}"[:160]}
    return res


def run_reference(args, rank, local, world):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "apexw")):
        return {"unavailable": "baseline/_ref is missing: the reference was not installed"}
    sys.path.insert(0, ref_dir)
    try:
        import apexw as ref
        import transformers  # noqa: F401
    except Exception as exc:
        return {"unavailable": f"reference or transformers not importable: {type(exc).__name__}: {exc}"[:200]}
    from apexw_b200.utils.timing import ClockSampler, time_steps
    from apexw_b200.models.llama import get_config
    dev = torch.device("cuda", local)
    c = get_config(args.model, **({"n_layers": args.layers} if args.layers else {}))
    model = build_hf_llama(c, args.seq, dev)
    accum = args.global_batch // (world * MICRO_BATCH)
    net = model
    if world > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP
        net = DDP(model, device_ids=[local], gradient_as_bucket_view=True)
    if args.optimizer == "hybrid":      # the reference's hybrid: every rank orthogonalises every matrix (DDP-averaged gradients)
        opt = ref.ApexW(model, lr=LR, weight_decay=WD, betas=(0.9, 0.95), precision=args.precision, use_muon=True)
    else:
        opt = ref.ApexWZeRO(model.parameters(), lr=LR, weight_decay=WD, betas=(0.9, 0.95), precision=args.precision)
    tokens = make_tokens(rank, accum * MICRO_BATCH, args.seq, c.vocab_size, 2 * args.steps + args.warmup)
    dev_buf = torch.empty(accum * MICRO_BATCH, args.seq + 1, dtype=torch.int64, device=dev)
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()
    events = []
    step_device, step_e2e = hf_step_fns(net, opt, accum, world, dev, dev_buf, loss_host, events)

    dev_tokens = [t.to(dev) for t in tokens]
    curve = []
    n = 0
    for i in range(args.warmup):
        curve.append(step_e2e(tokens[n % len(tokens)]))
        n += 1
    torch.cuda.reset_peak_memory_stats(dev)
    del events[:]
    sampler = ClockSampler(local)
    sampler.start()
    dev_losses = []
    ms = time_steps(lambda i: dev_losses.append(step_device(dev_tokens[(n + i) % len(dev_tokens)])), args.steps, dev)
    clocks = sampler.stop()
    opt_ms = median_event_ms(events, dev)
    curve += [float(x) for x in dev_losses]
    n += args.steps
    losses = []
    e2e_ms = time_steps(lambda i: losses.append(step_e2e(tokens[(n + i) % len(tokens)])), args.steps, dev)
    n_params = sum(p.numel() for p in model.parameters())
    return dict(ms=ms, e2e_ms=e2e_ms, clocks=clocks, launches=0, opt_ms=opt_ms, loss=losses[-1], curve=curve + losses,
                tokens_per_step=args.global_batch * args.seq, n_params=n_params,
                h2d=accum * MICRO_BATCH * (args.seq + 1) * 8, d2h=4, peak_bytes=torch.cuda.max_memory_allocated(dev),
                state_bpp=opt.get_state_memory_mb() * 2 ** 20 * (world if args.optimizer == "zero" else 1) / n_params,
                fused=False, accum=accum, init="tensors of the seed-0 transformers Llama",
                model=args.model if not args.layers else f"{args.model}[{args.layers} layers]")


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def main():
    args = parse()
    rank, local, world = init_dist(args.gpus)
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}; using {world}", file=sys.stderr)
    try:
        res = run_reference(args, rank, local, world) if args.impl == "reference" else run_ours(args, rank, local, world)
    except torch.cuda.OutOfMemoryError as exc:
        res = {"unavailable": f"out of memory: {str(exc)[:120]}"} if args.impl == "reference" else None
        if res is None:
            raise
    if rank == 0:
        if "unavailable" in res:
            print(json.dumps({"impl": "reference", "unavailable": res["unavailable"]}))
        else:
            tps = res["tokens_per_step"] / (res["ms"] / args.steps / 1e3)
            e2e = res["tokens_per_step"] / (res["e2e_ms"] / args.steps / 1e3)
            line = {
                "metric": "llama3_8b_train_tokens_per_s" if args.model == MODEL else f"{args.model}_train_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms"] / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic uniform-random tokens (a fresh batch every step), random-init weights", "impl": args.impl,
                "config": {"model": res["model"], "global_batch": args.global_batch, "seq_len": args.seq,
                           "micro_batch": MICRO_BATCH, "grad_accum_per_rank": res["accum"],
                           "parallelism": f"dp{world}+zero1" if args.optimizer == "zero" else f"dp{world}+dist-muon+zero1",
                           "optimizer_state": args.precision,
                           "l2": "no flush needed: each step streams all parameters and activations, GBs against a 126 MB L2",
                           "fused_zero_kernel": res["fused"], "initial_weights": res["init"],
                           **({"zero_transport": res["transport"], "overlap_backward": res["overlap"]} if "transport" in res else {})},
                "clocks": {"sm_mhz": res["clocks"]["sm_mhz"], "sm_max_mhz": res["clocks"]["sm_max_mhz"],
                           "reasons": res["clocks"]["reasons"]},
                "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": res["h2d"], "d2h_bytes_per_step": res["d2h"],
                        "ms_per_step": res["e2e_ms"] / args.steps},
                "gpu_launches": res["launches"],
                "optimizer_step_ms": res["opt_ms"], "peak_hbm_bytes_per_param": res["peak_bytes"] / res["n_params"],
                "optimizer_state_bytes_per_param": res["state_bpp"], "loss": res["loss"],
                "loss_curve": [round(x, 4) for x in res["curve"]],
            }
            if "swap" in res:
                line["optimizer_only_swap"] = res["swap"]
            print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
