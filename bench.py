#!/usr/bin/env python
"""Headline benchmark: full-parameter bf16 SFT throughput (tokens/s) of the
SenseNova-U1-8B-MoT architecture on packed 16384-token multimodal sequences,
random-init weights, synthetic data, one process per GPU.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Two timed regions, both K steps after W warm-up steps, barrier + synchronize on both
sides, CUDA events on the launching stream, max over ranks:
  * value: batches resident on the device (kernel / collective time of the step);
  * e2e:   the public ``Trainer.train_step`` call: pinned host batch -> device copy,
           forward, backward, gradient reduce-scatter, AdamW, parameter all-gather,
           loss read back to the host, every step.
Every step includes the optimizer; nothing is cached between steps.  Each step streams
the whole weight set (35 GB at 8B) through the SMs, far more than the 126 MB L2, so no
explicit L2 flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="8b-mot")
    ap.add_argument("--seq-len", type=int, default=16384)
    ap.add_argument("--layers", type=int, default=None, help="debug only: override the layer count")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-fixed-policy", action="store_true",
                    help="skip the extra timed steps under the fixed 'every layer recomputed' activation policy")
    ap.add_argument("--breakdown", action="store_true", help="also report the optimizer-step share (CUDA events)")
    ap.add_argument("--kernel-table", default=None, metavar="PATH",
                    help="after all timed regions, run one more step on rank 0 under the torch profiler and write the "
                         "per-kernel device-time table there (shares only: never a bench value)")
    ap.add_argument("--recompute", default="auto", choices=["auto", "full", "attention", "none"],
                    help="activation policy of the training engine (auto: by free memory)")
    ap.add_argument("--task", default="sft", choices=["sft", "t2i"],
                    help="sft: the headline training throughput; t2i: seconds per 2048x2048 image (50 Euler steps, CFG 4)")
    ap.add_argument("--image", type=int, default=2048)
    ap.add_argument("--denoise-steps", type=int, default=50)
    ap.add_argument("--parallel", default="auto",
                    help="auto: wp from 2 GPUs up (the configuration the baseline names: ZeRO-1 + ISP weight parallel of "
                         "degree N), single GPU otherwise; tp<T>pp<P>: tensor x pipeline parallel (1F1B, 8 micro-batches); "
                         "dp: data parallel + ZeRO-1 (weights replicated); wp: weight parallel = the reference's ISP mode "
                         "with wp = N, tp = 1 (weights, gradients and optimizer state sharded 1/N, layers gathered by "
                         "peer loads one layer ahead, gradients reduce-scattered from staging slots); cp<N>: context parallel, "
                         "one packed sequence of --seq-len tokens over the N ranks")
    ap.add_argument("--micro", type=int, default=8, help="micro-batches per step of the tp x pp configuration")
    ap.add_argument("--comm", default="peer", choices=["peer", "nccl"],
                    help="peer: ZeRO collectives by this package's NVLink peer-memory kernels; nccl: NCCL baseline")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while running."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 7:
                    continue
                try:
                    sm.append(float(f[0])); mx = max(mx, float(f[1]))
                except ValueError:
                    continue
                for n, v in zip(names, f[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except OSError:
            pass
        sm.sort()
        # the busiest half of the samples is "under load"
        load = sm[len(sm) // 2:] if sm else []
        med = load[len(load) // 2] if load else None
        return {"sm_mhz": med, "sm_max_mhz": mx or None, "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    """Runs the unmodified reference (the copy under baseline/_ref) through its own public entry points for the same
    metric and configuration; nothing of this package is imported on that path (baseline/reference_runner.py)."""
    from baseline import reference_runner
    if args.task == "t2i":
        return reference_runner.run_t2i(args, ClockSampler)
    return reference_runner.run_sft(args, ClockSampler)


def t2i_bench(args):
    """Secondary metric of the baseline: 8B-MoT text-to-image, batch 1, 256 random prompt ids, 50 Euler steps
    with CFG 4, single GPU.  Published reference: 22.108 s / image on one H100 through transformers
    (docs/gpu_mem_profiler.md:27-34), 0.312 s / step with LightX2V (docs/inference_infra.md:116)."""
    import torch
    import torch.distributed as dist
    from sensenova_u1_b200.config import get_config
    from sensenova_u1_b200.inference.engine import InferenceEngine
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.ops import _lib
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    # rank = (guidance branch, token slice): 2 ranks sample guidance-parallel (one per branch); 4 and 8 ranks
    # additionally split every image's tokens over 2 / 4 ranks per branch (sequence parallel)
    if world not in (1, 2, 4, 8):
        raise SystemExit("the T2I task runs on 1, 2, 4 or 8 GPUs")
    from sensenova_u1_b200.inference.parallel import init_sampling_groups
    groups = init_sampling_groups(2, torch.device("cuda", local))
    group, sp_group, par_group, sp = groups.cfg_group, groups.sp_group, groups.par_group, groups.sp
    kw = {"num_layers": args.layers} if args.layers is not None else {}
    cfg = get_config(args.model, **kw)
    store = ParamStore(cfg, device="cuda", with_grads=False)
    store.init_weights(1234)
    eng = InferenceEngine(cfg, store)
    if sp_group is not None:
        eng.enable_sequence_parallel(sp_group)
    g = torch.Generator().manual_seed(0)
    cond = torch.randint(8, cfg.vocab_size, (256,), generator=g).pin_memory()
    uncond = torch.randint(8, cfg.vocab_size, (8,), generator=g).pin_memory()

    def run(seed):
        img = eng.t2i(cond, uncond, image_size=(args.image, args.image), num_steps=args.denoise_steps, cfg_scale=4.0,
                      timestep_shift=3.0, seed=seed, cfg_group=group, par_group=par_group)
        return img.cpu()          # the device -> host read of the result
    for i in range(max(1, args.warmup // 3)):
        run(i)
    _lib.check_status()
    sampler = ClockSampler(local)
    sampler.start()
    l0 = _lib.LAUNCHES
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = max(1, args.steps // 3)
    e0.record()
    for i in range(n):
        out = run(100 + i)
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / 1e3 / n
    if world > 1:
        t = torch.tensor([sec], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t)
    clocks = sampler.stop()
    _lib.check_status()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return 0
    print(json.dumps({
        "metric": f"T2I seconds per image ({args.image}x{args.image}, {args.denoise_steps} Euler steps, CFG 4, batch 1)",
        "value": sec, "unit": "s/image",
        "n_gpus": world, "steps": n, "warmup": max(1, args.warmup // 3), "ms_per_step": sec * 1e3 / args.denoise_steps,
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: 256 uniform-random prompt ids, N(0,1) pixel noise, random-init weights", "impl": "ours",
        "config": {"model": cfg.name, "layers": cfg.num_layers, "image": args.image, "denoise_steps": args.denoise_steps,
                   "cfg_scale": 4.0, "parallelism": "single" if world == 1 else "guidance-parallel x2 (peer memory)" + (
                       f" x sequence-parallel x{sp} (K/V and predictions through peer memory)" if sp > 1 else ""), "l2": "35 GB of weights streamed per denoise step"},
        "clocks": clocks, "gpu_launches": _lib.LAUNCHES - l0,
        "e2e": {"value": sec, "unit": "s/image", "h2d_bytes_per_step": int(cond.numel() + uncond.numel()) * 8,
                "d2h_bytes_per_step": int(out.numel() * 4)},
        "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 1e9, 2)}))
    return 0


def tp_pp_bench(args, tp: int, pp: int):
    """Long-context configuration of the baseline: tensor parallel x pipeline parallel (1F1B, ``--micro`` micro-batches
    per step), interleaved sequences with 8 images of 512 x 512.  tokens/s = micro-batches x seq_len / step time."""
    import torch
    import torch.distributed as dist
    from sensenova_u1_b200.config import get_config
    from sensenova_u1_b200.data.synthetic import interleaved_batch
    from sensenova_u1_b200.ops import _lib
    from sensenova_u1_b200.parallel.pipeline_engine import PipelineTrainer
    from sensenova_u1_b200.train.optimizer import AdamConfig
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    if world != tp * pp:
        raise SystemExit(f"--parallel tp{tp}pp{pp} needs {tp * pp} ranks, got {world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    kw = {"num_layers": args.layers} if args.layers is not None else {}
    cfg = get_config(args.model, **kw)
    pt = PipelineTrainer(cfg, tp, pp, dev, AdamConfig(lr=2e-4, beta2=0.95, clip_grad_norm=1.0), init_seed=1234,
                         max_tokens=args.seq_len)
    n_micro = args.micro
    host = [[interleaved_batch(cfg, args.seq_len, seed=100 * s + i).pin() for i in range(n_micro)] for s in range(2)]
    devb = [[b.to(dev) for b in hs] for hs in host]
    last = {}

    def dev_step(i):
        last["out"] = pt.step(devb[i % 2])

    def e2e_step(i):
        o = pt.step([b.to(dev, non_blocking=True) for b in host[i % 2]])
        last["e2e"] = {k: float(v) for k, v in o.items()}           # device -> host read (last stage's ranks)

    def timed(fn, steps):
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        dist.barrier(); torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)
    for i in range(args.warmup):
        dev_step(i)
    _lib.check_status()
    sampler = ClockSampler(local)
    if rank == world - 1:
        sampler.start()
    l0 = _lib.LAUNCHES
    ms_dev = timed(dev_step, args.steps)
    launches = _lib.LAUNCHES - l0
    clocks = sampler.stop() if rank == world - 1 else None
    _lib.check_status()
    tokens = n_micro * args.seq_len
    e2e = None
    if not args.no_e2e:
        e2e_step(0)
        ms_e2e = timed(e2e_step, args.steps)
        e2e = {"value": tokens * args.steps / (ms_e2e / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": sum(b.nbytes() for b in host[0]), "d2h_bytes_per_step": 4 * max(1, len(last.get("e2e", {}))),
               "ms_per_step": ms_e2e / args.steps}
    if rank == world - 1:          # a rank of the last stage holds the loss
        print(json.dumps({
            "metric": "8B-MoT long-context SFT tokens/s (device, max over ranks)", "value": tokens * args.steps / (ms_dev / 1e3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "impl": "ours",
            "data": "synthetic interleaved sequences (8 images 512x512 between Zipf text), random-init weights",
            "config": {"model": cfg.name, "layers": cfg.num_layers, "seq_len": args.seq_len, "micro_batches": n_micro,
                       "global_batch": n_micro, "parallelism": f"tp{tp} x pp{pp} (1F1B; peer-memory all-reduce, NCCL p2p on two communicators)",
                       "optimizer": "AdamW fp32 master, clip 1.0", "activation_checkpointing": "every layer recomputed in backward",
                       "l2": "inputs larger than L2 (whole weight set streamed every step)"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "final_loss": float(last["out"]["loss"]),
            "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 1e9, 2)}))
    dist.barrier()
    dist.destroy_process_group()
    return 0


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    if args.task == "t2i":
        return t2i_bench(args)
    import re
    m = re.fullmatch(r"tp(\d+)pp(\d+)", args.parallel)
    if m:
        return tp_pp_bench(args, int(m.group(1)), int(m.group(2)))
    import torch
    import torch.distributed as dist
    from sensenova_u1_b200.config import get_config
    from sensenova_u1_b200.data.synthetic import synthetic_batch
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.ops import _lib
    from sensenova_u1_b200.train.optimizer import AdamConfig
    from sensenova_u1_b200.train.trainer import Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    host_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        host_group = dist.new_group(backend="gloo")
    _lib.load()

    kw = {}
    if args.layers is not None:
        kw["num_layers"] = args.layers
    cfg = get_config(args.model, **kw)
    if args.parallel == "auto":
        args.parallel = "wp" if (world > 1 and not cfg.is_moe) else "dp"
    m_cp = re.fullmatch(r"cp(\d+)", args.parallel)
    cp = int(m_cp.group(1)) if m_cp else 1
    if cp > 1 and (cp != world or cfg.is_moe):
        raise SystemExit(f"--parallel cp{cp}: one packed sequence over all {world} ranks of a dense model")
    if cfg.is_moe and world > 1:
        # MoE family: experts split over all ranks (expert parallel = world), rows exchanged through
        # peer memory; everything else is data parallel + ZeRO-1
        kw["ep_size"] = world
        cfg = get_config(args.model, **kw)
    if args.parallel == "wp":
        from sensenova_u1_b200.parallel.weight_parallel import WeightParallelStore
        store = WeightParallelStore(cfg, dev)
    else:
        store = ParamStore(cfg, device=dev, shard_multiple=8 * 128 * max(world, 1),
                           symmetric_group=True if (world > 1 and args.comm == "peer") else None, ep_rank=rank)
    store.init_weights(seed=1234)
    trainer = Trainer(cfg, store, AdamConfig(lr=2e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0,
                                             clip_grad_norm=1.0), dp_group=None, host_group=host_group,
                      comm=args.comm, max_tokens=args.seq_len // cp, cp_group=dist.group.WORLD if cp > 1 else None)

    trainer.engine.recompute = args.recompute
    monitor = None
    if cfg.is_moe:
        from sensenova_u1_b200.utils.moe_monitor import MoEMonitor
        monitor = trainer.engine.monitor = MoEMonitor(ep_size=cfg.ep_size)
    n_distinct = 4
    if cp > 1:
        # context parallel: every rank builds the same packed sequence and keeps its zigzag share of the 128-row tiles
        from sensenova_u1_b200.data.batch import split_context_parallel
        host = [split_context_parallel(synthetic_batch(cfg, args.seq_len, seed=i), cp, rank, cfg).pin()
                for i in range(n_distinct)]
    else:
        host = [synthetic_batch(cfg, args.seq_len, seed=1000 * rank + i).pin() for i in range(n_distinct)]
    devb = [b.to(dev) for b in host]
    torch.cuda.synchronize()

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    host_ms = {}

    def timed(fn, steps):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        host_ms[fn.__name__] = (time.perf_counter() - t0) * 1e3 / steps     # host time to enqueue one step
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    last = {}

    def dev_step(i):
        last["out"] = trainer.step_on_device([devb[i % n_distinct]])

    def e2e_step(i):
        last["e2e"] = trainer.train_step([host[i % n_distinct]])

    for i in range(args.warmup):
        dev_step(i)
    if args.breakdown:
        trainer.profile_events = []
    _lib.check_status()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = _lib.LAUNCHES
    ms_dev = timed(dev_step, args.steps)
    launches = _lib.LAUNCHES - l0
    clocks = sampler.stop() if rank == 0 else None
    _lib.check_status()
    loss_val = float(last["out"]["loss"])

    tokens_per_step = args.seq_len * (world // cp)
    value = tokens_per_step * args.steps / (ms_dev / 1e3)
    e2e = None
    if not args.no_e2e:
        for i in range(2):
            e2e_step(i)
        ms_e2e = timed(e2e_step, args.steps)
        e2e = {"value": tokens_per_step * args.steps / (ms_e2e / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": host[0].nbytes(), "d2h_bytes_per_step": 4 * len(last["e2e"]),
               "ms_per_step": ms_e2e / args.steps}
    policy_label = {"full": "every layer recomputed in backward", "attention": "attention outputs kept, rest recomputed",
                    "none": "activations kept (no recompute)"}.get(getattr(trainer.engine, "_mode", "full"), "every layer")
    fixed = None
    # every rank picks its activation policy from its own free memory, so near a threshold the ranks can differ; the
    # extra fixed-policy steps below are collective work (flags / reductions between the ranks), so whether they run
    # must be the same decision everywhere: they run if any rank keeps activations
    keeps = getattr(trainer.engine, "_mode", "full") != "full"
    if world > 1:
        flag = torch.tensor([1.0 if keeps else 0.0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        keeps = bool(flag.item() > 0)
    if args.recompute == "auto" and not args.no_fixed_policy and keeps:
        # the automatic activation policy keeps more as memory allows, so the work per token changes with N; this second
        # figure pins the policy ("every layer recomputed", what the reference runs: checkpoint=1) so that values at
        # different N compare equal work
        trainer.engine.recompute = "full"
        trainer.engine._mode = None
        for i in range(2):
            dev_step(i)
        nfix = max(3, args.steps // 2)
        ms_fix = timed(dev_step, nfix)
        fixed = {"recompute": "full", "value": tokens_per_step * nfix / (ms_fix / 1e3), "unit": "tokens/s",
                 "ms_per_step": ms_fix / nfix, "steps": nfix}
        trainer.engine.recompute = args.recompute
        trainer.engine._mode = None
    elif args.recompute == "auto" and not args.no_fixed_policy:
        fixed = {"recompute": "full", "value": value, "unit": "tokens/s", "ms_per_step": ms_dev / args.steps,
                 "steps": args.steps, "note": "the automatic policy chose full recompute: same run as value"}
    if args.kernel_table:
        from torch.profiler import ProfilerActivity, profile
        sync_all()
        if rank == 0:
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                dev_step(0)
                torch.cuda.synchronize()
            rows = sorted(prof.key_averages(), key=lambda r: -r.device_time_total)
            busy = sum(r.device_time_total for r in rows)
            with open(args.kernel_table, "w") as f:
                f.write(f"# one step, rank 0 of {world}; sum of kernel time {busy / 1e3:.1f} ms "
                        f"(timed step {ms_dev / args.steps:.1f} ms); {sum(r.count for r in rows)} device activities\n")
                for r in rows[:60]:
                    f.write(f"{r.device_time_total / 1e3:10.2f} ms {100 * r.device_time_total / max(busy, 1):5.1f}% "
                            f"{r.count:6d}x  {r.key[:110]}\n")
        else:
            dev_step(0)
        sync_all()
    moe_load = None
    if monitor is not None:
        sm_ = monitor.summary()
        moe_load = {k.replace("moe/", "").replace("/mean_", "_"): round(v, 3) for k, v in sm_.items()
                    if "/mean_" in k and k.rsplit("mean_", 1)[1] in ("rank_max_over_mean", "max_over_mean", "idle_experts")}
    if rank == 0:
        line = {
            "metric": ("8B-MoT" if not cfg.is_moe else cfg.name) + " SFT tokens/s (device, max over ranks)", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev / args.steps,
            "higher_is_better": True, "scaling": "strong" if cp > 1 else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic packed text+image sequences, random-init weights",
            "impl": "ours",
            "config": {"model": cfg.name, "layers": cfg.num_layers, "params_b": round(cfg.num_params() / 1e9, 3),
                       "global_batch": world // cp, "seq_len": args.seq_len,
                       "parallelism": (f"cp{cp}+zero1({args.comm}): one packed sequence over {cp} GPUs, key / value blocks "
                                       "pulled from peer memory" if cp > 1 else
                                       f"wp{world}+zero1 (weight parallel over peer memory, tp1 pp1)" if args.parallel == "wp" else
                                       (f"dp{world}+zero1({args.comm})" + (f"+ep{world}(peer)" if cfg.ep_size > 1 else ""))
                                       if world > 1 else "single"),
                       "optimizer": f"AdamW fp32 master, {str(trainer.optim.state_dtype).split('.')[-1]} moments, clip 1.0",
                       "l2": "inputs larger than L2 (whole weight set streamed every step)",
                       "activation_checkpointing": policy_label},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "final_loss": loss_val,
            **({"fixed_policy": fixed} if fixed else {}),
            **({"moe_load": moe_load} if moe_load else {}),
            **({"breakdown": {"optimizer_ms_per_step": round(sum(a.elapsed_time(b) for a, b in trainer.profile_events)
                                                              / max(1, len(trainer.profile_events)), 2),
                              "host_ms_in_step_calls": round(host_ms.get("dev_step", 0.0), 1)}}
               if args.breakdown and trainer.profile_events else {}),
            "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 1e9, 2),
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
