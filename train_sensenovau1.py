#!/usr/bin/env python
"""Training entry point: ``torchrun ... train_sensenovau1.py --config C --launcher torch --backend nccl``.

Same command line and config schema as the reference (training/train_sensenovau1.py:46-89,
initialize/launch.py:36-66).  Data: the jsonl meta file named by ``data.meta_path`` when a tokenizer is
available, otherwise synthetic packed sequences of the configured length.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def get_parser():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--launcher", default="torch", choices=["torch", "slurm"])
    ap.add_argument("--host", default=None)
    ap.add_argument("--port", type=int, default=8888)
    ap.add_argument("--world_size", type=int, default=None)
    ap.add_argument("--rank", type=int, default=None)
    ap.add_argument("--local_rank", type=int, default=None)
    ap.add_argument("--backend", default="nccl")
    ap.add_argument("--seed", type=int, default=1024)
    ap.add_argument("--profiling", action="store_true")
    ap.add_argument("--dataloader_resume_mode", default="v1")
    ap.add_argument("--enable_ali_topology", action="store_true", help="accepted for compatibility: rank order follows the launcher")
    ap.add_argument("--disable_volc_topology", action="store_true", help="accepted for compatibility: rank order follows the launcher")
    ap.add_argument("--max_steps", type=int, default=None, help="stop early (smoke runs)")
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (smoke runs)")
    return ap


def launch_env(args):
    if args.launcher == "slurm":
        os.environ.setdefault("RANK", os.environ.get("SLURM_PROCID", "0"))
        os.environ.setdefault("WORLD_SIZE", os.environ.get("SLURM_NTASKS", os.environ.get("SLURM_NPROCS", "1")))
        os.environ.setdefault("LOCAL_RANK", os.environ.get("SLURM_LOCALID", "0"))
        os.environ.setdefault("MASTER_ADDR", args.host or "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(args.port))
    for k, v in (("RANK", args.rank), ("WORLD_SIZE", args.world_size), ("LOCAL_RANK", args.local_rank)):
        if v is not None:
            os.environ[k] = str(v)
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))


def make_batches(cfg, mcfg, seq_len, seed, data_rank, data_world):
    """Endless iterator of packed batches for this data-parallel rank: the annotation files named by
    ``data.meta_path`` (tokenised, condition-dropped, packed best-fit into ``seq_len`` rows), or
    synthetic packed sequences when no meta file is configured."""
    from sensenova_u1_b200.data.synthetic import synthetic_batch
    meta = (cfg.data.get("meta_path") if hasattr(cfg.data, "get") else None) or None
    folder = (cfg.data.get("train_folder") if hasattr(cfg.data, "get") else None) or None
    text_stream = None
    if folder and os.path.isdir(str(folder)):
        # text-only data (data.train_folder): one-document-per-line token files, packed by cutting (or by padding with
        # data.pack_sample_into_one = False and text_pack_mode=pad), rows dealt over the data-parallel ranks
        import glob as _glob
        from sensenova_u1_b200.data.tokenized import JsonlTokenFile, PackedDocumentDataset
        files = sorted(_glob.glob(os.path.join(str(folder), "**", "*.jsonl"), recursive=True))
        if not files:
            raise FileNotFoundError(f"data.train_folder {folder}: no *.jsonl token files")
        min_len = int(cfg.data.get("min_length", 0) or 0)
        text_stream = iter(PackedDocumentDataset([JsonlTokenFile(f, min_len) for f in files], mcfg, seq_len,
                                                 mode=os.environ.get("text_pack_mode", "cut"), seed=seed, rank=data_rank,
                                                 world=data_world, epochs=int(cfg.data.get("total_epochs", -1) or -1)))
        if not meta or not os.path.isfile(str(meta)):
            return text_stream
    if not meta or not os.path.isfile(str(meta)):
        def synth():
            i = 0
            while True:
                yield synthetic_batch(mcfg, seq_len, seed=seed + i * data_world + data_rank)
                i += 1
        return synth()
    from sensenova_u1_b200.data.multimodal import CfgDrop, ConversationDataset
    from sensenova_u1_b200.data.options import DataOptions, image_loader_from_options
    from sensenova_u1_b200.data.packing import PackedDataset, RestartableLoader
    opts = DataOptions.from_config(cfg.data)
    tok_path = cfg.data.get("tokenizer_path")
    if tok_path and os.path.isdir(str(tok_path)):
        from transformers import AutoTokenizer
        tk = AutoTokenizer.from_pretrained(tok_path, trust_remote_code=True)
        tokenize = lambda s: tk(s, add_special_tokens=False)["input_ids"]
    else:
        from sensenova_u1_b200.inference.api import ByteTokenizer
        tokenize = ByteTokenizer(mcfg.vocab_size).encode
    E = os.environ.get
    drop = CfgDrop(float(E("cfg_txt_uncond_drop_prob", 0.0)), float(E("cfg_img_uncond_drop_prob", 0.0)),
                   float(E("cfg_txtimg_uncond_drop_prob", 0.0)),
                   str(E("cfg_is_uncond_drop_independent", "true")).lower() in ("1", "true", "yes"))
    load = image_loader_from_options(opts)       # pixel budgets of understanding / generation images, shared per sample
    from sensenova_u1_b200.data.multimodal import ChatOptions
    g = lambda k, d: cfg.get(k, d) if hasattr(cfg, "get") else d
    chat_opts = ChatOptions(thinking_method=str(g("thinking_method", "sys")), st_prompt_ratio=float(g("st_prompt_ratio", 0.0) or 0.0),
                            rm_all_think_token=bool(g("rm_all_think_token", False)),
                            image_token_position_random=str(g("image_token_position_random", "none")))

    def dataset_weights():
        """Sampling weight per annotation file when the config mixes by kind (caption pairs / plain pairs / the
        rest, ``data.mm_cc_data_weights`` ...); otherwise the meta file's ``repeat_time``."""
        if not (opts.mm_cc_data_weights or opts.mm_plain_pair_data_weights or opts.llm_data_weights):
            return None
        import json
        m = json.loads(open(meta).read())
        names = sorted(m)
        kinds = [m[n].get("kind", "cc" if m[n].get("data_type") == "mm_cc" else "paired") for n in names]
        lengths = [int(m[n].get("length", 0)) or sum(1 for ln in open(m[n]["annotation"]) if ln.strip()) for n in names]
        return opts.mixing_weights(kinds, lengths)

    def make():
        src = ConversationDataset(meta, tokenize, load, drop, rank=data_rank, world=data_world, seed=seed,
                                  und_loss=opts.enabel_und_loss and str(E("enable_und_loss", "true")).lower() in ("1", "true", "yes"),
                                  min_length=opts.min_length, weights=dataset_weights(), max_epochs=opts.total_epochs,
                                  chat=chat_opts, min_num_frame=opts.min_num_frame, max_num_frame=opts.max_num_frame,
                                  frame_max_pixels=max(opts.min_pixels, opts.max_pixels // max(1, opts.max_num_frame)))
        return iter(PackedDataset(src, mcfg, opts.packed_tokens if opts.max_packed_tokens else seq_len,
                                  num_images_expected=opts.num_images_expected, max_buffer_size=opts.max_buffer_size,
                                  max_age=opts.packed_buffer_stale_threshold, seed=seed + data_rank,
                                  loss_reduction=opts.loss_reduction))
    mm_stream = iter(RestartableLoader(make))
    share = float(opts.llm_data_weights or 0.0)
    if text_stream is None or share <= 0.0:
        return mm_stream

    def mixed():
        """Each micro-batch is a text-only row with probability data.llm_data_weights, else a multimodal row."""
        import random
        rng = random.Random(seed * 7919 + data_rank)
        while True:
            try:
                yield next(text_stream) if rng.random() < share else next(mm_stream)
            except StopIteration:              # one of the streams has used up its epochs: the mix ends with it
                return
    return mixed()


def main(argv=None):
    args = get_parser().parse_args(argv)
    rank, world, local = launch_env(args)
    import torch
    import torch.distributed as dist
    from sensenova_u1_b200.data.synthetic import synthetic_batch
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.parallel.context import ParallelContext, ParallelMode, init_distributed
    from sensenova_u1_b200.train import config as C
    from sensenova_u1_b200.train.checkpoint import CheckpointManager, LoadMask, import_hf
    from sensenova_u1_b200.train.metrics import (AccPerplex, ThroughputStats, Timers, TrainRecord, WandbWriter, Writer, RankLog, step_tflops,
                                                  format_line)
    from sensenova_u1_b200.train.schedulers import Beta2Scheduler, FineTuneCosineAnnealingWarmupLR
    from sensenova_u1_b200.train.trainer import Trainer
    from sensenova_u1_b200.utils.watchdog import Watchdog

    use_cuda = args.backend == "nccl" and torch.cuda.is_available()
    dev = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(local)
    if world > 1:
        init_distributed(args.backend if use_cuda else "gloo", device=dev if use_cuda else None)
    cfg = C.sanity_check(C.Config.from_file(args.config), world)
    torch.manual_seed(args.seed)
    torch.backends.cudnn.benchmark = bool(cfg.get("cudnn_benchmark", False))
    torch.backends.cudnn.deterministic = bool(cfg.get("cudnn_deterministic", False))
    pc = ParallelContext(C.parallel_config_from(cfg), rank=rank, world_size=world, create_groups=world > 1)
    tp, pp = pc.get_world_size(ParallelMode.TENSOR), pc.get_world_size(ParallelMode.PIPELINE)
    use_pipe = tp > 1 or pp > 1
    if use_pipe:
        # tensor x pipeline parallel (parallel/pipeline_engine.py): rank = pp_rank * tp + tp_rank, every rank steps the
        # same micro-batches, the last stage holds the losses
        if not use_cuda:
            raise SystemExit("tensor / pipeline parallel training runs on the CUDA engine (backend nccl)")
        if tp * pp != world:
            raise SystemExit(f"tp_size {tp} x pp_size {pp} must equal the {world} ranks of the job "
                             "(no data-parallel replicas of a tensor x pipeline group in this build)")
    wp = pc.get_world_size(ParallelMode.WEIGHT)
    use_wp = False
    if wp > 1:
        # weight parallel (the reference's ISP mode with tp = 1): every rank keeps 1/wp of each weight, gathers a layer
        # right before it is used and reduce-scatters its gradients (parallel/weight_parallel.py).  Built for the case
        # the shipped configs use, one weight-parallel group over all ranks; other splits run as data parallel + ZeRO-1
        # over the same ranks, which computes the same update with replicated weights.
        use_wp = use_cuda and wp == world and os.environ.get("weight_parallel", "on") != "off"
        if rank == 0 and not use_wp:
            print(f"note: weight parallel size {wp} on {world} ranks runs as data parallel + ZeRO-1 "
                  "(same global batch and gradients; weights replicated, optimizer state sharded)", flush=True)
    if cfg.parallel.zero1.get("fsdp") and world > 1 and use_cuda and not use_pipe and not use_wp:
        # fully-sharded mode (the reference's parallel.zero1.fsdp): parameters, gradients and optimizer states sharded
        # over all ranks, a layer's weights gathered right before use: that is the weight-parallel engine over the world
        use_wp = os.environ.get("weight_parallel", "on") != "off"
        if rank == 0 and use_wp:
            print("parallel.zero1.fsdp: running the weight-parallel (fully sharded) engine over all ranks", flush=True)
    if use_wp and any(cfg.model.get(k) for k in ("freeze_llm", "freeze_backbone")):
        use_wp = False                                 # frozen ranges live in the replicated-weight optimizer
        if rank == 0:
            print("note: frozen branches run as data parallel + ZeRO-1 (weight-parallel mode updates every weight)", flush=True)
    over = {"num_layers": args.layers} if args.layers else {}
    ep = pc.get_world_size(ParallelMode.EXPERT) if use_cuda else 1
    if ep > 1:
        if ep != world:
            raise SystemExit(f"expert parallel size {ep}: this entry point splits the experts over all {world} ranks "
                             "(set ep_size to the world size or to 1)")
        over["ep_size"] = ep
    mcfg = C.model_config_from(cfg, **over)
    # context parallel: cp_size consecutive ranks share one packed sequence (tiles dealt zigzag)
    cp = int(os.environ.get("cp_size", "1")) if use_cuda else 1
    if cp > 1 and (world % cp or mcfg.is_moe):
        raise SystemExit("cp_size must divide the world size (dense model only)")
    cp_group, cp_rank, data_rank, data_world = None, 0, rank, world
    if cp > 1:
        for g0 in range(0, world, cp):
            grp = dist.new_group(list(range(g0, g0 + cp)))
            if g0 <= rank < g0 + cp:
                cp_group = grp
        cp_rank, data_rank, data_world = rank % cp, rank // cp, world // cp
    hf_dir = cfg.model.get("model_name_or_path")
    if use_wp and (ep > 1 or cp > 1):
        raise SystemExit("weight parallel is combined with neither expert nor context parallel in this build")
    if use_pipe and (use_wp or ep > 1 or cp > 1 or mcfg.is_moe):
        raise SystemExit("tensor / pipeline parallel is combined with neither weight, expert nor context parallel "
                         "(dense model only) in this build")
    pt = None
    if use_pipe:
        from sensenova_u1_b200.parallel.pipeline_engine import PipelineTrainer
        full = import_hf(hf_dir, device=dev, with_grads=False, strict=False) if (hf_dir and os.path.isdir(hf_dir)) else None
        store = None                                   # built by the pipeline trainer: this rank's stage and slice
    elif use_wp:
        from sensenova_u1_b200.parallel.weight_parallel import WeightParallelStore
        store = WeightParallelStore(mcfg, dev)
        if hf_dir and os.path.isdir(hf_dir):
            store.load_from(import_hf(hf_dir, device=dev, with_grads=False, strict=False))
        else:
            store.init_weights(args.seed)
    elif hf_dir and os.path.isdir(hf_dir):
        store = import_hf(hf_dir, device=dev, with_grads=True, strict=False)
    else:
        store = ParamStore(mcfg, device=dev, shard_multiple=8 * 128 * max(world, 1),
                           dtype=torch.bfloat16 if use_cuda else torch.float32,
                           grad_dtype_mat=None if use_cuda else torch.float32,
                           symmetric_group=True if (use_cuda and world > 1) else None, ep_rank=rank if ep > 1 else 0)
        store.init_weights(args.seed)
    host_group = dist.new_group(backend="gloo") if (world > 1 and use_cuda) else None
    if use_pipe:
        data_rank, data_world = 0, 1                   # one stream for the whole tensor x pipeline group
    ema = float(cfg.averaged_model.decay) if (cfg.get("averaged_model") or {}).get("enable") and world > 1 else 0.0
    seq_len, micro = int(cfg.data.seq_len), int(cfg.data.micro_num)
    from sensenova_u1_b200.data.options import DataOptions
    dopts = DataOptions.from_config(cfg.data)      # validated view of the data section
    from sensenova_u1_b200.data.options import BatchSkipper
    skip_batch = BatchSkipper(dopts.skip_batches)
    consumed = 0                                   # micro-batches this rank has drawn (checkpointed)
    comm = os.environ.get("zero_comm", "peer") if (use_cuda and world > 1) else "nccl"
    adam_cfg = C.adam_config_from(cfg)
    mm = cfg.model
    if use_pipe and any(mm.get(k) for k in ("freeze_llm", "freeze_backbone")):
        raise SystemExit("freeze_llm / freeze_backbone are not combined with tensor / pipeline parallel in this build")
    if any(mm.get(k) for k in ("freeze_llm", "freeze_backbone")):
        from sensenova_u1_b200.train.freeze import count_frozen, frozen_ranges
        adam_cfg.frozen = frozen_ranges(store, bool(mm.get("freeze_llm")), bool(mm.get("freeze_backbone")),
                                        bool(mm.get("unfreeze_lm_head")), bool(mm.get("unfreeze_mot_gen")))
        if rank == 0:
            print(f"frozen parameters: {count_frozen(adam_cfg.frozen) / 1e9:.3f} B", flush=True)
    if use_pipe:
        pt = PipelineTrainer(mcfg, tp, pp, dev, adam_cfg, init_seed=args.seed, full_store=full,
                             schedule=os.environ.get("pp_schedule", "zero_bubble" if cfg.parallel.pipeline.get("zero_bubble") else "1f1b"),
                             max_tokens=seq_len)
        del full
        tr, store = pt.trainer, pt.store
    else:
        tr = Trainer(mcfg, store, adam_cfg, host_group=host_group, grad_accum=micro,
                     ema_decay=ema, comm=comm, max_tokens=seq_len // cp, cp_group=cp_group)
    log_rank = world - 1 if use_pipe else 0            # with pipeline stages the losses live on the last one
    if tr.engine is not None and not use_pipe:
        # activation policy: "auto" (by free memory), "full" (every layer recomputed in backward; what the
        # reference's model.checkpoint = 1 does), "attention" (attention outputs kept), "none" (no recompute)
        policy = os.environ.get("activation_policy", mm.get("activation_policy", "auto"))
        if policy not in ("auto", "full", "attention", "none"):
            raise ValueError(f"unknown activation policy {policy!r}")
        tr.engine.recompute = policy
    if tr.engine is not None and mm.get("freeze_llm") and not mcfg.is_moe:
        # frozen understanding branch (and frozen generation branch unless unfreeze_mot_gen): no weight gradients
        tr.engine.skip_wgrad_groups = (0,) if mm.get("unfreeze_mot_gen") else (0, 1)
    batches_iter = make_batches(cfg, mcfg, seq_len, args.seed, data_rank, data_world)
    ls = cfg.lr_scheduler
    sched = FineTuneCosineAnnealingWarmupLR(float(cfg.adam.lr), int(ls.total_steps), int(ls.get("init_steps", 0)),
                                            float(ls.get("warmup_ratio", 0)), float(ls.get("eta_min", 0)),
                                            cfg.get("lr_scheduler_type", "cosine"), int(cfg.get("lr_scheduler_offset", 0)))
    b2 = Beta2Scheduler(**{k: v for k, v in dict(cfg.beta2_scheduler).items() if k in ("init_beta2", "c", "cur_iter")})
    run_dir = f"RUN/{cfg.get('JOB_NAME', 'job')}/{time.strftime('%Y%m%d-%H%M%S')}"
    writer = Writer(run_dir, rank, enable_tb=bool(cfg.get("enable_tb", True)), report_rank=log_rank,
                    tensorboard_folder=cfg.get("tensorboard_folder") or os.environ.get("tensorboard_folder"),
                    resume_tb_folder=cfg.get("resume_tb_folder") or os.environ.get("resume_tb_folder"))
    rlog = RankLog(run_dir, rank, echo=False)      # echo is decided per line: the logging rank depends on the layout
    wandb_writer = WandbWriter(name=str(cfg.get("JOB_NAME", "job")), rank=0 if rank == log_rank else 1)
    record = TrainRecord(dp_world=data_world if world > 1 else 1, group=None if use_pipe else host_group)
    acc_metric = AccPerplex(("all",), group=None if use_pipe else host_group)
    if tr.engine is not None:
        tr.engine.per_task_losses = True
    ck = cfg.ckpt
    mgr = CheckpointManager(ck.save_ckpt_folder, int(ck.checkpoint_every), 0 if ck.oss_snapshot_freq == float("inf") else int(ck.oss_snapshot_freq),
                            ck.get("stop_file_path"), bool(ck.auto_resume), dp_rank=0 if (use_wp or use_pipe) else rank,
                            zero_rank=0 if use_pipe else rank, wp_rank=rank if use_wp else None, wp_size=world if use_wp else 1,
                            ep_rank=rank if ep > 1 else 0, tp_rank=pt.tp_rank if use_pipe else 0, tp_size=tp if use_pipe else 1,
                            pp_rank=pt.pp_rank if use_pipe else 0, layer_offset=pt.layers[0] if use_pipe else 0,
                            local_work_folder=ck.get("async_upload_tmp_folder") if ck.get("async_upload", True) else None) \
        if ck.enable_save_ckpt else None
    step = 0
    if mgr is not None:
        mgr.ping()                                     # an unwritable checkpoint folder ends the job before step 1
        res = mgr.try_resume(store, tr.optim, LoadMask.parse((ck.get("load_ckpt_info") or {}).get("content", "all")))
        if res is not None:
            d, (ts, ss, ds) = res
            step = int((ts or {}).get("step", 0))
            if (ts or {}).get("record"):
                record.load_state_dict(ts["record"])
            if (ts or {}).get("moe_selection_bias") and getattr(tr.engine, "sel_bias", None):
                tr.engine.load_selection_bias_state(ts["moe_selection_bias"])
            if ss:
                sched.load_state_dict(ss)
            saved_ema = mgr.load_ema(d) if tr.ema is not None else None
            if saved_ema is not None and all(k in tr.ema and saved_ema[k].shape == tr.ema[k].shape for k in saved_ema):
                for k, v in saved_ema.items():         # the averaged weights continue instead of restarting from the weights
                    tr.ema[k].copy_(v.to(tr.ema[k].device))
            # data: replay the stream up to the batches this rank had consumed (the streams are deterministic in
            # their seed; the reference's "v0" dataloader resume, core/trainer_builder.py:67-120)
            consumed = int((ds or {}).get("consumed_batches", step * micro))
            for _ in range(consumed):
                next(batches_iter)
            if rank == log_rank:
                print(f"resumed from {d} at step {step}", flush=True)
    from sensenova_u1_b200.utils.diagnostics import (MemoryWatch, bind_to_gpu_numa_node, check_replicas_equal,
                                                     warmup_process_groups)
    if use_cuda and os.environ.get("bind_numa", "on") != "off":
        node = bind_to_gpu_numa_node(local)            # host threads next to the GPU; a no-op where sysfs says nothing
        if node is not None and rank == log_rank:
            print(f"rank {rank}: host threads bound to NUMA node {node}", flush=True)
    if world > 1:
        warmup_process_groups([dist.group.WORLD, host_group, cp_group])
        if not (use_wp or use_pipe or ep > 1 or cp > 1) and os.environ.get("check_replicas", "on") != "off":
            # data-parallel replicas must start from identical weights (a missed broadcast or a rank-dependent seed
            # shows here, not as a slow divergence)
            check_replicas_equal(store.p.items(), group=host_group)
    memwatch = MemoryWatch(int(cfg.data.get("empty_cache_and_diag_interval", 50) or 50),
                           log=(lambda line: print(line, flush=True)) if rank == log_rank else (lambda line: None))
    wd = Watchdog()
    hb = None
    if world > 1:
        # every rank reports its step into the rendezvous store; when a phase runs out of time the watchdog says which
        # ranks went quiet before it acts (a dead peer shows up as "rank 5 silent", not only as "my collective hangs")
        try:
            from sensenova_u1_b200.utils.watchdog import Heartbeat
            hb = Heartbeat(dist.distributed_c10d._get_default_store(), rank, world)
            act = wd.on_timeout

            def on_timeout(phase, late, _act=act):
                try:
                    quiet = hb.silent_ranks(float(os.environ.get("heartbeat_max_age_s", 120)))
                    sys.stderr.write(f"[watchdog] rank {rank}: phase {phase!r} late by {late:.1f} s; silent ranks: {quiet}\n")
                    sys.stderr.flush()
                finally:
                    if _act is not None:
                        _act(phase, late)
            wd.on_timeout = on_timeout
        except Exception:
            hb = None
    timers, tput = Timers(), ThroughputStats()
    total = int(args.max_steps or ls.total_steps)
    prof = None
    if args.profiling:
        from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler
        prof = profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA],
                       schedule=schedule(skip_first=3, wait=1, warmup=1, active=1),
                       on_trace_ready=tensorboard_trace_handler(f"{run_dir}/traces/rank{rank}"))
        prof.start()
    while step < total:
        t0 = time.perf_counter()
        with wd.phase("load_batch"):
            # micro-batches of this step: the full count, or the ramp-up schedule's (data.rampup_batch_size)
            n_micro = dopts.batch_size_at(step, micro)
            try:
                batches = [next(batches_iter) for _ in range(n_micro)]
            except StopIteration:          # data.total_epochs passes over the data are done
                if rank == 0:
                    print(f"data exhausted after step {step}", flush=True)
                break
            consumed += n_micro
            if cp > 1:
                from sensenova_u1_b200.data.batch import split_context_parallel
                batches = [split_context_parallel(b, cp, cp_rank, mcfg) for b in batches]
            if use_cuda:
                batches = [b.pin() for b in batches]
        if skip_batch(step):                           # data.skip_batches: drawn, not trained on; schedules move on
            sched.step()
            b2.step()
            step += 1
            if rank == log_rank:
                print(f"step={step} skipped (data.skip_batches)", flush=True)
            continue
        lr = sched.step()
        tr.optim.cfg.beta2 = b2.step()
        t_fb = time.perf_counter()
        with wd.phase("fwd_bwd_step"):
            if use_pipe:
                out_t = pt.step([b.to(dev, non_blocking=True) for b in batches], lr=lr)
                out = {k: float(v) for k, v in out_t.items()}            # filled on the last stage's ranks
            else:
                out = tr.train_step(batches, lr=lr)
        fb_time = time.perf_counter() - t_fb           # forward, backward and update (the host read of the loss ends it)
        step += 1
        dt = time.perf_counter() - t0
        m = dict(out, lr=lr, step_time=dt)
        n_tok = sum(b.n_tokens for b in batches)
        # data parallel: each rank steps its own batches; tensor x pipeline: the whole group steps one set
        m.update(tput.update(n_tok, 1 if use_pipe else world, world, dt))
        m.update(step_tflops(mcfg, n_tok, dt, world=world if use_pipe else 1))
        m.update(record.update(batches, skipped_steps=int(tr.optim.skipped)))
        pad = int(getattr(record, "last", {}).get("num_padding_tokens", 0))
        m["tgs_wo_padding"] = (n_tok - pad) * (1 if use_pipe else world) / world / max(dt, 1e-9)
        m["fwd_bwd_time"] = fb_time
        m["loss_scale"] = 1.0                          # bf16 training: no loss scaling (the key is logged for parity)
        if "ce_rows" in out:
            acc_metric.update(out.get("ce_correct", 0.0), out["ce_rows"], out.get("ce", 0.0) * out["ce_rows"])
            m.update(acc_metric.get_metric())
        m["adam_beta2"] = float(tr.optim.cfg.beta2)
        writer.add_scalars(m, step)
        wandb_writer.add_scalars(m, step)
        if step % max(1, int(os.environ.get("LOG_EVERY", 1))) == 0 or step == total:
            rlog(format_line(step, m), echo=rank == log_rank)
        if prof is not None:
            prof.step()
        if hb is not None:
            hb.beat(step)
        if use_cuda:
            memwatch.step(step, tag=f"rank {rank}")
        every = int(os.environ.get("check_replicas_every", 500))
        if world > 1 and every > 0 and step % every == 0 and not (use_wp or use_pipe or ep > 1 or cp > 1) \
                and os.environ.get("check_replicas", "on") != "off":
            check_replicas_equal(store.p.items(), group=host_group)      # replicated weights must not drift apart
        if mgr is not None:
            save, kind, stop = mgr.decide(step, total)
            if save:
                with wd.phase("save_checkpoint"):
                    ts_out = {"step": step, "record": record.state_dict()}
                    if getattr(tr.engine, "sel_bias", None):
                        ts_out["moe_selection_bias"] = tr.engine.selection_bias_state()
                    mgr.save(step, store, tr.optim, ts_out, sched.state_dict(),
                             {"consumed_batches": consumed, "data_rank": data_rank}, tr.ema, kind,
                             model_cfg=mcfg if use_pipe else None)
            if stop:
                break
    if prof is not None:
        prof.stop()
    if mgr is not None:
        mgr.close()                                    # a remote checkpoint folder: outstanding uploads and the last marker
    writer.close()
    rlog.close()
    wandb_writer.close()
    wd.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    try:
        sys.exit(main())
    except Exception:
        # which machine and rank failed: the first thing needed when one of many ranks dies
        # (the reference wraps its entry point the same way, utils/common.py:489-498)
        import socket
        import traceback
        sys.stderr.write(f"[{socket.gethostname()}] rank {os.environ.get('RANK', '0')} failed:\n{traceback.format_exc()}")
        sys.stderr.flush()
        raise
