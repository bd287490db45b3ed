"""Reference arm of ``bench.py``: runs the unmodified reference (a plain copy of its ``src`` and
``training`` trees under ``baseline/_ref``) through its own public entry points and stock code
path, on the same metric and configuration as this package's arm.

Nothing of ``sensenova_u1_b200`` is imported here.

* SFT: ``initialize_distributed_env`` -> ``get_model`` -> ``TrainerBuilder`` and, per step, the
  trainer's own batch preparation, ``execute_schedule`` (forward + backward) and optimizer step
  (training/train_sensenovau1.py:46-74, sensenovalm/core/trainer_builder.py:528-689), driven with
  the shipped 8B config file, ``wp_size = N`` (the shipped 8B mode, shell/train_u1/8B.sh:35-38),
  random-init weights and synthetic packed batches assembled by the reference's own collate
  function (sensenovavl/data/dataset_interleaved_iterable.py:1735-1947).
* T2I: ``NEOChatModel(NEOChatConfig(<8B dims>))`` random-init in bf16, flash-attn backend, stock
  ``t2i_generate`` (src/sensenova_u1/models/neo_unify/modeling_neo_chat.py:1691-1860) with a
  stand-in tokenizer that returns fixed random ids.

Third-party modules that the reference imports but the image lacks (``timm``, ``imageio``,
``decord``) are satisfied by the stand-ins in ``baseline/ref_shims`` (never reached by these
paths); apex / grouped_gemm / flash-attn's fused dense, rotary and cross-entropy extensions are
absent too, so the reference runs its own in-tree PyTorch fall-backs for those; the JSON line
lists them.
"""
from __future__ import annotations

import json
import math
import os
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"


def _unavailable(why: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def _paths(training: bool):
    if not (REF / "src" / "sensenova_u1").is_dir():
        return ("baseline/_ref holds no copy of the reference (pip install of the project fails offline: its build "
                "backend hatchling is not in the wheelhouse; copy src/ and training/ there with baseline/install_reference.py)")
    sys.path.insert(0, str(REF / "src"))
    if training:
        sys.path.insert(0, str(REF / "training"))
        sys.path.append(str(HERE / "ref_shims"))
    return None


def _max_over_ranks(x: float, device) -> float:
    import torch
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([x], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)
    return x


# ----------------------------------------------------------------------------------------------
# text-to-image
# ----------------------------------------------------------------------------------------------
class FixedIdsTokenizer:
    """The reference only calls ``tokenizer(query, return_tensors="pt")``.  The conditional query (system
    message + prompt) maps to 256 fixed random ids, the unconditional one to 8."""

    def __init__(self, vocab: int, seed: int = 0):
        import torch
        g = torch.Generator().manual_seed(seed)
        self.cond = torch.randint(8, vocab, (1, 256), generator=g)
        self.uncond = torch.randint(8, vocab, (1, 8), generator=g)

    def __call__(self, text, return_tensors="pt", **kw):
        return {"input_ids": (self.cond if len(text) > 200 else self.uncond).clone()}


def neo_8b_hf_config(layers=None):
    llm = dict(architectures=["Qwen3ForCausalLM"], hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
               head_dim=128, intermediate_size=12288, num_hidden_layers=layers or 42, vocab_size=151936,
               rms_norm_eps=1e-6, rope_theta=5_000_000.0, rope_theta_hw=10_000.0, max_position_embeddings=262144,
               tie_word_embeddings=False, attention_bias=False)
    vis = dict(patch_size=16, hidden_size=1024, llm_hidden_size=4096, downsample_ratio=0.5, rope_theta_vision=10_000.0)
    return dict(llm_config=llm, vision_config=vis, downsample_ratio=0.5, noise_scale=1.0, noise_scale_mode="resolution",
                noise_scale_base_image_seq_len=64, noise_scale_max_value=8.0, add_noise_scale_embedding=True,
                t_eps=0.05, time_schedule="standard", time_shift_type="exponential", base_shift=0.5, max_shift=1.15,
                base_image_seq_len=64, max_image_seq_len=4096, use_pixel_head=False, fm_head_dim=4096,
                fm_head_layers=2, fm_head_mlp_ratio=1, concat_time_token_num=0)


def run_t2i(args, ClockSampler) -> int:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        return _unavailable("the reference has no multi-GPU sampling path in-tree: its TP2/CFG2 numbers come from the external "
                            "LightLLM + LightX2V servers (docs/inference_infra.md:20-21); only N=1 runs")
    why = _paths(training=False)
    if why:
        return _unavailable(why)
    import torch
    from sensenova_u1.models.neo_unify import modeling_qwen3
    from sensenova_u1.models.neo_unify.configuration_neo_chat import NEOChatConfig
    from sensenova_u1.models.neo_unify.conversation import conv_templates
    from sensenova_u1.models.neo_unify.modeling_neo_chat import NEOChatModel
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    conf = neo_8b_hf_config(args.layers)
    conf["template"] = "sensenova-u1" if "sensenova-u1" in conv_templates else next(iter(conv_templates))
    rcfg = NEOChatConfig(**conf)
    torch.manual_seed(1234)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(dev):
            model = NEOChatModel(rcfg)
    finally:
        torch.set_default_dtype(old)
    model = model.to(dev, torch.bfloat16).eval()
    backend = "flash" if getattr(modeling_qwen3, "_HAS_FLASH_ATTN", False) else "sdpa"
    modeling_qwen3.set_attn_backend(backend)
    tok = FixedIdsTokenizer(conf["llm_config"]["vocab_size"])

    def run(seed):
        with torch.no_grad():
            img = model.t2i_generate(tok, "a synthetic prompt", cfg_scale=4.0, timestep_shift=3.0,
                                     image_size=(args.image, args.image), num_steps=args.denoise_steps, seed=seed)
        return img.float().cpu()
    warm = max(1, args.warmup // 3)
    n = max(1, args.steps // 3)
    for i in range(warm):
        run(i)
    sampler = ClockSampler(dev.index)
    sampler.start()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        out = run(100 + i)
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) / 1e3 / n
    clocks = sampler.stop()
    print(json.dumps({
        "metric": f"T2I seconds per image ({args.image}x{args.image}, {args.denoise_steps} Euler steps, CFG 4, batch 1)",
        "value": sec, "unit": "s/image", "n_gpus": 1, "steps": n, "warmup": warm,
        "ms_per_step": sec * 1e3 / args.denoise_steps, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "impl": "reference",
        "data": "synthetic: 256 fixed random prompt ids, N(0,1) pixel noise, random-init weights",
        "config": {"model": "SenseNova-U1-8B-MoT", "layers": conf["llm_config"]["num_hidden_layers"], "image": args.image,
                   "denoise_steps": args.denoise_steps, "cfg_scale": 4.0, "parallelism": "single",
                   "attention": backend, "path": "NEOChatModel.t2i_generate (transformers path)",
                   "l2": "35 GB of weights streamed per denoise step"},
        "clocks": clocks, "e2e": {"value": sec, "unit": "s/image", "h2d_bytes_per_step": 264 * 8,
                                  "d2h_bytes_per_step": int(out.numel() * 4)},
        "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 1e9, 2)}))
    return 0


# ----------------------------------------------------------------------------------------------
# supervised fine-tuning
# ----------------------------------------------------------------------------------------------
IMG_START, IMG_END, IMG_CONTEXT = 151670, 151671, 151669        # the reference's special-token ids


def _sft_env(args, world: int, job: str):
    """The knobs of training/shell/train_u1/8B.sh that the config file reads from the environment."""
    env = dict(JOB_NAME=job, zero1_size="-1", wp_size=str(world), tp_size="1", pp_size="1", lr="2e-4", weight_decay="0.0",
               grad_accm="1", total_steps="100000", init_steps="0", min_lr_ratio="0.1", mlp_lr_scale="1.0",
               num_imgs="144", seq_len=str(args.seq_len), max_pixels=str(1024 * 1024), min_pixels=str(256 * 256),
               add_noise_scale_embedding="true", noise_scale_mode="resolution", P_mean="-0.8", P_std="0.8",
               dataset_replacement="false", load_optimizer="model", SENSENOVALM_ENABLE_TIMEOUT="0")
    for k, v in env.items():
        os.environ.setdefault(k, v)


def _synthetic_feature(seq_len: int, seed: int, patch: int = 16, merge: int = 2):
    """One packed sequence in the form the reference's ``PackedDataset`` hands to its collate function: ~60 %
    Zipf(1.1) text ids, 1-4 images of 512-1024 px (one of them a generation target, followed by its
    understanding duplicate as the reference's t2i samples carry it), pixels uniform in [-1, 1]."""
    import numpy as np
    import torch
    rng = np.random.default_rng(seed)
    tp = patch * merge
    n_img = int(rng.integers(1, 5))
    ids, labels, data_index = [], [], []
    pixel_values, image_flags, gen_flags, gen_loss_flags, dup_flags, seq_lens = [], [], [], [], [], []
    budget_img = int(0.4 * seq_len)
    doc = 0

    def text(n):
        z = rng.zipf(1.1, size=n)
        t = (z % (IMG_CONTEXT - 8)) + 8
        ids.extend(t.tolist()); labels.extend(t.tolist()); data_index.extend([doc] * n)

    def image(h, w, gen):
        gh, gw = h // tp, w // tp
        n = gh * gw
        px = torch.from_numpy(rng.uniform(-1, 1, size=(3, h, w)).astype("float32"))
        copies = [(True, False)] + ([(False, True)] if gen else [])      # generation image, then its understanding duplicate
        if not gen:
            copies = [(False, False)]
        for is_gen, is_dup in copies:
            ids.extend([IMG_START] + [IMG_CONTEXT] * n + [IMG_END])
            labels.extend([-100] * (n + 2))
            data_index.extend([doc] * (n + 2))
            pixel_values.append(px)
            image_flags.append(1); gen_flags.append(1 if is_gen else 0); gen_loss_flags.append(1 if is_gen else 0)
            dup_flags.append(1 if is_dup else 0); seq_lens.append(n)
        return (n + 2) * len(copies)

    used_img = 0
    text(64)
    for i in range(n_img):
        h = int(rng.integers(512 // tp, 1024 // tp + 1)) * tp
        w = int(rng.integers(512 // tp, 1024 // tp + 1)) * tp
        gen = (i == 0)
        cost = ((h // tp) * (w // tp) + 2) * (2 if gen else 1)
        if used_img + cost > budget_img:
            break
        used_img += image(h, w, gen)
        text(int(rng.integers(64, 512)))
        if rng.random() < 0.5:
            doc += 1
    remaining = seq_len - len(ids)
    while remaining > 0:
        n = min(remaining, int(rng.integers(256, 2048)))
        text(n)
        remaining -= n
        doc += 1
    ids, labels, data_index = ids[:seq_len], labels[:seq_len], data_index[:seq_len]
    L = torch.long
    return {"input_ids": torch.tensor(ids, dtype=L), "labels": torch.tensor(labels, dtype=L),
            "type_ids": torch.zeros(len(ids), dtype=L), "data_index": torch.tensor(data_index, dtype=L),
            "pixel_values": pixel_values, "image_seq_lens": torch.tensor(seq_lens, dtype=L),
            "image_flags": torch.tensor(image_flags, dtype=L), "image_con_flags": None,
            "image_for_gen_flags": torch.tensor(gen_flags, dtype=torch.bool),
            "image_for_gen_loss_flags": torch.tensor(gen_loss_flags, dtype=torch.bool),
            "is_image_duplicated_for_und_flags": torch.tensor(dup_flags, dtype=torch.bool),
            "worker_state_key": "w0", "worker_state_dict": {}, "custom_infos": None}


class SyntheticLoader:
    """Stands where the reference's DataLoader stands: an endless iterator of collated batches."""

    def __init__(self, collate, seq_len, rank, distinct=4):
        self.batches = [collate([_synthetic_feature(seq_len, 1000 * rank + i)]) for i in range(distinct)]
        self.dataset = self
        self.batch_sampler = None
        self.i = 0

    def __iter__(self):
        return self

    def __next__(self):
        import copy
        b = self.batches[self.i % len(self.batches)]
        self.i += 1
        return copy.deepcopy(b)

    def __len__(self):
        return 1 << 30


def _transformers5_compat():
    """The reference training model sets ``self.tp_size`` on a ``PreTrainedModel`` subclass; it was written for
    transformers 4.43, where that name is free.  transformers 5 defines ``tp_size`` as a read-only property, so the
    assignment raises.  The installed library (not the reference) is given a setter that stores the value."""
    from transformers import PreTrainedModel
    prop = PreTrainedModel.__dict__.get("tp_size")
    if isinstance(prop, property) and prop.fset is None:
        def fget(self, _orig=prop.fget):
            return self.__dict__["_snu1_tp_size"] if "_snu1_tp_size" in self.__dict__ else _orig(self)

        def fset(self, value):
            self.__dict__["_snu1_tp_size"] = value
        PreTrainedModel.tp_size = property(fget, fset)
        return ["transformers 5: PreTrainedModel.tp_size made assignable"]
    return []


def sft_state_bytes(n_params: float, world: int) -> float:
    """Per-GPU bytes of the reference's training state under weight parallel ``world``: bf16 weights + bf16
    gradients + fp32 master + fp32 Adam moments (HybridZeroOptimizer) + the bf16 EMA copy the shipped config
    enables (averaged_model), all sharded 1/world."""
    return n_params * (2 + 2 + 4 + 4 + 4 + 2) / world


def run_sft(args, ClockSampler) -> int:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    n_params = 17.552e9 if args.layers is None else 1.3e9 + args.layers * 0.386e9
    # + two gathered layers + the fp32 logits of 16384 tokens x 151936 words with their gradient and bf16 copy
    # (parallel_output logits are materialised: 10 + 10 + 5 GB) + layer-input checkpoints and workspaces
    need = sft_state_bytes(n_params, world) + 2 * 0.772e9 * 2 + 30e9
    if need > 178e9:
        return _unavailable(f"the reference keeps bf16 weights and gradients, fp32 master weights, fp32 Adam moments "
                            f"(HybridZeroOptimizer) and a bf16 EMA copy: 18 bytes x 17.552 B parameters / {world} GPU(s) = "
                            f"{sft_state_bytes(n_params, world) / 1e9:.0f} GB per GPU, plus about 30 GB of logits and "
                            f"activations at 16384 tokens: more than the 180 GB of one B200; a rank that ran out of "
                            f"memory would leave the others waiting in a collective, so it is not attempted below 4 GPUs "
                            f"(weight parallel = N)")
    why = _paths(training=True)
    if why:
        return _unavailable(why)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29513")
    os.environ.setdefault("RANK", "0"); os.environ.setdefault("LOCAL_RANK", "0"); os.environ.setdefault("WORLD_SIZE", "1")
    run_dir = Path(os.environ.get("SNU1_REF_RUN_DIR", "/tmp/snu1_ref_run"))
    run_dir.mkdir(parents=True, exist_ok=True)
    os.chdir(run_dir)                       # the reference writes RUN/<job>/ logs and tensorboard files to the cwd
    _sft_env(args, world, job=f"bench_ref_n{world}")
    import torch
    import sensenovalm  # noqa: F401
    from sensenovalm.core.context import ParallelMode
    from sensenovalm.core.context import global_context as gpc
    from sensenovalm.initialize import initialize_distributed_env
    config_path = str(REF / "training" / "configs" / "sensenovavl_qwen3_gen" / "sensenovau1_8b_mot_sft.py")
    initialize_distributed_env(config=config_path, launcher="torch", master_port=int(os.environ["MASTER_PORT"]), seed=1024)
    if args.layers is not None:             # debugging aid only (a smaller stack): never a bench value
        gpc.config.model.num_layers = args.layers
    if os.environ.get("SNU1_REF_DEBUG_DIMS"):      # debugging aid only: tiny dims for a CPU dry run of this driver
        gpc.config.model.update(json.loads(os.environ["SNU1_REF_DEBUG_DIMS"]))
    gpc.config.ckpt.enable_save_ckpt = False
    # the shipped vit_cfg leaves the patch size to the class default (14) and relies on the released checkpoint's
    # config for 16; with random init the value of data.patch_size (16, what the released models use) is written in
    gpc.config.model.vit_cfg["patch_size"] = int(gpc.config.data.patch_size)
    compat = _transformers5_compat()
    from sensenovalm.core.trainer_builder import TrainerBuilder
    from sensenovalm.utils.common import get_current_device
    from sensenovavl.data.build_dataloader import len2weight
    from sensenovavl.data.dataset_interleaved_iterable import internevo_collate_fn
    from sensenovavl.train.pipeline import get_model
    import functools
    dev = get_current_device()
    data = gpc.config.data
    data.img_context_token_id, data.img_start_token_id = IMG_CONTEXT, IMG_START
    collate = functools.partial(
        internevo_collate_fn, max_item_length=args.seq_len, img_start_token_id=IMG_START, img_token_id=IMG_CONTEXT,
        img_end_token_id=IMG_END, ignored_token_ids=[IMG_START, IMG_END, IMG_CONTEXT], pad_id=0, micro_num=1,
        len2weight=functools.partial(len2weight, loss_reduction=data.loss_reduction),
        loss_reduction_all_gather=data.loss_reduction_all_gather, patch_size=data.patch_size)
    loader = SyntheticLoader(collate, args.seq_len, rank)
    model = get_model(gpc.config.model, gpc.config.data).to(dev)
    trainer = TrainerBuilder(model, loader, None, config=config_path, profiling=False, dataset_types=["en"],
                             dataloader_resume_mode="v0", very_begining_time=time.time(), launcher="torch",
                             seed=1024, port=int(os.environ["MASTER_PORT"]), backend="nccl")
    trainer.train()
    it = iter(loader)
    state = {"i": 0, "loss": None}

    def step():
        nonlocal it
        gpc.config.batch_count = state["i"]
        batch, it, _, _ = trainer._load_and_prepare_batch(state["i"], it)
        loss, *_ = trainer._forward_backward(batch)
        trainer._update_parameters()
        state["i"] += 1
        state["loss"] = loss
    import torch.distributed as dist

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for _ in range(args.warmup):
        step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        step()
        loss_host = float(state["loss"])            # the device -> host read of the step's loss
    e1.record()
    sync()
    wall = time.perf_counter() - t0
    ms = _max_over_ranks(e0.elapsed_time(e1), dev)
    clocks = sampler.stop() if rank == 0 else None
    tokens = args.seq_len * gpc.get_world_size(ParallelMode.DATA)
    value = tokens * args.steps / (ms / 1e3)
    b0 = loader.batches[0]
    h2d = int(b0[0]["input_ids"].numel() * 8 + b0[1].numel() * 8 + sum(x.numel() * 4 for x in b0[0]["images"] if x is not None))
    fallbacks = []
    import importlib.util as iu
    for mod, what in (("apex", "RMSNorm / l2-norm: in-tree PyTorch (no apex)"),
                      ("grouped_gemm", "grouped GEMM: unused by the dense model (no grouped_gemm)"),
                      ("fused_dense_lib", "linear wgrad: torch.matmul (no flash-attn fused_dense_lib)"),
                      ("rotary_emb", "RoPE: in-tree PyTorch (no flash-attn rotary_emb)"),
                      ("xentropy_cuda_lib", "cross entropy: in-tree vocab-parallel CE (no flash-attn xentropy)")):
        if iu.find_spec(mod) is None:
            fallbacks.append(what)
    if rank == 0:
        print(json.dumps({
            "metric": "8B-MoT SFT tokens/s (device, max over ranks)", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": "reference",
            "data": "synthetic packed text+image sequences (reference collate function), random-init weights",
            "config": {"model": "SenseNova-U1-8B-MoT", "layers": int(gpc.config.model.num_layers), "seq_len": args.seq_len,
                       "global_batch": gpc.get_world_size(ParallelMode.DATA),
                       "parallelism": f"wp{world}+zero1 (ISP weight parallel, the shipped 8B mode), tp1 pp1",
                       "attention": "torch.compile(flex_attention) with the reference BlockMask",
                       "optimizer": "HybridZeroOptimizer, fp32 master + fp32 moments, clip 1.0", "activation_checkpointing": "every layer (checkpoint=1)",
                       "fallbacks": fallbacks + compat, "torch": torch.__version__,
                       "l2": "inputs larger than L2 (whole weight set streamed every step)"},
            "clocks": clocks, "final_loss": loss_host,
            "e2e": {"value": tokens * args.steps / wall, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 1e9, 2)}))
    if world > 1:
        dist.barrier()
    return 0
