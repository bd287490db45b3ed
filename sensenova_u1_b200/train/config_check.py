"""Checks of the config sections whose keys select behaviour this package fixes.

The reference's model / loss / lr_scale / grad_scaler / ckpt sections carry switches for code paths of its generic
LLM trainer (norm type, biases, sliding window, interleaved rotary layout, fp16 loss scaling, layer-wise lr decay ...)
that the shipped SenseNova-U1 configs leave at one value (training/configs/sensenovavl_qwen3_gen/*.py,
sensenovalm/initialize/launch.py:69-691).  This package implements that one value.  Rather than ignore such a key, the
config loader checks it here: the shipped value passes, any other value raises with the reason, and keys that only
tune the reference's own runtime (fused-kernel toggles, upload queues, alert hooks) are listed as having no
counterpart.  ``check_sections`` returns the notes for keys that were accepted without effect."""
from __future__ import annotations

from typing import Any, Dict, List, Mapping, Tuple

# key -> (accepted values, what this package does)
_MODEL_FIXED: Dict[str, Tuple[tuple, str]] = {
    "norm_type": (("rmsnorm",), "RMSNorm kernels only"),
    "qkv_bias": ((False,), "projections have no bias"),
    "use_sliding_window": ((False,), "no sliding-window attention"),
    "qk_interleaved": ((False,), "rotary halves are contiguous, not interleaved"),
    "apply_post_layer_norm": ((False,), "pre-norm decoder"),
    "mlp_layer_fusion": ((False, True), "gate / up projections are always one fused matrix"),
    "rope_scaling_factor": ((1.0, 1), "no rotary scaling"),
    "multiple_of": ((1, 128, 256), "FFN width comes from mlp_ratio / the checkpoint"),
    "pure_llm": ((False,), "the multimodal model is always built"),
    "mot_model": ((True,), "Mixture-of-Transformers decoder (understanding + generation weights)"),
    "moe_location": (("llm",), "experts live in the decoder FFN"),
    "ps_version": (("v2",), "pixel-unshuffle layout v2"),
    "vision_select_layer": ((-1,), "the vision front-end has no encoder layers to select from"),
    "image_fold": ((None,), "no image folding"),
    "num_chunks": ((1,), "the vocabulary head is chunked by rows, not by this key"),
    "embed_split_hidden": ((True, False), "the embedding is sharded by the weight-parallel store"),
    "parallel_output": ((True, False), "the loss is fused with the head"),
    "use_cache": ((False,), "training never keeps a KV cache"),
    "embed_grad_scale": ((1, 1.0), "no embedding gradient scaling"),
    "unfreeze_vit_layers": ((0,), "the vision front-end has no encoder layers"),
}
_MODEL_NO_EFFECT = {
    "extra_num_layers": "num_layers already counts them; the split only matters when layers are initialised from a "
                        "shorter base LLM checkpoint",
    "extra_num_layers_post": "num_layers already counts them",
    "use_flash_attn": "attention is this package's tcgen05 kernel",
    "attention_type": "one attention module (MoT, packed mixed mask)",
    "attention_selective_checkpoint": "activation policy is full / attention / none (engine.recompute)",
    "vision_path": "weights come from model_name_or_path / the checkpoint folder",
    "mlp_path": "weights come from model_name_or_path / the checkpoint folder",
    "freeze_mlp": "freeze policy: train/freeze.py switches",
    "train_buffer": "no trainable buffers",
    "unfreeze_post_buffer": "no trainable buffers",
    "mot_random_init": "generation branch initialised from the understanding branch or at random by train/checkpoint.py",
}
_MOE_FIXED = {
    "moe_type": (("QwenDropless", "GShard"), "dropless top-k (engine) or capacity gating (models/gshard.py)"),
    "num_shared_experts": ((0,), "no shared experts"),
    "moe_layer_freq": ((1,), "every layer is a MoE layer"),
    "param_jitter_epsilon": ((0.0, 0), "no router jitter"),
    "first_k_dense_replace": ((0,), "no leading dense layers"),
}
_MOE_LAYER_FIXED = {
    "capacity_factor": ((None,), "dropless routing"),
    "normalize_expert_weights": ((True, False), "norm_topk_prob"),
    "scoring_func": (("softmax",), "softmax router"),
    "routed_scaling_factor": ((1.0, 1), "no routed scaling"),
}
_VIT_FIXED = {
    "num_hidden_layers": ((0,), "encoder-free vision front-end (patch embed + merge only)"),
    "use_moe": ((False,), "no experts in the vision front-end"),
    "drop_path_rate": ((0.0, 0), "no stochastic depth"),
    "dropout": ((0.0, 0), "no dropout"),
}
_LR_SCALE_UNIT = ("vit_layer_decay_rate", "moe_layer_decay_rate", "vit_woinit_layer_decay_rate")
_RUNTIME_ONLY = {
    "ckpt": ("async_upload", "async_upload_tmp_folder", "resume_ds"),
    "hybrid_zero_optimizer": ("reduce_bucket_size", "overlap_sync_grad", "overlap_sync_param"),
    "parallel": ("memory_pool",),
    "monitor": ("alert", "enable_feishu_alert", "feishu_alert_address", "light_monitor_address", "alert_file_path",
                "queue_max_length", "interval_step"),
    "tensorboard": ("queue_max_length",),
    "averaged_model": ("use_buffers",),
}


def _check_table(section: str, d: Mapping, table: Mapping[str, Tuple[tuple, str]], errors: List[str]) -> None:
    for k, (ok, what) in table.items():
        if k in d and d[k] not in ok:
            errors.append(f"{section}.{k}={d[k]!r} is not supported ({what}; accepted: {', '.join(map(repr, ok))})")


def check_sections(cfg: Mapping) -> List[str]:
    """Raises ``ValueError`` listing every unsupported setting; returns notes on keys accepted without effect."""
    errors: List[str] = []
    notes: List[str] = []
    model = dict(cfg.get("model") or {})
    _check_table("model", model, _MODEL_FIXED, errors)
    for k, why in _MODEL_NO_EFFECT.items():
        if k in model:
            notes.append(f"model.{k}: no effect ({why})")
    _check_table("model.moe_kwargs", dict(model.get("moe_kwargs") or {}), _MOE_FIXED, errors)
    _check_table("model.moe_layer_kwargs", dict(model.get("moe_layer_kwargs") or {}), _MOE_LAYER_FIXED, errors)
    _check_table("model.vit_cfg", dict(model.get("vit_cfg") or {}), _VIT_FIXED, errors)
    ls = dict(cfg.get("lr_scale") or {})
    for k in _LR_SCALE_UNIT:
        if float(ls.get(k, 1.0)) != 1.0:
            errors.append(f"lr_scale.{k}={ls[k]!r}: layer-wise learning-rate decay is not implemented (accepted: 1.0)")
    if float(ls.get("moe_coeff_lr_scale", 1.0)) != 1.0:
        errors.append("lr_scale.moe_coeff_lr_scale: there is no residual-expert coefficient to scale (accepted: 1.0)")
    loss = dict(cfg.get("loss") or {})
    if float(loss.get("label_smoothing", 0) or 0) != 0:
        errors.append("loss.label_smoothing: the fused cross-entropy kernel has no label smoothing (accepted: 0)")
    if float(loss.get("expert_coef_balance_coef", 0) or 0) != 0:
        errors.append("loss.expert_coef_balance_coef: no residual-expert coefficient loss (accepted: 0)")
    gs = dict(cfg.get("grad_scaler") or {})
    dtype = str(model.get("dtype", "torch.bfloat16"))
    if dtype.endswith("float16") and "bfloat16" not in dtype:
        errors.append("model.dtype=float16 needs dynamic loss scaling, which is not implemented (bf16 training needs none)")
    elif gs:
        notes.append("grad_scaler: no effect (bf16 training uses a constant loss scale of 1)")
    adam = dict(cfg.get("adam") or {})
    if float(adam.get("adam_beta2_c", 0) or 0) != 0:
        notes.append("adam.adam_beta2_c: the beta2 schedule is beta2_scheduler.c")
    avg = dict(cfg.get("averaged_model") or {})
    if avg.get("enable") and avg.get("multi_avg_fn", "ema") != "ema":
        errors.append(f"averaged_model.multi_avg_fn={avg.get('multi_avg_fn')!r}: only 'ema' is implemented")
    ck = dict(cfg.get("ckpt") or {})
    info = dict(ck.get("load_ckpt_info") or {})
    if info.get("ckpt_type") not in (None, "internevo", "sensenovalm", "hf"):
        errors.append(f"ckpt.load_ckpt_info.ckpt_type={info.get('ckpt_type')!r}: 'internevo' (training shards) or 'hf'")
    for section, keys in _RUNTIME_ONLY.items():
        present = [k for k in keys if k in dict(cfg.get(section) or {})]
        if present:
            notes.append(f"{section}.{{{', '.join(present)}}}: no counterpart (the reference's own runtime plumbing)")
    if errors:
        raise ValueError("unsupported config settings:\n  " + "\n  ".join(errors))
    return notes
