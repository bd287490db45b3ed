"""Model configurations of the NEO-unify Mixture-of-Transformers family.

Field values of the presets come from the reference configs:
8B-MoT  training/configs/sensenovavl_qwen3_gen/sensenovau1_8b_mot_sft.py:161-173, 283-316
A3B-MoT training/configs/sensenovavl_qwen3_gen/sensenovau1_a3b_mot_sft.py:163-201, 363-382
vision  src/sensenova_u1/models/neo_unify/configuration_neo_vit.py
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field


@dataclass
class ModelConfig:
    name: str = "tiny-mot"
    vocab_size: int = 1024
    hidden_size: int = 256
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 128
    ffn_size: int = 1024
    num_layers: int = 2
    rms_eps: float = 1e-6
    rope_base: float = 5_000_000.0
    rope_base_hw: float = 10_000.0
    max_position_embeddings: int = 262144
    # vision front-end (patch 16, 2x2 merge => one token per 32x32 pixels)
    patch_size: int = 16
    merge_size: int = 2
    vision_hidden: int = 1024
    rope_theta_vision: float = 10_000.0
    # generation head: MLP (H -> fm_head_dim -> token_dim) or, with use_pixel_head, the convolutional
    # decoder (pixel-shuffle 2, conv3x3, GELU, pixel-shuffle 2, conv3x3, pixel-shuffle token_pixels/4)
    use_pixel_head: bool = False
    pixel_head_dim: int = 1024
    fm_head_dim: int = 4096
    timestep_freq_dim: int = 256
    add_noise_scale_embedding: bool = True
    noise_scale: float = 1.0
    noise_scale_mode: str = "resolution"
    noise_scale_base_image_seq_len: int = 64
    noise_scale_max_value: float = 8.0
    t_eps: float = 0.05
    P_mean: float = -0.8
    P_std: float = 0.8
    time_schedule: str = "standard"
    time_shift_type: str = "exponential"
    timestep_shift: float = 1.0
    base_shift: float = 0.5
    max_shift: float = 1.15
    base_image_seq_len: int = 64
    max_image_seq_len: int = 4096
    # MoE (0 experts => dense FFN)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    gen_num_experts: int = 0
    gen_num_experts_per_tok: int = 0
    # expert parallelism: every rank holds num_experts / ep_size experts of each mixture (1 = replicated)
    ep_size: int = 1
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    router_aux_loss_coef: float = 0.0
    # understanding branch: the balance loss is taken over image tokens and text tokens separately and mixed with
    # these ratios (both 0: one loss over all tokens); router z-loss coefficient; step of the bias-based
    # ("aux-free") balancing of the selection scores (0 = off)
    moe_balance_image_ratio: float = 0.0
    moe_balance_text_ratio: float = 0.0
    # weights of the generation / understanding mixtures' balance losses in their sum (the reference's loose config
    # globals of the same names, modeling_qwen3_moe_mot.py:695-708)
    moe_balance_gen_ratio: float = 1.0
    moe_balance_und_ratio: float = 1.0
    router_z_loss_coef: float = 0.0
    router_bias_update_rate: float = 0.0
    # multi-token prediction heads (0 = off): head k predicts the token k + 2 positions ahead
    num_mtp_layers: int = 0
    mtp_loss_coeff: float = 0.3
    # losses
    ce_loss_weight: float = 0.1
    image_gen_loss_weight: float = 1.0

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def token_pixels(self) -> int:
        return self.patch_size * self.merge_size

    @property
    def patch_dim(self) -> int:
        return 3 * self.patch_size * self.patch_size

    @property
    def token_dim(self) -> int:
        return 3 * self.token_pixels * self.token_pixels

    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    def replace(self, **kw) -> "ModelConfig":
        return dataclasses.replace(self, **kw)

    def num_params(self) -> int:
        """Parameters of the whole model (every expert of every rank under expert parallelism)."""
        from .models.params import build_specs
        ep = max(1, self.ep_size)
        return sum(s.numel * (ep if s.arena == "exp" else 1) for s in build_specs(self))


def tiny_mot(**kw) -> ModelConfig:
    """2 layers, hidden 256, 4 heads of 64, FFN 1024, vocab 1024: the CPU / gloo test
    model.  The CUDA kernels need head_dim 128 (as every released model has), so GPU
    tests pass ``head_dim=128``."""
    base = ModelConfig(name="tiny-mot", vocab_size=1024, hidden_size=256, num_heads=4, num_kv_heads=2,
                       head_dim=64, ffn_size=1024, num_layers=2, vision_hidden=64, fm_head_dim=128,
                       patch_size=8, merge_size=2)
    return base.replace(**kw)


def neo_8b_mot(**kw) -> ModelConfig:
    base = ModelConfig(name="SenseNova-U1-8B-MoT", vocab_size=151936, hidden_size=4096, num_heads=32,
                       num_kv_heads=8, head_dim=128, ffn_size=12288, num_layers=42,
                       rope_base=5_000_000.0, vision_hidden=1024, fm_head_dim=4096)
    return base.replace(**kw)


def neo_a3b_mot(**kw) -> ModelConfig:
    base = ModelConfig(name="SenseNova-U1-A3B-MoT", vocab_size=151936, hidden_size=2048, num_heads=32,
                       num_kv_heads=4, head_dim=128, ffn_size=6144, num_layers=48,
                       rope_base=10_000_000.0, num_experts=128, num_experts_per_tok=8,
                       gen_num_experts=32, gen_num_experts_per_tok=8, moe_intermediate_size=768,
                       router_aux_loss_coef=0.001)
    return base.replace(**kw)


PRESETS = {"tiny-mot": tiny_mot, "8b-mot": neo_8b_mot, "a3b-mot": neo_a3b_mot}


def get_config(name: str, **kw) -> ModelConfig:
    try:
        return PRESETS[name.lower()](**kw)
    except KeyError as e:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)}") from e
