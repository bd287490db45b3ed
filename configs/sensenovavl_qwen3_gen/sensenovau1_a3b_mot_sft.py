"""SenseNova-U1-A3B-MoT (MoE) SFT: 48 layers, hidden 2048, 128 understanding / 32 generation
experts, top-8, expert FFN 768 (reference: training/configs/sensenovavl_qwen3_gen/sensenovau1_a3b_mot_sft.py)."""
import os
import runpy

_base = runpy.run_path(os.path.join(os.path.dirname(__file__), "sensenovau1_8b_mot_sft.py"))
globals().update({k: v for k, v in _base.items() if not k.startswith("_")})
E = os.environ.get
JOB_NAME = E("JOB_NAME", "sensenovau1_a3b_sft")
HIDDEN_SIZE, NUM_KV_ATTENTION_HEAD, NUM_LAYER = 2048, 4, 48
model = dict(model, hidden_size=HIDDEN_SIZE, num_kv_attention_heads=NUM_KV_ATTENTION_HEAD, num_layers=NUM_LAYER,
             mlp_ratio=3.0, rope_base=10000000.0,
             moe_kwargs=dict(num_experts=128, top_k=8, gen_num_experts=32, gen_top_k=8, moe_intermediate_size=768,
                             moe_type="QwenDropless", num_shared_experts=0, normalize_expert_weights=True,
                             first_k_dense_replace=0))
loss = dict(loss, expert_balance_coef=float(E("expert_balance_coef", 0.001)))
parallel = dict(parallel, expert=dict(size=int(E("ep_size", 8))), expert_weight=dict(size=int(E("ewp_size", 1))))
ckpt = dict(ckpt, save_ckpt_folder=f"local:RUN/{JOB_NAME}")
