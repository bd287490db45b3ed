"""SenseNova-U1-8B-MoT full-parameter SFT.  Same keys and environment knobs as the reference
config of the same name (training/configs/sensenovavl_qwen3_gen/sensenovau1_8b_mot_sft.py);
every knob has a default here so that the file also evaluates outside a launcher script."""
import os

from sensenova_u1_b200.train.config import env_bool

E = os.environ.get
JOB_NAME = E("JOB_NAME", "sensenovau1_8b_sft")
MODEL_NAME_OR_PATH = E("MODEL_NAME_OR_PATH")          # HF checkpoint directory or None (random init)
TOKENIZER_PATH = E("TOKENIZER_PATH") or E("VOCAB_FILE")   # the reference's launcher names it VOCAB_FILE
MODEL_ONLY_FOLDER = E("MODEL_ONLY_FOLDER")
mm_data_path = E("mm_data_path")                       # meta json; None => synthetic packed data

zero1_size, wp_size = int(E("zero1_size", -1)), int(E("wp_size", 1))
tp_size, pp_size = int(E("tp_size", 1)), int(E("pp_size", 1))
lr, weight_decay = float(E("lr", 2e-4)), float(E("weight_decay", 0))
grad_accm, total_steps, init_steps = int(E("grad_accm", 1)), int(E("total_steps", 200000)), int(E("init_steps", 2000))
min_lr_ratio = float(E("min_lr_ratio", 0.5))
mlp_lr_scale = float(E("mlp_lr_scale", 1.0))
fm_modules_lr_scale = float(E("fm_modules_lr_scale", 1.0))
mot_gen_lr_scale = float(E("mot_gen_lr_scale", 1.0))
lr_scheduler_type = E("lr_scheduler_type", "constant")
lr_scheduler_offset = int(E("lr_scheduler_offset", 0))
load_optimizer = E("load_optimizer", "model")
ce_loss_weight = float(E("ce_loss_weight", 0.1))
SEQ_LEN = int(E("seq_len", 28672))
num_imgs = int(E("num_imgs", 144))
max_pixels, min_pixels = int(E("max_pixels", 2048 * 2048)), int(E("min_pixels", 256 * 256))
max_pixels_gen, min_pixels_gen = int(E("max_pixels_gen", 512 * 512)), int(E("min_pixels_gen", 256 * 256))
down_sample_ratio = float(E("down_sample_ratio", 0.5))
dataset_replacement = env_bool("dataset_replacement", True)
thinking_method = E("thinking_method", "tag")
pad_dummy_image_gen = env_bool("pad_dummy_image_gen", True)
ema_decay = float(E("ema_decay", 0.9999))
auto_resume, resume_ds = env_bool("auto_resume", False), env_bool("resume_ds", False)
freeze_llm, freeze_backbone = env_bool("freeze_llm", False), env_bool("freeze_backbone", False)
unfreeze_mot_gen, mot_random_init = env_bool("unfreeze_mot_gen", True), env_bool("mot_random_init", True)

VOCAB_SIZE, HIDDEN_SIZE, HEAD_DIM = 151936, 4096, 128
NUM_ATTENTION_HEAD, NUM_KV_ATTENTION_HEAD = 32, 8
MLP_RATIO = 12288 / 4096
NUM_LAYER = 36 + 6 + int(E("post_layer_num", 0))
model_type = "QWEN3_MoEMoT"

ckpt = dict(enable_save_ckpt=True, save_ckpt_folder=f"local:RUN/{JOB_NAME}", load_ckpt_folder=MODEL_ONLY_FOLDER,
            load_ckpt_info=dict(path=MODEL_ONLY_FOLDER, content=(load_optimizer,), ckpt_type="internevo"),
            auto_resume=auto_resume, resume_ds=resume_ds, checkpoint_every=100, oss_snapshot_freq=1000,
            async_upload=True, async_upload_tmp_folder="/dev/shm/sensenovalm_tmp_ckpt/")

data = dict(type="multimodal_streaming", use_packed_ds=True, seq_len=SEQ_LEN, micro_num=grad_accm, micro_bsz=1,
            total_steps=total_steps, num_workers=8, meta_path=mm_data_path, tokenizer_path=TOKENIZER_PATH,
            patch_size=16, down_sample_ratio=down_sample_ratio, max_pixels=max_pixels, min_pixels=min_pixels,
            max_pixels_gen=max_pixels_gen, min_pixels_gen=min_pixels_gen, num_images_expected=num_imgs,
            max_packed_tokens=SEQ_LEN, max_buffer_size=10, replacement=dataset_replacement,
            loss_reduction="square", loss_reduction_all_gather=True, empty_cache_and_diag_interval=200,
            cfg_txt_uncond_drop_prob=float(E("cfg_txt_uncond_drop_prob", 0.1)),
            cfg_img_uncond_drop_prob=float(E("cfg_img_uncond_drop_prob", 0)),
            cfg_txtimg_uncond_drop_prob=float(E("cfg_txtimg_uncond_drop_prob", 0.1)),
            # launcher knobs of the reference's 8B.sh: chat template, dataset mixing by kind, batch-size ramp-up
            conv_style=E("CONV_STYLE", "sensenovalm2-chat-v3"), llm_data_weights=float(E("LLM_DATA_WEIGHTS", 0)),
            mm_cc_data_weights=float(E("MM_CC_DATA_WEIGHTS", 0)), rampup_batch_size=E("rampup_batch_size") or None,
            min_length=int(E("min_length", 0)), total_epochs=int(E("total_epochs", -1)),
            dynamic_image_size=True, dynamic_image_version="native_resolution")
if E("time_base_dist", "logit_normal") != "logit_normal":
    raise ValueError("time_base_dist: denoising times are drawn logit-normal (P_mean, P_std); no other base distribution")

model = dict(head_dim=HEAD_DIM, num_attention_heads=NUM_ATTENTION_HEAD, num_kv_attention_heads=NUM_KV_ATTENTION_HEAD,
             hidden_size=HIDDEN_SIZE, mlp_ratio=MLP_RATIO, vocab_size=VOCAB_SIZE, num_layers=NUM_LAYER,
             max_position_embeddings=262144, norm_type="rmsnorm", layer_norm_epsilon=1e-6, qkv_bias=False,
             rope_base=5000000.0, parallel_output=True, checkpoint=1, use_flash_attn=True, dtype="torch.bfloat16",
             model_name_or_path=MODEL_NAME_OR_PATH, freeze_llm=freeze_llm, freeze_backbone=freeze_backbone,
             unfreeze_mot_gen=unfreeze_mot_gen, mot_random_init=mot_random_init,
             P_mean=float(E("P_mean", -0.8)), P_std=float(E("P_std", 0.8)), time_schedule=E("time_schedule", "standard"),
             time_shift_type=E("time_shift_type", "exponential"), base_shift=float(E("base_shift", 0.5)),
             max_shift=float(E("max_shift", 1.15)), base_image_seq_len=int(E("base_image_seq_len", 64)),
             max_image_seq_len=int(E("max_image_seq_len", 4096)), noise_scale_mode=E("noise_scale_mode", "resolution"),
             noise_scale=float(E("noise_scale", 1)), noise_scale_base_image_seq_len=int(E("noise_scale_base_image_seq_len", 64)),
             noise_scale_max_value=float(E("noise_scale_max_value", 8)),
             add_noise_scale_embedding=env_bool("add_noise_scale_embedding", True), t_eps=0.05)

averaged_model = dict(enable=ema_decay > 0, decay=ema_decay, multi_avg_fn="ema", use_buffers=False)
adam = dict(lr=lr, adam_beta1=0.9, adam_beta2=0.95, adam_eps=1e-08, adam_beta2_c=0, weight_decay=weight_decay)
lr_scale = dict(mlp_lr_scale=mlp_lr_scale, mot_gen_lr_scale=mot_gen_lr_scale, fm_modules_lr_scale=fm_modules_lr_scale,
                moe_wg_lr_scale=1.0)
lr_scheduler = dict(total_steps=total_steps, init_steps=init_steps, warmup_ratio=0.0, last_epoch=-1, eta_min=min_lr_ratio)
beta2_scheduler = dict(init_beta2=adam["adam_beta2"], c=adam["adam_beta2_c"], cur_iter=-1)
grad_scaler = dict(fp16=dict(initial_scale=1, min_scale=1, growth_interval=1000), growth_factor=1, backoff_factor=1,
                   max_scale=1, hysteresis=2)
hybrid_zero_optimizer = dict(overlap_sync_grad=True, overlap_sync_param=False, reduce_bucket_size=256 * 1024 * 1024,
                             clip_grad_norm=1.0)
loss = dict(label_smoothing=0, image_gen_loss_coef=1.0)
parallel = dict(zero1=dict(size=zero1_size), tensor=dict(size=tp_size, mode="isp"), pipeline=dict(size=pp_size),
                weight=dict(size=wp_size, overlap=True, launch_allgather_before="wo", forward_overlap_per="layer"))
monitor = dict(alert=dict(enable_feishu_alert=False))
cudnn_deterministic, cudnn_benchmark = False, False
