#!/bin/bash
# SenseNova-U1.5 8B-MoT generation pre-training with the convolutional pixel head on one node of B200s
# (language model and understanding front-end frozen, generation branch and generation modules train).  Every knob is an environment
# variable read by the config module (same names as the reference launcher,
# training/shell/train_u1/U1.5_8B.sh:1-119); override them before calling this script.
set -e
cd "$(dirname "$0")/../.."  # repo root

export NPROC_PER_NODE=${NPROC_PER_NODE:-8}
export NNODES=${NNODES:-1}
export NODE_RANK=${NODE_RANK:-0}
export MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
export MASTER_PORT=${MASTER_PORT:-29500}
export CONFIG_NAME=${CONFIG_NAME:-"configs/sensenovavl_qwen3_gen/sensenovau1_5_8b_mot_pt.py"}

# model / tokenizer / data
export MODEL_NAME_OR_PATH=${MODEL_NAME_OR_PATH:-"/path/to/SenseNova-U1-8B-MoT"}
export TOKENIZER_PATH=${TOKENIZER_PATH:-"/path/to/qwen3/tokenizer"}
export mm_data_path=${mm_data_path:-"data/sample/sample_data_meta.json"}
export load_optimizer=${load_optimizer:-"model"}

# parallelism: 180 GB parts hold weights + gradients + 1/N optimizer state, so the default is data
# parallel + ZeRO-1 over every rank (zero1_size=-1); cp_size > 1 splits one packed sequence over ranks
export zero1_size=${zero1_size:--1}
export tp_size=${tp_size:-1}
export pp_size=${pp_size:-1}
export cp_size=${cp_size:-1}
export zero_comm=${zero_comm:-peer}      # peer: NVLink peer-memory kernels, nccl: NCCL collectives
export activation_policy=${activation_policy:-auto}   # auto (by free memory), full, attention, none

# optimisation
export SEED=${SEED:-42}
export lr=${lr:-2e-4}
export lr_scheduler_type=${lr_scheduler_type:-constant}
export min_lr_ratio=${min_lr_ratio:-0.5}
export weight_decay=${weight_decay:-0}
export grad_accm=${grad_accm:-1}
export total_steps=${total_steps:-200000}
export init_steps=${init_steps:-2000}
export ema_decay=${ema_decay:-0.9999}

# data shape
export num_imgs=${num_imgs:-144}
export seq_len=${seq_len:-8192}
export max_sample_tokens=${max_sample_tokens:-8192}
export max_pixels=${max_pixels:-$((1024 * 1024))}
export min_pixels=${min_pixels:-$((256 * 256))}
export max_pixels_gen=${max_pixels_gen:-$((1024 * 1024))}
export min_pixels_gen=${min_pixels_gen:-$((256 * 256))}

# freeze policy
export mot_random_init=${mot_random_init:-true}
export freeze_llm=${freeze_llm:-true}
export freeze_backbone=${freeze_backbone:-true}
export use_pixel_head=${use_pixel_head:-true}
export unfreeze_mot_gen=${unfreeze_mot_gen:-true}

# flow matching
export time_schedule=${time_schedule:-standard}
export time_shift_type=${time_shift_type:-exponential}
export base_shift=${base_shift:-0.5}
export max_shift=${max_shift:-1.15}
export base_image_seq_len=${base_image_seq_len:-64}
export max_image_seq_len=${max_image_seq_len:-4096}
export noise_scale_mode=${noise_scale_mode:-resolution}
export noise_scale_base_image_seq_len=${noise_scale_base_image_seq_len:-64}
export add_noise_scale_embedding=${add_noise_scale_embedding:-true}
export noise_scale_max_value=${noise_scale_max_value:-16}
export P_mean=${P_mean:--0.8}
export P_std=${P_std:-0.8}
export cfg_txt_uncond_drop_prob=${cfg_txt_uncond_drop_prob:-0.1}
export cfg_img_uncond_drop_prob=${cfg_img_uncond_drop_prob:-0}
export cfg_txtimg_uncond_drop_prob=${cfg_txtimg_uncond_drop_prob:-0.1}
export cfg_is_uncond_drop_independent=${cfg_is_uncond_drop_independent:-false}

# understanding branch
export ce_loss_weight=${ce_loss_weight:-0}
export enable_und_loss=${enable_und_loss:-false}
export pad_dummy_image_gen=${pad_dummy_image_gen:-false}

export JOB_NAME=${JOB_NAME:-"sensenovau1_5_8b_pt"}
export PYTHONPATH="${PYTHONPATH}:$(pwd)"
export TORCH_SYMM_MEM_DISABLE_MULTICAST=${TORCH_SYMM_MEM_DISABLE_MULTICAST:-1}

python -m torch.distributed.run \
    --nproc-per-node=${NPROC_PER_NODE} \
    --nnodes=${NNODES} \
    --node-rank=${NODE_RANK} \
    --master-addr=${MASTER_ADDR} \
    --master-port=${MASTER_PORT} \
    train_sensenovau1.py \
        --config "${CONFIG_NAME}" \
        --launcher torch \
        --seed "${SEED}" \
        --backend nccl "$@"
