#!/bin/bash
# SenseNova-U1-8B-MoT full-parameter SFT on one node of B200s.  Every knob is an environment
# variable read by the config module (same names as the reference launcher,
# training/shell/train_u1/8B.sh:1-118); override them before calling this script.
set -e
cd "$(dirname "$0")/../.."  # repo root

export NPROC_PER_NODE=${NPROC_PER_NODE:-8}
export NNODES=${NNODES:-1}
export NODE_RANK=${NODE_RANK:-0}
export MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
export MASTER_PORT=${MASTER_PORT:-29500}
export CONFIG_NAME=${CONFIG_NAME:-"configs/sensenovavl_qwen3_gen/sensenovau1_8b_mot_sft.py"}

# model / tokenizer / data
export MODEL_NAME_OR_PATH=${MODEL_NAME_OR_PATH:-"/path/to/SenseNova-U1-8B-MoT-SFT"}
export TOKENIZER_PATH=${TOKENIZER_PATH:-"/path/to/qwen3/tokenizer"}
export mm_data_path=${mm_data_path:-"data/sample/sample_data_meta.json"}
export load_optimizer=${load_optimizer:-"model"}

# parallelism: the reference's shipped mode, ZeRO-1 + weight parallel over every rank (wp_size = world: each rank
# keeps 1/N of every weight, layers are gathered one ahead over NVLink peer memory).  wp_size=1 runs data parallel +
# ZeRO-1 with replicated weights (180 GB parts hold them); cp_size > 1 splits one packed sequence over ranks;
# tp_size x pp_size = world runs tensor x pipeline parallel
export zero1_size=${zero1_size:--1}
export tp_size=${tp_size:-1}
export pp_size=${pp_size:-1}
export cp_size=${cp_size:-1}
if [ "$((tp_size * pp_size * cp_size))" -gt 1 ]; then
  export wp_size=${wp_size:-1}                      # tensor / pipeline / context parallel: weights whole per rank
else
  export wp_size=${wp_size:-$((NPROC_PER_NODE * NNODES))}
fi
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
export seq_len=${seq_len:-28672}
export max_sample_tokens=${max_sample_tokens:-28672}
export max_pixels=${max_pixels:-$((2048 * 2048))}
export min_pixels=${min_pixels:-$((256 * 256))}
export max_pixels_gen=${max_pixels_gen:-$((512 * 512))}
export min_pixels_gen=${min_pixels_gen:-$((256 * 256))}

# freeze policy
export mot_random_init=${mot_random_init:-true}
export freeze_llm=${freeze_llm:-false}
export freeze_backbone=${freeze_backbone:-false}
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
export noise_scale_max_value=${noise_scale_max_value:-8}
export P_mean=${P_mean:--0.8}
export P_std=${P_std:-0.8}
export cfg_txt_uncond_drop_prob=${cfg_txt_uncond_drop_prob:-0.1}
export cfg_img_uncond_drop_prob=${cfg_img_uncond_drop_prob:-0}
export cfg_txtimg_uncond_drop_prob=${cfg_txtimg_uncond_drop_prob:-0.1}
export cfg_is_uncond_drop_independent=${cfg_is_uncond_drop_independent:-false}

# understanding branch
export ce_loss_weight=${ce_loss_weight:-0.1}
export enable_und_loss=${enable_und_loss:-true}
export pad_dummy_image_gen=${pad_dummy_image_gen:-true}

export JOB_NAME=${JOB_NAME:-"sensenovau1_8b_sft"}
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
