"""SenseNova-U1.5 8B-MoT generation pre-training: the 8B-MoT SFT configuration with the
convolutional pixel head (``use_pixel_head``) and the language model / understanding front-end
frozen by default, so that only the generation branch and the generation modules train (reference:
training/configs/sensenovavl_qwen3_gen/sensenovau1_5_8b_mot_pt.py:104-130, :323-326).

The pixel head runs on the sm_100a engine (``models/engine.py::_pixel_head_fwd``: pixel shuffle and 3x3 patch
gather in ``csrc/pixel_head.cu``, the convolutions as tcgen05 GEMMs); ``use_pixel_head=false`` selects the MLP
head instead."""
import os
import runpy
from types import SimpleNamespace

from sensenova_u1_b200.train.config import env_bool

# the base file is found beside this one (a package import of ``configs`` could pick up another tree on sys.path)
_base_ns = runpy.run_path(os.path.join(os.path.dirname(__file__), "sensenovau1_8b_mot_sft.py"))
globals().update({k: v for k, v in _base_ns.items() if not k.startswith("_")})
_base = SimpleNamespace(**_base_ns)

E = os.environ.get
JOB_NAME = E("JOB_NAME", "sensenovau1_5_8b_mot_pt")
freeze_llm, freeze_backbone = env_bool("freeze_llm", True), env_bool("freeze_backbone", True)
unfreeze_mot_gen, unfreeze_lm_head = env_bool("unfreeze_mot_gen", True), env_bool("unfreeze_lm_head", False)
use_pixel_head = env_bool("use_pixel_head", True)
ce_loss_weight = float(E("ce_loss_weight", 0.0))

ckpt = dict(_base.ckpt, save_ckpt_folder=f"local:RUN/{JOB_NAME}")
model = dict(_base.model, use_pixel_head=use_pixel_head, pixel_head_dim=int(E("pixel_head_dim", 1024)),
             freeze_llm=freeze_llm, freeze_backbone=freeze_backbone, unfreeze_mot_gen=unfreeze_mot_gen,
             unfreeze_lm_head=unfreeze_lm_head)
