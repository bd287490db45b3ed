"""Parameter inventory, flat storage arenas and checkpoint name mapping.

Every weight of the model lives in one of two flat device buffers ("arenas"):
``mat`` (matrices; bf16 weights and bf16 gradient accumulators) and ``vec``
(gains and biases; bf16 weights, fp32 gradient accumulators).  Parameters are
views into them.  A flat layout makes ZeRO-1 a contiguous range per rank, lets
reduce-scatter / all-gather run on the buffer itself, and lets the optimizer
kernels sweep long ranges (the reference flattens per rank at every step:
training/sensenovalm/solver/optimizer/hybrid_zero_optim.py:363-404, 626-690).

MoT twins are stacked on a leading axis of size 2: index 0 is the understanding
branch, index 1 the generation branch (``*_mot_gen`` in HF checkpoints:
src/sensenova_u1/models/neo_unify/modeling_qwen3.py:380-429, training
tools/key_mappings.json).  q/k/v and gate/up projections are stored fused.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterator, List, Tuple

import torch

from ..config import ModelConfig

UND, GEN = 0, 1
ALIGN = 128  # elements; keeps every tensor 256-byte aligned inside an arena


@dataclass
class ParamSpec:
    name: str
    shape: Tuple[int, ...]
    arena: str            # "mat" | "vec" | "exp" (expert weights held by this rank only)
    init: str             # "normal" | "ones" | "zeros" | "out_normal"
    role: str             # lr-scale / weight-decay group: llm, vit, fm_modules, embed, norm, bias
    decay: bool = True

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


def build_specs(cfg: ModelConfig) -> List[ParamSpec]:
    H, D = cfg.hidden_size, cfg.head_dim
    qkv = cfg.q_dim + 2 * cfg.kv_dim
    F = cfg.ffn_size
    sp: List[ParamSpec] = []
    add = sp.append
    add(ParamSpec("embed_tokens", (cfg.vocab_size, H), "mat", "normal", "embed"))
    Cv = cfg.vision_hidden
    for br in ("und", "gen"):
        p = f"vision_{br}."
        add(ParamSpec(p + "patch_w", (Cv, cfg.patch_dim), "mat", "normal", "vit"))
        add(ParamSpec(p + "patch_b", (Cv,), "vec", "zeros", "vit", False))
        add(ParamSpec(p + "merge_w", (H, cfg.merge_size ** 2 * Cv), "mat", "normal", "vit"))
        add(ParamSpec(p + "merge_b", (H,), "vec", "zeros", "vit", False))
    embedders = ["timestep_embedder"] + (["noise_scale_embedder"] if cfg.add_noise_scale_embedding else [])
    for e in embedders:
        add(ParamSpec(f"{e}.w1", (H, cfg.timestep_freq_dim), "mat", "normal", "fm_modules"))
        add(ParamSpec(f"{e}.b1", (H,), "vec", "zeros", "fm_modules", False))
        add(ParamSpec(f"{e}.w2", (H, H), "mat", "normal", "fm_modules"))
        add(ParamSpec(f"{e}.b2", (H,), "vec", "zeros", "fm_modules", False))
    def add_layer(p):
        add(ParamSpec(p + "attn_norm", (2, H), "vec", "ones", "norm", False))
        add(ParamSpec(p + "wqkv", (2, qkv, H), "mat", "normal", "llm"))
        add(ParamSpec(p + "qk_norm", (2, 4, D // 2), "vec", "ones", "norm", False))
        add(ParamSpec(p + "wo", (2, H, cfg.q_dim), "mat", "out_normal", "llm"))
        add(ParamSpec(p + "ffn_norm", (2, H), "vec", "ones", "norm", False))
        if not cfg.is_moe:
            add(ParamSpec(p + "w13", (2, 2 * F, H), "mat", "normal", "llm"))
            add(ParamSpec(p + "w2", (2, H, F), "mat", "out_normal", "llm"))
        else:
            Fe = cfg.moe_intermediate_size
            ep = max(1, cfg.ep_size)
            ea = "exp" if ep > 1 else "mat"
            for br, ne in (("und", cfg.num_experts), ("gen", cfg.gen_num_experts)):
                if ne % ep:
                    raise ValueError(f"{ne} experts do not split over ep_size={ep}")
                add(ParamSpec(p + f"moe_{br}.gate", (ne, H), "mat", "normal", "moe_gate"))
                add(ParamSpec(p + f"moe_{br}.w13", (ne // ep, 2 * Fe, H), ea, "normal", "moe_expert"))
                add(ParamSpec(p + f"moe_{br}.w2", (ne // ep, H, Fe), ea, "out_normal", "moe_expert"))

    for l in range(cfg.num_layers):
        add_layer(f"layers.{l}.")
    add(ParamSpec("final_norm", (2, H), "vec", "ones", "norm", False))
    add(ParamSpec("lm_head", (cfg.vocab_size, H), "mat", "normal", "embed"))
    if cfg.use_pixel_head:
        # convolutional pixel decoder (training/sensenovavl/model/modules/fm_modules.py:44-61)
        if H % 4 or cfg.pixel_head_dim % 4 or cfg.token_pixels % 4:
            raise ValueError("the pixel head needs hidden size, pixel_head_dim and token size divisible by 4")
        r3 = cfg.token_pixels // 4
        add(ParamSpec("fm_head.conv1_w", (cfg.pixel_head_dim, H // 4, 3, 3), "mat", "normal", "fm_modules"))
        add(ParamSpec("fm_head.conv1_b", (cfg.pixel_head_dim,), "vec", "zeros", "fm_modules", False))
        add(ParamSpec("fm_head.conv2_w", (3 * r3 * r3, cfg.pixel_head_dim // 4, 3, 3), "mat", "normal", "fm_modules"))
        add(ParamSpec("fm_head.conv2_b", (3 * r3 * r3,), "vec", "zeros", "fm_modules", False))
    else:
        add(ParamSpec("fm_head.w1", (cfg.fm_head_dim, H), "mat", "normal", "fm_modules"))
        add(ParamSpec("fm_head.b1", (cfg.fm_head_dim,), "vec", "zeros", "fm_modules", False))
        add(ParamSpec("fm_head.w2", (cfg.token_dim, cfg.fm_head_dim), "mat", "normal", "fm_modules"))
        add(ParamSpec("fm_head.b2", (cfg.token_dim,), "vec", "zeros", "fm_modules", False))
    for k in range(cfg.num_mtp_layers):
        # multi-token-prediction head k: two norms, a 2H -> H projection and one decoder layer
        # (training/sensenovalm/model/mtp.py:11-55); embedding, final norm and LM head are shared.
        # They sit after the heads so that their gradients join the "head" communication bucket.
        add(ParamSpec(f"mtp.{k}.norm_hidden", (H,), "vec", "ones", "norm", False))
        add(ParamSpec(f"mtp.{k}.norm_embed", (H,), "vec", "ones", "norm", False))
        add(ParamSpec(f"mtp.{k}.proj", (H, 2 * H), "mat", "normal", "llm"))
        add_layer(f"mtp.{k}.layer.")
    return sp


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class ParamStore:
    """Owns the arenas and hands out named views.

    ``with_grads`` allocates gradient accumulators (``mat``: bf16, ``vec``: fp32).
    Arena sizes are padded to a multiple of ``shard_multiple`` elements so that
    they split evenly over data-parallel ranks.  With expert parallelism (``cfg.ep_size > 1``)
    the expert weights sit in a third arena, ``exp``, that holds this rank's experts only
    (experts ``ep_rank * E / ep_size ...``): it is neither reduced nor gathered across ranks.
    """

    def __init__(self, cfg: ModelConfig, device="cpu", dtype=torch.bfloat16, with_grads=True,
                 shard_multiple: int = 8 * ALIGN, grad_dtype_mat=None, symmetric_group=None,
                 ep_rank: int = 0):
        self.cfg = cfg
        self.ep_rank = ep_rank
        self.specs = build_specs(cfg)
        self.device = torch.device(device)
        self.dtype = dtype
        self.offsets: Dict[str, Tuple[str, int]] = {}
        sizes = {"mat": 0, "vec": 0}
        if any(s.arena == "exp" for s in self.specs):
            sizes["exp"] = 0
        for s in self.specs:
            self.offsets[s.name] = (s.arena, sizes[s.arena])
            sizes[s.arena] += _round_up(s.numel, ALIGN)
        self.sizes = {k: _round_up(max(v, ALIGN), shard_multiple) for k, v in sizes.items()}
        # symmetric_group: allocate the arenas in NVLink peer-mapped (symmetric) memory of that
        # process group right away (``True`` = the default group), for the peer-memory collectives
        self.symm = None
        if symmetric_group is not None:
            from ..parallel.symm import SymmetricBuffer
            grp = None if symmetric_group is True else symmetric_group
            self.symm = {"arena": {}, "grad": {}}

            def alloc(kind, name, n, dt):
                if name == "exp":       # rank-local, no peer ever reads it
                    return torch.zeros(n, dtype=dt, device=self.device)
                sb = SymmetricBuffer(n, dt, self.device, grp)
                self.symm[kind][name] = sb
                return sb.tensor
        else:
            def alloc(kind, name, n, dt):
                return torch.zeros(n, dtype=dt, device=self.device)
        self.arena = {k: alloc("arena", k, n, dtype) for k, n in self.sizes.items()}
        self.grad_arena = None
        if with_grads:
            gm = grad_dtype_mat or dtype
            self.grad_arena = {"mat": alloc("grad", "mat", self.sizes["mat"], gm),
                               "vec": alloc("grad", "vec", self.sizes["vec"], torch.float32)}
            if "exp" in self.sizes:
                self.grad_arena["exp"] = alloc("grad", "exp", self.sizes["exp"], gm)
        self.by_name = {s.name: s for s in self.specs}
        self.p: Dict[str, torch.Tensor] = {}
        self.g: Dict[str, torch.Tensor] = {}
        self.rebind_views()

    def rebind_views(self) -> None:
        """(Re)creates the named views after an arena was replaced (e.g. moved to symmetric memory)."""
        for s in self.specs:
            a, off = self.offsets[s.name]
            self.p[s.name] = self.arena[a][off:off + s.numel].view(s.shape)
            if self.grad_arena is not None:
                self.g[s.name] = self.grad_arena[a][off:off + s.numel].view(s.shape)

    # -- initialisation -----------------------------------------------------
    def init_weights(self, seed: int = 0, std: float = 0.02) -> None:
        """Random init, streamed tensor by tensor (never a full fp32 copy)."""
        g = torch.Generator(device=self.device).manual_seed(seed)
        ge = torch.Generator(device=self.device).manual_seed(seed + 7919 * (self.ep_rank + 1))
        L = max(1, self.cfg.num_layers)
        for s in self.specs:
            t = self.p[s.name]
            if s.arena == "exp":        # every rank's experts are different weights
                sd = std / (2 * L) ** 0.5 if s.init == "out_normal" else std
                t.view(-1).copy_((torch.randn(t.numel(), device=self.device, generator=ge) * sd).to(self.dtype))
                continue
            if s.init == "ones":
                t.fill_(1.0)
            elif s.init == "zeros":
                t.zero_()
            else:
                sd = std / (2 * L) ** 0.5 if s.init == "out_normal" else std
                flat = t.view(-1)
                step = 1 << 26
                for i in range(0, flat.numel(), step):
                    n = min(step, flat.numel() - i)
                    flat[i:i + n] = (torch.randn(n, device=self.device, generator=g) * sd).to(self.dtype)

    def zero_grads(self, keep_layer_matrices: bool = False) -> None:
        """Clears the gradient arenas.  ``keep_layer_matrices``: the decoder layers' matrices are left as they are,
        for a caller whose first micro-batch *stores* those gradients instead of adding to them (saves clearing and
        re-reading two bytes per parameter and step)."""
        for a, t in self.grad_arena.items():
            if a == "mat" and keep_layer_matrices:
                for key, lo, hi in self.buckets("mat"):
                    if not key.startswith("layer."):
                        t[lo:hi].zero_()
            else:
                t.zero_()

    def named_parameters(self) -> Iterator[Tuple[str, torch.Tensor]]:
        for s in self.specs:
            yield s.name, self.p[s.name]

    def segments(self, arena: str) -> List[Tuple[int, int, ParamSpec]]:
        """(start, end, spec) of every tensor in ``arena`` (padding excluded)."""
        out = []
        for s in self.specs:
            a, off = self.offsets[s.name]
            if a == arena:
                out.append((off, off + s.numel, s))
        return out

    def buckets(self, arena: str) -> List[Tuple[str, int, int]]:
        """Gradient-communication buckets (name, start, end) that tile the whole arena in
        order: ``front`` (token embedding, pixel front-ends, scalar embedders: complete at the
        very end of backward), one per decoder layer, and ``head`` (lm head, generation head:
        complete first).  The small ``vec`` arena is a single bucket."""
        if arena in ("vec", "exp"):
            return [(arena, 0, self.sizes[arena])]
        marks = []
        for s in self.specs:
            a, off = self.offsets[s.name]
            if a != "mat":
                continue
            if s.name.startswith("layers."):
                key = "layer." + s.name.split(".")[1]
            elif s.name in ("lm_head",) or s.name.startswith("fm_head.") or s.name.startswith("mtp."):
                key = "head"
            else:
                key = "front"
            if not marks or marks[-1][0] != key:
                marks.append([key, off])
        out = []
        for i, (key, off) in enumerate(marks):
            end = marks[i + 1][1] if i + 1 < len(marks) else self.sizes["mat"]
            out.append((key, off, end))
        return out

    def copy_from(self, other: "ParamStore") -> None:
        for k in self.arena:
            self.arena[k].copy_(other.arena[k].to(self.dtype))


# ---------------------------------------------------------------------------
# HF checkpoint names (inference layout, src/sensenova_u1 and tools/revert2hf.py)
# ---------------------------------------------------------------------------
def hf_state_dict(store: ParamStore) -> Dict[str, torch.Tensor]:
    """Splits the fused / stacked tensors into the per-module HF tensors."""
    cfg, p = store.cfg, store.p
    out: Dict[str, torch.Tensor] = {}
    sfx = {UND: "", GEN: "_mot_gen"}
    lm = "language_model.model."
    out[lm + "embed_tokens.weight"] = p["embed_tokens"]
    out["language_model.lm_head.weight"] = p["lm_head"]
    for b in (UND, GEN):
        out[lm + f"norm{sfx[b]}.weight"] = p["final_norm"][b]
    qd, kd = cfg.q_dim, cfg.kv_dim
    for l in range(cfg.num_layers):
        s, d = f"layers.{l}.", lm + f"layers.{l}."
        for b in (UND, GEN):
            x = sfx[b]
            w = p[s + "wqkv"][b]
            out[d + f"self_attn.q_proj{x}.weight"] = w[:qd]
            out[d + f"self_attn.k_proj{x}.weight"] = w[qd:qd + kd]
            out[d + f"self_attn.v_proj{x}.weight"] = w[qd + kd:]
            out[d + f"self_attn.o_proj{x}.weight"] = p[s + "wo"][b]
            n = p[s + "qk_norm"][b]
            out[d + f"self_attn.q_norm{x}.weight"] = n[0]
            out[d + f"self_attn.q_norm_hw{x}.weight"] = n[1]
            out[d + f"self_attn.k_norm{x}.weight"] = n[2]
            out[d + f"self_attn.k_norm_hw{x}.weight"] = n[3]
            out[d + f"input_layernorm{x}.weight"] = p[s + "attn_norm"][b]
            out[d + f"post_attention_layernorm{x}.weight"] = p[s + "ffn_norm"][b]
            if not cfg.is_moe:
                F = cfg.ffn_size
                out[d + f"mlp{x}.gate_proj.weight"] = p[s + "w13"][b][:F]
                out[d + f"mlp{x}.up_proj.weight"] = p[s + "w13"][b][F:]
                out[d + f"mlp{x}.down_proj.weight"] = p[s + "w2"][b]
            else:
                br = "und" if b == UND else "gen"
                Fe = cfg.moe_intermediate_size
                out[d + f"mlp{x}.gate.weight"] = p[s + f"moe_{br}.gate"]
                w13, w2 = p[s + f"moe_{br}.w13"], p[s + f"moe_{br}.w2"]
                e0 = store.ep_rank * w13.shape[0] if cfg.ep_size > 1 else 0   # global expert index
                for e in range(w13.shape[0]):
                    out[d + f"mlp{x}.experts.{e0 + e}.gate_proj.weight"] = w13[e][:Fe]
                    out[d + f"mlp{x}.experts.{e0 + e}.up_proj.weight"] = w13[e][Fe:]
                    out[d + f"mlp{x}.experts.{e0 + e}.down_proj.weight"] = w2[e]
    Cv, ps, ms = cfg.vision_hidden, cfg.patch_size, cfg.merge_size
    for br, pre in (("und", "vision_model."), ("gen", "fm_modules.vision_model_mot_gen.")):
        e = pre + "embeddings."
        out[e + "patch_embedding.weight"] = p[f"vision_{br}.patch_w"].view(Cv, 3, ps, ps)
        out[e + "patch_embedding.bias"] = p[f"vision_{br}.patch_b"]
        # stored [H, kh, kw, Cv] (K-major for the merge GEMM); conv layout is [H, Cv, kh, kw]
        out[e + "dense_embedding.weight"] = (
            p[f"vision_{br}.merge_w"].view(-1, ms, ms, Cv).permute(0, 3, 1, 2))
        out[e + "dense_embedding.bias"] = p[f"vision_{br}.merge_b"]
    for emb in ("timestep_embedder", "noise_scale_embedder"):
        if emb + ".w1" in p:
            out[f"fm_modules.{emb}.mlp.0.weight"] = p[emb + ".w1"]
            out[f"fm_modules.{emb}.mlp.0.bias"] = p[emb + ".b1"]
            out[f"fm_modules.{emb}.mlp.2.weight"] = p[emb + ".w2"]
            out[f"fm_modules.{emb}.mlp.2.bias"] = p[emb + ".b2"]
    if cfg.use_pixel_head:
        out["fm_modules.fm_head.conv1.weight"] = p["fm_head.conv1_w"]
        out["fm_modules.fm_head.conv1.bias"] = p["fm_head.conv1_b"]
        out["fm_modules.fm_head.conv2.weight"] = p["fm_head.conv2_w"]
        out["fm_modules.fm_head.conv2.bias"] = p["fm_head.conv2_b"]
    else:
        out["fm_modules.fm_head.0.weight"] = p["fm_head.w1"]
        out["fm_modules.fm_head.0.bias"] = p["fm_head.b1"]
        out["fm_modules.fm_head.2.weight"] = p["fm_head.w2"]
        out["fm_modules.fm_head.2.bias"] = p["fm_head.b2"]
    return out


def load_hf_state_dict(store: ParamStore, sd: Dict[str, torch.Tensor], strict: bool = True) -> List[str]:
    """Copies HF-named tensors into the arenas; returns the names it did not find."""
    missing = []
    for name, view in hf_state_dict(store).items():
        if name in sd:
            view.copy_(sd[name].to(view.dtype).reshape(view.shape) if view.is_contiguous()
                       else sd[name].to(view.dtype))
        else:
            missing.append(name)
    if strict and missing:
        raise KeyError(f"{len(missing)} tensors missing from checkpoint, e.g. {missing[:4]}")
    return missing
