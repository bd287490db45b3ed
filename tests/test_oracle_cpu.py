"""CPU checks of the PyTorch oracle: mask rule, rotary conventions, losses, packing."""
import math

import torch

from sensenova_u1_b200.config import tiny_mot
from sensenova_u1_b200.data import batch as B
from sensenova_u1_b200.data.synthetic import synthetic_batch, tiny_batch
from sensenova_u1_b200.models import oracle
from sensenova_u1_b200.models.params import ParamStore, hf_state_dict, load_hf_state_dict
from sensenova_u1_b200.ops.attention import dense_mask, make_meta


def _store(cfg, seed=0):
    st = ParamStore(cfg, dtype=torch.float32, with_grads=True)
    st.init_weights(seed)
    return st


def test_mask_rule_text_causal_image_bidirectional():
    # doc 0: 3 text tokens, an und image of 4 tokens sharing one position, 2 text tokens
    doc = torch.zeros(9, dtype=torch.int32)
    pos = torch.tensor([0, 1, 2, 3, 3, 3, 3, 4, 5])
    img = torch.tensor([0, 0, 0, 7, 7, 7, 7, 0, 0])
    m = dense_mask(make_meta(doc, pos, img), make_meta(doc, pos, img))
    assert m[1, 0] and not m[0, 1]                 # causal text
    assert m[3, 6] and m[6, 3]                     # image tokens see each other
    assert not m[2, 3]                             # text before the image does not see it
    assert m[7, 4]                                 # later text sees the image


def test_mask_generation_gating():
    doc = torch.zeros(8, dtype=torch.int32)
    #      txt txt | gen image (2 tok) | clean copy (2 tok, same pos) | txt txt
    pos = torch.tensor([0, 1, 2, 2, 2, 2, 3, 4])
    img = torch.tensor([0, 0, 5, 5, 6, 6, 0, 0])
    gen = torch.tensor([0, 0, 1, 1, 0, 0, 0, 0]).bool()
    meta = make_meta(doc, pos, img, gen)
    m = dense_mask(meta, meta)
    assert m[2, 3] and m[3, 2]                      # generation tokens of one image see each other
    assert m[2, 0] and m[2, 1]                      # and the text prefix
    assert not m[6, 2] and not m[7, 3]              # nobody else sees generation keys
    assert not m[2, 4] and not m[3, 5]              # generation queries skip the clean copy at their own position
    assert m[6, 4] and m[7, 5]                      # later text reads the clean copy
    blocked = torch.tensor([0, 1, 0, 0, 0, 0, 0, 0]).bool()
    m2 = dense_mask(make_meta(doc, pos, img, gen, blocked), make_meta(doc, pos, img, gen, blocked))
    assert not m2[:, 1].any()


def test_documents_do_not_mix():
    doc = torch.tensor([0, 0, 1, 1], dtype=torch.int32)
    pos = torch.tensor([0, 1, 0, 1])
    m = dense_mask(make_meta(doc, pos), make_meta(doc, pos))
    assert not m[2, 0] and not m[3, 1] and m[3, 2]


def test_rope_frequency_rule():
    cfg = tiny_mot(head_dim=128)
    inv_t, inv_hw = oracle.rope_inv_freq(cfg, "cpu")
    assert inv_t.numel() == 32 and inv_hw.numel() == 16
    # "keep frequency range": rotary of twice the width, every other entry
    full_t = 1.0 / (cfg.rope_base ** (torch.arange(0, 128, 2).float() / 128))
    assert torch.allclose(inv_t, full_t[::2])
    full_hw = 1.0 / (cfg.rope_base_hw ** (torch.arange(0, 64, 2).float() / 64))
    assert torch.allclose(inv_hw, full_hw[::2])


def test_rope3d_is_rotation_and_position_zero_identity():
    cfg = tiny_mot(head_dim=128)
    x = torch.randn(5, 2, 128)
    pos0 = torch.zeros(3, 5, dtype=torch.int32)
    assert torch.allclose(oracle.rope3d(x, pos0, cfg), x, atol=1e-6)
    pos = torch.randint(0, 50, (3, 5), dtype=torch.int32)
    y = oracle.rope3d(x, pos, cfg)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)
    # only the h block moves when only h changes
    pos_h = pos0.clone(); pos_h[1] = 3
    yh = oracle.rope3d(x, pos_h, cfg)
    assert torch.allclose(yh[..., :64], x[..., :64]) and torch.allclose(yh[..., 96:], x[..., 96:])
    assert not torch.allclose(yh[..., 64:96], x[..., 64:96])


def test_patch_token_layout_roundtrip():
    px = torch.rand(3, 64, 96)
    p16, gx, gy, th, tw = B.patchify_block_major(px, 16, 2)
    assert p16.shape == (th * tw * 4, 768) and (th, tw) == (2, 3)
    tok = B.patches_to_tokens(p16, 16, 2)
    # token (ty, tx) holds the 32x32 pixel block in (row, col, channel) order
    blk = px[:, 32:64, 32:64].permute(1, 2, 0).reshape(-1)
    assert torch.equal(tok[1 * tw + 1], blk)
    assert torch.equal(B.tokens_to_patches(tok, 16, 2), p16)
    # grid coordinates of the 4 patches of token (1, 2)
    i = (1 * tw + 2) * 4
    assert gy[i:i + 4].tolist() == [2, 2, 3, 3] and gx[i:i + 4].tolist() == [4, 5, 4, 5]


def test_packed_layout_invariants():
    cfg = tiny_mot()
    b = synthetic_batch(cfg.replace(patch_size=16), 2048, seed=3, image_sizes=(64, 128), max_images=2)
    assert b.S == 2048 and b.S % 128 == 0 and b.n_gen_pad % 128 == 0
    kinds = b.kind
    assert (kinds[: b.n_gen_pad] != B.KIND_TEXT).all()             # generation partition first
    assert ((kinds[b.n_gen_pad:] != B.KIND_GEN_IMG)).all()
    assert (b.tile_group[: b.n_gen_pad // 128] == 1).all()
    assert b.labels[b.label_rows].min() >= 0
    assert abs(b.loss_w[b.label_rows].sum().item() - b.ce_weight_sum) < 1e-3
    pad = kinds == B.KIND_PAD
    assert ((b.meta[pad, 3] & B.FLAG_BLOCKED) != 0).all()
    # labels are the next token of the same document
    assert b.n_label > 0 and b.n_tokens <= b.S


def test_time_schedule_and_noise_scale():
    cfg = tiny_mot()
    t = torch.linspace(0, 1, 5)
    out = B.apply_time_schedule(t, 64, cfg, timestep_shift=3.0)
    sigma = 1 - t
    assert torch.allclose(out, 1 - 3 * sigma / (1 + 2 * sigma))
    assert B.noise_scale_for(cfg, 256) == min(math.sqrt(256 / 64) * cfg.noise_scale, cfg.noise_scale_max_value)


def test_training_loss_backward_is_finite_and_decreases():
    cfg = tiny_mot()
    st = _store(cfg)
    b = tiny_batch(cfg, with_und_image=True)
    noise = torch.randn(b.gen_x16.shape, generator=torch.Generator().manual_seed(1))
    p = {k: v.clone().requires_grad_(True) for k, v in st.p.items()}
    loss, parts = oracle.training_loss(p, b, cfg, noise)
    loss.backward()
    assert torch.isfinite(loss) and set(parts) == {"ce", "fm"}
    assert abs(parts["ce"].item() - math.log(cfg.vocab_size)) < 0.5     # random init ~ uniform
    with torch.no_grad():
        for v in p.values():
            if v.grad is not None:
                v -= 0.5 * v.grad
    loss2, _ = oracle.training_loss({k: v.detach() for k, v in p.items()}, b, cfg, noise)
    assert loss2 < loss


def test_moe_oracle_runs():
    cfg = tiny_mot(num_experts=8, num_experts_per_tok=2, gen_num_experts=4, gen_num_experts_per_tok=2,
                   moe_intermediate_size=64, router_aux_loss_coef=0.01)
    st = _store(cfg)
    b = tiny_batch(cfg)
    noise = torch.randn(b.gen_x16.shape, generator=torch.Generator().manual_seed(1))
    p = {k: v.clone().requires_grad_(True) for k, v in st.p.items()}
    loss, parts = oracle.training_loss(p, b, cfg, noise)
    loss.backward()
    assert "moe_aux" in parts and torch.isfinite(loss)
    assert p["layers.0.moe_und.gate"].grad.abs().sum() > 0


def test_hf_state_dict_roundtrip_and_param_count():
    from sensenova_u1_b200.config import neo_8b_mot
    assert neo_8b_mot().num_params() == 17_552_340_992
    cfg = tiny_mot()
    a, b = _store(cfg, 1), _store(cfg, 2)
    sd = {k: v.clone() for k, v in hf_state_dict(a).items()}
    assert "language_model.model.layers.0.self_attn.q_proj_mot_gen.weight" in sd
    assert "fm_modules.vision_model_mot_gen.embeddings.dense_embedding.weight" in sd
    assert sd["vision_model.embeddings.dense_embedding.weight"].shape == (cfg.hidden_size, cfg.vision_hidden, 2, 2)
    load_hf_state_dict(b, sd)
    for k in a.p:
        assert torch.equal(a.p[k], b.p[k]), k


def test_mtp_heads_shift_and_train():
    """Multi-token prediction: lookahead rows stay inside one run of text, the extra loss is
    finite, depends on the MTP parameters only through its own term, and gets gradients."""
    import torch
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.synthetic import tiny_batch
    from sensenova_u1_b200.models import oracle
    from sensenova_u1_b200.models.params import ParamStore
    cfg = tiny_mot(num_mtp_layers=2)
    store = ParamStore(cfg, device="cpu", dtype=torch.float32)
    store.init_weights(0, std=0.05)
    assert "mtp.1.layer.wqkv" in store.p and [b[0] for b in store.buckets("mat")][-1] == "head"
    batch = tiny_batch(cfg, seed=1, n_text=96, image_px=64, with_und_image=True)
    ok, tgt = oracle.mtp_shift(batch, 2)
    doc, pos = batch.meta[:, 0], batch.meta[:, 1]
    assert ok.any()
    assert bool(((doc[tgt[ok]] == doc[ok]) & (pos[tgt[ok]] == pos[ok] + 2) & (batch.kind[tgt[ok]] == 1)).all())
    p = {k: v.detach().clone().requires_grad_(True) for k, v in store.p.items()}
    g = torch.Generator().manual_seed(0)
    noise = torch.randn(batch.gen_x16.shape, generator=g)
    loss, parts = oracle.training_loss(p, batch, cfg, noise)
    assert torch.isfinite(loss) and parts["mtp"] > 0
    loss.backward()
    assert p["mtp.0.proj"].grad.abs().sum() > 0 and p["mtp.1.layer.wo"].grad.abs().sum() > 0
    base, _ = oracle.training_loss(p, batch, tiny_mot(), noise)
    want = base + cfg.mtp_loss_coeff * cfg.ce_loss_weight * parts["mtp"]
    assert abs(float(loss) - float(want)) < 1e-5


def test_capacity_gating_drops_in_choice_major_order():
    import torch
    from sensenova_u1_b200.models.gshard import capacity_moe_ffn, capacity_topk_gating, dense_dispatch
    torch.manual_seed(0)
    S, E, k = 16, 4, 2
    logits = torch.randn(S, E)
    logits[:, 0] += 4.0                                   # everybody's first choice is expert 0
    r = capacity_topk_gating(logits, k, capacity_factor=1.0, min_capacity=1)
    assert r.capacity == 8
    first0 = (r.expert[:, 0] == 0)
    assert bool(first0.all())
    assert r.keep[:8, 0].all() and not r.keep[8:, 0].any()       # rows 0..7 fill expert 0, the rest are dropped
    assert torch.equal(r.slot[:8, 0], torch.arange(8))
    kept = r.keep.float().sum(1)
    w = r.weight.sum(1)
    assert torch.allclose(w[kept > 0], torch.ones(int((kept > 0).sum())), atol=1e-6)   # survivors renormalised
    comb, mask = dense_dispatch(r, E)
    assert comb.shape == (S, E, 8) and int(mask.sum()) == int(r.keep.sum())
    assert int(mask.sum(dim=(0,)).max()) <= 1                     # one token copy per (expert, slot)
    assert torch.allclose(comb.sum(dim=(1, 2)), w, atol=1e-6)
    # with ample capacity nothing is dropped and the layer equals the dropless mixture
    from sensenova_u1_b200.models import oracle
    H, Fd = 8, 16
    x = torch.randn(S, H)
    gate_w, w13, w2 = torch.randn(E, H), torch.randn(E, 2 * Fd, H) * 0.2, torch.randn(E, H, Fd) * 0.2
    y, aux = capacity_moe_ffn(x, gate_w, w13, w2, k, capacity_factor=8.0)
    y_ref, _ = oracle.moe_ffn(x, gate_w, w13, w2, k, True)
    assert torch.allclose(y, y_ref, atol=1e-4) and aux > 0


def test_pixel_head_layout_and_training():
    """Convolutional pixel decoder: output pixel blocks are in (row, col, channel) order per token,
    images of different grids are decoded independently, and the flow-matching loss trains it."""
    import torch
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.synthetic import tiny_batch
    from sensenova_u1_b200.models import oracle
    from sensenova_u1_b200.models.params import ParamStore, hf_state_dict
    cfg = tiny_mot(use_pixel_head=True, pixel_head_dim=32)
    store = ParamStore(cfg, device="cpu", dtype=torch.float32)
    store.init_weights(0, std=0.05)
    assert "fm_head.conv1_w" in store.p and "fm_head.w1" not in store.p
    assert "fm_modules.fm_head.conv2.weight" in hf_state_dict(store)
    tp = cfg.token_pixels
    h = torch.randn(2 * 3 + 1 * 2, cfg.hidden_size)
    y = oracle.pixel_head(store.p, h, [(2, 3), (1, 2)], cfg)
    assert y.shape == (8, cfg.token_dim)
    # reference: decode image 0 as a picture, then cut token (1, 2)'s block out of it
    x = h[:6].view(1, 2, 3, -1).permute(0, 3, 1, 2)
    F = torch.nn.functional
    x = F.gelu(F.conv2d(F.pixel_shuffle(x, 2), store.p["fm_head.conv1_w"], store.p["fm_head.conv1_b"], padding=1))
    img = F.pixel_shuffle(F.conv2d(F.pixel_shuffle(x, 2), store.p["fm_head.conv2_w"], store.p["fm_head.conv2_b"], padding=1), tp // 4)[0]
    block = img[:, tp:2 * tp, 2 * tp:3 * tp].permute(1, 2, 0).reshape(-1)
    assert torch.allclose(y[1 * 3 + 2], block, atol=1e-6)
    # the second image does not see the first one
    y2 = oracle.pixel_head(store.p, h[6:], [(1, 2)], cfg)
    assert torch.allclose(y[6:], y2, atol=1e-6)
    batch = tiny_batch(cfg, seed=2, n_text=64, image_px=4 * tp)
    assert oracle.gen_image_grids(batch) == [(4, 4)]
    p = {k: v.detach().clone().requires_grad_(True) for k, v in store.p.items()}
    noise = torch.randn(batch.gen_x16.shape, generator=torch.Generator().manual_seed(0))
    loss, parts = oracle.training_loss(p, batch, cfg, noise)
    loss.backward()
    assert torch.isfinite(loss) and parts["fm"] > 0 and p["fm_head.conv1_w"].grad.abs().sum() > 0


def test_balance_loss_weights_of_the_two_mixtures():
    """``moe_balance_gen_ratio`` / ``moe_balance_und_ratio`` weigh the two mixtures' balance losses in their sum."""
    import torch
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.synthetic import tiny_batch
    from sensenova_u1_b200.models import oracle
    from sensenova_u1_b200.models.params import ParamStore
    base = dict(num_layers=1, num_experts=4, num_experts_per_tok=2, gen_num_experts=4, gen_num_experts_per_tok=2,
                moe_intermediate_size=64)
    aux = {}
    for g, u in ((1.0, 1.0), (1.0, 0.0), (0.0, 1.0), (2.0, 3.0)):
        cfg = tiny_mot(**base, moe_balance_gen_ratio=g, moe_balance_und_ratio=u)
        st = ParamStore(cfg, dtype=torch.float32, grad_dtype_mat=torch.float32)
        st.init_weights(0)
        b = tiny_batch(cfg, seed=1, n_text=64)
        noise = torch.randn(b.gen_x16.shape, generator=torch.Generator().manual_seed(0))
        _, parts = oracle.training_loss(st.p, b, cfg, noise)
        aux[(g, u)] = float(parts["moe_aux"])
    gen, und = aux[(1.0, 0.0)], aux[(0.0, 1.0)]
    assert gen > 0 and und > 0 and abs(aux[(1.0, 1.0)] - (gen + und)) < 1e-5
    assert abs(aux[(2.0, 3.0)] - (2 * gen + 3 * und)) < 1e-5
