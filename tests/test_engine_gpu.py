"""CUDA engine (explicit forward/backward on sm_100a kernels) against the PyTorch oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(with_und=True, layers=2, seed=0, **cfg_kw):
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.synthetic import tiny_batch
    from sensenova_u1_b200.models.params import ParamStore
    cfg = tiny_mot(head_dim=128, num_heads=4, num_kv_heads=2, hidden_size=256, num_layers=layers,
                   patch_size=16, merge_size=2, vision_hidden=64, fm_head_dim=128, **cfg_kw)
    store = ParamStore(cfg, device="cuda", dtype=torch.bfloat16)
    store.init_weights(seed, std=0.05)
    # make gains / biases non-trivial so their gradients are exercised
    g = torch.Generator(device="cuda").manual_seed(seed + 1)
    for sp in store.specs:
        if sp.arena == "vec":
            t = store.p[sp.name]
            t.add_((torch.randn(t.shape, device="cuda", generator=g) * 0.1).to(t.dtype))
    batch = tiny_batch(cfg, seed=seed, n_text=200, image_px=8 * 32, with_und_image=with_und).to("cuda")
    noise = torch.randn(batch.gen_x16.shape, device="cuda", generator=g)
    return cfg, store, batch, noise


def _oracle(cfg, store, batch, noise):
    from sensenova_u1_b200.models import oracle
    p = {k: v.detach().float().clone().requires_grad_(True) for k, v in store.p.items()}
    loss, parts = oracle.training_loss(p, batch, cfg, noise)
    loss.backward()
    return loss, parts, {k: v.grad for k, v in p.items()}


def _note(test: str, name: str, err: float) -> None:
    """With SNU1_TEST_ERRLOG=<file> the worst relative error of every comparison is appended there (one JSON line
    per entry), to set the bounds from measurements."""
    import json
    import os
    path = os.environ.get("SNU1_TEST_ERRLOG")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"test": test, "name": name, "err": err}) + "\n")


def test_forward_backward_matches_oracle():
    from sensenova_u1_b200.models.engine import MoTEngine
    from sensenova_u1_b200.ops import _lib
    cfg, store, batch, noise = _setup()
    eng = MoTEngine(cfg, store)
    store.zero_grads()
    out = eng.forward_backward(batch, noise)
    _lib.check_status()
    loss_ref, parts_ref, grads_ref = _oracle(cfg, store, batch, noise)
    assert abs(out["ce"].item() - parts_ref["ce"].item()) < 3e-2 * abs(parts_ref["ce"].item())
    assert abs(out["fm"].item() - parts_ref["fm"].item()) < 3e-2 * abs(parts_ref["fm"].item())
    bad = []
    for name, gref in grads_ref.items():
        if gref is None:
            continue
        got = store.g[name].float()
        den = gref.norm().item()
        err = (got - gref).norm().item() / (den + 1e-8)
        if den > 1e-6:
            _note("dense", name, err)
        if den > 1e-6 and err > 0.025:        # measured worst: 1.1 % (bf16 activations through two layers)
            bad.append((name, err, den))
    assert not bad, bad


def test_convolutional_pixel_head_matches_oracle():
    """The ConvDecoder head (pixel-shuffle + 3x3 convolutions as patch gather + tcgen05 GEMM) in the CUDA engine:
    loss and every gradient against the PyTorch oracle, whose head is ``F.pixel_shuffle`` / ``F.conv2d``."""
    from sensenova_u1_b200.models.engine import MoTEngine
    from sensenova_u1_b200.ops import _lib
    cfg, store, batch, noise = _setup(use_pixel_head=True, pixel_head_dim=256)
    eng = MoTEngine(cfg, store)
    store.zero_grads()
    out = eng.forward_backward(batch, noise)
    _lib.check_status()
    loss_ref, parts_ref, grads_ref = _oracle(cfg, store, batch, noise)
    assert abs(out["fm"].item() - parts_ref["fm"].item()) < 3e-2 * abs(parts_ref["fm"].item())
    assert abs(out["ce"].item() - parts_ref["ce"].item()) < 3e-2 * abs(parts_ref["ce"].item())
    bad = []
    for name, gref in grads_ref.items():
        if gref is None:
            continue
        got = store.g[name].float()
        den = gref.norm().item()
        err = (got - gref).norm().item() / (den + 1e-8)
        if den > 1e-6 and err > 0.08:
            bad.append((name, round(err, 3), den))
    assert not bad, bad
    for name in ("fm_head.conv1_w", "fm_head.conv2_w", "fm_head.conv1_b", "fm_head.conv2_b"):
        assert grads_ref[name].norm().item() > 0


@pytest.mark.parametrize("mode", ["full", "none"])
def test_mtp_heads_match_oracle(mode):
    """Two multi-token-prediction heads on top of the decoder: loss and every gradient (heads, shared LM head /
    final norm / embedding, and the decoder below) against the PyTorch model."""
    from sensenova_u1_b200.models.engine import MoTEngine
    from sensenova_u1_b200.ops import _lib
    cfg, store, batch, noise = _setup(num_mtp_layers=2, mtp_loss_coeff=0.5)
    eng = MoTEngine(cfg, store)
    eng.recompute = mode
    store.zero_grads()
    out = eng.forward_backward(batch, noise)
    _lib.check_status()
    loss_ref, parts_ref, grads_ref = _oracle(cfg, store, batch, noise)
    assert parts_ref["mtp"].item() > 0
    assert abs(out["mtp"].item() - parts_ref["mtp"].item()) < 3e-2 * abs(parts_ref["mtp"].item())
    assert abs(out["loss"].item() - loss_ref.item()) < 3e-2 * abs(loss_ref.item())
    bad = []
    for name, gref in grads_ref.items():
        if gref is None:
            continue
        got = store.g[name].float()
        den = gref.norm().item()
        err = (got - gref).norm().item() / (den + 1e-8)
        if den > 1e-6 and err > 0.08:
            bad.append((name, round(err, 3), den))
    assert not bad, bad
    assert any(n.startswith("mtp.1.") for n in grads_ref)


def test_gradient_accumulation_and_determinism():
    from sensenova_u1_b200.models.engine import MoTEngine
    cfg, store, batch, noise = _setup(layers=1)
    eng = MoTEngine(cfg, store)
    store.zero_grads()
    eng.forward_backward(batch, noise)
    g1 = {k: v.clone() for k, v in store.grad_arena.items()}
    store.zero_grads()
    eng.forward_backward(batch, noise)
    # big matrices come from deterministic tensor-core reductions
    assert torch.equal(store.grad_arena["mat"][: store.offsets["final_norm"][1] if False else 1024],
                       g1["mat"][:1024])
    eng.forward_backward(batch, noise)
    w = store.g["layers.0.w13"].float()
    ref = 2 * torch.stack([g1["mat"][store.offsets["layers.0.w13"][1]:][: w.numel()].view(w.shape).float()])[0]
    assert ((w - ref).norm() / ref.norm()).item() < 2e-2


def test_moe_engine_matches_oracle():
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.synthetic import tiny_batch
    from sensenova_u1_b200.models.engine_moe import MoEMoTEngine
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.ops import _lib
    cfg = tiny_mot(head_dim=128, patch_size=16, num_layers=2, num_experts=8, num_experts_per_tok=2,
                   gen_num_experts=8, gen_num_experts_per_tok=2, moe_intermediate_size=128,
                   router_aux_loss_coef=0.01)
    store = ParamStore(cfg, device="cuda")
    store.init_weights(0, std=0.05)
    batch = tiny_batch(cfg, seed=0, n_text=200, image_px=8 * 32, with_und_image=True).to("cuda")
    g = torch.Generator(device="cuda").manual_seed(5)
    noise = torch.randn(batch.gen_x16.shape, device="cuda", generator=g)
    eng = MoEMoTEngine(cfg, store)
    store.zero_grads()
    out = eng.forward_backward(batch, noise)
    _lib.check_status()
    loss_ref, parts_ref, grads_ref = _oracle(cfg, store, batch, noise)
    assert abs(out["ce"].item() - parts_ref["ce"].item()) < 3e-2 * abs(parts_ref["ce"].item())
    assert abs(out["fm"].item() - parts_ref["fm"].item()) < 3e-2 * abs(parts_ref["fm"].item())
    assert abs(out["moe_aux"].item() - parts_ref["moe_aux"].item()) < 3e-2 * abs(parts_ref["moe_aux"].item())
    bad = []
    for name, gref in grads_ref.items():
        if gref is None:
            continue
        got = store.g[name].float()
        den = gref.norm().item()
        err = (got - gref).norm().item() / (den + 1e-8)
        # a token whose k-th and (k+1)-th gate probabilities are within bf16 noise may route
        # differently; expert tensors get a wider band
        # measured worst: router gates 12 %, expert matrices 5.7 %, everything else 5 %
        tol = 0.2 if name.endswith(".gate") else (0.1 if "moe_" in name else 0.08)
        if den > 1e-6:
            _note("moe", name, err)
        if den > 1e-6 and err > tol:
            bad.append((name, round(err, 3), den))
    assert not bad, bad


def test_moe_training_extras_match_oracle():
    """Class-weighted balance loss (text / image tokens of the understanding branch), router z-loss and the bias of
    bias-based balancing: loss terms and gate gradients against the PyTorch oracle; the bias moves against the load."""
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.synthetic import tiny_batch
    from sensenova_u1_b200.models.engine_moe import MoEMoTEngine
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.ops import _lib
    cfg = tiny_mot(head_dim=128, patch_size=16, num_layers=2, num_experts=8, num_experts_per_tok=2,
                   gen_num_experts=8, gen_num_experts_per_tok=2, moe_intermediate_size=128,
                   router_aux_loss_coef=0.05, moe_balance_image_ratio=0.3, moe_balance_text_ratio=0.7,
                   router_z_loss_coef=0.01)
    store = ParamStore(cfg, device="cuda")
    store.init_weights(0, std=0.05)
    batch = tiny_batch(cfg, seed=0, n_text=200, image_px=8 * 32, with_und_image=True).to("cuda")
    g = torch.Generator(device="cuda").manual_seed(5)
    noise = torch.randn(batch.gen_x16.shape, device="cuda", generator=g)
    eng = MoEMoTEngine(cfg, store)
    store.zero_grads()
    out = eng.forward_backward(batch, noise)
    _lib.check_status()
    loss_ref, parts_ref, grads_ref = _oracle(cfg, store, batch, noise)
    for k in ("moe_aux", "moe_z_loss"):
        assert abs(out[k].item() - parts_ref[k].item()) < 3e-2 * abs(parts_ref[k].item()), (k, out[k].item(), parts_ref[k].item())
    assert abs(out["loss"].item() - loss_ref.item()) < 3e-2 * abs(loss_ref.item())
    for name in ("layers.0.moe_und.gate", "layers.1.moe_und.gate", "layers.1.moe_gen.gate"):
        got, gref = store.g[name].float(), grads_ref[name]
        err = (got - gref).norm().item() / (gref.norm().item() + 1e-8)
        assert err < 0.25, (name, err)
    # bias-based balancing: overloaded experts get a lower selection bias, starved ones a higher one
    cfg2 = cfg.replace(router_bias_update_rate=1e-2)
    eng2 = MoEMoTEngine(cfg2, store)
    store.zero_grads()
    eng2.forward_backward(batch, noise)
    _lib.check_status()
    assert eng2.sel_bias[(0, "und")].abs().max().item() == 0        # moves at the end of the step, not per micro-batch
    eng2.update_selection_bias()
    assert eng2.sel_counts[(0, "und")].abs().max().item() == 0
    saved = eng2.selection_bias_state()
    eng3 = MoEMoTEngine(cfg2, store)
    eng3.load_selection_bias_state(saved)
    assert torch.equal(eng3.sel_bias[(1, "gen")], eng2.sel_bias[(1, "gen")])
    b = eng2.sel_bias[(0, "und")]
    assert b.abs().max().item() > 0 and abs(b.sum().item()) <= 8 * 1e-2 * 2
    for v in torch.unique(b.abs()).tolist():          # one signed step of the update rate per expert
        assert min(abs(v - m * 1e-2) for m in (0, 1)) < 1e-6, v


@pytest.mark.parametrize("mode", ["attention", "none"])
def test_activation_policies_give_the_same_gradients(mode):
    from sensenova_u1_b200.models.engine import MoTEngine
    cfg, store, batch, noise = _setup()
    eng = MoTEngine(cfg, store)
    eng.recompute = "full"
    store.zero_grads()
    ref_out = eng.forward_backward(batch, noise)
    ref = {k: v.clone() for k, v in store.grad_arena.items()}
    eng2 = MoTEngine(cfg, store)
    eng2.recompute = mode
    store.zero_grads()
    out = eng2.forward_backward(batch, noise)
    # same kernels on the same data; the loss and the gain gradients are summed with fp32 atomics
    assert torch.allclose(out["loss"], ref_out["loss"], rtol=1e-5)
    dm = (store.grad_arena["mat"].float() - ref["mat"].float()).norm() / ref["mat"].float().norm()
    assert dm.item() < 1e-3, dm.item()
    assert torch.allclose(store.grad_arena["vec"], ref["vec"], rtol=1e-3, atol=1e-6)   # fp32 atomics


def test_moe_engine_with_kept_attention_outputs():
    """The MoE engine under the "attention" activation policy (attention outputs kept, the expert FFN with
    its routing recomputed in backward) gives the gradients and the auxiliary loss of full recompute."""
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.synthetic import tiny_batch
    from sensenova_u1_b200.models.engine_moe import MoEMoTEngine
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.ops import _lib
    cfg = tiny_mot(head_dim=128, patch_size=16, num_layers=2, num_experts=8, num_experts_per_tok=2,
                   gen_num_experts=8, gen_num_experts_per_tok=2, moe_intermediate_size=128,
                   router_aux_loss_coef=0.01)
    store = ParamStore(cfg, device="cuda")
    store.init_weights(0, std=0.05)
    batch = tiny_batch(cfg, seed=0, n_text=200, image_px=8 * 32, with_und_image=True).to("cuda")
    g = torch.Generator(device="cuda").manual_seed(5)
    noise = torch.randn(batch.gen_x16.shape, device="cuda", generator=g)
    res = {}
    for mode in ("full", "attention"):
        eng = MoEMoTEngine(cfg, store)
        eng.recompute = mode
        store.zero_grads()
        out = eng.forward_backward(batch, noise)
        _lib.check_status()
        assert eng._mode == mode
        res[mode] = (out, {k: v.clone() for k, v in store.grad_arena.items()})
    (o1, g1), (o2, g2) = res["full"], res["attention"]
    assert torch.allclose(o1["loss"], o2["loss"], rtol=1e-5)
    assert torch.allclose(o1["moe_aux"], o2["moe_aux"], rtol=1e-5)
    dm = (g1["mat"].float() - g2["mat"].float()).norm() / g1["mat"].float().norm()
    assert dm.item() < 1e-3, dm.item()
    # automatic policy: the first step recomputes everything, the second keeps the attention outputs once the
    # steady-state free memory is known
    eng = MoEMoTEngine(cfg, store)
    modes = []
    for _ in range(3):
        store.zero_grads()
        out = eng.forward_backward(batch, noise)
        modes.append(eng._mode)
    _lib.check_status()
    assert modes == ["full", "attention", "attention"], modes
    dm = (g1["mat"].float() - store.grad_arena["mat"].float()).norm() / g1["mat"].float().norm()
    assert dm.item() < 1e-3, dm.item()


@pytest.mark.parametrize("shape", ["text_only", "image_only"])
def test_degenerate_partitions_match_oracle(shape):
    """A packed batch without any generation row (the generation partition is empty) and one that is
    almost only a generation image: both partitions may be empty or fill the sequence."""
    from sensenova_u1_b200.data.batch import Sample, Segment, build_packed_batch
    from sensenova_u1_b200.models.engine import MoTEngine
    from sensenova_u1_b200.ops import _lib
    cfg, store, _, _ = _setup()
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(8, cfg.vocab_size, (333,), generator=g)          # ragged: not a multiple of 128
    if shape == "text_only":
        segs = [Segment("text", ids=ids[:100], loss=False), Segment("text", ids=ids[100:], loss=True)]
    else:
        segs = [Segment("text", ids=ids[:5], loss=False),
                Segment("gen_image", pixels=torch.rand(3, 12 * 32, 10 * 32, generator=g) * 2 - 1)]
    batch = build_packed_batch([Sample(segs)], cfg, seed=1).to("cuda")
    assert (batch.n_gen_pad == 0) == (shape == "text_only")
    noise = torch.randn(batch.gen_x16.shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(2))
    eng = MoTEngine(cfg, store)
    store.zero_grads()
    out = eng.forward_backward(batch, noise)
    torch.cuda.synchronize(); _lib.check_status()
    loss_ref, parts_ref, grads_ref = _oracle(cfg, store, batch, noise)
    assert abs(out["loss"].item() - loss_ref.item()) < 3e-2 * abs(loss_ref.item())
    bad = []
    for name, gref in grads_ref.items():
        if gref is None or gref.norm().item() < 1e-6:
            continue
        err = (store.g[name].float() - gref).norm().item() / gref.norm().item()
        if err > 0.1:
            bad.append((name, round(err, 3)))
    assert not bad, bad


def test_moe_routing_with_empty_experts():
    """Experts that receive no token: empty segments, no tile, zero weight gradient, finite output."""
    from sensenova_u1_b200.ops import _lib, gemm, moe
    from sensenova_u1_b200.ops.gemm import OUT_BF16_ACC
    R, E, K, H, Fe = 300, 8, 2, 256, 128
    g = torch.Generator(device="cuda").manual_seed(0)
    logits = torch.randn(R, E, device="cuda", generator=g)
    logits[:, 4:] -= 50.0                                      # experts 4..7 are never chosen
    r = moe.route(logits.contiguous(), K, True)
    counts = r.counts.cpu()
    assert counts[4:].sum() == 0 and counts[:4].sum() == R * K
    ss, se = r.seg_start.cpu(), r.seg_end.cpu()
    assert all(int(se[e]) == int(ss[e]) for e in range(4, 8))
    x = (torch.randn(R, H, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    xp = torch.zeros(r.max_rows, H, dtype=torch.bfloat16, device="cuda")
    moe.gather(x, r, xp)
    w = (torch.randn(E, Fe, H, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    y = gemm.gemm_nt(xp, w, tile_group=r.tile_group)
    dy = (torch.randn(r.max_rows, Fe, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    dy[int(r.total_rows.item()):] = 0
    gw = torch.zeros(E, Fe, H, dtype=torch.bfloat16, device="cuda")
    gemm.gemm_tn(dy, xp, out=gw, k_begin=r.seg_start, k_end=r.seg_end, num_groups=E, out_mode=OUT_BF16_ACC)
    torch.cuda.synchronize(); _lib.check_status()
    used = int(r.total_rows.item())                       # rows past the last segment are never written
    assert torch.isfinite(y[:used].float()).all() and float(gw[4:].float().abs().max()) == 0.0
    e0 = 0
    ref = dy[int(ss[e0]):int(se[e0])].float().t() @ xp[int(ss[e0]):int(se[e0])].float()
    assert ((gw[e0].float() - ref).norm() / ref.norm()).item() < 2e-2


def test_frozen_branch_skips_its_weight_gradients():
    """With the understanding branch marked frozen its weight-gradient slices stay zero while the
    generation slices and every activation gradient are unchanged."""
    from sensenova_u1_b200.models.engine import MoTEngine
    from sensenova_u1_b200.ops import _lib
    cfg, store, batch, noise = _setup()
    eng = MoTEngine(cfg, store)
    store.zero_grads()
    eng.forward_backward(batch, noise)
    ref = {k: v.clone() for k, v in store.g.items()}
    eng2 = MoTEngine(cfg, store)
    eng2.skip_wgrad_groups = (0,)
    store.zero_grads()
    eng2.forward_backward(batch, noise)
    torch.cuda.synchronize(); _lib.check_status()
    for name in ("layers.0.wqkv", "layers.1.w13", "layers.0.wo", "layers.1.w2"):
        assert float(store.g[name][0].float().abs().max()) == 0.0, name
        assert torch.equal(store.g[name][1], ref[name][1]), name
    assert torch.equal(store.g["embed_tokens"], ref["embed_tokens"])        # activation gradients unchanged


def test_first_micro_batch_stores_layer_gradients():
    """The trainer does not clear the decoder layers' matrix gradients: the first micro-batch stores them.  Two
    steps of two micro-batches give exactly the weights of the clear-then-add path, also when the gradient arena
    starts out full of NaN."""
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.data.synthetic import tiny_batch
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.ops import _lib
    from sensenova_u1_b200.train.optimizer import AdamConfig
    from sensenova_u1_b200.train.trainer import Trainer
    cfg = tiny_mot(head_dim=128, patch_size=16, num_layers=2)
    stores = []
    for fast in (True, False):
        store = ParamStore(cfg, device="cuda")
        store.init_weights(0, std=0.05)
        tr = Trainer(cfg, store, AdamConfig(lr=1e-2, state_dtype="fp32", clip_grad_norm=0.0))
        tr.store_first_enabled = fast
        if fast:
            store.grad_arena["mat"].fill_(float("nan"))
        for step in range(2):
            batches = [tiny_batch(cfg, seed=10 * step + i, n_text=200, image_px=8 * 32).to("cuda") for i in range(2)]
            g = torch.Generator(device="cuda").manual_seed(step)
            noise = [torch.randn(b.gen_x16.shape, device="cuda", generator=g) for b in batches]
            out = tr.step_on_device(batches, lr=1e-2, noise=noise)
        _lib.check_status()
        assert torch.isfinite(out["loss"]).item()
        stores.append(store)
    a, b = stores
    assert torch.isfinite(a.arena["mat"].float()).all()
    for name in ("layers.0.wqkv", "layers.1.w13", "layers.1.w2", "layers.0.wo"):
        assert torch.equal(a.p[name], b.p[name]), name
    rel = (a.arena["mat"].float() - b.arena["mat"].float()).norm() / b.arena["mat"].float().norm()
    # embeddings / heads: their gradients are summed with fp32 atomics in an order that differs from run to run, so a
    # few bf16 weights land on the other side of a rounding boundary (one ulp = 4e-3 relative); a gradient that was
    # lost or counted twice would move every weight by about the learning rate instead
    assert rel.item() < 2e-3, rel.item()
