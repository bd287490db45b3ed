"""CUDA inference engine (KV-cached prefix, packed CFG branches, fused sampler step)
against the cache-free PyTorch sampling oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _model(seed=0):
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.models.params import ParamStore
    cfg = tiny_mot(head_dim=128, patch_size=16, num_layers=2)
    store = ParamStore(cfg, device="cuda", with_grads=False)
    store.init_weights(seed, std=0.05)
    return cfg, store


@pytest.mark.parametrize("cfg_norm", ["none", "global", "channel", "cfg_zero_star"])
def test_t2i_matches_oracle(cfg_norm):
    from sensenova_u1_b200.inference.engine import InferenceEngine
    from sensenova_u1_b200.models import oracle
    from sensenova_u1_b200.ops import _lib
    cfg, store = _model()
    eng = InferenceEngine(cfg, store)
    g = torch.Generator().manual_seed(1)
    cond = torch.randint(8, cfg.vocab_size, (37,), generator=g)
    uncond = torch.randint(8, cfg.vocab_size, (5,), generator=g)
    noise = torch.randn(1, 3, 128, 96, generator=g).cuda()
    kw = dict(image_size=(96, 128), num_steps=3, cfg_scale=3.0, timestep_shift=3.0, cfg_norm=cfg_norm)
    got = eng.t2i(cond, uncond, noise=noise, **kw)
    _lib.check_status()
    p32 = {k: v.float() for k, v in store.p.items()}
    ref = oracle.t2i_reference(p32, cfg, cond, uncond, noise=noise, **kw)
    err = ((got - ref).norm() / ref.norm()).item()
    assert got.shape == (1, 3, 128, 96) and err < 3e-2, err


def test_greedy_decode_matches_full_recompute():
    from sensenova_u1_b200.inference.engine import InferenceEngine
    from sensenova_u1_b200.models import oracle
    from sensenova_u1_b200.ops.attention import make_meta
    cfg, store = _model(3)
    eng = InferenceEngine(cfg, store)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(8, cfg.vocab_size, (21,), generator=g)
    lay, h = eng.prefill([prompt], reserve_image_tokens=8)
    toks = eng.decode_greedy(lay, h, max_new_tokens=4)[0]
    p32 = {k: v.float() for k, v in store.p.items()}
    ids = prompt.cuda()
    ref = []
    for _ in range(4):
        n = ids.numel()
        x = p32["embed_tokens"][ids]
        pos = torch.arange(n, device="cuda")
        meta = make_meta(torch.zeros(n, device="cuda"), pos)
        mask = oracle.dense_mask(meta, meta)
        pos3 = torch.stack([pos, torch.zeros_like(pos), torch.zeros_like(pos)])
        isg = torch.zeros(n, dtype=torch.bool, device="cuda")
        for l in range(cfg.num_layers):
            x = oracle.decoder_layer(p32, l, x, isg, pos3, mask, cfg)
        logits = oracle.rmsnorm(x[-1:], p32["final_norm"][0], cfg.rms_eps) @ p32["lm_head"].t()
        nxt = int(logits.argmax())
        ref.append(nxt)
        ids = torch.cat([ids, torch.tensor([nxt], device="cuda")])
    assert toks == ref


def test_public_api_t2i_editing_chat_and_interleave():
    import sensenova_u1_b200 as pkg
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.inference.api import ByteTokenizer
    from sensenova_u1_b200.ops import _lib
    cfg = tiny_mot(head_dim=128, patch_size=16, num_layers=2)
    model = pkg.NEOChatModel.from_config(cfg, device="cuda", seed=1)
    tok = ByteTokenizer(cfg.vocab_size)
    img = model.t2i_generate(tok, "a red cube", cfg_scale=3.0, timestep_shift=3.0, image_size=(64, 96), num_steps=2)
    assert img.shape == (1, 3, 96, 64) and torch.isfinite(img).all()
    src = torch.randn(3, 64, 64)
    ed = model.it2i_generate(tok, "make it blue", [src], cfg_scale=3.0, img_cfg_scale=1.5, num_steps=2)
    assert ed.shape == (1, 3, 64, 64) and torch.isfinite(ed).all()
    # the three-branch guidance reduces to two-branch guidance when the image-only branch is ignored
    ans = model.chat(tok, src, "what is this?", dict(max_new_tokens=4))
    assert isinstance(ans, str)
    text, imgs = model.interleave_gen(tok, "draw", max_rounds=1, max_new_tokens=3, image_size=(64, 64), num_steps=1)
    assert isinstance(text, str) and isinstance(imgs, list)
    _lib.check_status()


def test_moe_t2i_matches_oracle():
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.inference.engine import InferenceEngine
    from sensenova_u1_b200.models import oracle
    from sensenova_u1_b200.models.params import ParamStore
    cfg = tiny_mot(head_dim=128, patch_size=16, num_layers=2, num_experts=8, num_experts_per_tok=2,
                   gen_num_experts=8, gen_num_experts_per_tok=2, moe_intermediate_size=128)
    store = ParamStore(cfg, device="cuda", with_grads=False)
    store.init_weights(0, std=0.05)
    eng = InferenceEngine(cfg, store)
    g = torch.Generator().manual_seed(1)
    cond = torch.randint(8, cfg.vocab_size, (33,), generator=g)
    noise = torch.randn(1, 3, 64, 64, generator=g).cuda()
    kw = dict(image_size=(64, 64), num_steps=2, cfg_scale=1.0, timestep_shift=3.0)
    got = eng.t2i(cond, None, noise=noise, **kw)
    ref = oracle.t2i_reference({k: v.float() for k, v in store.p.items()}, cfg, cond, None, noise=noise, **kw)
    assert ((got - ref).norm() / ref.norm()).item() < 5e-2


def test_graph_decode_equals_eager_decode():
    """The CUDA-graph replay of the decode step yields the same tokens as launching it eagerly,
    for two documents of different length, with an early stop."""
    from sensenova_u1_b200.inference.engine import InferenceEngine
    from sensenova_u1_b200.ops import _lib
    cfg, store = _model(3)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(8, cfg.vocab_size, (n,), generator=g) for n in (17, 33)]
    outs = []
    for use_graph in (False, True):
        eng = InferenceEngine(cfg, store)
        lay, h = eng.prefill(prompts, reserve_image_tokens=24)
        outs.append(eng.decode_greedy(lay, h, max_new_tokens=20, use_graph=use_graph))
        torch.cuda.synchronize(); _lib.check_status()
        assert eng.last_decode_graph == use_graph and eng.last_decode_steps == 20
        assert lay[0].next_pos == 17 + 20
    assert outs[0] == outs[1] and all(len(o) == 20 for o in outs[0])
    # a stop id ends the loop at the next host check and trims the output
    stop = outs[0][0][3]
    eng = InferenceEngine(cfg, store)
    lay, h = eng.prefill(prompts[:1], reserve_image_tokens=24)
    got = eng.decode_greedy(lay, h, max_new_tokens=20, stop_ids=(stop,), check_every=4)[0]
    assert got == outs[0][0][: outs[0][0].index(stop) + 1] and eng.last_decode_steps <= 8


@pytest.mark.parametrize("vram_mode", ["balanced", "low"])
def test_layer_offload_gives_identical_images(vram_mode):
    """Decoder layers streamed from pinned host memory: the image is bit-identical to the resident run."""
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.inference.api import ByteTokenizer, NEOChatModel
    from sensenova_u1_b200.ops import _lib
    cfg = tiny_mot(head_dim=128, patch_size=16, num_layers=4)
    tok = ByteTokenizer(cfg.vocab_size)
    kw = dict(cfg_scale=3.0, timestep_shift=3.0, image_size=(128, 96), num_steps=3, seed=4)
    from sensenova_u1_b200.models.params import ParamStore
    host = ParamStore(cfg, device="cpu", with_grads=False)
    host.init_weights(7, std=0.05)
    dev = ParamStore(cfg, device="cuda", with_grads=False)
    dev.copy_from(host)
    full = NEOChatModel(cfg, dev).t2i_generate(tok, "a small boat", **kw)
    m = NEOChatModel(cfg, host, vram_mode=vram_mode, device="cuda")
    off = m.t2i_generate(tok, "a small boat", **kw)
    torch.cuda.synchronize(); _lib.check_status()
    assert torch.equal(full, off)
    assert m.engine.offload.bytes_streamed > 0
