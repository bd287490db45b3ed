"""Pins this package's model maths to the reference's own code (CPU, tiny sizes, fp32).

The reference inference package is imported from a plain copy of its ``src`` tree and its
``NEOChatModel`` is driven through its stock entry points; nothing of it is restated here.
A tiny parameter store of this package is exported with ``export_hf``, loaded into the
reference model by name (strict), and then compared:

* the key set of the exported checkpoint against the reference module's ``state_dict``;
* ``t2i_generate`` (prefix cache, block-causal prefix mask, 3-axis RoPE, qk half-norms,
  generation-branch weights, timestep / noise-scale embedders, MLP head, Euler steps, CFG)
  against ``oracle.t2i_reference`` from the same noise;
* prefix logits of a text prompt against the oracle's decoder stack;
* the training attention mask: the reference's ``mask_mod`` evaluated densely against
  ``ops.attention.dense_mask`` on a packed batch with two documents, an understanding image, a
  generation image and its understanding duplicate.
"""
import json
import math
import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
_CANDIDATES = [ROOT / "baseline" / "_ref", Path("/root/reference")]
REF = next((c for c in _CANDIDATES if (c / "src" / "sensenova_u1").is_dir()), None)

pytestmark = pytest.mark.skipif(REF is None, reason="no copy of the reference source tree is available")


def _ref_inference():
    p = str(REF / "src")
    if p not in sys.path:
        sys.path.append(p)
    from sensenova_u1.models.neo_unify import modeling_neo_chat, modeling_qwen3
    from sensenova_u1.models.neo_unify.configuration_neo_chat import NEOChatConfig
    return modeling_neo_chat, modeling_qwen3, NEOChatConfig


def _ref_training_mask():
    """The mask builder module of the training model, loaded alone (the package around it pulls the whole
    distributed stack)."""
    p = str(REF / "training")
    if p not in sys.path:
        sys.path.append(p)          # behind this repository: both trees have `configs` and `train_sensenovau1`
    shim = str(ROOT / "baseline" / "ref_shims")
    if shim not in sys.path:
        sys.path.append(shim)
    import sensenovalm.initialize  # noqa: F401  (this import order avoids a circular import inside the reference)
    from sensenovavl.model.sensenovavl_moe_chat import modeling_sensenovavl_chat_mot as m
    return m


@pytest.fixture(scope="module", autouse=True)
def _leave_no_reference_modules_behind():
    """The reference's trees go on ``sys.path`` for this module only: afterwards their entries and every module
    loaded from them are dropped, so later tests import this repository's modules of the same names."""
    yield
    roots = tuple(str(c) for c in _CANDIDATES) + (str(ROOT / "baseline" / "ref_shims"),)
    sys.path[:] = [p for p in sys.path if not p.startswith(roots)]
    for name, mod in list(sys.modules.items()):
        f = getattr(mod, "__file__", None) or ""
        if f.startswith(roots):
            del sys.modules[name]


class FixedTokenizer:
    """Stand-in tokenizer: the conditional query maps to ``cond`` ids, the short unconditional query to
    ``uncond`` ids (the reference only calls ``tokenizer(query, return_tensors='pt')``)."""

    def __init__(self, cond, uncond):
        self.cond, self.uncond = cond, uncond

    def __call__(self, text, return_tensors="pt", **kw):
        ids = self.cond if len(text) > 200 else self.uncond
        return {"input_ids": ids.view(1, -1).clone()}


@pytest.fixture(scope="module")
def tiny_pair(tmp_path_factory):
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.models.params import ParamStore
    from sensenova_u1_b200.train.checkpoint import export_hf, hf_config_dict
    mnc, mq3, NEOChatConfig = _ref_inference()
    cfg = tiny_mot(vocab_size=512, hidden_size=128, num_heads=4, num_kv_heads=2, head_dim=32, ffn_size=256,
                   num_layers=2, vision_hidden=64, fm_head_dim=4096, patch_size=16, merge_size=2,
                   noise_scale_mode="resolution", add_noise_scale_embedding=True)
    store = ParamStore(cfg, device="cpu", dtype=torch.float32, with_grads=False)
    store.init_weights(seed=3, std=0.05)
    # random gains / biases so that every tensor matters
    g = torch.Generator().manual_seed(5)
    for s in store.specs:
        if s.arena == "vec":
            store.p[s.name].copy_(1.0 + 0.2 * torch.randn(store.p[s.name].shape, generator=g)
                                  if s.init == "ones" else 0.1 * torch.randn(store.p[s.name].shape, generator=g))
    out = tmp_path_factory.mktemp("hf")
    export_hf(store, str(out))
    hf = hf_config_dict(cfg)
    hf["llm_config"]["architectures"] = ["Qwen3ForCausalLM"]
    hf["llm_config"]["tie_word_embeddings"] = False
    hf.update(template="sensenova-u1" if False else hf.get("template"), fm_head_layers=2, fm_head_mlp_ratio=1,
              concat_time_token_num=0)
    return cfg, store, out, hf, (mnc, mq3, NEOChatConfig)


def _build_ref_model(hf, out, mnc, NEOChatConfig):
    from safetensors import safe_open
    conf = dict(hf)
    conf.pop("model_type", None)
    conf.pop("architectures", None)
    if conf.get("template") is None:
        from sensenova_u1.models.neo_unify.conversation import conv_templates
        conf["template"] = next(iter(conv_templates))
    rcfg = NEOChatConfig(**conf)
    torch.manual_seed(0)
    model = mnc.NEOChatModel(rcfg).float().eval()
    sd = {}
    for f in sorted(Path(out).glob("*.safetensors")):
        with safe_open(str(f), framework="pt") as fh:
            for k in fh.keys():
                sd[k] = fh.get_tensor(k)
    return model, sd


def test_exported_keys_are_the_reference_modules_keys(tiny_pair):
    cfg, store, out, hf, (mnc, mq3, NEOChatConfig) = tiny_pair
    model, sd = _build_ref_model(hf, out, mnc, NEOChatConfig)
    ref_keys = {k for k in model.state_dict().keys() if "rotary_emb" not in k and "inv_freq" not in k}
    assert set(sd) == ref_keys, (sorted(set(sd) - ref_keys)[:5], sorted(ref_keys - set(sd))[:5])
    for k, v in model.state_dict().items():
        if k in sd:
            assert tuple(v.shape) == tuple(sd[k].shape), k
    model.load_state_dict(sd, strict=False)


def test_t2i_generate_matches_oracle(tiny_pair):
    from sensenova_u1_b200.models import oracle
    cfg, store, out, hf, (mnc, mq3, NEOChatConfig) = tiny_pair
    model, sd = _build_ref_model(hf, out, mnc, NEOChatConfig)
    model.load_state_dict(sd, strict=False)
    mq3.set_attn_backend("sdpa")
    g = torch.Generator().manual_seed(11)
    cond = torch.randint(8, cfg.vocab_size, (37,), generator=g)
    uncond = torch.randint(8, cfg.vocab_size, (6,), generator=g)
    W = Hh = 128
    steps, scale, shift, seed = 3, 4.0, 3.0, 21
    with torch.no_grad():
        ref_img = model.t2i_generate(FixedTokenizer(cond, uncond), "x" * 10, cfg_scale=scale, timestep_shift=shift,
                                     image_size=(W, Hh), num_steps=steps, seed=seed, t_eps=0.02)
    noise = torch.randn((1, 3, Hh, W), generator=torch.Generator("cpu").manual_seed(seed), dtype=torch.float32)
    with torch.no_grad():
        ours = oracle.t2i_reference(store.p, cfg, cond, uncond, (W, Hh), steps, scale, shift, noise, t_eps=0.02)
    err = (ours - ref_img.float()).abs().max().item()
    assert err < 2e-3 * max(1.0, ref_img.abs().max().item()), err


def test_prefix_logits_match_oracle(tiny_pair):
    from sensenova_u1_b200.models import oracle
    from sensenova_u1_b200.ops.attention import dense_mask, make_meta
    cfg, store, out, hf, (mnc, mq3, NEOChatConfig) = tiny_pair
    model, sd = _build_ref_model(hf, out, mnc, NEOChatConfig)
    model.load_state_dict(sd, strict=False)
    n = 29
    ids = torch.randint(8, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(2))
    t = torch.arange(n)
    idx = torch.stack([t, torch.zeros_like(t), torch.zeros_like(t)])
    with torch.no_grad():
        ref = model.language_model(input_ids=ids.view(1, -1), indexes=idx,
                                   attention_mask={"full_attention": mq3.create_block_causal_mask(idx[0])}).logits[0]
        p = store.p
        x = p["embed_tokens"][ids]
        is_gen = torch.zeros(n, dtype=torch.bool)
        meta = make_meta(torch.zeros(n), t)
        mask = dense_mask(meta, meta)
        for l in range(cfg.num_layers):
            x = oracle.decoder_layer(p, l, x, is_gen, idx, mask, cfg)
        from sensenova_u1_b200.models.params import UND
        ours = torch.nn.functional.linear(oracle.rmsnorm(x, p["final_norm"][UND], cfg.rms_eps), p["lm_head"])
    assert (ours - ref).abs().max().item() < 2e-3


def test_thw_indexes_match(tiny_pair):
    from sensenova_u1_b200.inference.api import NEOChatModel as Ours
    cfg, store, out, hf, (mnc, mq3, NEOChatConfig) = tiny_pair
    model, _ = _build_ref_model(hf, out, mnc, NEOChatConfig)
    ctx, start = 500, 501
    model.img_context_token_id, model.img_start_token_id = ctx, start
    grids = [(2, 3), (4, 2)]
    ids = [5, 6, start] + [ctx] * 6 + [9, 10, start] + [ctx] * 8 + [11]
    ids = torch.tensor(ids)
    merged = torch.tensor(grids)
    try:
        ref = model.get_thw_indexes(ids, merged * 2)          # the reference takes patch grids (before the 2x2 merge)
    except Exception:
        pytest.skip("reference get_thw_indexes has another calling convention in this version")
    ours = Ours.get_thw_indexes(ids, grids, ctx)
    assert torch.equal(ours.cpu(), ref.cpu().reshape(ours.shape))


def test_training_mask_matches_reference_mask_mod():
    from sensenova_u1_b200.ops.attention import dense_mask, make_meta
    try:
        m = _ref_training_mask()
    except Exception as e:      # the training package needs optional third-party modules at import
        pytest.skip(f"reference training model module does not import here: {type(e).__name__}: {e}")
    doc, pos, img, gen, blocked = [], [], [], [], []

    def text(d, n, p0):
        for i in range(n):
            doc.append(d); pos.append(p0 + i); img.append(0); gen.append(0); blocked.append(0)
        return p0 + n

    def image(d, n, p0, iid, is_gen, blocked_last=False):
        for i in range(n):
            doc.append(d); pos.append(p0); img.append(iid); gen.append(is_gen)
            blocked.append(1 if (blocked_last and i == n - 1) else 0)
        return p0 + 1

    # doc 0: 5 text, a generated image (4 tokens), its understanding duplicate at the same position (its last
    # token is a key nobody may read), 3 text; doc 1: 2 text, an understanding image, 3 text; then padding
    p0 = text(0, 5, 0)
    image(0, 4, p0, 1, 1)
    p0 = image(0, 4, p0, 2, 0, blocked_last=True)
    text(0, 3, p0)
    p1 = text(1, 2, 0)
    p1 = image(1, 4, p1, 3, 0)
    text(1, 3, p1)
    t = lambda x, dt=torch.long: torch.tensor(x, dtype=dt)
    S = len(doc)
    # the reference lets torch's create_block_mask default to device="cuda"; on a CPU-only box bind it to the CPU
    # (the mask_mod closure, which is what is compared, is the reference's own)
    import functools
    from torch.nn.attention.flex_attention import create_block_mask
    if not torch.cuda.is_available():
        m.create_block_mask = functools.partial(create_block_mask, device="cpu")
    bm, padlen = m.create_flex_mask_padding_image_gen(
        t(doc), t(img), t(gen, torch.bool), t(pos), t(blocked, torch.bool), div_num=128, compile_mask=False)
    ref = m.dense_from_flex_mask(bm.mask_mod, S + padlen, device="cpu")[:S, :S]
    meta = make_meta(t(doc), t(pos), t(img), t(gen), t(blocked))
    ours = dense_mask(meta, meta)
    assert torch.equal(ours, ref), (ours != ref).nonzero()[:8]
    # the same rule in [generation rows | understanding rows] storage order, which the engine uses
    perm = torch.cat([t(gen).nonzero().flatten(), (t(gen) == 0).nonzero().flatten()])
    meta_p = meta[perm]
    assert torch.equal(dense_mask(meta_p, meta_p), ref[perm][:, perm])
