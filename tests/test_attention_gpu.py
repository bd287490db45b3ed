"""Packed mixed-mask attention (tcgen05) forward and backward against dense fp32 softmax."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _meta(S, kind):
    from sensenova_u1_b200.ops import attention as A
    idx = torch.arange(S, device=DEV)
    if kind == "causal":
        return A.make_meta(torch.zeros_like(idx), idx)
    if kind == "full":
        return A.make_meta(torch.zeros_like(idx), torch.zeros_like(idx))
    if kind == "docs":
        return A.make_meta(idx // 200, idx)
    doc = idx // 300
    r = idx % 300
    isimg = (r >= 100) & (r < 164)
    pos = torch.where(r < 100, r, torch.where(isimg, torch.full_like(r, 100), r - 63))
    img = torch.where(isimg, doc + 1, torch.zeros_like(doc))
    gen = isimg & (doc % 2 == 0)
    blocked = (r == 99) & (doc % 3 == 0)
    return A.make_meta(doc, pos, img, gen, blocked)


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("S,Hq,Hkv,kind", [(128, 1, 1, "full"), (512, 4, 1, "causal"), (1000, 8, 2, "docs"),
                                           (1500, 4, 1, "mixed"), (2048, 8, 2, "causal")])
def test_forward_backward(S, Hq, Hkv, kind):
    from sensenova_u1_b200.ops import _lib, attention as A
    g = torch.Generator(device=DEV).manual_seed(S)
    mk = lambda h: torch.randn(S, h, 128, device=DEV, generator=g).to(torch.bfloat16)
    q, k, v, do = mk(Hq), mk(Hkv), mk(Hkv), mk(Hq)
    meta = _meta(S, kind)
    plan = A.build_plan(meta)
    sc = 128 ** -0.5
    o, lse = A.attention_fwd(q, k, v, plan, sc)
    dq, dk, dv = A.attention_bwd(q, k, v, o, do, lse, plan, sc)
    _lib.check_status()
    qf, kf, vf = [t.float().requires_grad_(True) for t in (q, k, v)]
    ref = A.reference_attention(qf, kf, vf, meta, meta, sc)
    ref.backward(do.float())
    assert _rel(o, ref) < 6e-3
    assert _rel(dq, qf.grad) < 1e-2 and _rel(dk, kf.grad) < 1e-2 and _rel(dv, vf.grad) < 1e-2


def test_tile_classes_and_cross_lengths():
    from sensenova_u1_b200.ops import _lib, attention as A
    S = 1024
    meta = _meta(S, "causal")
    plan = A.build_plan(meta)
    cls = plan.cls.cpu()
    for qt in range(8):
        for kt in range(8):
            want = 0 if kt > qt else (1 if kt == qt else 2)
            assert cls[qt, kt].item() == want
    assert plan.kv_count.tolist() == list(range(1, 9))
    assert plan.q_count.tolist() == list(range(8, 0, -1))
    # generation step of inference: 300 queries against 1000 keys, no mask
    g = torch.Generator(device=DEV).manual_seed(1)
    q = torch.randn(300, 4, 128, device=DEV, generator=g).to(torch.bfloat16)
    k = torch.randn(1000, 1, 128, device=DEV, generator=g).to(torch.bfloat16)
    v = torch.randn(1000, 1, 128, device=DEV, generator=g).to(torch.bfloat16)
    mq, mk = _meta(300, "full"), _meta(1000, "full")
    plan = A.build_plan(mq, mk)
    o, _ = A.attention_fwd(q, k, v, plan, 128 ** -0.5)
    _lib.check_status()
    assert _rel(o, A.reference_attention(q, k, v, mq, mk, 128 ** -0.5)) < 6e-3


def test_rows_without_keys_and_determinism():
    from sensenova_u1_b200.ops import attention as A
    S = 256
    idx = torch.arange(S, device=DEV)
    blocked = idx >= 128                       # second tile: keys nobody may read, queries of another doc
    meta = A.make_meta((idx >= 128).int(), idx, blocked=blocked)
    g = torch.Generator(device=DEV).manual_seed(2)
    q = torch.randn(S, 2, 128, device=DEV, generator=g).to(torch.bfloat16)
    k = torch.randn(S, 2, 128, device=DEV, generator=g).to(torch.bfloat16)
    v = torch.randn(S, 2, 128, device=DEV, generator=g).to(torch.bfloat16)
    plan = A.build_plan(meta)
    o1, lse = A.attention_fwd(q, k, v, plan, 0.1)
    o2, _ = A.attention_fwd(q, k, v, plan, 0.1)
    assert torch.equal(o1, o2)
    assert o1[128:].abs().max().item() == 0 and torch.isinf(lse[:, 128:]).all()
    do = torch.randn_like(o1)
    a = A.attention_bwd(q, k, v, o1, do, lse, plan, 0.1)
    b = A.attention_bwd(q, k, v, o1, do, lse, plan, 0.1)
    for x, y in zip(a, b):
        assert torch.equal(x, y) and torch.isfinite(x.float()).all()


@pytest.mark.parametrize("kind,blocks", [("causal", 2), ("mixed", 3), ("docs", 4)])
def test_blockwise_attention_with_ring_merge(kind, blocks):
    """Keys split into blocks, one forward per block, partial results folded with the ring-merge
    kernel: equal to attention over all keys at once; the backward kernel, given the merged
    log-sum-exp and output, yields per-block gradients that sum to the full gradient."""
    from sensenova_u1_b200.ops import _lib, attention as A
    from sensenova_u1_b200.parallel.context_attention import ring_merge
    S, Hq, Hkv = 1536, 4, 2
    g = torch.Generator(device=DEV).manual_seed(11)
    mk = lambda h: torch.randn(S, h, 128, device=DEV, generator=g).to(torch.bfloat16)
    q, k, v, do = mk(Hq), mk(Hkv), mk(Hkv), mk(Hq)
    meta = _meta(S, kind)
    sc = 128 ** -0.5
    o_ref, lse_ref = A.attention_fwd(q, k, v, A.build_plan(meta), sc)
    B = S // blocks
    o_acc = torch.empty(S, Hq, 128, dtype=torch.float32, device=DEV)
    lse = torch.empty(Hq, S, dtype=torch.float32, device=DEV)
    out = torch.empty_like(q)
    plans = []
    for j in range(blocks):
        sl = slice(j * B, (j + 1) * B)
        plans.append(A.build_plan(meta, meta[sl].contiguous()))
        o_j, lse_j = A.attention_fwd(q, k[sl].contiguous(), v[sl].contiguous(), plans[j], sc)
        ring_merge(o_acc, lse, o_j, lse_j, out=out, first=j == 0)
    _lib.check_status()
    assert _rel(out, o_ref) < 4e-3
    fin = torch.isfinite(lse_ref)
    assert torch.equal(fin, torch.isfinite(lse))
    assert (lse[fin] - lse_ref[fin]).abs().max().item() < 2e-3
    dq_ref, dk_ref, dv_ref = A.attention_bwd(q, k, v, o_ref, do, lse_ref, A.build_plan(meta), sc)
    dq = torch.zeros(S, Hq, 128, dtype=torch.float32, device=DEV)
    dk, dv = torch.empty_like(k), torch.empty_like(v)
    for j in range(blocks):
        sl = slice(j * B, (j + 1) * B)
        dq_j, dk_j, dv_j = A.attention_bwd(q, k[sl].contiguous(), v[sl].contiguous(), out, do, lse, plans[j], sc)
        dq += dq_j.float()
        dk[sl], dv[sl] = dk_j, dv_j
    _lib.check_status()
    assert _rel(dq, dq_ref) < 1e-2 and _rel(dk, dk_ref) < 1e-2 and _rel(dv, dv_ref) < 1e-2
