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
    if S >= 128:
        for got, want in ((o, ref.detach()), (dq, qf.grad), (dk, kf.grad), (dv, vf.grad)):
            worst, max_abs = _row_tile_err(got, want)
            assert worst < 2e-2 and max_abs < 2e-2, (worst, max_abs)


def _row_tile_err(got, ref, rows=128):
    """Worst relative error over blocks of 128 rows (one query / key tile) and the largest absolute error in units
    of the reference's largest magnitude (bf16 rounding of the output alone gives up to 2^-8 there)."""
    d = (got.float() - ref.float()).flatten(1)
    r = ref.float().flatten(1)
    n = d.shape[0] // rows * rows
    blk = lambda t: t[:n].view(-1, rows * t.shape[1]).norm(dim=1)
    worst = (blk(d) / (blk(r) + 1e-3 * r.norm() / max(1, n // rows) ** 0.5)).max().item()
    return worst, (d.abs().max() / r.abs().max()).item()


@pytest.mark.parametrize("n_gen", [0, 128, 16384])
def test_training_size_mixed_mask_in_branch_order(n_gen):
    """16,384 packed rows in the engine's row order (generation rows first, understanding rows after them): documents
    of 2,048 tokens; with ``n_gen`` > 0 the first rows are noised-image tokens (full attention inside their image,
    causal towards the text before it)."""
    from sensenova_u1_b200.ops import _lib, attention as A
    S, Hq, Hkv, L = 16384, 2, 1, 2048
    idx = torch.arange(S, device=DEV)
    doc, r = idx // L, idx % L
    if n_gen == 0:
        pos, img, gen = r, torch.zeros_like(r), torch.zeros_like(r, dtype=torch.bool)
    elif n_gen == S:                                     # every document is one generated image
        pos, img, gen = torch.zeros_like(r), doc + 1, torch.ones_like(r, dtype=torch.bool)
    else:                                                # document 0: 1,000 text tokens, a 128-token image, text
        isimg = (doc == 0) & (r >= 1000) & (r < 1000 + n_gen)
        after = (doc == 0) & (r >= 1000 + n_gen)
        pos = torch.where(isimg, torch.full_like(r, 1000), torch.where(after, r - n_gen + 1, r))
        img, gen = isimg.long(), isimg
    order = torch.cat([idx[gen], idx[~gen]])             # [gen rows | und rows]
    meta = A.make_meta(doc[order], pos[order], img[order], gen[order])
    g = torch.Generator(device=DEV).manual_seed(77)
    mk = lambda h: torch.randn(S, h, 128, device=DEV, generator=g).to(torch.bfloat16)
    q, k, v, do = mk(Hq), mk(Hkv), mk(Hkv), mk(Hq)
    plan = A.build_plan(meta)
    sc = 128 ** -0.5
    o, lse = A.attention_fwd(q, k, v, plan, sc)
    dq, dk, dv = A.attention_bwd(q, k, v, o, do, lse, plan, sc)
    _lib.check_status()
    qf, kf, vf = [t.float().requires_grad_(True) for t in (q, k, v)]
    ref = A.reference_attention(qf, kf, vf, meta, meta, sc)
    ref.backward(do.float())
    for name, got, want, tol in (("o", o, ref.detach(), 8e-3), ("dq", dq, qf.grad, 1.5e-2), ("dk", dk, kf.grad, 1.5e-2),
                                 ("dv", dv, vf.grad, 1.5e-2)):
        worst, max_abs = _row_tile_err(got, want)
        assert _rel(got, want) < tol and worst < 2 * tol and max_abs < 2e-2, (name, _rel(got, want), worst, max_abs)


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


@pytest.mark.parametrize("slots", [0, 3])
def test_mask_bits_equal_the_rule(slots):
    """Partial tiles read their mask as bits written by the tile classifier.  With no table (0 slots) every partial
    tile evaluates the mask rule per element; with 3 slots most partial tiles find the table full and fall back.
    Both must give exactly the results of the default table."""
    from sensenova_u1_b200.ops import _lib, attention as A
    S, Hq, Hkv = 1500, 4, 2
    g = torch.Generator(device=DEV).manual_seed(5)
    mk = lambda h: torch.randn(S, h, 128, device=DEV, generator=g).to(torch.bfloat16)
    q, k, v, do = mk(Hq), mk(Hkv), mk(Hkv), mk(Hq)
    meta = _meta(S, "mixed")
    sc = 128 ** -0.5
    plan = A.build_plan(meta)
    assert plan.tile_slot is not None
    n_partial = int((plan.cls == 1).sum())
    assert int(plan.slot_counter.item()) == n_partial and n_partial > 3
    # the bits themselves against the dense oracle mask, both orientations
    dense = A.dense_mask(meta, meta)
    nq = (S + 127) // 128
    pad = torch.zeros(nq * 128, nq * 128, dtype=torch.bool, device=DEV)
    pad[:S, :S] = dense
    shifts = torch.arange(32, device=DEV)
    for qt, kt in [(0, 0), (3, 2), (nq - 1, nq - 1)]:
        if plan.cls[qt, kt].item() != 1:
            continue
        slot = int(plan.tile_slot[qt, kt])
        blk = pad[qt * 128:(qt + 1) * 128, kt * 128:(kt + 1) * 128]
        unpack = lambda words: ((words.view(128, 4, 1) >> shifts) & 1).bool().view(128, 128)
        assert torch.equal(unpack(plan.bits_q[slot]), blk)
        assert torch.equal(unpack(plan.bits_k[slot]), blk.t())
    ref_o, ref_lse = A.attention_fwd(q, k, v, plan, sc)
    ref_g = A.attention_bwd(q, k, v, ref_o, do, ref_lse, plan, sc)
    plan2 = A.build_plan(meta, mask_slots=slots)
    o, lse = A.attention_fwd(q, k, v, plan2, sc)
    grads = A.attention_bwd(q, k, v, o, do, lse, plan2, sc)
    _lib.check_status()
    assert torch.equal(o, ref_o) and torch.equal(lse, ref_lse)
    for a, b in zip(grads, ref_g):
        assert torch.equal(a, b)


def test_launch_order_is_by_list_length_and_does_not_change_results():
    from sensenova_u1_b200.ops import _lib, attention as A
    S, Hq, Hkv = 2000, 4, 2
    g = torch.Generator(device=DEV).manual_seed(9)
    mk = lambda h: torch.randn(S, h, 128, device=DEV, generator=g).to(torch.bfloat16)
    q, k, v, do = mk(Hq), mk(Hkv), mk(Hkv), mk(Hq)
    plan = A.build_plan(_meta(S, "docs"))
    for order, count in ((plan.pair_order, plan.pair_count), (plan.q_order, plan.kv_count), (plan.kv_order, plan.q_count)):
        assert sorted(order.tolist()) == list(range(count.numel()))
        c = count[order.long()].tolist()
        assert c == sorted(c, reverse=True)
    sc = 128 ** -0.5
    o, lse = A.attention_fwd(q, k, v, plan, sc)
    grads = A.attention_bwd(q, k, v, o, do, lse, plan, sc)
    plan.pair_order = plan.q_order = plan.kv_order = None          # natural order
    o2, lse2 = A.attention_fwd(q, k, v, plan, sc)
    grads2 = A.attention_bwd(q, k, v, o2, do, lse2, plan, sc)
    _lib.check_status()
    assert torch.equal(o, o2) and torch.equal(lse, lse2)
    for a, b in zip(grads, grads2):
        assert torch.equal(a, b)
