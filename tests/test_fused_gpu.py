"""Memory-bound sm_100a kernels against plain fp32 PyTorch."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _bf(*shape, seed=0, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, device=DEV, generator=g) * scale).to(torch.bfloat16)


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("H", [512, 4096, 384])      # warp-per-row kernels (2 and 16 vectors per lane), generic kernel
def test_rmsnorm_fwd_bwd_dual_gain(H):
    from sensenova_u1_b200.models import oracle
    from sensenova_u1_b200.ops import fused
    S = 384
    x, dy = _bf(S, H, seed=1), _bf(S, H, seed=2)
    gain = (1 + 0.1 * torch.randn(2, H, device=DEV)).to(torch.bfloat16)
    tg = torch.tensor([1, 0, 0], dtype=torch.int32, device=DEV)
    y = torch.empty_like(x); rstd = torch.empty(S, device=DEV)
    fused.rmsnorm_fwd(x, gain, tg, y, rstd, 1e-6)
    xf = x.float().requires_grad_(True)
    gf = gain.float().requires_grad_(True)
    rows_g = tg.repeat_interleave(128).long()
    ref = oracle.rmsnorm(xf, gf[rows_g], 1e-6)
    assert _rel(y, ref) < 5e-3
    ref.backward(dy.float())
    dx = torch.empty_like(x); dg = torch.zeros(2, H, device=DEV)
    res = _bf(S, H, seed=3)
    fused.rmsnorm_bwd(dy, x, gain, rstd, tg, res, dx, dg)
    assert _rel(dx, xf.grad + res.float()) < 1e-2
    assert _rel(dg, gf.grad) < 1e-2


def test_rmsnorm_many_tiles_and_alternating_gain_sets():
    """74 tiles, the gain set alternating from tile to tile, some of them padding tiles (which take no part in the
    gain gradient)."""
    from sensenova_u1_b200.models import oracle
    from sensenova_u1_b200.ops import fused
    tiles, H = 74, 1024
    S = tiles * 128
    x, dy = _bf(S, H, seed=11), _bf(S, H, seed=12)
    gain = (1 + 0.1 * torch.randn(2, H, device=DEV)).to(torch.bfloat16)
    tg = (torch.arange(tiles, device=DEV) % 2).int()
    tg[5] = -1
    tg[40] = -1
    y = torch.empty_like(x); rstd = torch.empty(S, device=DEV)
    fused.rmsnorm_fwd(x, gain, tg, y, rstd, 1e-6)
    xf = x.float().requires_grad_(True)
    gf = gain.float().requires_grad_(True)
    rows_g = tg.clamp(min=0).repeat_interleave(128).long()
    live = (tg >= 0).repeat_interleave(128)
    ref = oracle.rmsnorm(xf, gf[rows_g], 1e-6)
    assert _rel(y, ref) < 5e-3
    (ref * dy.float() * live[:, None]).sum().backward()
    dx = torch.empty_like(x); dg = torch.zeros(2, H, device=DEV)
    fused.rmsnorm_bwd(dy, x, gain, rstd, tg, None, dx, dg)
    assert _rel(dx[live], xf.grad[live]) < 1e-2
    assert _rel(dg, gf.grad) < 1e-2


def test_qknorm_rope_fwd_bwd():
    from sensenova_u1_b200.config import tiny_mot
    from sensenova_u1_b200.models import oracle
    from sensenova_u1_b200.ops import fused
    cfg = tiny_mot(head_dim=128, num_heads=4, num_kv_heads=2)
    S = 256
    qkv = _bf(S, cfg.q_dim + 2 * cfg.kv_dim, seed=4)
    gains = (1 + 0.1 * torch.randn(2, 4, 64, device=DEV)).to(torch.bfloat16)
    tg = torch.tensor([1, 0], dtype=torch.int32, device=DEV)
    pos3 = torch.stack([torch.randint(0, 5000, (S,)), torch.randint(0, 64, (S,)), torch.randint(0, 64, (S,))]).to(DEV).int()
    inv_t, inv_hw = oracle.rope_inv_freq(cfg, DEV)
    out = torch.empty(S, cfg.q_dim + cfg.kv_dim, dtype=torch.bfloat16, device=DEV)
    fused.qknorm_rope_fwd(qkv, out, gains, tg, pos3, inv_t, inv_hw, 4, 2, 1e-6)
    qf = qkv.float().requires_grad_(True)
    gf = gains.float().requires_grad_(True)
    refs = []
    for t, grp in enumerate(tg.tolist()):
        r = slice(t * 128, (t + 1) * 128)
        q, k, _ = oracle.qk_norm_rope(qf[r], gf[grp], pos3[:, r], cfg)
        refs.append(torch.cat([q.reshape(128, -1), k.reshape(128, -1)], 1))
    ref = torch.cat(refs)
    assert _rel(out, ref) < 6e-3
    d = _bf(S, cfg.q_dim + cfg.kv_dim, seed=5)
    ref.backward(d.float())
    dgains = torch.zeros(2, 4, 64, device=DEV)
    dbuf = torch.zeros(S, cfg.q_dim + 2 * cfg.kv_dim, dtype=torch.bfloat16, device=DEV)
    dbuf[:, : cfg.q_dim + cfg.kv_dim] = d
    fused.qknorm_rope_bwd(qkv, dbuf, gains, dgains, tg, pos3, inv_t, inv_hw, 4, 2, 1e-6)
    assert _rel(dbuf[:, : cfg.q_dim + cfg.kv_dim], qf.grad[:, : cfg.q_dim + cfg.kv_dim]) < 1.5e-2
    assert _rel(dgains, gf.grad) < 1.5e-2


def test_swiglu_and_gelu():
    from sensenova_u1_b200.ops import fused
    gu, da = _bf(300, 512, seed=6), _bf(300, 256, seed=7)
    act = torch.empty(300, 256, dtype=torch.bfloat16, device=DEV)
    fused.swiglu_fwd(gu, act)
    gf = gu.float().requires_grad_(True)
    ref = F.silu(gf[:, :256]) * gf[:, 256:]
    assert _rel(act, ref) < 5e-3
    ref.backward(da.float())
    dgu = torch.empty_like(gu)
    fused.swiglu_bwd(gu, da, dgu)
    assert _rel(dgu, gf.grad) < 1e-2
    x = _bf(64, 128, seed=8)
    y = torch.empty_like(x)
    fused.gelu_fwd(x, y)
    xf = x.float().requires_grad_(True)
    r = F.gelu(xf)
    assert _rel(y, r) < 5e-3
    r.backward(torch.ones_like(r))
    dx = torch.empty_like(x)
    fused.gelu_bwd(x, torch.ones_like(x), dx)
    assert _rel(dx, xf.grad) < 1e-2


def test_cross_entropy_fused_gradient():
    from sensenova_u1_b200.ops import fused
    R, V = 37, 1000
    logits = _bf(R, V, seed=9, scale=2.0)
    labels = torch.randint(0, V, (R,), device=DEV).int()
    labels[3] = -100
    w = torch.rand(R, device=DEV)
    lf = logits.float().requires_grad_(True)
    valid = labels >= 0
    ref_rows = F.cross_entropy(lf[valid], labels[valid].long(), reduction="none")
    ref = (ref_rows * w[valid]).sum() * 0.25
    ref.backward()
    acc = torch.zeros(4, device=DEV)
    work = logits.clone()
    fused.ce_fwd_bwd(work, labels, w, 0.25, acc)
    assert abs(acc[0].item() * 0.25 - ref.item()) < 2e-3 * abs(ref.item())
    assert abs(acc[1].item() - w[valid].sum().item()) < 1e-4
    assert acc[3].item() == valid.sum().item()
    assert (acc[2].item() == (lf[valid].argmax(-1) == labels[valid]).sum().item())
    assert _rel(work, lf.grad) < 1e-2
    assert work[3].abs().max().item() == 0


def test_fm_loss_fused_gradient():
    from sensenova_u1_b200.ops import fused
    R, D = 20, 768
    xp = _bf(R, D, seed=10)
    z, v = torch.randn(R, D, device=DEV), torch.randn(R, D, device=DEV)
    t = torch.rand(R, device=DEV); t[0] = 0.99
    w = torch.rand(R, device=DEV)
    xf = xp.float().requires_grad_(True)
    den = (1 - t[:, None]).clamp_min(0.05)
    rows = (((xf - z) / den - v) ** 2).mean(1)
    ref = (rows * w).sum() * 0.5
    ref.backward()
    dx = torch.empty_like(xp); acc = torch.zeros(1, device=DEV); rl = torch.empty(R, device=DEV)
    fused.fm_loss(xp, z, v, t, w, 0.05, 0.5, dx, acc, rl)
    assert abs(acc.item() * 0.5 - ref.item()) < 1e-3 * abs(ref.item())
    assert _rel(rl, rows) < 1e-4
    assert _rel(dx, xf.grad) < 1e-2


def test_rope2d_and_colsum():
    from sensenova_u1_b200.models import oracle
    from sensenova_u1_b200.ops import fused
    P, C = 48, 64
    x = _bf(P, C, seed=11)
    px, py = torch.randint(0, 30, (P,), device=DEV).int(), torch.randint(0, 30, (P,), device=DEV).int()
    inv = (1.0 / (10000.0 ** (torch.arange(0, C // 2, 2, device=DEV).float() / (C // 2)))).contiguous()
    y = torch.empty_like(x)
    fused.rope2d(x, y, px, py, inv)
    assert _rel(y, oracle.rope2d(x.float(), px, py, 10000.0)) < 5e-3
    back = torch.empty_like(x)
    fused.rope2d(y, back, px, py, inv, inverse=True)
    assert _rel(back, x) < 1e-2
    out = torch.zeros(C, device=DEV)
    fused.colsum(x, out)
    assert _rel(out, x.float().sum(0)) < 1e-4


@pytest.mark.parametrize("state_dtype", [torch.float32, torch.bfloat16])
def test_adamw_master_split(state_dtype):
    from sensenova_u1_b200.ops import fused
    n = 8 * 1024
    w32 = torch.randn(n, device=DEV) * 0.1
    hi = torch.empty(n, dtype=torch.bfloat16, device=DEV); lo = torch.empty(n, dtype=torch.int16, device=DEV)
    fused.split_master(w32, hi, lo)
    back = torch.empty_like(w32)
    fused.join_master(hi, lo, back)
    assert torch.equal(back, w32)                       # the split is exact
    assert _rel(hi, w32) < 4e-3                         # and the bf16 half is the rounded weight
    g = _bf(n, seed=12, scale=0.01)
    m = torch.zeros(n, dtype=state_dtype, device=DEV); v = torch.zeros(n, dtype=state_dtype, device=DEV)
    ref = torch.nn.Parameter(w32.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    nsq = torch.zeros(1, device=DEV); skipped = torch.zeros(1, dtype=torch.int32, device=DEV)
    for step in range(1, 4):
        nsq.zero_()
        fused.sumsq(g, nsq)
        assert abs(nsq.item() - g.float().pow(2).sum().item()) < 1e-3 * nsq.item()
        coef = min(1.0, 0.5 / (math.sqrt(nsq.item()) + 1e-6))
        ref.grad = g.float() * coef
        opt.step()
        fused.adamw(hi, lo, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                    step=step, norm_sq=nsq, max_norm=0.5, skipped=skipped)
    fused.join_master(hi, lo, back)
    tol = 1e-5 if state_dtype == torch.float32 else 2e-3
    assert _rel(back, ref.data) < tol
    assert skipped.item() == 0
    nsq.fill_(float("inf"))
    before = back.clone()
    fused.adamw(hi, lo, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                step=4, norm_sq=nsq, max_norm=0.5, skipped=skipped)
    fused.join_master(hi, lo, back)
    assert skipped.item() == 1 and torch.equal(before, back)


@pytest.mark.parametrize("n,dtype", [(8 * 1000 + 3, torch.bfloat16), (4096, torch.float32), (5, torch.bfloat16)])
def test_sumsq_vector_body_and_scalar_tail(n, dtype):
    from sensenova_u1_b200.ops import fused
    g = torch.Generator(device="cuda").manual_seed(n)
    x = (torch.randn(n + 8, device="cuda", generator=g)).to(dtype)
    for view in (x[:n], x[8:8 + n], x[1:1 + n] if dtype == torch.float32 else x[8:8 + n]):   # aligned / offset starts
        out = torch.zeros(1, device="cuda")
        fused.sumsq(view, out)
        ref = view.float().pow(2).sum()
        assert abs(out.item() - ref.item()) < 1e-3 * ref.item() + 1e-6


def test_peer_flag_wait_runs_out_and_the_device_keeps_answering():
    """A wait on a flag that nobody sets, with a 50 ms limit given at launch: the kernel records the timeout in the
    status word and returns, ``check_status`` raises, and the context is still usable afterwards."""
    import time
    import torch
    from sensenova_u1_b200.ops import _lib
    from sensenova_u1_b200.ops._lib import c_int, c_ll, c_void_p
    _lib.load()
    _lib.check_status()
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    st = c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.time()
    _lib.call("wait_flags_limit", c_void_p(flags.data_ptr()), c_int(2), c_int(0), c_int(1), c_ll(50_000_000), st)
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    with pytest.raises(_lib.NativeLibraryError) as e:
        _lib.check_status()
    assert "peer flag" in str(e.value)
    _lib.check_status()                       # the status word was cleared by the read
    x = torch.arange(1024, device="cuda", dtype=torch.float32)
    assert float((x * 2).sum()) == 1023 * 1024.0      # the device still answers
    flags.fill_(1)                            # and the same wait returns at once when the flag is there
    _lib.call("wait_flags_limit", c_void_p(flags.data_ptr()), c_int(2), c_int(0), c_int(1), c_ll(50_000_000), st)
    _lib.check_status()
