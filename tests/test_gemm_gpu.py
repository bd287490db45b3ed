"""mot_gemm (tcgen05) against an fp32 PyTorch product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["pair", "single"])
def kernel_variant(request):
    """Every test runs on the two-SM pair kernel and on the single-CTA kernel."""
    from sensenova_u1_b200.ops import gemm
    old = gemm.set_pair_mode(request.param == "pair")
    yield request.param
    gemm.set_pair_mode(old)


def _rel_err(got, ref):
    return ((got.float() - ref).norm() / (ref.norm() + 1e-12)).item()


def _tile_err(got, ref, tm=128, tn=256):
    """Worst relative error of one output tile (a wrong tile hardly moves the whole-matrix norm) and the largest
    absolute error in units of the reference's largest magnitude (bf16 output rounding alone: up to 2^-8)."""
    d = got.float() - ref
    M, N = ref.shape
    Mp, Np = (M + tm - 1) // tm * tm, (N + tn - 1) // tn * tn
    pad = lambda t: torch.nn.functional.pad(t, (0, Np - N, 0, Mp - M))
    tiles = lambda t: pad(t).view(Mp // tm, tm, Np // tn, tn).pow(2).sum((1, 3)).sqrt()
    worst = (tiles(d) / (tiles(ref) + 1e-6 * ref.norm())).max().item()
    return worst, (d.abs().max() / ref.abs().max()).item()


def _mk(*shape, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * 0.5).to(torch.bfloat16)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 1024, 1088), (200, 264, 72),
                                   (1024, 4096, 4096), (4096, 4096, 512), (2944, 1280, 192)])
def test_nt(M, N, K):
    from sensenova_u1_b200.ops import _lib, gemm
    x, w = _mk(M, K, seed=1), _mk(N, K, seed=2)
    out = gemm.gemm_nt(x, w)
    _lib.check_status()
    ref = x.float() @ w.float().t()
    assert _rel_err(out, ref) < 1e-2
    worst_tile, max_abs = _tile_err(out, ref)
    assert worst_tile < 1e-2 and max_abs < 1e-2, (worst_tile, max_abs)      # bf16 output rounding: 2^-9 relative


def test_nt_at_training_size():
    """The fused gate/up projection of the 8B model at 16,384 rows (the largest product of the training step)."""
    from sensenova_u1_b200.ops import _lib, gemm
    M, N, K = 16384, 24576, 4096
    x, w = _mk(M, K, seed=11), _mk(N, K, seed=12)
    out = gemm.gemm_nt(x, w)
    _lib.check_status()
    torch.backends.cuda.matmul.allow_tf32 = False
    for r0 in (0, 8192, M - 2048):                       # fp32 reference in row slabs (1.6 GB for the whole product)
        ref = x[r0:r0 + 2048].float() @ w.float().t()
        worst_tile, max_abs = _tile_err(out[r0:r0 + 2048], ref)
        assert worst_tile < 1e-2 and max_abs < 1e-2, (r0, worst_tile, max_abs)


def test_output_beyond_two_to_the_31_elements():
    """An output of 16,384 x 151,936 (the vocabulary head at training size): element offsets pass 2^31."""
    from sensenova_u1_b200.ops import _lib, gemm
    M, N, K = 16384, 151936, 256
    assert M * N > 2 ** 31
    x, w = _mk(M, K, seed=13), _mk(N, K, seed=14)
    out = gemm.gemm_nt(x, w)
    _lib.check_status()
    for r0 in (0, 14080, M - 256):                       # 14,135 is the first row whose elements sit past 2^31
        ref = x[r0:r0 + 256].float() @ w.float().t()
        worst_tile, max_abs = _tile_err(out[r0:r0 + 256], ref)
        assert worst_tile < 1e-2 and max_abs < 1e-2, (r0, worst_tile, max_abs)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (200, 264, 72), (512, 4096, 1024)])
def test_nn(M, N, K):
    from sensenova_u1_b200.ops import _lib, gemm
    dy, w = _mk(M, K, seed=3), _mk(K, N, seed=4)   # out[M,N] = dy[M,K] @ w[K,N]
    out = gemm.gemm_nn(dy, w)
    _lib.check_status()
    ref = dy.float() @ w.float()
    assert _rel_err(out, ref) < 1e-2


@pytest.mark.parametrize("S,No,Ki", [(64, 128, 256), (256, 256, 512), (1000, 264, 200), (2048, 1024, 4096)])
def test_tn(S, No, Ki):
    from sensenova_u1_b200.ops import _lib, gemm
    dy, x = _mk(S, No, seed=5), _mk(S, Ki, seed=6)
    out = gemm.gemm_tn(dy, x)
    _lib.check_status()
    ref = dy.float().t() @ x.float()
    assert out.dtype == torch.float32
    assert _rel_err(out, ref) < 1e-2


def test_grouped_rows_and_residual():
    from sensenova_u1_b200.ops import _lib, gemm
    M, N, K, G = 640, 512, 320, 2
    x, w, res = _mk(M, K, seed=7), _mk(G, N, K, seed=8), _mk(M, N, seed=9)
    tg = torch.tensor([0, 0, 1, -1, 1], dtype=torch.int32, device="cuda")
    out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    gemm.gemm_nt(x, w, out=out, tile_group=tg, residual=res)
    _lib.check_status()
    ref = torch.zeros(M, N, device="cuda")
    for t, g in enumerate(tg.tolist()):
        if g >= 0:
            r = slice(t * 128, (t + 1) * 128)
            ref[r] = x[r].float() @ w[g].float().t() + res[r].float()
    assert _rel_err(out, ref) < 1e-2
    assert out[384:512].abs().max().item() == 0  # skipped tile untouched
    dx = gemm.gemm_nn(out, w, tile_group=tg)  # [M,N] @ [G,N,K]
    _lib.check_status()
    refdx = torch.zeros(M, K, device="cuda")
    for t, g in enumerate(tg.tolist()):
        if g >= 0:
            r = slice(t * 128, (t + 1) * 128)
            refdx[r] = out[r].float() @ w[g].float()
    got = dx.float()
    got[384:512] = 0
    assert _rel_err(got, refdx) < 1e-2


def test_grouped_wgrad_and_accumulate():
    from sensenova_u1_b200.ops import _lib, gemm
    S, No, Ki = 768, 256, 384
    dy, x = _mk(S, No, seed=10), _mk(S, Ki, seed=11)
    kb = torch.tensor([0, 256, 768], dtype=torch.int32, device="cuda")
    ke = torch.tensor([256, 768, 768], dtype=torch.int32, device="cuda")
    out = gemm.gemm_tn(dy, x, k_begin=kb, k_end=ke, num_groups=3)
    _lib.check_status()
    for g, (b, e) in enumerate(zip(kb.tolist(), ke.tolist())):
        ref = dy[b:e].float().t() @ x[b:e].float()
        if e > b:
            assert _rel_err(out[g], ref) < 1e-2
        else:
            assert out[g].abs().max().item() == 0
    before = out.clone()
    gemm.gemm_tn(dy, x, out=out, k_begin=kb, k_end=ke, num_groups=3, out_mode=gemm.OUT_F32_ACC)
    _lib.check_status()
    assert _rel_err(out, 2 * before) < 1e-5


def test_deterministic():
    from sensenova_u1_b200.ops import gemm
    x, w = _mk(512, 1024, seed=12), _mk(768, 1024, seed=13)
    a = gemm.gemm_nt(x, w)
    b = gemm.gemm_nt(x, w)
    assert torch.equal(a, b)


def test_output_buffer_must_match_the_output_mode():
    from sensenova_u1_b200.ops import gemm
    a = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        gemm.gemm_tn(a, b, out=torch.empty(64, 64, dtype=torch.bfloat16, device="cuda"))          # default mode is fp32
    with pytest.raises(ValueError):
        gemm.gemm_nt(a, b, out=torch.empty(128, 64, dtype=torch.bfloat16, device="cuda"))         # too few columns
    with pytest.raises(ValueError):
        gemm.gemm_nt(a, b, out=torch.empty(128, 128, dtype=torch.float32, device="cuda"))


def test_many_groups_with_odd_tile_runs_and_row_bound():
    """Expert-style grouping: runs of 1..3 row tiles per weight set (pairs of tiles straddle sets), skipped
    tiles, and a device-side bound on the rows in use."""
    from sensenova_u1_b200.ops import _lib, gemm
    G, N, K = 5, 384, 256
    tgl = [0, 1, 1, 1, 2, -1, 3, 3, 4, 4, 4, 0, 2]
    M = 128 * len(tgl)
    x, w = _mk(M, K, seed=21), _mk(G, N, K, seed=22)
    tg = torch.tensor(tgl, dtype=torch.int32, device="cuda")
    ref = torch.zeros(M, N, device="cuda")
    for t, g in enumerate(tgl):
        if g >= 0:
            r = slice(t * 128, (t + 1) * 128)
            ref[r] = x[r].float() @ w[g].float().t()
    out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    gemm.gemm_nt(x, w, out=out, tile_group=tg)
    _lib.check_status()
    assert _rel_err(out, ref) < 1e-2
    used = 128 * 7 + 40          # the bound falls inside tile 7
    rows = torch.tensor([used], dtype=torch.int32, device="cuda")
    out2 = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    gemm.gemm_nt(x, w, out=out2, tile_group=tg, rows_dev=rows)
    _lib.check_status()
    assert _rel_err(out2[:128 * 8], ref[:128 * 8]) < 1e-2
    assert out2[128 * 8:].abs().max().item() == 0     # tiles past the bound are not visited
