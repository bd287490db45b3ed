"""Python face of ``mot_gemm`` (csrc/gemm_sm100.cu): bf16 tcgen05 GEMM with
K-major or MN-major operands and per-tile / per-range grouping.

The three products of a linear layer ``y = x W^T`` run on the row-major tensors
as stored (reference call sites: training/sensenovalm/model/ops/linear.py:108-165,
training/sensenovalm/model/modules/linear.py:169-295):

    forward   y  = x  W^T      gemm_nt(x, W)
    dgrad     dx = dy W        gemm_nn(dy, W)
    wgrad     dW = dy^T x      gemm_tn(dy, x)
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import c_float, c_int, c_ll, c_void_p

OUT_BF16_STORE, OUT_BF16_ACC, OUT_F32_STORE, OUT_F32_ACC = 0, 1, 2, 3


def set_pair_mode(on: bool) -> bool:
    """Selects the kernel for products without a fused collective: the two-SM pair kernel
    (tcgen05 ``cta_group::2``, 256x256 tiles; default) or the single-CTA kernel (128x256 tiles).
    Returns the previous setting."""
    lib = _lib.load()
    return bool(lib.snu1_gemm_set_pair_mode(c_int(1 if on else 0)))


def _check(t: torch.Tensor, name: str):
    if not t.is_cuda or t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be a CUDA bf16 tensor")
    if t.stride(-1) != 1:
        raise ValueError(f"{name} must have a contiguous last dimension")


def _raw(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, group_mode, num_groups, tile_group,
         k_begin, k_end, b_group_stride, c_group_stride, out_mode, residual, ldr, alpha,
         a_rows, b_rows):
    _lib.call(
        "gemm_bf16", c_void_p(A.data_ptr()), c_void_p(B.data_ptr()), c_void_p(C.data_ptr()),
        c_int(M), c_int(N), c_int(K), c_ll(lda), c_ll(ldb), c_ll(ldc), c_int(a_mn), c_int(b_mn),
        c_int(group_mode), c_int(num_groups),
        c_void_p(_lib.ptr(tile_group)), c_void_p(_lib.ptr(k_begin)), c_void_p(_lib.ptr(k_end)),
        c_ll(b_group_stride), c_ll(c_group_stride), c_int(out_mode),
        c_void_p(_lib.ptr(residual)), c_ll(ldr), c_float(alpha), c_ll(a_rows), c_ll(b_rows),
        c_void_p(_lib.stream()))


def _ldr(residual):
    if residual is None:
        return 0
    return 0 if residual.dim() == 1 else residual.stride(0)   # 1-D: a bias broadcast over rows


def _check_out(C, rows, N, out_mode):
    """The kernel writes ``rows x N`` elements of the output mode's type: a caller-provided buffer of
    another type or size would be overrun, so it is refused here."""
    want = torch.bfloat16 if out_mode <= 1 else torch.float32
    if C.dtype != want:
        raise ValueError(f"output buffer is {C.dtype} but out_mode {out_mode} writes {want}")
    if C.shape[-1] < N or C.shape[-2] < rows or C.stride(-1) != 1:
        raise ValueError(f"output buffer {tuple(C.shape)} cannot hold a {rows} x {N} result")


def _out(C, rows, N, out_mode, device):
    if C is None:
        dt = torch.bfloat16 if out_mode <= 1 else torch.float32
        C = torch.empty(rows, N, dtype=dt, device=device)
    else:
        _check_out(C, rows, N, out_mode)
    return C


def _raw_rows(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, grouped, G, tile_group, bgs, out_mode, alpha, a_rows,
              b_rows, rows_dev):
    _lib.call("gemm_bf16_rows", c_void_p(A.data_ptr()), c_void_p(B.data_ptr()), c_void_p(C.data_ptr()), c_int(M),
              c_int(N), c_int(K), c_ll(lda), c_ll(ldb), c_ll(ldc), c_int(a_mn), c_int(b_mn), c_int(1 if grouped else 0),
              c_int(G), c_void_p(None if tile_group is None else tile_group.data_ptr()), c_ll(bgs), c_int(out_mode),
              c_float(alpha), c_ll(a_rows), c_ll(b_rows), c_void_p(rows_dev.data_ptr()), c_void_p(_lib.stream()))


def gemm_nt(x, w, out=None, *, tile_group=None, residual=None, out_mode=OUT_BF16_STORE, alpha=1.0, rows_dev=None):
    """``out[M,N] = x[M,K] @ w[(G,)N,K]^T``; ``tile_group[M/128]`` picks the weight set.
    ``rows_dev`` (int32 device scalar): only that many rows of ``x`` / ``out`` are in use."""
    _check(x, "x"); _check(w, "w")
    M, K = x.shape
    grouped = w.dim() == 3
    G = w.shape[0] if grouped else 1
    N = w.shape[-2]
    assert w.shape[-1] == K
    if grouped and tile_group is None:
        raise ValueError("grouped weights need tile_group")
    out = _out(out, M, N, out_mode, x.device)
    if rows_dev is not None:
        assert residual is None
        _raw_rows(x, w, out, M, N, K, x.stride(0), w.stride(-2), out.stride(0), 0, 0, grouped, G, tile_group,
                  w.stride(0) if grouped else 0, out_mode, alpha, M, N, rows_dev)
        return out
    _raw(x, w, out, M, N, K, x.stride(0), w.stride(-2), out.stride(0), 0, 0,
         1 if grouped else 0, G, tile_group, None, None,
         w.stride(0) if grouped else 0, 0, out_mode, residual,
         _ldr(residual), alpha, M, N)
    return out


def gemm_nn(dy, w, out=None, *, tile_group=None, residual=None, out_mode=OUT_BF16_STORE, alpha=1.0, rows_dev=None):
    """``out[M,Kin] = dy[M,Nout] @ w[(G,)Nout,Kin]``  (w is read MN-major)."""
    _check(dy, "dy"); _check(w, "w")
    M, Nout = dy.shape
    grouped = w.dim() == 3
    G = w.shape[0] if grouped else 1
    assert w.shape[-2] == Nout
    Kin = w.shape[-1]
    if grouped and tile_group is None:
        raise ValueError("grouped weights need tile_group")
    out = _out(out, M, Kin, out_mode, dy.device)
    if rows_dev is not None:
        assert residual is None
        _raw_rows(dy, w, out, M, Kin, Nout, dy.stride(0), w.stride(-2), out.stride(0), 0, 1, grouped, G, tile_group,
                  w.stride(0) if grouped else 0, out_mode, alpha, M, Nout, rows_dev)
        return out
    _raw(dy, w, out, M, Kin, Nout, dy.stride(0), w.stride(-2), out.stride(0), 0, 1,
         1 if grouped else 0, G, tile_group, None, None,
         w.stride(0) if grouped else 0, 0, out_mode, residual,
         _ldr(residual), alpha, M, Nout)
    return out


def gemm_tn(dy, x, out=None, *, k_begin=None, k_end=None, num_groups=1,
            out_mode=OUT_F32_STORE, alpha=1.0):
    """``out[(G,)Nout,Kin] = dy[S,Nout]^T @ x[S,Kin]``; with ``k_begin/k_end``
    (device int32 ``[G]``) output ``g`` reduces over rows ``[k_begin[g], k_end[g])``."""
    _check(dy, "dy"); _check(x, "x")
    S, Nout = dy.shape
    assert x.shape[0] == S
    Kin = x.shape[1]
    grouped = k_begin is not None
    G = num_groups if grouped else 1
    if out is None:
        dt = torch.bfloat16 if out_mode <= 1 else torch.float32
        shape = (G, Nout, Kin) if grouped else (Nout, Kin)
        out = torch.empty(*shape, dtype=dt, device=dy.device)
    else:
        _check_out(out, Nout, Kin, out_mode)
        if grouped and (out.dim() != 3 or out.shape[0] < G):
            raise ValueError(f"grouped weight gradient needs an output of {G} groups, got {tuple(out.shape)}")
    ldc = out.stride(-2)
    cgs = out.stride(0) if grouped else 0
    _raw(dy, x, out, Nout, Kin, S, dy.stride(0), x.stride(0), ldc, 1, 1,
         2 if grouped else 0, G, None, k_begin, k_end, 0, cgs, out_mode, None, 0, alpha, S, S)
    return out
