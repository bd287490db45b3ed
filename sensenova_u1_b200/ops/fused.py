"""Thin Python faces of the memory-bound sm_100a kernels (csrc/elementwise.cu,
csrc/losses.cu, csrc/optim.cu).  All of them work in place on caller-provided
buffers; shapes are checked here, alignment by the native side."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import c_float, c_int, c_ll, c_void_p

P = lambda t: c_void_p(_lib.ptr(t))
ST = lambda: c_void_p(_lib.stream())


def rmsnorm_fwd(x, gain, tile_group, out, rstd, eps):
    rows, H = x.shape
    _lib.call("rmsnorm_fwd", P(x), P(gain), P(tile_group), P(out), P(rstd), c_int(rows), c_int(H),
              c_float(eps), ST())
    return out


def rmsnorm_bwd(dy, x, gain, rstd, tile_group, dres, dx, dgain):
    rows, H = x.shape
    _lib.call("rmsnorm_bwd", P(dy), P(x), P(gain), P(rstd), P(tile_group), P(dres), P(dx), P(dgain),
              c_int(rows), c_int(H), ST())
    return dx


def qknorm_rope_fwd(qkv, out, gains, tile_group, pos3, inv_t, inv_hw, n_q, n_kv, eps):
    rows = qkv.shape[0]
    _lib.call("qknorm_rope_fwd", P(qkv), c_ll(qkv.stride(0)), P(out), c_ll(out.stride(0)), P(gains),
              P(tile_group), P(pos3), P(inv_t), P(inv_hw), c_int(rows), c_int(n_q), c_int(n_kv),
              c_float(eps), ST())
    return out


def qknorm_rope_bwd(qkv, d, gains, dgains, tile_group, pos3, inv_t, inv_hw, n_q, n_kv, eps):
    rows = qkv.shape[0]
    _lib.call("qknorm_rope_bwd", P(qkv), c_ll(qkv.stride(0)), P(d), c_ll(d.stride(0)), P(gains),
              P(dgains), P(tile_group), P(pos3), P(inv_t), P(inv_hw), c_int(rows), c_int(n_q),
              c_int(n_kv), c_float(eps), ST())
    return d


def swiglu_fwd(gu, act, rows_dev=None):
    """``rows_dev``: optional int32 device scalar, only that many rows are in use (buffers sized for a
    worst case whose fill is known on the device only)."""
    rows, F2 = gu.shape
    _lib.call("swiglu_fwd_dyn", P(gu), P(act), c_ll(rows), c_int(F2 // 2), P(rows_dev), ST())
    return act


def swiglu_bwd(gu, dact, dgu, rows_dev=None):
    rows, F2 = gu.shape
    _lib.call("swiglu_bwd_dyn", P(gu), P(dact), P(dgu), c_ll(rows), c_int(F2 // 2), P(rows_dev), ST())
    return dgu


def ce_fwd_bwd(logits, labels, weights, grad_scale, loss_out, row_loss=None):
    """Overwrites ``logits`` [R,V] (bf16) with d loss / d logits; ``loss_out`` [4] fp32
    accumulates (weighted loss sum, weight sum, correct top-1 count, valid rows)."""
    rows, V = logits.shape
    _lib.call("ce_fwd_bwd", P(logits), c_ll(logits.stride(0)), P(labels), P(weights),
              c_float(grad_scale), P(loss_out), P(row_loss), c_int(rows), c_int(V), ST())


def fm_loss(x_pred, z, v_tgt, t, w, t_eps, grad_scale, dx, loss_out, row_loss=None):
    rows, D = x_pred.shape
    _lib.call("fm_loss", P(x_pred), P(z), P(v_tgt), P(t), P(w), c_float(t_eps), c_float(grad_scale),
              P(dx), P(loss_out), P(row_loss), c_int(rows), c_int(D), ST())


def gelu_fwd(x, y):
    _lib.call("gelu_fwd", P(x), P(y), c_ll(x.numel()), ST())
    return y


def gelu_bwd(x, dy, dx):
    _lib.call("gelu_bwd", P(x), P(dy), P(dx), c_ll(x.numel()), ST())
    return dx


def colsum(x, out):
    rows, cols = x.shape
    _lib.call("colsum", P(x), c_ll(x.stride(0)), P(out), c_int(rows), c_int(cols), ST())


def rope2d(x, y, px, py, inv_freq, inverse=False):
    rows, C = x.shape
    _lib.call("rope2d", P(x), P(y), P(px), P(py), P(inv_freq), c_int(rows), c_int(C),
              c_int(1 if inverse else 0), ST())
    return y


def sumsq(g, out):
    _lib.call("sumsq", P(g), c_ll(g.numel()), c_int(0 if g.dtype == torch.bfloat16 else 1), P(out), ST())


def adamw(p_hi, p_lo, g, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_prescale=1.0,
          norm_sq=None, max_norm=0.0, skipped=None):
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    _lib.call("adamw", P(p_hi), P(p_lo), P(g), P(m), P(v), c_ll(p_hi.numel()),
              c_int(0 if g.dtype == torch.bfloat16 else 1), c_int(0 if m.dtype == torch.bfloat16 else 1),
              c_float(lr), c_float(beta1), c_float(beta2), c_float(eps), c_float(weight_decay),
              c_float(bc1), c_float(bc2), c_float(grad_prescale), P(norm_sq), c_float(max_norm),
              P(skipped), ST())


def ema(ema_buf, p_hi, p_lo, decay):
    _lib.call("ema", P(ema_buf), P(p_hi), P(p_lo), c_ll(ema_buf.numel()), c_float(decay), ST())


def split_master(w32, hi, lo):
    _lib.call("split_master", P(w32), P(hi), P(lo), c_ll(w32.numel()), ST())


def join_master(hi, lo, w32):
    _lib.call("join_master", P(hi), P(lo), P(w32), c_ll(w32.numel()), ST())


# ---- convolutional pixel head (csrc/pixel_head.cu) ---------------------------------------------------------
def ps_im2col(x, A, h: int, w: int, C: int):
    """Pixel-shuffle(2) + 3x3 patch gather: x [h*w, 4C] -> A [(2h)(2w), 9C] (tap-major, channel-minor columns)."""
    _lib.call("ps_im2col", P(x), P(A), c_int(h), c_int(w), c_int(C), ST())
    return A


def ps_col2im(dA, dx, h: int, w: int, C: int, accumulate: bool = False):
    """Adjoint of :func:`ps_im2col`: dA [(2h)(2w), 9C] -> dx [h*w, 4C]."""
    _lib.call("ps_col2im", P(dA), P(dx), c_int(h), c_int(w), c_int(C), c_int(1 if accumulate else 0), ST())
    return dx


def pixel_regroup(y, tok, h: int, w: int, r: int, to_y: bool = False):
    """Last pixel shuffle + token blocking: y [(4h)(4w), 3 r r] <-> tok [h*w, (4r)(4r) 3] ((row, column, channel))."""
    _lib.call("pixel_regroup", P(y), P(tok), c_int(h), c_int(w), c_int(r), c_int(1 if to_y else 0), ST())
    return y if to_y else tok
