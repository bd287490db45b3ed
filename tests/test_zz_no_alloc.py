"""The allocation-free attention-backward entry point (csrc/snu1_noalloc.h).

Some users of the native library cannot allocate device memory where they need the
attention backward pass (a serving loop that must not hit cudaMalloc, a plugin that is
only handed pre-allocated buffers, a process whose allocator is locked after start-up).
For them the library exports ``snu1_attn_bwd_noalloc``: same inputs and outputs as
``snu1_attn_bwd``, but the delta scratch and the status word live in a fixed array inside
the library, so the call allocates nothing.

This test calls the exported C symbol directly through ctypes, twice in a row with
different data (the second call finds the first call's leftovers in the shared scratch),
and compares every gradient with the regular entry point, which gets caller-allocated
scratch.  Both run the same deterministic kernels, so the results must be identical; the
comparison still uses the tolerance of the other attention tests.  It also checks that a
problem larger than the built-in capacity is refused with a clear message.
"""
import ctypes
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_DELTA = 1 << 20


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _case(S, Hq, Hkv, seed, causal):
    from sensenova_u1_b200.ops import attention as A
    g = torch.Generator(device=DEV).manual_seed(seed)
    mk = lambda h: torch.randn(S, h, 128, device=DEV, generator=g).to(torch.bfloat16)
    q, k, v, do = mk(Hq), mk(Hkv), mk(Hkv), mk(Hq)
    idx = torch.arange(S, device=DEV)
    meta = A.make_meta(idx // 300 if not causal else torch.zeros_like(idx), idx)
    plan = A.build_plan(meta)
    o, lse = A.attention_fwd(q, k, v, plan, 128 ** -0.5)
    return q, k, v, o, do, lse, plan


def _call_noalloc(lib, q, k, v, o, do, lse, plan, scale, status, dq, dk, dv):
    Sq, Hq, _ = q.shape
    Sk, Hkv, _ = k.shape
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    LL = ctypes.c_longlong
    fn = lib.snu1_attn_bwd_noalloc
    fn.restype = ctypes.c_int
    rc = fn(P(q), LL(q.stride(0)), P(k), LL(k.stride(0)), P(v), LL(v.stride(0)), P(o), LL(o.stride(0)),
            P(do), LL(do.stride(0)), P(lse), P(dq), LL(dq.stride(0)), P(dk), LL(dk.stride(0)), P(dv),
            LL(dv.stride(0)), P(plan.meta_q), P(plan.meta_k), P(plan.kv_list), P(plan.kv_count),
            P(plan.q_list), P(plan.q_count), ctypes.c_int(Sq), ctypes.c_int(Sk), ctypes.c_int(Hq),
            ctypes.c_int(Hkv), ctypes.c_float(scale), P(status),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc


def test_noalloc_matches_regular_entry_point_twice():
    from sensenova_u1_b200.ops import _lib, attention as A
    lib = _lib.load()
    status = torch.full((1,), -1, dtype=torch.int32).pin_memory()
    scale = 128 ** -0.5
    for seed, (S, Hq, Hkv, causal) in enumerate([(1000, 8, 2, True), (700, 4, 4, False)]):
        q, k, v, o, do, lse, plan = _case(S, Hq, Hkv, seed, causal)
        ref = A.attention_bwd(q, k, v, o, do, lse, plan, scale)       # caller-allocated scratch
        dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
        if seed == 1:
            # second case = the entry point's second use on this device: its one-time set-up is behind it, so a raw
            # cudaMalloc inside the library (which PyTorch's counters cannot see) would show in the driver's free bytes
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
        gc.collect()      # tensors of earlier tests that a later collection would free must not move the counters
        before = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
        rc = _call_noalloc(lib, q, k, v, o, do, lse, plan, scale, status, dq, dk, dv)
        assert rc == 0, lib.snu1_last_error()
        torch.cuda.synchronize()
        assert status.item() == 0
        # the call took nothing from PyTorch's allocator either: outputs were made before it
        after = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
        assert after[0] <= before[0] and after[1] <= before[1], (before, after)
        if seed == 1:
            assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was allocated during the call"
        for got, want in zip((dq, dk, dv), ref):
            assert torch.isfinite(got.float()).all()
            assert _rel(got, want) < 1e-2
            assert torch.equal(got, want)


def test_noalloc_rejects_problems_beyond_capacity():
    from sensenova_u1_b200.ops import _lib
    lib = _lib.load()
    lib.snu1_last_error.restype = ctypes.c_char_p
    S, Hq = 8192 + 128, 128            # Hq * Sq > 2^20
    assert S * Hq > MAX_DELTA
    q = torch.zeros(1, device=DEV)     # never dereferenced: the size check comes first
    fn = lib.snu1_attn_bwd_noalloc
    fn.restype = ctypes.c_int
    P = ctypes.c_void_p(q.data_ptr())
    LL = ctypes.c_longlong
    rc = fn(P, LL(Hq * 128), P, LL(Hq * 128), P, LL(Hq * 128), P, LL(Hq * 128), P, LL(Hq * 128), P, P,
            LL(Hq * 128), P, LL(Hq * 128), P, LL(Hq * 128), P, P, P, P, P, P, ctypes.c_int(S),
            ctypes.c_int(S), ctypes.c_int(Hq), ctypes.c_int(Hq), ctypes.c_float(0.1), None, None)
    assert rc == -4
    assert b"exceeds the built-in scratch" in lib.snu1_last_error()
