"""GEMMs fused with their collective over NVLink peer memory (csrc/gemm_sm100.cu).

* :class:`AllGatherGemm` — ``y = x @ W^T`` with ``W`` split by rows over the ranks (the weight-parallel
  / ZeRO-3-like layout of the reference's ISP mode, training/sensenovalm/model/modules/linear.py:169-229,
  core/parallel/comm/isp.py:548-582).  One kernel: a few CTAs stream every rank's shard into a local
  staging buffer with bulk TMA copies while the other CTAs already multiply the shards that have landed,
  local shard first, ring order after that.
* :func:`gemm_reduce_scatter` — a product whose rows are owned by ranks in equal blocks; every output tile
  is added into its owner's fp32 buffer from the GEMM epilogue (peer ``red.global.add``).  Serves the
  weight-gradient reduce-scatter of weight parallelism (linear.py:265-290, isp.py:805-850) and the
  row-parallel output reduce-scatter of tensor / sequence parallelism (core/parallel/comm/tensor.py:148-217).

The NCCL equivalents (all_gather_into_tensor + GEMM, GEMM + reduce_scatter_tensor) are the baselines
these are measured against in ``tests/test_multigpu_gpu.py`` and ``profiles/``.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import c_float, c_int, c_ll, c_void_p
from .symm import SymmetricBuffer


class AllGatherGemm:
    def __init__(self, shard: SymmetricBuffer, shard_rows: int, K: int, chunk_rows: int = 256, num_copy_ctas: int = 8):
        self.shard, self.shard_rows, self.K = shard, shard_rows, K
        self.world, self.rank = shard.world, shard.rank
        self.chunk_rows, self.num_copy_ctas = chunk_rows, num_copy_ctas
        dev = shard.tensor.device
        self.N = self.world * shard_rows
        self.staging = torch.empty(self.N, K, dtype=torch.bfloat16, device=dev)
        self.flags = torch.zeros(self.N // chunk_rows, dtype=torch.int32, device=dev)
        self.seq = 0

    def __call__(self, x: torch.Tensor, out=None, residual=None) -> torch.Tensor:
        M, K = x.shape
        assert K == self.K and x.dtype == torch.bfloat16 and x.stride(1) == 1
        if out is None:
            out = torch.empty(M, self.N, dtype=torch.bfloat16, device=x.device)
        self.seq += 1
        _lib.call("gemm_allgather_bf16", c_void_p(x.data_ptr()), c_ll(x.stride(0)), c_int(M), c_int(K),
                  self.shard.c_ptrs, c_int(self.world), c_int(self.rank), c_int(self.shard_rows),
                  c_void_p(self.staging.data_ptr()), c_void_p(self.flags.data_ptr()), c_int(self.seq),
                  c_int(self.chunk_rows), c_int(self.num_copy_ctas), c_void_p(out.data_ptr()), c_ll(out.stride(0)),
                  c_int(0), c_void_p(_lib.ptr(residual)), c_ll(0 if residual is None else residual.stride(0)),
                  c_void_p(_lib.stream()))
        return out


def gemm_reduce_scatter(a: torch.Tensor, b: torch.Tensor, dst: SymmetricBuffer, rs_rows: int, ldc: int,
                        a_mn: bool = False, b_mn: bool = False, alpha: float = 1.0) -> None:
    """Adds this rank's product into the owners' buffers ``dst`` (fp32 [rs_rows, ldc] per rank).
    ``a_mn=b_mn=False``: C = a[M,K] @ b[N,K]^T;  ``a_mn=b_mn=True``: C = a[S,M]^T @ b[S,N] (weight gradient)."""
    if a_mn:
        S, M = a.shape
        N = b.shape[1]
        K, a_rows, b_rows = S, S, S
    else:
        M, K = a.shape
        N = b.shape[0]
        a_rows, b_rows = M, N
    _lib.call("gemm_reducescatter_bf16", c_void_p(a.data_ptr()), c_void_p(b.data_ptr()), c_int(M), c_int(N), c_int(K),
              c_ll(a.stride(0)), c_ll(b.stride(0)), c_int(int(a_mn)), c_int(int(b_mn)), dst.c_ptrs,
              c_int(dst.world), c_int(rs_rows), c_ll(ldc), c_float(alpha), c_ll(a_rows), c_ll(b_rows),
              c_void_p(_lib.stream()))


class GemmReduceScatter:
    """Staged fused GEMM + reduce-scatter: every rank stores its bf16 partial rows straight from the GEMM
    epilogue into its slab of the owning rank's staging buffer (plain 16-byte peer stores, no atomics,
    half the wire bytes of the fp32 form above); after a device-side flag barrier the owner sums its
    ``world`` slabs into the output.  Reference counterpart: the GEMM followed by ``reduce_scatter`` of
    the weight-parallel / sequence-parallel linears (training/sensenovalm/model/modules/linear.py:51-163)."""

    def __init__(self, group, device, rs_rows: int, ldc: int):
        import torch.distributed as dist
        from .symm import FlagBarrier
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.rs_rows, self.ldc = rs_rows, ldc
        # two staging sets: a fast rank may already store the next product while a slow one still sums this one
        self.stage = [SymmetricBuffer(self.world * rs_rows * ldc, torch.bfloat16, device, self.group) for _ in range(2)]
        self.bar = FlagBarrier(self.group, device)
        self.calls = 0

    def __call__(self, a, b, out, a_mn: bool = False, b_mn: bool = False, alpha: float = 1.0, accumulate: bool = False):
        """out ([rs_rows, ldc] fp32 or bf16, this rank's rows) (+)= rows of sum over ranks of the product."""
        if a_mn:
            S, M = a.shape
            N = b.shape[1]
            K, a_rows, b_rows = S, S, S
        else:
            M, K = a.shape
            N = b.shape[0]
            a_rows, b_rows = M, N
        st = self.stage[self.calls & 1]
        self.calls += 1
        _lib.call("gemm_reducescatter_staged_bf16", c_void_p(a.data_ptr()), c_void_p(b.data_ptr()), c_int(M), c_int(N),
                  c_int(K), c_ll(a.stride(0)), c_ll(b.stride(0)), c_int(int(a_mn)), c_int(int(b_mn)), st.c_ptrs,
                  c_int(self.world), c_int(self.rank), c_int(self.rs_rows), c_ll(self.ldc), c_float(alpha),
                  c_ll(a_rows), c_ll(b_rows), c_void_p(_lib.stream()))
        self.bar.barrier()
        _lib.call("sum_slabs", c_void_p(st.tensor.data_ptr()), c_int(self.world), c_ll(self.rs_rows * self.ldc),
                  c_void_p(out.data_ptr()), c_int(1 if out.dtype == torch.float32 else 0), c_int(int(accumulate)),
                  c_void_p(_lib.stream()))
        return out
