"""Times the fused compute+collective kernels against their NCCL + GEMM baselines.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m sensenova_u1_b200.parallel.bench_fused

Device-timed with CUDA events after warm-up, barrier + synchronize on both sides, max over ranks.
Shapes are the weight-parallel projections of the 8B model at 16384 tokens per rank.
"""
import json
import os
import sys

import torch
import torch.distributed as dist


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    dist.init_process_group("nccl", device_id=dev)
    from sensenova_u1_b200.ops import _lib, gemm
    from sensenova_u1_b200.parallel.fused_ops import AllGatherGemm, gemm_reduce_scatter
    from sensenova_u1_b200.parallel.symm import SymmetricBuffer

    def timed(fn, it=10, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(it):
            fn()
        e1.record()
        torch.cuda.synchronize(); dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / it], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    M = int(os.environ.get("BENCH_M", 16384))
    rows = []
    for name, N, K in (("w13", 24576, 4096), ("wqkv", 6144, 4096), ("w2", 4096, 12288)):
        if (N // world) % 256:
            continue
        sr = N // world
        sb = SymmetricBuffer(sr * K, torch.bfloat16, dev)
        sb.tensor.copy_((torch.randn(sr * K, device=dev) * 0.02).to(torch.bfloat16))
        x = (torch.randn(M, K, device=dev) * 0.5).to(torch.bfloat16)
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        full = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize(); dist.barrier()
        for ncopy in (4, 8, 16):
            op = AllGatherGemm(sb, sr, K, chunk_rows=256, num_copy_ctas=ncopy)
            t_f = timed(lambda: op(x, out=y))
            rows.append(dict(op="allgather+gemm fused", proj=name, copy_ctas=ncopy, ms=t_f))

        def base():
            dist.all_gather_into_tensor(full, sb.tensor.view(sr, K))
            gemm.gemm_nt(x, full, out=y)
        t_b = timed(base)
        t_g = timed(lambda: gemm.gemm_nt(x, full, out=y))
        flops = 2.0 * M * N * K
        wire = (world - 1) / world * N * K * 2
        roof = max(flops / 1368.6e12, wire / 770e9) * 1e3
        rows.append(dict(op="nccl all_gather then gemm", proj=name, ms=t_b))
        rows.append(dict(op="gemm only (weights local)", proj=name, ms=t_g, roofline_ms=roof))
        # weight-gradient GEMM + reduce-scatter: dW[N,K] = dy[M,N]^T x[M,K], rows of dW owned in blocks
        dy = (torch.randn(M, N, device=dev) * 0.1).to(torch.bfloat16)
        dst = SymmetricBuffer(sr * K, torch.float32, dev)
        torch.cuda.synchronize(); dist.barrier()
        t_rs = timed(lambda: gemm_reduce_scatter(dy, x, dst, sr, K, a_mn=True, b_mn=True), it=5)
        dwf = torch.empty(N, K, dtype=torch.float32, device=dev)
        outs = torch.empty(sr, K, dtype=torch.float32, device=dev)

        def base_rs():
            gemm.gemm_tn(dy, x, out=dwf)
            dist.reduce_scatter_tensor(outs, dwf)
        t_brs = timed(base_rs, it=5)
        rows.append(dict(op="wgrad gemm+reduce_scatter fused", proj=name, ms=t_rs,
                         roofline_ms=max(flops / 1368.6e12, (world - 1) / world * N * K * 4 / 770e9) * 1e3))
        rows.append(dict(op="wgrad gemm then nccl reduce_scatter(fp32)", proj=name, ms=t_brs))
        # staged form: bf16 partial rows stored into the owner's per-source slabs, summed by the owner
        from sensenova_u1_b200.parallel.fused_ops import GemmReduceScatter
        grs = GemmReduceScatter(None, dev, sr, K)
        outb = torch.empty(sr, K, dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize(); dist.barrier()
        t_st = timed(lambda: grs(dy, x, outb, a_mn=True, b_mn=True), it=5)
        dwb = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
        outsb = torch.empty(sr, K, dtype=torch.bfloat16, device=dev)

        def base_rs_bf16():
            gemm.gemm_tn(dy, x, out=dwb, out_mode=gemm.OUT_BF16_STORE)
            dist.reduce_scatter_tensor(outsb, dwb)
        t_bb = timed(base_rs_bf16, it=5)
        rows.append(dict(op="wgrad gemm+reduce_scatter staged (bf16 slabs, owner sums)", proj=name, ms=t_st,
                         roofline_ms=max(flops / 1368.6e12, (world - 1) / world * N * K * 2 / 770e9) * 1e3))
        rows.append(dict(op="wgrad gemm then nccl reduce_scatter(bf16)", proj=name, ms=t_bb))
        del sb, dst, dy, dwf, grs, outb, dwb, outsb
    _lib.check_status()
    if rank == 0:
        print(json.dumps({"world": world, "M": M, "rows": rows}, indent=1))
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
