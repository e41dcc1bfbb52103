"""One rank of the two-process test of the column-split Gemm (started by test_tp_gpu.py through torch.distributed.run).
Checks this rank's full-width result against a torch fp32 product of the same bf16 operands and prints one JSON line."""
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from sofie_b200 import lib as L
from sofie_b200 import replicas, tp
from sofie_b200.ops import Context, GemmPlan, make_epilogue


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rep = replicas.init_from_env("nccl")
    dev = torch.device("cuda", rep.local_rank)
    ctx = Context(rep.local_rank)
    bf = torch.bfloat16
    out = {"rank": rep.rank, "cases": []}
    for M, N, K, iters in ((4096 + 37, 1024, 512, 0), (65536, 2048, 512, 10), (8192, 8192, 8192, 5)):
        g = torch.Generator(device="cpu").manual_seed(1234 + M)          # the same operands on every rank
        a = (torch.randn(M, K, generator=g) * 0.5).to(bf).to(dev)
        w = (torch.randn(N, K, generator=g) * 0.05).to(bf).to(dev)
        cs = (torch.rand(N, generator=g) + 0.5).to(dev)
        bias = (torch.randn(N, generator=g) * 0.1).to(dev)
        split = tp.ColumnParallelGemm(ctx, M, N, K, bf, bf)
        n0, n = split.n0, split.n
        ep, keep = make_epilogue(col_scale=cs[n0:n0 + n].contiguous(), bias=bias[n0:n0 + n].contiguous(), act=L.ACT_RELU)
        w_shard = w[n0:n0 + n].contiguous()
        ys = [split(a, w_shard, ep).clone() for _ in range(3)]          # three calls: both buffers, and the first one again
        rows = slice(0, min(M, 2048))
        ref = torch.relu((a[rows].float() @ w.float().t()) * cs + bias)
        err = max(float(((y[rows].float() - ref).abs() / (1e-2 + 2e-2 * ref.abs())).max()) for y in ys)
        tail = torch.relu((a[-64:].float() @ w.float().t()) * cs + bias)
        err = max(err, float(((ys[-1][-64:].float() - tail).abs() / (1e-2 + 2e-2 * tail.abs())).max()))
        case = {"M": M, "N": N, "K": K, "kernel": split.plan.kernel, "err_over_tol": err, "same": bool(torch.equal(ys[0], ys[2]))}
        if iters:
            # device time of the fused kernel (max over ranks) beside the same shard without the peer stores
            def timed(fn):
                for _ in range(3):
                    fn()
                ctx.sync()
                dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(iters):
                    fn()
                e1.record()
                ctx.sync()
                torch.cuda.synchronize()
                return replicas.max_over_ranks(rep, e0.elapsed_time(e1) * 1e3 / iters)
            local = GemmPlan(ctx, M, n, K, bf, bf, trans_b=True, ldy=N)
            y_local = torch.empty(M, N, dtype=bf, device=dev)
            case["us_with_peer_stores"] = timed(lambda: split.enqueue(a, w_shard, ep))
            case["us_local_only"] = timed(lambda: local.enqueue(a, w_shard, y_local[:, n0:], ep))
            narrow = tp.ColumnParallelGemm(ctx, M, N, K, bf, bf, wide_stores=False)
            case["us_with_peer_stores_64_byte_rows"] = timed(lambda: narrow.enqueue(a, w_shard, ep))
            case["same_narrow"] = bool(torch.equal(narrow(a, w_shard, ep), ys[0]))
            narrow.close()
            case["peer_bytes"] = M * n * 2 * (rep.world - 1)
            local.close()
        out["cases"].append(case)
        split.close()
    print("\nTP_RESULT " + json.dumps(out) + "\n", flush=True)
    ctx.close()
    replicas.shutdown(rep)


if __name__ == "__main__":
    main()
