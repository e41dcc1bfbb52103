"""The column-split Gemm whose epilogue stores into every GPU's result (sofie_b200_gemm_enqueue_peers).  Needs two GPUs."""
import json
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu

two_gpus = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@two_gpus
@pytest.mark.parametrize("flags", [0, 2], ids=["rows64", "rows128"])
def test_one_process_two_gpus_each_writes_its_columns_into_both_results(flags):
    from sofie_b200 import lib as L
    from sofie_b200.ops import Context, GemmPlan, make_epilogue
    M, N, K = 1000, 512, 256          # 1000 rows: the last 32-row segment is clipped by the tensor map
    bf = torch.bfloat16
    g = torch.Generator().manual_seed(7)
    a = (torch.randn(M, K, generator=g) * 0.5).to(bf)
    w = (torch.randn(N, K, generator=g) * 0.1).to(bf)
    bias = torch.randn(N, generator=g) * 0.1
    ctxs, ys, keep = [], [], []
    for d in range(2):
        torch.cuda.set_device(d)
        ctxs.append(Context(d))
        ys.append(torch.full((M, N), float("nan"), dtype=bf, device=f"cuda:{d}"))
    for d in range(2):
        ctxs[d].enable_peer(1 - d)
    torch.cuda.synchronize(0)
    torch.cuda.synchronize(1)
    n = N // 2
    for d in range(2):
        torch.cuda.set_device(d)
        n0 = d * n
        plan = GemmPlan(ctxs[d], M, n, K, bf, bf, trans_b=True, ldy=N, flags=flags)
        ep, k = make_epilogue(bias=bias[n0:n0 + n].contiguous().to(f"cuda:{d}"), act=L.ACT_GELU_ERF)
        ad, wd = a.to(f"cuda:{d}"), w[n0:n0 + n].contiguous().to(f"cuda:{d}")
        keep += [plan, k, ad, wd]
        plan.enqueue_peers(ad, wd, ys[d].data_ptr() + n0 * 2, [ys[1 - d].data_ptr() + n0 * 2], ep)
    for d in range(2):
        torch.cuda.set_device(d)
        ctxs[d].sync()
    ref = torch.nn.functional.gelu(a.float() @ w.float().t() + bias)
    for d in range(2):
        got = ys[d].float().cpu()
        assert not torch.isnan(got).any()                       # every element of both results was written
        assert ((got - ref).abs() <= 1e-2 + 2e-2 * ref.abs()).all()   # bf16 tolerance: 2e-2 relative + 1e-2 absolute
    assert torch.equal(ys[0].cpu(), ys[1].cpu())                # the two copies are the same bytes
    torch.cuda.set_device(0)


@two_gpus
def test_peer_stores_are_refused_for_int8_and_for_ragged_widths():
    from sofie_b200 import lib as L
    from sofie_b200.ops import Context, GemmPlan
    ctx = Context(0)
    a = torch.zeros(256, 128, dtype=torch.int8, device="cuda:0")
    w = torch.zeros(128, 128, dtype=torch.int8, device="cuda:0")
    y = torch.zeros(256, 128, dtype=torch.int8, device="cuda:0")
    plan = GemmPlan(ctx, 256, 128, 128, torch.int8, torch.int8, trans_b=True)
    with pytest.raises(RuntimeError, match="floating-point"):
        plan.enqueue_peers(a, w, y.data_ptr(), [y.data_ptr()], None)
    ab = torch.zeros(256, 128, dtype=torch.bfloat16, device="cuda:0")
    wb = torch.zeros(96, 128, dtype=torch.bfloat16, device="cuda:0")
    yb = torch.zeros(256, 96, dtype=torch.bfloat16, device="cuda:0")
    plan = GemmPlan(ctx, 256, 96, 128, torch.bfloat16, torch.bfloat16, trans_b=True)
    with pytest.raises(RuntimeError, match="multiple of 64"):
        plan.enqueue_peers(ab, wb, yb.data_ptr(), [yb.data_ptr()], None)


@two_gpus
def test_two_processes_hold_the_whole_result_after_one_kernel_each():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(ROOT / "tests" / "tp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    # (the two ranks' lines may arrive glued together: cut at the marker, not at line ends)
    lines = [json.JSONDecoder().raw_decode(part)[0] for part in r.stdout.split("TP_RESULT ")[1:]]
    assert sorted(x["rank"] for x in lines) == [0, 1]
    for x in lines:
        for case in x["cases"]:
            assert case["err_over_tol"] <= 1.0, case          # bf16 tolerance (2e-2 relative + 1e-2 absolute) = 1.0
            assert case["same"], case                         # call 3 reuses call 1's buffer and reproduces it bit for bit
            assert case["kernel"].startswith("umma"), case
