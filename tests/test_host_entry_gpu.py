"""The host-operand entry points of the C ABI (sofie_b200_gemm_run_host, sofie_b200_gemm_run_host_many) against the CPU
checker: int8, bit for bit."""
import numpy as np
import pytest
import torch

from oracle_api import Oracle
from sofie_b200 import lib as L

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("pinned", [True, False])
def test_run_host_many_matches_checker(b200_lib, oracle_lib, pinned):
    from sofie_b200.ops import Context, GemmPlan, make_epilogue
    o = Oracle(oracle_lib)
    ctx = Context(0)
    M, N, K, count = 300, 264, 512, 5
    rng = np.random.default_rng(4)
    mult = 3e-4
    plan = GemmPlan(ctx, M, N, K, torch.int8, torch.int8)
    ep, keep = make_epilogue(alpha=mult)
    hold = (lambda t: t.pin_memory()) if pinned else (lambda t: t)
    As = [hold(torch.from_numpy(rng.integers(-127, 128, size=(M, K), dtype=np.int8))) for _ in range(count)]
    Bs = [hold(torch.from_numpy(rng.integers(-127, 128, size=(K, N), dtype=np.int8))) for _ in range(count)]
    Bs[3] = Bs[1]                                   # a pointer may repeat
    Ys = [hold(torch.zeros((M, N), dtype=torch.int8)) for _ in range(count)]
    n0 = ctx.launches
    plan.run_host_many(As, Bs, Ys, ep)
    assert ctx.launches - n0 == count
    for a, b, y in zip(As, Bs, Ys):
        want = o.gemm(a.numpy(), b.numpy(), M, N, K, L.I8, L.I8, ep=o.epilogue(alpha=mult))
        assert np.array_equal(y.numpy(), want)
    # the one-inference call afterwards (it shares the first staging set), then an empty and a one-entry queue
    y1 = hold(torch.zeros((M, N), dtype=torch.int8))
    plan.run_host(As[2], Bs[2], y1, ep)
    assert torch.equal(y1, Ys[2])
    plan.run_host_many([], [], [], ep)
    y2 = hold(torch.zeros((M, N), dtype=torch.int8))
    plan.run_host_many([As[4]], [Bs[4]], [y2], ep)
    assert torch.equal(y2, Ys[4])
    plan.close()
    ctx.close()
