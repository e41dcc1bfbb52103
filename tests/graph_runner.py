"""Runs the small ONNX graphs of the golden fixtures on one of two backends.

Test infrastructure.  `OracleBackend` evaluates every operator with the CPU restatement
(oracle/libsofie_oracle.so); `B200Backend` evaluates them through the C ABI of libsofie_b200.so on
cuda:0, folding a following Relu / LeakyRelu / Sigmoid into the producing Gemm / Conv /
BatchNormalization the way the reference's parser and GPU planner do
(parsers/src/RModelParser_ONNX.cxx:1182-1219, core/src/RModel_Fusion_ALPAKA.cxx:367-416).
Operator attribute rules follow the reference's operators (cited per function).
"""
from __future__ import annotations

import ctypes as C
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from sofie_b200 import lib as L  # noqa: E402  (struct definitions and enums only)

ACT_OF = {"Relu": L.ACT_RELU, "LeakyRelu": L.ACT_LEAKY_RELU, "Sigmoid": L.ACT_SIGMOID}


def load_fixture(name: str) -> dict:
    z = np.load(ROOT / "tests" / "golden" / f"{name}.npz", allow_pickle=False)
    fx = {k: z[k] for k in z.files}
    fx["graph"] = json.loads(str(fx["graph"]))
    fx["weights"] = {k[2:]: fx[k] for k in list(fx) if k.startswith("w:")}
    return fx


def conv_geometry(attrs: dict, xshape, wshape):
    """Pads / strides / dilations / groups / output extent as ROperator_Conv.hxx:123-262 derives them
    (2-D only).  Quirk kept: auto_pad NOTSET without a pads attribute means pads of 1."""
    dil = list(attrs.get("dilations", [1, 1]))
    strides = list(attrs.get("strides", [1, 1]))
    group = attrs.get("group", 0) or xshape[1] // wshape[1]
    kh, kw = wshape[2], wshape[3]
    ekh, ekw = kh + (dil[0] - 1) * (kh - 1), kw + (dil[1] - 1) * (kw - 1)
    auto = attrs.get("auto_pad", "NOTSET")
    if auto == "NOTSET":
        pads = list(attrs.get("pads", [1, 1, 1, 1]))
    elif auto in ("SAME_UPPER", "SAME_LOWER"):
        pads = [0, 0, 0, 0]
        for d, (insz, st, ek) in enumerate(((xshape[2], strides[0], ekh), (xshape[3], strides[1], ekw))):
            out = (insz + st - 1) // st
            total = max(0, (out - 1) * st + ek - insz)
            lo, hi = (total // 2, total - total // 2) if auto == "SAME_UPPER" else (total - total // 2, total // 2)
            pads[d], pads[d + 2] = lo, hi
    elif auto == "VALID":
        pads = [0, 0, 0, 0]
    else:
        raise ValueError(f"invalid auto_pad {auto}")
    ho = (xshape[2] + pads[0] + pads[2] - ekh) // strides[0] + 1
    wo = (xshape[3] + pads[1] + pads[3] - ekw) // strides[1] + 1
    return dict(pads=pads, strides=strides, dil=dil, group=group, ho=ho, wo=wo)


def conv_desc(geo, xshape, wshape, x_dtype=L.F32, y_dtype=L.F32) -> L.ConvDesc:
    d = L.ConvDesc()
    d.N, d.C, d.H, d.W = xshape
    d.K, d.R, d.S = wshape[0], wshape[2], wshape[3]
    d.pad_top, d.pad_left, d.pad_bottom, d.pad_right = geo["pads"]
    d.stride_h, d.stride_w = geo["strides"]
    d.dil_h, d.dil_w = geo["dil"]
    d.groups = geo["group"]
    d.x_dtype, d.y_dtype, d.x_zero_point, d.precise = x_dtype, y_dtype, 0, 1
    return d


def _single_consumer(graph, tensor):
    return sum(tensor in n["in"] for n in graph["nodes"]) == 1 and tensor not in graph["outputs"]


# ------------------------------------------------------------------------------------------------
class OracleBackend:
    """numpy in / numpy out through oracle/libsofie_oracle.so."""

    def __init__(self):
        path = ROOT / "oracle" / "libsofie_oracle.so"
        if not path.exists():
            raise RuntimeError(f"{path} missing: run `make -C oracle oracle`")
        self.lib = C.CDLL(str(path))

    @staticmethod
    def _p(a):
        return a.ctypes.data_as(C.c_void_p) if a is not None else None

    def gemm(self, a, b, bias, alpha, beta, ta, tb, act, act_alpha):
        M, K = (a.shape[1], a.shape[0]) if ta else a.shape
        N = b.shape[0] if tb else b.shape[1]
        d = L.GemmDesc()
        d.M, d.N, d.K, d.batch = M, N, K, 1
        d.trans_a, d.trans_b, d.ab_dtype, d.y_dtype, d.precise = int(ta), int(tb), L.F32, L.F32, 1
        d.lda, d.ldb, d.ldy = a.shape[1], b.shape[1], N
        e = L.Epilogue()
        e.alpha, e.beta, e.out_scale, e.act, e.act_alpha = alpha, beta, 1.0, act, act_alpha
        keep = None
        if bias is not None:
            # broadcast rules of ROperator_Gemm.hxx:270-301; beta scales C before it is added
            keep = np.ascontiguousarray(np.broadcast_to(bias.astype(np.float32) * np.float32(beta), (M, N)))
            e.bias_mode, e.bias, e.ldc, e.beta = L.BIAS_FULL_F32, self._p(keep), N, 1.0
        y = np.zeros((M, N), dtype=np.float32)
        self.lib.so_gemm(C.byref(d), self._p(a), self._p(b), self._p(y), C.byref(e))
        return y

    def conv(self, x, w, bias, geo, act, act_alpha):
        d = conv_desc(geo, x.shape, w.shape)
        e = L.Epilogue()
        e.alpha, e.beta, e.out_scale, e.act, e.act_alpha = 1.0, 1.0, 1.0, act, act_alpha
        if bias is not None:
            e.bias_mode, e.bias = L.BIAS_COL_F32, self._p(bias)
        y = np.zeros((x.shape[0], w.shape[0], geo["ho"], geo["wo"]), dtype=np.float32)
        self.lib.so_conv(C.byref(d), self._p(x), self._p(w), self._p(y), C.byref(e))
        return y

    def batchnorm(self, x, scale, bias, mean, var, eps, act):
        fs = np.zeros_like(scale)
        self.lib.so_batchnorm_fold(self._p(scale), self._p(var), C.c_float(eps), C.c_int64(scale.size), self._p(fs))
        y = np.zeros_like(x)
        inner = int(np.prod(x.shape[2:])) if x.ndim > 2 else 1
        self.lib.so_batchnorm(self._p(x), self._p(y), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]), C.c_int64(inner),
                              self._p(fs), self._p(bias), self._p(mean), act)
        return y

    def layernorm(self, x, scale, bias, eps, cols):
        y = np.zeros_like(x)
        self.lib.so_layernorm(self._p(x), self._p(y), L.F32, L.F32, C.c_int64(x.size // cols), C.c_int64(cols),
                              self._p(scale), self._p(bias), C.c_float(eps), None, None)
        return y

    def softmax_last(self, x, cols):
        y = np.zeros_like(x)
        self.lib.so_softmax(self._p(x), self._p(y), L.F32, L.F32, C.c_int64(x.size // cols), C.c_int64(cols), 0)
        return y

    def softmax_axis(self, x, axis):
        y = np.zeros_like(x)
        outer, inner = int(np.prod(x.shape[:axis])), int(np.prod(x.shape[axis + 1:]))
        self.lib.so_softmax_axis(self._p(x), self._p(y), C.c_int64(outer), C.c_int64(x.shape[axis]), C.c_int64(inner), 0)
        return y

    def sdpa(self, q, k, v, mask):
        B, H, S, D = q.shape
        y = np.zeros((B, H, S, v.shape[3]), dtype=np.float32)
        self.lib.so_sdpa(self._p(q), self._p(k), self._p(v), self._p(mask), self._p(y), C.c_int64(B), C.c_int64(H), C.c_int64(S),
                         C.c_int64(D), C.c_int64(v.shape[3]), C.c_float(0.0), 0)
        return y

    def unary(self, x, act, act_alpha=0.0):
        y = np.zeros_like(x)
        self.lib.so_unary(self._p(x), self._p(y), L.F32, C.c_int64(x.size), act, C.c_float(act_alpha))
        return y

    def binary(self, a, b, op):
        y = np.zeros_like(a)
        self.lib.so_binary(self._p(a), self._p(np.ascontiguousarray(b)), self._p(y), L.F32, C.c_int64(a.size),
                           C.c_int64(b.size), op, 0)
        return y

    def to_backend(self, a):
        return np.ascontiguousarray(a, dtype=np.float32)

    def to_numpy(self, a):
        return a

    def transpose_copy(self, a, perm):
        return np.ascontiguousarray(np.transpose(a, perm))


class B200Backend:
    """torch CUDA tensors through libsofie_b200.so (cuda:0)."""

    fuses = True

    def __init__(self):
        import torch
        from sofie_b200.ops import Context
        self.torch = torch
        self.ctx = Context(0)
        self.lib = self.ctx._lib

    def gemm(self, a, b, bias, alpha, beta, ta, tb, act, act_alpha):
        from sofie_b200.ops import GemmPlan, make_epilogue
        t = self.torch
        M, K = (a.shape[1], a.shape[0]) if ta else a.shape
        N = b.shape[0] if tb else b.shape[1]
        kw = dict(alpha=alpha, act=act, act_alpha=act_alpha)
        if bias is not None:
            # ROperator_Gemm.hxx:270-301: C broadcasts as [N], [M,1], scalar or full [M,N]
            bs = tuple(bias.shape)
            if bias.numel() == 1:
                kw.update(bias=(bias.reshape(1) * beta).contiguous(), bias_mode=L.BIAS_SCALAR_F32)
            elif bs in ((N,), (1, N)):
                kw.update(bias=(bias.reshape(N) * beta).contiguous(), bias_mode=L.BIAS_COL_F32)
            elif bs == (M, 1):
                kw.update(bias=(bias.reshape(M) * beta).contiguous(), bias_mode=L.BIAS_ROW_F32)
            else:
                kw.update(bias=bias.contiguous(), bias_mode=L.BIAS_FULL_F32, beta=beta, ldc=N)
        ep, keep = make_epilogue(**kw)
        y = t.empty((M, N), dtype=t.float32, device="cuda:0")
        plan = GemmPlan(self.ctx, M, N, K, t.float32, t.float32, trans_a=ta, trans_b=tb, precise=True)
        plan.enqueue(a, b, y, ep)
        self.ctx.sync()
        plan.close()
        return y

    def conv(self, x, w, bias, geo, act, act_alpha):
        from sofie_b200.ops import make_epilogue
        t = self.torch
        d = conv_desc(geo, tuple(x.shape), tuple(w.shape))
        h = C.c_void_p()
        L.check(self.lib.sofie_b200_conv_plan_create(self.ctx._h, C.byref(d), w.data_ptr(), C.byref(h)), "conv_plan_create")
        ws = t.empty(max(16, self.lib.sofie_b200_conv_workspace_bytes(h)), dtype=t.uint8, device="cuda:0")
        y = t.empty((x.shape[0], w.shape[0], geo["ho"], geo["wo"]), dtype=t.float32, device="cuda:0")
        ep, keep = make_epilogue(bias=bias, act=act, act_alpha=act_alpha)
        L.check(self.lib.sofie_b200_conv_enqueue(h, x.data_ptr(), y.data_ptr(), ws.data_ptr(), C.byref(ep)), "conv_enqueue")
        self.ctx.sync()
        self.lib.sofie_b200_conv_plan_destroy(h)
        return y

    def batchnorm(self, x, scale, bias, mean, var, eps, act):
        t = self.torch
        # fused_scale is a code-generation-time constant in the reference (ROperator_BatchNormalization.hxx:100-109)
        fs = (scale / t.sqrt(var + t.tensor(eps, dtype=t.float32, device=var.device))).contiguous()
        y = t.empty_like(x)
        self.ctx.batchnorm(x, y, fs, bias, mean, act)
        self.ctx.sync()
        return y

    def layernorm(self, x, scale, bias, eps, cols):
        y = self.torch.empty_like(x)
        self.ctx.layernorm(x.reshape(-1, cols), y.reshape(-1, cols), scale, bias, eps)
        self.ctx.sync()
        return y

    def softmax_last(self, x, cols):
        y = self.torch.empty_like(x)
        self.ctx.softmax(x.reshape(-1, cols), y.reshape(-1, cols))
        self.ctx.sync()
        return y

    def softmax_axis(self, x, axis):
        y = self.torch.empty_like(x)
        self.ctx.softmax_axis(x, y, axis)
        self.ctx.sync()
        return y

    def sdpa(self, q, k, v, mask):
        y = self.torch.empty((q.shape[0], q.shape[1], q.shape[2], v.shape[3]), dtype=q.dtype, device=q.device)
        self.ctx.sdpa(q, k, v, y, mask=mask)
        return y

    def unary(self, x, act, act_alpha=0.0):
        y = self.torch.empty_like(x)
        self.ctx.unary(x, y, act, act_alpha)
        self.ctx.sync()
        return y

    def binary(self, a, b, op):
        y = self.torch.empty_like(a)
        self.ctx.binary(a, b.contiguous(), y, op)
        self.ctx.sync()
        return y

    def to_backend(self, a):
        return self.torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to("cuda:0")

    def to_numpy(self, a):
        return a.detach().cpu().numpy()

    def transpose_copy(self, a, perm):
        return a.permute(*perm).contiguous()  # layout plumbing only


# ------------------------------------------------------------------------------------------------
def run_graph(fx: dict, inputs: list, backend) -> np.ndarray:
    """Evaluates fx['graph'] on `inputs` (numpy) and returns the first graph output (numpy, flat)."""
    g = fx["graph"]
    env = {k: backend.to_backend(v) for k, v in fx["weights"].items()}
    for (name, _), val in zip(g["inputs"], inputs):
        env[name] = backend.to_backend(val)
    nodes = g["nodes"]
    skip = set()
    for idx, n in enumerate(nodes):
        if idx in skip:
            continue
        op, at = n["op"], n["attrs"]
        ins = [env[i] if i else None for i in n["in"]]
        out_name = n["out"][0]
        # fold a following activation into the producer (B200 backend only)
        act, act_alpha = L.ACT_NONE, 0.0
        if getattr(backend, "fuses", False) and op in ("Gemm", "Conv", "BatchNormalization") and idx + 1 < len(nodes):
            nx = nodes[idx + 1]
            if nx["op"] in ACT_OF and nx["in"] == [out_name] and _single_consumer(g, out_name):
                act, act_alpha = ACT_OF[nx["op"]], float(nx["attrs"].get("alpha", 0.01))
                out_name = nx["out"][0]
                skip.add(idx + 1)
        if op == "Gemm":
            bias = ins[2] if len(ins) > 2 else None
            y = backend.gemm(ins[0], ins[1], bias, float(at.get("alpha", 1.0)), float(at.get("beta", 1.0)),
                             bool(at.get("transA", 0)), bool(at.get("transB", 0)), act, act_alpha)
        elif op == "Conv":
            x, w = ins[0], ins[1]
            three_d = x.ndim == 5
            if three_d:
                # [N, C, D, H, W]: the depth taps become channels (x [N*Do, C*T, H, W], w [K, C*T, R, S] as it lies in memory), a
                # 2-D convolution runs over the slices and its result [N*Do, K, Ho, Wo] is transposed to [N, K, Do, Ho, Wo]
                xn, wn = backend.to_numpy(x), backend.to_numpy(w)
                N3, C3, D3 = xn.shape[:3]
                T = wn.shape[2]
                at = dict(at)
                dil3, st3 = list(at.get("dilations", [1, 1, 1])), list(at.get("strides", [1, 1, 1]))
                p3 = list(at.get("pads", [1] * 6)) if at.get("auto_pad", "NOTSET") == "NOTSET" else None
                if p3 is None:
                    raise NotImplementedError("auto_pad on a 3-D convolution")
                et = T + (dil3[0] - 1) * (T - 1)
                Do3 = (D3 + p3[0] + p3[3] - et) // st3[0] + 1
                xs = np.zeros((N3, Do3, C3, T) + xn.shape[3:], dtype=xn.dtype)
                for od in range(Do3):
                    for t in range(T):
                        z = od * st3[0] - p3[0] + t * dil3[0]
                        if 0 <= z < D3:
                            xs[:, od, :, t] = xn[:, :, z]
                x = backend.to_backend(np.ascontiguousarray(xs.reshape((N3 * Do3, C3 * T) + xn.shape[3:])))
                w = backend.to_backend(np.ascontiguousarray(wn.reshape((wn.shape[0], wn.shape[1] * T) + wn.shape[3:])))
                at["dilations"], at["strides"], at["pads"] = dil3[1:], st3[1:], [p3[1], p3[2], p3[4], p3[5]]
                if "kernel_shape" in at:
                    at["kernel_shape"] = list(at["kernel_shape"])[1:]
                if "group" not in at or not at["group"]:
                    at["group"] = C3 // wn.shape[1]
            one_d = x.ndim == 3   # [N, C, L]: a 2-D convolution of height 1 (ROperator_Conv.hxx:123-262 treats the ranks alike)
            if one_d:
                x, w = x.reshape(x.shape[0], x.shape[1], 1, x.shape[2]), w.reshape(w.shape[0], w.shape[1], 1, w.shape[2])
                at = dict(at)
                for key, fill in (("dilations", 1), ("strides", 1)):
                    if key in at:
                        at[key] = [fill] + list(at[key])
                if at.get("auto_pad", "NOTSET") == "NOTSET":
                    b, e = at.get("pads", [1, 1])   # the pads-default quirk: no pads attribute means 1
                    at["pads"] = [0, b, 0, e]
            geo = conv_geometry(at, tuple(x.shape), tuple(w.shape))
            y = backend.conv(x, w, ins[2] if len(ins) > 2 else None, geo, act, act_alpha)
            if one_d:
                y = y.reshape(y.shape[0], y.shape[1], y.shape[3])
            if three_d:
                yn = backend.to_numpy(y)
                y = backend.to_backend(np.ascontiguousarray(yn.reshape((N3, Do3) + yn.shape[1:]).transpose(0, 2, 1, 3, 4)))
        elif op == "BatchNormalization":
            y = backend.batchnorm(ins[0], ins[1], ins[2], ins[3], ins[4], float(at.get("epsilon", 1e-5)), act)
        elif op == "LayerNormalization":
            # normalises over the dimensions [axis, rank): ROperator_LayerNormalization.hxx:186-247
            x = ins[0]
            axis = at.get("axis", -1)
            axis = axis + x.ndim if axis < 0 else axis
            cols = int(np.prod(x.shape[axis:]))
            sc = ins[1].reshape(-1) if len(ins) > 1 and ins[1] is not None else None
            bi = ins[2].reshape(-1) if len(ins) > 2 and ins[2] is not None else None
            y = backend.layernorm(x, sc, bi, float(at.get("epsilon", 1e-5)), cols)
        elif op == "Softmax":
            x = ins[0]
            axis = at.get("axis", -1)
            axis = axis + x.ndim if axis < 0 else axis
            if axis == x.ndim - 1:
                y = backend.softmax_last(x, x.shape[-1])
            else:
                y = backend.softmax_axis(x, axis)
        elif op == "ScaledDotProductAttention":
            y = backend.sdpa(ins[0], ins[1], ins[2], ins[3] if len(ins) > 3 else None)
        elif op in ACT_OF:
            y = backend.unary(ins[0], ACT_OF[op], float(at.get("alpha", 0.01)))
        elif op == "Gelu":
            y = backend.unary(ins[0], L.ACT_GELU_TANH if at.get("approximate", "none") == "tanh" else L.ACT_GELU_ERF)
        elif op == "Add":
            y = backend.binary(ins[0], ins[1], 0)
        else:
            raise NotImplementedError(f"operator {op} is outside the hot path")
        env[out_name] = y
    return backend.to_numpy(env[g["outputs"][0]]).reshape(-1)
