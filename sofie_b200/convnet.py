"""The conv-net configuration on libsofie_b200: weights, work count and the device assembly.

Eight Conv 3x3 (pad 1) layers 3-64-64-128-128-256-256-512-512 with strides 1,2,1,2,1,2,1,2, each with a folded
BatchNormalization (per-channel scale and shift in the contraction epilogue) and Relu, global average pool,
Gemm 512 -> 1000.  Two variants: fp32 (precise: 3xTF32 on the tensor cores where large enough) and per-channel
int8 (QLinearConv: int32 accumulation, fp32 multiplier a_scale * w_scale[c] / y_scale, int32 bias, Relu, int8 out).
Plans, weights and every activation buffer are created once; a step only enqueues kernels.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

CHANNELS = [3, 64, 64, 128, 128, 256, 256, 512, 512]
STRIDES = [1, 2, 1, 2, 1, 2, 1, 2]
CLASSES = 1000
Y_SCALE = np.float32(0.05)        # activation scale of every int8 layer output
IN_SCALE = np.float32(1.0 / 127)  # U(0,1) input quantised to 0..127


def conv_desc(n, c, h, w, k, stride, x_dtype, y_dtype, x_layout=0, y_layout=0, flags=0):
    from sofie_b200 import lib as L
    d = L.ConvDesc()
    d.N, d.C, d.H, d.W, d.K, d.R, d.S = n, c, h, w, k, 3, 3
    d.pad_top = d.pad_left = d.pad_bottom = d.pad_right = 1
    d.stride_h = d.stride_w = stride
    d.dil_h = d.dil_w = 1
    d.groups = 1
    d.x_dtype, d.y_dtype, d.x_zero_point, d.precise = x_dtype, y_dtype, 0, 1
    d.x_layout, d.y_layout, d.flags = x_layout, y_layout, flags
    return d


def raw_parameters(seed: int):
    """The fp32 network as ONNX would hold it, from the reproducible generator of sofie_b200/synth.py (oracle/ref_emit.cxx
    builds the reference's model from the same draws): per layer He-normal weights N(0, sqrt(2/fan_in)) and the
    BatchNormalization parameters gamma ~ U(0.5, 1.5), beta ~ N(0, 0.1), mean ~ N(0, 0.1), var ~ U(0.5, 1.5); the classifier
    N(0, sqrt(2/512)) with a zero bias."""
    from . import synth
    layers = []
    for i in range(8):
        cin, cout = CHANNELS[i], CHANNELS[i + 1]
        ts = lambda j: synth.tensor_seed(seed, 10 * i + j)
        layers.append(dict(w=synth.normal_f32(ts(0), (cout, cin, 3, 3), np.sqrt(2.0 / (cin * 9))),
                           gamma=synth.uniform_f32(ts(1), cout, 0.5, 1.5), beta=synth.normal_f32(ts(2), cout, 0.1),
                           mean=synth.normal_f32(ts(3), cout, 0.1), var=synth.uniform_f32(ts(4), cout, 0.5, 1.5)))
    fc_w = synth.normal_f32(synth.tensor_seed(seed, 100), (512, CLASSES), np.sqrt(2.0 / 512))
    return layers, fc_w, np.zeros(CLASSES, dtype=np.float32)


def make_weights(seed: int, int8: bool):
    """raw_parameters() with BatchNormalization folded to a per-channel scale and shift (the fold the generator's fusion
    pass makes); the int8 variant quantises the weights per output channel and turns the fold into a multiplier and an
    int32 bias."""
    raw, fc_w, fc_b = raw_parameters(seed)
    layers = []
    a_scale = IN_SCALE
    for i, r in enumerate(raw):
        cout = CHANNELS[i + 1]
        wf = r["w"]
        scale = (r["gamma"] / np.sqrt(r["var"] + np.float32(1e-5))).astype(np.float32)
        shift = (r["beta"] - r["mean"] * scale).astype(np.float32)
        if not int8:
            layers.append(dict(w=wf, scale=scale, bias=shift))
        else:
            wfold = wf * scale[:, None, None, None]                     # BN scale folded into the weights before quantising
            w_scale = (np.abs(wfold).reshape(cout, -1).max(axis=1) / 127.0).astype(np.float32)
            wq = np.clip(np.rint(wfold / w_scale[:, None, None, None]), -127, 127).astype(np.int8)
            mult = (a_scale * w_scale / Y_SCALE).astype(np.float32)
            bias = np.rint(shift / (a_scale * w_scale)).astype(np.int32)   # shift at the accumulator's scale
            layers.append(dict(w=wq, scale=mult, bias=bias))
            a_scale = Y_SCALE
    return layers, fc_w, fc_b


def flops_per_image(img: int) -> float:
    f, hw = 0.0, img
    for i, st in enumerate(STRIDES):
        hw = (hw + 2 - 3) // st + 1
        f += 2.0 * CHANNELS[i + 1] * hw * hw * CHANNELS[i] * 9
    return f + 2.0 * 512 * CLASSES


class ConvNetB200:
    """The network on one GPU through the C ABI.  `ctx` is a sofie_b200.ops.Context on that GPU."""

    @property
    def launches(self) -> int:
        """Kernels one call enqueues: per convolution 1 (direct first layer; implicit convolution "umma_im2col"), else an
        unfold and a contraction plus, for an NCHW input of whole 16-byte channel vectors, its channels-last copy (the
        3-channel first layer unfolds straight from NCHW); then the pool and the classifier."""
        n = 2
        for i, (kern, xl) in enumerate(zip(self.kernels, self.x_layouts)):
            n += 1 if kern in ("direct", "umma_im2col", "umma3x_im2col") else (2 if xl or i == 0 or kern == "umma_im2col_x2" else 3)
        if self.kernels[0] == "umma" and self.int8 and self.channels_last and self.first_pixels % 2 == 0:
            n += 1   # the int8 first layer on the tensor cores packs 2 or 4 pixels per row: one kernel repeats its per-channel vectors
        return n

    def __init__(self, ctx, weights, batch: int, img: int, int8: bool, device: str, channels_last: bool = True):
        """channels_last: the activations between the convolutions are kept [N,H,W,C] (what a layout pass of the generator
        would emit for a conv -> conv chain, the pool reading the last one in that layout); the network's input stays NCHW."""
        import torch
        from sofie_b200 import lib as L
        from sofie_b200.ops import GemmPlan, make_epilogue
        self.ctx, self.batch, self.int8, self.channels_last = ctx, batch, int8, channels_last
        self.first_pixels = batch * img * img
        self.lib = lib = ctx._lib
        t = torch
        adt = t.int8 if int8 else t.float32
        code = L.I8 if int8 else L.F32
        layers, fc_w, fc_b = weights
        self.plans, self.eps, self.keep, self.acts, self.kernels, self.x_layouts = [], [], [], [], [], []
        hw, ws_bytes = img, 16
        self.x_in = t.empty((batch, 3, img, img), dtype=adt, device=device)
        for i, (ly, st, cin, cout) in enumerate(zip(layers, STRIDES, CHANNELS[:-1], CHANNELS[1:])):
            # channels-last chain; the fp32 net passes TF32 pairs (layout 2: [N,H,W,2C], hi then lo channels) between the
            # convolutions, which the 3xTF32 contraction reads without an unfold, and a plain channels-last tensor to the pool
            inner = 1 if int8 else 2
            xl = (inner if i > 0 else 0) if channels_last else 0
            yl = (inner if i < 7 else 1) if channels_last else 0
            d = conv_desc(batch, cin, hw, hw, cout, st, code, code, xl, yl)
            w = t.from_numpy(ly["w"]).to(device)
            h = C.c_void_p()
            L.check(lib.sofie_b200_conv_plan_create(ctx._h, C.byref(d), w.data_ptr(), C.byref(h)), "conv_plan_create")
            ws_bytes = max(ws_bytes, lib.sofie_b200_conv_workspace_bytes(h))
            hw = (hw + 2 - 3) // st + 1
            ep, keep = make_epilogue(col_scale=t.from_numpy(ly["scale"]).to(device), bias=t.from_numpy(ly["bias"]).to(device), act=L.ACT_RELU)
            self.plans.append(h); self.eps.append(ep); self.keep.append((keep, w))
            self.acts.append(t.empty((batch, hw, hw, cout * (2 if yl == 2 else 1)) if yl else (batch, cout, hw, hw), dtype=adt, device=device))
            self.kernels.append(lib.sofie_b200_conv_plan_kernel(h).decode())
            self.x_layouts.append(xl)
        ctx.sync()   # weight re-layout kernels read `w`
        self.workspace = t.empty(ws_bytes, dtype=t.uint8, device=device)
        self.pooled = t.empty((batch, 512), dtype=t.float32, device=device)
        self.logits = t.empty((batch, CLASSES), dtype=t.float32, device=device)
        self.fc_w = t.from_numpy(fc_w).to(device)
        self.fc = GemmPlan(ctx, batch, CLASSES, 512, t.float32, t.float32, trans_b=False)
        self.fc_ep, k = make_epilogue(alpha=float(Y_SCALE) if int8 else 1.0, bias=t.from_numpy(fc_b).to(device))
        self.keep.append(k)

    def __call__(self, x):
        """x: [batch, 3, img, img] on the device; returns the logits buffer (owned here, overwritten by the next call)."""
        from sofie_b200 import lib as L
        cur = x
        for h, ep, y in zip(self.plans, self.eps, self.acts):
            L.check(self.lib.sofie_b200_conv_enqueue(h, cur.data_ptr(), y.data_ptr(), self.workspace.data_ptr(), C.byref(ep)), "conv_enqueue")
            cur = y
        if self.channels_last:
            self.ctx.global_avgpool_nhwc(cur, self.pooled)
        else:
            self.ctx.global_avgpool(cur, self.pooled)
        self.fc.enqueue(self.pooled, self.fc_w, self.logits, self.fc_ep)
        return self.logits

    def close(self):
        for h in self.plans:
            self.lib.sofie_b200_conv_plan_destroy(h)
        self.fc.close()


def onnx_model(seed: int, batch: int, img: int, int8: bool):
    """The network as an ONNX graph for the C++ generator (sofie_b200/onnx_min.save).  fp32: Conv -> BatchNormalization -> Relu
    per layer, as a framework exports it (the generator folds the normalisation and the Relu into the convolution and keeps
    the chain channels-last).  int8: QLinearConv (per-channel weight scales, int32 bias) -> Relu per layer on int8 tensors
    of scale Y_SCALE, then DequantizeLinear -> GlobalAveragePool; both end in Flatten -> Gemm 512 -> 1000.
    Returns (nodes, initializers, inputs, outputs, input_types)."""
    raw, fc_w, fc_b = raw_parameters(seed)
    init = {"fc_w": fc_w, "fc_b": fc_b}
    nodes = []
    x = "X"
    if not int8:
        for i, (r, st) in enumerate(zip(raw, STRIDES)):
            for k in ("w", "gamma", "beta", "mean", "var"):
                init[f"{k}{i}"] = r[k]
            nodes.append({"op": "Conv", "in": [x, f"w{i}"], "out": [f"c{i}"], "attrs": {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1], "strides": [st, st]}})
            nodes.append({"op": "BatchNormalization", "in": [f"c{i}", f"gamma{i}", f"beta{i}", f"mean{i}", f"var{i}"], "out": [f"n{i}"], "attrs": {"epsilon": 1e-5}})
            nodes.append({"op": "Relu", "in": [f"n{i}"], "out": [f"r{i}"], "attrs": {}})
            x = f"r{i}"
        types = {}
    else:
        layers, _, _ = make_weights(seed, True)
        init.update({"zp": np.array(0, dtype=np.int8), "in_scale": np.array(IN_SCALE), "act_scale": np.array(Y_SCALE)})
        a_scale = IN_SCALE
        for i, (ly, r, st) in enumerate(zip(layers, raw, STRIDES)):
            cout = CHANNELS[i + 1]
            bn_scale = (r["gamma"] / np.sqrt(r["var"] + np.float32(1e-5))).astype(np.float32)
            wfold = r["w"] * bn_scale[:, None, None, None]
            w_scale = (np.abs(wfold).reshape(cout, -1).max(axis=1) / 127.0).astype(np.float32)
            init[f"wq{i}"], init[f"ws{i}"], init[f"wz{i}"], init[f"b{i}"] = ly["w"], w_scale, np.zeros(cout, dtype=np.int8), ly["bias"]
            nodes.append({"op": "QLinearConv", "in": [x, "in_scale" if i == 0 else "act_scale", "zp", f"wq{i}", f"ws{i}", f"wz{i}", "act_scale", "zp", f"b{i}"],
                          "out": [f"q{i}"], "attrs": {"kernel_shape": [3, 3], "pads": [1, 1, 1, 1], "strides": [st, st]}})
            nodes.append({"op": "Relu", "in": [f"q{i}"], "out": [f"r{i}"], "attrs": {}})
            x = f"r{i}"
            a_scale = Y_SCALE
        nodes.append({"op": "DequantizeLinear", "in": [x, "act_scale", "zp"], "out": ["deq"], "attrs": {}})
        x = "deq"
        types = {"X": 3}
    nodes.append({"op": "GlobalAveragePool", "in": [x], "out": ["pool"], "attrs": {}})
    nodes.append({"op": "Flatten", "in": ["pool"], "out": ["flat"], "attrs": {"axis": 1}})
    nodes.append({"op": "Gemm", "in": ["flat", "fc_w", "fc_b"], "out": ["Y"], "attrs": {}})
    return nodes, init, [("X", [batch, 3, img, img])], ["Y"], types
