"""int8 ResNet-50 v1.5 as an nGraph Function (client-side graph construction for tests and bench).

The reference ships no model files, so the graph is built here with nGraph ops, the way a framework
bridge would after nGraph's quantization builders and the CPU backend's fusion pass have run:
every convolution is a QuantizedConvolutionBias (+Relu, or +Add+Relu for the residual joins) with
u8 activations, i8 per-output-channel weights and i32 bias; MaxPool on u8; the head is
Dequantize -> global AvgPool -> Quantize -> QuantizedDot 2048->1000 -> Dequantize.

Weights are random (He-normal, seeded; batch-norm folded away, i.e. conv + bias), quantised per
output channel (scale = maxabs/127).  Activation scales come from a seeded calibration batch pushed
through a float simulation of the quantised network (torch on the host, deterministic), scale =
max/255 per tensor.  The network input is f32 NCHW, already normalised by the ImageNet mean/std, and
is quantised to i8 (the normalised image is signed) by the first node of the graph.
"""
import numpy as np

MEAN = np.array([0.485, 0.456, 0.406], np.float32)
STD = np.array([0.229, 0.224, 0.225], np.float32)
STAGES = [(3, 64, 256, 1), (4, 128, 512, 2), (6, 256, 1024, 2), (3, 512, 2048, 2)]  # blocks, mid, out, stride


def synthetic_images(batch, seed, size=224):
    """uniform [0,1) pixels normalised per channel; stands in for ImageNet images"""
    rng = np.random.default_rng(seed)
    x = rng.random((batch, 3, size, size), dtype=np.float32)
    return ((x - MEAN[None, :, None, None]) / STD[None, :, None, None]).astype(np.float32)


def conv_specs():
    """(name, cin, cout, kernel, stride, pad, relu, residual) in execution order; residual names the
    tensor added before the ReLU ('' = none)."""
    specs = [("stem", 3, 64, 7, 2, 3, True, "")]
    cin = 64
    for si, (blocks, mid, cout, stride) in enumerate(STAGES):
        for b in range(blocks):
            s = stride if b == 0 else 1
            pre = "s%db%d" % (si + 1, b)
            if b == 0:
                specs.append((pre + "_down", cin, cout, 1, s, 0, False, ""))
            specs.append((pre + "_c1", cin, mid, 1, 1, 0, True, ""))
            specs.append((pre + "_c2", mid, mid, 3, s, 1, True, ""))  # v1.5: the stride sits on the 3x3
            specs.append((pre + "_c3", mid, cout, 1, 1, 0, True, pre + "_down" if b == 0 else "block_in"))
            cin = cout
    return specs


def _rne(x):
    return np.rint(x)


class QuantizedResNet50:
    def __init__(self, seed=0, calibration_batch=8, classes=1000, image_size=224, calibration_size=None):
        self.seed, self.classes, self.image_size = seed, classes, image_size
        rng = np.random.default_rng(seed)
        self.layers = {}
        for name, cin, cout, k, stride, pad, relu, res in conv_specs():
            w = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
            bias = (rng.standard_normal(cout) * 0.05).astype(np.float32)
            s_w = (np.abs(w).reshape(cout, -1).max(axis=1) / np.float32(127)).astype(np.float32)
            w_q = np.clip(_rne(w / s_w[:, None, None, None]), -127, 127).astype(np.int8)
            self.layers[name] = dict(cin=cin, cout=cout, k=k, stride=stride, pad=pad, relu=relu, res=res, w_q=w_q, s_w=s_w,
                                     bias_f=bias)
        fc = (rng.standard_normal((2048, classes)) * np.sqrt(1.0 / 2048)).astype(np.float32)
        self.s_fc = np.float32(np.abs(fc).max() / 127)
        self.fc_q = np.clip(_rne(fc / self.s_fc), -127, 127).astype(np.int8)
        self._calibrate(calibration_batch, calibration_size or image_size)

    # ------------------------------------------------------------------ calibration (host, float simulation)
    def _calibrate(self, batch, size):
        import torch
        import torch.nn.functional as F
        torch.manual_seed(0)
        x = synthetic_images(batch, self.seed + 1000, size)
        self.s_input = np.float32(np.abs(x).max() / 127)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
        xq = torch.clamp(torch.round(t(x) / float(self.s_input)), -128, 127)
        acts = {}   # name -> (integer-valued float tensor, scale)

        def conv(name, inp, s_in, res=None, res_signed=False):
            L = self.layers[name]
            mult = (np.float32(s_in) * L["s_w"]).astype(np.float32)                  # s_in * s_w[k]
            L["bias_q"] = _rne(L["bias_f"] / mult).astype(np.int32)                  # Quantize(bias, s_in*s_w, i32, RNE)
            acc = F.conv2d(inp, t(L["w_q"]).float(), stride=L["stride"], padding=L["pad"])
            v = (acc + t(L["bias_q"]).float()[None, :, None, None]) * t(mult)[None, :, None, None]
            if res is not None:
                v = v + res[0] * float(res[1])
            if L["relu"]:
                # QuantizedConvolutionBiasSignedAdd (i8 residual) produces i8: its ReLU output tops out at 127
                top = 127 if res_signed else 255
                v = torch.clamp(v, min=0)
                s_out = np.float32(max(float(v.max()), 1e-6) / top)
                q = torch.clamp(torch.round(v / float(s_out)), 0, top)
            else:
                s_out = np.float32(max(float(v.abs().max()), 1e-6) / 127)
                q = torch.clamp(torch.round(v / float(s_out)), -128, 127)
            L["s_in"], L["s_out"] = np.float32(s_in), s_out
            L["scale"] = (mult / s_out).astype(np.float32)                           # requantisation scale per channel
            if res is not None:
                L["sum_scale"] = np.array([np.float32(res[1]) / s_out], np.float32)
            return q.float(), s_out

        a, s = conv("stem", xq.float(), self.s_input)
        a = F.max_pool2d(a, 3, 2, 1)
        for si, (blocks, mid, cout, stride) in enumerate(STAGES):
            for b in range(blocks):
                pre = "s%db%d" % (si + 1, b)
                block_in = (a, s)
                short = conv(pre + "_down", a, s) if b == 0 else block_in
                y, sy = conv(pre + "_c1", a, s)
                y, sy = conv(pre + "_c2", y, sy)
                a, s = conv(pre + "_c3", y, sy, res=short, res_signed=(b == 0))
        self.s_feat = s
        pooled = (a * float(s)).mean(dim=(2, 3))
        self.s_pool = np.float32(max(float(pooled.max()), 1e-6) / 255)
        pq = torch.clamp(torch.round(pooled / float(self.s_pool)), 0, 255)
        logits = (pq @ t(self.fc_q).float()) * float(self.s_pool) * float(self.s_fc)
        # 2x headroom: other inputs exceed the calibration maximum, and where the device saturates the
        # reference's QuantizedDot wraps (runtime/reference/dot.hpp:156 casts without clamping)
        self.s_logits = np.float32(2.0 * max(float(logits.abs().max()), 1e-6) / 127)

    # ------------------------------------------------------------------ graph
    def layer_work(self, hw=None):
        """per contraction node in execution order: (name, multiply-accumulates, bytes read + written) for ONE image; bytes =
        input and output activations (one byte each), the residual where there is one; weights are added per batch by the
        caller (they are read once per launch, not per image)"""
        h, w = hw or (self.image_size, self.image_size)
        out = lambda n, k, s, p: (n + 2 * p - k) // s + 1
        rows = []
        hs, ws = out(h, 7, 2, 3), out(w, 7, 2, 3)
        rows.append(("stem", hs * ws * 64 * 3 * 49, h * w * 3 * 4 + hs * ws * 64, 64 * 3 * 49))  # reads the f32 image
        h, w = out(hs, 3, 2, 1), out(ws, 3, 2, 1)
        cin = 64
        for si, (blocks, mid, cout, stride) in enumerate(STAGES):
            for b in range(blocks):
                s = stride if b == 0 else 1
                ho, wo = out(h, 3, s, 1), out(w, 3, s, 1)
                pre = "s%db%d" % (si + 1, b)
                if b == 0:
                    rows.append((pre + "_down", ho * wo * cin * cout, h * w * cin + ho * wo * cout, cin * cout))
                rows.append((pre + "_c1", h * w * cin * mid, h * w * cin + h * w * mid, cin * mid))
                rows.append((pre + "_c2", ho * wo * mid * mid * 9, h * w * mid + ho * wo * mid, mid * mid * 9))
                rows.append((pre + "_c3", ho * wo * mid * cout, ho * wo * mid + 2 * ho * wo * cout, mid * cout))
                h, w, cin = ho, wo, cout
        rows.append(("fc", 2048 * self.classes, 2048 + self.classes, 2048 * self.classes))
        return rows

    def macs_per_image(self, hw=None):
        """multiply-accumulates of the convolutions and the final QuantizedDot for one image of size hw"""
        h, w = hw or (self.image_size, self.image_size)
        out = lambda n, k, s, p: (n + 2 * p - k) // s + 1
        h, w = out(h, 7, 2, 3), out(w, 7, 2, 3)
        total = h * w * 64 * 3 * 49
        h, w = out(h, 3, 2, 1), out(w, 3, 2, 1)
        cin = 64
        for blocks, mid, cout, stride in STAGES:
            for b in range(blocks):
                s = stride if b == 0 else 1
                ho, wo = out(h, 3, s, 1), out(w, 3, s, 1)
                if b == 0:
                    total += ho * wo * cin * cout
                total += h * w * cin * mid + ho * wo * mid * mid * 9 + ho * wo * mid * cout
                h, w, cin = ho, wo, cout
        return total + 2048 * self.classes

    def build(self, ng, batch, fused=True, decomposed=None, image_hw=None, intermediate_results=False, framework_style=False):
        """Returns (Function, parameter).  fused=True: the graph a client hands to the B200 backend.
        fused=False: every fused op replaced by `decomposed` (oracle.interpreter), for INTERPRETER.
        framework_style=True: the graph a framework bridge emits before any backend fusion: every convolution is a
        QuantizedConvolutionBias WITHOUT relu followed by Dequantize -> [Add(Dequantize(shortcut))] -> Relu -> Quantize,
        with the same scales; a backend's quantisation fusion is expected to turn it back into the fused graph."""
        h, w = image_hw or (self.image_size, self.image_size)
        x = ng.parameter(np.float32, (batch, 3, h, w))
        a = ng.quantize(x, self.s_input, np.int8(0), np.int8, (), 4)
        scale_of, alive = {}, []  # id of a quantized value -> its scale (for the shortcut's Dequantize); values kept alive

        def conv(name, inp, res=None):
            L = self.layers[name]
            geom = dict(stride=(L["stride"],) * 2, pad_below=(L["pad"],) * 2)
            out_dtype = np.uint8 if L["relu"] else np.int8
            if framework_style:
                y = ng.quantized_conv_bias(inp, L["w_q"], L["bias_q"], L["scale"], False, **geom)  # i8, scale s_out
                if L["relu"]:
                    f = ng.dequantize(y, L["s_out"], np.int8(0))
                    if res is not None:
                        f = ng.add(f, ng.dequantize(res, scale_of[id(res)], np.zeros((), np.dtype(res.dtype))))
                    y = ng.quantize(ng.relu(f), L["s_out"], np.uint8(0), np.uint8, (), 4)
                scale_of[id(y)] = L["s_out"]
                alive.append(y)
                return y
            if fused:
                if res is None:
                    return ng.quantized_conv_bias(inp, L["w_q"], L["bias_q"], L["scale"], L["relu"], **geom)
                signed = np.dtype(res.dtype) == np.int8
                y = ng.quantized_conv_bias_add(inp, L["w_q"], L["bias_q"], res, L["scale"], L["sum_scale"], True, signed, **geom)
                return ng.convert(y, np.uint8) if signed else y
            kw = {}
            if res is not None:
                kw = dict(sum_in=res, sum_scale=ng.constant(L["sum_scale"]), signed=np.dtype(res.dtype) == np.int8)
            return decomposed.decomposed_conv(inp, ng.constant(L["w_q"]), ng.constant(L["bias_q"]), ng.constant(L["scale"]),
                                              out_dtype, L["relu"], **geom, **kw)

        taps = []
        a = conv("stem", a)
        taps.append(a)
        stem_out = a
        a = ng.max_pool(a, (3, 3), (2, 2), (1, 1))
        scale_of[id(a)] = scale_of.get(id(stem_out))
        alive.append(a)
        taps.append(a)
        for si, (blocks, mid, cout, stride) in enumerate(STAGES):
            for b in range(blocks):
                pre = "s%db%d" % (si + 1, b)
                short = conv(pre + "_down", a) if b == 0 else a
                y = conv(pre + "_c1", a)
                y = conv(pre + "_c2", y)
                a = conv(pre + "_c3", y, res=short)
                taps.append(a)
        fh, fw = a.shape[2], a.shape[3]
        pooled = ng.quantize(ng.avg_pool(ng.dequantize(a, self.s_feat, np.uint8(0)), (fh, fw)), self.s_pool, np.uint8(0),
                             np.uint8, (), 4)
        flat = ng.reshape(pooled, (0, 1, 2, 3), (batch, 2048))
        logits = ng.quantized_dot(flat, ng.constant(self.fc_q), self.s_pool, 0, self.s_fc, 0, self.s_logits, 0, np.int8)
        out = ng.dequantize(logits, self.s_logits, np.int8(0))
        if intermediate_results:  # stem, maxpool, the 16 block outputs, pooled features, i8 logits, f32 logits
            return ng.Function(taps + [pooled, logits, out], [x]), x
        return ng.Function([out], [x]), x


class OneDnnProxy:
    """The same int8 ResNet-50 (weights, per-channel weight scales, calibrated activation scales) on the host cores through
    the oneDNN int8 primitives that ship inside PyTorch (torch.ops.quantized.* with the 'onednn' engine).

    nGraph's own CPU backend drives the same library family (DNNL int8 convolution_forward / inner_product with output
    scales, sum and ReLU post-ops: src/ngraph/runtime/cpu/builder/quantized_conv.cpp, dnnl_emitter.hpp) but cannot be
    built without its downloaded dependencies, so this stands in for it as a TIMING baseline only: the residual add is a
    separate quantized add here and activations are uint8 with zero point 128 where the nGraph graph uses int8, so
    results are close to, not identical with, the reference's."""

    def __init__(self, model):
        import torch
        torch.backends.quantized.engine = "onednn"
        self.torch, self.model = torch, model
        self.packed = {}
        for name, L in model.layers.items():
            w = torch.from_numpy(L["w_q"].astype(np.float32) * L["s_w"][:, None, None, None])
            qw = torch.quantize_per_channel(w, torch.from_numpy(L["s_w"].astype(np.float64)), torch.zeros(L["cout"], dtype=torch.int64),
                                            0, torch.qint8)
            self.packed[name] = torch.ops.quantized.conv2d_prepack(qw, torch.from_numpy(L["bias_f"]), [L["stride"]] * 2,
                                                                   [L["pad"]] * 2, [1, 1], 1)
        fc = torch.from_numpy(model.fc_q.T.astype(np.float32) * float(model.s_fc)).contiguous()
        self.fc = torch.ops.quantized.linear_prepack(torch.quantize_per_tensor(fc, float(model.s_fc), 0, torch.qint8), None)

    def forward(self, x):
        torch, m = self.torch, self.model
        q = torch.ops.quantized
        a = torch.quantize_per_tensor(torch.from_numpy(x), float(m.s_input), 128, torch.quint8).contiguous(memory_format=torch.channels_last)

        def conv(name, inp, relu=None):
            L = m.layers[name]
            relu = L["relu"] if relu is None else relu
            if relu:
                return q.conv2d_relu(inp, self.packed[name], float(L["s_out"]), 0)
            return q.conv2d(inp, self.packed[name], float(L["s_out"]), 128)

        a = conv("stem", a)
        a = torch.nn.functional.max_pool2d(a, 3, 2, 1)
        for si, (blocks, mid, cout, stride) in enumerate(STAGES):
            for b in range(blocks):
                pre = "s%db%d" % (si + 1, b)
                short = conv(pre + "_down", a) if b == 0 else a
                y = conv(pre + "_c1", a)
                y = conv(pre + "_c2", y)
                L = m.layers[pre + "_c3"]
                y = conv(pre + "_c3", y, relu=False)
                a = q.add_relu(y, short, float(L["s_out"]), 0)
        pooled = torch.nn.functional.adaptive_avg_pool2d(a, 1).flatten(1)
        logits = q.linear(pooled, self.fc, float(m.s_logits), 128)
        return logits.dequantize().numpy()

    def images_per_second(self, batch=16, seconds=8.0):
        import time
        x = synthetic_images(batch, 5, self.model.image_size)
        self.forward(x)
        t0, n = time.time(), 0
        while time.time() - t0 < seconds:
            self.forward(x)
            n += batch
        return n / (time.time() - t0)
