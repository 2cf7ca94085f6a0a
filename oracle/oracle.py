"""CPU oracle for libgpx — TEST INFRASTRUCTURE ONLY (see gpx_oracle.c for the full header).

Only tests/, the smoke check and the CPU-baseline leg of bench.py may import this module.
PARITY UNPINNED: the reference stores no expected outputs and its arithmetic (TVM-generated
kernels, apache/tvm @ 513c2be0c3b853) is not in its tree; the layer functions here are checked
against PyTorch CPU operators by tests/test_oracle.py instead.

The model definitions below restate the published architectures independently of the
product's graph builder: ResNet v1.5 bottleneck networks and VGG, with batch norm folded into
a per-convolution bias, NCHW activations and OIHW filters as the reference's graphs use
(scripts/compile/compile.py:27-44).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libgpx_oracle.so")
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_f64p = ctypes.POINTER(ctypes.c_double)
_i32p = ctypes.POINTER(ctypes.c_int)


def build() -> str:
    """Compiles gpx_oracle.c when the shared object is missing or stale."""
    src = os.path.join(_HERE, "gpx_oracle.c")
    if not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        conv_args = [_f32p, _f32p, _f32p, _f32p, _f32p] + [ctypes.c_int] * 10
        _lib.orc_conv2d_nchw.argtypes = conv_args
        _lib.orc_conv2d_nchw_fast.argtypes = conv_args
        _lib.orc_conv2d_nchw_hw.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p] + [ctypes.c_int] * 11
        _lib.orc_pool2d_nchw.argtypes = [_f32p, _f32p] + [ctypes.c_int] * 8
        _lib.orc_dwconv2d_nchw.argtypes = [_f32p, _f32p, _f32p, _f32p] + [ctypes.c_int] * 9
        _lib.orc_axpy_f32.argtypes = [ctypes.c_float, _f32p, _f32p, ctypes.c_size_t]
        _lib.orc_f32_to_bf16.argtypes = [_f32p, _u16p, ctypes.c_size_t]
        _lib.orc_bf16_to_f32.argtypes = [_u16p, _f32p, ctypes.c_size_t]
        _lib.orc_gemm_bf16_nt.argtypes = [_u16p, _u16p, _f64p] + [ctypes.c_int] * 3
        _lib.orc_gemm_bf16_nt_fast.argtypes = [_u16p, _u16p, _f32p] + [ctypes.c_int] * 3
        _lib.orc_gemm_bf16_nt_samples.argtypes = [_u16p, _u16p, _i32p, _i32p, ctypes.c_int,
                                                  _f64p, ctypes.c_int]
    return _lib


def _p(a: np.ndarray | None, typ):
    if a is None:
        return ctypes.cast(None, typ)
    return a.ctypes.data_as(typ)


def _c(a, dtype=np.float32) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


# ---- layer functions ---------------------------------------------------------------------------

def conv2d(x, w, bias=None, stride=1, pad=0, relu=False, residual=None, fast=False):
    """Fused conv2d + bias + residual + activation.  x NCHW, w OIHW; `relu` is False/True or
    the string "relu6"."""
    x, w = _c(x), _c(w)
    n, cin, h, wd = x.shape
    cout, cin2, kh, kw = w.shape
    assert cin == cin2
    ph, pw = (pad, pad) if np.isscalar(pad) else pad   # (vertical, horizontal) for one-sided kernels
    ho = (h + 2 * ph - kh) // stride + 1
    wo = (wd + 2 * pw - kw) // stride + 1
    out = np.empty((n, cout, ho, wo), np.float32)
    b = _c(bias) if bias is not None else None
    r = _c(residual) if residual is not None else None
    if r is not None:
        assert r.shape == out.shape
    act = 3 if relu == "relu6" else int(bool(relu))
    if fast and ph == pw:
        lib().orc_conv2d_nchw_fast(_p(x, _f32p), _p(w, _f32p), _p(b, _f32p), _p(r, _f32p), _p(out, _f32p), n, cin,
                                   h, wd, cout, kh, kw, stride, ph, act)
    else:
        lib().orc_conv2d_nchw_hw(_p(x, _f32p), _p(w, _f32p), _p(b, _f32p), _p(r, _f32p), _p(out, _f32p), n, cin,
                                 h, wd, cout, kh, kw, stride, ph, pw, act)
    return out


def dwconv2d(x, w, bias=None, stride=1, pad=0, relu=False):
    """Depthwise conv2d + bias + activation.  x NCHW, w [C][1][kh][kw]."""
    x, w = _c(x), _c(w)
    n, c, h, wd = x.shape
    assert w.shape[0] == c and w.shape[1] == 1
    kh, kw = w.shape[2], w.shape[3]
    ho = (h + 2 * pad - kh) // stride + 1
    wo = (wd + 2 * pad - kw) // stride + 1
    out = np.empty((n, c, ho, wo), np.float32)
    b = _c(bias) if bias is not None else None
    lib().orc_dwconv2d_nchw(_p(x, _f32p), _p(w, _f32p), _p(b, _f32p), _p(out, _f32p), n, c, h, wd,
                            kh, kw, stride, pad, 3 if relu == "relu6" else int(bool(relu)))
    return out


def pool2d(x, k, stride, pad, mode):
    x = _c(x)
    n, c, h, w = x.shape
    ho = (h + 2 * pad - k) // stride + 1
    wo = (w + 2 * pad - k) // stride + 1
    out = np.empty((n, c, ho, wo), np.float32)
    # "avg" divides by the number of taps inside the image, "avg_pad" by the whole window
    lib().orc_pool2d_nchw(_p(x, _f32p), _p(out, _f32p), n, c, h, w, k, stride, pad,
                          {"max": 0, "avg": 1, "avg_pad": 2}[mode])
    return out


def axpy(a, x, y):
    """Returns fma(a, x, y) element-wise in fp32 (y is not modified)."""
    x = _c(x)
    out = _c(y).copy()
    lib().orc_axpy_f32(np.float32(a), _p(x, _f32p), _p(out, _f32p), x.size)
    return out


def f32_to_bf16(x):
    x = _c(x)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16(_p(x, _f32p), _p(out, _u16p), x.size)
    return out


def bf16_to_f32(x):
    x = _c(x, np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().orc_bf16_to_f32(_p(x, _u16p), _p(out, _f32p), x.size)
    return out


def gemm_bf16_nt(a_bits, b_bits):
    """Exact (fp64) A[M][K] x B[N][K]^T for bf16 bit patterns; returns float64 [M][N]."""
    a, b = _c(a_bits, np.uint16), _c(b_bits, np.uint16)
    m, k = a.shape
    n, k2 = b.shape
    assert k == k2
    out = np.empty((m, n), np.float64)
    lib().orc_gemm_bf16_nt(_p(a, _u16p), _p(b, _u16p), _p(out, _f64p), m, n, k)
    return out


def gemm_bf16_nt_fast(a_bits, b_bits):
    a, b = _c(a_bits, np.uint16), _c(b_bits, np.uint16)
    m, k = a.shape
    n, _ = b.shape
    out = np.empty((m, n), np.float32)
    lib().orc_gemm_bf16_nt_fast(_p(a, _u16p), _p(b, _u16p), _p(out, _f32p), m, n, k)
    return out


def gemm_bf16_nt_samples(a_bits, b_bits, rows, cols):
    a, b = _c(a_bits, np.uint16), _c(b_bits, np.uint16)
    rows, cols = _c(rows, np.int32), _c(cols, np.int32)
    out = np.empty(rows.size, np.float64)
    lib().orc_gemm_bf16_nt_samples(_p(a, _u16p), _p(b, _u16p), _p(rows, _i32p), _p(cols, _i32p),
                                   rows.size, _p(out, _f64p), a.shape[1])
    return out


# ---- model definitions -------------------------------------------------------------------------

def resnet_param_shapes(layers=(3, 4, 6, 3), num_classes=1000):
    """Ordered {name: shape} of a bottleneck ResNet with folded batch norm."""
    shapes = {"conv1.weight": (64, 3, 7, 7), "conv1.bias": (64,)}
    inplanes, planes = 64, 64
    for li, nblocks in enumerate(layers):
        for b in range(nblocks):
            p = f"layer{li + 1}.{b}"
            if b == 0:
                shapes[f"{p}.downsample.weight"] = (planes * 4, inplanes, 1, 1)
                shapes[f"{p}.downsample.bias"] = (planes * 4,)
            shapes[f"{p}.conv1.weight"] = (planes, inplanes, 1, 1)
            shapes[f"{p}.conv1.bias"] = (planes,)
            shapes[f"{p}.conv2.weight"] = (planes, planes, 3, 3)
            shapes[f"{p}.conv2.bias"] = (planes,)
            shapes[f"{p}.conv3.weight"] = (planes * 4, planes, 1, 1)
            shapes[f"{p}.conv3.bias"] = (planes * 4,)
            inplanes = planes * 4
        planes *= 2
    shapes["fc.weight"] = (num_classes, inplanes, 1, 1)
    shapes["fc.bias"] = (num_classes,)
    return shapes


def resnet_forward(params, data, layers=(3, 4, 6, 3), fast=False, taps=None):
    """ResNet v1.5 forward.  `taps`, when a dict, receives every intermediate by node name."""
    def keep(name, v):
        if taps is not None:
            taps[name] = v
        return v

    x = keep("conv1", conv2d(data, params["conv1.weight"], params["conv1.bias"], 2, 3, True,
                             fast=fast))
    x = keep("maxpool", pool2d(x, 3, 2, 1, "max"))
    for li, nblocks in enumerate(layers):
        for b in range(nblocks):
            p = f"layer{li + 1}.{b}"
            stride = 2 if (b == 0 and li > 0) else 1
            identity = x
            if b == 0:
                identity = keep(f"{p}.downsample",
                                conv2d(x, params[f"{p}.downsample.weight"],
                                       params[f"{p}.downsample.bias"], stride, 0, False, fast=fast))
            y = keep(f"{p}.conv1", conv2d(x, params[f"{p}.conv1.weight"], params[f"{p}.conv1.bias"],
                                          1, 0, True, fast=fast))
            y = keep(f"{p}.conv2", conv2d(y, params[f"{p}.conv2.weight"], params[f"{p}.conv2.bias"],
                                          stride, 1, True, fast=fast))
            x = keep(f"{p}.conv3", conv2d(y, params[f"{p}.conv3.weight"], params[f"{p}.conv3.bias"],
                                          1, 0, True, residual=identity, fast=fast))
    x = keep("avgpool", pool2d(x, x.shape[2], 1, 0, "avg"))
    x = conv2d(x, params["fc.weight"], params["fc.bias"], 1, 0, False, fast=fast)
    return keep("heads", x.reshape(x.shape[0], -1))


VGG_CFG = {
    "vgg16": (64, 64, 0, 128, 128, 0, 256, 256, 256, 0, 512, 512, 512, 0, 512, 512, 512, 0),
    "vgg19": (64, 64, 0, 128, 128, 0, 256, 256, 256, 256, 0, 512, 512, 512, 512, 0,
              512, 512, 512, 512, 0),
}


def vgg_forward(params, data, cfg="vgg16", fast=False, taps=None):
    x = data
    ci = 0
    for c in VGG_CFG[cfg]:
        if c == 0:
            x = pool2d(x, 2, 2, 0, "max")
        else:
            x = conv2d(x, params[f"features.{ci}.weight"], params[f"features.{ci}.bias"], 1, 1,
                       True, fast=fast)
            ci += 1
    # The first dense layer sees the (C, H, W)-flattened feature map: a 7x7 "valid" convolution.
    x = conv2d(x, params["classifier.0.weight"], params["classifier.0.bias"], 1, 0, True, fast=fast)
    x = conv2d(x, params["classifier.3.weight"], params["classifier.3.bias"], 1, 0, True, fast=fast)
    x = conv2d(x, params["classifier.6.weight"], params["classifier.6.bias"], 1, 0, False,
               fast=fast)
    out = x.reshape(x.shape[0], -1)
    if taps is not None:
        taps["heads"] = out
    return out


# MobileNetV2 (Sandler et al. 2018): (expansion t, output channels c, repeats n, first stride s).
MOBILENET_V2_CFG = ((1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1),
                    (6, 160, 3, 2), (6, 320, 1, 1))


def mobilenet_v2_param_shapes(num_classes=1000):
    s = {"features.0.weight": (32, 3, 3, 3), "features.0.bias": (32,)}
    cin, idx = 32, 1
    for t, c, n, _ in MOBILENET_V2_CFG:
        for _r in range(n):
            p = f"features.{idx}"
            hid = cin * t
            if t != 1:
                s[f"{p}.expand.weight"] = (hid, cin, 1, 1)
                s[f"{p}.expand.bias"] = (hid,)
            s[f"{p}.dw.weight"] = (hid, 1, 3, 3)
            s[f"{p}.dw.bias"] = (hid,)
            s[f"{p}.project.weight"] = (c, hid, 1, 1)
            s[f"{p}.project.bias"] = (c,)
            cin = c
            idx += 1
    s["features.18.weight"] = (1280, cin, 1, 1)
    s["features.18.bias"] = (1280,)
    s["classifier.weight"] = (num_classes, 1280, 1, 1)
    s["classifier.bias"] = (num_classes,)
    return s


def mobilenet_v2_forward(params, data, fast=False, taps=None):
    """Inverted-residual network with batch norm folded into the biases: 1x1 expand + ReLU6, 3x3
    depthwise + ReLU6, linear 1x1 projection, identity shortcut when stride 1 keeps the shape."""
    def keep(name, v):
        if taps is not None:
            taps[name] = v
        return v

    P = params
    x = keep("features.0", conv2d(data, P["features.0.weight"], P["features.0.bias"], 2, 1, "relu6",
                                  fast=fast))
    cin, idx = 32, 1
    for t, c, n, s0 in MOBILENET_V2_CFG:
        for r in range(n):
            p = f"features.{idx}"
            stride = s0 if r == 0 else 1
            y = x
            if t != 1:
                y = keep(f"{p}.expand", conv2d(y, P[f"{p}.expand.weight"], P[f"{p}.expand.bias"], 1, 0,
                                               "relu6", fast=fast))
            y = keep(f"{p}.dw", dwconv2d(y, P[f"{p}.dw.weight"], P[f"{p}.dw.bias"], stride, 1, "relu6"))
            res = x if (stride == 1 and cin == c) else None
            x = keep(f"{p}.project", conv2d(y, P[f"{p}.project.weight"], P[f"{p}.project.bias"], 1, 0,
                                            False, residual=res, fast=fast))
            cin = c
            idx += 1
    x = keep("features.18", conv2d(x, P["features.18.weight"], P["features.18.bias"], 1, 0, "relu6",
                                   fast=fast))
    x = keep("avgpool", pool2d(x, x.shape[2], 1, 0, "avg"))
    x = conv2d(x, P["classifier.weight"], P["classifier.bias"], 1, 0, False, fast=fast)
    return keep("heads", x.reshape(x.shape[0], -1))


DENSENET_CFG = {"densenet201": (6, 12, 48, 32), "densenet_tiny": (2, 2, 4, 2)}


def densenet_param_shapes(cfg="densenet201", growth=32, init_features=64, num_classes=1000):
    s = {"features.conv0.weight": (init_features, 3, 7, 7), "features.conv0.bias": (init_features,)}
    c = init_features
    blocks = DENSENET_CFG[cfg]
    for b, nl in enumerate(blocks):
        for l in range(nl):
            p = f"features.denseblock{b + 1}.denselayer{l + 1}"
            cin = c + growth * l
            s[f"{p}.norm1.weight"] = (cin,)
            s[f"{p}.norm1.bias"] = (cin,)
            s[f"{p}.conv1.weight"] = (4 * growth, cin, 1, 1)
            s[f"{p}.conv1.bias"] = (4 * growth,)
            s[f"{p}.conv2.weight"] = (growth, 4 * growth, 3, 3)
            s[f"{p}.conv2.bias"] = (growth,)
        c += growth * nl
        if b != len(blocks) - 1:
            t = f"features.transition{b + 1}"
            s[f"{t}.norm.weight"] = (c,)
            s[f"{t}.norm.bias"] = (c,)
            s[f"{t}.conv.weight"] = (c // 2, c, 1, 1)
            s[f"{t}.conv.bias"] = (c // 2,)
            c //= 2
    s["features.norm5.weight"] = (c,)
    s["features.norm5.bias"] = (c,)
    s["classifier.weight"] = (num_classes, c, 1, 1)
    s["classifier.bias"] = (num_classes,)
    return s


def _affine_relu(x, scale, shift):
    """relu(x * scale + shift) per channel of an NCHW tensor, in float64, rounded to fp32."""
    x = np.asarray(x, np.float64)
    y = x * np.asarray(scale, np.float64)[None, :, None, None] + np.asarray(shift, np.float64)[None, :, None, None]
    return np.maximum(y, 0.0).astype(np.float32)


def densenet_forward(params, data, cfg="densenet201", fast=False, taps=None):
    """DenseNet-BC forward: stem, dense blocks whose layers see the concatenation of everything
    before them (norm-ReLU-1x1-norm-ReLU-3x3, the inner norm folded into the 1x1 bias), transitions
    (norm-ReLU-1x1-avgpool2), final norm-ReLU, global average pool, classifier."""
    def keep(name, v):
        if taps is not None:
            taps[name] = v
        return v

    P = params
    x = keep("features.conv0", conv2d(data, P["features.conv0.weight"], P["features.conv0.bias"], 2, 3,
                                      True, fast=fast))
    x = keep("features.pool0", pool2d(x, 3, 2, 1, "max"))
    blocks = DENSENET_CFG[cfg]
    for b, nl in enumerate(blocks):
        for l in range(nl):
            p = f"features.denseblock{b + 1}.denselayer{l + 1}"
            a = keep(f"{p}.norm1", _affine_relu(x, P[f"{p}.norm1.weight"], P[f"{p}.norm1.bias"]))
            y = keep(f"{p}.conv1", conv2d(a, P[f"{p}.conv1.weight"], P[f"{p}.conv1.bias"], 1, 0, True,
                                          fast=fast))
            z = keep(f"{p}.conv2", conv2d(y, P[f"{p}.conv2.weight"], P[f"{p}.conv2.bias"], 1, 1, False,
                                          fast=fast))
            x = np.concatenate([x, z], axis=1)
        keep(f"features.denseblock{b + 1}", x)
        if b != len(blocks) - 1:
            t = f"features.transition{b + 1}"
            a = keep(f"{t}.norm", _affine_relu(x, P[f"{t}.norm.weight"], P[f"{t}.norm.bias"]))
            y = keep(f"{t}.conv", conv2d(a, P[f"{t}.conv.weight"], P[f"{t}.conv.bias"], 1, 0, False,
                                         fast=fast))
            x = keep(f"{t}.pool", pool2d(y, 2, 2, 0, "avg"))
    x = _affine_relu(x, P["features.norm5.weight"], P["features.norm5.bias"])
    x = keep("avgpool", pool2d(x, x.shape[2], 1, 0, "avg"))
    x = conv2d(x, P["classifier.weight"], P["classifier.bias"], 1, 0, False, fast=fast)
    return keep("heads", x.reshape(x.shape[0], -1))


MODELS = {
    "densenet201": lambda p, d, **kw: densenet_forward(p, d, "densenet201", **kw),
    "densenet_tiny": lambda p, d, **kw: densenet_forward(p, d, "densenet_tiny", **kw),
    "mobilenet_v2": lambda p, d, **kw: mobilenet_v2_forward(p, d, **kw),
    "resnet50": lambda p, d, **kw: resnet_forward(p, d, (3, 4, 6, 3), **kw),
    "resnet152": lambda p, d, **kw: resnet_forward(p, d, (3, 8, 36, 3), **kw),
    "resnet_tiny": lambda p, d, **kw: resnet_forward(p, d, (1, 1, 1, 1), **kw),
    "vgg16": lambda p, d, **kw: vgg_forward(p, d, "vgg16", **kw),
    "vgg19": lambda p, d, **kw: vgg_forward(p, d, "vgg19", **kw),
    "inception_v3": lambda p, d, **kw: inception_v3_forward(p, d, **kw),
}


# ---- Inception-v3 -------------------------------------------------------------------------------
# Szegedy et al. 2016 in the torchvision layer schedule and parameter names (one of the models the
# reference compiles, scripts/compile/compile.py:27-36, from relay.testing.inception_v3 with
# 3x299x299 inputs; that definition uses max pooling in the last block's pooling branch where
# torchvision, followed here, averages).  Every BasicConv2d is convolution + folded batch norm
# (a bias) + ReLU.  INCEPTION_CONVS lists (name, cin, cout, (kh, kw), stride, (ph, pw)) in
# execution order.

def _inception_blocks():
    convs = [("Conv2d_1a_3x3", 3, 32, (3, 3), 2, (0, 0)), ("Conv2d_2a_3x3", 32, 32, (3, 3), 1, (0, 0)),
             ("Conv2d_2b_3x3", 32, 64, (3, 3), 1, (1, 1)), ("Conv2d_3b_1x1", 64, 80, (1, 1), 1, (0, 0)),
             ("Conv2d_4a_3x3", 80, 192, (3, 3), 1, (0, 0))]

    def a(p, cin, pf):
        return [(f"{p}.branch1x1", cin, 64, (1, 1), 1, (0, 0)),
                (f"{p}.branch5x5_1", cin, 48, (1, 1), 1, (0, 0)), (f"{p}.branch5x5_2", 48, 64, (5, 5), 1, (2, 2)),
                (f"{p}.branch3x3dbl_1", cin, 64, (1, 1), 1, (0, 0)), (f"{p}.branch3x3dbl_2", 64, 96, (3, 3), 1, (1, 1)),
                (f"{p}.branch3x3dbl_3", 96, 96, (3, 3), 1, (1, 1)), (f"{p}.branch_pool", cin, pf, (1, 1), 1, (0, 0))]

    def b(p, cin):
        return [(f"{p}.branch3x3", cin, 384, (3, 3), 2, (0, 0)),
                (f"{p}.branch3x3dbl_1", cin, 64, (1, 1), 1, (0, 0)), (f"{p}.branch3x3dbl_2", 64, 96, (3, 3), 1, (1, 1)),
                (f"{p}.branch3x3dbl_3", 96, 96, (3, 3), 2, (0, 0))]

    def c(p, cin, c7):
        return [(f"{p}.branch1x1", cin, 192, (1, 1), 1, (0, 0)),
                (f"{p}.branch7x7_1", cin, c7, (1, 1), 1, (0, 0)), (f"{p}.branch7x7_2", c7, c7, (1, 7), 1, (0, 3)),
                (f"{p}.branch7x7_3", c7, 192, (7, 1), 1, (3, 0)),
                (f"{p}.branch7x7dbl_1", cin, c7, (1, 1), 1, (0, 0)), (f"{p}.branch7x7dbl_2", c7, c7, (7, 1), 1, (3, 0)),
                (f"{p}.branch7x7dbl_3", c7, c7, (1, 7), 1, (0, 3)), (f"{p}.branch7x7dbl_4", c7, c7, (7, 1), 1, (3, 0)),
                (f"{p}.branch7x7dbl_5", c7, 192, (1, 7), 1, (0, 3)), (f"{p}.branch_pool", cin, 192, (1, 1), 1, (0, 0))]

    def d(p, cin):
        return [(f"{p}.branch3x3_1", cin, 192, (1, 1), 1, (0, 0)), (f"{p}.branch3x3_2", 192, 320, (3, 3), 2, (0, 0)),
                (f"{p}.branch7x7x3_1", cin, 192, (1, 1), 1, (0, 0)), (f"{p}.branch7x7x3_2", 192, 192, (1, 7), 1, (0, 3)),
                (f"{p}.branch7x7x3_3", 192, 192, (7, 1), 1, (3, 0)), (f"{p}.branch7x7x3_4", 192, 192, (3, 3), 2, (0, 0))]

    def e(p, cin):
        return [(f"{p}.branch1x1", cin, 320, (1, 1), 1, (0, 0)),
                (f"{p}.branch3x3_1", cin, 384, (1, 1), 1, (0, 0)), (f"{p}.branch3x3_2a", 384, 384, (1, 3), 1, (0, 1)),
                (f"{p}.branch3x3_2b", 384, 384, (3, 1), 1, (1, 0)),
                (f"{p}.branch3x3dbl_1", cin, 448, (1, 1), 1, (0, 0)), (f"{p}.branch3x3dbl_2", 448, 384, (3, 3), 1, (1, 1)),
                (f"{p}.branch3x3dbl_3a", 384, 384, (1, 3), 1, (0, 1)), (f"{p}.branch3x3dbl_3b", 384, 384, (3, 1), 1, (1, 0)),
                (f"{p}.branch_pool", cin, 192, (1, 1), 1, (0, 0))]

    convs += a("Mixed_5b", 192, 32) + a("Mixed_5c", 256, 64) + a("Mixed_5d", 288, 64) + b("Mixed_6a", 288)
    convs += c("Mixed_6b", 768, 128) + c("Mixed_6c", 768, 160) + c("Mixed_6d", 768, 160) + c("Mixed_6e", 768, 192)
    convs += d("Mixed_7a", 768) + e("Mixed_7b", 1280) + e("Mixed_7c", 2048)
    return convs


INCEPTION_CONVS = _inception_blocks()


def inception_v3_param_shapes(num_classes=1000):
    s = {}
    for name, cin, cout, (kh, kw), _, _ in INCEPTION_CONVS:
        s[f"{name}.weight"] = (cout, cin, kh, kw)
        s[f"{name}.bias"] = (cout,)
    s["fc.weight"] = (num_classes, 2048, 1, 1)
    s["fc.bias"] = (num_classes,)
    return s


def inception_v3_forward(params, data, fast=False, taps=None):
    """Inception-v3 forward on [N][3][299][299]; returns the logits [N][1000]."""
    spec = {c[0]: c for c in INCEPTION_CONVS}

    def keep(name, v):
        if taps is not None:
            taps[name] = v
        return v

    def cv(name, x):
        _, _, _, _, stride, pad = spec[name]
        return keep(name, conv2d(x, params[f"{name}.weight"], params[f"{name}.bias"], stride, pad, True, fast=fast))

    x = cv("Conv2d_1a_3x3", data)
    x = cv("Conv2d_2a_3x3", x)
    x = cv("Conv2d_2b_3x3", x)
    x = keep("maxpool1", pool2d(x, 3, 2, 0, "max"))
    x = cv("Conv2d_3b_1x1", x)
    x = cv("Conv2d_4a_3x3", x)
    x = keep("maxpool2", pool2d(x, 3, 2, 0, "max"))
    for p in ("Mixed_5b", "Mixed_5c", "Mixed_5d"):
        b1 = cv(f"{p}.branch1x1", x)
        b5 = cv(f"{p}.branch5x5_2", cv(f"{p}.branch5x5_1", x))
        b3 = cv(f"{p}.branch3x3dbl_3", cv(f"{p}.branch3x3dbl_2", cv(f"{p}.branch3x3dbl_1", x)))
        bp = cv(f"{p}.branch_pool", pool2d(x, 3, 1, 1, "avg_pad"))
        x = keep(p, np.concatenate([b1, b5, b3, bp], 1))
    p = "Mixed_6a"
    b3 = cv(f"{p}.branch3x3", x)
    bd = cv(f"{p}.branch3x3dbl_3", cv(f"{p}.branch3x3dbl_2", cv(f"{p}.branch3x3dbl_1", x)))
    x = keep(p, np.concatenate([b3, bd, pool2d(x, 3, 2, 0, "max")], 1))
    for p in ("Mixed_6b", "Mixed_6c", "Mixed_6d", "Mixed_6e"):
        b1 = cv(f"{p}.branch1x1", x)
        b7 = cv(f"{p}.branch7x7_3", cv(f"{p}.branch7x7_2", cv(f"{p}.branch7x7_1", x)))
        bd = x
        for i in range(1, 6):
            bd = cv(f"{p}.branch7x7dbl_{i}", bd)
        bp = cv(f"{p}.branch_pool", pool2d(x, 3, 1, 1, "avg_pad"))
        x = keep(p, np.concatenate([b1, b7, bd, bp], 1))
    p = "Mixed_7a"
    b3 = cv(f"{p}.branch3x3_2", cv(f"{p}.branch3x3_1", x))
    b7 = x
    for i in range(1, 5):
        b7 = cv(f"{p}.branch7x7x3_{i}", b7)
    x = keep(p, np.concatenate([b3, b7, pool2d(x, 3, 2, 0, "max")], 1))
    for p in ("Mixed_7b", "Mixed_7c"):
        b1 = cv(f"{p}.branch1x1", x)
        t = cv(f"{p}.branch3x3_1", x)
        b3 = np.concatenate([cv(f"{p}.branch3x3_2a", t), cv(f"{p}.branch3x3_2b", t)], 1)
        t = cv(f"{p}.branch3x3dbl_2", cv(f"{p}.branch3x3dbl_1", x))
        bd = np.concatenate([cv(f"{p}.branch3x3dbl_3a", t), cv(f"{p}.branch3x3dbl_3b", t)], 1)
        bp = cv(f"{p}.branch_pool", pool2d(x, 3, 1, 1, "avg_pad"))
        x = keep(p, np.concatenate([b1, b3, bd, bp], 1))
    x = keep("avgpool", pool2d(x, x.shape[2], 1, 0, "avg"))
    x = conv2d(x, params["fc.weight"].reshape(-1, 2048, 1, 1), params["fc.bias"], 1, 0, False, fast=fast)
    return keep("heads", x.reshape(x.shape[0], -1))


def forward(model, params, data, **kw):
    return MODELS[model](params, data, **kw)


# ---- block-level preemption protocol (scripts/compile/convert_to_blp.py:39-70) -----------------

def blp_simulate(total_tiles, n_ctas, tile_cost, raise_at, cursor=0, stop_index=-1, kernel_id=0):
    """Discrete-event restatement of the persistent-CTA loop.

    Every CTA repeats: read the flag; if clear, claim tile `cursor++` (tiles >= total end the
    CTA) and spend tile_cost(tile) time units on it; if raised, record kernel_id into the stop
    index when that is still -1, and return.  `raise_at` is the time the flag flips to 1 (None =
    never).  Returns (tiles in completion order, cursor, stop_index, drain_time).
    """
    import heapq

    ready = [(0.0, c) for c in range(n_ctas)]
    heapq.heapify(ready)
    done = []
    last_exit = 0.0
    while ready:
        t, c = heapq.heappop(ready)
        if raise_at is not None and t >= raise_at:
            if stop_index == -1:
                stop_index = kernel_id
            last_exit = max(last_exit, t)
            continue
        idx = cursor
        cursor += 1
        if idx >= total_tiles:
            last_exit = max(last_exit, t)
            continue
        t_end = t + tile_cost(idx)
        done.append(idx)
        heapq.heappush(ready, (t_end, c))
    return done, cursor, stop_index, last_exit


# ---- BERT encoder (post-LayerNorm transformer, Devlin et al. 2018) ------------------------------
# Parameter names follow the Hugging Face BertModel state dict, which is what the reference's
# compile script traces (scripts/compile/compile-bert.py:33-52 uses a DistilBERT checkpoint; the
# baseline configuration asks for BERT-base).  All arithmetic is numpy float64.

def bert_param_shapes(layers=12, hidden=768, heads=12, ffn=3072, vocab=30522, max_pos=512):
    s = {
        "embeddings.word_embeddings.weight": (vocab, hidden),
        "embeddings.position_embeddings.weight": (max_pos, hidden),
        "embeddings.token_type_embeddings.weight": (2, hidden),
        "embeddings.LayerNorm.weight": (hidden,),
        "embeddings.LayerNorm.bias": (hidden,),
    }
    for i in range(layers):
        p = f"encoder.layer.{i}"
        for nm in ("query", "key", "value"):
            s[f"{p}.attention.self.{nm}.weight"] = (hidden, hidden)
            s[f"{p}.attention.self.{nm}.bias"] = (hidden,)
        s[f"{p}.attention.output.dense.weight"] = (hidden, hidden)
        s[f"{p}.attention.output.dense.bias"] = (hidden,)
        s[f"{p}.attention.output.LayerNorm.weight"] = (hidden,)
        s[f"{p}.attention.output.LayerNorm.bias"] = (hidden,)
        s[f"{p}.intermediate.dense.weight"] = (ffn, hidden)
        s[f"{p}.intermediate.dense.bias"] = (ffn,)
        s[f"{p}.output.dense.weight"] = (hidden, ffn)
        s[f"{p}.output.dense.bias"] = (hidden,)
        s[f"{p}.output.LayerNorm.weight"] = (hidden,)
        s[f"{p}.output.LayerNorm.bias"] = (hidden,)
    return s


def _layer_norm(x, g, b, eps=1e-12):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * g + b


def _gelu(x):
    from math import sqrt

    import scipy.special as sp

    return 0.5 * x * (1.0 + sp.erf(x / sqrt(2.0)))


def bert_forward(params, ids, layers=12, heads=12, taps=None):
    """ids: int64 [B][S]; returns the last hidden state [B][S][H] as float32."""
    P = {k: np.asarray(v, np.float64).reshape(v.shape[0], -1) if np.ndim(v) > 1 else np.asarray(v, np.float64)
         for k, v in params.items()}
    ids = np.asarray(ids, np.int64)
    B, S = ids.shape
    x = (P["embeddings.word_embeddings.weight"][ids] +
         P["embeddings.position_embeddings.weight"][np.arange(S)][None, :, :] +
         P["embeddings.token_type_embeddings.weight"][0][None, None, :])
    x = _layer_norm(x, P["embeddings.LayerNorm.weight"], P["embeddings.LayerNorm.bias"])
    if taps is not None:
        taps["embeddings"] = x.astype(np.float32)
    H = x.shape[-1]
    dh = H // heads
    for i in range(layers):
        p = f"encoder.layer.{i}"
        q = x @ P[f"{p}.attention.self.query.weight"].T + P[f"{p}.attention.self.query.bias"]
        k = x @ P[f"{p}.attention.self.key.weight"].T + P[f"{p}.attention.self.key.bias"]
        v = x @ P[f"{p}.attention.self.value.weight"].T + P[f"{p}.attention.self.value.bias"]
        qh = q.reshape(B, S, heads, dh).transpose(0, 2, 1, 3)
        kh = k.reshape(B, S, heads, dh).transpose(0, 2, 1, 3)
        vh = v.reshape(B, S, heads, dh).transpose(0, 2, 1, 3)
        sc = qh @ kh.transpose(0, 1, 3, 2) / np.sqrt(dh)
        sc = sc - sc.max(-1, keepdims=True)
        pr = np.exp(sc)
        pr = pr / pr.sum(-1, keepdims=True)
        ctx = (pr @ vh).transpose(0, 2, 1, 3).reshape(B, S, H)
        if taps is not None:
            taps[f"{p}.attention.context"] = ctx.astype(np.float32)
        a = ctx @ P[f"{p}.attention.output.dense.weight"].T + P[f"{p}.attention.output.dense.bias"]
        x = _layer_norm(a + x, P[f"{p}.attention.output.LayerNorm.weight"],
                        P[f"{p}.attention.output.LayerNorm.bias"])
        h = _gelu(x @ P[f"{p}.intermediate.dense.weight"].T + P[f"{p}.intermediate.dense.bias"])
        o = h @ P[f"{p}.output.dense.weight"].T + P[f"{p}.output.dense.bias"]
        x = _layer_norm(o + x, P[f"{p}.output.LayerNorm.weight"], P[f"{p}.output.LayerNorm.bias"])
        if taps is not None and i != layers - 1:
            taps[f"{p}.output"] = x.astype(np.float32)
    out = x.astype(np.float32)
    if taps is not None:
        taps["heads"] = out
    return out


# ---- DistilBERT -------------------------------------------------------------------------------
# The sequence model the reference compiles (scripts/compile/compile-bert.py:33-52: Hugging Face
# DistilBertModel, last hidden state, traced on a 6-token input).  Same post-LayerNorm encoder as
# BERT without token-type embeddings; parameter names follow the DistilBertModel state dict.

def distilbert_param_shapes(layers=6, hidden=768, heads=12, ffn=3072, vocab=30522, max_pos=512):
    s = {
        "embeddings.word_embeddings.weight": (vocab, hidden),
        "embeddings.position_embeddings.weight": (max_pos, hidden),
        "embeddings.LayerNorm.weight": (hidden,),
        "embeddings.LayerNorm.bias": (hidden,),
    }
    for i in range(layers):
        p = f"transformer.layer.{i}"
        for nm in ("q_lin", "k_lin", "v_lin", "out_lin"):
            s[f"{p}.attention.{nm}.weight"] = (hidden, hidden)
            s[f"{p}.attention.{nm}.bias"] = (hidden,)
        s[f"{p}.sa_layer_norm.weight"] = (hidden,)
        s[f"{p}.sa_layer_norm.bias"] = (hidden,)
        s[f"{p}.ffn.lin1.weight"] = (ffn, hidden)
        s[f"{p}.ffn.lin1.bias"] = (ffn,)
        s[f"{p}.ffn.lin2.weight"] = (hidden, ffn)
        s[f"{p}.ffn.lin2.bias"] = (hidden,)
        s[f"{p}.output_layer_norm.weight"] = (hidden,)
        s[f"{p}.output_layer_norm.bias"] = (hidden,)
    return s


def distilbert_forward(params, ids, layers=6, heads=12, taps=None):
    """ids: int64 [B][S]; returns the last hidden state [B][S][H] as float32 (numpy float64 inside)."""
    P = {k: np.asarray(v, np.float64).reshape(v.shape[0], -1) if np.ndim(v) > 1 else np.asarray(v, np.float64)
         for k, v in params.items()}
    ids = np.asarray(ids, np.int64)
    B, S = ids.shape
    x = P["embeddings.word_embeddings.weight"][ids] + P["embeddings.position_embeddings.weight"][np.arange(S)][None, :, :]
    x = _layer_norm(x, P["embeddings.LayerNorm.weight"], P["embeddings.LayerNorm.bias"])
    if taps is not None:
        taps["embeddings"] = x.astype(np.float32)
    H = x.shape[-1]
    dh = H // heads
    for i in range(layers):
        p = f"transformer.layer.{i}"
        lin = lambda name, t: t @ P[f"{p}.{name}.weight"].T + P[f"{p}.{name}.bias"]  # noqa: E731
        split = lambda t: t.reshape(B, S, heads, dh).transpose(0, 2, 1, 3)  # noqa: E731
        qh, kh, vh = split(lin("attention.q_lin", x)), split(lin("attention.k_lin", x)), split(lin("attention.v_lin", x))
        sc = qh @ kh.transpose(0, 1, 3, 2) / np.sqrt(dh)
        sc = sc - sc.max(-1, keepdims=True)
        pr = np.exp(sc)
        pr = pr / pr.sum(-1, keepdims=True)
        ctx = (pr @ vh).transpose(0, 2, 1, 3).reshape(B, S, H)
        if taps is not None:
            taps[f"{p}.attention.context"] = ctx.astype(np.float32)
        x = _layer_norm(lin("attention.out_lin", ctx) + x, P[f"{p}.sa_layer_norm.weight"], P[f"{p}.sa_layer_norm.bias"])
        o = lin("ffn.lin2", _gelu(lin("ffn.lin1", x)))
        x = _layer_norm(o + x, P[f"{p}.output_layer_norm.weight"], P[f"{p}.output_layer_norm.bias"])
        if taps is not None and i != layers - 1:
            taps[f"{p}.output"] = x.astype(np.float32)
    out = x.astype(np.float32)
    if taps is not None:
        taps["heads"] = out
    return out
