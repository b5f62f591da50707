"""Synthetic ResNet generators (random-initialised, real file formats).

``resnet50_onnx`` writes the classification model of the CPU benchmark configuration:
ResNet-50 v1.5 (stride 2 in the 3x3 of each down-sampling bottleneck), ONNX opset 11,
seed-0 fp32 weights, 1000 classes, input ``[N,3,224,224]``. The reference ships no
network definitions - its models arrive as downloaded files
(tests/models/test_ppyoloe.py:24-30) - so the generators stand in for those files.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np

from ..importer.onnx_format import save_onnx
from ..ir.graph import Graph


def _he(rng, shape):
    fan_in = int(np.prod(shape[1:]))
    return (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)


def _conv_bn(g: Graph, rng, x: str, cin: int, cout: int, k: int, stride: int, relu: bool, name: str) -> str:
    w = g.add_initializer(f"{name}.weight", _he(rng, (cout, cin, k, k)))
    y = g.op("Conv", x, w, kernel_shape=[k, k], strides=[stride, stride], pads=[k // 2] * 4, dilations=[1, 1], group=1)
    scale = g.add_initializer(f"{name}.bn.scale", (1.0 + 0.1 * rng.standard_normal(cout)).astype(np.float32))
    bias = g.add_initializer(f"{name}.bn.bias", (0.1 * rng.standard_normal(cout)).astype(np.float32))
    mean = g.add_initializer(f"{name}.bn.mean", (0.1 * rng.standard_normal(cout)).astype(np.float32))
    var = g.add_initializer(f"{name}.bn.var", (1.0 + 0.1 * rng.random(cout)).astype(np.float32))
    y = g.op("BatchNormalization", y, scale, bias, mean, var, epsilon=1e-5)
    return g.op("Relu", y) if relu else y


def build_resnet(layers: Sequence[int] = (3, 4, 6, 3), num_classes: int = 1000, seed: int = 0, width: int = 64,
                 batch="N", image: int = 224, softmax: bool = False) -> Graph:
    rng = np.random.default_rng(seed)
    g = Graph("resnet", opset=11)
    x = g.add_input("input", "float32", [batch, 3, image, image])
    y = _conv_bn(g, rng, x, 3, width, 7, 2, True, "conv1")
    y = g.op("MaxPool", y, kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1])
    cin = width
    for si, n in enumerate(layers):
        mid = width * (2 ** si)
        cout = mid * 4
        for bi in range(n):
            stride = 2 if (bi == 0 and si > 0) else 1
            name = f"layer{si + 1}.{bi}"
            identity = y
            z = _conv_bn(g, rng, y, cin, mid, 1, 1, True, name + ".conv1")
            z = _conv_bn(g, rng, z, mid, mid, 3, stride, True, name + ".conv2")     # v1.5: stride on the 3x3
            z = _conv_bn(g, rng, z, mid, cout, 1, 1, False, name + ".conv3")
            if bi == 0:
                identity = _conv_bn(g, rng, y, cin, cout, 1, stride, False, name + ".downsample")
            y = g.op("Relu", g.op("Add", z, identity))
            cin = cout
    y = g.op("GlobalAveragePool", y)
    y = g.op("Flatten", y, axis=1)
    w = g.add_initializer("fc.weight", (rng.standard_normal((num_classes, cin)) * 0.01).astype(np.float32))
    b = g.add_initializer("fc.bias", np.zeros(num_classes, np.float32))
    y = g.op("Gemm", y, w, b, alpha=1.0, beta=1.0, transB=1)
    if softmax:
        y = g.op("Softmax", y, axis=1)
    g.nodes[-1].outputs = ["output"]
    g.add_output("output", "float32", [batch, num_classes])
    return g


def resnet50_onnx(path: Optional[str] = None, seed: int = 0, **kw) -> bytes:
    data = save_onnx(build_resnet((3, 4, 6, 3), seed=seed, **kw))
    if path:
        with open(path, "wb") as f:
            f.write(data)
    return data


def resnet18_like_onnx(path: Optional[str] = None, seed: int = 0, **kw) -> bytes:
    """A small bottleneck ResNet for fast tests."""
    kw.setdefault("width", 16)
    kw.setdefault("num_classes", 10)
    kw.setdefault("image", 64)
    data = save_onnx(build_resnet((1, 1, 1, 1), seed=seed, **kw))
    if path:
        with open(path, "wb") as f:
            f.write(data)
    return data
