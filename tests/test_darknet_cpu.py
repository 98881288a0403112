"""The darknet weight-file loader against its description in gorgonia's example
(examples/tiny-yolo-v2-coco/weights_darknet.go:13-99, net.go:88-137): five header words skipped, per
batch-normalised layer biases / gammas / means / variances / kernels in that order, the last layer
biases / kernels, batch normalisation folded on the host in float32 with epsilon 1e-6."""
import numpy as np
import pytest

from gorgonia_b200 import darknet

SMALL = (3, 4, 6, 8, 6, 4, 6, 8, 6, 5)


def _layers(seed, channels):
    g = np.random.Generator(np.random.Philox(seed))
    layers = []
    for i, shape in enumerate(darknet.layer_shapes(channels)):
        L = {"bias": g.standard_normal(shape[0]).astype(np.float32),
             "kernel": (g.standard_normal(shape) * 0.1).astype(np.float32)}
        if i < 8:
            L["gamma"] = (1 + 0.1 * g.standard_normal(shape[0])).astype(np.float32)
            L["mean"] = g.standard_normal(shape[0]).astype(np.float32)
            L["var"] = (g.random(shape[0]) + 0.5).astype(np.float32)
        layers.append(L)
    return layers


def test_file_layout_and_folding(tmp_path):
    path = str(tmp_path / "tiny.weights")
    layers = _layers(1, SMALL)
    darknet.write_tiny_yolo_v2(path, layers, seen=12345)
    words = darknet.parse(path)
    assert words[:3].view("<i4").tolist() == [0, 2, 0] and words[3:5].view("<i8")[0] == 12345
    # the first payload word is the first bias of layer 0 (lastIdx := 5 in the reference)
    assert words[5] == layers[0]["bias"][0]
    kernels, biases = darknet.load_tiny_yolo_v2(path, SMALL)
    assert [k.shape for k in kernels] == darknet.layer_shapes(SMALL)
    for i, L in enumerate(layers):
        if i == 8:
            assert np.array_equal(kernels[i], L["kernel"]) and np.array_equal(biases[i], L["bias"])
            continue
        # DenormalizeWeights restated element by element, as the Go loop runs it
        for k in range(L["bias"].size):
            scale = np.float32(L["gamma"][k] / np.float32(np.sqrt(np.float64(np.float32(L["var"][k] + np.float32(1e-6))))))
            assert biases[i][k] == np.float32(L["bias"][k] - np.float32(L["mean"][k] * scale))
            assert np.array_equal(kernels[i][k], (L["kernel"][k] * scale).astype(np.float32))
    # folding is what it claims to be: conv + batch norm == folded conv, in double
    i, L = 2, layers[2]
    x = np.random.Generator(np.random.Philox(2)).standard_normal(L["kernel"].shape[1:]).astype(np.float64)
    raw = (L["kernel"].astype(np.float64) * x[None]).sum(axis=(1, 2, 3))
    bn = (raw - L["mean"]) * L["gamma"] / np.sqrt(L["var"].astype(np.float64) + 1e-6) + L["bias"]
    folded = (kernels[i].astype(np.float64) * x[None]).sum(axis=(1, 2, 3)) + biases[i]
    assert np.allclose(folded, bn, rtol=1e-5, atol=1e-5)


def test_truncated_or_ragged_files_are_errors(tmp_path):
    path = str(tmp_path / "tiny.weights")
    darknet.write_tiny_yolo_v2(path, _layers(3, SMALL))
    raw = open(path, "rb").read()
    open(path, "wb").write(raw[:-40])
    with pytest.raises(ValueError):
        darknet.load_tiny_yolo_v2(path, SMALL)
    open(path, "wb").write(raw[:-3])
    with pytest.raises(ValueError):
        darknet.parse(path)
