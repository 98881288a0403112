"""Darknet (v2) weight files for the tiny-YOLOv2 tape.

Restates the host-side loader of gorgonia's example (examples/tiny-yolo-v2-coco/weights_darknet.go:13-99,
net.go:88-137): the file is a flat array of little-endian float32 words; the first five are the
header (major, minor, revision as int32 and the 64-bit `seen` counter) and are skipped; every
batch-normalised layer then stores biases, gammas, rolling means, rolling variances (one value per
output channel each) and its kernels (K, C, kh, kw); the last layer stores biases and kernels only.
Batch normalisation is folded into kernel and bias on the host, in float32 as the reference does:

    scale = gamma / float32(sqrt(float64(var + eps)))      eps = 1e-6
    bias  = bias - mean * scale
    kernel[k, :, :, :] *= scale

The folded arrays go to the device once (TinyYolo.load_weights); nothing else is computed here.
"""
import numpy as np

HEADER_WORDS = 5
EPSILON = np.float32(0.000001)


def parse(path):
    """The whole file as float32 words (ParseTinyYOLOv2). A trailing partial word is an error."""
    raw = np.fromfile(path, dtype=np.uint8)
    if raw.size % 4:
        raise ValueError(f"{path}: {raw.size} bytes is not a whole number of float32 words")
    return raw.view("<f4")


def layer_shapes(channels=(3, 16, 32, 64, 128, 256, 512, 1024, 1024, 125)):
    """(K, C, kh, kw) of the nine convolutions: 3x3 except the last, which is 1x1. The reference
    graph uses (…, 1024, 512, 425); pass its channel list for a COCO file."""
    k = [3] * 8 + [1]
    return [(channels[i + 1], channels[i], k[i], k[i]) for i in range(9)]


def fold(bias, gamma, mean, var, kernel, eps=EPSILON):
    """DenormalizeWeights: batch normalisation folded into (kernel, bias), float32 throughout except
    the square root, which the reference takes in float64."""
    bias, gamma, mean, var = (np.asarray(a, np.float32) for a in (bias, gamma, mean, var))
    root = np.sqrt((var + eps).astype(np.float64)).astype(np.float32)
    scale = (gamma / root).astype(np.float32)
    new_bias = (bias - (mean * scale).astype(np.float32)).astype(np.float32)
    new_kernel = (np.asarray(kernel, np.float32) * scale[:, None, None, None]).astype(np.float32)
    return new_kernel, new_bias


def load_tiny_yolo_v2(path, channels=(3, 16, 32, 64, 128, 256, 512, 1024, 1024, 125)):
    """-> (kernels, biases): nine float32 arrays each, batch normalisation folded in for the first eight
    layers (PrepareData + DenormalizeWeights in file order)."""
    data = parse(path)
    pos = HEADER_WORDS
    kernels, biases = [], []
    shapes = layer_shapes(channels)
    for i, shape in enumerate(shapes):
        nb, nk = shape[0], int(np.prod(shape))
        need = (4 * nb + nk) if i < 8 else (nb + nk)
        if pos + need > data.size:
            raise ValueError(f"{path}: layer {i} needs {need} words at word {pos}, the file has {data.size}")
        b = data[pos:pos + nb]
        pos += nb
        if i < 8:
            g, m, v = data[pos:pos + nb], data[pos + nb:pos + 2 * nb], data[pos + 2 * nb:pos + 3 * nb]
            pos += 3 * nb
        w = data[pos:pos + nk].reshape(shape)
        pos += nk
        if i < 8:
            w, b = fold(b, g, m, v, w)
        kernels.append(np.ascontiguousarray(w, np.float32))
        biases.append(np.ascontiguousarray(b, np.float32))
    return kernels, biases


def write_tiny_yolo_v2(path, layers, seen=0):
    """Writes a file in the same format (tests, and exporting weights): layers = nine dicts with
    'bias' and 'kernel', the first eight also 'gamma', 'mean', 'var'."""
    words = [np.array([0, 2, 0], "<i4").view("<f4"), np.array([seen], "<i8").view("<f4")]
    for i, L in enumerate(layers):
        words.append(np.asarray(L["bias"], "<f4").reshape(-1))
        if i < 8:
            for key in ("gamma", "mean", "var"):
                words.append(np.asarray(L[key], "<f4").reshape(-1))
        words.append(np.asarray(L["kernel"], "<f4").reshape(-1))
    np.concatenate(words).astype("<f4").tofile(path)
