"""numpy forward of a model description (tacker_b200.nnf / the host runtime's GraphTask).  Test infrastructure.

fp16-rounded GEMM operands with binary32 accumulation, fp32 bias and activation, activations between convolutions kept
as fp16 (the bordered images of the runtime), NHWC; constants read from the files the description names."""
import json
import os

import numpy as np


def _f16(a):
    return a.astype(np.float16).astype(np.float32)


def forward(description_path, input_array):
    d = json.load(open(description_path))
    cdir = os.path.join(os.path.dirname(description_path), d.get("constants", "."))
    load = lambda name, shape: np.fromfile(os.path.join(cdir, name), dtype="<f4").reshape(shape)
    h, w, c = d["input"]["h"], d["input"]["w"], d["input"]["c"]
    x = input_array.reshape(h, w, c).astype(np.float32)
    row = None
    for l in d["layers"]:
        if l["op"] == "conv3x3":
            wt, b = load(l["weight"], (3, 3, c, l["out"])), load(l["bias"], (l["out"],))
            xp = np.zeros((h + 2, w + 2, c), np.float32)
            xp[1:-1, 1:-1] = _f16(x)
            cols = np.concatenate([xp[i:i + h, j:j + w] for i in range(3) for j in range(3)], axis=2).reshape(h * w, 9 * c)
            y = cols @ _f16(wt.reshape(9 * c, l["out"])) + b
            if l.get("act", "relu") == "relu":
                y = np.maximum(y, 0.0)
            x = _f16(y.astype(np.float32)).reshape(h, w, l["out"])     # stored as an fp16 image
            c = l["out"]
        elif l["op"] == "maxpool":
            x = x.reshape(h // 2, 2, w // 2, 2, c).max(axis=(1, 3))
            h, w = h // 2, w // 2
        elif l["op"] == "dense":
            if row is None:
                row = x.reshape(1, h * w * c)
            wt, b = load(l["weight"], (row.shape[1], l["out"])), load(l["bias"], (l["out"],))
            y = _f16(row) @ _f16(wt) + b
            row = (np.maximum(y, 0.0) if l.get("act", "none") == "relu" else y).astype(np.float32)
        elif l["op"] == "softmax":
            e = np.exp(row[0] - row[0].max())
            return row[0], (e / e.sum()).astype(np.float32)
    return row[0], None
