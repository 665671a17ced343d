"""Model descriptions for the host runtime's GraphTask (`aker -m <dir>/model.json`).

The reference compiles its models in: NNFusion emits one CUDA source per model, `src/nnf/gen_code.py` rewrites it
into kernel classes, and the classes read their weights from `Constant/Constant_<n>_0.bin` (raw fp32).  Here a model is
a JSON description interpreted at start-up plus the same kind of constant files, in NNFusion's layouts: convolution
filters [3][3][Cin][Cout], dense weights [in][out], biases [out].  `write_model` emits both from numpy arrays;
`vgg16_description` is the layer list of VGG16.

    python -m tacker_b200.nnf --vgg16 out_dir [--seed 1]     # VGG16 with He-initialised random constants
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np


def vgg16_description(num_classes: int = 1000) -> list:
    layers = []
    for c in (64, 64, -1, 128, 128, -1, 256, 256, 256, -1, 512, 512, 512, -1, 512, 512, 512, -1):
        layers.append({"op": "maxpool"} if c < 0 else {"op": "conv3x3", "out": c, "act": "relu"})
    layers += [{"op": "dense", "out": 4096, "act": "relu"}, {"op": "dense", "out": 4096, "act": "relu"},
               {"op": "dense", "out": num_classes, "act": "none"}, {"op": "softmax"}]
    return layers


def random_constants(layers: list, h: int, w: int, c: int, seed: int = 1) -> list:
    """One (weight, bias) pair of float32 arrays per conv3x3 / dense layer, He-initialised; None for the others."""
    rng = np.random.default_rng(seed)
    out, features = [], None
    for l in layers:
        if l["op"] == "conv3x3":
            k = 9 * c
            out.append((rng.standard_normal((3, 3, c, l["out"])).astype(np.float32) * np.float32(np.sqrt(2.0 / k)),
                        rng.uniform(-0.05, 0.05, l["out"]).astype(np.float32)))
            c = l["out"]
        elif l["op"] == "maxpool":
            h, w = h // 2, w // 2
            out.append(None)
        elif l["op"] == "dense":
            k = features if features is not None else h * w * c
            out.append((rng.standard_normal((k, l["out"])).astype(np.float32) * np.float32(np.sqrt(2.0 / k)),
                        rng.uniform(-0.05, 0.05, l["out"]).astype(np.float32)))
            features = l["out"]
        else:
            out.append(None)
    return out


def write_model(out_dir: str, name: str, h: int, w: int, c: int, layers: list, constants: list, config: str = "vgg16",
                input_array: np.ndarray | None = None, input_seed: int = 42) -> str:
    """Writes <out_dir>/model.json and <out_dir>/Constant/Constant_<n>_0.bin; returns the path of the description."""
    cdir = os.path.join(out_dir, "Constant")
    os.makedirs(cdir, exist_ok=True)
    n, described = 0, []
    for l, cst in zip(layers, constants):
        d = dict(l)
        if cst is not None:
            for key, arr in (("weight", cst[0]), ("bias", cst[1])):
                n += 1
                fname = f"Constant_{n}_0.bin"
                np.ascontiguousarray(arr, dtype="<f4").tofile(os.path.join(cdir, fname))
                d[key] = fname
        described.append(d)
    inp = {"h": h, "w": w, "c": c, "seed": input_seed}
    if input_array is not None:
        np.ascontiguousarray(input_array, dtype="<f4").reshape(h, w, c).tofile(os.path.join(cdir, "input_0.bin"))
        inp["file"] = "input_0.bin"
    path = os.path.join(out_dir, "model.json")
    with open(path, "w") as f:
        json.dump({"name": name, "config": config, "input": inp, "constants": "Constant", "layers": described}, f, indent=1)
        f.write("\n")
    return path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--vgg16", metavar="DIR", required=True, help="write the VGG16 description and random constants there")
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--classes", type=int, default=1000)
    args = ap.parse_args(argv)
    layers = vgg16_description(args.classes)
    print(write_model(args.vgg16, "vgg16_file", 224, 224, 3, layers, random_constants(layers, 224, 224, 3, args.seed)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
