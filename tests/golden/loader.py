"""Loads a golden fixture (tests/golden/<name>.npz) as a dict of torch tensors.

Large ternary-layer weights are stored as int8 grid indices under `<key>__i8`; the value the
reference saw is index * GRID in fp32, reproduced here bit for bit."""
import os

import numpy as np
import torch

GRID = np.float32(0.02 / 32.0)
_DIR = os.path.dirname(os.path.abspath(__file__))


def load(name: str) -> dict:
    out = {}
    with np.load(os.path.join(_DIR, name + ".npz")) as z:
        for k in z.files:
            a = z[k]
            if k.endswith("__i8"):
                out[k[:-4]] = torch.from_numpy(a.astype(np.float32) * GRID)
            else:
                out[k] = torch.from_numpy(np.ascontiguousarray(a))
    return out
