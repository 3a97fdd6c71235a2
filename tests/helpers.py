"""Shared helpers of the test-suite."""
import glob
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.astype(np.int16)).view(torch.bfloat16)


def load_golden(name: str) -> dict:
    d = dict(np.load(os.path.join(GOLDEN, name + ".npz")))
    out = {}
    for k, v in d.items():
        if k.endswith("_bf16"):
            out[k[:-5]] = bf16_from_bits(v)
        elif k == "block":
            out[k] = int(v)
        else:
            out[k] = torch.from_numpy(v)
    return out


def golden_names(prefix: str):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))
