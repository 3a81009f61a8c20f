"""Tiny Kolisun configurations of the tests and helpers around them.

K has sizes no kernel likes (nothing a multiple of 8, keys and values of different sizes, a rotation over part of
a head, a window shorter than a page, one group, one norm part, three taps, a layer without feed-forward, rates
without rescaling).  L has sizes the fast kernels take.  M makes things equal or 1 that the others keep apart (one
key/value head, one head of state, as many groups as heads, two taps, a window of one page).
"""
import copy
import json
import os

import torch

from prelude_b200.weights.random_init import random_tensors, write_random_model
from prelude_b200.weights.safetensors_io import write_safetensors


def bands(factor, low, high, original):
    return {"factor": factor, "low": low, "high": high, "original": original}


def ramp(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def left(heads, kv, dim, vdim, scale, window, rot_dims, base=10000.0, scaling=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"dims": rot_dims, "base": base}}
    if window is not None:
        m["mask"] = {"size": window}
    if scaling is not None:
        m["rot"]["scaling"] = scaling
    return m


def right(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def parallel(l, r, ls, rs, ff):
    return {"type": "parallel", "mixer": {"left": l, "right": r, "left_scale": ls, "right_scale": rs},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, ff, base=10000.0, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": {"dims": rot_dim, "base": base}}
    if scaling is not None:
        m["rot"]["scaling"] = scaling
    return {"type": "latent_attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


KOLISUN_K = {
    "architecture": "Kolisun", "vocab": 97, "width": 40, "norm": {"eps": 1e-5},
    "layers": [
        latent(3, 12, 6, 20, 10, 14, 0.3, 56, base=50.0, scaling=ramp(3.0, 16, 8.0, 1.0)),
        parallel(left(4, 2, 12, 20, 0.3, 7, 8, base=100.0, scaling=bands(5.0, 1.0, 3.0, 24)), right(4, 6, 5, 1, 3, 1), 0.7, 1.3, 24),
        parallel(left(2, 1, 10, 6, 0.35, 19, 10, base=40.0), right(3, 11, 9, 3, 5, 3), 1.2, 0.5, None),
        latent(2, 7, 4, 9, 13, 5, 0.4, 18),
    ],
}

KOLISUN_L = {
    "architecture": "Kolisun", "vocab": 211, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        parallel(left(8, 2, 64, 64, 0.125, 50, 64, base=10000.0, scaling=bands(8.0, 1.0, 4.0, 64)), right(4, 32, 64, 2, 4, 4), 0.9, 1.1, 256),
        latent(4, 32, 16, 48, 64, 40, 0.14, 192, base=10000.0, scaling=ramp(6.0, 48, 16.0, 2.0)),
        latent(8, 16, 32, 16, 32, 64, 0.2, None, base=300.0),
        parallel(left(4, 4, 32, 32, 0.17, 33, 16, base=1000.0), right(8, 16, 16, 4, 4, 1), 1.0, 1.0, 96),
    ],
}

KOLISUN_M = {
    "architecture": "Kolisun", "vocab": 50, "width": 32, "norm": {"eps": 1e-6},
    "layers": [
        parallel(left(2, 1, 16, 16, 0.25, 8, 16, base=20.0), right(1, 16, 16, 1, 2, 1), 1.0, 1.0, 32),
        latent(1, 16, 16, 16, 16, 16, 0.2, 32, base=20.0, scaling=ramp(2.0, 8, 4.0, 1.0)),
        parallel(left(4, 4, 8, 8, 0.3, 1, 2, base=20.0), right(4, 8, 24, 4, 4, 4), 0.5, 2.0, 40),
    ],
}

# configuration, random-weight options, page size
PARAMS = {"K": (KOLISUN_K, dict(seed=31, std=0.25, norm_jitter=0.3), 4),
          "L": (KOLISUN_L, dict(seed=32, std=0.12, norm_jitter=0.2), 16),
          "M": (KOLISUN_M, dict(seed=33, std=0.2, norm_jitter=0.2), 8)}


def make_folder(tmp_path, which: str, dtype=torch.float32, config=None, **overrides):
    cfg, init, _ = PARAMS[which]
    cfg = copy.deepcopy(config or cfg)
    init = dict(init, **overrides)
    d = os.path.join(str(tmp_path), f"kolisun_{which}_{str(dtype).split('.')[-1]}_{abs(hash(str(cfg) + str(init))) % 10**8}")
    return write_random_model(d, cfg, dtype=dtype, **init)


def make_folder_from_tensors(tmp_path, name: str, cfg: dict, tensors: dict) -> str:
    """A folder with the given tensors (made or changed by a test so that a fault would show)."""
    d = os.path.join(str(tmp_path), name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors, {"format": "pt"})
    return d


__all__ = ["KOLISUN_K", "KOLISUN_L", "KOLISUN_M", "PARAMS", "make_folder", "make_folder_from_tensors", "random_tensors"]
