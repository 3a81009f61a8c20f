"""Tiny Pabelix configurations of the tests and helpers around them.

P differs from Q in every size; both use values that a real folder may happen
to make equal or 1 (one key/value head, one expert chosen, one group, a layer
without feed-forward, key size times two unequal to the value size, sizes that
are no multiple of 8 or 32).  Q has the sizes the tensor-core kernels take.
"""
import copy
import os

import torch

from prelude_b200.weights.random_init import random_tensors, write_random_model
from prelude_b200.weights.safetensors_io import write_safetensors


def _attn(heads, kv, dim, vdim, scale, diff, coef, every, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff,
         "q_temp": {"coef": coef, "every": every}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, ff, top, count=None, keep=None):
    r = {"experts": experts, "top": top}
    if count is not None:
        r["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


PABELIX_P = {
    "architecture": "Pabelix", "vocab": 97, "width": 40, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _attn(4, 2, 12, 20, 0.3, 0.4, 0.7, 4), "mlp": _dense(56, 0.8)},
        {"type": "attention", "mixer": _attn(2, 1, 16, 8, 0.21, 0.25, 0.3, 5), "mlp": _moe(6, 24, 2, 3, 2)},
        {"type": "attention", "mixer": _attn(4, 2, 12, 20, 0.35, 0.5, 0.2, 7, kv_from=0), "mlp": None},
        {"type": "attention", "mixer": _attn(2, 1, 16, 8, 0.25, 0.1, 0.9, 3, kv_from=1), "mlp": _moe(4, 16, 1, 1, 1)},
        {"type": "attention", "mixer": _attn(3, 3, 7, 33, 0.4, 0.7, 0.5, 16), "mlp": _moe(8, 10, 3)},
    ],
}

PABELIX_Q = {
    "architecture": "Pabelix", "vocab": 211, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _attn(4, 2, 64, 64, 0.125, 0.6, 0.5, 32), "mlp": _moe(8, 64, 2, 4, 2)},
        {"type": "attention", "mixer": _attn(2, 2, 32, 128, 0.18, 0.3, 0.25, 20), "mlp": _dense(256, 1.2)},
        {"type": "attention", "mixer": _attn(8, 2, 64, 64, 0.11, 0.45, 0.4, 50, kv_from=0), "mlp": _moe(16, 32, 4, 2, 1)},
        {"type": "attention", "mixer": _attn(4, 1, 16, 48, 0.25, 0.2, 1.0, 9), "mlp": _dense(96, 3.0)},
    ],
}

PARAMS = {"P": (PABELIX_P, dict(seed=11, std=0.25, norm_jitter=0.3), 4),
          "Q": (PABELIX_Q, dict(seed=12, std=0.12, norm_jitter=0.2), 16)}


def make_folder(tmp_path, which: str, dtype=torch.float32, config=None, **overrides):
    cfg, init, _ = PARAMS[which]
    cfg = copy.deepcopy(config or cfg)
    init = dict(init, **overrides)
    d = os.path.join(str(tmp_path), f"pabelix_{which}_{str(dtype).split('.')[-1]}_{abs(hash(str(cfg) + str(init))) % 10**8}")
    return write_random_model(d, cfg, dtype=dtype, **init)


def make_folder_from_tensors(tmp_path, name: str, cfg: dict, tensors: dict) -> str:
    """A folder with the given tensors (made or changed by a test so that a fault would show)."""
    import json
    d = os.path.join(str(tmp_path), name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors, {"format": "pt"})
    return d


__all__ = ["PABELIX_P", "PABELIX_Q", "PARAMS", "make_folder", "make_folder_from_tensors", "random_tensors"]
