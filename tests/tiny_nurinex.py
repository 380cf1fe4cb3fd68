"""Tiny Nurinex configurations that differ in every size, constant and in the order of layers, and a
writer of model folders with seeded random weights (bfloat16 storage) whose scales make the attention
sharp and the recurrence's memory long enough that a wrong key, a lost state or a missing sink shows.

P: key size != value size, a layer without feed-forward, a layer that runs another's tensors.
Q: every layer its own sizes; as many kv heads as heads in one layer and a single kv head in the other;
   a temperature that grows every token; a chain of layers running another's tensors.
R: sizes that are multiples of 4 but not of 8, an odd vocabulary.
S: head sizes of real models (128 for attention, 64 for the recurrence).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import numpy as np
import torch


def _left(heads, kv, dim, vdim, scale, rows, reach, coef, every):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": reach,
            "q_temp": {"coef": coef, "every": every}, "_rows": rows}


def _layer(left, right_heads, right_dim, rank, ff, weights_of=None):
    e = {"type": "parallel", "mixer": {"left": dict(left), "right": {"heads": right_heads, "dim": right_dim, "_rank": rank}},
         "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


_PL = _left(4, 2, 16, 32, 0.3, 8, 50, 0.7, 8)
_Q0 = _left(6, 6, 24, 16, 0.21, 16, 40.5, 0.25, 1)
_Q1 = _left(2, 1, 40, 48, 0.16, 4, 1000, 0.4, 100)
_RL = _left(5, 5, 20, 12, 0.25, 12, 30, 0.3, 5)
_SL = _left(4, 1, 128, 128, 0.09, 32, 128, 0.5, 32)

# keys that begin with "_" are sizes that only the tensors' shapes carry; they are not written to config.json
CONFIGS: Dict[str, dict] = {
    "P": {"architecture": "Nurinex", "vocab": 211, "width": 64, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
          "layers": [_layer(_PL, 2, 32, 8, 96), _layer(_PL, 2, 32, 8, None), _layer(_PL, 2, 32, 8, 96, weights_of=0)]},
    "Q": {"architecture": "Nurinex", "vocab": 300, "width": 96, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-6},
          "layers": [_layer(_Q0, 3, 32, 4, 130), _layer(_Q1, 6, 16, 12, 72), _layer(_Q1, 6, 16, 12, 72, weights_of=1),
                     _layer(_Q1, 6, 16, 12, 72, weights_of=2), _layer(_Q0, 3, 32, 4, 130, weights_of=0)]},
    "R": {"architecture": "Nurinex", "vocab": 257, "width": 100, "embedding": {"scale": 10.0}, "norm": {"eps": 3e-5},
          "layers": [_layer(_RL, 5, 20, 6, 76), _layer(_RL, 5, 20, 6, 76)]},
    "S": {"architecture": "Nurinex", "vocab": 512, "width": 256, "embedding": {"scale": 16.0}, "norm": {"eps": 1e-5},
          "layers": [_layer(_SL, 4, 64, 32, 512), _layer(_SL, 4, 64, 32, 512)]},
}
SEEDS = {"P": 3, "Q": 5, "R": 8, "S": 13}
PAGE = {"P": 16, "Q": 8, "R": 16, "S": 32}


def public_config(cfg: dict) -> dict:
    """config.json as a checkpoint carries it: without the sizes that stand in the shapes alone."""
    def strip(o):
        if isinstance(o, dict):
            return {k: strip(v) for k, v in o.items() if not k.startswith("_")}
        if isinstance(o, list):
            return [strip(v) for v in o]
        return o
    return strip(cfg)


def random_tensors(cfg: dict, seed: int, overrides: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    t: Dict[str, torch.Tensor] = {}

    def mat(out, inp, gain=1.0):
        return torch.randn(out, inp, generator=g) * (gain / inp ** 0.5)

    def uni(n, lo, hi):
        return torch.rand(n, generator=g) * (hi - lo) + lo

    t["embed"] = torch.randn(cfg["vocab"], W, generator=g) / cfg["embedding"]["scale"]
    t["head"] = mat(cfg["vocab"], W)
    t["final.norm"] = uni(W, 0.8, 1.2)
    for i, L in enumerate(cfg["layers"]):
        if L.get("weights_of") is not None:
            continue
        lf, rt = L["mixer"]["left"], L["mixer"]["right"]
        p = f"l{i}."
        t[p + "norm1"] = uni(W, 0.8, 1.2)
        H, G, dk, dv = lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"]
        sharp = (2.5 / (lf["scale"] * dk ** 0.5)) ** 0.5           # scores of a few units: a sharp softmax
        t[p + "mix.left.q"] = mat(H * dk, W, sharp)
        t[p + "mix.left.k"] = mat(G * dk, W, sharp)
        t[p + "mix.left.v"] = mat(G * dv, W)
        t[p + "mix.left.o"] = mat(W, H * dv)
        t[p + "mix.left.rel"] = torch.randn(lf["_rows"], H, generator=g)
        t[p + "mix.left.talk"] = torch.eye(H) + 0.3 * torch.randn(H, H, generator=g)
        t[p + "mix.left.sink"] = torch.randn(H, generator=g)
        t[p + "mix.left.out"] = uni(W, 0.8, 1.2)
        Hh, n, rank = rt["heads"], rt["dim"], rt["_rank"]
        for s in "rkvgw":
            t[p + "mix.right.mu." + s] = uni(W, 0.2, 0.8)
        for s in "rkvg":
            t[p + "mix.right." + s] = mat(Hh * n, W)
        t[p + "mix.right.w1"] = mat(rank, W)
        t[p + "mix.right.w2"] = mat(Hh * n, rank)
        t[p + "mix.right.w0"] = torch.randn(Hh * n, generator=g) * 1.5 - 2.5     # decays from ~0.5 to ~0.999
        t[p + "mix.right.u"] = torch.randn(Hh, n, generator=g) * 0.5
        t[p + "mix.right.norm"] = uni(Hh * n, 0.8, 1.2)
        t[p + "mix.right.o"] = mat(W, Hh * n)
        t[p + "mix.right.out"] = uni(W, 0.8, 1.2)
        if L["mlp"] is not None:
            t[p + "mlp.up"] = mat(L["mlp"]["ff"], W)
            t[p + "mlp.down"] = mat(W, L["mlp"]["ff"], 0.5)
            t[p + "mlp.act"] = torch.randn(2, generator=g)
    if overrides:
        for k, v in overrides.items():
            assert t[k].shape == v.shape, k
            t[k] = v
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def write_model(cfg: dict, model_dir: str, seed: int, overrides: Optional[Dict[str, torch.Tensor]] = None) -> None:
    from safetensors.torch import save_file

    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(public_config(cfg), f, indent=1)
    save_file(random_tensors(cfg, seed, overrides), os.path.join(model_dir, "model.safetensors"), metadata={"format": "pt"})


def prompts(cfg: dict, lengths: List[int], seed: int) -> List[List[int]]:
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]
