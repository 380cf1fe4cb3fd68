"""Tiny Mugulorn configurations that differ in every size, constant and in the order of layers, and a writer of
model folders with seeded random weights (bfloat16 storage) whose scales make the attention sharp and the
recurrence's memory long, so that a wrong key, a window that is one token off, a lost state or a missing sink shows.

A: attention first; a later attention layer reads the first one's cache with a WIDER window than its owner's; a
   recurrent layer with a feed-forward and one without; residual factor 0.5.
B: a recurrent layer first (one block, two taps); attention without YaRN and with fewer rotated numbers than the
   rotated part holds; a window of 7; an attention layer without any window whose cache a windowed layer reads;
   residual factor 1 and embedding scale 1.
C: sizes that are multiples of 4 but not of 8, an odd vocabulary, five blocks, a convolution of one tap and one of
   eight, a window of one token.
D: sizes of the order of real models' heads (64 + 32 numbers per head, a latent of 128).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import numpy as np
import torch

_YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}


def _att(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window, base=10000.0, dims=None, scaling=_YARN, kv_from=None,
         ff=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if scaling is not None:
        m["rot"]["scaling"] = dict(scaling)
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _rec(width, blocks, taps, ff=None):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": taps},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIGS: Dict[str, dict] = {
    "A": {"architecture": "Mugulorn", "vocab": 211, "width": 64, "residual_mult": 0.5, "embedding": {"scale": 2.0},
          "norm": {"eps": 1e-5},
          "layers": [_att(4, 16, 8, 24, 48, 32, 0.2, 24, ff=96), _rec(96, 3, 3, ff=128),
                     _att(4, 16, 8, 24, 48, 32, 0.2, 40, kv_from=0), _rec(96, 3, 3)]},
    "B": {"architecture": "Mugulorn", "vocab": 300, "width": 96, "residual_mult": 1.0, "embedding": {"scale": 1.0},
          "norm": {"eps": 1e-6},
          "layers": [_rec(128, 1, 2), _att(2, 24, 16, 16, 64, 48, 0.15, 7, base=500.0, dims=8, scaling=None, ff=72),
                     _att(3, 8, 4, 40, 24, 16, 0.3, None, scaling={"factor": 16.0, "original": 32, "fast": 4.0, "slow": 2.0}),
                     _att(6, 8, 4, 8, 32, 16, 0.35, 1000, kv_from=2, ff=130,
                          scaling={"factor": 16.0, "original": 32, "fast": 4.0, "slow": 2.0})]},
    "C": {"architecture": "Mugulorn", "vocab": 257, "width": 100, "residual_mult": 0.3, "embedding": {"scale": 10.0},
          "norm": {"eps": 3e-5},
          "layers": [_att(5, 20, 12, 28, 44, 36, 0.18, 1, ff=76), _rec(60, 5, 1), _rec(140, 4, 8, ff=52),
                     _att(1, 12, 20, 4, 20, 60, 0.25, 33, base=77.0)]},
    "D": {"architecture": "Mugulorn", "vocab": 512, "width": 256, "residual_mult": 0.7, "embedding": {"scale": 16.0},
          "norm": {"eps": 1e-5},
          "layers": [_att(8, 64, 32, 64, 128, 128, 0.1, 128, ff=512), _rec(384, 4, 4),
                     _att(8, 64, 32, 64, 128, 128, 0.1, 64, kv_from=0, ff=512)]},
}
SEEDS = {"A": 3, "B": 5, "C": 8, "D": 13}
PAGE = {"A": 16, "B": 8, "C": 16, "D": 32}


def random_tensors(cfg: dict, seed: int, overrides: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    t: Dict[str, torch.Tensor] = {}

    def mat(out, inp, gain=1.0):
        return torch.randn(out, inp, generator=g) * (gain / inp ** 0.5)

    def uni(n, lo, hi):
        return torch.rand(n, generator=g) * (hi - lo) + lo

    t["embed"] = torch.randn(cfg["vocab"], W, generator=g) / cfg["embedding"]["scale"]
    t["final.norm"] = uni(W, 0.8, 1.2)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        t[p + "norm1"] = uni(W, 0.8, 1.2)
        if L["type"] == "latent_attention":
            H, dn, rd, dv, Rq, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            sharp = (3.0 / (m["scale"] * (dn + rd) ** 0.5)) ** 0.5            # scores of a few units: a sharp softmax
            t[p + "mix.dq"] = mat(Rq, W)
            t[p + "mix.dq.norm"] = uni(Rq, 0.8, 1.2)
            t[p + "mix.uq"] = mat(H * (dn + rd), Rq, sharp)
            if m.get("kv_from") is None:
                d = mat(R + rd, W)
                d[R:] *= sharp
                t[p + "mix.dkv"] = d
                t[p + "mix.dkv.norm"] = uni(R, 0.8, 1.2)
            t[p + "mix.uk"] = mat(H * dn, R, sharp)
            t[p + "mix.uv"] = mat(H * dv, R)
            t[p + "mix.sink"] = torch.randn(H, generator=g) * 1.5
            t[p + "mix.g"] = mat(H * dv, W, 2.0)
            t[p + "mix.o"] = mat(W, H * dv, 2.0)
        else:
            C, B, taps = m["width"], m["blocks"], m["conv"]
            bw = C // B
            t[p + "mix.y"] = mat(C, W)
            t[p + "mix.y.b"] = torch.randn(C, generator=g) * 0.3
            t[p + "mix.x"] = mat(C, W)
            t[p + "mix.x.b"] = torch.randn(C, generator=g) * 0.3
            t[p + "mix.conv"] = torch.randn(C, taps, generator=g) * (0.8 / taps ** 0.5)
            t[p + "mix.conv.b"] = torch.randn(C, generator=g) * 0.2
            t[p + "mix.ra"] = torch.randn(B, bw, bw, generator=g) * (1.5 / bw ** 0.5)
            t[p + "mix.ra.b"] = torch.randn(B, bw, generator=g)
            t[p + "mix.ri"] = torch.randn(B, bw, bw, generator=g) * (1.5 / bw ** 0.5)
            t[p + "mix.ri.b"] = torch.randn(B, bw, generator=g)
            t[p + "mix.lam"] = uni(C, -6.0, -0.5)              # decays from ~0.1 to ~0.99 a token
            t[p + "mix.o"] = mat(W, C, 2.0)
        if L["mlp"] is not None:
            ff = L["mlp"]["ff"]
            t[p + "norm2"] = uni(W, 0.8, 1.2)
            t[p + "mlp.gate"] = mat(ff, W, 1.5)
            t[p + "mlp.up"] = mat(ff, W)
            t[p + "mlp.down"] = mat(W, ff, 1.5)
    if overrides:
        for k, v in overrides.items():
            assert t[k].shape == v.shape, k
            t[k] = v
    return {k: v.to(torch.bfloat16).contiguous() for k, v in t.items()}


def write_model(cfg: dict, model_dir: str, seed: int, overrides: Optional[Dict[str, torch.Tensor]] = None) -> None:
    from safetensors.torch import save_file

    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    save_file(random_tensors(cfg, seed, overrides), os.path.join(model_dir, "model.safetensors"), metadata={"format": "pt"})


def read_model(model_dir: str):
    """(config dict, {name: float64 tensor}) for the plain implementation."""
    from safetensors.torch import load_file

    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, {k: v.double() for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}


def prompts(cfg: dict, lengths: List[int], seed: int) -> List[List[int]]:
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]
