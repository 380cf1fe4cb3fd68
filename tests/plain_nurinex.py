"""A plain, slow implementation of the Nurinex design on the CPU: whole sequences, no cache, no
batching, one function per mechanism, float64 on the values the checkpoint stores (bfloat16 widens
exactly).  It shares no code with ``atom_b200``: it reads config.json and model.safetensors itself.

The design in this file's notation.  A layer reads one normalised copy a = rmsnorm(x; g) of the residual
stream x and adds to x the mean of two mixers' outputs, each normalised over the width with a weight of
its own, plus a feed-forward of the same a (when the layer has one):
    x <- x + (rmsnorm(A(a); g_A) + rmsnorm(R(a); g_R)) / 2 + F(a)
A is attention without any rotation (``attention``), R a recurrence over a matrix state per head
(``recurrence``), F a two-matrix feed-forward with a two-parameter activation (``feed_forward``).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- loading


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def read_tensors(model_dir: str) -> Dict[str, torch.Tensor]:
    from safetensors import safe_open

    out = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt", device="cpu") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k).to(F64)
    return out


# ----------------------------------------------------------------------------- small pieces


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over the root of (mean square + eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * g


def bias_row(n: int, rows: int, reach: float) -> int:
    """Row of the distance-bias table for a distance n >= 0: the first half of the rows stand for the
    distances 0 .. rows/2 - 1 themselves, the second half for ranges that grow geometrically until
    ``reach``; everything beyond falls into the last row."""
    half = rows // 2
    if n < half:
        return n
    step = math.log(n / half) / math.log(reach / half) * (rows - half)
    return min(rows - 1, half + int(math.floor(step)))


def query_temperature(pos: int, coef: float, every: int) -> float:
    """Factor on the query at position pos: grows with the logarithm of the number of whole blocks of
    ``every`` tokens that the sequence holds up to and including this one."""
    return 1.0 + coef * math.log((pos + 1) // every + 1)


def softplus(v: float) -> float:
    return max(v, 0.0) + math.log1p(math.exp(-abs(v)))


def xielu(z: torch.Tensor, p: float, q: float) -> torch.Tensor:
    """Quadratic above zero, a shifted exponential below, joined smoothly (value 0, slope 1/2 at zero)."""
    up = softplus(p) * z * z + 0.5 * z
    down = (0.5 + softplus(q)) * (torch.expm1(z) - z) + 0.5 * z
    return torch.where(z > 0, up, down)


# ----------------------------------------------------------------------------- attention


def attention_scores(q: torch.Tensor, k: torch.Tensor, c: dict, rel: Optional[torch.Tensor],
                     talk: Optional[torch.Tensor], first_pos: int = 0) -> torch.Tensor:
    """Scores [heads, T, T] before the softmax (entries above the diagonal are meaningless):
    temperature on the query, scaled dot product, distance bias (not scaled), then every head's score
    replaced by a fixed linear combination of all heads' scores of the same (query, key) pair.  A test of one
    mechanism alone may leave the bias or the combination out (None)."""
    T, H, _ = q.shape
    G = k.shape[1]
    temp = torch.tensor([query_temperature(first_pos + i, c["q_temp"]["coef"], c["q_temp"]["every"]) for i in range(T)], dtype=F64)
    kh = k.repeat_interleave(H // G, dim=1)           # query head h reads kv head h // (H / G)
    s = torch.einsum("ihd,jhd->hij", q * temp[:, None, None], kh) * c["scale"]
    if rel is not None:
        by_distance = torch.tensor([bias_row(n, rel.shape[0], c["bias_max"]) for n in range(T)])
        idx = torch.arange(T)
        row = by_distance[(idx[:, None] - idx[None, :]).clamp(min=0)]
        s = s + rel[row].permute(2, 0, 1)
    return s if talk is None else torch.einsum("hg,gij->hij", talk, s)


def sink_softmax(s: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """Causal softmax over keys with one more term exp(sink_h) in every row's denominator."""
    H, T, _ = s.shape
    keep = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~keep, -math.inf)
    top = torch.maximum(s.max(dim=-1, keepdim=True).values, sink.view(H, 1, 1))
    e = torch.exp(s - top)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink.view(H, 1, 1) - top))


def attention(a: torch.Tensor, w: Dict[str, torch.Tensor], p: str, c: dict, eps: float) -> torch.Tensor:
    """a: [T, width].  p: prefix of the mixer's tensors ('l3.mix.left.')."""
    T = a.shape[0]
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = (a @ w[p + "q"].T).view(T, H, dk)
    k = (a @ w[p + "k"].T).view(T, G, dk)
    v = unit_rms((a @ w[p + "v"].T).view(T, G, dv), eps)          # every value head has unit rms
    weights = sink_softmax(attention_scores(q, k, c, w[p + "rel"], w[p + "talk"]), w[p + "sink"])
    vh = v.repeat_interleave(H // G, dim=1)
    o = torch.einsum("hij,jhd->ihd", weights, vh).reshape(T, H * dv)
    return o @ w[p + "o"].T


# ----------------------------------------------------------------------------- recurrence


def shifted(a: torch.Tensor) -> torch.Tensor:
    """Row t holds row t - 1 of a; row 0 holds zeros."""
    return torch.cat([torch.zeros_like(a[:1]), a[:-1]], dim=0)


def blend(a: torch.Tensor, mu: torch.Tensor) -> torch.Tensor:
    """Each token moved towards the token before it, by mu per channel."""
    return a + (shifted(a) - a) * mu


def decay(x: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    """Per token and key channel a factor in (0, 1): exp(-exp(low-rank(x) + offset))."""
    return torch.exp(-torch.exp(torch.tanh(x @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]))


def state_scan(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, d: torch.Tensor, u: torch.Tensor,
               state: Optional[torch.Tensor] = None):
    """r, k, v, d: [T, heads, n]; u: [heads, n].  Per head a matrix S [n, n] (key channel x value channel):
    the token reads S plus its own outer product weighted by u, then S decays per key channel and takes
    the outer product.  Returns (outputs [T, heads, n], final state)."""
    T, Hh, n = r.shape
    S = torch.zeros(Hh, n, n, dtype=F64) if state is None else state.clone()
    out = torch.zeros(T, Hh, n, dtype=F64)
    for t in range(T):
        outer = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * outer)
        S = d[t][:, :, None] * S + outer
    return out, S


def recurrence(a: torch.Tensor, w: Dict[str, torch.Tensor], p: str, c: dict, eps: float) -> torch.Tensor:
    T = a.shape[0]
    Hh, n = c["heads"], c["dim"]
    r = (blend(a, w[p + "mu.r"]) @ w[p + "r"].T).view(T, Hh, n)
    k = (blend(a, w[p + "mu.k"]) @ w[p + "k"].T).view(T, Hh, n)
    v = (blend(a, w[p + "mu.v"]) @ w[p + "v"].T).view(T, Hh, n)
    gate = torch.nn.functional.silu(blend(a, w[p + "mu.g"]) @ w[p + "g"].T)
    d = decay(blend(a, w[p + "mu.w"]), w, p).view(T, Hh, n)
    out, _ = state_scan(r, k, v, d, w[p + "u"])
    y = unit_rms(out, eps).reshape(T, Hh * n) * w[p + "norm"] * gate
    return y @ w[p + "o"].T


# ----------------------------------------------------------------------------- feed-forward, layer, model


def feed_forward(a: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    pq = w[p + "act"].tolist()
    return xielu(a @ w[p + "up"].T, pq[0], pq[1]) @ w[p + "down"].T


def layer(x: torch.Tensor, w: Dict[str, torch.Tensor], entry: dict, owner: int, eps: float) -> torch.Tensor:
    if entry["type"] != "parallel":
        raise ValueError(f"layer type {entry['type']!r}")
    p = f"l{owner}."
    a = rms_norm(x, w[p + "norm1"], eps)
    left = rms_norm(attention(a, w, p + "mix.left.", entry["mixer"]["left"], eps), w[p + "mix.left.out"], eps)
    right = rms_norm(recurrence(a, w, p + "mix.right.", entry["mixer"]["right"], eps), w[p + "mix.right.out"], eps)
    y = 0.5 * (left + right)
    if entry.get("mlp") is not None:
        if entry["mlp"]["kind"] != "dense":
            raise ValueError(f"feed-forward kind {entry['mlp']['kind']!r}")
        y = y + feed_forward(a, w, p + "mlp.")
    return x + y


def owner_of(entries: List[dict], i: int) -> int:
    while entries[i].get("weights_of") is not None:
        i = entries[i]["weights_of"]
    return i


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(list(tokens))] * cfg["embedding"]["scale"]
    for i, entry in enumerate(cfg["layers"]):
        x = layer(x, w, entry, owner_of(cfg["layers"], i), eps)
        if residuals is not None:
            residuals.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
