"""A plain, slow implementation of the Mugulorn design in float64 on the CPU: one function per mechanism,
whole sequences at once, no cache.  It shares no code with the package; the tests compare the engine with it.

A model is (config dict as in config.json, {tensor name: float64 tensor}).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequency of every pair, factor on cos and sin)."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:      # the pair index whose wave makes ``turns`` turns over the original length
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=F)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, mag: float) -> torch.Tensor:
    """x [..., T, dims] with pair (i, i + dims/2); positions [T]."""
    half = x.shape[-1] // 2
    ang = positions.to(F)[:, None] * freq[None, :]
    c, s = torch.cos(ang) * mag, torch.sin(ang) * mag
    u, v = x[..., :half], x[..., half:]
    return torch.cat([u * c - v * s, v * c + u * s], dim=-1)


def latent_kv(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict, eps: float):
    """What a latent-attention layer keeps of its input h [T, width]: the normed latent [T, kv_rank] and the
    rotated key part [T, rot_dim] that all heads share."""
    T = h.shape[0]
    R, rd = m["kv_rank"], m["rot_dim"]
    d = h @ P["dkv"].T
    c = rms_norm(d[:, :R], P["dkv.norm"], eps)
    freq, mag = yarn_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    kr = d[:, R:R + rd].clone()
    nrot = m["rot"]["dims"]
    kr[:, :nrot] = rotate_half(kr[:, :nrot], torch.arange(T), freq, mag)
    return c, kr


def latent_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict, eps: float, kv) -> torch.Tensor:
    """h [T, width]; kv = (latent, rotated key part), this layer's own or another layer's."""
    T = h.shape[0]
    H, dn, rd, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = kv
    cq = rms_norm(h @ P["dq"].T, P["dq.norm"], eps)
    q = (cq @ P["uq"].T).view(T, H, dn + rd)
    qn, qr = q[..., :dn], q[..., dn:].clone()
    freq, mag = yarn_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    nrot = m["rot"]["dims"]
    qr[..., :nrot] = rotate_half(qr[..., :nrot].transpose(0, 1), torch.arange(T), freq, mag).transpose(0, 1)
    kn = (c @ P["uk"].T).view(T, H, dn)
    v = (c @ P["uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i)
    if m.get("mask") and m["mask"].get("size"):
        seen = seen & (i - j < m["mask"]["size"])
    s = s.masked_fill(~seen[None], -math.inf)
    sink = P["sink"].view(H, 1, 1)
    top = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - top)
    a = e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))
    o = torch.einsum("hij,jhd->ihd", a, v).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ P["g"].T)
    return o @ P["o"].T


def causal_conv(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """x [T, C]; w [C, taps], the last column meets the present token; zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x], 0)
    out = b.expand(T, -1).clone()
    for k in range(taps):
        out = out + pad[k:k + T] * w[:, k]
    return out


def rglru(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict) -> torch.Tensor:
    T = h.shape[0]
    W, B = m["width"], m["blocks"]
    y = gelu_tanh(h @ P["y"].T + P["y.b"])
    u = causal_conv(h @ P["x"].T + P["x.b"], P["conv"], P["conv.b"])
    ub = u.view(T, B, W // B)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, P["ra"]) + P["ra.b"]).reshape(T, W)
    g = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, P["ri"]) + P["ri.b"]).reshape(T, W)
    a = torch.exp(-8.0 * r * torch.nn.functional.softplus(P["lam"]))
    S = torch.zeros(W, dtype=F)
    out = []
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * g[t] * u[t]
        out.append(S)
    return (torch.stack(out) * y) @ P["o"].T


def gated_gelu(h: torch.Tensor, P: Dict[str, torch.Tensor]) -> torch.Tensor:
    return (gelu_tanh(h @ P["gate"].T) * (h @ P["up"].T)) @ P["down"].T


def _sub(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its first token on."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = tensors["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        h = rms_norm(x, tensors[f"l{i}.norm1"], eps)
        P, m = _sub(tensors, f"l{i}.mix."), L["mixer"]
        if L["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latent_kv(h, P, m, eps)
                kv = kept[i]
            else:
                kv = kept[m["kv_from"]]
            x = x + mult * latent_attention(h, P, m, eps, kv)
        elif L["type"] == "rglru":
            x = x + mult * rglru(h, P, m)
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            x = x + mult * gated_gelu(rms_norm(x, tensors[f"l{i}.norm2"], eps), _sub(tensors, f"l{i}.mlp."))
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, tensors["final.norm"], eps) @ tensors["embed"].T
