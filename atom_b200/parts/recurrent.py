"""A recurrent mixer with a matrix state per head, a decay per key channel that depends on the token,
and a bonus for the present token (time mixing in the manner of RWKV).

With h' the token before h in the request (zeros before the first), each of the five branches reads its own blend
   m_s = h + (h' - h) * mu_s,   s in (r, k, v, g, w)
   r, k, v = W_r m_r, W_k m_k, W_v m_v   (heads x head_dim each);   gate = silu(W_g m_g)
   decay w = exp(-exp(W_w2 tanh(W_w1 m_w) + w0))                     per head and key channel
   o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t;    S_t = diag(w_t) S_(t-1) + k_t v_t^T      per head
   y = W_o (concat_heads(o / rms(o)) * norm * gate)
The state (S in 32-bit, and the last h of the step in the activation type) lives in the request's state slot;
the recurrence, the decay and the unit norm are 32-bit in both precisions.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import native
from .base import Mixer
from .linear import linear
from .registry import register
from .spec import CacheEntry, CacheNeed, ParamSpec

_BRANCHES = ("r", "k", "v", "g", "w")


@register("mixer", "decayed_state_mixing")
class DecayedStateMixing(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, decay_rank: int, norm_eps: float):
        if not native.wkv_supports(head_dim, head_dim):
            raise ValueError(f"decayed_state_mixing: head_dim {head_dim} is beyond what the kernel takes (128)")
        self.hidden_size, self.nh, self.hd, self.rank, self.norm_eps = hidden_size, num_heads, head_dim, decay_rank, norm_eps

    def params(self) -> Dict[str, ParamSpec]:
        W, D = self.hidden_size, self.nh * self.hd
        return {
            "mu": ParamSpec((len(_BRANCHES), W), role="vector", init="half", rows=(1,) * len(_BRANCHES),
                            members_lack_axis=True),
            "r.weight": ParamSpec((D, W)), "k.weight": ParamSpec((D, W)), "v.weight": ParamSpec((D, W)),
            "g.weight": ParamSpec((D, W)),
            "w1.weight": ParamSpec((self.rank, W)), "w2.weight": ParamSpec((D, self.rank)),
            "w0": ParamSpec((D,), role="vector", init="zeros"),
            "u": ParamSpec((self.nh, self.hd), role="vector", init="normal"),
            "norm": ParamSpec((D,), role="vector", init="norm"),
            "o.weight": ParamSpec((W, D)),
        }

    def cache_need(self) -> CacheNeed:
        return CacheNeed("state", states=(
            CacheEntry("wkv", (self.nh, self.hd, self.hd), "float32"),
            CacheEntry("shift", (self.hidden_size,), "compute")))

    def forward(self, x, step, cache, writes_cache):
        T, W = x.shape
        D = self.nh * self.hd
        ws, dt = self.rt.workspace, self.rt.dtype
        mixes = ws.get("dsm.mixes", (len(_BRANCHES), T, W), dt)
        native.token_shift_mix(mixes, x, self.w_mu, cache.states["shift"], step.seq_of_token, step.cu_q,
                               step.state_slots, writes_cache)
        r = linear(mixes[0], self.w_r_weight, None, ws.get("dsm.r", (T, D), dt))
        k = linear(mixes[1], self.w_k_weight, None, ws.get("dsm.k", (T, D), dt))
        v = linear(mixes[2], self.w_v_weight, None, ws.get("dsm.v", (T, D), dt))
        g = linear(mixes[3], self.w_g_weight, None, ws.get("dsm.g", (T, D), dt))
        a = linear(mixes[4], self.w_w1_weight, None, ws.get("dsm.a", (T, self.rank), dt))
        native.tanh_(a)
        d = linear(a, self.w_w2_weight, None, ws.get("dsm.d", (T, D), torch.float32))
        y = ws.get("dsm.y", (T, D), dt)
        native.wkv(y, r, k, v, d, g, self.w_w0, self.w_u, self.w_norm, cache.states["wkv"], step.cu_q,
                   step.state_slots, step.num_seqs, self.nh, self.hd, self.hd, self.norm_eps, writes_cache)
        return linear(y, self.w_o_weight, None, ws.get("dsm.out", (T, W), dt))
