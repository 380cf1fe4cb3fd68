"""A recurrent mixer with one real number of state per channel, gated by the input (the recurrent block of
Griffin, De et al. 2024, with its real-gated linear recurrent unit).

   [yp | xp] = W_in h                                   two branches of ``width`` channels, one product
   y = gelu_tanh(yp + b_y)
   u = conv(xp + b_x)                                   causal, per channel, ``taps`` taps, zeros before the start
   per block b of width / blocks channels:  r = sigmoid(A_b u_b + a_b),  i = sigmoid(I_b u_b + i_b)
   a = exp(-decay * r * softplus(lam)),   S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t       S = 0 before the first token
   out = W_o (S * y)
A request's state is S (32-bit) and the last taps - 1 inputs of the convolution; both live in its state slot and
are zero at its first token.  Gates, decay and state are 32-bit in both precisions; the gates' products hand
their sums over in 32-bit.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import native
from .base import Mixer
from .linear import PendingProduct, linear, may_defer
from .registry import register
from .spec import CacheEntry, CacheNeed, ParamSpec


@register("mixer", "rglru")
class GatedLinearRecurrence(Mixer):
    graph_safe = True
    takes_scaled_rows = True      # x may be ScaledRows: the branches' product finishes the norm
    defers_output = True          # forward(..., defer=True) may hand the output projection on unrun

    def __init__(self, hidden_size: int, width: int, blocks: int, taps: int, decay: float = 8.0):
        if width % blocks:
            raise ValueError(f"rglru: width {width} is no multiple of its {blocks} blocks")
        if not 1 <= taps <= 32:
            raise ValueError(f"rglru: {taps} taps are beyond what the kernels take (1 to 32)")
        self.hidden_size, self.width, self.blocks, self.taps, self.decay = hidden_size, width, blocks, taps, float(decay)

    def params(self) -> Dict[str, ParamSpec]:
        H, W, B = self.hidden_size, self.width, self.blocks
        bw = W // B
        return {
            "in.weight": ParamSpec((2 * W, H), rows=(W, W)),
            "y.bias": ParamSpec((W,), role="vector", init="zeros"),
            "x.bias": ParamSpec((W,), role="vector", init="zeros"),
            "conv.weight": ParamSpec((W, self.taps), role="vector", init="half"),
            "conv.bias": ParamSpec((W,), role="vector", init="zeros"),
            "gates.weight": ParamSpec((B, 2 * bw, bw), rows=(bw, bw), stack_dim=1),
            "gates.bias": ParamSpec((B, 2 * bw), role="vector", init="zeros", rows=(bw, bw), stack_dim=1),
            "lam": ParamSpec((W,), role="vector", init="normal"),
            "o.weight": ParamSpec((H, W)),
        }

    def cache_need(self) -> CacheNeed:
        return CacheNeed("state", states=(
            CacheEntry("h", (self.width,), "float32"),
            CacheEntry("conv", (max(self.taps - 1, 1), self.width), "compute")))

    def forward(self, x, step, cache, writes_cache, defer=False):
        T = x.shape[0]
        W, B = self.width, self.blocks
        bw = W // B
        ws, dt = self.rt.workspace, self.rt.dtype
        proj = linear(x, self.w_in_weight, None, ws.get("rg.in", (T, 2 * W), dt))
        yp, xp = proj[:, :W], proj[:, W:]
        conv_state = cache.states["conv"][:, : self.taps - 1]
        u = ws.get("rg.u", (T, W), dt)
        native.causal_conv(u, xp, self.w_x_bias, self.w_conv_weight, self.w_conv_bias, conv_state, step.seq_of_token,
                           step.cu_q, step.state_slots)
        gates = ws.get("rg.gates", (T, B, 2 * bw), torch.float32)
        native.gemm_batched(gates, u.view(T, B, bw), self.w_gates_weight)
        out = ws.get("rg.s", (T, W), dt)
        native.rglru_scan(out, gates, self.w_gates_bias, self.w_lam, u, yp, xp, self.w_y_bias, self.w_x_bias,
                          cache.states["h"], conv_state, step.cu_q, step.state_slots, step.num_seqs, self.taps,
                          self.decay, writes_cache)
        res = ws.get("rg.out", (T, self.hidden_size), dt)
        if defer and may_defer(out, self.w_o_weight):
            return PendingProduct(out, self.w_o_weight, None, res)
        return linear(out, self.w_o_weight, None, res)
