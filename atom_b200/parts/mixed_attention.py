"""Grouped-query attention over the paged cache whose heads see one another's scores.

   [q | k | v] = x W_qkv^T;  q_h, k_g of size key_dim, v_g of size value_dim (they may differ)
   v_g <- v_g / rms(v_g)                          if value_norm; the cache holds the normalised values
   s_g[i, j]  = scale * temp(i) * (q_g[i] . k[j]) + rel[bucket(i - j), g]          j <= i
   s'_h[i, j] = sum_g talk[h, g] * s_g[i, j]                                      if head_mixing
   a_h[i, j]  = exp(s'_h[i, j]) / (exp(sink_h) + sum_j' exp(s'_h[i, j']))         (sink_h absent without sink)
   y = concat_h(sum_j a_h[i, j] v[j]) W_o^T
temp(i) = 1 + coef * ln(floor((i + 1) / every) + 1) is the query temperature; bucket(n) is the row of the
distance-bias table: n itself below half the table, logarithmic steps up to max_distance above
(``distance_thresholds``).  Positions enter through temp and rel alone; nothing is rotated.  Scores,
weights and sums are 32-bit in both precisions.  Every extra is an option of the constructor, so a
model may use any subset.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .. import native
from .base import Mixer
from .linear import linear
from .registry import register
from .spec import CacheEntry, CacheNeed, ParamSpec


def distance_thresholds(rows: int, max_distance: float) -> List[int]:
    """For a distance-bias table of ``rows`` rows: row(n) = n for n < rows/2, else
    min(rows - 1, rows/2 + floor(ln(n / (rows/2)) / ln(max_distance / (rows/2)) * (rows - rows/2))).
    Returns the distances at which rows rows/2 + 1, rows/2 + 2, ... begin (ascending), found by
    evaluating the formula in 64-bit around the place where each row must begin, so that the kernel
    compares integers and never takes a logarithm."""
    if rows < 2 or rows % 2:
        raise ValueError(f"a distance-bias table needs an even number of rows (>= 2), got {rows}")
    half = rows // 2
    if max_distance <= half:
        raise ValueError(f"max_distance ({max_distance}) must exceed half the table ({half})")
    steps = rows - half
    denom = math.log(max_distance / half)

    def row(n: int) -> int:
        return min(rows - 1, half + int(math.floor(math.log(n / half) / denom * steps)))

    out = []
    for r in range(half + 1, rows):
        # near half * (max_distance / half) ** ((r - half) / steps); the formula itself decides the exact place
        n = max(half, int(half * (max_distance / half) ** ((r - half) / steps)) - 2)
        while n > half and row(n - 1) >= r:
            n -= 1
        while row(n) < r:
            n += 1
        out.append(n)
    return out


@register("mixer", "mixed_head_attention")
class MixedHeadAttention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                 scale: Optional[float] = None, norm_eps: float = 0.0, value_norm: bool = False,
                 head_mixing: bool = False, sink: bool = False, bias_rows: int = 0, bias_max_distance: float = 0.0,
                 temp_coef: float = 0.0, temp_every: int = 0, window: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden_size, self.nh, self.nkv, self.dk, self.dv = hidden_size, num_heads, num_kv_heads, key_dim, value_dim
        self.scale = float(scale) if scale is not None else key_dim ** -0.5
        self.norm_eps, self.value_norm, self.head_mixing, self.sink = norm_eps, value_norm, head_mixing, sink
        self.bias_rows, self.bias_max_distance = int(bias_rows), float(bias_max_distance)
        self.temp_coef, self.temp_every = float(temp_coef), int(temp_every)
        self.window = window
        self._thr_host = distance_thresholds(self.bias_rows, self.bias_max_distance) if self.bias_rows else []
        self._thr = self._rel = self._talk = self._sink = None

    def params(self) -> Dict[str, ParamSpec]:
        q, k, v = self.nh * self.dk, self.nkv * self.dk, self.nkv * self.dv
        p = {
            "qkv.weight": ParamSpec((q + k + v, self.hidden_size), rows=(q, k, v)),
            "o.weight": ParamSpec((self.hidden_size, self.nh * self.dv)),
        }
        if self.bias_rows:
            p["rel"] = ParamSpec((self.bias_rows, self.nh), role="vector", init="normal")
        if self.head_mixing:
            p["talk"] = ParamSpec((self.nh, self.nh), role="vector", init="eye")
        if self.sink:
            p["sink"] = ParamSpec((self.nh,), role="vector", init="normal")
        return p

    def cache_need(self) -> CacheNeed:
        return CacheNeed("pages", window=self.window, entries=(
            CacheEntry("k", (self.nkv, self.dk)), CacheEntry("v", (self.nkv, self.dv))))

    def after_load(self) -> None:
        # the kernel reads its small tables in 32-bit (a bfloat16 value widens exactly)
        dev = self.rt.device
        self._rel = self.w_rel.float().contiguous() if self.bias_rows else None
        self._talk = self.w_talk.float().contiguous() if self.head_mixing else None
        self._sink = self.w_sink.float().contiguous() if self.sink else None
        self._thr = torch.tensor(self._thr_host, dtype=torch.int32, device=dev) if self._thr_host else None

    def forward(self, x, step, cache, writes_cache):
        T = x.shape[0]
        ws, dt = self.rt.workspace, self.rt.dtype
        nh, nkv, dk, dv = self.nh, self.nkv, self.dk, self.dv
        qkv = linear(x, self.w_qkv_weight, None, ws.get("mha.qkv", (T, nh * dk + nkv * (dk + dv)), dt))
        bt = step.block_tables[cache.group]
        if writes_cache:
            native.kv_write(qkv, nh * dk, (nh + nkv) * dk, nkv, dk, dv, self.value_norm, self.norm_eps,
                            step.positions, step.seq_of_token, bt, cache.page_size, cache.k_pages, cache.v_pages,
                            step.status)
        o = ws.get("mha.o", (T, nh * dv), dt)
        tc, nsplit = self.launch_plan(step)
        scratch = None
        if nsplit > 1:
            scratch = ws.get("mha.splits", (native.attention_mixed_scratch_elems(T, nh, dv, nsplit),), torch.float32)
        if tc:
            native.attention_mixed_tc(o, qkv, cache.k_pages, cache.v_pages, bt, step.positions, step.seq_of_token,
                                      step.cu_q, step.num_seqs, nh, nkv, dk, dv, self.scale, self.window or 0, self._rel,
                                      self.bias_rows // 2, self._thr, self._talk, self._sink, self.temp_coef,
                                      self.temp_every, nsplit, scratch)
        else:
            native.attention_mixed(o, qkv, cache.k_pages, cache.v_pages, bt, step.positions, step.seq_of_token,
                                   nh, nkv, dk, dv, self.scale, self.window or 0, self._rel, self.bias_rows // 2,
                                   self._thr, self._talk, self._sink, self.temp_coef, self.temp_every, nsplit, scratch)
        return linear(o, self.w_o_weight, None, ws.get("mha.out", (T, self.hidden_size), dt))

    def launch_plan(self, step):
        """(whether the tensor-core kernel runs, into how many shares every token's or tile's keys are cut), from
        the step's shape and its longest context (windowed layers never look further back than their window)."""
        key = ("mixed_head_attention", self.nh, self.nkv, self.dk, self.dv, self.window or 0)
        plan = step.plans.get(key)
        if plan is None:
            longest = min(step.max_ctx_len, self.window) if self.window else step.max_ctx_len
            tc = native.MIXED_TC and native.attention_mixed_tc_supports(
                self.nh, self.nkv, self.dk, self.dv, len(self._thr_host), self.head_mixing, self.rt.dtype)
            if tc:      # CTAs are tiles of 16 tokens of one request
                units = max(step.num_seqs, -(-step.num_tokens // 16))
                plan = (True, native.attention_mixed_splits(units, longest, per_sm=2, min_share=128))
            else:
                plan = (False, native.attention_mixed_splits(step.num_tokens, longest))
            step.plans[key] = plan
        return plan
