"""Two mixers side by side on the same input, their outputs each passed through an RMSNorm of its own
(plain weight) and averaged:   y = (rmsnorm(left(h); w_left) + rmsnorm(right(h); w_right)) / 2.

The members are mixers of any registered kind, given as PartSpecs; their parameters appear under
``<member>.<name>``, the two output-norm weights as ``<member>.out``.  What the members keep between
steps is put together into one need (``CacheNeed.merged``: the pages of the one that keeps pages, every
member's state arrays), and each member sees its own share of the run entry's cache slot.  An arrangement
that adds the mixer's output to the residual stream anyway may pass ``add_to=(residual, extra)``: norms,
average, the optional extra addend and the residual add are then one kernel in 32-bit; ``extra`` may be a
function that computes the addend, which then runs while the second member is busy on its own stream.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import native
from . import registry
from .base import Mixer
from .registry import register
from .spec import CacheNeed, ParamSpec, PartSpec


# Rows of a step from which the second member runs on a stream of its own (0: never).
OVERLAP_MIN_ROWS = 256
_side_streams = {}


def side_by_side_spec(hidden_size: int, norm_eps: float, members: Mapping[str, PartSpec],
                      out_sources: Mapping[str, str]) -> PartSpec:
    """The PartSpec of a pair of mixers: the members' checkpoint names move under ``<member>.``;
    out_sources: member -> checkpoint tensor of its output-norm weight."""
    sources = {}
    for name, m in members.items():
        sources.update({f"{name}.{k}": v for k, v in m.sources.items()})
        sources[f"{name}.out"] = (out_sources[name],)
    return PartSpec("side_by_side", {"hidden_size": hidden_size, "norm_eps": norm_eps,
                                     "members": {n: PartSpec(m.kind, dict(m.args)) for n, m in members.items()}},
                    sources)


@register("mixer", "side_by_side")
class SideBySide(Mixer):
    adds_to_residual = True       # forward takes add_to=(residual, extra addend or None) and then returns None

    def __init__(self, hidden_size: int, norm_eps: float, members: Mapping[str, PartSpec]):
        if len(members) != 2:
            raise ValueError("side_by_side takes exactly two members")
        self.hidden_size, self.norm_eps = hidden_size, norm_eps
        self.members = {n: registry.build("mixer", m) for n, m in members.items()}
        self._side = None

    @property
    def graph_safe(self) -> bool:
        return all(m.graph_safe for m in self.members.values())

    def params(self) -> Dict[str, ParamSpec]:
        p = {}
        for n, m in self.members.items():
            p.update({f"{n}.{k}": v for k, v in m.params().items()})
            p[f"{n}.out"] = ParamSpec((self.hidden_size,), role="vector", init="norm")
        return p

    def cache_need(self):
        return CacheNeed.merged({n: m.cache_need() for n, m in self.members.items()})

    def bind(self, tensors, rt):
        self.rt = rt
        self._out_w = {}
        for n, m in self.members.items():
            m.bind({k[len(n) + 1:]: v for k, v in tensors.items() if k.startswith(n + ".") and k != f"{n}.out"}, rt)
            self._out_w[n] = tensors[f"{n}.out"]

    def after_load(self) -> None:
        for m in self.members.values():
            m.after_load()

    def launch_plan(self, step) -> None:
        for m in self.members.values():
            m.launch_plan(step)

    def _members_forward(self, x, step, cache, writes_cache, meanwhile=None):
        """Both members' outputs.  In an eager step of many rows the second member runs on a stream of its own
        beside the first (and beside ``meanwhile``, work of the caller that reads the same rows): the two share
        nothing but their input, and a member that cannot fill the device (a recurrence with one CTA per request
        and head) would otherwise hold everything else up.  Captured steps keep to one stream."""
        (na, ma), (nb, mb) = self.members.items()
        T = x.shape[0]
        if not (OVERLAP_MIN_ROWS and T >= OVERLAP_MIN_ROWS) or torch.cuda.is_current_stream_capturing():
            a = ma.forward(x, step, cache.member(na), writes_cache)
            b = mb.forward(x, step, cache.member(nb), writes_cache)
            return (na, a), (nb, b), (meanwhile() if meanwhile is not None else None)
        main = torch.cuda.current_stream()
        if self._side is None:      # one for all layers of a device: layers run one after another
            key = x.device.index
            if key not in _side_streams:
                _side_streams[key] = torch.cuda.Stream(device=x.device, priority=-1)     # its blocks are placed first
            self._side = _side_streams[key]
        fork, join = torch.cuda.Event(), torch.cuda.Event()
        fork.record(main)
        self._side.wait_event(fork)
        with torch.cuda.stream(self._side):
            b = mb.forward(x, step, cache.member(nb), writes_cache)
            join.record(self._side)
        # the caller's work first: by the time the first member's long kernels take the SMs, the second member's
        # chain of short ones has reached its own long kernel
        extra = meanwhile() if meanwhile is not None else None
        a = ma.forward(x, step, cache.member(na), writes_cache)
        main.wait_event(join)
        return (na, a), (nb, b), extra

    def forward(self, x, step, cache, writes_cache, add_to=None):
        if add_to is not None:
            residual, extra = add_to
            (na, a), (nb, b), extra = self._members_forward(x, step, cache, writes_cache,
                                                            extra if callable(extra) else (lambda: extra))
            native.pair_rmsnorm_add(residual, a, self._out_w[na], b, self._out_w[nb], extra, self.norm_eps)
            return None
        (na, a), (nb, b), _ = self._members_forward(x, step, cache, writes_cache)
        T = x.shape[0]
        ws = self.rt.workspace
        acc = ws.get("sbs.acc", (T, self.hidden_size), torch.float32)
        acc.zero_()
        native.pair_rmsnorm_add(acc, a, self._out_w[na], b, self._out_w[nb], None, self.norm_eps)
        out = ws.get("sbs.out", (T, self.hidden_size), self.rt.dtype)
        out.copy_(acc)
        return out
