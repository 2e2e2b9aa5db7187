"""A mixer that is the weighted sum of several mixers reading the same input:
``out = sum_i scale_i * mixer_i(h)``.  Every member keeps the cache it asks for (the run's cache
then carries the members' needs one after the other) and writes its output to a float32 buffer of
its own; the sum is taken in float32.
"""
from __future__ import annotations

from typing import Mapping, Sequence

import torch

from ..cache.cache import KVView, RunCache, needs_of
from ..kernels import ops
from .base import MIXERS, Mixer, PartSpec


@MIXERS.register("weighted_sum")
class WeightedSumMixer(Mixer):
    def __init__(self, members: Mapping[str, PartSpec], scales: Mapping[str, float]):
        if len(members) != 2:
            raise ValueError("a weighted sum of mixers takes two members")
        if set(members) != set(scales):
            raise ValueError("a weighted sum of mixers wants one scale per member")
        self.names = tuple(members)
        self.members = {n: MIXERS.build(members[n]) for n in self.names}
        self.scales = {n: float(scales[n]) for n in self.names}

    @property
    def graph_safe(self):       # as safe as its members (the block asks all_graph_safe, which asks them too)
        return True

    def children(self):
        return dict(self.members)

    def cache_need(self):
        out = ()
        for n in self.names:
            out += needs_of(self.members[n].cache_need())
        return out

    def prepare(self, runtime, max_positions: int) -> None:
        for m in self.members.values():
            m.prepare(runtime, max_positions)

    def _member_runs(self, run) -> Sequence[RunCache]:
        """The run's cache cut into the members' shares, in the order the needs were declared."""
        out, at = [], 0
        for n in self.names:
            k = len(needs_of(self.members[n].cache_need()))
            entries = tuple(run.entries[at:at + k])
            at += k
            kv = next((e for e in entries if isinstance(e, KVView)), None)
            state = next((e for e in entries if not isinstance(e, KVView)), None)
            out.append(RunCache(kv=kv, state=state, writes_cache=run.writes_cache, entries=entries))
        return out

    def forward_store(self, ctx, h, out, run) -> None:
        runs = self._member_runs(run)
        parts = []
        for i, n in enumerate(self.names):
            y = ctx.rows(f"sum.member{i}", out.shape[1], torch.float32)
            self.members[n].forward_store(ctx, h, y, runs[i])
            parts.append(y)
        a, b = (self.scales[n] for n in self.names)
        ops.weighted_sum(out, parts[0], a, parts[1], b)

    def forward(self, ctx, h, residual, run) -> None:
        y = ctx.rows("sum.out", residual.shape[1], torch.float32)
        self.forward_store(ctx, h, y, run)
        ops.residual_add(residual, y)
