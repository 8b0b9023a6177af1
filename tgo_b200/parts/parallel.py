"""Mixers that share an input: several mixers read the same rows and the layer's mixer output is the
weighted sum of theirs,

    y = sum_i scale_i * mixer_i(x),

summed in float32. The branches are ordinary registered mixers, each with its own spec
(`MixerSpec.branches`, with `branch_scales`); each gets the layer's tensor-name prefix and
names its tensors through its own `tensors` table. At most one branch may keep a paged cache
and at most one a per-request state: the layer call's cache group and state row are handed to
every branch, and each takes what it asked for.
"""
from __future__ import annotations

from typing import List

import torch

from ..config.spec import MixerSpec
from ..kernels import ops
from ..registry import MIXERS
from .base import LayerCache, Part, offered


class ParallelMixers(Part):
    out_dtype = None

    def __init__(self, spec: MixerSpec, hidden: int, prefix: str, device=None):
        if not spec.branches or len(spec.branches) != len(spec.branch_scales):
            raise ValueError("parallel mixers: the spec needs branches and one scale for each")
        self.hidden = hidden
        self.scales = [float(s) for s in spec.branch_scales]
        self.branches = [MIXERS.get(b.kind)(b, hidden, prefix, device) for b in spec.branches]
        needs = [b.cache_need() for b in self.branches if hasattr(b, "cache_need")]
        states = [b.state_need() for b in self.branches if hasattr(b, "state_need")]
        if sum(n is not None for n in needs) > 1 or sum(s is not None for s in states) > 1:
            raise ValueError("parallel mixers: at most one branch may keep a paged cache and at "
                             "most one a per-request state")
        self._cache_need = next((n for n in needs if n is not None), None)
        self._state_need = next((s for s in states if s is not None), None)
        # the weighted sum is float32: the branches' last products keep float32 rows
        for b in self.branches:
            if hasattr(b, "out_dtype"):
                b.out_dtype = torch.float32

    def parts(self):
        return list(self.branches)

    def weight_specs(self):
        out = []
        for b in self.branches:
            out += b.weight_specs()
        return out

    def bind(self, weights):
        for b in self.branches:
            b.bind(weights)

    def cache_need(self):
        return self._cache_need

    def state_need(self):
        return self._state_need

    def libraries(self, dtype, page_size) -> List[str]:
        out = ["layer_ops"]
        for b in self.branches:
            out += offered(b, "libraries")(dtype, page_size)
        return out

    def prepare_capture(self, ctx, cache) -> None:
        for b in self.branches:
            offered(b, "prepare_capture")(ctx, cache)

    def flops(self, extents, first_positions, writes_cache: bool = True) -> float:
        return sum(offered(b, "flops")(extents, first_positions, writes_cache)
                   for b in self.branches)

    def cache_bytes_read(self, context_len: float, width: int) -> float:
        return sum(offered(b, "cache_bytes_read")(context_len, width) for b in self.branches)

    def forward(self, x, ctx, cache: LayerCache):
        x = ops.rows_of(x)
        outs = [b.forward(x, ctx, cache) for b in self.branches]
        y = torch.empty((x.shape[0], self.hidden), dtype=torch.float32, device=x.device)
        ops.weighted_sum(outs, self.scales, y)
        want = self.out_dtype or ctx.act_dtype
        return y if want == torch.float32 else _narrow(y, want)


def _narrow(y: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    out = torch.empty(y.shape, dtype=dtype, device=y.device)
    ops.cast_rows(y, out)
    return out


MIXERS.register("parallel", ParallelMixers)
