"""A selective state-space mixer (the form known as Mamba-2): H heads of P channels, a state
of N per head and channel, B and C shared by the heads of each of G groups.

    [z | x B C | dt] = W_in h                       inner = H P; widths inner, inner + 2 G N, H
    x B C  <- silu(causal convolution per channel, `conv_taps` taps with a bias)
    dt     <- softplus(dt + dt_bias)                                          (unbounded)
    S_t    = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T                 S is [N, P]
    y_t    = S_t^T C_t + D_h x_t
    out    = W_o ( gain * group_rmsnorm(y * silu(z), `norm_groups` parts) )

The projections and the convolution's input are in the activation type; the convolution's sum,
dt, the decays, the scan, its state and the norm are float32. Per request the mixer keeps, as
one float32 state row, S [H, N, P] and the convolution's last taps - 1 inputs [taps - 1, C].

Spec fields: num_heads = H, value_dim = P, head_dim = N, num_kv_heads = G, conv_taps,
norm_groups, norm_eps. Tensor roles: in, conv, conv_bias, dt_bias, a_log, d, norm, o.
"""
from __future__ import annotations

from typing import List

import torch

from ..config.spec import MixerSpec, tensor_names
from ..kernels import ops
from ..registry import MIXERS
from ..weights.binder import WeightSpec
from .base import LayerCache, Part, StateNeed


class SelectiveStateSpace(Part):
    out_dtype = None                 # dtype of the output product's rows (None: activations')

    def __init__(self, spec: MixerSpec, hidden: int, prefix: str, device=None):
        self.hidden = hidden
        self.H, self.P, self.N, self.G = spec.num_heads, spec.value_dim, spec.head_dim, spec.num_kv_heads
        self.taps, self.norm_groups = int(spec.conv_taps), int(spec.norm_groups or 1)
        if min(self.H, self.P or 0, self.N, self.G, self.taps) <= 0 or self.H % self.G:
            raise ValueError(f"state-space mixer: heads {self.H}, channels {self.P}, state {self.N}, "
                             f"groups {self.G}, taps {self.taps}")
        self.inner = self.H * self.P
        if self.inner % self.norm_groups:
            raise ValueError(f"state-space mixer: {self.norm_groups} norm parts do not divide "
                             f"{self.inner} channels")
        self.C = self.inner + 2 * self.G * self.N            # channels through the convolution
        self.eps = float(spec.norm_eps)
        self.ssm_floats = self.H * self.N * self.P
        self.names = tensor_names(spec.tensors, prefix,
                                  ["in", "conv", "conv_bias", "dt_bias", "a_log", "d", "norm", "o"],
                                  "state-space mixer")
        self.w_in = self.w_o = self.conv = self.conv_bias = None
        self.dt_bias = self.a_log = self.d_skip = self.gain = None

    def weight_specs(self):
        n, d = self.names, self.hidden
        return [WeightSpec(n["in"], (2 * self.inner + 2 * self.G * self.N + self.H, d)),
                WeightSpec(n["conv"], (self.C, self.taps), "constant"),
                WeightSpec(n["conv_bias"], (self.C,), "gain"),
                WeightSpec(n["dt_bias"], (self.H,), "gain"), WeightSpec(n["a_log"], (self.H,), "gain"),
                WeightSpec(n["d"], (self.H,), "gain"), WeightSpec(n["norm"], (self.inner,), "gain"),
                WeightSpec(n["o"], (d, self.inner))]

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed((self.ssm_floats + (self.taps - 1) * self.C,))

    def bind(self, weights):
        n = self.names
        self.w_in = weights.pop(n["in"]).contiguous()
        self.w_o = weights.pop(n["o"]).contiguous()
        f32 = lambda r: weights.pop(n[r]).to(torch.float32).contiguous()     # noqa: E731
        self.conv, self.conv_bias = f32("conv"), f32("conv_bias")
        self.dt_bias, self.a_log, self.d_skip, self.gain = f32("dt_bias"), f32("a_log"), f32("d"), f32("norm")

    def libraries(self, dtype, page_size) -> List[str]:
        return ["sgemm" if dtype == torch.float32 else "gemm_skinny", "layer_ops", "state_space"]

    def flops(self, extents, first_positions, writes_cache: bool = True) -> float:
        n = sum(extents)
        products = 2.0 * n * self.hidden * (2 * self.inner + 2 * self.G * self.N + self.H) + \
            2.0 * n * self.inner * self.hidden
        return products + 2.0 * n * self.C * self.taps + 6.0 * n * self.H * self.N * self.P

    def cache_bytes_read(self, context_len: float, width: int) -> float:
        return 4.0 * (self.ssm_floats + (self.taps - 1) * self.C)      # the state, whatever the length

    def forward(self, x, ctx, cache: LayerCache):
        x = ops.rows_of(x)
        T, inner = x.shape[0], self.inner
        zall = ops.linear(x, self.w_in)
        z, xbc_in, dt_raw = zall[:, :inner], zall[:, inner:inner + self.C], zall[:, inner + self.C:]
        state = cache.state
        xbc = torch.empty((T, self.C), dtype=torch.float32, device=x.device)
        ops.causal_conv_act(xbc_in, self.conv, self.conv_bias, xbc, ctx.num_seqs, ctx.seq_ids,
                            ctx.q_start, ctx.state_slots, state, self.ssm_floats)
        y = torch.empty((T, inner), dtype=torch.float32, device=x.device)
        ops.selective_scan(xbc, dt_raw, self.dt_bias, self.a_log, self.d_skip, y, ctx.num_seqs,
                           self.H, self.G, self.N, self.P, ctx.q_start, ctx.state_slots, state, 0)
        g = torch.empty((T, inner), dtype=x.dtype, device=x.device)
        ops.gated_group_norm(y, z, self.gain, g, self.norm_groups, self.eps, "silu", True)
        return ops.linear(g, self.w_o, out_dtype=self.out_dtype)


MIXERS.register("selective_state_space", SelectiveStateSpace)
