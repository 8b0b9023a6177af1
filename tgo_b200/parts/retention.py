"""Retention: linear attention with one fixed decay per head, no softmax and no denominator,
as a mixer with a fixed-size float32 state per request instead of a cache that grows.

    q = Wq x, k = Wk x (heads x dk), v = Wv x (heads x dv); q and k rotated, k * dk^-1/2
    S_t = decay_h S_(t-1) + k_t v_t^T            (per head; S is [dk, dv], starts at zero)
    o_t = S_t^T q_t
    y   = Wo ( o_t / rms(o_t per head) * silu(Wg x) )

The projections may run in the activation type; the rotation, the scaling of k, the
recurrence and the per-head norm are float32. Tensor roles: q, k, v, o and, with
`output_gate`, gate. The decays are constants of the spec.

What a spec may change (the form known as lightning attention changes all four):
`input_activation` "silu" puts q, k and v through SiLU as the recurrence reads them; `scale`
replaces the dk^-1/2 on k (1 for none); `output_norm` "joint_gain" norms the heads' outputs as
one row and multiplies by a gain (tensor role out_norm) instead of norming each head alone;
`gate_activation` "sigmoid" gates with the logistic function instead of SiLU.
"""
from __future__ import annotations

from typing import List

import torch

from ..config.spec import MixerSpec, tensor_names
from ..kernels import ops
from ..registry import MIXERS, POSITIONS
from ..weights.binder import WeightSpec
from .attention import step_tiles
from .base import LayerCache, Part, StateNeed


USE_CHUNKED = True


def step_chunks(ctx, tokens_per_chunk: int):
    """Chunk lists of a step: first token row and token count of each chunk (a chunk holds
    tokens of one request), and each request's first chunk; made once per step on the host
    and kept in ctx.aux (under keys that a graph capture keeps)."""
    tok0, ntok = step_tiles(ctx, tokens_per_chunk)
    key = ("tiles", tokens_per_chunk, "first")
    first = ctx.aux.get(key)
    if first is None:
        at, firsts = 0, []
        for n in ctx.extents:
            firsts.append(at)
            at += -(-n // tokens_per_chunk)
        first = torch.tensor(firsts, dtype=torch.int32).to(ctx.token_ids.device, non_blocking=True)
        ctx.aux[key] = first
    return tok0, ntok, first


class Retention(Part):
    out_dtype = None                 # dtype of the output product's rows (None: activations')

    def __init__(self, spec: MixerSpec, hidden: int, prefix: str, device=None):
        self.hidden = hidden
        self.H, self.dk = spec.num_heads, spec.head_dim
        self.dv = spec.value_dim or spec.head_dim
        if len(spec.decay) != self.H:
            raise ValueError(f"retention: {len(spec.decay)} decays for {self.H} heads")
        self.gated = bool(spec.output_gate)
        self.eps = float(spec.norm_eps)
        self.k_scale = float(self.dk) ** -0.5 if spec.scale is None else float(spec.scale)
        self.act = {None: 0, "silu": 1}.get(spec.input_activation, -1)
        if self.act < 0:
            raise ValueError(f"retention: input_activation {spec.input_activation!r}; silu or None")
        self.output_norm = spec.output_norm or "head_unit"
        if self.output_norm not in ("head_unit", "joint_gain"):
            raise ValueError(f"retention: output_norm {self.output_norm!r}; head_unit or joint_gain")
        self.gate_activation = spec.gate_activation or "silu"
        if self.gate_activation not in ("silu", "sigmoid"):
            raise ValueError(f"retention: gate_activation {self.gate_activation!r}; silu or sigmoid")
        pos = spec.position
        self.position = POSITIONS.get(pos.kind)(pos, self.dk, device) if pos is not None else None
        if self.position is not None and not getattr(self.position, "fusable", False):
            raise ValueError("retention: the rotation is done inside the kernel and needs a "
                             "position encoding that offers rotary()")
        self.decay = torch.tensor([float(d) for d in spec.decay], dtype=torch.float32,
                                  device=device)
        roles = ["q", "k", "v", "o"] + (["gate"] if self.gated else []) + \
            (["out_norm"] if self.output_norm == "joint_gain" else [])
        self.names = tensor_names(spec.tensors, prefix, roles, "retention")
        self.w_in = self.w_o = self.out_gain = None

    def weight_specs(self):
        n, d = self.names, self.hidden
        out = [WeightSpec(n["q"], (self.H * self.dk, d)), WeightSpec(n["k"], (self.H * self.dk, d)),
               WeightSpec(n["v"], (self.H * self.dv, d))]
        if self.gated:
            out.append(WeightSpec(n["gate"], (self.H * self.dv, d)))
        if self.output_norm == "joint_gain":
            out.append(WeightSpec(n["out_norm"], (self.H * self.dv,), "gain"))
        return out + [WeightSpec(n["o"], (d, self.H * self.dv))]

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed((self.H, self.dk, self.dv))

    def bind(self, weights):
        n = self.names
        mats = [weights.pop(n["q"]), weights.pop(n["k"]), weights.pop(n["v"])]
        if self.gated:
            mats.append(weights.pop(n["gate"]))
        self.w_in = torch.cat(mats, dim=0).contiguous()      # one product makes q, k, v, gate
        self.w_o = weights.pop(n["o"]).contiguous()
        if self.output_norm == "joint_gain":
            self.out_gain = weights.pop(n["out_norm"]).to(torch.float32).contiguous()
        self.decay = self.decay.to(self.w_o.device)

    def libraries(self, dtype, page_size) -> List[str]:
        return ["sgemm" if dtype == torch.float32 else "gemm_skinny", "elementwise", "layer_ops",
                "retention"]

    def prepare_capture(self, ctx, cache) -> None:
        if not ctx.decode_only and USE_CHUNKED and \
                ops.retention_chunked_supports(self.H, self.dk, self.dv):
            step_chunks(ctx, ops.retention_chunk_tokens())

    def flops(self, extents, first_positions, writes_cache: bool = True) -> float:
        n = sum(extents)
        qk, vw = self.H * self.dk, self.H * self.dv
        products = 2.0 * n * self.hidden * (2 * qk + vw * (2 if self.gated else 1)) + \
            2.0 * n * vw * self.hidden
        return products + 4.0 * n * self.H * self.dk * self.dv     # the state's update and read

    def cache_bytes_read(self, context_len: float, width: int) -> float:
        return 4.0 * self.H * self.dk * self.dv                     # the state, whatever the length

    def forward(self, x, ctx, cache: LayerCache):
        H, dk, dv = self.H, self.dk, self.dv
        qk, vw = H * dk, H * dv
        x = ops.rows_of(x)
        z = ops.linear(x, self.w_in)
        q, k, v = z[:, :qk], z[:, qk:2 * qk], z[:, 2 * qk:2 * qk + vw]
        gate = z[:, 2 * qk + vw:] if self.gated else None
        rope, rot = self.position.rotary(ctx) if self.position is not None else (None, 0)
        o = torch.empty((x.shape[0], vw), dtype=torch.float32, device=x.device)
        args = (q, k, v, o, ctx.num_seqs, H, dk, dv, self.decay, self.k_scale, rope, rot,
                ctx.q_start, ctx.state_slots, cache.state)
        if not USE_CHUNKED or not ops.retention_chunked_supports(H, dk, dv):
            ops.retention(*args, act=self.act)   # a block per (request, head, columns), in order
        elif ctx.decode_only:
            ops.retention_chunked(*args, act=self.act)   # single tokens: the state streamed through once
        else:
            ops.retention_chunked(*args, *step_chunks(ctx, ops.retention_chunk_tokens()),
                                  act=self.act)
        y = torch.empty((x.shape[0], vw), dtype=x.dtype, device=x.device)
        if self.output_norm == "head_unit" and self.gate_activation == "silu":
            ops.head_norm_gate(o, gate, y, H, dv, self.eps)
        else:
            ops.gated_group_norm(o, gate, self.out_gain, y,
                                 1 if self.output_norm == "joint_gain" else H, self.eps,
                                 self.gate_activation, False)
        return ops.linear(y, self.w_o, out_dtype=self.out_dtype)


MIXERS.register("retention", Retention)
