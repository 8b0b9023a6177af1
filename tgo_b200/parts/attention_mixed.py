"""Grouped-query causal softmax attention over the paged cache with four things beside the
plain one (`parts/attention.py`), each switched by its spec:

  - keys `head_dim` wide and values `value_dim` wide (two cache planes with rows of their own);
  - `value_norm`: each head's value divided by its root mean square before it is stored;
  - `value_share`: the first layer that has it ("source") leaves its normed values of the
    step's tokens for the later ones ("blend"), which store (1 - b) v + b v_source with their
    own learned scalar b; what is cached is the blended value;
  - `head_mix`: the softmax weights of the H heads are mixed by a learned [H, H] matrix,
    w_h = sum_g M[h, g] p_g, and head h applies w_h to the values of its own kv head.

q and k are normed per head (plain gain) before the rotation; no bias anywhere. Tensor roles:
q, k, v, o, q_norm, k_norm, head_mix, value_share.
"""
from __future__ import annotations

import math
from typing import List

import torch

from ..config.spec import MixerSpec, tensor_names
from ..kernels import ops
from ..registry import MIXERS, POSITIONS
from ..weights.binder import WeightSpec
from .attention import step_tiles
from .base import CacheNeed, LayerCache, Part

SHARED_VALUES = "shared_values"      # ctx.aux: the source layer's values of this step's tokens


class MixedHeadAttention(Part):
    out_dtype = None                 # dtype of the output product's rows (None: activations')

    def __init__(self, spec: MixerSpec, hidden: int, prefix: str, device=None):
        self.hidden = hidden
        self.H, self.Hkv, self.dk = spec.num_heads, spec.num_kv_heads, spec.head_dim
        self.dv = spec.value_dim or spec.head_dim
        if self.H <= 0 or self.Hkv <= 0 or self.H % self.Hkv:
            raise ValueError(f"attention: {self.H} query heads do not group over {self.Hkv}")
        self.qk_norm = spec.qk_norm
        self.value_norm = spec.value_norm
        self.head_mix = spec.head_mix
        self.share = spec.value_share
        if self.share not in (None, "source", "blend"):
            raise ValueError(f"attention: value_share is {self.share!r}; source, blend or None")
        self.eps = float(spec.norm_eps)
        self.window = spec.window
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(self.dk)
        pos = spec.position
        self.position = POSITIONS.get(pos.kind)(pos, self.dk, device) if pos is not None else None
        if self.position is not None and not getattr(self.position, "fusable", False):
            raise ValueError("attention: this mixer rotates inside its own kernel and needs a "
                             "position encoding that offers rotary()")
        roles = ["q", "k", "v", "o"] + (["q_norm", "k_norm"] if self.qk_norm else []) + \
            (["head_mix"] if self.head_mix else []) + (["value_share"] if self.share else [])
        self.names = tensor_names(spec.tensors, prefix, roles, "attention")
        # a layer outside the sharing has no use for a blend factor; a checkpoint that ships
        # one for it anyway is not refused for that
        self.unused_blend = None if self.share else dict(spec.tensors).get("value_share")
        if self.unused_blend is not None:
            self.unused_blend = prefix + self.unused_blend
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = self.mix = self.blend = None

    def weight_specs(self):
        n, d = self.names, self.hidden
        out = [WeightSpec(n["q"], (self.H * self.dk, d)), WeightSpec(n["k"], (self.Hkv * self.dk, d)),
               WeightSpec(n["v"], (self.Hkv * self.dv, d)), WeightSpec(n["o"], (d, self.H * self.dv))]
        if self.qk_norm:
            out += [WeightSpec(n["q_norm"], (self.dk,), "gain"),
                    WeightSpec(n["k_norm"], (self.dk,), "gain")]
        if self.head_mix:
            out.append(WeightSpec(n["head_mix"], (self.H, self.H), "constant"))
        if self.share:
            out.append(WeightSpec(n["value_share"], (), "constant"))
        elif self.unused_blend is not None:
            out.append(WeightSpec(self.unused_blend, (), "constant", optional=True))
        return out

    def cache_need(self):
        return CacheNeed.keys_and_values_of(self.window, self.Hkv, self.dk, self.dv)

    def state_need(self):
        return None

    def bind(self, weights):
        n = self.names
        self.w_qkv = torch.cat([weights.pop(n["q"]), weights.pop(n["k"]), weights.pop(n["v"])],
                               dim=0).contiguous()
        self.w_o = weights.pop(n["o"]).contiguous()
        if self.qk_norm:
            self.q_gain = weights.pop(n["q_norm"]).contiguous()
            self.k_gain = weights.pop(n["k_norm"]).contiguous()
        if self.head_mix:
            self.mix = weights.pop(n["head_mix"]).contiguous()
        if self.share:
            self.blend = weights.pop(n["value_share"]).reshape(1).contiguous()

    def libraries(self, dtype, page_size) -> List[str]:
        return ["sgemm" if dtype == torch.float32 else "gemm_skinny", "elementwise", "layer_ops",
                "attention_mixed"]

    def prepare_capture(self, ctx, cache) -> None:
        """The tile list of a step with prompt portions is made on the host: before a capture."""
        if not ctx.decode_only and cache is not None and \
                tile_kernel_takes(ctx.act_dtype, self.H, self.Hkv, self.dk, self.dv, self.window or 0):
            step_tiles(ctx, TILE_TOKENS)

    def flops(self, extents, first_positions, writes_cache: bool = True) -> float:
        n = sum(extents)
        qw, kw, vw = self.H * self.dk, self.Hkv * self.dk, self.H * self.dv
        total = 2.0 * n * self.hidden * (qw + kw + self.Hkv * self.dv) + 2.0 * n * vw * self.hidden
        keys = 0
        for first, extent in zip(first_positions, extents):
            if self.window:
                keys += sum(min(first + t + 1, self.window) for t in range(extent))
            else:
                keys += extent * first + extent * (extent + 1) // 2
        mix = 2.0 * self.H * self.H if self.head_mix else 0.0
        return total + (2.0 * qw + 2.0 * vw + mix) * keys

    def cache_bytes_read(self, context_len: float, width: int) -> float:
        reach = min(context_len, self.window) if self.window else context_len
        return self.Hkv * (self.dk + self.dv) * width * reach

    def forward(self, x, ctx, cache: LayerCache):
        H, Hkv, dk, dv = self.H, self.Hkv, self.dk, self.dv
        qw, kw = H * dk, Hkv * dk
        x = ops.rows_of(x)
        qkv = ops.linear(x, self.w_qkv)
        q, k, v = qkv[:, :qw], qkv[:, qw:qw + kw], qkv[:, qw + kw:]
        rope, rot = self.position.rotary(ctx) if self.position is not None else (None, 0)
        # q in place; k normed, rotated and stored in the key plane
        ops.qk_norm_rope_cache(q, k, None, H, Hkv, dk, self.q_gain, self.k_gain, self.eps, rope,
                               rot, cache.slots, cache.k, None, cache.page_size)
        shared, mode = None, 0
        if self.share == "source":
            shared = torch.empty((x.shape[0], Hkv * dv), dtype=torch.float32, device=x.device)
            ctx.aux[SHARED_VALUES] = shared
            mode = 1
        elif self.share == "blend":
            shared = ctx.aux.get(SHARED_VALUES)
            if shared is None or shared.shape != (x.shape[0], Hkv * dv):
                raise RuntimeError("attention: a layer blends its values with an earlier "
                                   "layer's, and none of the same shape ran before it")
            mode = 2
        ops.value_norm_share_cache(v, Hkv, dv, self.value_norm, self.eps, self.blend, shared, mode,
                                   cache.slots, cache.v, cache.page_size)
        a = torch.empty((x.shape[0], H * dv), dtype=q.dtype, device=q.device)
        mixed_attention(q, a, H, Hkv, dk, dv, cache, ctx, self.mix, self.scale, self.window or 0)
        return ops.linear(a, self.w_o, out_dtype=self.out_dtype)


USE_DECODE_KERNELS = True


def decode_ranges(tokens: int, max_context: int, num_sms: int) -> int:
    """Into how many key ranges a decode step cuts each token's keys: enough blocks (token x
    range) for four a multiprocessor, no range shorter than 64 keys, at most 32."""
    want = max(1, (4 * num_sms) // max(1, tokens))
    return max(1, min(want, max(1, max_context // 64), 32))


TILE_TOKENS = 16                     # tokens of one request a block of the tile kernel takes
USE_TILE_KERNEL = True


def tile_kernel_takes(dtype, H, Hkv, dk, dv, window) -> bool:
    return USE_TILE_KERNEL and dtype == torch.bfloat16 and \
        ops.attention_mixed_tile_supports(H, Hkv, dk, dv, window)


def mixed_attention(q, out, H, Hkv, dk, dv, cache, ctx, mix, scale, window) -> None:
    """Which kernel runs the attention of a step: bfloat16 steps with prompt portions take the
    tensor-core tile kernel (single tokens beside them are tiles of one); float32, and sizes
    the tile kernel has no instance for, the generic kernel (a block a token, keys in a fixed
    order)."""
    if ctx.decode_only and USE_DECODE_KERNELS and q.dtype == torch.bfloat16 and \
            ops.attention_mixed_decode_supports(H, Hkv, dk, dv, window):
        ops.attention_mixed_decode(q, out, H, Hkv, dk, dv, cache.k, cache.v, cache.page_size,
                                   cache.block_tables, ctx.seq_ids, ctx.positions, mix, scale,
                                   decode_ranges(ctx.num_seqs, ctx.max_context, ops.num_sms(q.device)),
                                   ctx.max_context)
        return
    if not ctx.decode_only and tile_kernel_takes(q.dtype, H, Hkv, dk, dv, window):
        tok0, ntok = step_tiles(ctx, TILE_TOKENS)
        ops.attention_mixed_tile(q, out, H, Hkv, dk, dv, cache.k, cache.v, cache.page_size,
                                 cache.block_tables, ctx.seq_ids, ctx.positions, mix, scale,
                                 tok0, ntok)
        return
    ops.attention_mixed(q, out, H, Hkv, dk, dv, cache.k, cache.v, cache.page_size,
                        cache.block_tables, ctx.seq_ids, ctx.positions, mix, scale, window)


MIXERS.register("mixed_head_attention", MixedHeadAttention)
