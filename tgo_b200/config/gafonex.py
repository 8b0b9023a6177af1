"""Typed reading of a Gafonex config.json, and its translation to a ModelSpec.

Gafonex is a decoder whose layers are listed one by one in the file: each entry names its
mixer ("attention": softmax attention over a paged cache with per-head q/k norm, a rotation
that may be stretched, normed values, attention weights mixed across heads and values blended
with an earlier layer's; "retention": linear attention with one fixed decay per head, a
32-bit state per request and a gated output), the mixer's sizes and its feed-forward
(a ReLU-gated dense one, or none). A layer adds the grouped RMS norm of each sublayer's
output, scaled per channel, to the stream; the sublayers read the stream itself. The logits
go through a soft cap.

Every size and constant comes from the file; a value the engine cannot honour is refused
with its key in the message.
"""
from __future__ import annotations

import math
from typing import Optional

from .qwen3 import ConfigError, _f32
from .spec import (FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec)

ARCHITECTURE = "Gafonex"


def _int(raw: dict, key: str, where: str, default: Optional[int] = None) -> int:
    v = raw.get(key, default)
    if v is None:
        raise ConfigError(f"config: {where}{key} is required")
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config: {where}{key} is {v!r}; it must be a positive integer")
    return v


def _number(raw: dict, key: str, where: str) -> float:
    v = raw.get(key)
    if v is None:
        raise ConfigError(f"config: {where}{key} is required")
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"config: {where}{key} is {v!r}; it must be a finite number")
    try:
        f = _f32(float(v))
    except OverflowError:
        f = math.inf
    if not math.isfinite(f):
        raise ConfigError(f"config: {where}{key} is {v}, which is not finite as a 32-bit float")
    return float(v)


def _positive(raw: dict, key: str, where: str) -> float:
    v = _number(raw, key, where)
    if not v > 0:
        raise ConfigError(f"config: {where}{key} is {v}; it must be positive")
    return v


def _position(rot, dim: int, where: str) -> Optional[PositionSpec]:
    """`rot` {dims, base, scaling?} -> PositionSpec; without `rot` positions do not enter."""
    if rot is None:
        return None
    if not isinstance(rot, dict):
        raise ConfigError(f"config: {where}rot must be an object")
    dims = _int(rot, "dims", where + "rot.")
    if dims % 2 or dims > dim:
        raise ConfigError(f"config: {where}rot.dims is {dims}; it must be even and at most the "
                          f"head's key size {dim}")
    base = _positive(rot, "base", where + "rot.")
    sc = rot.get("scaling")
    if sc is None:
        return PositionSpec("rope_half_split", rotary_dim=dims, theta=base)
    if not isinstance(sc, dict):
        raise ConfigError(f"config: {where}rot.scaling must be an object or null")
    w = where + "rot.scaling."
    scaling = (_positive(sc, "factor", w), _positive(sc, "original", w), _positive(sc, "fast", w),
               _positive(sc, "slow", w))
    if base == 1.0:
        raise ConfigError(f"config: {where}rot.base is 1; the stretched rotation divides by its "
                          "logarithm")
    return PositionSpec("rope_stretched", rotary_dim=dims, theta=base, scaling=scaling)


ATTENTION_TENSORS = (("q", "mix.q"), ("k", "mix.k"), ("v", "mix.v"), ("o", "mix.o"),
                     ("q_norm", "mix.q.norm"), ("k_norm", "mix.k.norm"),
                     ("head_mix", "mix.talk"), ("value_share", "mix.vmix"))
RETENTION_TENSORS = (("q", "mix.q"), ("k", "mix.k"), ("v", "mix.v"), ("gate", "mix.g"),
                     ("o", "mix.o"))
FEED_FORWARD_TENSORS = (("gate", "mlp.gate"), ("up", "mlp.up"), ("down", "mlp.down"))
BLOCK_TENSORS = (("mixer_norm", "norm1"), ("ffn_norm", "norm2"),
                 ("mixer_scale", "ls1"), ("ffn_scale", "ls2"))


def _attention(m: dict, where: str, eps: float, share: Optional[str]) -> MixerSpec:
    H = _int(m, "heads", where)
    G = _int(m, "kv_heads", where, default=H)
    if H % G:
        raise ConfigError(f"config: {where}heads ({H}) is not a multiple of kv_heads ({G})")
    dim = _int(m, "dim", where)
    vdim = _int(m, "vdim", where, default=dim)
    scale = _positive(m, "scale", where) if m.get("scale") is not None else None   # None: dim^-1/2
    return MixerSpec("mixed_head_attention", num_heads=H, num_kv_heads=G, head_dim=dim,
                     qk_norm=True, window=None, scale=scale,
                     position=_position(m.get("rot"), dim, where), norm_eps=eps,
                     tensors=ATTENTION_TENSORS, value_dim=vdim, value_norm=True, head_mix=True,
                     value_share=share)


def _retention(m: dict, where: str, eps: float) -> MixerSpec:
    H = _int(m, "heads", where)
    dim = _int(m, "dim", where)
    vdim = _int(m, "vdim", where, default=dim)
    decay = m.get("decay")
    if not isinstance(decay, list) or len(decay) != H:
        raise ConfigError(f"config: {where}decay must list one decay per head ({H})")
    for j in range(H):
        d = _number({"decay": decay[j]}, "decay", where)
        if not 0.0 <= d <= 1.0:
            raise ConfigError(f"config: {where}decay[{j}] is {d}; a decay lies in [0, 1]")
    return MixerSpec("retention", num_heads=H, num_kv_heads=H, head_dim=dim,
                     position=_position(m.get("rot"), dim, where), norm_eps=eps,
                     tensors=RETENTION_TENSORS, value_dim=vdim,
                     decay=tuple(float(d) for d in decay), output_gate=True)


def gafonex_model_spec(raw: dict) -> ModelSpec:
    """config.json (as a dict) -> ModelSpec. Tensor names: `embed`, `l<i>.norm1|norm2|ls1|ls2`,
    `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`."""
    if not isinstance(raw, dict):
        raise ConfigError("config: the top level must be an object")
    d = _int(raw, "width", "")
    V = _int(raw, "vocab", "")
    norm = raw.get("norm")
    if not isinstance(norm, dict):
        raise ConfigError("config: norm is required (eps, groups)")
    eps = _positive(norm, "eps", "norm.")
    groups = _int(norm, "groups", "norm.", default=1)
    if d % groups:
        raise ConfigError(f"config: norm.groups is {groups}; it must divide width ({d})")
    nspec = NormSpec("group_rmsnorm", eps, groups)
    cap = raw.get("logit_softcap")
    if cap is not None:
        cap = _positive(raw, "logit_softcap", "")
    entries = raw.get("layers")
    if not isinstance(entries, list) or not entries:
        raise ConfigError("config: layers must list at least one layer")
    layers, shared = [], False
    for i, e in enumerate(entries):
        where = f"layers[{i}]."
        if not isinstance(e, dict) or not isinstance(e.get("mixer"), dict):
            raise ConfigError(f"config: {where}mixer is required")
        kind, m = e.get("type"), e["mixer"]
        if kind == "attention":
            share = None
            if m.get("v_mix"):
                share = "blend" if shared else "source"
                shared = True
            mixer = _attention(m, where + "mixer.", eps, share)
        elif kind == "retention":
            mixer = _retention(m, where + "mixer.", eps)
        else:
            raise ConfigError(f"config: {where}type is {kind!r}; known mixers are attention, "
                              "retention")
        mlp = e.get("mlp")
        ffn = None
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"config: {where}mlp.kind is "
                                  f"{mlp.get('kind') if isinstance(mlp, dict) else mlp!r}; "
                                  "known kinds: dense")
            ffn = FeedForwardSpec("gated_dense", intermediate_size=_int(mlp, "ff", where + "mlp."),
                                  tensors=FEED_FORWARD_TENSORS, activation="relu")
        layers.append(LayerSpec("postnorm_scaled_residual", f"l{i}.", mixer, ffn, nspec,
                                BLOCK_TENSORS))
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=d, vocab_size=V, layers=layers,
        run_order=[LayerCall(i) for i in range(len(layers))], final_norm=nspec,
        embedding_name="embed", final_norm_name="final.norm", head_name="head",
        logit_softcap=cap, source=dict(raw))
    spec.validate()
    return spec
