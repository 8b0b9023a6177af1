"""Typed reading of a Totatar config.json, and its translation to a ModelSpec.

Totatar is a decoder whose layers are listed one by one in the file. A layer norms the input
AND the output of each sublayer (zero-centred norm weights: the gain is 1 + w):

    x <- x + norm1b(mixer(norm1(x)));  x <- x + norm2b(feed_forward(norm2(x)))

Its mixers: "mamba2", a selective state-space mixer (a short causal convolution, a scan with a
32-bit state per request, a gated group norm); "parallel", two mixers on one input whose
results are added with a factor each: softmax attention with biased projections, a rotation
of neighbouring channel pairs that may be slowed by a factor, a sliding window and a learned
sink per head, and linear attention with a fixed decay per head (q, k, v through SiLU, one
norm over all heads, a logistic gate). Its feed-forwards: dense (the gate through the tanh
form of GELU), a mixture of experts (SiLU) with a router bias and a shared expert, or none.
The head is the embedding table.

Every size and constant comes from the file; a value the engine cannot honour is refused
with its key in the message.
"""
from __future__ import annotations

from typing import Optional

from .gafonex import _int, _number, _positive
from .qwen3 import ConfigError
from .spec import (FeedForwardSpec, LayerCall, LayerSpec, MixerSpec, ModelSpec, NormSpec,
                   PositionSpec)

ARCHITECTURE = "Totatar"

SOFTMAX_TENSORS = (("q", "mix.left.q"), ("k", "mix.left.k"), ("v", "mix.left.v"),
                   ("o", "mix.left.o"), ("q_bias", "mix.left.q.b"), ("k_bias", "mix.left.k.b"),
                   ("v_bias", "mix.left.v.b"), ("sink", "mix.left.sink"))
LINEAR_TENSORS = (("q", "mix.right.q"), ("k", "mix.right.k"), ("v", "mix.right.v"),
                  ("gate", "mix.right.g"), ("o", "mix.right.o"), ("out_norm", "mix.right.norm"))
STATE_SPACE_TENSORS = (("in", "mix.in"), ("conv", "mix.conv"), ("conv_bias", "mix.conv.b"),
                       ("dt_bias", "mix.dt_bias"), ("a_log", "mix.A_log"), ("d", "mix.D"),
                       ("norm", "mix.norm"), ("o", "mix.o"))
DENSE_TENSORS = (("gate", "mlp.gate"), ("up", "mlp.up"), ("down", "mlp.down"))
SHARED_TENSORS = (("gate", "mlp.shared.gate"), ("up", "mlp.shared.up"), ("down", "mlp.shared.down"))
ROUTED_TENSORS = (("expert_gate", "mlp.e{e}.gate"), ("expert_up", "mlp.e{e}.up"),
                  ("expert_down", "mlp.e{e}.down"), ("router", "mlp.router"),
                  ("router_bias", "mlp.router.b"))
BLOCK_TENSORS = (("mixer_norm", "norm1"), ("mixer_out_norm", "norm1b"), ("ffn_norm", "norm2"),
                 ("ffn_out_norm", "norm2b"))


def _object(raw, key: str, where: str, required: bool = True) -> Optional[dict]:
    v = raw.get(key)
    if v is None and not required:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config: {where}{key} must be an object")
    return v


def _rotation(rot, dim: int, where: str) -> Optional[PositionSpec]:
    """`rot` {dims, base, scaling: {factor}?} -> the neighbouring-pair rotation; without `rot`
    positions do not enter."""
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
    scaling = None
    if sc is not None:
        if not isinstance(sc, dict):
            raise ConfigError(f"config: {where}rot.scaling must be an object or null")
        unknown = sorted(set(sc) - {"factor"})
        if unknown:
            raise ConfigError(f"config: {where}rot.scaling.{unknown[0]} is not known; this "
                              "rotation is slowed by rot.scaling.factor alone")
        scaling = (_positive(sc, "factor", where + "rot.scaling."),)
    return PositionSpec("rope_interleaved", rotary_dim=dims, theta=base, scaling=scaling)


def _softmax_branch(m: dict, where: str) -> MixerSpec:
    H = _int(m, "heads", where)
    G = _int(m, "kv_heads", where, default=H)
    if H % G:
        raise ConfigError(f"config: {where}heads ({H}) is not a multiple of kv_heads ({G})")
    dim = _int(m, "dim", where)
    vdim = _int(m, "vdim", where, default=dim)
    scale = _positive(m, "scale", where) if m.get("scale") is not None else None
    mask = _object(m, "mask", where, required=False)
    window = _int(mask, "size", where + "mask.") if mask is not None else None
    return MixerSpec("sink_attention", num_heads=H, num_kv_heads=G, head_dim=dim, window=window,
                     scale=scale, position=_rotation(m.get("rot"), dim, where),
                     tensors=SOFTMAX_TENSORS, value_dim=vdim, bias=True, sink=True)


def _linear_branch(m: dict, where: str, eps: float) -> MixerSpec:
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
    return MixerSpec("retention", num_heads=H, num_kv_heads=H, head_dim=dim, scale=1.0,
                     norm_eps=eps, tensors=LINEAR_TENSORS, value_dim=vdim,
                     decay=tuple(float(d) for d in decay), output_gate=True,
                     gate_activation="sigmoid", input_activation="silu", output_norm="joint_gain")


def _parallel(m: dict, where: str, eps: float) -> MixerSpec:
    left = _softmax_branch(_object(m, "left", where), where + "left.")
    right = _linear_branch(_object(m, "right", where), where + "right.", eps)
    scales = tuple(_number(m, key, where) if m.get(key) is not None else 1.0
                   for key in ("left_scale", "right_scale"))
    return MixerSpec("parallel", branches=(left, right), branch_scales=scales)


def _state_space(m: dict, where: str, eps: float) -> MixerSpec:
    H = _int(m, "heads", where)
    G = _int(m, "groups", where, default=1)
    if H % G:
        raise ConfigError(f"config: {where}heads ({H}) is not a multiple of groups ({G})")
    P, N = _int(m, "vdim", where), _int(m, "state", where)
    if N > 256:
        raise ConfigError(f"config: {where}state is {N}; the scan keeps at most 256 per channel")
    parts = _int(m, "norm_groups", where, default=1)
    if (H * P) % parts:
        raise ConfigError(f"config: {where}norm_groups is {parts}; it must divide heads * vdim "
                          f"({H * P})")
    return MixerSpec("selective_state_space", num_heads=H, num_kv_heads=G, head_dim=N,
                     value_dim=P, conv_taps=_int(m, "conv", where), norm_groups=parts,
                     norm_eps=eps, tensors=STATE_SPACE_TENSORS)


def _feed_forward(mlp, where: str) -> Optional[FeedForwardSpec]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config: {where}mlp must be an object or null")
    kind = mlp.get("kind")
    if kind == "dense":
        return FeedForwardSpec("gated_dense", intermediate_size=_int(mlp, "ff", where + "mlp."),
                               tensors=DENSE_TENSORS, activation="gelu_tanh")
    if kind == "moe":
        router = _object(mlp, "router", where + "mlp.")
        E = _int(router, "experts", where + "mlp.router.")
        top = _int(router, "top", where + "mlp.router.")
        if top > E or top > 32:
            raise ConfigError(f"config: {where}mlp.router.top is {top}; at most the number of "
                              f"experts ({E}) and at most 32")
        expert = _object(mlp, "expert", where + "mlp.")
        shared = _object(mlp, "shared", where + "mlp.", required=False)
        shared_spec = None
        if shared is not None:
            shared_spec = FeedForwardSpec("gated_dense",
                                          intermediate_size=_int(shared, "ff", where + "mlp.shared."),
                                          tensors=SHARED_TENSORS, activation="silu")
        return FeedForwardSpec("routed_experts",
                               intermediate_size=_int(expert, "ff", where + "mlp.expert."),
                               tensors=ROUTED_TENSORS, activation="silu", experts=E, top=top,
                               router_bias=True, shared=shared_spec)
    raise ConfigError(f"config: {where}mlp.kind is {kind!r}; known kinds: dense, moe")


def totatar_model_spec(raw: dict) -> ModelSpec:
    """config.json (as a dict) -> ModelSpec. Tensor names: `embed`, `l<i>.norm1|norm1b|norm2|
    norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`; the head is `embed`."""
    if not isinstance(raw, dict):
        raise ConfigError("config: the top level must be an object")
    d = _int(raw, "width", "")
    V = _int(raw, "vocab", "")
    norm = raw.get("norm")
    if not isinstance(norm, dict):
        raise ConfigError("config: norm is required (eps)")
    eps = _positive(norm, "eps", "norm.")
    nspec = NormSpec("group_rmsnorm", eps, 1, unit_offset=True)
    entries = raw.get("layers")
    if not isinstance(entries, list) or not entries:
        raise ConfigError("config: layers must list at least one layer")
    layers = []
    for i, e in enumerate(entries):
        where = f"layers[{i}]."
        if not isinstance(e, dict) or not isinstance(e.get("mixer"), dict):
            raise ConfigError(f"config: {where}mixer is required")
        kind, m = e.get("type"), e["mixer"]
        if kind == "parallel":
            mixer = _parallel(m, where + "mixer.", eps)
        elif kind == "mamba2":
            mixer = _state_space(m, where + "mixer.", eps)
        else:
            raise ConfigError(f"config: {where}type is {kind!r}; known mixers are mamba2, parallel")
        layers.append(LayerSpec("sandwich_norm_residual", f"l{i}.", mixer,
                                _feed_forward(e.get("mlp"), where), nspec, BLOCK_TENSORS))
    spec = ModelSpec(
        architecture=ARCHITECTURE, hidden_size=d, vocab_size=V, layers=layers,
        run_order=[LayerCall(i) for i in range(len(layers))], final_norm=nspec,
        embedding_name="embed", final_norm_name="final.norm", head_name=None, source=dict(raw))
    spec.validate()
    return spec
