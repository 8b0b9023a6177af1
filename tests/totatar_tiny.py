"""Small Totatar configurations with weights of the tests' own making.

  T1: every size different from every other: parallel layers with 4/2 and 3/1 attention heads,
      keys and values of different widths, windows of 9 and 20 tokens (shorter and longer than
      a page), a partial rotation slowed by a factor and a full plain one, linear attention
      with decays 0.5, 0.9, 1; state-space layers with two groups and 4 taps, one group and 2
      taps; a dense feed-forward, experts with and without a shared one, and none.
  T2: the values a model may happen to make equal or 1: kv heads = heads, key size = value
      size, no window in one layer and one longer than any request in the other, no rotation
      in one layer, one linear-attention head, scales of 1, one expert taken of one, one tap
      (no convolution state), groups = heads, one norm part, nine attention heads.
  T3: state-space layers only: no layer owns a paged cache.
  T4: sizes that no kernel's fast form takes (a width, key and value sizes, channel counts,
      expert widths and a vocabulary that are not multiples of 8; a state that is not a
      multiple of 4; a window of 1), and a parallel layer without a feed-forward.
  T5: a width the fast products take (a multiple of 8) with odd numbers of output columns (three
      state-space heads, an odd vocabulary) and a feed-forward width that is not a multiple of 8.
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch


def _left(H, G, a, b, window, rot, scale):
    m = {"heads": H, "kv_heads": G, "dim": a, "vdim": b, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = rot
    return m


def _par(left, H, a, b, decay, ls, rs):
    return {"left": left, "right": {"heads": H, "dim": a, "vdim": b, "decay": decay},
            "left_scale": ls, "right_scale": rs}


def _ssm(H, P, N, G, taps, parts):
    return {"heads": H, "vdim": P, "state": N, "groups": G, "conv": taps, "norm_groups": parts}


def _moe(E, top, ff, shared):
    m = {"kind": "moe", "router": {"experts": E, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


T1 = {
    "architecture": "Totatar", "vocab": 97, "width": 48, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "parallel",
         "mixer": _par(_left(4, 2, 12, 20, 9, {"dims": 8, "base": 500.0, "scaling": {"factor": 4.0}}, 0.4),
                       3, 8, 12, [0.5, 0.9, 1.0], 0.7, 1.3),
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "mamba2", "mixer": _ssm(4, 6, 10, 2, 4, 2), "mlp": _moe(5, 2, 24, 16)},
        {"type": "parallel",
         "mixer": _par(_left(3, 1, 16, 8, 20, {"dims": 16, "base": 50.0}, 0.3),
                       2, 16, 4, [0.97, 0.75], 1.1, 0.6),
         "mlp": _moe(7, 3, 8, None)},
        {"type": "mamba2", "mixer": _ssm(3, 8, 16, 1, 2, 1), "mlp": None},
    ],
}

T2 = {
    "architecture": "Totatar", "vocab": 70, "width": 40, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mamba2", "mixer": _ssm(2, 20, 9, 2, 1, 1), "mlp": _moe(1, 1, 32, 40)},
        {"type": "parallel",
         "mixer": _par(_left(9, 9, 20, 20, None, None, 0.25), 1, 24, 24, [0.99], 1.0, 1.0),
         "mlp": {"kind": "dense", "ff": 72}},
        {"type": "parallel",
         "mixer": _par(_left(2, 2, 8, 8, 1000, {"dims": 2, "base": 7.0, "scaling": {"factor": 1.0}}, 0.5),
                       4, 4, 8, [0.5, 0.8, 0.95, 1.0], 1.0, 1.0),
         "mlp": _moe(4, 4, 16, None)},
    ],
}

T3 = {
    "architecture": "Totatar", "vocab": 50, "width": 32, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "mamba2", "mixer": _ssm(2, 16, 20, 1, 3, 2), "mlp": {"kind": "dense", "ff": 48}},
        {"type": "mamba2", "mixer": _ssm(8, 4, 6, 4, 5, 4), "mlp": None},
    ],
}

T4 = {
    "architecture": "Totatar", "vocab": 53, "width": 36, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "mamba2", "mixer": _ssm(3, 5, 7, 3, 3, 3), "mlp": _moe(3, 2, 12, 20)},
        {"type": "parallel",
         "mixer": _par(_left(6, 3, 10, 6, 1, {"dims": 6, "base": 30.0}, 0.35), 2, 6, 10, [0.9, 0.6], 0.5, 2.0),
         "mlp": None},
        {"type": "parallel",
         "mixer": _par(_left(2, 1, 14, 18, 33, {"dims": 14, "base": 100.0, "scaling": {"factor": 3.0}}, 0.3),
                       3, 10, 6, [1.0, 0.8, 0.2], 1.0, 1.0),
         "mlp": {"kind": "dense", "ff": 44}},
    ],
}

T5 = {
    "architecture": "Totatar", "vocab": 61, "width": 40, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mamba2", "mixer": _ssm(3, 8, 12, 1, 4, 3), "mlp": {"kind": "dense", "ff": 44}},
        {"type": "parallel",
         "mixer": _par(_left(3, 1, 8, 24, 50, {"dims": 4, "base": 200.0, "scaling": {"factor": 2.0}}, 0.4),
                       1, 8, 8, [0.95], 0.9, 1.2),
         "mlp": _moe(6, 2, 24, 8)},
    ],
}

CONFIGS = {"T1": (T1, 8), "T2": (T2, 16), "T3": (T3, 16), "T4": (T4, 4), "T5": (T5, 16)}   # config, page size


def bf16_values(x: np.ndarray) -> np.ndarray:
    """float64 values that bfloat16 holds exactly (what a checkpoint would store)."""
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).to(torch.bfloat16).double().numpy()


def make_weights(cfg, seed):
    """name -> float64 array of bfloat16-exact values; lively enough that tokens differ, that
    sinks and biases matter and that the experts a token takes change from token to token."""
    rng = np.random.default_rng(seed)
    d, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, out, inp, gain=1.0):
        W[name] = rng.normal(0, gain / np.sqrt(inp), (out, inp))

    def vec(name, n, mean=0.0, sd=0.2):
        W[name] = mean + sd * rng.normal(0, 1, n)

    def ffn(p, f):
        mat(p + "gate", f, d, 1.5)
        mat(p + "up", f, d)
        mat(p + "down", d, f)
    W["embed"] = rng.normal(0, 1.0, (V, d))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", d)
        vec(p + "norm1b", d)
        if L["type"] == "parallel":
            lf, rt = m["left"], m["right"]
            H, a = lf["heads"], lf["dim"]
            G, b = lf.get("kv_heads", H), lf.get("vdim", a)
            for nm, n in (("q", H * a), ("k", G * a), ("v", G * b)):
                mat(p + "mix.left." + nm, n, d, 1.5)
                vec(p + "mix.left." + nm + ".b", n, 0.0, 0.3)
            vec(p + "mix.left.sink", H, 0.5, 1.0)
            mat(p + "mix.left.o", d, H * b)
            H, a = rt["heads"], rt["dim"]
            b = rt.get("vdim", a)
            for nm, n in (("q", H * a), ("k", H * a), ("v", H * b), ("g", H * b)):
                mat(p + "mix.right." + nm, n, d, 2.0)
            vec(p + "mix.right.norm", H * b, 1.0)
            mat(p + "mix.right.o", d, H * b)
        else:
            H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m.get("groups", 1), m["conv"]
            C = H * P + 2 * G * N
            mat(p + "mix.in", 2 * H * P + 2 * G * N + H, d, 1.5)
            W[p + "mix.conv"] = rng.normal(0, 0.6, (C, taps))
            vec(p + "mix.conv.b", C, 0.0, 0.2)
            vec(p + "mix.dt_bias", H, -0.5, 0.5)
            vec(p + "mix.A_log", H, -1.0, 0.7)
            vec(p + "mix.D", H, 1.0, 0.3)
            vec(p + "mix.norm", H * P, 1.0)
            mat(p + "mix.o", d, H * P)
        mlp = L.get("mlp")
        if mlp:
            vec(p + "norm2", d)
            vec(p + "norm2b", d)
            if mlp["kind"] == "dense":
                ffn(p + "mlp.", mlp["ff"])
            else:
                E = mlp["router"]["experts"]
                for e in range(E):
                    ffn(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
                mat(p + "mlp.router", E, d, 3.0)
                vec(p + "mlp.router.b", E, 0.0, 0.5)
                if mlp.get("shared"):
                    ffn(p + "mlp.shared.", mlp["shared"]["ff"])
    vec("final.norm", d)
    return {k: bf16_values(v) for k, v in W.items()}


def write_model_dir(path, cfg, W):
    """config.json + model.safetensors (bfloat16) of these weights."""
    from tgo_b200.weights.safetensors import write_safetensors
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      {k: torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16)
                       for k, v in W.items()})
    return str(path)


def bind_model(cfg, W, dtype, device):
    """A tgo_b200 Model with these weights, without a folder."""
    from tgo_b200.engine.model import Model
    from tgo_b200.registry import model_spec_from_config
    model = Model(model_spec_from_config(cfg), dtype, device)
    weights = {}
    for ws in model.weight_specs():
        if ws.optional and ws.name not in W:
            continue
        store = torch.float32 if ws.role in ("gain", "constant") else dtype
        weights[ws.name] = torch.from_numpy(np.asarray(W[ws.name], dtype=np.float32)).to(
            device=device, dtype=store)
    model.bind(weights)
    return model
