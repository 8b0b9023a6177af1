"""Small Gafonex configurations with weights of the tests' own making.

  G1: every size different from every other (3 norm groups; retention 3 heads of 8 x 12 with
      a partial rotation and decays 0.5, 0.9, 1; attention 4/2 heads of 12 x 20, one layer with
      a stretched partial rotation, one with a full plain one; value sharing over two layers
      and a third attention layer outside it; one layer without feed-forward).
  G2: the values a model may happen to make equal or 1: one norm group, one retention head,
      kv heads = heads, key size = value size, an attention layer first, 9 query heads (more
      than the generic kernel has warps), value size above 32, no soft cap, one sharing layer
      only (a source that nobody reads).
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch


def _att(H, G, a, b, rot, scale, v_mix=None):
    m = {"heads": H, "kv_heads": G, "dim": a, "vdim": b, "rot": rot, "scale": scale}
    if v_mix is not None:
        m["v_mix"] = v_mix
    return m


def _ret(H, a, b, rot, decay):
    m = {"heads": H, "dim": a, "vdim": b, "decay": decay}
    if rot is not None:
        m["rot"] = rot
    return m


STRETCH = {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}

G1 = {
    "architecture": "Gafonex", "vocab": 97, "width": 48, "logit_softcap": 12.0,
    "norm": {"eps": 1e-5, "groups": 3},
    "layers": [
        {"type": "retention", "mixer": _ret(3, 8, 12, {"dims": 4, "base": 100.0}, [0.5, 0.9, 1.0]),
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "attention", "mixer": _att(4, 2, 12, 20, {"dims": 8, "base": 500.0,
                                                           "scaling": STRETCH}, 0.4, True),
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "attention", "mixer": _att(4, 2, 12, 20, {"dims": 12, "base": 50.0}, 0.3, True),
         "mlp": None},
        {"type": "retention", "mixer": _ret(2, 16, 4, {"dims": 16, "base": 10.0}, [0.97, 0.75]),
         "mlp": {"kind": "dense", "ff": 56}},
        {"type": "attention", "mixer": _att(2, 1, 8, 8, {"dims": 2, "base": 7.0}, 0.5, False),
         "mlp": {"kind": "dense", "ff": 24}},
    ],
}

G2 = {
    "architecture": "Gafonex", "vocab": 70, "width": 40,
    "norm": {"eps": 1e-6, "groups": 1},
    "layers": [
        {"type": "attention", "mixer": _att(9, 9, 20, 40, {"dims": 20, "base": 1000.0,
                                                           "scaling": {"factor": 2.0, "original": 8,
                                                                       "fast": 2.0, "slow": 0.5}},
                                           0.2, True),
         "mlp": {"kind": "dense", "ff": 72}},
        {"type": "retention", "mixer": _ret(1, 24, 24, {"dims": 24, "base": 1e4}, [0.99]),
         "mlp": None},
        {"type": "attention", "mixer": _att(3, 3, 16, 16, {"dims": 8, "base": 20.0}, 0.25),
         "mlp": {"kind": "dense", "ff": 72}},
    ],
}

# retention only: no layer owns a paged cache, every layer a state
G3 = {
    "architecture": "Gafonex", "vocab": 50, "width": 32, "logit_softcap": 20.0,
    "norm": {"eps": 1e-5, "groups": 2},
    "layers": [
        {"type": "retention", "mixer": _ret(2, 8, 8, {"dims": 8, "base": 100.0}, [0.9, 0.99]),
         "mlp": {"kind": "dense", "ff": 48}},
        {"type": "retention", "mixer": _ret(4, 4, 8, None, [0.5, 0.8, 0.95, 1.0]), "mlp": None},
    ],
}

CONFIGS = {"G1": (G1, 8), "G2": (G2, 16), "G3": (G3, 16)}           # config, page size


def bf16_values(x: np.ndarray) -> np.ndarray:
    """float64 values that bfloat16 holds exactly (what a checkpoint would store)."""
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).to(torch.bfloat16).double().numpy()


def make_weights(cfg, seed):
    """name -> float64 array of bfloat16-exact values; lively enough that tokens differ."""
    rng = np.random.default_rng(seed)
    d, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, out, inp, gain=1.0):
        W[name] = rng.normal(0, gain / np.sqrt(inp), (out, inp))

    def gain(name, n):
        W[name] = 1.0 + 0.2 * rng.normal(0, 1, n)
    W["embed"] = rng.normal(0, 1.0, (V, d))
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        gain(p + "norm1", d)
        W[p + "ls1"] = 0.5 + 0.2 * rng.normal(0, 1, d)
        H, a = m["heads"], m["dim"]
        b = m.get("vdim", a)
        if L["type"] == "attention":
            G = m.get("kv_heads", H)
            mat(p + "mix.q", H * a, d)
            mat(p + "mix.k", G * a, d)
            mat(p + "mix.v", G * b, d)
            gain(p + "mix.q.norm", a)
            gain(p + "mix.k.norm", a)
            W[p + "mix.talk"] = np.eye(H) * 0.7 + 0.3 * rng.normal(0, 1, (H, H))
            if m.get("v_mix"):
                W[p + "mix.vmix"] = np.array(0.35 + 0.1 * rng.normal())
            mat(p + "mix.o", d, H * b)
        else:
            for nm, n in (("q", H * a), ("k", H * a), ("v", H * b), ("g", H * b)):
                mat(p + "mix." + nm, n, d, 2.0)
            mat(p + "mix.o", d, H * b)
        if L.get("mlp"):
            f = L["mlp"]["ff"]
            gain(p + "norm2", d)
            W[p + "ls2"] = 0.5 + 0.2 * rng.normal(0, 1, d)
            mat(p + "mlp.gate", f, d)
            mat(p + "mlp.up", f, d)
            mat(p + "mlp.down", d, f)
    gain("final.norm", d)
    mat("head", V, d, 3.0)
    return {k: bf16_values(v) for k, v in W.items()}


def write_model_dir(path, cfg, W):
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
