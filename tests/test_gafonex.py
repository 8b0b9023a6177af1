"""Gafonex without a GPU: the config reader, the plain implementation against values worked
out by hand, and the engine's host side (cache, state slots, batching, cutting) with the torch
stand-ins for the kernels, against the plain implementation."""
import copy
import math

import numpy as np
import pytest
import torch

import emulated_kernels
import gafonex_tiny as gt
import plain_gafonex as plain
import tiny


# ------------------------------------------------------------------------------ the reader
def test_reader_builds_the_layers_the_file_lists():
    from tgo_b200.registry import model_spec_from_config
    spec = model_spec_from_config(gt.G1)
    assert spec.architecture == "Gafonex" and spec.hidden_size == 48 and spec.vocab_size == 97
    assert spec.logit_softcap == 12.0 and spec.final_norm.groups == 3
    kinds = [l.mixer.kind for l in spec.layers]
    assert kinds == ["retention", "mixed_head_attention", "mixed_head_attention", "retention",
                     "mixed_head_attention"]
    assert [l.mixer.value_share for l in spec.layers] == [None, "source", "blend", None, None]
    assert spec.layers[2].feed_forward is None and spec.layers[1].feed_forward.activation == "relu"
    assert spec.layers[0].mixer.decay == (0.5, 0.9, 1.0) and spec.layers[0].mixer.value_dim == 12
    assert spec.layers[1].mixer.position.kind == "rope_stretched"
    assert spec.layers[2].mixer.position.kind == "rope_half_split"
    assert model_spec_from_config(gt.G2).logit_softcap is None


@pytest.mark.parametrize("path,value,word", [
    (("width",), 0, "width"), (("norm", "groups"), 5, "norm.groups"),
    (("layers", 0, "type"), "conv", "layers[0].type"),
    (("layers", 0, "mixer", "decay"), [0.5], "decay"),
    (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 1, "mixer", "scale"), -1.0, "scale"),
    (("layers", 1, "mlp", "kind"), "moe", "mlp.kind"),
    (("logit_softcap",), 0.0, "logit_softcap")])
def test_reader_refuses_by_key(path, value, word):
    from tgo_b200.config.qwen3 import ConfigError
    from tgo_b200.registry import model_spec_from_config
    cfg = copy.deepcopy(gt.G1)
    at = cfg
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word.replace("[", r"\[").replace("]", r"\]")):
        model_spec_from_config(cfg)


def test_declared_tensors_are_the_checkpoints_names():
    from tgo_b200.engine.model import Model
    from tgo_b200.registry import model_spec_from_config
    for cfg in (gt.G1, gt.G2):
        W = gt.make_weights(cfg, 0)
        model = Model(model_spec_from_config(cfg), torch.float32, "cpu")
        need = {w.name: tuple(w.shape) for w in model.weight_specs() if not w.optional}
        assert need == {k: tuple(v.shape) for k, v in W.items()}


def test_a_written_folder_loads_with_its_scalars(tmp_path):
    from tgo_b200.engine.model import Model
    from tgo_b200.registry import model_spec_from_config
    from tgo_b200.weights.binder import load_weights
    from tgo_b200.weights.safetensors import SafetensorsRepo
    W = gt.make_weights(gt.G1, 0)
    d = gt.write_model_dir(str(tmp_path / "m"), gt.G1, W)
    model = Model(model_spec_from_config(gt.G1), torch.bfloat16, "cpu")
    repo = SafetensorsRepo(d)
    got = load_weights(model.weight_specs(), repo, torch.bfloat16, "cpu")
    repo.close()
    assert got["l2.mix.vmix"].shape == () and got["l2.mix.vmix"].dtype == torch.float32
    assert float(got["l2.mix.vmix"]) == float(W["l2.mix.vmix"])
    assert got["l1.mix.talk"].dtype == torch.float32 and got["l1.mix.q"].dtype == torch.bfloat16
    assert "l4.mix.vmix" not in got                     # outside the sharing: none shipped, none asked


# ------------------------------------------------------------- the plain statement by hand
def test_plain_pieces_by_hand():
    x = np.array([[3.0, 4.0, 0.0, 2.0]])
    got = plain.group_norm(x, np.array([1.0, 2.0, 1.0, 0.5]), 0.0, 2)
    r1, r2 = math.sqrt(12.5), math.sqrt(2.0)
    assert np.allclose(got, [[3 / r1, 8 / r1, 0.0, 1 / r2]])
    # two tokens of retention, one head, sizes 2 x 1
    q = np.array([[[1.0, 0.0]], [[1.0, 1.0]]])
    k = np.array([[[2.0, 1.0]], [[0.0, 3.0]]])
    v = np.array([[[5.0]], [[7.0]]])
    o = plain.retention_outputs(q, k, v, [0.5])
    assert np.allclose(o[:, 0, 0], [10.0, 0.5 * (10.0 + 5.0) + 21.0])
    # the stretched rotation: pair 0 turns fast (kept), the last pair slow (divided)
    rot = {"dims": 8, "base": 500.0, "scaling": gt.STRETCH}
    f, mag = plain.rotary_frequencies(rot)
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert f[0] == pytest.approx(1.0)
    base = [500.0 ** (-2.0 * i / 8) for i in range(4)]
    turns = lambda t: 8 * math.log(16 / (2 * math.pi * t)) / (2 * math.log(500.0))   # noqa: E731
    lo, hi = max(math.floor(turns(4.0)), 0), min(math.ceil(turns(1.0)), 7)
    for i in range(4):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0), 1)
        assert f[i] == pytest.approx(base[i] * (1 - ramp) + base[i] / 4.0 * ramp)
    # head mixing with the identity changes nothing; rows of mixed weights sum to the table's
    w = plain.attention_weights(np.random.default_rng(0).normal(size=(5, 2, 3)),
                                np.random.default_rng(1).normal(size=(5, 1, 3)), 0.7)
    assert np.allclose(plain.mix_heads(w, np.eye(2)), w)
    table = np.array([[0.2, 0.5], [1.0, -1.0]])
    assert np.allclose(plain.mix_heads(w, table).sum(-1), table.sum(1)[:, None] * np.ones((2, 5)))


# ---------------------------------------------------- the engine's host side on the CPU
@pytest.fixture()
def emulated(monkeypatch):
    emulated_kernels.install(monkeypatch)


def _engine(cfg, W, page_size, max_tokens, slots=4):
    from tgo_b200.engine.step import Engine
    model = gt.bind_model(cfg, W, torch.float32, "cpu")
    return Engine(model, page_size=page_size, max_tokens=max_tokens, num_slots=slots, graphs=False)


def _check(got, cfg, W, requests, tol=2e-4):
    for rid, toks in requests.items():
        want = plain.forward(cfg, W, toks)
        for p in range(len(toks)):
            assert np.abs(got[(rid, p)] - want[p]).max() <= tol * max(1.0, np.abs(want[p]).max()), \
                (rid, p)


@pytest.mark.parametrize("name", ["G1", "G2", "G3"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_engine_host_side_against_plain(emulated, name, family):
    cfg, page = gt.CONFIGS[name]
    W = gt.make_weights(cfg, 3)
    requests = tiny.random_requests(cfg["vocab"], [37, 9, 1, 50, 18, 26], seed=5)
    trace = {"whole": tiny.trace_whole, "tail": lambda r: tiny.trace_tail(r, 6),
             "portions": tiny.trace_portions,
             "mixed": lambda r: tiny.trace_mixed(r, seed=2, max_live=3, tail=5)}[family](requests)
    # a pool for what is live at once, three state slots: pages and slots come back and go out again
    eng = _engine(cfg, W, page, tiny.max_tokens_of(trace, page), slots=3)
    owners = [dict() for _ in eng.cache.groups]
    got = tiny.run_trace_engine(eng, trace, poison=True, owners=owners)
    _check(got, cfg, W, requests)
    if family == "mixed" and eng.cache.groups:
        assert any(len(ids) > 1 for g in owners for ids in g.values())      # a page was reused


def test_a_reused_state_slot_starts_from_zero(emulated):
    cfg, page = gt.CONFIGS["G1"]
    W = gt.make_weights(cfg, 4)
    eng = _engine(cfg, W, page, 64, slots=1)
    reqs = tiny.random_requests(cfg["vocab"], [20, 20], seed=9)
    got = tiny.run_trace_engine(eng, tiny.trace_whole(reqs))
    _check(got, cfg, W, reqs)


def test_a_failing_step_leaves_the_state_alone(emulated, monkeypatch):
    from tgo_b200.engine.step import StepEntry
    from tgo_b200.kernels import ops
    cfg, page = gt.CONFIGS["G1"]
    W = gt.make_weights(cfg, 5)
    eng = _engine(cfg, W, page, 64)
    toks = tiny.random_requests(cfg["vocab"], [12], seed=1)["r0"]
    eng.admit("a")
    eng.step([StepEntry("a", toks[:6], [])])
    real = ops.softcap

    def boom(*a):
        raise RuntimeError("boom")
    monkeypatch.setattr(ops, "softcap", boom)
    with pytest.raises(RuntimeError):
        eng.step([StepEntry("a", toks[6:], [5])])
    monkeypatch.setattr(ops, "softcap", real)
    assert eng.length("a") == 6
    got = eng.step([StepEntry("a", toks[6:], [5])])[0].numpy()
    want = plain.forward(cfg, W, toks)[-1]
    assert np.abs(got - want).max() < 2e-4 * np.abs(want).max()
