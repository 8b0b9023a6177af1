"""Totatar without a GPU: the config reader and its refusals, the declared tensor names, the
plain statement's pieces against values worked out by hand, and the engine's host side (cache
groups, state rows, packing, portions, mixed batches, reused pages and slots) with torch
stand-ins for the kernels, against the plain statement."""
import math

import numpy as np
import pytest
import torch

import emulated_kernels
import plain_totatar as plain
import tiny
import totatar_tiny as tt


def test_reader_builds_the_layers_the_file_lists():
    from tgo_b200.registry import model_spec_from_config
    spec = model_spec_from_config(tt.T1)
    assert spec.architecture == "Totatar" and spec.tied_head and len(spec.layers) == 4
    assert [ls.block for ls in spec.layers] == ["sandwich_norm_residual"] * 4
    assert spec.final_norm.unit_offset and spec.final_norm.groups == 1
    par = spec.layers[0].mixer
    assert par.kind == "parallel" and par.branch_scales == (0.7, 1.3)
    left, right = par.branches
    assert (left.kind, left.num_heads, left.num_kv_heads, left.head_dim, left.value_dim) == \
        ("sink_attention", 4, 2, 12, 20)
    assert left.window == 9 and left.bias and left.sink and left.scale == 0.4
    assert left.position.kind == "rope_interleaved" and left.position.rotary_dim == 8
    assert left.position.scaling == (4.0,)
    assert (right.kind, right.decay, right.input_activation, right.output_norm,
            right.gate_activation, right.scale) == \
        ("retention", (0.5, 0.9, 1.0), "silu", "joint_gain", "sigmoid", 1.0)
    ssm = spec.layers[1].mixer
    assert (ssm.kind, ssm.num_heads, ssm.value_dim, ssm.head_dim, ssm.num_kv_heads, ssm.conv_taps,
            ssm.norm_groups) == ("selective_state_space", 4, 6, 10, 2, 4, 2)
    ffn = spec.layers[1].feed_forward
    assert (ffn.kind, ffn.experts, ffn.top, ffn.intermediate_size, ffn.shared.intermediate_size) == \
        ("routed_experts", 5, 2, 24, 16)
    assert spec.layers[0].feed_forward.activation == "gelu_tanh"
    assert spec.layers[2].feed_forward.shared is None and spec.layers[3].feed_forward is None
    no_window = model_spec_from_config(tt.T2).layers[1].mixer.branches[0]
    assert no_window.window is None and no_window.position is None


def _changed(path, value):
    import copy
    cfg = copy.deepcopy(tt.T1)
    at = cfg
    for key in path[:-1]:
        at = at[key]
    if value is ...:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value,word", [
    (("width",), 0, "width"), (("vocab",), ..., "vocab"), (("norm", "eps"), -1.0, "norm.eps"),
    (("layers", 0, "type"), "conv", "layers[0].type"),
    (("layers", 0, "mixer", "left", "heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 7, "rot.dims"),
    (("layers", 0, "mixer", "left", "rot", "scaling"), {"factor": 2.0, "slow": 1.0}, "rot.scaling.slow"),
    (("layers", 0, "mixer", "left", "mask", "size"), 0, "mask.size"),
    (("layers", 0, "mixer", "right", "decay"), [0.5, 0.9], "decay"),
    (("layers", 0, "mixer", "right", "decay"), [0.5, 0.9, 1.5], "decay[2]"),
    (("layers", 1, "mixer", "groups"), 3, "groups"),
    (("layers", 1, "mixer", "norm_groups"), 5, "norm_groups"),
    (("layers", 1, "mixer", "state"), 1000, "state"),
    (("layers", 1, "mlp", "router", "top"), 6, "router.top"),
    (("layers", 1, "mlp", "kind"), "sparse", "mlp.kind"),
    (("layers", 0, "mlp", "ff"), ..., "mlp.ff"),
])
def test_reader_refuses_by_key(path, value, word):
    from tgo_b200.config.qwen3 import ConfigError
    from tgo_b200.registry import model_spec_from_config
    with pytest.raises(ConfigError) as err:
        model_spec_from_config(_changed(path, value))
    assert word in str(err.value)


@pytest.mark.parametrize("name", ["T1", "T2", "T3", "T4", "T5"])
def test_declared_tensors_are_the_weights_the_tests_make(name):
    from tgo_b200.engine.model import Model
    from tgo_b200.registry import model_spec_from_config
    cfg, _ = tt.CONFIGS[name]
    W = tt.make_weights(cfg, 1)
    model = Model(model_spec_from_config(cfg), torch.float32, "cpu")
    declared = {w.name: tuple(w.shape) for w in model.weight_specs() if not w.optional}
    assert declared == {k: tuple(v.shape) for k, v in W.items()}


def test_a_written_folder_loads(tmp_path):
    from tgo_b200.engine.model import Model
    from tgo_b200.registry import model_spec_from_config
    from tgo_b200.weights.binder import WeightError, load_weights
    from tgo_b200.weights.safetensors import SafetensorsRepo
    W = tt.make_weights(tt.T1, 2)
    d = tt.write_model_dir(str(tmp_path / "m"), tt.T1, W)
    model = Model(model_spec_from_config(tt.T1), torch.bfloat16, "cpu")
    repo = SafetensorsRepo(d)
    weights = load_weights(model.weight_specs(), repo, torch.bfloat16, "cpu", None, log=None)
    assert weights["l1.mlp.router"].dtype == torch.float32          # the router stays 32-bit
    assert weights["l0.mix.left.sink"].dtype == torch.float32
    assert weights["l1.mix.conv"].shape == (4 * 6 + 2 * 2 * 10, 4)
    model.bind(dict(weights))
    blk = model.blocks[0]
    assert torch.allclose(blk.norm1.gain, 1.0 + torch.from_numpy(W["l0.norm1"]).float())
    # a layer without a feed-forward may ship its second pair of norms; nothing else may be extra
    W2 = dict(W)
    W2["l3.norm2"] = W["l0.norm2"]
    d2 = tt.write_model_dir(str(tmp_path / "m2"), tt.T1, W2)
    load_weights(model.weight_specs(), SafetensorsRepo(d2), torch.bfloat16, "cpu", None, log=None)
    W2["l3.mlp.gate"] = W["l0.mlp.gate"]
    d3 = tt.write_model_dir(str(tmp_path / "m3"), tt.T1, W2)
    with pytest.raises(WeightError):
        load_weights(model.weight_specs(), SafetensorsRepo(d3), torch.bfloat16, "cpu", None, log=None)


def test_plain_pieces_by_hand():
    # the norm's weight is zero-centred: the gain is 1 + w
    x = np.array([[3.0, 4.0]])
    assert np.allclose(plain.offset_norm(x, np.array([0.0, 1.0]), 0.0), [[3 / math.sqrt(12.5), 8 / math.sqrt(12.5)]])
    # neighbouring channels turn together; a quarter turn at position 1, base 1, slowed by 2 is an eighth
    v = np.zeros((2, 1, 4))
    v[:, 0] = [1.0, 0.0, 5.0, 6.0]
    r = plain.rotate_interleaved(v, [0, 1], {"dims": 2, "base": 1.0, "scaling": {"factor": 2.0}})
    assert np.allclose(r[0, 0], [1, 0, 5, 6])
    assert np.allclose(r[1, 0], [math.cos(0.5), math.sin(0.5), 5, 6])
    # a sink takes its share of the softmax and gives nothing back; a window of one sees only itself
    q = np.ones((3, 1, 1))
    k = np.zeros((3, 1, 1))
    val = np.array([1.0, 2.0, 4.0]).reshape(3, 1, 1)
    out = plain.sink_window_attention(q, k, val, 1.0, None, np.array([0.0]))
    assert np.allclose(out[:, 0, 0], [1 / 2, 3 / 3, 7 / 4])
    out = plain.sink_window_attention(q, k, val, 1.0, 1, np.array([math.log(3.0)]))
    assert np.allclose(out[:, 0, 0], [1 / 4, 2 / 4, 4 / 4])
    out = plain.sink_window_attention(q, k, val, 1.0, 2, None)
    assert np.allclose(out[:, 0, 0], [1, 1.5, 3])
    # the convolution's last column meets the current token, zeros lie before the start
    y = plain.causal_conv(np.array([[1.0], [2.0], [3.0]]), np.array([[10.0, 1.0]]), np.array([0.5]))
    assert np.allclose(y[:, 0], [1.5, 12.5, 23.5])
    # the scan: S <- exp(-A dt) S + dt B x^T, y = S^T C + D x
    y = plain.selective_scan(np.ones((2, 1, 1)), np.array([[1.0], [2.0]]), np.array([math.log(2.0)]),
                             np.ones((2, 1, 1)), np.array([[[1.0]], [[3.0]]]), np.array([0.5]), 1)
    assert np.allclose(y[:, 0, 0], [1 + 0.5, (0.25 * 1 + 2) * 3 + 0.5])
    # fixed decay
    o = plain.decayed_linear_attention(np.ones((2, 1, 1)), np.ones((2, 1, 1)),
                                       np.array([2.0, 3.0]).reshape(2, 1, 1), [0.5])
    assert np.allclose(o[:, 0, 0], [2, 4])
    # routing: the top two by logit (ties to the lower index), softmax over those two alone
    W = {"r.router": np.array([[1.0], [3.0], [3.0]]), "r.router.b": np.array([0.0, 0.0, 0.0])}
    for e, g in enumerate([1.0, 2.0, 4.0]):
        W[f"r.e{e}.gate"] = np.array([[30.0]])
        W[f"r.e{e}.up"] = np.array([[1.0 / 30.0]])          # silu(30) is 30 to 1e-11
        W[f"r.e{e}.down"] = np.array([[g]])
    out = plain.routed(np.array([[1.0]]), W, "r.", {"router": {"experts": 3, "top": 2}})
    assert np.allclose(out, [[0.5 * 2 + 0.5 * 4]])
    out = plain.routed(np.array([[1.0]]), W, "r.", {"router": {"experts": 3, "top": 1}})
    assert np.allclose(out, [[2.0]])


# ---------------------------------------------------- the engine's host side on the CPU
@pytest.fixture()
def emulated(monkeypatch):
    emulated_kernels.install(monkeypatch)


def _engine(cfg, W, page_size, max_tokens, slots=4):
    from tgo_b200.engine.step import Engine
    model = tt.bind_model(cfg, W, torch.float32, "cpu")
    return Engine(model, page_size=page_size, max_tokens=max_tokens, num_slots=slots, graphs=False)


def _check(got, cfg, W, requests, tol=2e-4):
    for rid, toks in requests.items():
        want = plain.forward(cfg, W, toks)
        for p in range(len(toks)):
            assert np.abs(got[(rid, p)] - want[p]).max() <= tol * max(1.0, np.abs(want[p]).max()), \
                (rid, p)


@pytest.mark.parametrize("name", ["T1", "T2", "T3", "T4"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_engine_host_side_against_plain(emulated, name, family):
    cfg, page = tt.CONFIGS[name]
    W = tt.make_weights(cfg, 3)
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
    from tgo_b200.engine.step import StepEntry
    cfg, page = tt.CONFIGS["T3"]
    W = tt.make_weights(cfg, 4)
    eng = _engine(cfg, W, page, 64, slots=1)
    first, second = [3, 7, 11, 2, 9, 30, 1], [5, 1, 8, 40]
    for rid, toks in (("a", first), ("b", second)):
        eng.admit(rid)
        got = eng.step([StepEntry(rid, toks, list(range(len(toks))))]).numpy()
        want = plain.forward(cfg, W, toks)
        assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())
        eng.finish(rid)


def test_a_failing_step_leaves_the_state_alone(emulated, monkeypatch):
    from tgo_b200.engine.step import StepEntry
    from tgo_b200.kernels import ops
    cfg, page = tt.CONFIGS["T1"]
    W = tt.make_weights(cfg, 5)
    eng = _engine(cfg, W, page, 64, slots=2)
    toks = [4, 9, 60, 33, 2, 17, 5, 80, 41]
    eng.admit("a")
    eng.step([StepEntry("a", toks[:4], [])])
    good = ops.gated_group_norm
    calls = []

    def failing(*a, **k):
        calls.append(1)
        if len(calls) == 3:              # the third layer's mixer: two states have moved already
            raise RuntimeError("no")
        return good(*a, **k)
    monkeypatch.setattr(ops, "gated_group_norm", failing)
    with pytest.raises(RuntimeError):
        eng.step([StepEntry("a", toks[4:], [])])
    monkeypatch.setattr(ops, "gated_group_norm", good)
    assert eng.length("a") == 4
    got = eng.step([StepEntry("a", toks[4:], list(range(5)))]).numpy()
    want = plain.forward(cfg, W, toks)[4:]
    assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())
