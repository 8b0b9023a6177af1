"""Totatar on the GPU: every new kernel alone against the plain statement of its mechanism
(with inputs made so that a far key, a window's edge, a sink or a lost state shows), then the
engine against the plain model: whole prompts, decoding, portions down to two tokens, mixed
batches with pages and state slots that come back, first tokens, long decoding, a long prompt,
and greedy generation through the library's entry point, the scheduler and the command line."""
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_totatar as plain
import tiny
import totatar_tiny as tt

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(x, dtype=torch.float32):
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).to(device=DEV, dtype=dtype)


def ints(x):
    return torch.tensor(list(x), dtype=torch.int32, device=DEV)


def close(got, want, tol, what=""):
    got = got.detach().float().cpu().numpy().astype(np.float64)
    err = np.abs(got - want).max()
    assert err <= tol * max(1.0, np.abs(want).max()), f"{what}: {err}"


TOL = {torch.float32: 3e-5, torch.bfloat16: 2e-2}


# ------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,groups,act,first,gain", [(48, 3, "silu", True, True), (40, 1, "sigmoid", False, True),
                                                     (2048, 2, "silu", False, False), (6, 6, None, False, True)])
def test_gated_group_norm(W, groups, act, first, gain, dtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(W)
    o = rng.normal(size=(5, W)) * 3
    z = tt.bf16_values(rng.normal(size=(5, 2 * W)))[:, W:]          # a column view of a wider row
    g = rng.normal(size=W) if gain else None
    zz = dev(np.concatenate([z, z], 1), dtype)[:, W:] if act else None
    out = torch.empty((5, W), dtype=dtype, device=DEV)
    ops.gated_group_norm(dev(o), zz, dev(g) if gain else None, out, groups, 1e-5, act, first)
    gate = plain.silu(z) if act == "silu" else plain.sigmoid(z) if act == "sigmoid" else 1.0
    want = plain.group_norm(o * gate if first else o, g if gain else 1.0, 1e-5, groups)
    want = want if first else want * gate
    close(out, want, TOL[dtype])


def test_weighted_sum_and_interleaved_table():
    from tgo_b200.config.spec import PositionSpec
    from tgo_b200.kernels import ops
    from tgo_b200.parts.position import RopeInterleaved
    rng = np.random.default_rng(0)
    a, b = rng.normal(size=(7, 33)), rng.normal(size=(7, 33))
    out = torch.empty((7, 33), dtype=torch.float32, device=DEV)
    ops.weighted_sum([dev(a), dev(b)], [0.8, -1.1], out)
    close(out, np.float32(0.8) * a + np.float32(-1.1) * b, 1e-6)
    ops.weighted_sum([dev(a)], [0.5], out)
    close(out, 0.5 * a, 1e-6)
    pos = RopeInterleaved(PositionSpec("rope_interleaved", rotary_dim=6, theta=100.0, scaling=(4.0,)),
                          8, DEV)
    want = np.array([100.0 ** (-2.0 * i / 6) / 4.0 for i in range(3)])
    assert np.allclose(pos.inv_freq.cpu().numpy(), want, rtol=1e-12)


def _paged(rows, page_size, table, pages_total, dtype):
    """rows [n, heads, width] of one request laid into a plane [pages, heads, page, width]
    through its block table; unheld pages are NaN."""
    n, heads, width = rows.shape
    plane = torch.full((pages_total, heads, page_size, width), float("nan"), dtype=dtype, device=DEV)
    for j in range(n):
        plane[table[j // page_size], :, j % page_size, :] = dev(rows[j], dtype)
    return plane


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,a,b,rot,inter,ps", [(4, 2, 12, 20, 8, True, 8), (3, 3, 16, 16, 16, True, 4),
                                                   (2, 1, 40, 8, 0, True, 16), (5, 1, 8, 48, 4, False, 8)])
def test_projection_rows_biased_rotated_and_stored(H, G, a, b, rot, inter, ps, dtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(H * a)
    n = 11
    positions = [0, 1, 2, 50, 51, 5000, 3, 4, 5, 6, 7]
    slots = [17, 3, 40, 41, 8, 9, -1, 2, 63, 0, 31]                # one row is not stored
    joined = tt.bf16_values(rng.normal(size=(n, H * a + G * a + G * b)))
    bq, bk, bv = (tt.bf16_values(rng.normal(size=m)) for m in (H * a, G * a, G * b))
    x = dev(joined, dtype)
    q, k, v = x[:, :H * a], x[:, H * a:H * a + G * a], x[:, H * a + G * a:]
    rope = None
    rot_cfg = None
    if rot:
        rot_cfg = {"dims": rot, "base": 50.0, "scaling": {"factor": 2.0}}
        freq = torch.tensor([50.0 ** (-2.0 * i / rot) / 2.0 for i in range(rot // 2)], dtype=torch.float64,
                            device=DEV)
        rope = ops.rope_table(ints(positions), freq)
    pages = 64 // ps                                               # the slots below lie within 64
    kc = torch.zeros((pages, G, ps, a), dtype=dtype, device=DEV)
    vc = torch.zeros((pages, G, ps, b), dtype=dtype, device=DEV)
    ops.qkv_bias_rope_cache(q, k, v, H, G, a, b, dev(bq), dev(bk), dev(bv), rope, rot, inter,
                            ints(slots), kc, vc, ps)
    turn = plain.rotate_interleaved if inter else _rotate_half
    want_q = turn((joined[:, :H * a] + bq).reshape(n, H, a), positions, rot_cfg)
    want_k = turn((joined[:, H * a:H * a + G * a] + bk).reshape(n, G, a), positions, rot_cfg)
    want_v = (joined[:, H * a + G * a:] + bv).reshape(n, G, b)
    close(q, want_q.reshape(n, -1), TOL[dtype], "q")
    for t, s in enumerate(slots):
        if s >= 0:
            close(kc[s // ps, :, s % ps], want_k[t], TOL[dtype], "k")
            close(vc[s // ps, :, s % ps], want_v[t], TOL[dtype], "v")
    stored = {(s // ps, s % ps) for s in slots if s >= 0}
    for pg in range(pages):
        for off in range(ps):
            if (pg, off) not in stored:
                assert float(kc[pg, :, off].abs().max()) == 0.0


def _rotate_half(x, positions, rot):
    if rot is None:
        return x
    dims, half = rot["dims"], rot["dims"] // 2
    out = x.copy()
    for t, p in enumerate(positions):
        for i in range(half):
            ang = p * (rot["base"] ** (-2.0 * i / dims) / rot["scaling"]["factor"])
            c, s = math.cos(ang), math.sin(ang)
            out[t, :, i] = x[t, :, i] * c - x[t, :, i + half] * s
            out[t, :, i + half] = x[t, :, i + half] * c + x[t, :, i] * s
    return out


def _attention_case(H, G, a, b, ps, n, loud, rng):
    """One request of n tokens whose key `loud` is made to stand out for every query (its key
    is a multiple of a direction every query shares), so that a window that is one token off,
    or a far key that is dropped, changes the result visibly."""
    q = rng.normal(size=(n, H, a))
    k = rng.normal(size=(n, G, a))
    v = rng.normal(size=(n, G, b))
    direction = rng.normal(size=a)
    direction /= np.linalg.norm(direction)
    q += 3.0 * direction
    if loud is not None:
        k[loud] = (4.0 + 1.5 * math.sqrt(a)) * direction
        v[loud] = 10.0
    return tt.bf16_values(q), tt.bf16_values(k), tt.bf16_values(v)


def _run_attention(fn, q, k, v, H, G, a, b, ps, dtype, positions, **kw):
    """Queries at `positions` of one request whose n keys lie in shuffled pages."""
    n = k.shape[0]
    pages = (n + ps - 1) // ps
    table = list(np.random.default_rng(7).permutation(np.arange(1, pages + 3))[:pages])
    kc, vc = _paged(k, ps, table, pages + 3, dtype), _paged(v, ps, table, pages + 3, dtype)
    bt = torch.zeros((2, pages + 2), dtype=torch.int32, device=DEV)
    bt[1, :pages] = ints(table)
    qq = dev(q[positions].reshape(len(positions), -1), dtype)
    out = torch.empty((len(positions), H * b), dtype=dtype, device=DEV)
    fn(qq, out, kc, vc, bt, ints([1] * len(positions)), ints(positions), **kw)
    return out


ATT_SIZES = [(4, 2, 12, 20, 8), (3, 1, 16, 8, 4), (9, 9, 20, 20, 16), (6, 2, 88, 72, 16), (8, 2, 64, 64, 16),
             (2, 2, 128, 128, 16)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,a,b,ps", ATT_SIZES)
def test_attention_with_window_and_sink_generic(H, G, a, b, ps, dtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(H + a)
    n, window = 150, 37
    sink = rng.normal(size=H) + 1.0

    def fn(qq, out, kc, vc, bt, seq, pos, **kw):
        ops.attention_generic(qq, out, H, G, a, kc, vc, ps, bt, seq, pos, 0.3, kw["window"],
                              value_dim=b, sinks=kw["sinks"])
    for loud in (0, 100 - window, 100 - window + 1, 99, None):
        q, k, v = _attention_case(H, G, a, b, ps, n, loud, rng)
        for w, sk in ((window, sink), (0, sink), (window, None), (1, sink)):
            want = plain.sink_window_attention(q, k, v, 0.3, w or None, sk).reshape(n, -1)
            picks = [0, 1, 36, 37, 99, 100, 101, 149]
            got = _run_attention(fn, q, k, v, H, G, a, b, ps, dtype, picks, window=w,
                                 sinks=dev(sk) if sk is not None else None)
            close(got, want[picks], TOL[dtype], f"loud {loud} window {w}")
    # the loud key just outside the window of query 100 must not be seen, just inside it must
    q, k, v = _attention_case(H, G, a, b, ps, n, 100 - window, rng)
    out_ = plain.sink_window_attention(q, k, v, 0.3, window, sink)[100]
    in_ = plain.sink_window_attention(q, k, v, 0.3, window + 1, sink)[100]
    assert np.abs(out_ - in_).max() > 1.0


TILE_SIZES = [(4, 2, 16, 24, 8), (3, 1, 16, 8, 4), (6, 2, 88, 72, 16), (8, 2, 64, 64, 16), (2, 2, 128, 128, 16),
              (16, 1, 32, 120, 16), (5, 5, 40, 40, 8), (40, 1, 8, 16, 16)]


@pytest.mark.parametrize("H,G,a,b,ps", TILE_SIZES)
def test_attention_with_window_and_sink_on_the_tensor_cores(H, G, a, b, ps):
    """The tile kernel over a whole request cut into tiles, over a portion that starts in the
    middle of a window and of a page, and over single tokens; windows shorter and longer than a
    key tile, none, and one; a loud key just inside and just outside the window."""
    from tgo_b200.kernels import ops
    assert ops.attention_sink_supports(H, G, a, b)
    rng = np.random.default_rng(H + a)
    n, bf = 333, torch.bfloat16
    sink = rng.normal(size=H) + 1.0
    per = ops.attention_sink_tile_tokens(H // G)

    def tiles_of(first, count):
        t0 = list(range(0, count, per))
        return ints(t0), ints([min(per, count - t) for t in t0])

    for window, loud in ((37, 200 - 37), (37, 200 - 36), (100, 3), (0, 0), (1, 199), (64, 136), (65, 136)):
        q, k, v = _attention_case(H, G, a, b, ps, n, loud, rng)
        for sk in (sink, None):
            want = plain.sink_window_attention(q, k, v, 0.3, window or None, sk).reshape(n, -1)
            for first, count in ((0, n), (123, 150), (200, 1)):
                def fn(qq, out, kc, vc, bt, seq, pos, **kw):
                    t0, nt = tiles_of(first, count)
                    ops.attention_sink_tile(qq, out, H, G, a, b, kc, vc, ps, bt, seq, pos, 0.3, window,
                                            dev(sk) if sk is not None else None, t0, nt)
                picks = list(range(first, first + count))
                got = _run_attention(fn, q, k, v, H, G, a, b, ps, bf, picks)
                close(got, want[picks], 2e-2, f"window {window} loud {loud} from {first}")

            for splits in (1, 2, 5):           # five shares: some of them hold no key at all
                def single(qq, out, kc, vc, bt, seq, pos, **kw):
                    ops.attention_sink_tile(qq, out, H, G, a, b, kc, vc, ps, bt, seq, pos, 0.3, window,
                                            dev(sk) if sk is not None else None, n_splits=splits)
                picks = [0, 1, 36, 37, 63, 64, 65, 199, 200, 201, 332]
                got = _run_attention(single, q, k, v, H, G, a, b, ps, bf, picks)
                close(got, want[picks], 2e-2, f"single tokens in {splits} shares, window {window} loud {loud}")


def _scan_inputs(H, P, N, G, taps, n, rng):
    C = H * P + 2 * G * N
    xin = tt.bf16_values(rng.normal(size=(n, C)))
    w, bias = rng.normal(size=(C, taps)) * 0.6, rng.normal(size=C) * 0.2
    dt_raw = tt.bf16_values(rng.normal(size=(n, H)))
    dt_bias, a_log, d = rng.normal(size=H) * 0.5 - 0.5, rng.normal(size=H) * 0.7 - 1.0, rng.normal(size=H)
    return C, xin, w, bias, dt_raw, dt_bias, a_log, d


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,P,N,G,taps", [(4, 6, 10, 2, 4), (3, 8, 16, 1, 2), (2, 20, 9, 2, 1), (8, 4, 6, 4, 5),
                                          (2, 64, 128, 1, 4), (1, 40, 200, 1, 3)])
def test_convolution_and_scan_over_portions(H, P, N, G, taps, dtype):
    """Two requests in one batch, cut into portions of many sizes (single tokens among them),
    their states in slots that were used before; against the plain convolution and scan of the
    whole sequences. A loud first token shows a state that is lost on the way."""
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(H * P + N)
    lens = (70, 23)
    data = [_scan_inputs(H, P, N, G, taps, n, rng) for n in lens]
    C = data[0][0]
    _, _, w, bias, _, dt_bias, a_log, d = data[0]
    for item in data:
        item[1][0] *= 4.0                                             # a loud first token
    floats = H * N * P + (taps - 1) * C
    state = torch.full((4, floats), 7.0, dtype=torch.float32, device=DEV)   # used before
    slot = [2, 0]
    for s in slot:
        state[s].zero_()
    want = []
    for (_, xin, _, _, dt_raw, _, _, _), n in zip(data, lens):
        xbc = plain.silu(plain.causal_conv(xin, w, bias))
        y = plain.selective_scan(xbc[:, :H * P].reshape(n, H, P), plain.softplus(dt_raw + dt_bias),
                                 np.exp(a_log), xbc[:, H * P:H * P + G * N].reshape(n, G, N),
                                 xbc[:, H * P + G * N:].reshape(n, G, N), d, H // G)
        want.append((xbc, y.reshape(n, H * P)))
    at = [0, 0]
    cuts = [[17, 1, 1, 2, 30, 1, 18], [1, 5, 1, 1, 2, 13]]
    step = 0
    while any(at[r] < lens[r] for r in range(2)):
        live = [r for r in range(2) if at[r] < lens[r] and step < len(cuts[r])]
        sizes = [cuts[r][step] for r in live]
        xin = np.concatenate([data[r][1][at[r]:at[r] + m] for r, m in zip(live, sizes)])
        dtr = np.concatenate([data[r][4][at[r]:at[r] + m] for r, m in zip(live, sizes)])
        T = sum(sizes)
        wide = dev(np.concatenate([np.zeros((T, 3)), xin, dtr], 1), dtype)      # views of a wider row
        q_start = ints(np.cumsum([0] + sizes))
        seq = ints(np.repeat(np.arange(len(live)), sizes))
        slots = ints([slot[r] for r in live])
        xbc = torch.empty((T, C), dtype=torch.float32, device=DEV)
        ops.causal_conv_act(wide[:, 3:3 + C], dev(w), dev(bias), xbc, len(live), seq, q_start, slots,
                            state, H * N * P)
        y = torch.empty((T, H * P), dtype=torch.float32, device=DEV)
        ops.selective_scan(xbc, wide[:, 3 + C:], dev(dt_bias), dev(a_log), dev(d), y, len(live), H, G, N, P,
                           q_start, slots, state, 0)
        o = 0
        for r, m in zip(live, sizes):
            close(xbc[o:o + m], want[r][0][at[r]:at[r] + m], 3e-5, "convolution")
            close(y[o:o + m], want[r][1][at[r]:at[r] + m], 1e-4, "scan")
            o += m
            at[r] += m
        step += 1
    assert float(state[1].min()) == 7.0 and float(state[3].max()) == 7.0     # others' rows untouched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,E,top,ff,T,shared", [(48, 5, 2, 24, 9, True), (40, 1, 1, 32, 3, False),
                                                 (32, 7, 7, 8, 70, False), (192, 10, 3, 80, 150, True),
                                                 (64, 40, 4, 16, 1, False), (36, 3, 2, 20, 11, False)])
def test_routed_experts(d, E, top, ff, T, shared, dtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(d + E)
    x = tt.bf16_values(rng.normal(size=(T, d)))
    W = {"r.router": tt.bf16_values(rng.normal(size=(E, d)) * 0.8), "r.router.b": rng.normal(size=E) * 0.5}
    for e in range(E):
        W[f"r.e{e}.gate"] = tt.bf16_values(rng.normal(size=(ff, d)) / math.sqrt(d))
        W[f"r.e{e}.up"] = tt.bf16_values(rng.normal(size=(ff, d)) / math.sqrt(d))
        W[f"r.e{e}.down"] = tt.bf16_values(rng.normal(size=(d, ff)) / math.sqrt(ff))
    extra = rng.normal(size=(T, d)) if shared else None
    stack = lambda r: dev(np.stack([W[f"r.e{e}.{r}"] for e in range(E)]), dtype)       # noqa: E731
    wide = dev(np.concatenate([x, x], 1), dtype)
    got = ops.moe_feed_forward(wide[:, d:], dev(W["r.router"]), dev(W["r.router.b"]), stack("gate"),
                               stack("up"), stack("down"), top, "silu", dev(extra) if shared else None)
    want = plain.routed(x, W, "r.", {"router": {"experts": E, "top": top}})
    if shared:
        want = want + extra
    close(got, want, TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunked", [False, True])
def test_linear_attention_with_activated_inputs(dtype, chunked):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(3)
    H, a, b, n = 3, 8, 12, 150
    q, k, v = (tt.bf16_values(rng.normal(size=(n, H * w))) for w in (a, a, b))
    decay = [0.5, 0.9, 1.0]
    want = plain.decayed_linear_attention(plain.silu(q).reshape(n, H, a), plain.silu(k).reshape(n, H, a),
                                          plain.silu(v).reshape(n, H, b), decay).reshape(n, -1)
    state = torch.zeros((2, H, a, b), dtype=torch.float32, device=DEV)
    got = torch.empty((n, H * b), dtype=torch.float32, device=DEV)
    at = 0
    for m in (70, 1, 1, 2, 76):
        o = torch.empty((m, H * b), dtype=torch.float32, device=DEV)
        args = (dev(q[at:at + m], dtype), dev(k[at:at + m], dtype), dev(v[at:at + m], dtype), o, 1, H, a, b,
                dev(decay), 1.0, None, 0, ints([0, m]), ints([1]), state)
        if not chunked:
            ops.retention(*args, act=1)
        elif m == 1:
            ops.retention_chunked(*args, act=1)
        else:
            c = ops.retention_chunk_tokens()
            tok0 = list(range(0, m, c))
            ops.retention_chunked(*args, ints(tok0), ints([min(c, m - t) for t in tok0]), ints([0]), act=1)
        got[at:at + m] = o
        at += m
    close(got, want, 2e-4)


# ------------------------------------------------------------------- the engine, end to end
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, page) in tt.CONFIGS.items():
        W = tt.make_weights(cfg, 11)
        d = tt.write_model_dir(str(tmp_path_factory.mktemp("totatar" + name)), cfg, W)
        out[name] = (d, cfg, W, page)
    return out


def spread(d):
    d = d - d.mean()
    return math.sqrt((d * d).mean())


def rows_close(got, cfg, W, requests, dtype):
    """Against the plain logits. float32: to rounding. bfloat16: within three times what
    rounding the activations to bfloat16 does to the plain model's own logits on the same
    requests (the largest over all their positions): a bound that follows the model."""
    want = {rid: plain.forward(cfg, W, toks) for rid, toks in requests.items()}
    allowed = None
    if dtype != "float32":
        allowed = 3.0 * max(spread(row - want[rid][p]) for rid, toks in requests.items()
                            for p, row in enumerate(plain.forward(cfg, W, toks, rnd=tt.bf16_values)))
    for rid, toks in requests.items():
        for p in range(len(toks)):
            err = spread(got[(rid, p)].astype(np.float64) - want[rid][p])
            bound = 1e-4 * want[rid][p].std() if allowed is None else allowed
            assert err <= bound, (rid, p, err, bound)


FAMILIES = {"whole": tiny.trace_whole, "tail": lambda r: tiny.trace_tail(r, 12),
            "portions": tiny.trace_portions,
            "mixed": lambda r: tiny.trace_mixed(r, seed=4, max_live=4, tail=9)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", list(FAMILIES))
@pytest.mark.parametrize("name", ["T1", "T2", "T3", "T4"])
def test_replay_against_plain(models, tmp_path, name, family, dtype):
    d, cfg, W, page = models[name]
    requests = tiny.random_requests(cfg["vocab"], [70, 9, 1, 45, 33, 21], seed=6)
    trace = FAMILIES[family](requests)
    got = tiny.run_trace_program(d, dtype, trace, tmp_path / "out", cfg["vocab"],
                                 extra=["--page-size", str(page), "--max-live", "4"])
    rows_close(got, cfg, W, requests, dtype)


@pytest.mark.parametrize("name", ["T1", "T2"])
def test_float32_cuts_agree_and_pages_and_slots_come_back(models, name):
    """Every cutting gives the same float32 logits to rounding, with NaN in every page nobody
    holds and three state slots for six requests."""
    import tgo_b200
    d, cfg, W, page = models[name]
    requests = tiny.random_requests(cfg["vocab"], [64, 17, 2, 40, 33, 65], seed=7)
    model = tgo_b200.open(d, dtype="float32")
    base = None
    for family in ("whole", "portions", "mixed"):
        trace = tiny.trace_mixed(requests, seed=1, max_live=3, tail=7) if family == "mixed" \
            else FAMILIES[family](requests)
        eng = model.new_engine(page_size=page, max_tokens=tiny.max_tokens_of(trace, page), num_slots=3)
        owners = [dict() for _ in eng.cache.groups]
        got = tiny.run_trace_engine(eng, trace, poison=True, owners=owners)
        rows_close(got, cfg, W, requests, "float32")
        if base is None:
            base = got
        for key, row in got.items():
            assert np.abs(row - base[key]).max() <= 2e-4 * max(1.0, np.abs(base[key]).max()), key
        if family == "mixed":
            assert any(len(ids) > 1 for g in owners for ids in g.values())


@pytest.mark.parametrize("name", ["T1", "T5"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_first_tokens_and_a_long_prompt(models, dtype, name):
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    d, cfg, W, page = models[name]
    model = tgo_b200.open(d, dtype=dtype)
    toks = tiny.random_requests(cfg["vocab"], [150], seed=3)["r0"]
    eng = model.new_engine(page_size=page, max_tokens=192, num_slots=2)
    eng.admit("a")
    got = {}
    for p, t in enumerate(toks):                       # from an empty cache, one by one (graphs)
        got[("a", p)] = eng.step([StepEntry("a", [t], [0])])[0].float().cpu().numpy()
    rows_close(got, cfg, W, {"a": toks}, dtype)
    # 1100 tokens in one step: the many-row products; then a few decoded
    long = tiny.random_requests(cfg["vocab"], [1106], seed=4)["r0"]
    eng = model.new_engine(page_size=page, max_tokens=1152, num_slots=2)
    eng.admit("b")
    want = plain.forward(cfg, W, long)
    picks = [0, 7, 511, 1023, 1024, 1099]
    lg = eng.step([StepEntry("b", long[:1100], picks)]).float().cpu().numpy()
    rows = {("b", p): lg[i] for i, p in enumerate(picks)}
    for p in range(1100, 1106):
        rows[("b", p)] = eng.step([StepEntry("b", [long[p]], [0])])[0].float().cpu().numpy()
    rounded = plain.forward(cfg, W, long, rnd=tt.bf16_values)
    allowed = 3.0 * max(spread(rounded[p] - want[p]) for p in range(len(long)))
    for (rid, p), g in rows.items():
        err = spread(g.astype(np.float64) - want[p])
        assert err <= (2e-4 * want[p].std() if dtype == "float32" else allowed), (p, err)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_equal_portions_replayed_from_a_graph(models, dtype):
    """Portions of 256 tokens of one prompt: from the second on they run as a captured graph
    (the routing, the scan's state and the convolution's kept inputs advance with every replay)."""
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    d, cfg, W, page = models["T1"]
    model = tgo_b200.open(d, dtype=dtype)
    toks = tiny.random_requests(cfg["vocab"], [256 * 4 + 5], seed=12)["r0"]
    eng = model.new_engine(page_size=page, max_tokens=1088, num_slots=2)
    eng.admit("p")
    got = {}
    for o in range(0, 1024, 256):
        lg = eng.step([StepEntry("p", toks[o:o + 256], [0, 255])]).float().cpu().numpy()
        got[("p", o)], got[("p", o + 255)] = lg[0], lg[1]
    assert len(eng._portion_graphs) >= 1
    for p in range(1024, len(toks)):
        got[("p", p)] = eng.step([StepEntry("p", [toks[p]], [0])])[0].float().cpu().numpy()
    want = plain.forward(cfg, W, toks)
    rounded = plain.forward(cfg, W, toks, rnd=tt.bf16_values)
    allowed = 3.0 * max(spread(rounded[p] - want[p]) for p in range(len(toks)))
    for (_, p), g in got.items():
        err = spread(g.astype(np.float64) - want[p])
        assert err <= (2e-4 * want[p].std() if dtype == "float32" else allowed), (p, err)


def test_greedy_generation_through_entry_point_scheduler_and_command_line(models):
    import tgo_b200
    from tgo_b200.sampling.policy import Policy
    d, cfg, W, page = models["T1"]
    prompts = list(tiny.random_requests(cfg["vocab"], [5, 17, 33, 1, 12], seed=8).values())
    want = [plain.greedy(cfg, W, p, 8) for p in prompts]
    assert len({t for o in want for t in o}) > 4
    model = tgo_b200.open(d, dtype="float32")
    assert model.generate(prompts, Policy(max_tokens=8), slots=3, chunk=16, page_size=page) == want
    # so few pages and slots that requests wait for others' to come back
    assert model.generate(prompts, Policy(max_tokens=8), slots=2, chunk=7, pool_tokens=96,
                          page_size=page) == want
    got = tgo_b200.open(d, dtype="bfloat16").generate(prompts, Policy(max_tokens=8), slots=4,
                                                      page_size=page)
    for p, o in zip(prompts, got):                       # bfloat16: each pick is near the best
        seq = list(p)
        for tok in o:
            z = plain.forward(cfg, W, seq)[-1]
            assert z.max() - z[tok] <= 0.25 * z.std()
            seq.append(tok)
    tgo = os.path.join(tiny.ROOT, "bin", "tgo")
    r = subprocess.run([sys.executable, tgo, "run", "--prompt", " ".join(map(str, prompts[1])),
                        "--max-tokens", "8", "--precision", "f32", "--context", "64", d],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert [int(t) for t in r.stdout.split()] == want[1]
    r = subprocess.run([sys.executable, tgo, "info", d], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "Totatar" in r.stdout
