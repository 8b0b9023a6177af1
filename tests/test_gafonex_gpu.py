"""Gafonex on the GPU: every new kernel alone against the plain statement of its mechanism,
then the engine against the plain model: whole prompts, decoding, portions, mixed batches with
pages and state slots that come back, far keys and page borders, first tokens, long decoding,
long prompts through the many-row products, and greedy generation through the library's entry
point, the scheduler and the command line."""
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import gafonex_tiny as gt
import plain_gafonex as plain
import tiny

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(x, dtype=torch.float32):
    return torch.from_numpy(np.asarray(x, dtype=np.float32)).to(device=DEV, dtype=dtype)


def close(got, want, tol, what=""):
    got = got.detach().float().cpu().numpy().astype(np.float64)
    err = np.abs(got - want).max()
    assert err <= tol * max(1.0, np.abs(want).max()), f"{what}: {err}"


TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


# ------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("y_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,groups", [(48, 3), (40, 1), (2048, 2), (6, 6)])
def test_group_norm_scale_add(d, groups, y_dtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(d)
    h0, y = rng.normal(size=(5, d)), gt.bf16_values(rng.normal(size=(5, d)) * 3)
    gain, scale = rng.normal(size=d), rng.normal(size=d)
    h, act = dev(h0), torch.empty((5, d), dtype=torch.bfloat16, device=DEV)
    ops.group_norm_scale_add(h, dev(y, y_dtype), dev(gain), dev(scale), 1e-5, groups, act)
    want = h0 + plain.group_norm(y, gain, 1e-5, groups) * scale
    close(h, want, 2e-5, "stream")
    close(act, want, 1e-2, "copy")
    h = dev(h0)
    ops.group_norm_scale_add(h, dev(y, y_dtype), dev(gain), None, 1e-5, groups, None)
    close(h, h0 + plain.group_norm(y, gain, 1e-5, groups), 2e-5, "no scale")
    out = torch.empty((2, d), dtype=torch.float32, device=DEV)
    ops.group_norm_rows(dev(h0), torch.tensor([4, 1], dtype=torch.int32, device=DEV), dev(gain),
                        1e-5, groups, out)
    close(out, plain.group_norm(h0[[4, 1]], gain, 1e-5, groups), 2e-5, "rows")


def test_gate_activations_soft_cap_and_cast():
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(0)
    g, u = rng.normal(size=(3, 24)) * 3, rng.normal(size=(3, 24))
    for act, fn in (("relu", lambda z: np.maximum(z, 0)), ("gelu_tanh", plain.gelu_tanh),
                    ("silu", lambda z: z / (1 + np.exp(-z)))):
        out = torch.empty((3, 24), dtype=torch.float32, device=DEV)
        ops.gated_act(dev(np.concatenate([g, u], 1)), out, False, act)
        close(out, fn(g) * u, 2e-6, act)
        inter = np.stack([g.reshape(3, 3, 8), u.reshape(3, 3, 8)], 2).reshape(3, 48)
        ops.gated_act(dev(inter), out, True, act)
        close(out, fn(g) * u, 2e-6, act + " interleaved")
        for wdt in (torch.bfloat16,):                 # the 16-byte form of bfloat16 rows
            gb, ub = gt.bf16_values(g), gt.bf16_values(u)
            outb = torch.empty((3, 24), dtype=wdt, device=DEV)
            ops.gated_act(dev(np.concatenate([gb, ub], 1), wdt), outb, False, act)
            close(outb, fn(gb) * ub, 1e-2, act + " bfloat16")
            interb = np.stack([gb.reshape(3, 3, 8), ub.reshape(3, 3, 8)], 2).reshape(3, 48)
            ops.gated_act(dev(interb, wdt), outb, True, act)
            close(outb, fn(gb) * ub, 1e-2, act + " bfloat16 interleaved")
    z = rng.normal(size=(4, 50)) * 40
    t = dev(z)
    ops.softcap(t, 12.0)
    close(t, plain.soft_cap(z, 12.0), 2e-6, "soft cap")
    b = torch.empty((4, 50), dtype=torch.bfloat16, device=DEV)
    ops.cast_rows(dev(z), b)
    assert torch.equal(b, dev(z).to(torch.bfloat16))


def test_stretched_rotation_table():
    from tgo_b200.config.spec import PositionSpec
    from tgo_b200.parts.base import StepContext
    from tgo_b200.parts.position import RopeStretched
    rot = {"dims": 8, "base": 500.0, "scaling": gt.STRETCH}
    part = RopeStretched(PositionSpec("rope_stretched", 8, 500.0, (4.0, 16, 4.0, 1.0)), 12, DEV)
    pos = torch.tensor([0, 1, 17, 300], dtype=torch.int32, device=DEV)
    ctx = StepContext(4, 1, pos, pos, pos, pos, pos, pos, pos, torch.float32)
    table, dims = part.rotary(ctx)
    f, mag = plain.rotary_frequencies(rot)
    want = np.concatenate([np.cos(np.outer([0, 1, 17, 300], f)), np.sin(np.outer([0, 1, 17, 300], f))], 1) * mag
    assert dims == 8
    close(table, want, 1e-6, "table")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_values_normed_blended_and_stored(dtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(1)
    T, G, b, ps = 7, 3, 20, 4
    v = gt.bf16_values(rng.normal(size=(T, G * b)) * 2)
    slots = [9, 10, 11, 4, -1, 5, 6]
    cache = torch.zeros((5, G, ps, b), dtype=dtype, device=DEV)
    shared = torch.zeros((T, G * b), dtype=torch.float32, device=DEV)
    wide = torch.zeros((T, G * b + 8), dtype=dtype, device=DEV)      # rows with a stride
    wide[:, 8:] = dev(v, dtype)
    sl = torch.tensor(slots, dtype=torch.int32, device=DEV)
    ops.value_norm_share_cache(wide[:, 8:], G, b, True, 1e-5, None, shared, 1, sl, cache, ps)
    normed = plain.unit_rms(v.reshape(T, G, b), 1e-5)
    close(shared, normed.reshape(T, -1), 2e-5, "source")
    v2 = gt.bf16_values(rng.normal(size=(T, G * b)))
    lam = torch.tensor([0.3], dtype=torch.float32, device=DEV)
    ops.value_norm_share_cache(dev(v2, dtype), G, b, True, 1e-5, lam, shared, 2, sl, cache, ps)
    mixed = 0.7 * plain.unit_rms(v2.reshape(T, G, b), 1e-5) + np.float32(0.3) * normed
    for t, s in enumerate(slots):
        if s >= 0:
            close(cache[s // ps, :, s % ps, :], mixed[t], TOL[dtype], f"slot {s}")
    assert float(cache[0].abs().sum()) == 0 and float(cache[3].abs().sum()) == 0   # nothing strays


def _paged(rows, page_size, pages_total, table, dtype):
    """rows [n, G, w] -> plane [pages_total, G, page_size, w] through `table` (page of block i)."""
    n, G, w = rows.shape
    plane = torch.full((pages_total, G, page_size, w), float("nan"), dtype=dtype, device=DEV)
    t = dev(rows, dtype)
    for j in range(n):
        plane[table[j // page_size], :, j % page_size, :] = t[j]
    return plane


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,a,b,ps", [(4, 2, 12, 20, 8), (9, 9, 20, 40, 16), (3, 1, 48, 8, 4),
                                        (16, 4, 64, 64, 16)])
def test_mixed_head_attention_kernel(H, G, a, b, ps, dtype):
    """Decoded tokens and prompt tokens of two requests whose pages interleave; one key is
    made to stand out (far back, on either side of a page border, the newest) so that a lost
    or misplaced key shows."""
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(H * 100 + a)
    n0, n1 = 5 * ps + 3, 2 * ps
    table = np.zeros((2, 6), dtype=np.int32)
    table[0] = [2, 4, 6, 8, 10, 12]
    table[1, :2] = [3, 1]
    mix = np.eye(H) * 0.6 + 0.4 * rng.normal(size=(H, H))
    for star in (0, ps - 1, ps, 3 * ps + 1, n0 - 1):
        k0 = gt.bf16_values(rng.normal(size=(n0, G, a)))
        v0 = gt.bf16_values(rng.normal(size=(n0, G, b)))
        k1 = gt.bf16_values(rng.normal(size=(n1, G, a)))
        v1 = gt.bf16_values(rng.normal(size=(n1, G, b)))
        # queries: the last 3 positions of request 0 and positions 0, ps-1, ps of request 1
        pos = [n0 - 3, n0 - 2, n0 - 1, 0, ps - 1, ps]
        seq = [0, 0, 0, 1, 1, 1]
        q = gt.bf16_values(rng.normal(size=(6, H, a)))
        k0[star] = gt.bf16_values(4.0 * q[2, ::H // G])       # the star key answers query 2
        kc = _paged(k0, ps, 13, table[0], dtype)
        vc = _paged(v0, ps, 13, table[0], dtype)
        kc1, vc1 = _paged(k1, ps, 13, table[1], dtype), _paged(v1, ps, 13, table[1], dtype)
        for pg in table[1, :2]:
            kc[pg], vc[pg] = kc1[pg], vc1[pg]
        out = torch.empty((6, H * b), dtype=dtype, device=DEV)
        scale = 0.9 / math.sqrt(a)
        ops.attention_mixed(dev(q.reshape(6, -1), dtype), out, H, G, a, b, kc, vc, ps,
                            torch.from_numpy(table).to(DEV), torch.tensor(seq, dtype=torch.int32, device=DEV),
                            torch.tensor(pos, dtype=torch.int32, device=DEV), dev(mix), scale, 0)
        for i, (p, s) in enumerate(zip(pos, seq)):
            kk, vv = (k0, v0) if s == 0 else (k1, v1)
            qq = np.zeros((p + 1, H, a))
            qq[p] = q[i]
            w = plain.mix_heads(plain.attention_weights(qq, kk[:p + 1], scale), mix)
            want = np.stack([w[h, p] @ vv[:p + 1, h // (H // G)] for h in range(H)]).reshape(-1)
            close(out[i], want, TOL[dtype] * 2, f"star {star} query {i}")
        # without the table of mixes: plain grouped attention
        ops.attention_mixed(dev(q.reshape(6, -1), dtype), out, H, G, a, b, kc, vc, ps,
                            torch.from_numpy(table).to(DEV), torch.tensor(seq, dtype=torch.int32, device=DEV),
                            torch.tensor(pos, dtype=torch.int32, device=DEV), None, scale, 0)
        p = pos[2]
        qq = np.zeros((p + 1, H, a))
        qq[p] = q[2]
        w = plain.attention_weights(qq, k0[:p + 1], scale)
        want = np.stack([w[h, p] @ v0[:p + 1, h // (H // G)] for h in range(H)]).reshape(-1)
        close(out[2], want, TOL[dtype] * 2, f"unmixed star {star}")


@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("H,G,a,b,ps", [(4, 2, 16, 24, 8), (9, 9, 24, 40, 16), (16, 1, 64, 128, 16),
                                        (8, 2, 128, 64, 32), (3, 3, 16, 16, 8), (15, 5, 8, 32, 4)])
def test_mixed_head_attention_decode_kernels(H, G, a, b, ps, splits):
    """Single tokens of four requests (1, 33, 64 and 200 keys; one padded row) through the
    split-key kernels; the loud key at the start, at range and page borders, and the newest."""
    from tgo_b200.kernels import ops
    assert ops.attention_mixed_decode_supports(H, G, a, b, 0)
    rng = np.random.default_rng(H * 7 + a)
    lens = [1, 33, 64, 200]
    nb = -(-max(lens) // ps)
    table = np.zeros((4, nb), dtype=np.int32)
    pages = list(rng.permutation(np.arange(1, 4 * nb + 1)))
    for b_ in range(4):
        for i in range(-(-lens[b_] // ps)):
            table[b_, i] = pages.pop()
    mix = np.eye(H) * 0.6 + 0.4 * rng.normal(size=(H, H))
    scale = 0.8 / math.sqrt(a)
    for star in (0, 31, 32, 63, 64, 95, 96, 199):
        ks = [gt.bf16_values(rng.normal(size=(n, G, a))) for n in lens]
        vs = [gt.bf16_values(rng.normal(size=(n, G, b))) for n in lens]
        qs = gt.bf16_values(rng.normal(size=(4, H, a)))
        ks[3][star] = gt.bf16_values(3.0 * qs[3, ::H // G])
        kc = torch.full((4 * nb + 1, G, ps, a), 1e30, dtype=torch.bfloat16, device=DEV)
        vc = torch.full((4 * nb + 1, G, ps, b), 1e30, dtype=torch.bfloat16, device=DEV)
        for b_ in range(4):
            kk, vv = _paged(ks[b_], ps, 4 * nb + 1, table[b_], torch.bfloat16), \
                _paged(vs[b_], ps, 4 * nb + 1, table[b_], torch.bfloat16)
            for j in range(lens[b_]):
                pg = table[b_, j // ps]
                kc[pg, :, j % ps], vc[pg, :, j % ps] = kk[pg, :, j % ps], vv[pg, :, j % ps]
        q = np.concatenate([qs.reshape(4, -1), np.zeros((1, H * a))])
        pos = np.array([n - 1 for n in lens] + [-1], dtype=np.int32)
        seq = np.array([0, 1, 2, 3, 0], dtype=np.int32)
        out = torch.full((5, H * b), 7.0, dtype=torch.bfloat16, device=DEV)
        ops.attention_mixed_decode(dev(q, torch.bfloat16), out, H, G, a, b, kc, vc, ps,
                                   torch.from_numpy(table).to(DEV), torch.from_numpy(seq).to(DEV),
                                   torch.from_numpy(pos).to(DEV), dev(mix), scale, splits, max(lens))
        for b_, n in enumerate(lens):
            qq = np.zeros((n, H, a))
            qq[-1] = qs[b_]
            w = plain.mix_heads(plain.attention_weights(qq, ks[b_], scale), mix)
            want = np.stack([w[h, n - 1] @ vs[b_][:, h // (H // G)] for h in range(H)])
            close(out[b_], want.reshape(-1), 2e-2, f"star {star} request {b_}")
        assert float(out[4].abs().max()) == 0                # the padded row: zeros


@pytest.mark.parametrize("H,G,a,b,ps", [(4, 2, 16, 24, 8), (9, 3, 32, 40, 16), (16, 4, 64, 128, 16),
                                        (8, 8, 128, 64, 32), (2, 1, 48, 8, 4)])
def test_mixed_head_attention_tile_kernel(H, G, a, b, ps):
    """The tensor-core kernel of prompt portions: two requests in one launch, one from an
    empty cache (tiles of 16, 16 and 5 tokens), one continued from position 70 by 19 tokens
    and, in the same launch, a third by a single token; a loud key at the start, at either
    side of a block of 32 and of a page, and the newest."""
    from tgo_b200.kernels import ops
    assert ops.attention_mixed_tile_supports(H, G, a, b, 0)
    rng = np.random.default_rng(H + a)
    lens = [37, 89, 41]                     # keys each request holds after the step
    first = [0, 70, 40]                     # first position each brings
    nb = -(-max(lens) // ps)
    table = np.zeros((3, nb), dtype=np.int32)
    pages = list(rng.permutation(np.arange(1, 3 * nb + 1)))
    for b_ in range(3):
        for i in range(-(-lens[b_] // ps)):
            table[b_, i] = pages.pop()
    mix = np.eye(H) * 0.6 + 0.4 * rng.normal(size=(H, H))
    scale = 0.8 / math.sqrt(a)
    for star in (0, 31, 32, ps - 1, ps, 69, 88):
        ks = [gt.bf16_values(rng.normal(size=(n, G, a))) for n in lens]
        vs = [gt.bf16_values(rng.normal(size=(n, G, b))) for n in lens]
        qs = [gt.bf16_values(rng.normal(size=(n - f, H, a))) for n, f in zip(lens, first)]
        ks[1][star] = gt.bf16_values(3.0 * qs[1][-1, ::H // G])
        kc = torch.full((3 * nb + 1, G, ps, a), float("nan"), dtype=torch.bfloat16, device=DEV)
        vc = torch.full((3 * nb + 1, G, ps, b), float("nan"), dtype=torch.bfloat16, device=DEV)
        for b_ in range(3):
            kk, vv = _paged(ks[b_], ps, 3 * nb + 1, table[b_], torch.bfloat16), \
                _paged(vs[b_], ps, 3 * nb + 1, table[b_], torch.bfloat16)
            for pg in table[b_, :-(-lens[b_] // ps)]:
                kc[pg], vc[pg] = kk[pg], vv[pg]
        kc, vc = torch.nan_to_num(kc, nan=1e30), torch.nan_to_num(vc, nan=1e30)   # stale rows: loud
        q = np.concatenate([x.reshape(x.shape[0], -1) for x in qs])
        pos = np.concatenate([np.arange(f, n) for n, f in zip(lens, first)]).astype(np.int32)
        seq = np.concatenate([[i] * (n - f) for i, (n, f) in enumerate(zip(lens, first))]).astype(np.int32)
        tok0, ntok, base = [], [], 0
        for n, f in zip(lens, first):
            for o in range(0, n - f, 16):
                tok0.append(base + o)
                ntok.append(min(16, n - f - o))
            base += n - f
        wide = torch.zeros((len(pos), H * a + 3), dtype=torch.bfloat16, device=DEV)   # odd stride
        wide[:, :H * a] = dev(q, torch.bfloat16)
        out = torch.empty((len(pos), H * b), dtype=torch.bfloat16, device=DEV)
        ops.attention_mixed_tile(wide[:, :H * a], out, H, G, a, b, kc, vc, ps,
                                 torch.from_numpy(table).to(DEV), torch.from_numpy(seq).to(DEV),
                                 torch.from_numpy(pos).to(DEV), dev(mix), scale,
                                 torch.tensor(tok0, dtype=torch.int32, device=DEV),
                                 torch.tensor(ntok, dtype=torch.int32, device=DEV))
        at = 0
        for b_, (n, f) in enumerate(zip(lens, first)):
            qq = np.zeros((n, H, a))
            qq[f:] = qs[b_]
            w = plain.mix_heads(plain.attention_weights(qq, ks[b_], scale), mix)
            for p in range(f, n):
                want = np.stack([w[h, p, :p + 1] @ vs[b_][:p + 1, h // (H // G)] for h in range(H)])
                close(out[at], want.reshape(-1), 3e-2, f"star {star} request {b_} position {p}")
                at += 1


@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,a,b,rot", [(3, 8, 12, 4), (1, 24, 24, 24), (2, 16, 4, 0), (4, 64, 80, 32),
                                       (2, 128, 200, 128)])
def test_retention_kernel(H, a, b, rot, dtype, chunked):
    """Both forms (a block per request and head in order; in parallel over chunks with a scan,
    and its single-token kernel). Requests of 1, 2, 31, 32, 33, 63, 64, 65 and 150 tokens in
    one launch (a chunk's edge on either
    side), then each continued token by token and by a portion from the state the first launch
    left; decays 0, 1 and between; a loud first token that only a decay of 1 keeps for ever."""
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(a)
    lens = [1, 2, 31, 32, 33, 63, 64, 65, 150]
    more = 5
    decay = np.array(([0.0, 1.0, 0.9, 0.999] * 2)[:H])
    if H == 1:
        decay = np.array([1.0])
    total = [n + more for n in lens]
    q = [gt.bf16_values(rng.normal(size=(n, H, a))) for n in total]
    k = [gt.bf16_values(rng.normal(size=(n, H, a))) for n in total]
    v = [gt.bf16_values(rng.normal(size=(n, H, b))) for n in total]
    for x in v:
        x[0] *= 50.0
    x = [gt.bf16_values(x_) for x_ in v]
    v = x
    rotd = {"dims": rot, "base": 30.0} if rot else None
    want = [plain.retention_outputs(plain.rotate(qq, range(len(qq)), rotd),
                                    plain.rotate(kk, range(len(kk)), rotd) * a ** -0.5, vv, decay)
            for qq, kk, vv in zip(q, k, v)]
    state = torch.full((len(lens) + 2, H, a, b), 7.0, dtype=torch.float32, device=DEV)
    slots = [5, 0, 3, 6, 1, 2, 10, 8, 9]
    state[slots] = 0
    dec = dev(decay)
    if rot:
        f, _ = plain.rotary_frequencies(rotd)

    def launch(pieces):
        """pieces: per request (first position, count)."""
        T = sum(c for _, c in pieces)
        pos = np.concatenate([np.arange(s, s + c) for s, c in pieces])
        cat = lambda arrs, w: dev(np.concatenate([x_[s:s + c].reshape(c, -1) for x_, (s, c) in   # noqa: E731
                                                  zip(arrs, pieces)]), dtype)
        table = None
        if rot:
            ang = np.outer(pos, f)
            table = dev(np.concatenate([np.cos(ang), np.sin(ang)], 1))
        out = torch.empty((T, H * b), dtype=torch.float32, device=DEV)
        starts = np.concatenate([[0], np.cumsum([c for _, c in pieces])]).astype(np.int32)
        args = (cat(q, a), cat(k, a), cat(v, b), out, len(pieces), H, a, b, dec, a ** -0.5, table, rot,
                torch.from_numpy(starts).to(DEV), torch.tensor(slots, dtype=torch.int32, device=DEV), state)
        if not chunked:
            ops.retention(*args)
        elif all(c == 1 for _, c in pieces):
            ops.retention_chunked(*args)
        else:
            C = ops.retention_chunk_tokens()
            tok0, ntok, first = [], [], []
            for i, (_, c) in enumerate(pieces):
                first.append(len(tok0))
                for o in range(0, c, C):
                    tok0.append(int(starts[i]) + o)
                    ntok.append(min(C, c - o))
            ops.retention_chunked(*args, *(torch.tensor(x, dtype=torch.int32, device=DEV)
                                           for x in (tok0, ntok, first)))
        return out, starts
    tol = 3e-5 if dtype == torch.float32 else 3e-5      # the inputs are bfloat16-exact either way
    out, starts = launch([(0, n) for n in lens])
    for i, n in enumerate(lens):
        close(out[starts[i]:starts[i + 1]], want[i][:n].reshape(n, -1), tol, f"prompt {n}")
    for step in range(2):                                # two single tokens each
        out, starts = launch([(n + step, 1) for n in lens])
        for i, n in enumerate(lens):
            close(out[i], want[i][n + step].reshape(-1), tol, f"decode {n}+{step}")
    out, starts = launch([(n + 2, more - 2) for n in lens])    # then a portion of three
    for i, n in enumerate(lens):
        close(out[starts[i]:starts[i + 1]], want[i][n + 2:].reshape(more - 2, -1), tol, f"portion {n}")
    assert float((state[[4, 7]] - 7.0).abs().max()) == 0       # other slots untouched
    # the state the launches left is the plain recurrence's, whichever form made it
    for i, n in enumerate(lens):
        kk = plain.rotate(k[i], range(n + more), rotd) * a ** -0.5
        S = np.zeros((H, a, b))
        for t_ in range(n + more):
            S = decay[:, None, None] * S + kk[t_][:, :, None] * v[i][t_][:, None, :]
        close(state[slots[i]], S, tol, f"state {n}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_and_gate(dtype):
    from tgo_b200.kernels import ops
    rng = np.random.default_rng(2)
    T, H, b = 5, 3, 12
    o, g = rng.normal(size=(T, H * b)) * 10, gt.bf16_values(rng.normal(size=(T, H * b)))
    wide = torch.zeros((T, H * b + 6), dtype=dtype, device=DEV)
    wide[:, 6:] = dev(g, dtype)
    out = torch.empty((T, H * b), dtype=dtype, device=DEV)
    ops.head_norm_gate(dev(o), wide[:, 6:], out, H, b, 1e-5)
    want = plain.unit_rms(np.float32(o).astype(np.float64).reshape(T, H, b), 1e-5).reshape(T, -1) * \
        (g / (1 + np.exp(-g)))
    close(out, want, TOL[dtype], "gated")


# ------------------------------------------------------------------- the engine as a whole
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, page) in gt.CONFIGS.items():
        W = gt.make_weights(cfg, 11)
        d = gt.write_model_dir(str(tmp_path_factory.mktemp("gafonex" + name)), cfg, W)
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
                            for p, row in enumerate(plain.forward(cfg, W, toks, rnd=gt.bf16_values)))
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
@pytest.mark.parametrize("name", ["G1", "G2", "G3"])
def test_replay_against_plain(models, tmp_path, name, family, dtype):
    d, cfg, W, page = models[name]
    requests = tiny.random_requests(cfg["vocab"], [70, 9, 1, 45, 33, 21], seed=6)
    trace = FAMILIES[family](requests)
    got = tiny.run_trace_program(d, dtype, trace, tmp_path / "out", cfg["vocab"],
                                 extra=["--page-size", str(page), "--max-live", "4"])
    rows_close(got, cfg, W, requests, dtype)


@pytest.mark.parametrize("name", ["G1", "G2"])
def test_float32_cuts_agree_and_pages_and_slots_come_back(models, name):
    """Every cutting gives the same float32 logits to rounding of the retention's chunks, with
    NaN in every page nobody holds and three state slots for six requests."""
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_first_tokens_and_a_long_prompt(models, dtype):
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    d, cfg, W, page = models["G1"]
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
    rounded = plain.forward(cfg, W, long, rnd=gt.bf16_values)
    allowed = 3.0 * max(spread(rounded[p] - want[p]) for p in range(len(long)))
    for (rid, p), g in rows.items():
        err = spread(g.astype(np.float64) - want[p])
        assert err <= (2e-4 * want[p].std() if dtype == "float32" else allowed), (p, err)
    eng.check_kernels()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_equal_portions_replayed_from_a_graph(models, dtype):
    """Portions of 256 tokens of one prompt: from the second on they run as a captured graph
    (chunk and tile lists made before the capture, the state advanced by every replay)."""
    import tgo_b200
    from tgo_b200.engine.step import StepEntry
    d, cfg, W, page = models["G1"]
    model = tgo_b200.open(d, dtype=dtype)
    toks = tiny.random_requests(cfg["vocab"], [256 * 4 + 5], seed=12)["r0"]
    eng = model.new_engine(page_size=page, max_tokens=1088, num_slots=2)
    eng.admit("p")
    got = {}
    for o in range(0, 1024, 256):
        lg = eng.step([StepEntry("p", toks[o:o + 256], [0, 255])]).float().cpu().numpy()
        got[("p", o)], got[("p", o + 255)] = lg[0], lg[1]
    assert len(eng._portion_graphs) >= 1           # a graph per block-table width the prompt reaches
    for p in range(1024, len(toks)):
        got[("p", p)] = eng.step([StepEntry("p", [toks[p]], [0])])[0].float().cpu().numpy()
    want = plain.forward(cfg, W, toks)
    rounded = plain.forward(cfg, W, toks, rnd=gt.bf16_values)
    allowed = 3.0 * max(spread(rounded[p] - want[p]) for p in range(len(toks)))
    for (_, p), g in got.items():
        err = spread(g.astype(np.float64) - want[p])
        assert err <= (2e-4 * want[p].std() if dtype == "float32" else allowed), (p, err)


def test_greedy_generation_through_entry_point_scheduler_and_command_line(models):
    import tgo_b200
    from tgo_b200.sampling.policy import Policy
    d, cfg, W, page = models["G1"]
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
    assert r.returncode == 0 and "Gafonex" in r.stdout
