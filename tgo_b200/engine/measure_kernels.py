"""Kernel by kernel: the kernels of the layers that norm their sublayers' outputs, mix the
heads' attention weights and carry a retention state, each timed alone beside the like kernel
of the plain pre-norm attention layer at equal sizes, with what each reaches of its roofline.

Timing: CUDA events around the replay of a CUDA graph that holds one call (one to three
launches), an L2 flush before each, the mean of `repeats` after three warm-up calls. Denominators: the
measured copy bandwidth and library bfloat16 product of this pool for memory- and tensor-bound
kernels; for the float32 recurrence, which no tensor-core mode computes in true 32 bits, the
float32 FMA rate of the device (multiprocessors x 128 lanes x 2 x the SM clock seen).
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

from ..kernels import ops
from ..parts.attention import splits_for, step_tiles
from ..parts.attention_mixed import decode_ranges
from ..parts.base import StepContext
from ..parts.retention import step_chunks
from .measure import L2Flusher, load_peaks


def _timed(fn, flush, repeats: int = 5) -> float:
    """Mean milliseconds of fn() on the device, cold L2: fn is captured into a CUDA graph after
    three plain calls and the replays are timed, so that the host's share of a call that makes
    scratch tensors and launches two or three kernels does not count."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    graph.replay()
    times = []
    for _ in range(repeats):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return sum(times) / len(times)


def _paged(requests: int, length: int, heads: int, width: int, page: int, dev):
    """A cache plane with `requests` requests of `length` keys, and its block tables."""
    per = -(-length // page)
    plane = torch.randn((requests * per + 1, heads, page, width), device=dev).to(torch.bfloat16)
    table = (torch.arange(requests * per, dtype=torch.int32, device=dev) + 1).view(requests, per)
    return plane, table.contiguous()


def _fma_tflops(dev) -> float:
    props = torch.cuda.get_device_properties(dev)
    mhz = getattr(props, "clock_rate", 1_965_000) / 1e3
    return props.multi_processor_count * 128 * 2 * mhz * 1e6 / 1e12


def measure_kernels(width: int, heads: int, kv_heads: int, key_dim: int, value_dim: int,
                    ret_heads: int, ret_key: int, ret_value: int, inter: int,
                    prompt: int = 2048, batch: int = 64, context: int = 1024,
                    page: int = 16, device="cuda:0") -> List[Dict[str, object]]:
    dev = torch.device(device)
    peaks = load_peaks()
    hbm, tc, fma = peaks["hbm_gbs"], peaks["bf16_tflops"], _fma_tflops(dev)
    flush = L2Flusher(dev)
    out: List[Dict[str, object]] = []
    bf = torch.bfloat16

    def row(name, ms, like, like_ms, bound, work, like_work=None):
        """work: bytes (bound 'hbm') or floating-point operations (bound 'tensor', 'fma')."""
        peak = {"hbm": hbm * 1e9, "tensor": tc * 1e12, "fma": fma * 1e12}[bound]
        rec = {"kernel": name, "us": round(ms * 1e3, 1), "bound": bound,
               "frac": round(work / (ms * 1e-3) / peak, 3)}
        if like:
            rec.update(like=like, like_us=round(like_ms * 1e3, 1),
                       like_frac=round((like_work or work) / (like_ms * 1e-3) / peak, 3))
        out.append(rec)

    def context_of(n_req, extent, first):
        T = n_req * extent
        pos = (torch.arange(extent, dtype=torch.int32, device=dev) + first).repeat(n_req)
        seq = torch.arange(n_req, dtype=torch.int32, device=dev).repeat_interleave(extent)
        qs = torch.arange(n_req + 1, dtype=torch.int32, device=dev) * extent
        z = torch.zeros(n_req, dtype=torch.int32, device=dev)
        return StepContext(T, n_req, pos, pos, seq, qs, z, torch.arange(n_req, dtype=torch.int32, device=dev),
                           z, bf, extents=[extent] * n_req, first_positions=[first] * n_req,
                           max_extent=extent, max_context=first + extent, decode_only=extent == 1)

    # ---- attention over a prompt: the mixed-head tile kernel beside the plain one
    H, G, dk, dv = heads, kv_heads, key_dim, value_dim
    mix = torch.eye(H, device=dev) * 0.7 + 0.3 * torch.randn(H, H, device=dev)
    scale = 1.0 / math.sqrt(dk)
    kc, table = _paged(1, prompt, G, dk, page, dev)
    vc, _ = _paged(1, prompt, G, dv, page, dev)
    ctx = context_of(1, prompt, 0)
    q = torch.randn((prompt, H * dk), device=dev).to(bf)
    o = torch.empty((prompt, H * dv), dtype=bf, device=dev)
    keys = prompt * (prompt + 1) / 2
    flops = 2.0 * H * (dk + dv) * keys
    tok0, ntok = step_tiles(ctx, 16)
    ms = _timed(lambda: ops.attention_mixed_tile(q, o, H, G, dk, dv, kc, vc, page, table, ctx.seq_ids,
                                                 ctx.positions, mix, scale, tok0, ntok), flush)
    like, like_ms, like_flops = None, 0.0, 4.0 * H * dk * keys
    vk, _ = _paged(1, prompt, G, dk, page, dev)
    o2 = torch.empty((prompt, H * dk), dtype=bf, device=dev)
    group = H // G
    if dk == 128 and ops.attention_tc_supports(dk, group, page):
        t0, n0 = step_tiles(ctx, 128 // group)
        like = "attention_tc_prefill"
        like_ms = _timed(lambda: ops.attention_tc_prefill(q, o2, H, G, dk, kc, vk, page, table, ctx.positions,
                                                          ctx.seq_ids, t0, n0, scale, 0), flush)
    elif ops.flash_supports(dk, group):
        t0, n0 = step_tiles(ctx, ops.flash_tile_rows() // group)
        like = "attention_flash (tiles)"
        like_ms = _timed(lambda: ops.attention_flash(q, o2, H, G, dk, kc, vk, page, table, ctx.positions,
                                                     ctx.seq_ids, t0, n0, scale, 0), flush)
    row(f"attention_mixed_tile, {prompt} tokens", ms, like, like_ms, "tensor", flops, like_flops)

    # ---- attention of a decode step
    kc, table = _paged(batch, context, G, dk, page, dev)
    vc, _ = _paged(batch, context, G, dv, page, dev)
    vk, _ = _paged(batch, context, G, dk, page, dev)
    ctx = context_of(batch, 1, context - 1)
    q = torch.randn((batch, H * dk), device=dev).to(bf)
    o = torch.empty((batch, H * dv), dtype=bf, device=dev)
    o2 = torch.empty((batch, H * dk), dtype=bf, device=dev)
    ranges = decode_ranges(batch, context, ops.num_sms(dev))
    ms = _timed(lambda: ops.attention_mixed_decode(q, o, H, G, dk, dv, kc, vc, page, table, ctx.seq_ids,
                                                   ctx.positions, mix, scale, ranges, context), flush)
    like, like_ms = None, 0.0
    if ops.flash_supports(dk, group):
        like = "attention_flash (decode)"
        n_splits = splits_for(batch * G, context, 0, ops.num_sms(dev))
        like_ms = _timed(lambda: ops.attention_flash(q, o2, H, G, dk, kc, vk, page, table, ctx.positions,
                                                     ctx.seq_ids, None, None, scale, 0, n_splits=n_splits), flush)
    row(f"attention_mixed_decode, batch {batch} x {context} keys", ms, like, like_ms, "hbm",
        2.0 * batch * context * G * (dk + dv), 2.0 * batch * context * G * 2 * dk)

    # ---- retention: a prompt, and a decode step
    Hr, a, b = ret_heads, ret_key, ret_value
    decay = torch.linspace(0.9, 0.999, Hr, device=dev)
    for n_req, extent, first, what in ((1, prompt, 0, f"{prompt} tokens"), (batch, 1, context - 1, f"batch {batch}")):
        ctx = context_of(n_req, extent, first)
        T = n_req * extent
        z = torch.randn((T, Hr * (2 * a + 2 * b)), device=dev).to(bf)
        qk = Hr * a
        state = torch.zeros((n_req + 1, Hr, a, b), dtype=torch.float32, device=dev)
        oo = torch.empty((T, Hr * b), dtype=torch.float32, device=dev)
        rope = torch.randn((T, a), device=dev)
        args = (z[:, :qk], z[:, qk:2 * qk], z[:, 2 * qk:2 * qk + Hr * b], oo, n_req, Hr, a, b, decay,
                a ** -0.5, rope, a, ctx.q_start, ctx.state_slots, state)
        lists = () if extent == 1 else step_chunks(ctx, ops.retention_chunk_tokens())
        ms = _timed(lambda: ops.retention_chunked(*args, *lists), flush)
        in_order = _timed(lambda: ops.retention(*args), flush, repeats=2)
        if extent > 1:
            # by the chunked form's own count: per token and head 2 dk dv for the summaries, as
            # much for the state's part of the outputs, and chunk x (dk + dv) inside the chunk
            C = ops.retention_chunk_tokens()
            row(f"retention (summaries, scan, outputs), {what}", ms, "retention in order", in_order, "fma",
                2.0 * T * Hr * (2 * a * b + C * (a + b) / 2.0))
        else:
            row(f"retention (single tokens), {what}", ms, "retention in order", in_order, "hbm",
                8.0 * n_req * Hr * a * b)
        y = torch.empty((T, Hr * b), dtype=bf, device=dev)
        ms = _timed(lambda: ops.head_norm_gate(oo, z[:, 2 * qk + Hr * b:], y, Hr, b, 1e-6), flush)
        row(f"head_norm_gate, {what}", ms, None, 0.0, "hbm", T * Hr * b * (4 + 2 + 2.0))

    # ---- the add into the stream with its norm, beside the pre-norm layer's
    for T in (prompt, batch):
        h = torch.randn((T, width), device=dev)
        y32 = torch.randn((T, width), device=dev)
        ybf = y32.to(bf)
        gain = torch.ones(width, device=dev)
        act = torch.empty((T, width), dtype=bf, device=dev)
        ms = _timed(lambda: ops.group_norm_scale_add(h, y32, gain, gain, 1e-6, 2, act), flush)
        like_ms = _timed(lambda: ops.add_rmsnorm(h, ybf, gain, 1e-6, act), flush)
        row(f"group_norm_scale_add, {T} rows", ms, "add_rmsnorm", like_ms, "hbm",
            T * width * (4 + 4 + 4 + 2.0), T * width * (4 + 2 + 4 + 2.0))
    T = prompt
    gu = torch.randn((T, 2 * inter), device=dev).to(bf)
    go = torch.empty((T, inter), dtype=bf, device=dev)
    ms = _timed(lambda: ops.gated_act(gu, go, True, "relu"), flush)
    like_ms = _timed(lambda: ops.swiglu(gu, go, True), flush)
    row(f"gated_act relu, {T} rows", ms, "swiglu", like_ms, "hbm", T * inter * 6.0)
    # ---- values normed, blended, stored, beside the q/k-norm kernel that stores k and v
    v = torch.randn((T, G * dv), device=dev).to(bf)
    shared = torch.empty((T, G * dv), dtype=torch.float32, device=dev)
    vcache, _ = _paged(1, T, G, dv, page, dev)
    slots = torch.arange(T, dtype=torch.int32, device=dev) + page
    lam = torch.tensor([0.3], device=dev)
    ops.value_norm_share_cache(v, G, dv, True, 1e-6, None, shared, 1, slots, vcache, page)
    ms = _timed(lambda: ops.value_norm_share_cache(v, G, dv, True, 1e-6, lam, shared, 2, slots, vcache, page),
                flush)
    row(f"value_norm_share_cache, {T} rows", ms, None, 0.0, "hbm", T * G * dv * (2 + 4 + 2.0))
    return out
