"""Time one kernel in isolation (CUDA events, after warm-up), for tuning and for ncu captures.

    python -m pagedserve_b200.kernels.microbench gemm --m 2048 --n 2304 --k 768 [--bn 0] [--impl tc|skinny|rows|simt]
    python -m pagedserve_b200.kernels.microbench attention --batch 64 --context 640 [--heads 12 --head-dim 64]
    python -m pagedserve_b200.kernels.microbench wkv --items 2 --tokens 1024 [--heads 16 --head-dim 64]

``gemm`` prints achieved TFLOP/s and the bytes-per-second of streaming the weight once;
``attention`` prints achieved GB/s over the K and V bytes of the contexts.  Inputs are rotated
over several buffers larger than L2 in total so that a repeat does not find its operands cached.
"""

from __future__ import annotations

import argparse
import math
import sys

import torch


def _time(fn, iters, warmup=3, graph=False):
    """Seconds per call.  ``graph``: the calls are captured into one CUDA graph and replayed, which takes
    the host's launch cost out of the figure (needed for kernels of a few microseconds)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        captured = torch.cuda.CUDAGraph()
        with torch.cuda.graph(captured):
            for i in range(iters):
                fn(i)
        captured.replay()
        torch.cuda.synchronize()
        start.record()
        for _ in range(5):
            captured.replay()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / (5 * iters) * 1e-3
    start.record()
    for i in range(iters):
        fn(i)
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters * 1e-3


def bench_gemm(args):
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    M, N, K = args.m, args.n, args.k
    per_set = (M * K + N * K) * 2 + M * N * 4
    copies = max(2, min(64, int(160e6 // per_set) + 1))          # rotate operands past the 126 MB L2
    a = [torch.randn(M, K, device="cuda").to(torch.bfloat16) for _ in range(copies)]
    w = [(torch.randn(N, K, device="cuda") / math.sqrt(K)).to(torch.bfloat16) for _ in range(copies)]
    bias = torch.randn(N, device="cuda")
    out_dtype = torch.float32 if args.out == "float32" else torch.bfloat16
    out = torch.empty(M, N, dtype=out_dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    acc = args.accumulate
    if args.norm:
        from types import SimpleNamespace

        from pagedserve_b200.parts.base import NormPrologue
        from pagedserve_b200.parts.norms import DeferredNorm

        prologue = NormPrologue(weight=torch.ones(K, device="cuda"), bias=torch.zeros(K, device="cuda"),
                                eps=1e-5, has_mean=True)
        norm = SimpleNamespace(fused_prologue=lambda: prologue)
        x32 = [t.float() for t in a]

    def run(i):
        j = i % copies
        if args.norm:
            ops.linear_skinny_fused(DeferredNorm(norm, x32[j]), w[j], bias, out, act=args.act, accumulate=acc)
        elif args.impl == "tc":
            ops.linear_tc(a[j], w[j], bias, out, act=args.act, accumulate=acc, status=status, bn=args.bn)
        elif args.impl == "skinny":
            ops.linear_skinny(a[j], w[j], bias, out, act=args.act, accumulate=acc)
        elif args.impl == "rows":
            ops.linear_rows_tc(a[j], w[j], bias, out, act=args.act, accumulate=acc, status=status, splits=args.splits)
        else:
            ops.linear_simt(a[j], w[j], bias, out, act=args.act, accumulate=acc)

    seconds = _time(run, args.iters, graph=args.graph)
    flops = 2.0 * M * N * K
    print(f"gemm {'skinny+norm' if args.norm else args.impl} M={M} N={N} K={K} bn={args.bn} out={args.out}"
          f"{' accumulate' if acc else ''}: {seconds * 1e6:.2f} us, "
          f"{flops / seconds / 1e12:.1f} TFLOP/s, weight stream {N * K * 2 / seconds / 1e9:.0f} GB/s, "
          f"status {int(status.item())}")


def bench_attention(args):
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    B, ctx, H, D, page = args.batch, args.context, args.heads, args.head_dim, args.page_size
    pages_per = -(-ctx // page)
    layers = max(1, min(48, int(200e6 // (B * pages_per * page * H * D * 4)) + 1))   # rotate layers past L2
    pool = torch.randn(B * pages_per + 1, layers, 2, H, page, D, device="cuda").to(torch.bfloat16)
    table = torch.randperm(B * pages_per, device="cuda").to(torch.int32).view(B, pages_per)
    q = torch.randn(B, H * D, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    token_item = torch.arange(B, dtype=torch.int32, device="cuda")
    positions = torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda")
    stride = layers * 2 * H * page * D
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def run(i):
        layer = i % layers
        ops.paged_attention_decode(q, out, pool[:, layer, 0], pool[:, layer, 1], stride, token_item, positions, table,
                                   H, H, D, page, None, D ** -0.5, args.max_context or ctx, status=status)

    seconds = _time(run, args.iters, graph=args.graph)
    nbytes = B * ctx * H * D * 2 * 2
    print(f"decode attention B={B} ctx={ctx} heads={H} hd={D} page={page}: {seconds * 1e6:.2f} us, "
          f"{nbytes / seconds / 1e9:.0f} GB/s of K+V, status {int(status.item())}")


# ------------------------------------------------------------------ kernels as functions (bench.py calls these)
def _paged_inputs(items, context, kv_heads, head_dim, page, rotate_mb=200, planes=2):
    """A pool of random pages with one table row per item; several layers so that repeats miss the L2.
    ``planes`` 1: a cache whose rows are read as keys and as values."""
    pages_per = -(-context // page)
    layer_bytes = items * pages_per * page * kv_heads * head_dim * 2 * planes
    layers = max(1, min(16, int(rotate_mb * 1e6 // layer_bytes) + 1))
    pool = torch.randn(items * pages_per + 1, layers, planes, kv_heads, page, head_dim, device="cuda").to(torch.bfloat16)
    table = torch.randperm(items * pages_per, device="cuda").to(torch.int32).view(items, pages_per)
    return pool, table, layers, layers * planes * kv_heads * page * head_dim


def time_decode_attention(batch, context, heads, kv_heads, head_dim, page=16, window=None, softcap=None,
                          sink=False, iters=20, planes=2, chunk=None):
    """One decode token per request over ``context`` keys (bfloat16 split-key kernel); GB/s over the K and V
    bytes a token may see (with one plane: over the rows once)."""
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    pool, table, layers, stride = _paged_inputs(batch, context, kv_heads, head_dim, page, planes=planes)
    q = torch.randn(batch, heads * head_dim, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    token_item = torch.arange(batch, dtype=torch.int32, device="cuda")
    positions = torch.full((batch,), context - 1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sinks = torch.randn(heads, device="cuda") if sink else None
    if chunk:                                           # a chunked mask travels as a negative window
        window = -chunk

    def run(i):
        layer = i % layers
        ops.paged_attention_decode(q, out, pool[:, layer, 0], pool[:, layer, planes - 1], stride, token_item, positions,
                                   table, heads, kv_heads, head_dim, page, window, head_dim ** -0.5, context,
                                   status=status, softcap=softcap, sink=sinks)

    seconds = _time(run, iters, graph=True)
    seen = min(context, window) if window and window > 0 else context
    if chunk:
        seen = (context - 1) % chunk + 1
    nbytes = batch * seen * kv_heads * head_dim * 2 * planes
    return {"us": seconds * 1e6, "gbs": nbytes / seconds / 1e9, "status": int(status.item())}


def time_prefill_attention(prompts, prompt_len, heads, kv_heads, head_dim, page=16, window=None, softcap=None,
                           sink=False, iters=10, planes=2, chunk=None):
    """Whole prompts through the tcgen05 prompt kernel (bfloat16, head size 64 or 128); TFLOP/s over the
    products of the keys a query may see."""
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    pool, table, layers, _ = _paged_inputs(prompts, prompt_len, kv_heads, head_dim, page, rotate_mb=0, planes=planes)
    total = prompts * prompt_len
    q = torch.randn(total, heads * head_dim, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    q_start = torch.arange(0, total + 1, prompt_len, dtype=torch.int32, device="cuda")
    kv_len = torch.full((prompts,), prompt_len, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sinks = torch.randn(heads, device="cuda") if sink else None
    blocks = prompts * -(-prompt_len // 128)
    if chunk:
        window = -chunk

    def run(i):
        ops.prefill_attention_tc(q, out, pool, 0, q_start, kv_len, table, 0, prompts, blocks, heads, kv_heads,
                                 head_dim, page, window, head_dim ** -0.5, status=status, softcap=softcap, sink=sinks)

    seconds = _time(run, iters, graph=True)
    if chunk:
        whole, rest = divmod(prompt_len, chunk)
        pairs = whole * chunk * (chunk + 1) / 2.0 + rest * (rest + 1) / 2.0
    elif window and window < prompt_len:
        pairs = window * (window + 1) / 2.0 + (prompt_len - window) * float(window)
    else:
        pairs = prompt_len * (prompt_len + 1) / 2.0
    flops = 4.0 * prompts * heads * head_dim * pairs
    return {"us": seconds * 1e6, "tflops": flops / seconds / 1e12, "status": int(status.item())}


def time_wkv(items, tokens_each, heads, head_dim, width, dtype=torch.bfloat16, iters=10):
    """The recurrence kernel alone on ``items`` entries of ``tokens_each`` tokens; GB/s over what it must move:
    five float32 streams in, one row out, and every entry's state matrix in and out."""
    from types import SimpleNamespace

    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(dtype)
    total, inner = items * tokens_each, heads * head_dim
    matrix = heads * head_dim * head_dim
    streams = torch.randn(5, total, inner, device="cuda")
    streams[3] = -1.0 + streams[3]                      # the decay's argument: decays spread over (0, 1)
    x = torch.randn(total, width, device="cuda").to(dtype)
    state = torch.zeros(items, matrix + width, device="cuda")
    u, gain = torch.randn(inner, device="cuda"), torch.ones(inner, device="cuda")
    out = torch.empty(total, inner, dtype=dtype, device="cuda")
    ctx = SimpleNamespace(q_start=torch.arange(0, total + 1, tokens_each, dtype=torch.int32, device="cuda"),
                          item_slot=torch.arange(items, dtype=torch.int32, device="cuda"), num_items=items)

    def run(i):
        ops.wkv_recurrence(streams[0], streams[1], streams[2], streams[3], streams[4], u, gain, 1e-5, x, state,
                           matrix, ctx, out, heads, head_dim)

    seconds = _time(run, iters, graph=True)
    nbytes = total * inner * (5 * 4 + out.element_size()) + items * matrix * 4 * 2
    return {"us": seconds * 1e6, "gbs": nbytes / seconds / 1e9, "tokens_per_s": total / seconds}


def time_cache_write(tokens, heads, kv_heads, head_dim, page=16, rot_dims=None, iters=20):
    """The kernel that turns queries and keys and fills the pages, beside the plain cache write (``kv_append``)
    of as many tokens; GB/s over queries and keys read and queries, keys and values written."""
    from types import SimpleNamespace

    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    pool, table, _, stride = _paged_inputs(1, tokens, kv_heads, head_dim, page, rotate_mb=0)
    q = torch.randn(tokens, heads * head_dim, device="cuda").to(torch.bfloat16)
    k = torch.randn(tokens, kv_heads * head_dim, device="cuda").to(torch.bfloat16)
    rot = head_dim if rot_dims is None else rot_dims
    inv_freq = (10000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1))).float().cuda()
    item = torch.zeros(tokens, dtype=torch.int32, device="cuda")
    positions = torch.arange(tokens, dtype=torch.int32, device="cuda")
    layer = SimpleNamespace(k_pool=pool[:, 0, 0], v_pool=pool[:, 0, 1], page_stride=stride, page_size=page,
                            block_table=table)
    ctx = SimpleNamespace(token_slot=item, positions=positions)
    turned = _time(lambda i: ops.rotary_cache_write(q, k, None, inv_freq, rot, True, ctx, layer, heads, kv_heads,
                                                    head_dim), iters, graph=True)
    plain = _time(lambda i: ops.kv_append(k, k, item, positions, table, layer.k_pool, layer.v_pool, stride, kv_heads,
                                          head_dim, page), iters, graph=True)
    moved = tokens * head_dim * 2 * (2 * heads + 3 * kv_heads)
    return {"us": turned * 1e6, "gbs": moved / turned / 1e9, "plain_write_us": plain * 1e6,
            "plain_write_gbs": tokens * head_dim * 2 * 4 * kv_heads / plain / 1e9}


def time_head_norm_cache_write(tokens, heads, kv_heads, head_dim, page=16, rot_dims=None, iters=20):
    """The kernel that norms and turns query and key heads (halves paired) and fills the pages with keys and
    values; GB/s over queries, keys and values read and written."""
    from types import SimpleNamespace

    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    pool, table, _, stride = _paged_inputs(1, tokens, kv_heads, head_dim, page, rotate_mb=0)
    q = torch.randn(tokens, heads * head_dim, device="cuda").to(torch.bfloat16)
    k = torch.randn(tokens, kv_heads * head_dim, device="cuda").to(torch.bfloat16)
    v = torch.randn(tokens, kv_heads * head_dim, device="cuda").to(torch.bfloat16)
    rot = head_dim if rot_dims is None else rot_dims
    freq = 10000.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1))
    high = freq.float()
    inv_freq = torch.stack([high, (freq - high.double()).float()], dim=1).contiguous().cuda()
    gain = torch.ones(head_dim, device="cuda")
    item = torch.zeros(tokens, dtype=torch.int32, device="cuda")
    positions = torch.arange(tokens, dtype=torch.int32, device="cuda")
    layer = SimpleNamespace(k_pool=pool[:, 0, 0], v_pool=pool[:, 0, 1], page_stride=stride, page_size=page,
                            block_table=table)
    ctx = SimpleNamespace(token_slot=item, positions=positions)
    seconds = _time(lambda i: ops.head_norm_rotary_cache_write(q, k, v, gain, gain, 1e-6, inv_freq, rot, False, head_dim,
                                                               ctx, layer, heads, kv_heads, head_dim), iters, graph=True)
    moved = tokens * head_dim * 2 * (2 * heads + 4 * kv_heads)
    return {"us": seconds * 1e6, "gbs": moved / seconds / 1e9}


def time_shared_position_attention(batch, context, heads, head_dim, page=16, window=None, iters=20):
    """One decode token per request whose ``heads`` query heads all read one cached row of ``head_dim`` numbers
    (a one-plane cache): the heads run as the query rows of one tile; GB/s over the rows a token may see, once."""
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    pool, table, layers, stride = _paged_inputs(batch, context, 1, head_dim, page, planes=1)
    q = torch.randn(batch, heads * head_dim, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    rows = torch.arange(batch, dtype=torch.int32, device="cuda")
    positions = torch.full((batch,), context - 1, dtype=torch.int32, device="cuda")

    def run(i):
        layer = i % layers
        ops.shared_position_attention(q, out, pool[:, layer, 0], pool[:, layer, 0], stride, positions, table, rows,
                                      heads, head_dim, page, window, head_dim ** -0.5, max_kv_len=context)

    seconds = _time(run, iters, graph=True)
    seen = min(context, window) if window else context
    return {"us": seconds * 1e6, "gbs": batch * seen * head_dim * 2 / seconds / 1e9}


def time_latent_prepare(tokens, heads, flat, turning, rank, page=16, iters=20):
    """The kernel between the input projection and attention of a latent-attention layer (norm of the latent,
    turns, cache write); GB/s over what it reads and writes."""
    from types import SimpleNamespace

    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    row = rank + turning
    pool, table, _, stride = _paged_inputs(1, tokens, 1, row, page, rotate_mb=0, planes=1)
    q = torch.randn(tokens, heads * (flat + turning), device="cuda").to(torch.bfloat16)
    down = torch.randn(tokens, row, device="cuda").to(torch.bfloat16)
    q_out = torch.empty(tokens, heads * row, dtype=torch.bfloat16, device="cuda")
    gain = torch.ones(rank, device="cuda")
    freq = 10000.0 ** (-2.0 * torch.arange(turning // 2, dtype=torch.float64) / max(turning, 1))
    inv_freq = torch.stack([freq.float(), (freq - freq.float().double()).float()], dim=1).contiguous().cuda()
    item = torch.zeros(tokens, dtype=torch.int32, device="cuda")
    layer = SimpleNamespace(k_pool=pool[:, 0, 0], page_stride=stride, page_size=page, block_table=table)
    ctx = SimpleNamespace(token_slot=item, positions=torch.arange(tokens, dtype=torch.int32, device="cuda"))
    seconds = _time(lambda i: ops.latent_prepare(q, down, gain, 1e-5, inv_freq, turning, ctx, layer, q_out, heads, flat,
                                                 turning, rank), iters, graph=True)
    moved = tokens * 2 * (2 * heads * turning + 2 * row)
    return {"us": seconds * 1e6, "gbs": moved / seconds / 1e9}


def time_hyper_step(tokens, width, streams, iters=20):
    """One pass over the residual streams (update of a sublayer and the read of the next); GB/s over the streams
    read and written, the sublayer's row read and zeroed, and the next input written."""
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    copies = max(1, int(200e6 // (streams * tokens * width * 4)) + 1)           # rotate past the L2
    x = torch.randn(copies, streams, tokens, width, device="cuda")
    y = torch.randn(copies, tokens, width, device="cuda")
    u = torch.empty(tokens, width, device="cuda")
    mix = (torch.eye(streams) + 0.1 * torch.randn(streams, streams)).cuda()
    w_out, w_in = torch.ones(streams, device="cuda"), torch.ones(streams, device="cuda")
    seconds = _time(lambda i: ops.hyper_step(x[i % copies], y[i % copies], mix, w_out, w_in, u), iters, graph=True)
    moved = tokens * width * 4 * (2 * streams + 3)
    return {"us": seconds * 1e6, "gbs": moved / seconds / 1e9}


def time_mingru(items, tokens_each, width, dtype=torch.bfloat16, iters=10):
    """The gated recurrence kernel alone on ``items`` entries of ``tokens_each`` tokens; GB/s over what it must move:
    three float32 projections in, one row out, and every entry's state in and out."""
    from types import SimpleNamespace

    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(dtype)
    total = items * tokens_each
    copies = max(1, int(200e6 // (total * width * 14)) + 1)                       # rotate past the L2
    zug = torch.randn(copies, total, 3 * width, device="cuda")
    state = torch.zeros(items + 1, width, device="cuda")
    out = torch.empty(total, width, dtype=dtype, device="cuda")
    ctx = SimpleNamespace(q_start=torch.arange(0, total + 1, tokens_each, dtype=torch.int32, device="cuda"),
                          item_slot=torch.arange(items, dtype=torch.int32, device="cuda"), num_items=items,
                          max_q_len=tokens_each)
    seconds = _time(lambda i: ops.mingru_scan(zug[i % copies], width, state, ctx, out), iters, graph=True)
    nbytes = total * width * (3 * 4 + out.element_size()) + items * width * 4 * 2
    return {"us": seconds * 1e6, "gbs": nbytes / seconds / 1e9, "tokens_per_s": total / seconds}


def time_post_norm_add(tokens, width, groups, entries, iters=20):
    """The kernel that closes a sublayer of a layer that norms its sublayers' results, with the average over
    ``entries`` rows of depth behind it; GB/s over the sublayer's row read and zeroed, the residual row read and
    written, the new entry written, the older entries read and the rounded copy written."""
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    copies = max(1, int(200e6 // ((entries + 2) * tokens * width * 4)) + 1)         # rotate past the L2
    history = torch.randn(copies, entries, tokens, width, device="cuda")
    x = torch.randn(copies, tokens, width, device="cuda")
    y = torch.randn(copies, tokens, width, device="cuda")
    cast = torch.empty(tokens, width, dtype=torch.bfloat16, device="cuda")
    gain = torch.ones(width, device="cuda")
    weight = torch.full((entries,), 1.0 / entries, device="cuda")
    seconds = _time(lambda i: ops.post_norm_add(y[i % copies], x[i % copies], gain, 1e-6, groups, cast,
                                                history[i % copies], entries, weight), iters, graph=True)
    moved = tokens * width * (4 * (4 + entries) + 2)
    return {"us": seconds * 1e6, "gbs": moved / seconds / 1e9}


def time_short_conv(tokens, items, heads, kv_heads, head_dim, taps, iters=20):
    """The short convolution over q | k | v (with the gate's columns passed through and the values blended) and the
    kernel that keeps the entries' last rows; GB/s over the float32 rows read once and the rounded rows written."""
    from types import SimpleNamespace

    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    conv = (heads + 2 * kv_heads) * head_dim
    channels = conv + heads * head_dim
    copies = max(1, int(200e6 // (tokens * channels * 6)) + 1)                     # rotate past the L2
    u = torch.randn(copies, tokens, channels, device="cuda")
    out = torch.empty(tokens, channels, dtype=torch.bfloat16, device="cuda")
    weight = torch.randn(conv, taps, device="cuda")
    state = torch.zeros(items + 1, (taps - 1) * conv, device="cuda")
    shared = torch.randn(tokens, kv_heads * head_dim, device="cuda")
    mix = torch.full((1,), 0.3, device="cuda")
    each = tokens // items
    ctx = SimpleNamespace(q_start=torch.arange(0, tokens + 1, each, dtype=torch.int32, device="cuda"),
                          item_slot=torch.arange(items, dtype=torch.int32, device="cuda"), num_items=items,
                          token_item=(torch.arange(tokens, device="cuda") // each).to(torch.int32))
    blend = ("mix", (heads + kv_heads) * head_dim, kv_heads, head_dim, head_dim, shared, mix)
    seconds = _time(lambda i: ops.short_conv(u[i % copies], weight, taps, conv, state, ctx, out, blend=blend), iters,
                    graph=True)
    moved = tokens * channels * 6 + tokens * kv_heads * head_dim * 4
    return {"us": seconds * 1e6, "gbs": moved / seconds / 1e9}


def time_experts(tokens, width, experts, top, ff, iters=10, score="softmax", normalize=True, form=None):
    """The routed part of a feed-forward of ``experts`` experts, rows sorted by expert: router, plan, gather, the
    two tcgen05 products over expert tiles, gate, combine; beside the two plain tcgen05 products of a dense
    feed-forward with the same inner size per token (top * ff).  TFLOP/s over the useful products.  ``score``,
    ``normalize`` and ``form`` as the router and the inner activation take them (sigmoid scores that are the
    weights; clamped experts)."""
    from pagedserve_b200.kernels.ops import Ops

    ops = Ops(torch.bfloat16)
    dev = "cuda"
    x = torch.randn(tokens, width, device=dev).to(torch.bfloat16)
    router = (torch.randn(experts, width, device=dev) * 0.05).to(torch.bfloat16)
    w_gu = (torch.randn(experts * 2 * ff, width, device=dev) * width ** -0.5).to(torch.bfloat16)
    w_down = (torch.randn(width, experts * ff, device=dev) * ff ** -0.5).to(torch.bfloat16)
    dense = torch.empty(tokens, experts, device=dev)
    chosen = torch.empty(tokens, top, dtype=torch.int32, device=dev)
    chosen_w = torch.empty(tokens, top, device=dev)
    rows_cap = ops.expert_rows(tokens, top, experts)
    row_of = torch.empty(tokens * top, dtype=torch.int32, device=dev)
    row_token = torch.empty(rows_cap, dtype=torch.int32, device=dev)
    row_weight = torch.empty(rows_cap, device=dev)
    tile_expert = torch.empty(rows_cap // ops.EXPERT_TILE, dtype=torch.int32, device=dev)
    rows = torch.empty(rows_cap, width, dtype=torch.bfloat16, device=dev)
    gate_up = torch.empty(rows_cap, 2 * ff, dtype=torch.bfloat16, device=dev)
    inner = torch.empty(rows_cap, ff, dtype=torch.bfloat16, device=dev)
    down = torch.empty(rows_cap, width, device=dev)
    y = torch.zeros(tokens, width, device=dev)
    status = ops.status_flag(dev)
    parts = {}

    def routed(i):
        ops.moe_route(x, router, None, dense, chosen, chosen_w, None, top, 0, 0, score=score, normalize=normalize)
        ops.moe_plan(chosen, chosen_w, experts, row_of, row_token, row_weight, tile_expert)
        ops.moe_gather(x, row_token, rows)
        ops.linear_experts(rows, w_gu, gate_up, tile_expert, experts)
        ops.moe_gate_mul_rows(gate_up, row_weight, inner, form=form)
        ops.linear_experts(inner, w_down, down, tile_expert, experts, along_k=True)
        ops.moe_combine(down, row_of, top, y)

    seconds = _time(routed, iters, graph=True)
    parts["route_us"] = _time(lambda i: ops.moe_route(x, router, None, dense, chosen, chosen_w, None, top, 0, 0, score=score, normalize=normalize), iters,
                              graph=True) * 1e6
    parts["plan_us"] = _time(lambda i: ops.moe_plan(chosen, chosen_w, experts, row_of, row_token, row_weight, tile_expert),
                             iters, graph=True) * 1e6
    parts["gather_us"] = _time(lambda i: ops.moe_gather(x, row_token, rows), iters, graph=True) * 1e6
    parts["gate_up_us"] = _time(lambda i: ops.linear_experts(rows, w_gu, gate_up, tile_expert, experts), iters,
                                graph=True) * 1e6
    parts["gate_mul_us"] = _time(lambda i: ops.moe_gate_mul_rows(gate_up, row_weight, inner, form=form), iters, graph=True) * 1e6
    parts["down_us"] = _time(lambda i: ops.linear_experts(inner, w_down, down, tile_expert, experts, along_k=True), iters,
                             graph=True) * 1e6
    parts["combine_us"] = _time(lambda i: ops.moe_combine(down, row_of, top, y), iters, graph=True) * 1e6
    # a dense feed-forward of the same inner size per token: up to 2 * top * ff columns, down from top * ff
    wide = top * ff
    w_up_d = (torch.randn(2 * wide, width, device=dev) * width ** -0.5).to(torch.bfloat16)
    w_down_d = (torch.randn(width, wide, device=dev) * wide ** -0.5).to(torch.bfloat16)
    up_d = torch.empty(tokens, 2 * wide, dtype=torch.bfloat16, device=dev)
    inner_d = up_d[:, :wide]

    def plain(i):
        ops.linear_tc(x, w_up_d, None, up_d, status=status)
        ops.linear_tc(inner_d, w_down_d, None, y, accumulate=True, status=status)

    plain_seconds = _time(plain, iters, graph=True)
    flops = 2.0 * tokens * top * (3 * ff) * width
    return {"us": seconds * 1e6, "tflops": flops / seconds / 1e12, "dense_us": plain_seconds * 1e6,
            "dense_tflops": flops / plain_seconds / 1e12, "status": int(status.item()), **parts}


def main(argv=None):
    parser = argparse.ArgumentParser(prog="python -m pagedserve_b200.kernels.microbench")
    sub = parser.add_subparsers(dest="kind", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=2048)
    g.add_argument("--n", type=int, default=2304)
    g.add_argument("--k", type=int, default=768)
    g.add_argument("--bn", type=int, default=0)
    g.add_argument("--impl", default="tc", choices=("tc", "skinny", "rows", "simt"))
    g.add_argument("--splits", type=int, default=0, help="rows: CTAs per column tile (0: the kernel chooses)")
    g.add_argument("--act", default=None)
    g.add_argument("--out", default="bfloat16", choices=("bfloat16", "float32"))
    g.add_argument("--accumulate", action="store_true", help="add the product to what the output holds")
    g.add_argument("--norm", action="store_true",
                   help="the few-rows kernel with a LayerNorm of float32 rows fused in front")
    g.add_argument("--iters", type=int, default=50)
    g.add_argument("--graph", action="store_true", help="replay the calls as one CUDA graph")
    a = sub.add_parser("attention")
    a.add_argument("--batch", type=int, default=64)
    a.add_argument("--context", type=int, default=640)
    a.add_argument("--max-context", type=int, default=0)
    a.add_argument("--heads", type=int, default=12)
    a.add_argument("--head-dim", type=int, default=64)
    a.add_argument("--page-size", type=int, default=16)
    a.add_argument("--iters", type=int, default=50)
    a.add_argument("--graph", action="store_true", help="replay the calls as one CUDA graph")
    w = sub.add_parser("wkv")
    w.add_argument("--items", type=int, default=2)
    w.add_argument("--tokens", type=int, default=1024, help="tokens of every entry")
    w.add_argument("--heads", type=int, default=16)
    w.add_argument("--head-dim", type=int, default=64)
    w.add_argument("--width", type=int, default=1024)
    w.add_argument("--iters", type=int, default=10)
    args = parser.parse_args(argv)
    if args.kind == "gemm":
        bench_gemm(args)
    elif args.kind == "wkv":
        run = time_wkv(args.items, args.tokens, args.heads, args.head_dim, args.width, iters=args.iters)
        print(f"wkv recurrence items={args.items} tokens={args.tokens} heads={args.heads} hd={args.head_dim}: "
              f"{run['us']:.2f} us, {run['gbs']:.0f} GB/s, {run['tokens_per_s'] / 1e6:.2f} M tokens/s")
    else:
        bench_attention(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
