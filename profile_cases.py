"""Small stand-alone launches of each kernel at the benchmark's shapes, for profilers:

    python profile_cases.py dense_attn [--reps 3] [--ctx 131072]
    ncu --set full --clock-control none -k regex:decode_attn_mma -c 3 python profile_cases.py dense_attn

    python -m omnikv_b200.build --trace     # once: the profiling build of the library
    OMNIKV_B200_LIB=omnikv_b200/_lib/libomnikv_b200_trace.so python -m torch.distributed.run --nnodes=1 \
        --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29533 profile_cases.py tp_timeline

Cases: tp_timeline (one graph-replayed decode step of the benchmark on N GPUs, or on one: per-kernel %globaltimer
stamps of the profiling build, with the wait for the peers' flags separated from the streaming time), dense_attn (filter layer: K and V of 8 KV heads x ctx rows, fused scores), sparse_attn
(8781 selected rows + tail), topk (ctx scores, 8 planes), score_window (16-slot window, exp),
offload_gather (30150 tokens x 12 layers from pinned host memory).  Each prints the CUDA-event time per launch.
"""
from __future__ import annotations

import argparse

import torch

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from omnikv_b200 import ops  # noqa: E402


def gemv_cases(reps: int, n_sets: int = 8):
    """The four weight-streaming kernels of a Llama-3-8B decoder layer, each over ``n_sets`` distinct weight
    sets back to back (so that no launch finds its weights in L2), timed per launch with CUDA events."""
    dev, dt = "cuda", torch.bfloat16
    hidden, inter, H, KVH = 4096, 14336, 32, 8
    mk = lambda n, k: [torch.randn(n, k, device=dev, dtype=torch.float32).mul_(k ** -0.5).to(dt) for _ in range(n_sets)]  # noqa: E731
    w_qkv, w_o, w_gu, w_d = mk((H + 2 * KVH) * 128, hidden), mk(hidden, hidden), mk(2 * inter, hidden), mk(hidden, inter)
    h = torch.randn(hidden, device=dev).to(dt)
    nw = torch.ones(hidden, device=dev, dtype=dt)
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))).to(dev)
    pos = torch.tensor([5], dtype=torch.int32, device=dev)
    q = torch.zeros(H * 128, dtype=dt, device=dev)
    kc = torch.zeros(KVH, 16, 128, dtype=dt, device=dev)
    vc = torch.zeros_like(kc)
    act = torch.zeros(inter, dtype=dt, device=dev)
    out = torch.zeros(hidden, dtype=dt, device=dev)
    def layer_separate(i):
        ops.decode_gemv_residual(w_o[i], q, h, out)
        ops.decode_gate_up(out, nw, 1e-5, w_gu[i], act)
        ops.decode_gemv_residual(w_d[i], act, out, out)
        ops.decode_qkv(out, nw, 1e-5, w_qkv[i], H, KVH, inv_freq, pos, q, kc, vc, pos)

    counters = torch.zeros(n_sets, 4, dtype=torch.int32, device=dev)

    def layer_chain(i):
        if i == 0:
            counters.zero_()
        ops.decode_chain(out, chunk_counters=counters[i], eps=1e-5, H=H, KVH=KVH, inter=inter, w_o=w_o[i], attn_out=q, post_norm_w=nw,
                         w_gate_up=w_gu[i], w_down=w_d[i], act=act, in_norm_w=nw, w_qkv=w_qkv[i], inv_freq=inv_freq,
                         rope_pos=pos, q_out=q, k_cache_seq=kc, v_cache_seq=vc, cache_pos=pos)

    layer_bytes = (w_qkv[0].numel() + w_o[0].numel() + w_gu[0].numel() + w_d[0].numel()) * 2
    kinds = {
        "qkv+rope+append": (lambda i: ops.decode_qkv(h, nw, 1e-5, w_qkv[i], H, KVH, inv_freq, pos, q, kc, vc, pos), w_qkv[0].numel() * 2),
        "o_proj+residual": (lambda i: ops.decode_gemv_residual(w_o[i], q, h, out), w_o[0].numel() * 2),
        "gate_up+silu": (lambda i: ops.decode_gate_up(h, nw, 1e-5, w_gu[i], act), w_gu[0].numel() * 2),
        "down+residual": (lambda i: ops.decode_gemv_residual(w_d[i], act, h, out), w_d[0].numel() * 2),
        "layer: 4 launches": (layer_separate, layer_bytes),
        "layer: 1 chained launch": (layer_chain, layer_bytes),
    }
    # every kind is captured in a CUDA graph (8 launches over 8 distinct weight sets) so that the host's
    # launch cost does not show in the per-launch time
    for name, (fn, nbytes) in kinds.items():
        fn(0)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(n_sets):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        for r in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / n_sets
            print(f"{name} rep {r}: {ms * 1e3:.1f} us per launch, {nbytes / 1e6:.1f} MB, {nbytes / ms / 1e6:.0f} GB/s")
    ops.check_status(dev)


def batched_linear_cases(reps: int, n_tokens: int = 16, n_sets: int = 8):
    """The projections of a Llama-3-8B decoder layer for ``n_tokens`` sequences decoding together: this package's
    tcgen05 weight stream and the library GEMM (plus the separate norm / activation / residual kernels it needs), each
    over ``n_sets`` distinct weight sets back to back inside a CUDA graph."""
    import torch.nn.functional as F
    dev, dt = "cuda", torch.bfloat16
    hidden, inter, H, KVH = 4096, 14336, 32, 8
    mk = lambda n, k: [torch.randn(n, k, device=dev, dtype=torch.float32).mul_(k ** -0.5).to(dt) for _ in range(n_sets)]  # noqa: E731
    w_qkv, w_o, w_gu, w_d = mk((H + 2 * KVH) * 128, hidden), mk(hidden, hidden), mk(2 * inter, hidden), mk(hidden, inter)
    x = torch.randn(n_tokens, hidden, device=dev).to(dt)
    a_in = torch.randn(n_tokens, inter, device=dev).to(dt)
    nw = torch.ones(hidden, device=dev, dtype=dt)
    h = torch.zeros(n_tokens, hidden, device=dev, dtype=dt)

    def lib_gate_up(i):
        gu = F.linear(F.rms_norm(x, (hidden,), nw, 1e-5), w_gu[i])
        return F.silu(gu[:, :inter]) * gu[:, inter:]

    kinds = {
        "qkv (norm in front)": (lambda i: ops.batched_linear(x, w_qkv[i], norm_w=nw),
                                lambda i: F.linear(F.rms_norm(x, (hidden,), nw, 1e-5), w_qkv[i]), w_qkv[0].numel() * 2),
        "o_proj + residual": (lambda i: ops.batched_linear(x, w_o[i], epilogue="residual", residual=h, out=h),
                              lambda i: h.add_(F.linear(x, w_o[i])), w_o[0].numel() * 2),
        "gate_up + silu (norm in front)": (lambda i: ops.batched_linear(x, w_gu[i], epilogue="swiglu", norm_w=nw),
                                           lib_gate_up, w_gu[0].numel() * 2),
        "down + residual": (lambda i: ops.batched_linear(a_in, w_d[i], epilogue="residual", residual=h, out=h),
                            lambda i: h.add_(F.linear(a_in, w_d[i])), w_d[0].numel() * 2),
    }
    for name, (mine, lib, nbytes) in kinds.items():
        for leg, fn in (("tcgen05 stream", mine), ("library GEMM + element-wise kernels", lib)):
            fn(0)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(n_sets):
                    fn(i)
            g.replay()
            torch.cuda.synchronize()
            for r in range(reps):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                g.replay()
                b.record()
                torch.cuda.synchronize()
                ms = a.elapsed_time(b) / n_sets
                print(f"{name} [{leg}] rep {r}: {ms * 1e3:.1f} us per call, {nbytes / 1e6:.1f} MB, {nbytes / ms / 1e6:.0f} GB/s")
    ops.check_status(dev)


def tp_timeline(ctx: int, replays: int = 6):
    """One decode step of the benchmark (Llama-3-8B shape, batch 1, ``ctx`` tokens of synthetic KV, fused kernels,
    peer-memory exchange, CUDA graph) on the ranks of this torchrun job, with the profiling build of the library:
    every weight-streaming and attention launch of the LAST replay reports, from its own %globaltimer stamps, when
    it started, when the previous kernel had completed, how long it waited for the peers' flags, when its first
    weights landed and when it ended.  Timers of different GPUs are not comparable: every figure is a difference
    on one GPU.  Rank 0 prints its table and a summary by kind; every rank prints its totals."""
    import ctypes
    import os

    import numpy as np

    from omnikv_b200 import abi, parallel
    from omnikv_b200.modeling import LlamaCompressorConfig, OmniKVMulLM
    from omnikv_b200.modeling.omnikv import DecodeRunner
    lib = abi.lib()
    if not hasattr(lib, "omnikv_debug_gemv_trace"):
        raise SystemExit("tp_timeline needs the profiling build: python -m omnikv_b200.build --trace and "
                         "OMNIKV_B200_LIB=omnikv_b200/_lib/libomnikv_b200_trace.so")
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    tp = parallel.init(world, rank, dev) if world > 1 else None
    if tp is not None:
        tp.enable_peer_exchange(4096, dev)
    cfg = LlamaCompressorConfig()
    cfg.set_config_of_compressor(model_cls="multi", cache_cls="multi", do_select_layers="2,8,18", num_wait_load_layers=1,
                                 real_offload=False, dense_more=True, num_of_selected_tokens=0.067, selector_cls="last",
                                 window_size=16, fused_decode=True, chained_decode=False)
    lm = OmniKVMulLM.from_config(cfg, dtype=torch.bfloat16, device=dev, seed=0, tp=tp)
    cache = lm.new_cache().init_synthetic(1, cfg.num_key_value_heads // world, cfg.head_dim, [ctx], torch.bfloat16, dev,
                                          seed=1 + rank, reserve=64)
    runner = DecodeRunner(lm, None, cache=cache, first_token=torch.ones(1, 1, dtype=torch.int64, device=dev),
                          max_new_tokens=40, use_cuda_graph=False)
    runner.run(2)
    torch.cuda.synchronize()
    lib.omnikv_debug_trace_reset()
    runner._capture()          # the capture issues the step's launches once: slots 0 .. launches-1
    n_launch = runner.launches_per_step
    if tp is not None:
        torch.distributed.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    runner.run(2)
    e0.record()
    runner.run(replays)
    e1.record()
    torch.cuda.synchronize()
    step_us = e0.elapsed_time(e1) * 1e3 / replays
    GS, GC, GW, AC, AW = 256, 160, 12, 320, 8
    gbuf = (ctypes.c_uint64 * (GS * GC * GW))()
    abuf = (ctypes.c_uint64 * (GS * AC * AW))()
    lib.omnikv_debug_gemv_trace.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.omnikv_debug_attn_trace.argtypes = [ctypes.c_void_p, ctypes.c_int]
    assert lib.omnikv_debug_gemv_trace(gbuf, GS * GC * GW) == 0 and lib.omnikv_debug_attn_trace(abuf, GS * AC * AW) == 0
    g = np.frombuffer(gbuf, dtype=np.uint64).astype(np.int64).reshape(GS, GC, GW)
    a = np.frombuffer(abuf, dtype=np.uint64).astype(np.int64).reshape(GS, AC, AW)
    names = {1000: "qkv", 1002: "qkv<-x", 1010: "resid", 1011: "resid->x", 1020: "gate_up", 1022: "gate_up<-x",
             1030: "logits", 1032: "logits<-x", 2000: "attn dense", 2001: "attn sparse"}
    rows = []
    for slot in range(GS):
        if 1000 <= g[slot, 0, 10] < 2000:
            t = g[slot]
            live = t[:, 0] > 0
            n_cta = int(live.sum())
            t = t[live]
            flags = t[:, 9][t[:, 9] > 0]
            rows.append(dict(slot=slot, kind=names.get(int(t[0, 10]), str(t[0, 10])), ctas=n_cta, start=t[:, 0].min(),
                             prev_done=np.median(t[:, 1]), wait=np.median(t[:, 7] - t[:, 6]), first=np.median(t[:, 3]),
                             rows_done=t[:, 8].max(), end=t[:, 4].max(), flags=int(flags.max()) if flags.size else 0))
        elif 2000 <= a[slot, 0, 6] < 3000:
            t = a[slot]
            kind = names[int(t[0, 6])]
            live = t[:, 0] > 0
            t = t[live]
            rows.append(dict(slot=slot, kind=kind, ctas=int(live.sum()), start=t[:, 0].min(), prev_done=np.median(t[:, 1]),
                             wait=0.0, first=np.median(t[:, 2]), rows_done=t[:, 3].max(), end=t[:, 5].max(), flags=0))
    rows.sort(key=lambda r: r["start"])
    rows = rows[-n_launch:] if len(rows) > n_launch else rows
    t0 = rows[0]["start"]
    out = [f"rank {rank} of {world}: step {step_us:.0f} us by CUDA events over {replays} replays; {len(rows)} stamped launches "
           f"(top-k, NCCL and element-wise kernels between them are not stamped and show as gaps)"]
    if rank == 0:
        out.append("  # kind          ctas  start   gap-to-prev-end  prev-complete  flag-wait+staging  first-data  rows-done  tail   end   duration (us)")
    agg = {}
    prev_end = None
    for i, r in enumerate(rows):
        us = lambda x: (x - t0) / 1e3  # noqa: E731
        gap = (r["start"] - prev_end) / 1e3 if prev_end is not None else 0.0
        dur = (r["end"] - r["start"]) / 1e3
        tail = (r["end"] - r["rows_done"]) / 1e3
        if rank == 0 and i < 40:
            out.append(f"{i:3d} {r['kind']:13s} {r['ctas']:4d} {us(r['start']):7.1f} {gap:10.1f} {us(r['prev_done']) - us(r['start']):14.1f} "
                       f"{r['wait'] / 1e3:14.1f} {us(r['first']) - us(r['start']):14.1f} {us(r['rows_done']) - us(r['start']):10.1f} {tail:6.1f} "
                       f"{us(r['end']):7.1f} {dur:7.1f}")
        k = agg.setdefault(r["kind"], dict(n=0, dur=0.0, gap=0.0, wait=0.0, tail=0.0, first=0.0, prev=0.0))
        k["n"] += 1
        k["dur"] += dur
        k["gap"] += max(gap, 0.0)
        k["wait"] += r["wait"] / 1e3
        k["tail"] += tail
        k["first"] += (r["first"] - r["start"]) / 1e3
        k["prev"] += (r["prev_done"] - r["start"]) / 1e3
        prev_end = r["end"]
    span = (rows[-1]["end"] - t0) / 1e3
    out.append(f"rank {rank} summary: first start to last end {span:.0f} us; per kind: launches, mean duration, mean gap after the "
               "previous stamped kernel's end (negative gaps, i.e. overlap by dependent launch, counted as 0), mean time from start "
               "until the previous kernel had completed, mean flag-wait+staging, mean time to first data, mean tail after the rows")
    for kind, k in sorted(agg.items()):
        n = k["n"]
        out.append(f"  {kind:13s} n={n:3d} dur {k['dur'] / n:6.1f}  gap {k['gap'] / n:6.1f}  prev-complete {k['prev'] / n:6.1f}  "
                   f"wait+staging {k['wait'] / n:6.1f}  first-data {k['first'] / n:6.1f}  tail {k['tail'] / n:5.1f}  (sum dur {k['dur']:.0f}, sum gap {k['gap']:.0f}, sum wait {k['wait']:.0f})")
    text = "\n".join(out)
    if tp is not None:
        for r_ in range(world):
            if r_ == rank:
                print(text, flush=True)
            torch.distributed.barrier()
        runner.graph = None
        torch.cuda.synchronize()
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
        os._exit(0)
    print(text)


def prefill_case(ctx: int, reps: int, library: bool):
    """Causal prefill attention of one Llama-3-8B layer (32 query heads, 8 KV heads) over ``ctx`` tokens: this
    package's tcgen05 kernel (and, with --library, PyTorch's fused attention on the same tensors)."""
    import torch.nn.functional as F
    dev, H, KVH, d = "cuda", 32, 8, 128
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)  # noqa: E731
    q, k, v = rnd(1, H, ctx, d), rnd(1, KVH, ctx, d), rnd(1, KVH, ctx, d)
    flops = 4.0 * H * d * ctx * (ctx + 1) / 2  # two products over the causal triangle
    legs = [("tcgen05 kernel", lambda: ops.prefill_attn(q, k, v)),
            ("tcgen05 kernel, one query tile per CTA", lambda: ops.prefill_attn(q, k, v, variant=1))]
    if library:
        legs.append(("torch sdpa", lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)))
    outs = {}
    for name, fn in legs:
        outs[name] = fn()
        torch.cuda.synchronize()
        for r in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            print(f"prefill_attn {name} ctx {ctx} rep {r}: {ms:.3f} ms, {flops / ms / 1e9:.0f} TFLOP/s")
    ops.check_status(q.device)
    if library:
        a, b = outs["tcgen05 kernel"].float(), outs["torch sdpa"].transpose(1, 2).float()
        print(f"max |kernel - sdpa| = {(a - b).abs().max().item():.4f}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["dense_attn", "sparse_attn", "topk", "score_window", "offload_gather", "gemv", "operator",
                                     "tp_timeline", "prefill_attn", "batched_linear"])
    ap.add_argument("--tokens", type=int, default=16, help="batched_linear: sequences decoding together")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--ctx", type=int, default=131072)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--contiguous-idx", action="store_true", help="sparse_attn: select rows 0..k-1 instead of random ones")
    ap.add_argument("--batch", type=int, default=1, help="sparse_attn: sequences (2048 selected rows + 64 tail rows each)")
    ap.add_argument("--library", action="store_true", help="prefill_attn: also time PyTorch's fused attention")
    ap.add_argument("--kv-layout", default="interleaved", choices=["interleaved", "planes"],
                    help="dense_attn / score_window: K|V rows of a head interleaved, or in two separate runs of rows")
    args = ap.parse_args()
    if args.case == "tp_timeline":
        return tp_timeline(args.ctx)
    dev = "cuda"
    B, H, KVH, d, L = 1, 32, 8, 128, args.ctx
    k_sel = int(0.067 * L)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)  # noqa: E731
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)  # noqa: E731
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)  # 256 MB, larger than L2; READ between launches
    sink = torch.zeros(1, dtype=torch.float32, device=dev)

    if args.case == "gemv":
        return gemv_cases(args.reps)
    if args.case == "batched_linear":
        return batched_linear_cases(args.reps, args.tokens)
    if args.case == "prefill_attn":
        return prefill_case(args.ctx if args.ctx != 131072 else 16384, args.reps, args.library)
    if args.case == "operator":
        # the single-layer operator in fp32: context 16384, selector `last` on a filter layer's K, 1098 selected rows,
        # decode attention over a second layer's K/V at those rows -- three launches
        L, k_op = 16384, 1098
        f32 = lambda *s: torch.randn(*s, generator=g, device=dev, dtype=torch.float32)  # noqa: E731
        q, k1, k2, v2 = f32(B, H, d), f32(B, KVH, L, d), f32(B, KVH, L, d), f32(B, KVH, L, d)
        hot = torch.randperm(L, generator=g, device=dev)[: L // 50]
        qm = q.mean(dim=1)
        k1[:, :, hot] += 4.0 * (qm / qm.norm())[:, None, None, :]
        planes = torch.empty(KVH, B, L, dtype=torch.float32, device=dev)
        idx = torch.empty(B, k_op + 6, dtype=torch.int32, device=dev)
        cnt = torch.empty(B, dtype=torch.int32, device=dev)
        n_p, kk = i32([L]), i32([k_op])
        out = torch.empty(B, H, d, dtype=torch.float32, device=dev)

        def fn():
            ops.score_last(q, k1, n_p, score_out=planes)
            ops.topk(planes, n_p, kk, idx_out=idx, count_out=cnt, max_len=L)
            ops.decode_attn(q, k2, v2, cnt, idx=idx, out=out, max_rows=k_op)

        nbytes = KVH * d * 4 * L + 2 * KVH * d * 4 * k_op
    # K and V share one buffer as in the package's cache: head-major with K|V rows interleaved for a dense layer,
    # token-major for a sparse layer
    if args.case in ("dense_attn", "score_window"):
        if args.kv_layout == "planes":  # K and V of a head in separate runs of rows (a filter layer under a window selector)
            kv = rnd(B, KVH, 2, L + 64, d)
            kc, vc, q = kv[:, :, 0], kv[:, :, 1], rnd(B, H, d)
        else:                            # K and V rows of a head interleaved (every other dense layer)
            kv = rnd(B, KVH, L + 64, 2, d)
            kc, vc, q = kv[:, :, :, 0, :], kv[:, :, :, 1, :], rnd(B, H, d)
    if args.case == "sparse_attn" and args.batch > 1:  # the sparse layers of the batch-16 workload: 2048 rows + tail each
        B, L, k_sel = args.batch, 32768, 2048
    if args.case == "sparse_attn":
        kv = rnd(B, L + 64, KVH, 2, d)
        kc, vc, q = kv[:, :, :, 0, :].permute(0, 2, 1, 3), kv[:, :, :, 1, :].permute(0, 2, 1, 3), rnd(B, H, d)
    if args.case == "operator":
        pass
    elif args.case == "dense_attn":
        planes = torch.empty(KVH, B, L, dtype=torch.float32, device=dev)
        n_all, n_p = i32([L + 1]), i32([L])
        fn = lambda: ops.decode_attn(q, kc, vc, n_all, score_out=planes, score_len=n_p, n_splits=args.splits or None)  # noqa: E731
        nbytes = 2 * KVH * d * 2 * (L + 1)
    elif args.case == "sparse_attn":
        if args.contiguous_idx:  # the same number of rows, but neighbours in memory: separates the cost of scattered DRAM
            idx = torch.arange(k_sel, device=dev, dtype=torch.int32)[None].repeat(B, 1).contiguous()  # reads from the copies
        else:
            idx = torch.stack([torch.sort(torch.randperm(L, generator=g, device=dev)[:k_sel]).values.to(torch.int32)
                               for _ in range(B)]).contiguous()
        cnt, n_p, one = i32([k_sel] * B), i32([L] * B), i32([64 if B > 1 else 1] * B)
        fn = lambda: ops.decode_attn(q, kc, vc, cnt, idx=idx, k_tail=kc, v_tail=vc, tail_start=n_p, tail_len=one,  # noqa: E731
                                     max_rows=k_sel + 64, n_splits=args.splits or None)
        nbytes = 2 * KVH * d * 2 * (k_sel + (64 if B > 1 else 1)) * B
    elif args.case == "topk":
        planes = torch.randn(KVH, B, L, generator=g, device=dev)
        n_p, kk = i32([L]), i32([k_sel])
        idx = torch.empty(B, k_sel + 16, dtype=torch.int32, device=dev)
        cnt = torch.empty(B, dtype=torch.int32, device=dev)
        fn = lambda: ops.topk(planes, n_p, kk, idx_out=idx, count_out=cnt, max_len=L)  # noqa: E731
        nbytes = KVH * L * 4
    elif args.case == "score_window":
        qw = rnd(B, H, 16, d)
        n_p = i32([L])
        out = torch.empty(B, L, dtype=torch.float32, device=dev)
        fn = lambda: ops.score_window(qw, kc, n_p, "exp", max_len=L, score_out=out)  # noqa: E731
        nbytes = 2 * KVH * d * 2 * L
    else:
        layers, n = 12, int(0.067 * 450000)
        tokens = 450000 if L == 131072 else L
        host = torch.empty(tokens, layers, 2, KVH, d, dtype=torch.bfloat16).pin_memory()
        host.view(torch.int16).random_(0, 1000)
        idx = torch.sort(torch.randperm(tokens, generator=g, device=dev)[:n]).values.to(torch.int32).contiguous()
        staged = torch.zeros(layers, 2, KVH, n, d, dtype=torch.bfloat16, device=dev)
        cnt = i32([n])
        fn = lambda: ops.offload_gather(host, idx, cnt, staged)  # noqa: E731
        nbytes = n * layers * 2 * KVH * d * 2

    fn()
    torch.cuda.synchronize()
    # timed inside a CUDA graph (L2 flush, then the launch) so that the host's launch cost does not show
    g = torch.cuda.CUDAGraph()
    ev = [torch.cuda.Event(enable_timing=True, external=True) for _ in range(2)]
    with torch.cuda.graph(g):
        torch.sum(flush, dim=0, keepdim=True, out=sink)  # evicts L2 with clean lines (a write flush would leave
        # dirty lines whose write-back then competes with the measured kernel)
        ev[0].record()
        fn()
        ev[1].record()
    for r in range(args.reps):
        g.replay()
        torch.cuda.synchronize()
        ms = ev[0].elapsed_time(ev[1])
        print(f"{args.case} rep {r}: {ms * 1e3:.1f} us, {nbytes / 1e6:.1f} MB algorithmic, {nbytes / ms / 1e6:.0f} GB/s")


if __name__ == "__main__":
    main()
