"""Small stand-alone launches of each kernel at the benchmark's shapes, for profilers:

    python profile_cases.py dense_attn [--reps 3] [--ctx 131072]
    ncu --set full --clock-control none -k regex:decode_attn_mma -c 3 python profile_cases.py dense_attn

Cases: dense_attn (filter layer: K and V of 8 KV heads x ctx rows, fused scores), sparse_attn
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["dense_attn", "sparse_attn", "topk", "score_window", "offload_gather", "gemv", "operator"])
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--ctx", type=int, default=131072)
    ap.add_argument("--splits", type=int, default=0)
    args = ap.parse_args()
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
        kv = rnd(B, KVH, L + 64, 2, d)
        kc, vc, q = kv[:, :, :, 0, :], kv[:, :, :, 1, :], rnd(B, H, d)
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
        idx = torch.sort(torch.randperm(L, generator=g, device=dev)[:k_sel]).values.to(torch.int32)[None].contiguous()
        cnt, n_p, one = i32([k_sel]), i32([L]), i32([1])
        fn = lambda: ops.decode_attn(q, kc, vc, cnt, idx=idx, k_tail=kc, v_tail=vc, tail_start=n_p, tail_len=one,  # noqa: E731
                                     max_rows=k_sel + 64, n_splits=args.splits or None)
        nbytes = 2 * KVH * d * 2 * (k_sel + 1)
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
