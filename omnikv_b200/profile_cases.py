"""Small stand-alone launches of each kernel at the benchmark's shapes, for profilers:

    python -m omnikv_b200.profile_cases dense_attn [--reps 3] [--ctx 131072]
    ncu --set full --clock-control none -k regex:decode_attn_mma -c 3 python -m omnikv_b200.profile_cases dense_attn

Cases: dense_attn (filter layer: K and V of 8 KV heads x ctx rows, fused scores), sparse_attn
(8781 selected rows + tail), topk (ctx scores, 8 planes), score_window (16-slot window, exp),
offload_gather (30150 tokens x 12 layers from pinned host memory).  Each prints the CUDA-event time per launch.
"""
from __future__ import annotations

import argparse

import torch

from . import ops


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["dense_attn", "sparse_attn", "topk", "score_window", "offload_gather"])
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
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than L2

    if args.case in ("dense_attn", "sparse_attn", "score_window"):
        kc, q = rnd(B, KVH, L + 64, d), rnd(B, H, d)
    if args.case == "dense_attn":
        vc = rnd(B, KVH, L + 64, d)
        planes = torch.empty(KVH, B, L, dtype=torch.float32, device=dev)
        n_all, n_p = i32([L + 1]), i32([L])
        fn = lambda: ops.decode_attn(q, kc, vc, n_all, score_out=planes, score_len=n_p, n_splits=args.splits or None)  # noqa: E731
        nbytes = 2 * KVH * d * 2 * (L + 1)
    elif args.case == "sparse_attn":
        vc = rnd(B, KVH, L + 64, d)
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
    for r in range(args.reps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        print(f"{args.case} rep {r}: {ms * 1e3:.1f} us, {nbytes / 1e6:.1f} MB algorithmic, {nbytes / ms / 1e6:.0f} GB/s")


if __name__ == "__main__":
    main()
