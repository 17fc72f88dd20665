"""Run the batched (window selector), the offload and the 70B-shape tensor-parallel decode workloads with
synthetic inputs:

    python -m omnikv_b200.run_config batch16   [--steps 64]     # batch 16, contexts U[16384, 32768], selector exp, k = 2048
    python -m omnikv_b200.run_config offload   [--steps 32]     # batch 1, context 450000, real_offload (pinned host KV)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29520 \
        -m omnikv_b200.run_config tp70b [--steps 64]             # Llama-3-70B shape, batch 8, context 65536, KV-head TP

Random-init Llama-3-8B (bf16; tp70b: 80 layers, hidden 8192, 64 query / 8 KV heads, FFN 28672, every rank holding
its shard), KV cache filled with seeded N(0,1) rows, greedy decoding captured in a CUDA graph.
Prints one JSON line with tokens/s, ms/step and the algorithmic bytes moved per step (HBM, and host link for
the offload run).
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch

from . import ops
from .modeling import LlamaCompressorConfig, OmniKVMulLM
from .modeling.omnikv import DecodeRunner


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("workload", choices=["batch16", "offload", "tp70b"])
    ap.add_argument("--steps", type=int, default=0)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--ctx", type=int, default=0, help="override the context length (offload: 450000)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--nccl-allreduce", action="store_true", help="tp70b: NCCL instead of the peer-memory all-reduce")
    ap.add_argument("--profile-step", action="store_true",
                    help="after the warm-up run ONE step between cudaProfilerStart/Stop and exit (for a launch list)")
    ap.add_argument("--skip-threshold", type=float, default=None,
                    help="offload: use cache_cls lazy with this threshold (0 keeps the first selection for good: "
                         "the step time without host-link traffic)")
    args = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    tp = None
    if world > 1:
        from . import parallel
        tp = parallel.init(world, rank, dev)
        if not args.nccl_allreduce:
            tp.enable_peer_reduce(8 * 8192 * 2, dev)  # a batch-8 hidden state of the 70B shape in bf16
    if args.workload == "tp70b":
        cfg = LlamaCompressorConfig(num_hidden_layers=80 if args.layers == 32 else args.layers, hidden_size=8192,
                                    intermediate_size=28672, num_attention_heads=64, num_key_value_heads=8)
    else:
        cfg = LlamaCompressorConfig(num_hidden_layers=args.layers)
    base = dict(model_cls="multi", cache_cls="multi", do_select_layers="2,8,18", num_wait_load_layers=1, dense_more=True,
                window_size=16)
    g = torch.Generator().manual_seed(0)
    if args.workload == "batch16":
        steps = args.steps or 64
        B = 16
        lens = torch.randint(16384, 32769, (B,), generator=g).tolist()
        cfg.set_config_of_compressor(**base, real_offload=False, selector_cls="exp", num_of_selected_tokens=2048)
    elif args.workload == "tp70b":
        steps = args.steps or 64
        B = 8
        lens = [args.ctx or 65536] * B
        base["do_select_layers"] = "5,20,45"
        cfg.set_config_of_compressor(**base, real_offload=False, selector_cls="last", num_of_selected_tokens=0.067)
    else:
        steps = args.steps or 32
        B, lens = 1, [args.ctx or 450000]
        if args.skip_threshold is not None:
            base.update(cache_cls="lazy", skip_threshold=args.skip_threshold)
        cfg.set_config_of_compressor(**base, real_offload=True, selector_cls="last", num_of_selected_tokens=0.067)
    lm = OmniKVMulLM.from_config(cfg, dtype=torch.bfloat16, device=dev, seed=0, tp=tp)
    total = 2 + args.warmup + steps + 2
    t0 = time.perf_counter()
    kvh_local = cfg.num_key_value_heads // world
    cache = lm.new_cache().init_synthetic(B, kvh_local, cfg.head_dim, lens, torch.bfloat16, dev, seed=1 + rank,
                                          reserve=total + 16)
    torch.cuda.synchronize()
    fill_s = time.perf_counter() - t0
    lm.prepare_synthetic_decode(B, seed=2)
    first = torch.ones(B, 1, dtype=torch.int64, device=dev)
    runner = DecodeRunner(lm, None, cache=cache, first_token=first, max_new_tokens=total,
                          use_cuda_graph=not args.no_graph, warmup_steps=2)
    runner.run(args.warmup)
    torch.cuda.synchronize()
    if args.profile_step:
        torch.cuda.profiler.start()
        runner.run(1)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        return
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    runner.run(steps)
    e1.record()
    torch.cuda.synchronize()
    ops.check_status(dev)
    ms = e0.elapsed_time(e1) / steps
    if tp is not None:  # the job's time is the slowest rank's
        t = torch.tensor([ms], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
    # algorithmic bytes per step (whole job, all ranks)
    dense = [i for i, s in cache.layer_state.items() if not s[0]]
    n_sparse = cfg.num_hidden_layers - len(dense)
    row = cfg.num_key_value_heads * cfg.head_dim * 2 * 2  # K + V bytes per token per layer
    k0 = [2048 if args.workload == "batch16" else int(0.067 * n) for n in lens]
    hbm = sum(len(dense) * row * n + n_sparse * row * k for n, k in zip(lens, k0))
    if args.workload == "batch16":
        hbm += 3 * sum(lens) * row // 2  # the window selectors read the filter layers' K a second time
    weights = 2 * world * sum(p.numel() for n_, p in lm.named_parameters() if "embed_tokens" not in n_ and p.dim() > 1)
    link = n_sparse * row * k0[0] if args.workload == "offload" else 0
    regathers = None
    if args.skip_threshold is not None and args.workload == "offload":
        # selections that replaced the one in use during the last step, out of the filter groups
        regathers = sum(cache.lazy_state(sel)["applied"][0] for sel in cache.groups)
        if regathers == 0:
            link = 0
    line = {"workload": args.workload, "batch": B, "context": lens if B > 1 else lens[0], "steps": steps,
            "ms_per_step": ms, "tokens_per_s": B * 1e3 / ms, "kv_bytes_per_step": hbm, "weight_bytes_per_step": weights,
            "hbm_gbs": (hbm + weights + link) / ms / 1e6, "host_link_bytes_per_step": link,
            "host_link_gbs": link / ms / 1e6 if link else None, "kv_fill_s": fill_s, "cuda_graph": not args.no_graph,
            "selector": cfg.selector_cls, "launches_per_step": runner.launches_per_step,
            "cache_cls": cfg.get("cache_cls"), "regathers_last_step": regathers}
    line["n_gpus"] = world
    line["allreduce"] = None if tp is None else ("peer memory" if tp.reducer is not None else "nccl")
    if rank == 0:
        print(json.dumps(line), flush=True)
    if tp is not None:  # leave in step: drop the graph, sync, barrier, destroy the group, exit without teardown hooks
        runner.graph = None
        torch.cuda.synchronize()
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
        os._exit(0)


if __name__ == "__main__":
    main()
