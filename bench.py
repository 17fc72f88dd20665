"""Decode throughput of OmniKV selection + sparse decode on a random-init Llama-3-8B at 128K context.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one greedy decode step (one token per sequence) through all 32 layers: 8 dense layers
(3 of them filter layers that emit selection scores and run the top-k), 24 sparse layers reading the
selected 8781 prompt rows + the decode-time tail.  The prompt is 131072 uniform-random token ids, prefilled
through the model before the timed region (PyTorch SDPA; --synthetic-kv fills the cache with seeded N(0,1)
values instead); weights are seeded N(0, 0.02) bf16.  Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CTX = 131072
OMNI = dict(model_cls="multi", cache_cls="multi", do_select_layers="2,8,18", num_wait_load_layers=1,
            real_offload=False, dense_more=True, num_of_selected_tokens=0.067, selector_cls="last", window_size=16)
WORKLOAD = "llama3-8b bf16, batch 1, ctx 131072, greedy decode, OmniKV 2,8,18 / wait 1 / 0.067 / last"


def measured_peak_gbs():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU baseline: the oracle (a port of the reference's CPU-runnable path) on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_baseline_sample(threads: int, seed: int = 0):
    """Times, on the host, the oracle's restatement of one decode step's pieces at the benchmark's
    sizes -- one filter layer (dense attention + selector ``last`` + top-k), one sparse layer (index_select
    gather of k rows + attention over them), one layer's weight GEMVs and the lm_head -- each ONCE, and
    scales by the step's layer counts (8 dense of which 3 filter, 24 sparse, 32 layers of GEMVs)."""
    import oracle

    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(seed)
    H, KVH, d, L, hidden, inter, vocab = 32, 8, 128, CTX, 4096, 14336, 128256
    k = int(0.067 * L)
    kc = torch.randn(1, KVH, L, d, generator=g).to(torch.bfloat16)
    vc = torch.randn(1, KVH, L, d, generator=g).to(torch.bfloat16)
    q = torch.randn(1, H, d, generator=g).to(torch.bfloat16)
    t = {}
    t0 = time.perf_counter()
    oracle.dense_attention(q, kc, vc)
    t["dense_attn"] = time.perf_counter() - t0
    t0 = time.perf_counter()
    s = oracle.score_last(q, kc, L)
    idx = oracle.topk_ascending(s, k)
    t["select"] = time.perf_counter() - t0
    t0 = time.perf_counter()
    oracle.sparse_attention(q, kc, vc, idx, kc[:, :, :1], vc[:, :, :1])
    t["sparse_attn"] = time.perf_counter() - t0
    x = torch.randn(1, hidden, generator=g).to(torch.bfloat16)
    ws = [torch.randn(n, m, generator=g).to(torch.bfloat16) for n, m in
          ((6144, hidden), (hidden, hidden), (2 * inter, hidden))]
    wd = torch.randn(hidden, inter, generator=g).to(torch.bfloat16)
    xi = torch.randn(1, inter, generator=g).to(torch.bfloat16)
    t0 = time.perf_counter()
    for w in ws:
        torch.nn.functional.linear(x, w)
    torch.nn.functional.linear(xi, wd)
    t["layer_gemv"] = time.perf_counter() - t0
    wl = torch.randn(vocab, hidden, generator=g).to(torch.bfloat16)
    t0 = time.perf_counter()
    torch.nn.functional.linear(x, wl)
    t["lm_head"] = time.perf_counter() - t0
    step = 8 * t["dense_attn"] + 3 * t["select"] + 24 * t["sparse_attn"] + 32 * t["layer_gemv"] + t["lm_head"]
    return step, t


_REAL_STDOUT = None


def quiet_stdout():
    """Everything libraries print on stdout (NCCL's version banner, for one) goes to stderr from here on; the one
    JSON line is written to the real stdout by emit()."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line: dict) -> None:
    out = _REAL_STDOUT or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def run_reference_arm(args):
    """The reference's CPU-runnable path (oracle port) with every host thread, as its own bench arm."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_baseline_sample(threads)
    times = [cpu_baseline_sample(threads, seed=i)[0] for i in range(max(1, min(args.steps, 3)))]
    step = statistics.median(times)
    sample = ("per step: 1 filter layer (dense attention + selector last + top-k), 1 sparse layer, 1 layer of weight "
              "GEMVs, lm_head timed once each at full size on the host, scaled by 8 dense / 3 filter / 24 sparse / 32 layers")
    line = {
        "impl": "reference", "metric": "decode tokens/s at 128K ctx (Llama-3-8B shape)", "value": 1.0 / step,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": len(times), "warmup": min(args.warmup, 1),
        "ms_per_step": step * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": {"workload": WORKLOAD, "batch": 1, "seq_len": CTX},
        "cpu_baseline": {"value": 1.0 / step, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": 1.0 / step, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ctx", type=int, default=CTX, help="prompt length (the benchmark's is 131072)")
    ap.add_argument("--layers", type=int, default=32, help="decoder layers (the benchmark's is 32)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--synthetic-kv", action="store_true", help="fill the prompt KV with seeded N(0,1) values instead of "
                    "prefilling a prompt of uniform-random token ids through the model (about 7 s at 128K on one GPU)")
    ap.add_argument("--chain", action="store_true", help="run the weight-streaming phases between two attention calls "
                    "as one cooperative multi-phase launch instead of one launch per phase (measured slower so far)")
    ap.add_argument("--nccl-allreduce", action="store_true", help="multi-GPU: NCCL all-reduce after the row-parallel "
                    "projections instead of the fused peer-memory exchange")
    ap.add_argument("--profile-step", action="store_true",
                    help="after the warm-up, run ONE step between cudaProfilerStart/Stop and exit (for ncu "
                         "--profile-from-start off); prints no benchmark line")
    args = ap.parse_args()
    quiet_stdout()
    if args.impl == "reference":
        return run_reference_arm(args)

    from omnikv_b200 import ops
    from omnikv_b200.modeling import LlamaCompressorConfig, OmniKVMulLM
    from omnikv_b200.modeling.omnikv import DecodeRunner
    from omnikv_b200 import parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    tp = parallel.init(world, rank, dev) if world > 1 else None
    if tp is not None and not args.nccl_allreduce:
        tp.enable_peer_exchange(4096, dev)

    warmup = max(3, args.warmup)
    cfg = LlamaCompressorConfig(num_hidden_layers=args.layers)
    cfg.set_config_of_compressor(**OMNI)
    cfg.set_config_of_compressor(fused_decode=True, chained_decode=args.chain)
    lm = OmniKVMulLM.from_config(cfg, dtype=torch.bfloat16, device=dev, seed=0, tp=tp)
    graph_warm = 2
    reserve = graph_warm + 2 * (warmup + args.steps) + 16
    kvh_local = cfg.num_key_value_heads // (world if tp else 1)
    prefill_s = None
    if not args.synthetic_kv:
        cache = lm.new_cache()
        cache.reserve = reserve
        gen = torch.Generator(device=dev).manual_seed(3)  # the same prompt on every rank
        ids = torch.randint(0, cfg.vocab_size, (1, args.ctx), generator=gen, device=dev)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = lm(input_ids=ids, past_key_values=cache)
        torch.cuda.synchronize()
        prefill_s = time.perf_counter() - t0
        first = out.logits[:, -1].argmax(-1, keepdim=True)
        del out, ids
    else:
        cache = lm.new_cache().init_synthetic(1, kvh_local, cfg.head_dim, [args.ctx], torch.bfloat16, dev,
                                              seed=1 + rank, reserve=reserve)
        first = torch.tensor([[1]], device=dev)
    total = graph_warm + 2 * (warmup + args.steps) + 2
    runner = DecodeRunner(lm, None, cache=cache, first_token=first, max_new_tokens=total,
                          use_cuda_graph=not args.no_graph, warmup_steps=graph_warm)

    def barrier():
        if tp is not None:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput -------------------------------------------------------------
    runner.run(warmup)
    barrier()
    if args.profile_step:
        torch.cuda.profiler.start()
        runner.run(1)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        return
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    runner.run(args.steps)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)

    # ---- end to end: token in from pinned host memory, logits + next token back to the host ------
    h_tok = torch.ones(1, 1, dtype=torch.int64).pin_memory()
    h_next = torch.zeros(1, 1, dtype=torch.int64).pin_memory()
    h_logits = torch.zeros(1, cfg.vocab_size, dtype=torch.float32).pin_memory()

    def e2e_step():
        runner.token.copy_(h_tok, non_blocking=True)
        runner.run(1)
        h_next.copy_(runner.token, non_blocking=True)
        h_logits.copy_(runner.logits, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        h_tok.copy_(h_next)

    for _ in range(warmup):
        e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        e2e_step()
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None

    if tp is not None:
        t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms, ms_e2e = t.tolist()

    # ---- roofline of the dominant kernel: dense decode attention, timed live on its stream -------
    dense_layers = [i for i, s in cache.layer_state.items() if not s[0]]
    q = torch.randn(1, cfg.num_attention_heads // (world if tp else 1), cfg.head_dim, device=dev).to(torch.bfloat16)
    # The dense layers' attention calls are captured in a CUDA graph (as they are in the timed step) and
    # bracketed by events on the launching stream, so the host's launch cost is not part of the duration; the
    # launches read 8 x 537 MB of distinct K/V, far more than L2 holds.
    for layer in dense_layers:
        cache.attend(q, layer)
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True, external=True) for _ in range(2)]
    g_att = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g_att):
        ev[0].record()
        for layer in dense_layers:
            cache.attend(q, layer)
        ev[1].record()
    durs = []
    for rep in range(4):
        g_att.replay()
        torch.cuda.synchronize()
        if rep > 0:
            durs.append(ev[0].elapsed_time(ev[1]) / len(dense_layers))
    rows = cache._seen_tokens
    alg_bytes = 2 * kvh_local * cfg.head_dim * 2 * rows  # K and V rows of every local KV head, read once
    dur_ms = statistics.mean(durs)
    peak, peak_kind = measured_peak_gbs()
    achieved = alg_bytes / (dur_ms * 1e-3) / 1e9
    # DRAM bytes per (row, KV head) of this kernel from the ncu capture summarised in profiles/decode_attn_dense.md
    # (dram__bytes_read + dram__bytes_write = 545.06 MB for 131073 rows x 8 KV heads), scaled to this launch
    traffic = 519.2 * rows * kvh_local
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "kernel": "decode_attn_mma_kernel (dense layer: TMA tensor-map tiles, split-K, merge by the last CTA)",
                "algorithmic_bytes_per_launch": alg_bytes, "launch_ms": dur_ms, "peak_kind": peak_kind}

    # whole-step algorithmic bytes (KV + weights) for context
    n_params_local = sum(p.numel() for p in lm.parameters())
    step_bytes = (len(dense_layers) * alg_bytes + (cfg.num_hidden_layers - len(dense_layers)) * 2 * kvh_local * 256 *
                  (int(0.067 * args.ctx) + runner.steps_done) + 2 * (n_params_local - cfg.vocab_size * cfg.hidden_size))
    step_gbs = step_bytes / (ms / args.steps * 1e-3) / 1e9

    def finish():
        """Leave in step on every rank: drop the captured graph, sync, barrier, destroy the group, then exit
        without running interpreter-exit hooks (NCCL teardown after a captured graph has hung there)."""
        sys.stdout.flush()
        if tp is None:
            return
        runner.graph = None
        torch.cuda.synchronize()
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
        sys.stderr.flush()
        os._exit(0)

    if rank != 0:
        return finish()
    line = {
        "metric": "decode tokens/s at 128K ctx (Llama-3-8B shape)", "value": args.steps / (ms * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch": 1, "seq_len": args.ctx, "layers": args.layers,
                   "parallelism": (f"kv-head tp{world}, " + ("fused peer-memory all-reduce" if tp.exchange is not None
                                                                    else "nccl all-reduce")) if world > 1 else "single gpu",
                   "l2": "inputs larger than L2 (about 20 GB of KV and weights are read per step)",
                   "cuda_graph": not args.no_graph,
                   "kv_fill": (f"real prefill of {args.ctx} uniform-random token ids ({prefill_s:.1f} s)" if prefill_s
                               else "seeded N(0,1), no prefill run")},
        "clocks": clocks,
        "e2e": {"value": args.steps / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 8,
                "d2h_bytes_per_step": 8 + cfg.vocab_size * 4, "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": runner.launches_per_step * args.steps,
        "roofline": roofline,
        "whole_step": {"algorithmic_bytes": step_bytes, "achieved_gbs": step_gbs, "frac_of_peak": step_gbs / peak},
    }
    if world == 1 and not args.no_cpu_baseline:
        threads = min(os.cpu_count() or 1, 8)  # the reference's cpu_num_threads default is 8 (configs/example.json)
        step_s, parts = cpu_baseline_sample(threads)
        line["cpu_baseline"] = {
            "value": 1.0 / step_s, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": "one filter layer, one sparse layer, one layer of weight GEMVs and the lm_head timed once each at "
                      "full size, scaled by the step's layer counts (8 dense / 3 filter / 24 sparse / 32)",
            "parts_s": parts}
    emit(line)
    finish()


if __name__ == "__main__":
    main()
