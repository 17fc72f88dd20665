"""Decode throughput of OmniKV selection + sparse decode on a random-init Llama-3-8B at 128K context.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workloads (``--workload``): ``decode128k`` (default; the benchmark: batch 1, context 131072, selector ``last``,
filter layers 2,8,18, one wait layer, 6.7 % of the prompt selected), ``batch16`` (batch 16, contexts U[16384, 32768],
selector ``exp``, window 16, k = 2048), ``offload`` (batch 1, context 450000, ``real_offload``), ``tp70b``
(Llama-3-70B shape, batch 8, context 65536, filter layers 5,20,45, KV-head tensor parallelism).

One "step" is one greedy decode step (one token per sequence) through every layer.  ``decode128k`` prefills a prompt
of uniform-random token ids through the model before the timed region (``--synthetic-kv`` fills the cache with
seeded N(0,1) values instead, as the other workloads always do); weights are seeded N(0, 0.02) bf16.  Prints ONE JSON
line (rank 0).
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
WORKLOADS = {
    "decode128k": "llama3-8b bf16, batch 1, ctx 131072, greedy decode, OmniKV 2,8,18 / wait 1 / 0.067 / last",
    "batch16": "llama3-8b bf16, batch 16, ctx U[16384,32768], greedy decode, OmniKV 2,8,18 / wait 1 / k 2048 / exp, window 16",
    "offload": "llama3-8b bf16, batch 1, ctx 450000, greedy decode, OmniKV 2,8,18 / wait 1 / 0.067 / last, real_offload",
    "tp70b": "llama3-70b shape bf16, batch 8, ctx 65536, greedy decode, OmniKV 5,20,45 / wait 1 / 0.067 / last, kv-head TP",
}
METRIC = "decode tokens/s at 128K ctx (Llama-3-8B shape)"


def measured_peak_gbs():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs (read-only query)."""

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


def config_block(args, world: int) -> dict:
    """The ``config`` object of the JSON line: identical from both arms for the same command line."""
    return {"workload": WORKLOADS[args.workload], "batch": {"batch16": 16, "tp70b": 8}.get(args.workload, 1),
            "seq_len": args.ctx, "layers": args.layers,
            "parallelism": f"kv-head tp{world}" if world > 1 else "single gpu",
            "l2": "inputs larger than L2 (tens of GB of KV and weights are read per step)"}


# ------------------------------------------------------------------------------------------------
# the reference arm and the CPU baseline: the path's CPU implementation on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_baseline_block(threads: int, all_threads: int, steps: int = 3):
    """``cpu_baseline`` of our arm (rank 0, one GPU): a bounded sample of the decode step on ``threads`` host threads
    (the reference's ``cpu_num_threads`` default) in tokens/s, plus the operator case stage by stage on ``threads``
    and on every host thread."""
    from oracle import cpu_baseline as cb
    torch.set_num_threads(threads)
    sample = cb.StepSample(CTX)
    sample.run()
    runs = [sample.run() for _ in range(steps)]
    step_s = statistics.median(r[0] for r in runs)
    op = [cb.operator_case_stats(threads)]
    if all_threads != threads:
        op.append(cb.operator_case_stats(all_threads))
    return {"value": 1.0 / step_s, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": sample.sample + f"; median of {steps} samples after one warm-up",
            "parts_s": runs[len(runs) // 2][1],
            "operator_case": {"what": "single-layer operator (fp32, ctx 16384, selector last, k 1098): score + top-k, gather "
                                      "of the second layer's rows, update + attention; 3 warm-ups, 20 repetitions",
                              "kind": op[0]["kind"], "runs": op}}


def run_reference_arm(args):
    """``--impl reference``: the CPU implementation of the path, with every host thread, as its own bench arm.  The
    reference is pure Python whose model classes need transformers 4.41.2 and flash-attn, so what runs here is the
    restatement in ``oracle/`` (kind "port"); each step is a bounded sample of the decode step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import cpu_baseline as cb
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    sample = cb.StepSample(args.ctx)
    for _ in range(args.warmup):
        sample.run()
    times = [sample.run()[0] for _ in range(args.steps)]
    step = statistics.median(times)
    line = {
        "impl": "reference", "metric": METRIC, "value": 1.0 / step, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_block(args, args.gpus),
        "cpu_baseline": {"value": 1.0 / step, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample.sample},
        "e2e": {"value": 1.0 / step, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


# ------------------------------------------------------------------------------------------------
# the reference's op sequence in PyTorch on the same GPU (one filter layer, one sparse layer)
# ------------------------------------------------------------------------------------------------
def gpu_torch_baseline(cache, q, dev, reps: int = 3):
    """What the reference runs on a GPU for one filter layer and one sparse layer of the decode step, in bf16 torch
    ops on the same device and the same cache contents, next to this package's launches for the same layers.

    Filter layer: ``cat`` re-copy of the dense cache (modeling/spec_cache.py:363-369), ``repeat_kv`` + matmul + max over
    heads + ``topk`` + ``sort`` (modeling/omnikv.py:37-48, :109), attention over the whole cache.  Sparse layer:
    ``index_select`` of K and V at the selected rows (modeling/spec_cache.py:297-303), ``cat`` with the tail (:349-356),
    attention over them.  CUDA-event times per layer, median of ``reps`` after one warm-up."""
    import math
    import torch.nn.functional as F
    from omnikv_b200 import ops
    f_layer = min(cache.groups)                 # a filter layer
    s_layer = cache.groups[f_layer][0]          # a sparse layer of its group
    P, n = cache.prefill_len, cache._seen_tokens
    H, KVH, d = q.shape[1], cache._k[f_layer].shape[1], q.shape[2]
    G = H // KVH
    Kf = cache._k[f_layer][:, :, :n - 1].contiguous()
    Vf = cache._v[f_layer][:, :, :n - 1].contiguous()
    Ks = cache._k[s_layer][:, :, :P].contiguous()
    Vs = cache._v[s_layer][:, :, :P].contiguous()
    k_new, v_new = Kf[:, :, -1:].clone(), Vf[:, :, -1:].clone()
    tail_k, tail_v = Ks[:, :, : n - P].clone(), Vs[:, :, : n - P].clone()
    k_sel = int(cache.sel_state[f_layer].k0[0].item())
    q4 = q[:, :, None, :]

    def repeat_kv(x):
        b, kvh, s, dd = x.shape
        return x[:, :, None].expand(b, kvh, G, s, dd).reshape(b, kvh * G, s, dd)

    def torch_filter():
        K2, V2 = torch.cat([Kf, k_new], dim=-2), torch.cat([Vf, v_new], dim=-2)
        sc = torch.matmul(q4, repeat_kv(K2[:, :, :P]).transpose(2, 3)) / math.sqrt(d)
        score = sc[:, :, -1, :].max(dim=1).values
        idx = torch.topk(score, k_sel, dim=-1, sorted=True).indices
        idx = torch.sort(idx, dim=-1).values
        o = F.scaled_dot_product_attention(q4, repeat_kv(K2), repeat_kv(V2))
        return idx, o

    idx, _ = torch_filter()

    def torch_sparse():
        pk, pv = torch.index_select(Ks, 2, idx.view(-1)), torch.index_select(Vs, 2, idx.view(-1))
        kk, vv = torch.cat([pk, tail_k], dim=-2), torch.cat([pv, tail_v], dim=-2)
        return F.scaled_dot_product_attention(q4, repeat_kv(kk), repeat_kv(vv))

    st = cache.sel_state[f_layer]

    def ours_filter():
        cache.attend(q, f_layer, score_out=st.planes, score_len=cache.prefill_len_dev)
        ops.topk(st.planes, cache.prefill_len_dev, st.k0, idx_out=st.idx, count_out=st.count, max_len=st.max_len)

    def ours_sparse():
        cache.attend(q, s_layer)

    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)  # 256 MB read between launches: evicts L2
    sink = torch.zeros(1, dtype=torch.float32, device=dev)

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            torch.sum(flush, dim=0, keepdim=True, out=sink)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return statistics.median(ts)

    res = {"torch_filter_layer_us": timed(torch_filter), "ours_filter_layer_us": timed(ours_filter),
           "torch_sparse_layer_us": timed(torch_sparse), "ours_sparse_layer_us": timed(ours_sparse)}
    res["filter_layer_speedup"] = res["torch_filter_layer_us"] / res["ours_filter_layer_us"]
    res["sparse_layer_speedup"] = res["torch_sparse_layer_us"] / res["ours_sparse_layer_us"]
    res["what"] = ("the reference's op sequence (cat re-copy, repeat_kv + matmul + max + topk + sort, index_select, cat, "
                   "attention through torch SDPA) in bf16 on this GPU and cache vs this package's launches for the same "
                   "layer; eager launches, L2 evicted before each, median of %d" % reps)
    return res


# ------------------------------------------------------------------------------------------------
# multi-GPU self-check: the sharded model against the unsharded one built on rank 0
# ------------------------------------------------------------------------------------------------
def tp_parity_check(lm, cfg_factory, tp, dev, rank, ctx: int = 8192, steps: int = 4):
    """Before the timed region of a multi-GPU run: the sharded model (the fused peer-exchange path when it is on)
    against the UNSHARDED model (same seed: the shards are slices of its weights) built on rank 0.

    Rank 0 prefills ``ctx`` tokens through the unsharded model and broadcasts the prompt's K/V; every rank's cache
    takes over its KV heads of it, so both models decode from identical prompts.  Then ``steps`` teacher-forced
    decode steps (the unsharded model's greedy tokens) through both.  Two depths:

    * ``depth2``: both models cut to their first two layers.  The exchange arithmetic is exercised at full width
      and the bound is the 16-bit one, 2e-2.
    * ``full_depth``: all layers.  Sums taken in another order differ in the last fp32 bit; each 16-bit rounding
      that such a difference flips is a 0.4 % change of that element, which flips more roundings downstream, so
      within a few layers two 16-bit runs that differ ONLY in summation order carry independent rounding noise.
      The figure is therefore reported next to a noise floor measured the same way on ONE GPU: the unsharded
      model against itself with the attention split count changed (nothing else)."""
    from types import SimpleNamespace
    import torch.distributed as dist
    from omnikv_b200 import ops
    from omnikv_b200.modeling import OmniKVMulLM
    cfg = lm.config
    gen = torch.Generator(device=dev).manual_seed(11)
    ids = torch.randint(0, cfg.vocab_size, (1, ctx), generator=gen, device=dev)
    lo, hi = tp.shard(cfg.num_key_value_heads)
    full = OmniKVMulLM.from_config(cfg_factory(), dtype=torch.bfloat16, device=dev, seed=0, tp=None) if rank == 0 else None

    def compare(model_s, model_f, n_layers, floor=False):
        """Teacher-forced decode of (sharded or second unsharded) model_s against model_f on rank 0."""
        tok = torch.zeros(1, 1, dtype=torch.int64, device=dev)
        cache_f = None
        if rank == 0:
            out_f = model_f(input_ids=ids)
            cache_f = out_f.past_key_values
            cache_f.stage = "decoding"
            tok = out_f.logits[:, -1].argmax(-1, keepdim=True)
            del out_f
        if not floor:  # the noise floor runs on rank 0 alone: no collective in that mode
            dist.broadcast(tok, src=0)
        buf = torch.empty(2, 1, cfg.num_key_value_heads, ctx, cfg.head_dim, dtype=torch.bfloat16, device=dev)
        keys, vals = [], []
        for layer in range(n_layers):
            if rank == 0:
                buf[0].copy_(cache_f._k[layer][:, :, :ctx])
                buf[1].copy_(cache_f._v[layer][:, :, :ctx])
            if not floor:
                dist.broadcast(buf, src=0)
                keys.append(buf[0, :, lo:hi].clone())
                vals.append(buf[1, :, lo:hi].clone())
            elif rank == 0:
                keys.append(buf[0].clone())
                vals.append(buf[1].clone())
        diff, same, overlap = 0.0, True, 1.0
        if floor and rank != 0:
            return None
        cache_s = model_s.new_cache(SimpleNamespace(key_cache=keys, value_cache=vals, _seen_tokens=ctx))
        cache_s.stage = "decoding"
        del keys, vals, buf
        for _ in range(steps):
            if floor:
                real = ops.default_splits
                ops.default_splits = lambda *a, **k: 2 * real(*a, **k)   # the only change: twice the attention splits
                try:
                    logits_s, _ = model_s._decode_step(tok, cache_s)
                finally:
                    ops.default_splits = real
            else:
                logits_s, _ = model_s._decode_step(tok, cache_s)
            logits_s = logits_s.clone()
            if rank == 0:
                logits_f, nxt = model_f._decode_step(tok, cache_f)
                diff = max(diff, (logits_s.view(-1) - logits_f.view(-1)).abs().max().item())
                for f in cache_f._idx:
                    a_, ca = cache_s._idx[f]
                    b_, cb = cache_f._idx[f]
                    sa, sb = set(a_[0, : int(ca[0])].tolist()), set(b_[0, : int(cb[0])].tolist())
                    same = same and sa == sb
                    overlap = min(overlap, len(sa & sb) / max(1, len(sb)))
                tok = nxt.clone().view(1, 1)
            if not floor:
                dist.broadcast(tok, src=0)
        return {"max_abs_logit_diff": diff, "index_sets_equal": bool(same), "min_index_set_overlap": overlap}

    def cut(model, n):
        """The model reduced to its first n layers (shares the weights)."""
        keep = model.model.layers
        model.model.layers = torch.nn.ModuleList(list(keep)[:n])
        model.config.num_hidden_layers = n
        return keep

    res = {"ctx": ctx, "steps": steps, "against": "the unsharded model (same seed) on rank 0, decoding from the same prompt "
                                                 "K/V, teacher-forced with its greedy tokens"}
    n_all = cfg.num_hidden_layers
    res["full_depth"] = compare(lm, full, n_all)
    if rank == 0:
        res["full_depth"]["noise_floor"] = dict(compare(full, full, n_all, floor=True),
                                                what="the unsharded model against itself with the attention split count changed")
    # reduced depth: the first two layers of both models
    keep_s = cut(lm, 2)
    keep_f = cut(full, 2) if rank == 0 else None
    sel = cfg.get("do_select_layers")
    for model in ([lm, full] if rank == 0 else [lm]):
        model.config.do_select_layers = "1"
        for i, layer in enumerate(model.model.layers):
            layer.do_select_layers, layer.is_filter = [1], i == 1
    try:
        res["depth2"] = compare(lm, full, 2)
    finally:
        lm.model.layers, cfg.num_hidden_layers, cfg.do_select_layers = keep_s, n_all, sel
        filt = [int(i) for i in sel.split(",")]
        for i, layer in enumerate(lm.model.layers):
            layer.do_select_layers, layer.is_filter = filt, i in filt
    ops.check_status(dev)
    del full
    torch.cuda.empty_cache()
    dist.barrier()
    return res


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def build_workload(args, world, rank, dev, tp):
    """(config, config factory, model, batch, context lengths) of the chosen workload."""
    from omnikv_b200.modeling import LlamaCompressorConfig, OmniKVMulLM
    wl = args.workload

    def make_cfg():
        if wl == "tp70b" and args.rank_shape_of > 1:  # one rank's share of the 70B shape on one GPU, no exchange
            n = args.rank_shape_of
            cfg = LlamaCompressorConfig(num_hidden_layers=args.layers, hidden_size=8192, intermediate_size=28672 // n,
                                        num_attention_heads=64 // n, num_key_value_heads=8 // n,
                                        vocab_size=128256 // n, head_dim=128)
        elif wl == "tp70b":
            cfg = LlamaCompressorConfig(num_hidden_layers=args.layers, hidden_size=8192, intermediate_size=28672,
                                        num_attention_heads=64, num_key_value_heads=8)
        elif args.rank_shape_of > 1:
            n = args.rank_shape_of
            cfg = LlamaCompressorConfig(num_hidden_layers=args.layers, num_attention_heads=32 // n, num_key_value_heads=8 // n,
                                        intermediate_size=14336 // n, vocab_size=128256 // n, head_dim=128)
        else:
            cfg = LlamaCompressorConfig(num_hidden_layers=args.layers)
        omni = dict(OMNI)
        if wl == "batch16":
            omni.update(selector_cls="exp", num_of_selected_tokens=2048)
        elif wl == "offload":
            omni.update(real_offload=True)
            if args.skip_threshold is not None:
                omni.update(cache_cls="lazy", skip_threshold=args.skip_threshold)
        elif wl == "tp70b":
            omni.update(do_select_layers="5,20,45")
        cfg.set_config_of_compressor(**omni)
        cfg.set_config_of_compressor(fused_decode=True, chained_decode=args.chain, prefill_kernel=args.prefill_kernel,
                                     tcgen05_linear=args.tcgen05_linear, fused_small_ops=not args.no_fused_adds)
        return cfg

    cfg = make_cfg()
    lm = OmniKVMulLM.from_config(cfg, dtype=torch.bfloat16, device=dev, seed=0, tp=tp)
    g = torch.Generator().manual_seed(0)
    if wl == "batch16":
        B, lens = 16, torch.randint(16384, 32769, (16,), generator=g).tolist()
    elif wl == "tp70b":
        B, lens = 8, [args.ctx] * 8
    else:
        B, lens = 1, [args.ctx]
    return cfg, make_cfg, lm, B, lens


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode128k", choices=sorted(WORKLOADS))
    ap.add_argument("--ctx", type=int, default=0, help="prompt length (default: the workload's)")
    ap.add_argument("--layers", type=int, default=0, help="decoder layers (default: the workload's: 32, tp70b 80)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-torch-baseline", action="store_true")
    ap.add_argument("--no-tp-parity", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--synthetic-kv", action="store_true", help="decode128k: fill the prompt KV with seeded N(0,1) values "
                    "instead of prefilling a prompt of uniform-random token ids through the model")
    ap.add_argument("--chain", action="store_true", help="run the weight-streaming phases between two attention calls "
                    "as one cooperative multi-phase launch instead of one launch per phase (measured slower so far)")
    ap.add_argument("--nccl-allreduce", action="store_true", help="multi-GPU: NCCL all-reduce after the row-parallel "
                    "projections instead of the peer-memory exchange")
    ap.add_argument("--skip-threshold", type=float, default=None, help="offload: cache_cls lazy with this threshold")
    ap.add_argument("--rank-shape-of", type=int, default=0, metavar="N",
                    help="decode128k on ONE GPU with the shapes one rank of an N-way tensor-parallel run holds (1/N of the "
                         "heads, the MLP and the vocabulary) and no exchange: the per-rank floor a multi-GPU step is "
                         "compared with.  The line is marked and is not a benchmark value")
    ap.add_argument("--real-prefill", action="store_true",
                    help="offload: run the prompt through the model (this package's prefill attention kernel, K/V handed "
                         "to pinned host memory layer by layer) instead of filling the cache with seeded values")
    ap.add_argument("--prefill-kernel", default="tcgen05", choices=["tcgen05", "sdpa"],
                    help="prompt attention: this package's kernel, or PyTorch's fused attention")
    ap.add_argument("--tcgen05-linear", action="store_true",
                    help="batched workloads: projections through this package's tcgen05 weight stream instead of the "
                         "library GEMM")
    ap.add_argument("--no-fused-adds", action="store_true",
                    help="batched workloads: separate residual-add and norm kernels (PyTorch) instead of one launch")
    ap.add_argument("--profile-step", action="store_true",
                    help="after the warm-up, run ONE step between cudaProfilerStart/Stop and exit (for ncu "
                         "--profile-from-start off); prints no benchmark line")
    args = ap.parse_args()
    args.ctx = args.ctx or {"decode128k": CTX, "batch16": 32768, "offload": 450000, "tp70b": 65536}[args.workload]
    args.layers = args.layers or (80 if args.workload == "tp70b" else 32)
    quiet_stdout()
    if args.impl == "reference":
        return run_reference_arm(args)

    from omnikv_b200 import ops, parallel
    from omnikv_b200.modeling.omnikv import DecodeRunner

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    tp = parallel.init(world, rank, dev) if world > 1 else None
    wl = args.workload
    batched = wl in ("batch16", "tp70b")
    if tp is not None and not args.nccl_allreduce:
        if batched:
            tp.enable_peer_reduce(8 * 8192 * 2, dev)  # a batch-8 hidden state of the 70B shape in bf16
        else:
            tp.enable_peer_exchange(4096, dev)
            # the filter layers' score planes (MAX) and the sharded logits (gather) through peer memory as well
            tp.enable_peer_reduce(max(8 // world * args.ctx * 4, 128256 // world * 4), dev)

    warmup = max(3, args.warmup)
    cfg, make_cfg, lm, B, lens = build_workload(args, world, rank, dev, tp)
    tp_parity = None
    if tp is not None and wl == "decode128k" and not args.no_tp_parity:
        tp_parity = tp_parity_check(lm, make_cfg, tp, dev, rank)

    graph_warm = 2
    total = graph_warm + 2 * (warmup + args.steps) + 2
    reserve = total + 16
    kvh_local = cfg.num_key_value_heads // (world if tp else 1)
    prefill_s, fill_s = None, None
    if (wl == "decode128k" and not args.synthetic_kv) or (args.real_prefill and B == 1):
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
        t0 = time.perf_counter()
        cache = lm.new_cache().init_synthetic(B, kvh_local, cfg.head_dim, lens, torch.bfloat16, dev, seed=1 + rank,
                                              reserve=reserve)
        torch.cuda.synchronize()
        fill_s = time.perf_counter() - t0
        lm.prepare_synthetic_decode(B, seed=2)
        first = torch.ones(B, 1, dtype=torch.int64, device=dev)
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
    ops.check_status(dev)  # a bounded wait that ran out would have left incomplete results behind

    # ---- end to end: tokens in from pinned host memory, logits + next tokens back to the host ------
    vocab_local = lm.lm_head.weight.shape[0] * (world if tp else 1)
    h_tok = torch.ones(B, 1, dtype=torch.int64).pin_memory()
    h_next = torch.zeros(B, 1, dtype=torch.int64).pin_memory()
    h_logits = torch.zeros(B, vocab_local, dtype=torch.float32).pin_memory()

    def e2e_step():
        runner.token.copy_(h_tok, non_blocking=True)
        runner.run(1)
        h_next.copy_(runner.token, non_blocking=True)
        h_logits.copy_(runner.logits.view(B, -1), non_blocking=True)
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
    ops.check_status(dev)
    clocks = sampler.stop() if rank == 0 else None

    if tp is not None:
        t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms, ms_e2e = t.tolist()

    # ---- roofline of the dominant kernel: dense decode attention, timed live on its stream -------
    dense_layers = [i for i, s in cache.layer_state.items() if not s[0]]
    q = torch.randn(B, cfg.num_attention_heads // (world if tp else 1), cfg.head_dim, device=dev).to(torch.bfloat16)
    # The dense layers' attention calls are captured in a CUDA graph (as they are in the timed step) and
    # bracketed by events on the launching stream, so the host's launch cost is not part of the duration; the
    # launches read distinct K/V of every dense layer, far more than L2 holds.
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
    for rep_i in range(4):
        g_att.replay()
        torch.cuda.synchronize()
        if rep_i > 0:
            durs.append(ev[0].elapsed_time(ev[1]) / len(dense_layers))
    row_bytes = 2 * kvh_local * cfg.head_dim * 2            # K and V rows of every local KV head
    rows_now = [n + runner.steps_done + 1 for n in lens]     # rows a dense layer reads per sequence
    alg_bytes = row_bytes * sum(rows_now)
    dur_ms = statistics.mean(durs)
    peak, peak_kind = measured_peak_gbs()
    achieved = alg_bytes / (dur_ms * 1e-3) / 1e9
    # DRAM traffic per (row, KV head) of this kernel, from an ncu capture of one dense-layer launch at the benchmark's
    # shape (dram__bytes_read.sum + dram__bytes_write.sum = 545.06 MB for 131073 rows x 8 KV heads), scaled by the
    # rows this launch reads
    traffic = 519.2 * sum(rows_now) * kvh_local
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "traffic_source": "ncu capture of one launch at 131073 rows x 8 KV heads, scaled by rows",
                "kernel": "decode_attn_mma_kernel (dense layer: TMA tensor-map tiles, split-K, merge by the last CTA)",
                "algorithmic_bytes_per_launch": alg_bytes, "launch_ms": dur_ms, "peak_kind": peak_kind}

    # whole-step algorithmic bytes (KV + weights; the job's, all ranks) for context
    n_sparse = cfg.num_hidden_layers - len(dense_layers)
    nsel = cfg.get("num_of_selected_tokens")
    k0 = [nsel if isinstance(nsel, int) else int(nsel * n) for n in lens]
    row_all = 2 * cfg.num_key_value_heads * cfg.head_dim * 2
    kv_bytes = sum(len(dense_layers) * row_all * r + n_sparse * row_all * (k + runner.steps_done) for r, k in zip(rows_now, k0))
    if cfg.get("selector_cls") not in ("last",):
        kv_bytes += 3 * sum(lens) * row_all // 2   # the window selectors read the filter layers' K a second time
    w_bytes = 2 * (world if tp else 1) * sum(p.numel() for n_, p in lm.named_parameters()
                                             if "embed_tokens" not in n_ and p.dim() > 1)
    link_bytes = n_sparse * row_all * k0[0] if wl == "offload" else 0
    step_bytes = kv_bytes + w_bytes + link_bytes  # staged rows are written and read once more: counted once
    ms_step = ms / args.steps
    step_gbs = step_bytes / (ms_step * 1e-3) / 1e9 / (world if tp else 1)

    torch_leg = None
    if rank == 0 and world == 1 and wl == "decode128k" and not args.no_torch_baseline:
        torch_leg = gpu_torch_baseline(cache, q, dev)

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
    if world > 1:
        par = ("peer-memory all-reduce kernel" if tp.reducer is not None else "nccl all-reduce") if batched else \
              ("fused peer-memory exchange" if tp.exchange is not None else "nccl all-reduce")
    line = {
        "metric": METRIC if wl == "decode128k" else f"decode tokens/s ({wl})", "value": B * args.steps / (ms * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_block(args, world),
        "run": {"exchange": par if world > 1 else None, "cuda_graph": not args.no_graph,
                "context_lengths": lens if B > 1 else lens[0],
                "kv_fill": (f"real prefill of {args.ctx} uniform-random token ids ({prefill_s:.1f} s, attention: {args.prefill_kernel})" if prefill_s
                            else f"seeded N(0,1), no prefill run ({fill_s:.1f} s)")},
        "clocks": clocks,
        "e2e": {"value": B * args.steps / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 8 * B,
                "d2h_bytes_per_step": B * (8 + vocab_local * 4), "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": runner.launches_per_step * args.steps,
        "launches_per_step": runner.launches_per_step,
        "roofline": roofline,
        "whole_step": {"algorithmic_bytes": step_bytes, "kv_bytes": kv_bytes, "weight_bytes": w_bytes,
                       "achieved_gbs_per_gpu": step_gbs, "frac_of_peak": step_gbs / peak},
    }
    if args.rank_shape_of > 1:
        line["metric"] = f"NOT A BENCHMARK VALUE: one rank's share of a {args.rank_shape_of}-way tensor-parallel step, no exchange"
    if link_bytes:
        line["host_link"] = {"bytes_per_step": link_bytes, "achieved_gbs": link_bytes / (ms_step * 1e-3) / 1e9}
    if tp_parity is not None:
        line["tp_parity"] = tp_parity
    if torch_leg is not None:
        line["gpu_torch_baseline"] = torch_leg
    if world == 1 and wl == "decode128k" and not args.no_cpu_baseline:
        threads = min(os.cpu_count() or 1, 8)  # the reference's cpu_num_threads default is 8 (configs/example.json)
        line["cpu_baseline"] = cpu_baseline_block(threads, os.cpu_count() or 1)
    emit(line)
    finish()


if __name__ == "__main__":
    main()
