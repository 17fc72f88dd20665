"""CPU timing harness for the decode-selection path: the baseline reported beside the GPU numbers.

TEST / MEASUREMENT INFRASTRUCTURE ONLY -- imported by ``bench.py`` for its ``cpu_baseline`` leg and its
``--impl reference`` arm, never by the product package.

Two things are timed on the host cores:

* ``operator_case_stats``: the single-layer operator case (32 query / 8 KV heads, head size 128, batch 1, context
  16384, fp32, selector ``last``, k = 1098, seeded N(0,1) inputs with 2 % boosted keys) stage by stage --
  score + top-k, gather of the second layer's rows, update + attention over them -- with 3 warm-ups and >= 20
  repetitions, median and p10 / p90 of ``time.perf_counter``.  When a checkout of the reference is reachable
  (``OMNIKV_REFERENCE``), the stages are the REFERENCE's own ``select_tokens_by_attn_universal``,
  ``OmniKVMultiStageCache.set_idx_on_gpu`` and ``.update`` (kind "reference"); otherwise the restatement in this
  folder (kind "port").
* ``StepSample``: a bounded sample of one decode step of the benchmark (Llama-3-8B shape, 128K context): one
  filter layer, one sparse layer, one layer of weight GEMVs and the lm_head at full size, scaled by the step's
  layer counts to tokens/s.  A whole step of an 8B model on a CPU is out of reach; the pieces are the port.
"""
from __future__ import annotations

import math
import statistics
import time
import types
from typing import Dict, List

import torch

from . import omnikv_oracle as oo
from . import ref_shim

OPERATOR = dict(L=16384, H=32, KVH=8, d=128, W=16, k=1098, seed=2024)


def operator_inputs(seed: int = OPERATOR["seed"]):
    """Seeded inputs of the operator case: Q [1,H,W,d], the filter layer's K and a second layer's K2, V2
    [1,KVH,L,d] ~ N(0,1); 2 % of the key positions get +4 u (u = unit vector of the mean query) in every KV head."""
    o = OPERATOR
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, o["H"], o["W"], o["d"], generator=g)
    k = torch.randn(1, o["KVH"], o["L"], o["d"], generator=g)
    k2 = torch.randn(1, o["KVH"], o["L"], o["d"], generator=g)
    v2 = torch.randn(1, o["KVH"], o["L"], o["d"], generator=g)
    k_new = torch.randn(1, o["KVH"], 1, o["d"], generator=g)
    v_new = torch.randn(1, o["KVH"], 1, o["d"], generator=g)
    u = q.mean(dim=(0, 1, 2))
    u = u / u.norm()
    hot = torch.randperm(o["L"], generator=g)[: int(round(0.02 * o["L"]))]
    k[:, :, hot, :] += 4.0 * u
    return dict(q=q, k=k, k2=k2, v2=v2, k_new=k_new, v_new=v_new)


class _Attn:
    """What the selector reads from ``self_attn``: identity projection and rotation reproduce Q exactly."""

    def __init__(self, o):
        self.num_heads, self.num_key_value_heads, self.head_dim, self.layer_idx = o["H"], o["KVH"], o["d"], 0
        self.num_key_value_groups = o["H"] // o["KVH"]
        self.config = types.SimpleNamespace(get=lambda key, default=None: default)

    def q_proj(self, x):
        return x

    def k_proj(self, x):
        return x[..., : self.num_key_value_heads * self.head_dim]

    def rotary_emb(self, x, position_ids):
        shape = (position_ids.shape[0], position_ids.shape[1], self.head_dim)
        return torch.ones(shape), torch.zeros(shape)


def _stats(xs: List[float]) -> Dict[str, float]:
    xs = sorted(xs)
    pick = lambda p: xs[min(len(xs) - 1, int(round(p * (len(xs) - 1))))]  # noqa: E731
    return {"median_ms": statistics.median(xs) * 1e3, "p10_ms": pick(0.1) * 1e3, "p90_ms": pick(0.9) * 1e3}


def operator_case_stats(threads: int, reps: int = 20, warmups: int = 3) -> Dict:
    """Stage timings of the operator case on ``threads`` host threads.  See the module docstring."""
    o = OPERATOR
    x = operator_inputs()
    root = ref_shim.reference_root()
    if root is not None:
        ref_omnikv, ref_cache = ref_shim.import_reference(root)
        select = ref_omnikv.select_tokens_by_attn_universal
        dyn = types.SimpleNamespace(key_cache=[], value_cache=[], _seen_tokens=0)
        cache = ref_cache.OmniKVMultiStageCache.from_dynamic_cache(dyn, [0, 2], 2, 0, False)
        kind = "reference"
    else:
        select = oo.select_tokens_by_attn_universal
        cache = oo.OracleMultiStageCache([0, 2], 2, 0, False)
        kind = "port"
    torch.set_num_threads(threads)
    attn = _Attn(o)
    hs = x["q"].transpose(1, 2).reshape(1, o["W"], o["H"] * o["d"])[:, -1:]
    pos = torch.tensor([[o["L"]]])
    cache.stage = "prefill"
    cache.update(x["k"], torch.zeros_like(x["k"]), 0)
    cache.update(x["k2"], x["v2"], 1)
    cache.stage = "decoding"
    view = types.SimpleNamespace(key_cache=cache.key_cache)
    qq = x["q"][:, :, -1, :]
    G = o["H"] // o["KVH"]
    t = {"score_topk": [], "gather": [], "update_attention": [], "total": []}
    for it in range(warmups + reps):
        t0 = time.perf_counter()
        idx = select(attn, hs, pos, view, o["k"], o["L"], 0, "last")
        t1 = time.perf_counter()
        cache.set_idx_on_gpu(idx, 0)
        t2 = time.perf_counter()
        kk, vv = cache.update(x["k_new"], x["v_new"], 1)
        n = kk.shape[2]
        kr = kk[:, :, None].expand(1, o["KVH"], G, n, o["d"]).reshape(1, o["H"], n, o["d"])
        vr = vv[:, :, None].expand(1, o["KVH"], G, n, o["d"]).reshape(1, o["H"], n, o["d"])
        s = torch.matmul(qq[:, :, None, :], kr.transpose(2, 3)) / math.sqrt(o["d"])
        torch.matmul(torch.softmax(s, dim=-1), vr)
        t3 = time.perf_counter()
        if it >= warmups:
            t["score_topk"].append(t1 - t0)
            t["gather"].append(t2 - t1)
            t["update_attention"].append(t3 - t2)
            t["total"].append(t3 - t0)
    return {"kind": kind, "threads": threads, "reps": reps, "warmups": warmups,
            "stages": {name: _stats(v) for name, v in t.items()}}


class StepSample:
    """A bounded sample of one decode step at the benchmark's sizes; inputs are built once, ``run`` times the pieces."""

    def __init__(self, ctx: int = 131072, seed: int = 0, row_fraction: int = 8):
        """``row_fraction``: the dense layer and the selector are timed on ``ctx / row_fraction`` rows and scaled
        back (their cost is linear in the rows), which keeps a sample near a second; the sparse layer, the weight
        GEMVs and the lm_head are timed at full size."""
        g = torch.Generator().manual_seed(seed)
        H, KVH, d, hidden, inter, vocab = 32, 8, 128, 4096, 14336, 128256
        self.ctx, self.k, self.frac = ctx, int(0.067 * ctx), row_fraction
        self.rows = max(self.k + 1, ctx // row_fraction)
        bf = torch.bfloat16
        self.kc = torch.randn(1, KVH, self.rows, d, generator=g).to(bf)
        self.vc = torch.randn(1, KVH, self.rows, d, generator=g).to(bf)
        self.q = torch.randn(1, H, d, generator=g).to(bf)
        self.x = torch.randn(1, hidden, generator=g).to(bf)
        self.xi = torch.randn(1, inter, generator=g).to(bf)
        mk = lambda n, m: (torch.randn(n, m, generator=g) * 0.02).to(bf)  # noqa: E731
        self.ws = [mk(6144, hidden), mk(hidden, hidden), mk(2 * inter, hidden)]
        self.wd = mk(hidden, inter)
        self.wl = mk(vocab, hidden)
        self.sample = (f"per step: dense attention and selector last + top-k on {self.rows} of {ctx} rows (scaled by "
                       f"{ctx / self.rows:.1f}), one sparse layer ({self.k} rows), one layer of weight GEMVs and the lm_head "
                       "at full size, combined as 8 dense / 3 filter / 24 sparse / 32 layers + lm_head")

    def run(self):
        """(seconds of one decode step extrapolated from the sample, seconds per piece)."""
        t = {}
        t0 = time.perf_counter()
        oo.dense_attention(self.q, self.kc, self.vc)
        t["dense_attn"] = time.perf_counter() - t0
        t0 = time.perf_counter()
        s = oo.score_last(self.q, self.kc, self.rows)
        idx = oo.topk_ascending(s, self.k)
        t["select"] = time.perf_counter() - t0
        t0 = time.perf_counter()
        oo.sparse_attention(self.q, self.kc, self.vc, idx, self.kc[:, :, :1], self.vc[:, :, :1])
        t["sparse_attn"] = time.perf_counter() - t0
        t0 = time.perf_counter()
        for w in self.ws:
            torch.nn.functional.linear(self.x, w)
        torch.nn.functional.linear(self.xi, self.wd)
        t["layer_gemv"] = time.perf_counter() - t0
        t0 = time.perf_counter()
        torch.nn.functional.linear(self.x, self.wl)
        t["lm_head"] = time.perf_counter() - t0
        up = self.ctx / self.rows
        step = (8 * t["dense_attn"] + 3 * t["select"]) * up + 24 * t["sparse_attn"] + 32 * t["layer_gemv"] + t["lm_head"]
        return step, t
