"""Seeded inputs shared by the fixture generator and by the tests.

Only OUTPUTS of the reference are committed as fixtures; inputs are rebuilt from
these functions.  numpy's PCG64 ``Generator`` stream is stable across library
versions, and every fixture stores a float64 checksum of its inputs so that a
drift would be caught rather than silently compared.
"""
from __future__ import annotations

import math

import numpy as np


def checksum(arrays) -> float:
    return float(sum(np.float64(a.astype(np.float64).sum()) + np.float64(np.abs(a.astype(np.float64)).sum()) for a in arrays))


def selector_case_list():
    """Groups of small selector cases: one input set per group, several k per group."""
    out = []
    seed = 100
    for sel in ("last", "softmax_before_last", "uniform", "exp"):
        for (b, L) in ((1, 1), (1, 17), (2, 255), (1, 1000), (3, 4097)):
            ws = (1,) if sel == "last" else (1, 5, 16)
            for w in ws:
                seed += 1
                ks = sorted({1, max(1, L - 1), L, L + 5, max(1, int(0.067 * L)), max(1, L // 2)})
                out.append(dict(name=f"{sel}_B{b}_L{L}_W{w}", B=b, H=8, KVH=2, d=32, L=L, W=w, ks=ks,
                                selector=sel, seed=seed, theta=10000.0, pos=L + 2))
    return out


def selector_inputs(case):
    """wq [H*d, hidden], wk [KVH*d, hidden], hs [B, W, hidden], kc [B, KVH, L+3, d] (fp32)."""
    rng = np.random.default_rng(case["seed"])
    h, kvh, d, b, w, L = case["H"], case["KVH"], case["d"], case["B"], case["W"], case["L"]
    hidden = h * d // 4
    wq = (rng.standard_normal((h * d, hidden), dtype=np.float32) / math.sqrt(hidden)).astype(np.float32)
    wk = (rng.standard_normal((kvh * d, hidden), dtype=np.float32) / math.sqrt(hidden)).astype(np.float32)
    hs = (rng.standard_normal((b, w, hidden), dtype=np.float32) * 2.0).astype(np.float32)
    kc = rng.standard_normal((b, kvh, L + 3, d), dtype=np.float32)  # 3 decode-time rows past consider_len
    return dict(wq=wq, wk=wk, hs=hs, kc=kc)


CACHE_FLOW = dict(n_layers=6, sel=[1, 3], wait=1, kvh=2, d=16, P=40, steps=3, n_idx=9, seed=7)


def cache_flow_inputs():
    c = CACHE_FLOW
    rng = np.random.default_rng(c["seed"])
    n, kvh, d, P, steps = c["n_layers"], c["kvh"], c["d"], c["P"], c["steps"]
    k_pre = [rng.standard_normal((1, kvh, P, d), dtype=np.float32) for _ in range(n)]
    v_pre = [rng.standard_normal((1, kvh, P, d), dtype=np.float32) for _ in range(n)]
    k_new = [[rng.standard_normal((1, kvh, 1, d), dtype=np.float32) for _ in range(n)] for _ in range(steps)]
    v_new = [[rng.standard_normal((1, kvh, 1, d), dtype=np.float32) for _ in range(n)] for _ in range(steps)]
    idx = {(s, f): np.sort(rng.choice(P, size=c["n_idx"], replace=False))[None, :].astype(np.int64)
           for s in range(steps) for f in c["sel"]}
    return dict(k_pre=k_pre, v_pre=v_pre, k_new=k_new, v_new=v_new, idx=idx)


LAZY_RULE = dict(seed=11, P=4000, k=300, steps=24, thresholds=[0.4, 0.7, 0.95])


def lazy_rule_inputs():
    """A drifting sequence of ascending index lists [steps][1, k]: each step replaces a random share
    (0 .. 80 %) of the previous list's entries, so consecutive overlaps cover the whole range."""
    c = LAZY_RULE
    rng = np.random.default_rng(c["seed"])
    cur = np.sort(rng.choice(c["P"], size=c["k"], replace=False))
    out = [cur[None, :].astype(np.int64)]
    for _ in range(c["steps"] - 1):
        n_new = int(rng.uniform(0.0, 0.8) * c["k"])
        keep = rng.choice(cur, size=c["k"] - n_new, replace=False)
        pool = np.setdiff1d(np.arange(c["P"]), keep)
        cur = np.sort(np.concatenate([keep, rng.choice(pool, size=n_new, replace=False)]))
        out.append(cur[None, :].astype(np.int64))
    return out


OPERATOR = dict(seed=2024, L=16384, H=32, KVH=8, d=128, W=16, k=1098)


def operator_inputs(seed: int = 2024, L: int = 16384, H: int = 32, KVH: int = 8, d: int = 128, W: int = 16):
    """Inputs of the single-layer operator case (batch 1, fp32).

    Q ``[1,H,W,d]`` (already rotated), the filter layer's K ``[1,KVH,L,d]`` and a second
    layer's K2, V2, all ~ N(0,1); 2 % of the key positions get ``+4 u`` (u = unit vector of
    the mean query) in every KV head; ``k_new, v_new`` is the current token's row of the
    second layer.
    """
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((1, H, W, d), dtype=np.float32)
    k = rng.standard_normal((1, KVH, L, d), dtype=np.float32)
    k2 = rng.standard_normal((1, KVH, L, d), dtype=np.float32)
    v2 = rng.standard_normal((1, KVH, L, d), dtype=np.float32)
    k_new = rng.standard_normal((1, KVH, 1, d), dtype=np.float32)
    v_new = rng.standard_normal((1, KVH, 1, d), dtype=np.float32)
    u = q.mean(axis=(0, 1, 2))
    u = (u / np.linalg.norm(u)).astype(np.float32)
    hot = np.sort(rng.choice(L, size=int(round(0.02 * L)), replace=False))
    k[:, :, hot, :] += 4.0 * u
    return dict(q=q, k=k, k2=k2, v2=v2, k_new=k_new, v_new=v_new, hot=hot)
