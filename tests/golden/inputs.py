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


# the same flow at the head size the CUDA kernels are built for; its fixture stores signatures, not tensors
CACHE_FLOW_D128 = dict(n_layers=6, sel=[1, 3], wait=1, kvh=2, d=128, P=300, steps=4, n_idx=41, seed=17)


def signature(a) -> list:
    """[shape..., sum, sum of magnitudes, position-weighted sum] in float64: equal for equal arrays, and changed by
    any swapped, missing or altered element (the cache returns copies of its inputs, never new values)."""
    f = np.ascontiguousarray(a).astype(np.float64).ravel()
    w = np.arange(1, f.size + 1, dtype=np.float64)
    return [*a.shape, float(f.sum()), float(np.abs(f).sum()), float((f * w).sum())]


def cache_flow_inputs(c=None):
    c = c or CACHE_FLOW
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


LAYER_HOOK = dict(seed=31, n_layers=6, sel=[1, 3], wait=0, hidden=512, H=4, KVH=2, d=128, inter=768, P=200, steps=20,
                  window=16, frac=0.25, theta=500000.0, eps=1e-5, qk_gain=3.0)


def layer_hook_inputs():
    """A 6-layer decoder stack for the filter-layer hook: per layer the Hugging Face named weights (fp32; q/k
    scaled up so that attention is peaked and the selection matters), the prompt's input hidden states
    ``x_pre [1, P, hidden]`` and one input hidden state per decode step ``x_dec [steps][1, 1, hidden]``."""
    c = LAYER_HOOK
    rng = np.random.default_rng(c["seed"])
    hid, d, H, KVH, inter = c["hidden"], c["d"], c["H"], c["KVH"], c["inter"]
    n = lambda *s: rng.standard_normal(s, dtype=np.float32)  # noqa: E731
    layers = []
    for _ in range(c["n_layers"]):
        layers.append({
            "self_attn.q_proj.weight": n(H * d, hid) * (c["qk_gain"] / math.sqrt(hid)),
            "self_attn.k_proj.weight": n(KVH * d, hid) * (c["qk_gain"] / math.sqrt(hid)),
            "self_attn.v_proj.weight": n(KVH * d, hid) / math.sqrt(hid),
            "self_attn.o_proj.weight": n(hid, H * d) / math.sqrt(H * d),
            "mlp.gate_proj.weight": n(inter, hid) / math.sqrt(hid),
            "mlp.up_proj.weight": n(inter, hid) / math.sqrt(hid),
            "mlp.down_proj.weight": n(hid, inter) / math.sqrt(inter),
            "input_layernorm.weight": (1.0 + 0.1 * n(hid)).astype(np.float32),
            "post_attention_layernorm.weight": (1.0 + 0.1 * n(hid)).astype(np.float32),
        })
    x_pre = n(1, c["P"], hid)
    x_dec = [n(1, 1, hid) for _ in range(c["steps"])]
    return dict(layers=layers, x_pre=x_pre, x_dec=x_dec)


ROPE_CASES = [
    dict(name="default", head_dim=128, rope_theta=500000.0, max_position_embeddings=8192, rope_scaling=None),
    dict(name="linear", head_dim=128, rope_theta=10000.0, max_position_embeddings=4096,
         rope_scaling={"rope_type": "linear", "factor": 4.0}),
    dict(name="dynamic_init", head_dim=128, rope_theta=500000.0, max_position_embeddings=8192,
         rope_scaling={"type": "dynamic", "factor": 4}),
    dict(name="llama3", head_dim=128, rope_theta=500000.0, max_position_embeddings=131072,
         rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                       "original_max_position_embeddings": 8192}),
    dict(name="yarn", head_dim=128, rope_theta=10000.0, max_position_embeddings=4096,
         rope_scaling={"rope_type": "yarn", "factor": 16.0}),
    dict(name="yarn_betas", head_dim=64, rope_theta=1000000.0, max_position_embeddings=32768,
         rope_scaling={"rope_type": "yarn", "factor": 4.0, "beta_fast": 16, "beta_slow": 2, "attention_factor": 1.25}),
    dict(name="longrope_long", head_dim=96, rope_theta=10000.0, max_position_embeddings=4096,
         rope_scaling={"rope_type": "longrope", "factor": 8.0,
                       "long_factor": [1.0 + 0.25 * i for i in range(48)], "short_factor": [1.0 + 0.01 * i for i in range(48)]}),
    dict(name="longrope_phi3", head_dim=96, rope_theta=10000.0, max_position_embeddings=131072,
         original_max_position_embeddings=4096,
         rope_scaling={"rope_type": "longrope", "long_factor": [1.0 + 0.5 * i for i in range(48)],
                       "short_factor": [1.0 + 0.02 * i for i in range(48)]}),
]

# dynamic NTK followed over a conversation: forwards given as (first position, number of positions)
ROPE_DYNAMIC_SEQ = dict(head_dim=128, rope_theta=500000.0, max_position_embeddings=1024,
                        rope_scaling={"type": "dynamic", "factor": 4.0},
                        forwards=[(0, 600), (600, 1), (0, 1500), (1500, 1), (1501, 1), (1502, 1), (0, 1200), (1200, 1),
                                  (0, 300), (300, 1), (0, 2000), (2000, 1)])


# The decode attention of the reference's LightLLM fork over a paged pool: one request of 3000 tokens for the
# selecting call (the fork asserts batch 1 there) and three ragged requests for the plain call.
LIGHTLLM = dict(seed=515, H=8, KVH=2, d=128, pool_tokens=6144, n_requests=5, max_seq=3200, k=2048,
                select=dict(req=3, L=3000), dense=dict(reqs=[1, 4, 0], lens=[700, 256, 1033]))


def lightllm_inputs():
    """pool / pool2 ``[tokens, 2*KVH, d]`` (two layers' KV with the same paging), the request table, queries."""
    c = LIGHTLLM
    rng = np.random.default_rng(c["seed"])
    H, KVH, d = c["H"], c["KVH"], c["d"]
    pool = rng.standard_normal((c["pool_tokens"], 2 * KVH, d)).astype(np.float32)
    pool2 = rng.standard_normal((c["pool_tokens"], 2 * KVH, d)).astype(np.float32)
    perm = rng.permutation(c["pool_tokens"]).astype(np.int32)
    table = np.zeros((c["n_requests"], c["max_seq"]), dtype=np.int32)
    used = 0
    for req, n in [(c["select"]["req"], c["select"]["L"])] + list(zip(c["dense"]["reqs"], c["dense"]["lens"])):
        table[req, :n] = perm[used:used + n]
        used += n
    q_sel = rng.standard_normal((1, H, d)).astype(np.float32)
    q_sparse = rng.standard_normal((1, H, d)).astype(np.float32)
    q_dense = rng.standard_normal((len(c["dense"]["reqs"]), H, d)).astype(np.float32)
    # a few keys stand out, so that membership in the top 2048 of 3000 is not decided by the last bits
    L = c["select"]["L"]
    hot = rng.permutation(L)[: L // 40]
    qm = q_sel[0].mean(axis=0)
    pool[table[c["select"]["req"], hot], :KVH] += (3.0 * qm / np.linalg.norm(qm)).astype(np.float32)
    return dict(pool=pool, pool2=pool2, table=table, q_sel=q_sel, q_sparse=q_sparse, q_dense=q_dense)
