"""Generate the golden fixtures in this folder by running the REFERENCE's own code.

Run where the reference checkout is available (it is not needed to run the tests):

    python tests/golden/make_golden.py --reference /path/to/OmniKV

It imports ``modeling.omnikv.select_tokens_by_attn_universal`` and
``modeling.spec_cache.{OmniKVMultiStageCache, WOPackCache}`` unchanged, feeds them
seeded inputs, and stores their outputs as small ``.npz`` / ``.json`` files.
Nothing of the reference is copied; the import goes through ``oracle/ref_shim.py`` (the
reference targets transformers 4.41.2: the shims it needs under a newer one are listed
there).  One more adaptation lives here: the 5.x ``DynamicCache`` has no ``key_cache`` list,
so caches are built through ``from_dynamic_cache`` on a namespace carrying the three
attributes it copies.

Only the reference's OUTPUTS are stored; the inputs are rebuilt from the seeded
functions of ``inputs.py`` (a checksum of them is stored beside each fixture).
What the restatement in ``oracle/`` returns is not stored either: the tests
recompute it, so a fixture can only come from the reference.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from inputs import (CACHE_FLOW, OPERATOR, cache_flow_inputs, checksum, operator_inputs,  # noqa: E402
                    selector_case_list, selector_inputs)
import inputs as gi  # noqa: E402


sys.path.insert(0, str(HERE.parent.parent))
from oracle.ref_shim import import_reference  # noqa: E402  (the import shims live there)


class _Cfg:
    def get(self, key, default=None):
        return default


class DuckAttn:
    """The attributes select_tokens_by_attn_universal reads from ``self_attn``."""

    def __init__(self, wq, wk, num_heads, num_kv_heads, head_dim, theta, layer_idx=0, identity_rope=False):
        self.num_heads = num_heads
        self.num_key_value_heads = num_kv_heads
        self.num_key_value_groups = num_heads // num_kv_heads
        self.head_dim = head_dim
        self.layer_idx = layer_idx
        self.config = _Cfg()
        self._wq, self._wk, self._theta, self._id = wq, wk, theta, identity_rope

    def q_proj(self, x):
        return x @ self._wq.T

    def k_proj(self, x):
        return x @ self._wk.T

    def rotary_emb(self, x, position_ids):
        if self._id:
            shape = (position_ids.shape[0], position_ids.shape[1], self.head_dim)
            return torch.ones(shape), torch.zeros(shape)
        inv_freq = 1.0 / (self._theta ** (torch.arange(0, self.head_dim, 2, dtype=torch.float32) / self.head_dim))
        freqs = position_ids.float()[:, :, None] * inv_freq[None, None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        return emb.cos(), emb.sin()


def make_selector_fixture(ref_omnikv):
    arrays, meta = {}, []
    for case in selector_case_list():
        x = selector_inputs(case)
        wq, wk, hs, kc = (torch.from_numpy(x[n]) for n in ("wq", "wk", "hs", "kc"))
        pos = torch.full((case["B"], 1), case["pos"], dtype=torch.long)
        attn = DuckAttn(wq, wk, case["H"], case["KVH"], case["d"], case["theta"])
        cache = types.SimpleNamespace(key_cache=[kc])
        for k in case["ks"]:
            idx = ref_omnikv.select_tokens_by_attn_universal(attn, hs, pos, cache, k, case["L"], 0, case["selector"])
            arrays[f"{case['name']}/k{k}"] = idx.numpy().astype(np.int32)
        meta.append(dict(case, input_checksum=checksum(x.values())))
    np.savez_compressed(HERE / "selector_small.npz", **arrays)
    (HERE / "selector_small.json").write_text(json.dumps(meta, indent=1))
    print("selector groups:", len(meta), "idx lists:", len(arrays))


def make_plan_fixture(ref_cache):
    rows = []
    grid = [
        (32, [2, 8, 18], 1), (32, [2, 8, 18], 2), (32, [2, 8, 18], 0), (80, [5, 20, 45], 1), (80, [5, 20, 45], 2),
        (6, [1, 3], 1), (4, [0], 0), (4, [0], 5), (8, [7], 1), (12, [3, 4, 5], 1), (16, [0, 15], 3),
    ]
    for n, sel, wait in grid:
        full = list(range(0, sel[0])) + sel + [n]
        for cls in (ref_cache.OmniKVMultiStageCache, ref_cache.WOPackCache):
            c = cls(full, n, wait, False)
            rows.append(dict(cls=cls.__name__, num_layers=n, do_select=sel, wait=wait, full_attn_layers=full,
                             layer_state={str(k): list(v) for k, v in sorted(c.layer_state.items())}))
    (HERE / "layer_plan.json").write_text(json.dumps(rows))
    print("plan rows:", len(rows))


def make_cache_flow_fixture(ref_cache):
    """Prefill -> set_idx_on_gpu -> three decode updates on a 6-layer plan, both cache classes."""
    c = CACHE_FLOW
    x = cache_flow_inputs()
    n_layers, sel, wait, steps = c["n_layers"], c["sel"], c["wait"], c["steps"]
    full = list(range(0, sel[0])) + sel + [n_layers]
    t = lambda a: torch.from_numpy(a)  # noqa: E731
    arrays = {}
    for cls in (ref_cache.OmniKVMultiStageCache, ref_cache.WOPackCache):
        dyn = types.SimpleNamespace(key_cache=[], value_cache=[], _seen_tokens=0)
        cache = cls.from_dynamic_cache(dyn, full, n_layers, wait, False)
        cache.stage = "prefill"
        for i in range(n_layers):
            cache.update(t(x["k_pre"][i]), t(x["v_pre"][i]), i)
        for s in range(steps):
            cache.stage = "decoding"
            for i in range(n_layers):
                if i in sel:
                    cache.set_idx_on_gpu(t(x["idx"][(s, i)]), i)
                kk, vv = cache.update(t(x["k_new"][s][i]), t(x["v_new"][s][i]), i)
                arrays[f"{cls.__name__}/ret_k/{s}/{i}"] = kk.numpy().copy()
                arrays[f"{cls.__name__}/ret_v/{s}/{i}"] = vv.numpy().copy()
        arrays[f"{cls.__name__}/seen"] = np.array([cache._seen_tokens])
    np.savez_compressed(HERE / "cache_flow.npz", **arrays)
    flat = x["k_pre"] + x["v_pre"] + [a for r in x["k_new"] for a in r] + [a for r in x["v_new"] for a in r]
    (HERE / "cache_flow.json").write_text(json.dumps(dict(c, full=full, input_checksum=checksum(flat))))
    print("cache flow arrays:", len(arrays))


def make_cache_flow_d128_fixture(ref_cache):
    """The same flow at head size 128 (what the CUDA kernels are built for), four decode steps; per returned
    tensor a signature (shape, sums) instead of the tensor itself, since the returns are pure copies of inputs."""
    from inputs import CACHE_FLOW_D128, signature
    c = CACHE_FLOW_D128
    x = cache_flow_inputs(c)
    n_layers, sel, wait, steps = c["n_layers"], c["sel"], c["wait"], c["steps"]
    full = list(range(0, sel[0])) + sel + [n_layers]
    t = lambda a: torch.from_numpy(a)  # noqa: E731
    sigs = {}
    for cls in (ref_cache.OmniKVMultiStageCache, ref_cache.WOPackCache):
        dyn = types.SimpleNamespace(key_cache=[], value_cache=[], _seen_tokens=0)
        cache = cls.from_dynamic_cache(dyn, full, n_layers, wait, False)
        cache.stage = "prefill"
        for i in range(n_layers):
            cache.update(t(x["k_pre"][i]), t(x["v_pre"][i]), i)
        for s in range(steps):
            cache.stage = "decoding"
            for i in range(n_layers):
                if i in sel:
                    cache.set_idx_on_gpu(t(x["idx"][(s, i)]), i)
                kk, vv = cache.update(t(x["k_new"][s][i]), t(x["v_new"][s][i]), i)
                sigs[f"{cls.__name__}/{s}/{i}"] = [signature(kk.numpy()), signature(vv.numpy())]
        sigs[f"{cls.__name__}/seen"] = int(cache._seen_tokens)
    flat = x["k_pre"] + x["v_pre"] + [a for r in x["k_new"] for a in r] + [a for r in x["v_new"] for a in r]
    (HERE / "cache_flow_d128.json").write_text(json.dumps(dict(c, full=full, input_checksum=checksum(flat), returns=sigs)))
    print("cache flow d128 returns:", len(sigs))


def make_operator_fixture(ref_omnikv, ref_cache):
    """The single-layer operator case through the reference: selector ``last`` (k = 1098), gather of the
    second layer's rows by OmniKVMultiStageCache, then fp32 attention over what ``update`` returns."""
    o = OPERATOR
    H, KVH, d, L, W, k = o["H"], o["KVH"], o["d"], o["L"], o["W"], o["k"]
    x = operator_inputs()
    q = torch.from_numpy(x["q"])
    # q_proj = identity on a [1, W, H*d] layout and an identity rotation reproduce Q exactly.
    hs = q.transpose(1, 2).reshape(1, W, H * d)
    attn = DuckAttn(torch.eye(H * d), torch.zeros(KVH * d, H * d), H, KVH, d, 1.0, identity_rope=True)
    dyn = types.SimpleNamespace(key_cache=[], value_cache=[], _seen_tokens=0)
    cache = ref_cache.OmniKVMultiStageCache.from_dynamic_cache(dyn, [0, 2], 2, 0, False)
    cache.stage = "prefill"
    kf = torch.from_numpy(x["k"])
    cache.update(kf, torch.zeros_like(kf), 0)
    cache.update(torch.from_numpy(x["k2"]), torch.from_numpy(x["v2"]), 1)
    cache.stage = "decoding"
    view = types.SimpleNamespace(key_cache=cache.key_cache)
    idx = ref_omnikv.select_tokens_by_attn_universal(attn, hs[:, -1:], torch.tensor([[L]]), view, k, L, 0, "last")
    cache.set_idx_on_gpu(idx, 0)
    kk, vv = cache.update(torch.from_numpy(x["k_new"]), torch.from_numpy(x["v_new"]), 1)
    assert kk.shape == (1, KVH, k + 1, d)
    qq = q[:, :, -1, :]
    kk = kk[:, :, None].expand(1, KVH, H // KVH, k + 1, d).reshape(1, H, k + 1, d)
    vv = vv[:, :, None].expand(1, KVH, H // KVH, k + 1, d).reshape(1, H, k + 1, d)
    s = torch.matmul(qq[:, :, None, :], kk.transpose(2, 3)) / math.sqrt(d)
    out = torch.matmul(torch.softmax(s, dim=-1), vv)[:, :, 0, :]
    # window selectors on the same inputs (all 16 window queries), k = 1098 as well
    extra = {}
    for sel in ("uniform", "exp"):
        extra[f"idx_{sel}"] = ref_omnikv.select_tokens_by_attn_universal(
            attn, hs, torch.tensor([[L]]), view, k, L, 0, sel).numpy().astype(np.int32)
    np.savez_compressed(HERE / "operator_cfg1.npz", idx=idx.numpy().astype(np.int32), out=out.numpy(), **extra)
    names = ("q", "k", "k2", "v2", "k_new", "v_new")
    (HERE / "operator_cfg1.json").write_text(json.dumps(dict(o, input_checksum=checksum([x[n] for n in names]))))
    print("operator: |idx & hot| =", len(set(idx[0].tolist()) & set(x["hot"].tolist())), "of", len(x["hot"]))


def make_lazy_rule_fixture(ref_cache):
    """The reference's OmniKVLazyCache.set_out_idx on a drifting index sequence: which steps re-gather and
    which keep the previous selection (modeling/spec_cache.py:539-557), plus the overlap score of :10-31."""
    from inputs import LAZY_RULE, lazy_rule_inputs
    c = LAZY_RULE
    seq = lazy_rule_inputs()
    res = {}
    for thr in c["thresholds"]:
        cache = ref_cache.OmniKVLazyCache(offload_start_id=1, num_total_layers=3, skip_threshold=thr)
        cache.mamba_k = torch.arange(c["P"] * 4, dtype=torch.float32).view(1, c["P"], 4)
        cache.mamba_v = -cache.mamba_k
        applied, scores, live_sum = [], [], []
        for idx in seq:
            t = torch.from_numpy(idx)
            scores.append(float(ref_cache.get_idx_iou_score(t.view(-1), cache.idx[1].view(-1))) if 1 in cache.idx else -1.0)
            cache.set_out_idx(t, 1)
            applied.append(bool(torch.equal(cache.idx[1], t)))
            # the staged rows follow the live selection: row j of part_key[1] is token live[j]
            live_sum.append(float(cache.part_key[1][0, 0, :].sum()))
        res[str(thr)] = dict(applied=applied, scores=scores, live_sum=live_sum)
    (HERE / "lazy_rule.json").write_text(json.dumps(dict(c, input_checksum=checksum(seq), results=res)))
    print("lazy rule:", {k: sum(v["applied"]) for k, v in res.items()}, "re-gathers of", c["steps"])


class _StubAttention(torch.nn.Module):
    """Stand-in for the third-party attention module the reference's layer calls (transformers 4.41.2
    ``LlamaAttention``, absent from the reference tree): projections, rotation, ``past_key_value.update`` and plain
    softmax attention, with that version's call signature and 3-tuple return.  Everything the FILTER HOOK does --
    window capture, k / consider_len / nptw bookkeeping, the selector call, the appended window positions,
    ``set_idx_on_gpu`` -- is the reference's own ``OmniKVMulLayer.forward`` running around it."""

    def __init__(self, w, c, layer_idx):
        super().__init__()
        self.config = _Cfg()
        self.layer_idx = layer_idx
        self.num_heads, self.num_key_value_heads, self.head_dim = c["H"], c["KVH"], c["d"]
        self.num_key_value_groups = c["H"] // c["KVH"]
        self._theta = c["theta"]
        for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
            lin = torch.nn.Linear(1, 1, bias=False)
            lin.weight = torch.nn.Parameter(torch.from_numpy(w[f"self_attn.{name}.weight"]), requires_grad=False)
            setattr(self, name, lin)

    def rotary_emb(self, x, position_ids):
        inv_freq = 1.0 / (self._theta ** (torch.arange(0, self.head_dim, 2, dtype=torch.float32) / self.head_dim))
        freqs = position_ids.float()[:, :, None] * inv_freq[None, None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        return emb.cos(), emb.sin()

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                output_attentions=False, use_cache=False, cache_position=None):
        B, n, _ = hidden_states.shape
        H, KVH, d = self.num_heads, self.num_key_value_heads, self.head_dim
        q = self.q_proj(hidden_states).view(B, n, H, d).transpose(1, 2)
        k = self.k_proj(hidden_states).view(B, n, KVH, d).transpose(1, 2)
        v = self.v_proj(hidden_states).view(B, n, KVH, d).transpose(1, 2)
        cos, sin = self.rotary_emb(v, position_ids)

        def rot(x):
            h = x.shape[-1] // 2
            return x * cos.unsqueeze(1) + torch.cat((-x[..., h:], x[..., :h]), dim=-1) * sin.unsqueeze(1)

        q, k = rot(q), rot(k)
        k, v = past_key_value.update(k, v, self.layer_idx)
        m = k.shape[2]
        k = k[:, :, None].expand(B, KVH, H // KVH, m, d).reshape(B, H, m, d)
        v = v[:, :, None].expand(B, KVH, H // KVH, m, d).reshape(B, H, m, d)
        s = torch.matmul(q, k.transpose(2, 3)) / math.sqrt(d)
        if n > 1:
            s = s + torch.full((n, m), float("-inf")).triu(1 + m - n)
        o = torch.matmul(torch.softmax(s, dim=-1), v).transpose(1, 2).reshape(B, n, H * d)
        return self.o_proj(o), None, past_key_value


def make_layer_hook_fixture(ref_omnikv, ref_cache):
    """The reference's ``OmniKVMulLayer.forward`` (modeling/omnikv.py:143-246) on a six-layer stack: a prefill of
    P hidden states, then 20 decode forwards, for the selectors ``last``, ``uniform`` and ``exp``.  The layer objects
    are created without transformers' constructor (whose signature changed after 4.41.2) and given exactly the
    attributes the reference's ``__init__`` sets (:114-141).  Stored: every filter layer's index list at every
    decode forward and the stack's output hidden state of every forward."""
    from inputs import LAYER_HOOK, layer_hook_inputs
    c = LAYER_HOOK
    x = layer_hook_inputs()
    # transformers 4.41.2's DynamicCache.__len__ is the number of layers held, which is what makes the reference's
    # `if past_key_value:` true; 5.x returns 0 for this subclass.  Restore that meaning on the reference classes.
    for cls in (ref_cache.OmniKVMultiStageCache, ref_cache.WOPackCache):
        cls.__len__ = lambda self: len(self.key_cache)

    class Cfg:
        def __init__(self, **kw):
            self.__dict__.update(kw)

        def get(self, key, default=None):
            return self.__dict__.get(key, default)

    class Norm(torch.nn.Module):
        def __init__(self, w):
            super().__init__()
            self.w = torch.from_numpy(w)

        def forward(self, h):
            return h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + c["eps"]) * self.w

    class MLP(torch.nn.Module):
        def __init__(self, w):
            super().__init__()
            self.g, self.u, self.d = (torch.from_numpy(w[f"mlp.{n}_proj.weight"]) for n in ("gate", "up", "down"))

        def forward(self, h):
            return torch.nn.functional.linear(torch.nn.functional.silu(torch.nn.functional.linear(h, self.g)) *
                                              torch.nn.functional.linear(h, self.u), self.d)

    arrays = {}
    full = list(range(0, c["sel"][0])) + c["sel"] + [c["n_layers"]]
    for selector in ("last", "uniform", "exp"):
        cfg = Cfg(cache_cls="multi", do_select_layers=",".join(map(str, c["sel"])), selector_cls=selector,
                  window_size=c["window"], num_of_selected_tokens=c["frac"], dense_more=True)
        layers = []
        for i, w in enumerate(x["layers"]):
            layer = object.__new__(ref_omnikv.OmniKVMulLayer)
            torch.nn.Module.__init__(layer)
            layer.self_attn = _StubAttention(w, c, i)
            layer.mlp = MLP(w)
            layer.input_layernorm = Norm(w["input_layernorm.weight"])
            layer.post_attention_layernorm = Norm(w["post_attention_layernorm.weight"])
            layer.config, layer.layer_idx, layer.prefill_len = cfg, i, None
            layer.cache_cls = ref_cache.get_cache_cls(cfg)
            layer.do_select_layers = list(c["sel"])
            layer.hidden_state_window, layer.selector_cls = None, selector
            layer.window_size, layer.decode_step = c["window"], 0
            layers.append(layer)
        dyn = types.SimpleNamespace(key_cache=[], value_cache=[], _seen_tokens=0)
        cache = ref_cache.OmniKVMultiStageCache.from_dynamic_cache(dyn, full, c["n_layers"], c["wait"], False)
        seen = {}
        orig_set = cache.set_idx_on_gpu

        def spy(idx, layer_idx, _orig=orig_set, _seen=seen):
            _seen[layer_idx] = idx.clone()
            return _orig(idx, layer_idx)

        cache.set_idx_on_gpu = spy
        P = c["P"]
        with torch.no_grad():
            cache.stage = "prefill"   # modeling/omnikv.py:343-346: the LM sets the stage from the number of tokens
            h = torch.from_numpy(x["x_pre"])
            pos = torch.arange(P)[None, :]
            for layer in layers:
                h = layer(h, position_ids=pos, past_key_value=cache, use_cache=True)[0]
            arrays[f"{selector}/h/prefill"] = h[:, -1].numpy().copy()
            for s in range(c["steps"]):
                cache.stage = "decoding"
                h = torch.from_numpy(x["x_dec"][s])
                pos = torch.tensor([[P + s]])
                for layer in layers:
                    h = layer(h, position_ids=pos, past_key_value=cache, use_cache=True)[0]
                arrays[f"{selector}/h/{s}"] = h[:, -1].numpy().copy()
                for f in c["sel"]:
                    arrays[f"{selector}/idx/{s}/{f}"] = seen[f].numpy().astype(np.int32)
    np.savez_compressed(HERE / "layer_hook.npz", **arrays)
    flat = [a for w in x["layers"] for a in w.values()] + [x["x_pre"]] + x["x_dec"]
    (HERE / "layer_hook.json").write_text(json.dumps(dict(c, full=full, input_checksum=checksum(flat))))
    print("layer hook arrays:", len(arrays))


def make_rope_fixture(ref_root):
    """inv_freq and attention scaling of every ``rope_type`` from the reference's ROPE_INIT_FUNCTIONS
    (modeling/patch_of_llama3_1.py:336-343), and the dynamic-NTK frequencies its PatchLlamaRotaryEmbedding
    (:545-629) holds after each forward of a conversation that grows past, and falls back under, the trained length."""
    import modeling.patch_of_llama3_1 as ref_rope
    from inputs import ROPE_CASES, ROPE_DYNAMIC_SEQ
    arrays, meta = {}, []
    for case in ROPE_CASES:
        cfg = types.SimpleNamespace(**{k: v for k, v in case.items() if k != "name"})
        cfg.hidden_size, cfg.num_attention_heads = case["head_dim"] * 4, 4
        kind = "default" if case["rope_scaling"] is None else case["rope_scaling"].get("rope_type", case["rope_scaling"].get("type"))
        inv, att = ref_rope.ROPE_INIT_FUNCTIONS[kind](cfg, "cpu")
        arrays[f"{case['name']}/inv_freq"] = inv.numpy().astype(np.float32)
        meta.append(dict(name=case["name"], attention_scaling=float(att)))
    d = ROPE_DYNAMIC_SEQ
    cfg = types.SimpleNamespace(**{k: v for k, v in d.items() if k != "forwards"})
    cfg.hidden_size, cfg.num_attention_heads = d["head_dim"] * 4, 4
    emb = ref_rope.PatchLlamaRotaryEmbedding(config=cfg)
    for i, (first, n) in enumerate(d["forwards"]):
        pos = torch.arange(first, first + n)[None, :]
        cos, sin = emb(torch.zeros(1, 1, dtype=torch.float32), pos)
        arrays[f"dynamic_seq/{i}/inv_freq"] = emb.inv_freq.numpy().astype(np.float32).copy()
        arrays[f"dynamic_seq/{i}/cos_last"] = cos[0, -1].numpy().copy()
    np.savez_compressed(HERE / "rope.npz", **arrays)
    (HERE / "rope.json").write_text(json.dumps(dict(cases=meta)))
    print("rope arrays:", len(arrays))


def make_lightllm_fixture(ref_root):
    """The fork's own Triton kernels (omnikv-lightllm/lightllm/models/llama_omnikv/triton_kernel/
    flash_decoding_stage1.py, flash_decoding_stage2.py), loaded by path and run on CPU tensors by Triton's
    interpreter (TRITON_INTERPRET=1, set in main() before triton is imported), called as
    token_decode_attention_flash_decoding calls them (flash_decoding.py:57-93 for the selecting call, :176-214 for
    the plain one): outputs, the per-position score (max over heads of what the kernel writes to Attn_Score), the
    top-2048 choice and the attention over the chosen rows of another layer's pool."""
    import importlib.util
    base = os.path.join(ref_root, "omnikv-lightllm", "lightllm", "models", "llama_omnikv", "triton_kernel")
    mods = {}
    for name in ("flash_decoding_stage1", "flash_decoding_stage2"):
        spec = importlib.util.spec_from_file_location("ref_" + name, os.path.join(base, name + ".py"))
        mods[name] = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mods[name])
    s1, s2 = mods["flash_decoding_stage1"], mods["flash_decoding_stage2"]
    c, x = gi.LIGHTLLM, gi.lightllm_inputs()
    H, KVH, d, BS = c["H"], c["KVH"], c["d"], 256  # BLOCK_SEQ of flash_decoding.py:24
    t = {k: torch.from_numpy(v) for k, v in x.items()}
    table = t["table"]

    def run(q, pool, tab, reqs, lens, with_score):
        B, max_len = q.shape[0], int(max(lens))
        b_req, b_len = torch.tensor(reqs, dtype=torch.int32), torch.tensor(lens, dtype=torch.int32)
        mid_o = torch.zeros(B, H, max_len // BS + 1, d)
        mid_l = torch.zeros(B, H, max_len // BS + 1)
        o = torch.zeros(B, H, d)
        k, v = pool[:, :KVH], pool[:, KVH:]
        score = None
        if with_score:
            score = torch.zeros(B, H, max_len)
            s1.flash_decode_stage1_with_score(q, k, v, tab, b_req, b_len, max_len, mid_o, mid_l, score, BS)
        else:
            s1.flash_decode_stage1(q, k, v, tab, b_req, b_len, max_len, mid_o, mid_l, BS)
        s2.flash_decode_stage2(mid_o, mid_l, b_len, o, BS)
        return o, score

    req, L = c["select"]["req"], c["select"]["L"]
    sel_out, score = run(t["q_sel"], t["pool"], table, [req], [L], True)
    score_max = score.max(dim=1).values[0]                      # flash_decoding.py:75
    n_imp = min(c["k"], L)                                       # :79
    _, topk_idx = torch.topk(score_max[:L], dim=-1, k=n_imp)     # :80-82
    imp = torch.zeros(c["n_requests"], c["k"], dtype=torch.int32)
    imp[req, :n_imp] = torch.index_select(table[req, :L], dim=-1, index=topk_idx)  # :85-93
    sparse_out, _ = run(t["q_sparse"], t["pool2"], imp, [req], [n_imp], False)    # a later layer over the chosen rows
    dense_out, _ = run(t["q_dense"], t["pool"], table, c["dense"]["reqs"], c["dense"]["lens"], False)
    np.savez_compressed(HERE / "lightllm.npz", sel_out=sel_out.numpy(), score_max=score_max.numpy(),
                        topk_idx=topk_idx.numpy().astype(np.int32),
                        sel_pos_sorted=np.sort(topk_idx.numpy()).astype(np.int32), sparse_out=sparse_out.numpy(),
                        dense_out=dense_out.numpy())
    (HERE / "lightllm.json").write_text(json.dumps(dict(cfg=c, inputs_checksum=gi.checksum(list(x.values())),
                                                        block_seq=BS, triton="interpreter mode on CPU tensors")))
    print("lightllm: selected", n_imp, "of", L)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the OmniKV checkout")
    ap.add_argument("--only", default="", help="generate one fixture only (e.g. lightllm)")
    args = ap.parse_args()
    os.environ["TRITON_INTERPRET"] = "1"  # the fork's Triton kernels run on CPU tensors (before triton is imported)
    if args.only == "lightllm":
        return make_lightllm_fixture(os.path.abspath(args.reference))
    ref_omnikv, ref_cache = import_reference(os.path.abspath(args.reference))
    torch.set_num_threads(8)
    make_selector_fixture(ref_omnikv)
    make_plan_fixture(ref_cache)
    make_cache_flow_fixture(ref_cache)
    make_cache_flow_d128_fixture(ref_cache)
    make_operator_fixture(ref_omnikv, ref_cache)
    make_lazy_rule_fixture(ref_cache)
    make_layer_hook_fixture(ref_omnikv, ref_cache)
    make_rope_fixture(os.path.abspath(args.reference))
    make_lightllm_fixture(os.path.abspath(args.reference))


if __name__ == "__main__":
    main()
