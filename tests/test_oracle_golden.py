"""The CPU oracle against the fixtures produced by the reference's own code."""
import json
import types
from pathlib import Path

import numpy as np
import pytest
import torch

import inputs as gi
import oracle

G = Path(__file__).resolve().parent / "golden"


class _Attn:
    def __init__(self, wq, h, kvh, d, theta):
        self.num_heads, self.num_key_value_heads, self.head_dim, self.layer_idx = h, kvh, d, 0
        self._wq, self._theta = wq, theta

    def q_proj(self, x):
        return x @ self._wq.T

    def rotary_emb(self, x, position_ids):
        return oracle.rope_cos_sin(position_ids, self.head_dim, self._theta)


SEL_META = json.loads((G / "selector_small.json").read_text())
SEL = np.load(G / "selector_small.npz")


def _sets_match_up_to_ties(scores, got, want, k):
    """Equal, or differing only on positions whose score ties the k-th one (torch.topk leaves ties open)."""
    if np.array_equal(got, want):
        return True
    for b in range(scores.shape[0]):
        s = scores[b]
        kth = np.sort(s)[::-1][min(k, len(s)) - 1]
        diff = set(got[b].tolist()) ^ set(want[b].tolist())
        if any(abs(s[i] - kth) > 1e-6 for i in diff):
            return False
    return True


@pytest.mark.parametrize("case", SEL_META, ids=[c["name"] for c in SEL_META])
def test_selector_matches_reference(case):
    x = gi.selector_inputs(case)
    assert gi.checksum(x.values()) == pytest.approx(case["input_checksum"], rel=1e-12)
    attn = _Attn(torch.from_numpy(x["wq"]), case["H"], case["KVH"], case["d"], case["theta"])
    cache = types.SimpleNamespace(key_cache=[torch.from_numpy(x["kc"])])
    hs = torch.from_numpy(x["hs"])
    pos = torch.full((case["B"], 1), case["pos"], dtype=torch.long)
    for k in case["ks"]:
        want = SEL[f"{case['name']}/k{k}"]
        got = oracle.select_tokens_by_attn_universal(attn, hs, pos, cache, k, case["L"], 0, case["selector"]).numpy()
        assert got.shape == want.shape and got.dtype == np.int64
        assert np.all(np.diff(got, axis=1) > 0)
        if not np.array_equal(got, want):
            # recompute the score to allow exact ties at the threshold only
            q = attn.q_proj(hs).view(case["B"], case["W"], case["H"], case["d"]).transpose(1, 2)
            q = oracle.apply_rope(q, *attn.rotary_emb(q, pos))
            kc = cache.key_cache[0]
            s = (oracle.score_last(q[:, :, -1], kc, case["L"]) if case["selector"] == "last"
                 else oracle.score_window(q, kc, case["L"], case["selector"])).numpy()
            assert _sets_match_up_to_ties(s, got, want, k), (case["name"], k)


def test_layer_plan_matches_reference():
    for row in json.loads((G / "layer_plan.json").read_text()):
        assert oracle.omnikv_oracle.full_attn_layers_of(row["do_select"], row["num_layers"]) == row["full_attn_layers"]
        got = oracle.layer_plan(row["full_attn_layers"], row["num_layers"], row["wait"])
        want = {int(k): (bool(v[0]), v[1], v[2]) for k, v in row["layer_state"].items()}
        assert got == want, row


@pytest.mark.parametrize("cls_name", ["OmniKVMultiStageCache", "WOPackCache"])
def test_cache_flow_matches_reference(cls_name):
    c = json.loads((G / "cache_flow.json").read_text())
    gold = np.load(G / "cache_flow.npz")
    x = gi.cache_flow_inputs()
    t = torch.from_numpy
    cls = oracle.OracleMultiStageCache if cls_name == "OmniKVMultiStageCache" else oracle.OracleWOPackCache
    cache = cls(c["full"], c["n_layers"], c["wait"], False)
    for i in range(c["n_layers"]):
        cache.update(t(x["k_pre"][i]), t(x["v_pre"][i]), i)
    for s in range(c["steps"]):
        cache.stage = "decoding"
        for i in range(c["n_layers"]):
            if i in c["sel"]:
                cache.set_idx_on_gpu(t(x["idx"][(s, i)]), i)
            kk, vv = cache.update(t(x["k_new"][s][i]), t(x["v_new"][s][i]), i)
            np.testing.assert_array_equal(kk.numpy(), gold[f"{cls_name}/ret_k/{s}/{i}"])
            np.testing.assert_array_equal(vv.numpy(), gold[f"{cls_name}/ret_v/{s}/{i}"])
    assert cache._seen_tokens == int(gold[f"{cls_name}/seen"][0])


def test_operator_case_matches_reference():
    o = json.loads((G / "operator_cfg1.json").read_text())
    gold = np.load(G / "operator_cfg1.npz")
    x = gi.operator_inputs()
    assert gi.checksum([x[n] for n in ("q", "k", "k2", "v2", "k_new", "v_new")]) == pytest.approx(o["input_checksum"], rel=1e-12)
    q = torch.from_numpy(x["q"])
    kf = torch.from_numpy(x["k"])
    s = oracle.score_last(q[:, :, -1], kf, o["L"])
    idx = oracle.topk_ascending(s, o["k"])
    assert _sets_match_up_to_ties(s.numpy(), idx.numpy(), gold["idx"].astype(np.int64), o["k"])
    out = oracle.sparse_attention(q[:, :, -1], torch.from_numpy(x["k2"]), torch.from_numpy(x["v2"]),
                                  torch.from_numpy(gold["idx"].astype(np.int64)),
                                  torch.from_numpy(x["k_new"]), torch.from_numpy(x["v_new"]))
    np.testing.assert_allclose(out.numpy(), gold["out"], atol=1e-5, rtol=0)
    for sel in ("uniform", "exp"):
        sw = oracle.score_window(q, kf, o["L"], sel)
        got = oracle.topk_ascending(sw, o["k"]).numpy()
        want = gold[f"idx_{sel}"].astype(np.int64)
        # fp32 summation order may differ: positions may differ only inside a 1e-7 band around the threshold
        diff = set(got[0].tolist()) ^ set(want[0].tolist())
        kth = np.sort(sw.numpy()[0])[::-1][o["k"] - 1]
        assert all(abs(sw.numpy()[0, i] - kth) < 1e-7 for i in diff)


def test_k_rule():
    # int() truncation of the fractional k (the reference's rule), window bookkeeping
    assert oracle.selector_k_rule(0.067, 16384, "last", 16, 1) == (1097, 16384, 0)
    assert oracle.selector_k_rule(0.067, 131072, "last", 16, 5) == (8781, 131072, 0)
    assert oracle.selector_k_rule(2048, 20000, "exp", 16, 1) == (2033, 19985, 15)
    assert oracle.selector_k_rule(2048, 20000, "exp", 16, 40) == (2048, 20000, 0)
    assert oracle.selector_k_rule(3, 100, "uniform", 16, 2) == (1, 86, 14)


@pytest.mark.parametrize("thr", ["0.4", "0.7", "0.95"])
def test_lazy_rule_matches_reference(thr):
    """Which steps re-gather, the overlap scores and the rows in use, against the reference's
    OmniKVLazyCache.set_out_idx run on the same drifting index sequence."""
    meta = json.loads((G / "lazy_rule.json").read_text())
    seq = gi.lazy_rule_inputs()
    assert abs(gi.checksum(seq) - meta["input_checksum"]) < 1e-6 * max(1.0, abs(meta["input_checksum"]))
    gold = meta["results"][thr]
    rule = oracle.OracleLazyRule(float(thr))
    for s, idx in enumerate(seq):
        taken, score = rule.offer(torch.from_numpy(idx), 1)
        assert taken == gold["applied"][s]
        assert abs(score - gold["scores"][s]) < 1e-9
        # fixture rows: feature 0 of token t is 4 t, so the sum identifies the list in use
        assert float(rule.live[1].sum()) * 4.0 == gold["live_sum"][s]


def hook_model_inputs():
    """(config dict, HF-named fp32 weights, x_pre, x_dec list) of the layer-hook fixture."""
    c = json.loads((G / "layer_hook.json").read_text())
    x = gi.layer_hook_inputs()
    flat = [a for w in x["layers"] for a in w.values()] + [x["x_pre"]] + x["x_dec"]
    assert gi.checksum(flat) == pytest.approx(c["input_checksum"], rel=1e-12)
    weights = {f"model.layers.{i}.{k}": torch.from_numpy(v) for i, w in enumerate(x["layers"]) for k, v in w.items()}
    cfg = dict(num_hidden_layers=c["n_layers"], hidden_size=c["hidden"], intermediate_size=c["inter"],
               num_attention_heads=c["H"], num_key_value_heads=c["KVH"], head_dim=c["d"], rope_theta=c["theta"],
               rms_norm_eps=c["eps"], do_select_layers=",".join(map(str, c["sel"])), num_wait_load_layers=c["wait"],
               num_of_selected_tokens=c["frac"], window_size=c["window"], cache_cls="multi", real_offload=False,
               dense_more=True)
    return c, cfg, weights, x


@pytest.mark.parametrize("selector", ["last", "uniform", "exp"])
def test_layer_hook_matches_reference(selector):
    """The restated filter-layer hook (oracle.llama_oracle.OracleLM._layer) against the reference's own
    OmniKVMulLayer.forward: same index lists at every decode forward of both filter layers, same hidden states."""
    from oracle.llama_oracle import OracleLM
    c, cfg, weights, x = hook_model_inputs()
    gold = np.load(G / "layer_hook.npz")
    lm = OracleLM(dict(cfg, selector_cls=selector), weights)
    h, cache = lm.forward_hidden(torch.from_numpy(x["x_pre"]))
    np.testing.assert_allclose(h[:, -1].numpy(), gold[f"{selector}/h/prefill"], atol=2e-5, rtol=0)
    for s in range(c["steps"]):
        h, cache = lm.forward_hidden(torch.from_numpy(x["x_dec"][s]), cache, fwd_no=s)
        for f in c["sel"]:
            want = gold[f"{selector}/idx/{s}/{f}"]
            got = lm.selected[(s, f)].numpy()
            assert got.shape == want.shape, (s, f)
            assert np.array_equal(got, want), (selector, s, f, len(set(got[0].tolist()) ^ set(want[0].tolist())))
        np.testing.assert_allclose(h[:, -1].numpy(), gold[f"{selector}/h/{s}"], atol=5e-5, rtol=0)


@pytest.mark.parametrize("cls_name", ["OmniKVMultiStageCache", "WOPackCache"])
def test_cache_flow_d128_matches_reference(cls_name):
    """The flow at head size 128 (the fixture the CUDA caches are checked against), by signature."""
    c = json.loads((G / "cache_flow_d128.json").read_text())
    x = gi.cache_flow_inputs(gi.CACHE_FLOW_D128)
    flat = x["k_pre"] + x["v_pre"] + [a for r in x["k_new"] for a in r] + [a for r in x["v_new"] for a in r]
    assert gi.checksum(flat) == pytest.approx(c["input_checksum"], rel=1e-12)
    t = torch.from_numpy
    cls = oracle.OracleMultiStageCache if cls_name == "OmniKVMultiStageCache" else oracle.OracleWOPackCache
    cache = cls(c["full"], c["n_layers"], c["wait"], False)
    for i in range(c["n_layers"]):
        cache.update(t(x["k_pre"][i]), t(x["v_pre"][i]), i)
    for s in range(c["steps"]):
        cache.stage = "decoding"
        for i in range(c["n_layers"]):
            if i in c["sel"]:
                cache.set_idx_on_gpu(t(x["idx"][(s, i)]), i)
            kk, vv = cache.update(t(x["k_new"][s][i]), t(x["v_new"][s][i]), i)
            assert [gi.signature(kk.numpy()), gi.signature(vv.numpy())] == c["returns"][f"{cls_name}/{s}/{i}"]
    assert cache._seen_tokens == c["returns"][f"{cls_name}/seen"]


def test_lightllm_oracle_matches_the_forks_triton_kernels():
    """oracle/lightllm_oracle.py against what the fork's own Triton kernels produced (run by Triton's interpreter
    when the fixture was made): outputs of the selecting call and of the plain ragged call, the raw-logit scores,
    the top-2048 positions, and the attention of a later layer over exactly those rows."""
    from oracle import lightllm_oracle as lo
    meta = json.loads((G / "lightllm.json").read_text())
    gold = np.load(G / "lightllm.npz")
    c, x = gi.LIGHTLLM, gi.lightllm_inputs()
    assert meta["cfg"] == json.loads(json.dumps(c))
    assert abs(meta["inputs_checksum"] - gi.checksum(list(x.values()))) < 1e-6 * abs(meta["inputs_checksum"])
    t = {k: torch.from_numpy(v) for k, v in x.items()}
    KVH = c["KVH"]
    pk, pv, table = t["pool"][:, :KVH], t["pool"][:, KVH:], t["table"]
    req, L = c["select"]["req"], c["select"]["L"]
    out = lo.paged_decode_attention(t["q_sel"], pk, pv, table, [req], [L])
    assert np.abs(out.numpy() - gold["sel_out"]).max() <= 1e-5
    score = lo.fork_scores(t["q_sel"], pk, table, [req], [L])[0]
    assert np.abs(score.numpy() - gold["score_max"]).max() <= 1e-4  # raw logits of magnitude up to 40
    pos = lo.select_positions(t["q_sel"], pk, table, [req], [L], c["k"])[0]
    assert np.array_equal(pos.numpy().astype(np.int32), gold["sel_pos_sorted"])
    assert set(gold["topk_idx"].tolist()) == set(gold["sel_pos_sorted"].tolist())
    p2k, p2v = t["pool2"][:, :KVH], t["pool2"][:, KVH:]
    sparse = lo.selected_decode_attention(t["q_sparse"], p2k, p2v, table, [req], [pos])
    assert np.abs(sparse.numpy() - gold["sparse_out"]).max() <= 1e-5
    dense = lo.paged_decode_attention(t["q_dense"], pk, pv, table, c["dense"]["reqs"], c["dense"]["lens"])
    assert np.abs(dense.numpy() - gold["dense_out"]).max() <= 1e-5
