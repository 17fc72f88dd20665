"""Host-side logic that needs no GPU: config semantics, layer plan, the C ABI's symbols."""
import ctypes
import json
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
G = ROOT / "tests" / "golden"


def test_config_get_writes_default_back():
    from omnikv_b200.modeling import LlamaCompressorConfig
    c = LlamaCompressorConfig()
    assert not hasattr(c, "window_size")
    assert c.get("window_size", 16) == 16
    assert c.window_size == 16            # written back, as modeling/omnikv_config.py:15-19
    assert c.get("window_size", 99) == 16
    c.set_config_of_compressor(**json.loads((ROOT / "tests" / "golden" / "example_config.json").read_text()))
    assert c.get("do_select_layers") == "2,8,18" and c.get("num_of_selected_tokens") == 0.067
    assert c.get("selector_cls", "softmax_before_last") == "last" and c.get("real_offload", True) is False


@pytest.mark.parametrize("cls_name", ["OmniKVMultiStageCache", "WOPackCache"])
def test_layer_plan_matches_reference_fixture(cls_name):
    from omnikv_b200.modeling import spec_cache
    cls = getattr(spec_cache, cls_name)
    rows = [r for r in json.loads((G / "layer_plan.json").read_text()) if r["cls"] == cls_name]
    assert rows
    for row in rows:
        assert spec_cache.full_attn_layers_of(row["do_select"], row["num_layers"]) == row["full_attn_layers"]
        c = cls.from_dynamic_cache(None, row["full_attn_layers"], row["num_layers"], row["wait"], False)
        want = {int(k): (bool(v[0]), v[1], v[2]) for k, v in row["layer_state"].items()}
        assert c.layer_state == want, row
        assert c.stage == "prefill" and c.device is None
    c = cls([0, 2], 2, 0, True)
    assert c.device == "cpu"


def test_llama3_8b_plan_counts():
    from omnikv_b200.modeling import spec_cache
    c = spec_cache.OmniKVMultiStageCache(spec_cache.full_attn_layers_of([2, 8, 18], 32), 32, 1, False)
    dense = sorted(i for i, s in c.layer_state.items() if not s[0])
    assert dense == [0, 1, 2, 3, 8, 9, 18, 19]
    assert c.groups == {2: [4, 5, 6, 7], 8: list(range(10, 18)), 18: list(range(20, 32))}


def test_get_cache_cls():
    from omnikv_b200.modeling import LlamaCompressorConfig, OmniKVMultiStageCache, WOPackCache, get_cache_cls
    c = LlamaCompressorConfig()
    c.set_config_of_compressor(cache_cls="multi")
    assert get_cache_cls(c) is OmniKVMultiStageCache
    c.cache_cls = "without_pack"
    assert get_cache_cls(c) is WOPackCache
    from omnikv_b200.modeling import OmniKVLazyCache
    c.cache_cls = "lazy"
    assert get_cache_cls(c) is OmniKVLazyCache
    lz = OmniKVLazyCache.from_dynamic_cache(None, [0, 1, 4], 4, 1, False, skip_threshold=0.7)
    assert lz.skip_threshold == 0.7 and lz.layer_state == OmniKVMultiStageCache([0, 1, 4], 4, 1, False).layer_state
    c.cache_cls = "eff"
    with pytest.raises(NotImplementedError):
        get_cache_cls(c)


def test_library_exports_every_declared_symbol():
    from omnikv_b200 import abi
    header = (ROOT / "include" / "omnikv_b200.h").read_text()
    declared = set(re.findall(r"\b(omnikv_[a-z0-9_]+)\s*\(", header))
    assert declared == set(abi.SIGNATURES), declared ^ set(abi.SIGNATURES)
    lib = abi.lib()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.omnikv_abi_version() == abi.ABI_VERSION == int(re.search(r"OMNIKV_ABI_VERSION (\d+)", header).group(1))
    assert b"workspace" in lib.omnikv_strerror(-3)
    assert lib.omnikv_decode_attn_workspace_bytes(1, 32, 37) == 16384 + (32 * 37 * 128 + 32 * 37 * 2) * 4
    assert lib.omnikv_topk_workspace_bytes(2, 1000) == 2 * 1000 * 4


def test_bad_arguments_are_rejected_on_the_host():
    """Validation happens before any launch, so it can be exercised without a GPU."""
    from omnikv_b200 import abi
    lib = abi.lib()
    p = abi.AttnParams()
    assert lib.omnikv_decode_attn(ctypes.byref(p), None) == -1          # null pointers
    p.q = p.kA = p.vA = p.lenA = p.out = 256
    p.B, p.H, p.KVH, p.head_dim, p.n_splits = 1, 32, 8, 64, 4
    assert lib.omnikv_decode_attn(ctypes.byref(p), None) == -2          # head_dim 64 unsupported
    p.head_dim = 128
    p.q_stride_b, p.q_stride_h, p.a_stride_b, p.a_stride_h, p.a_stride_row = 4096, 128, 1 << 20, 1 << 17, 128
    p.dtype = abi.BF16
    assert lib.omnikv_decode_attn(ctypes.byref(p), None) == -3          # no workspace
    p.H = 30
    assert lib.omnikv_decode_attn(ctypes.byref(p), None) == -1          # H % KVH != 0
    assert lib.omnikv_topk(None, 1, 0, 0, None, None, None, 1, 10, None, 10, None, None, 0, None) == -1
    with pytest.raises(abi.OmniKVError):
        abi.check(-2, "x")


def test_ops_refuse_cpu_tensors():
    from omnikv_b200 import abi, ops
    q = torch.zeros(1, 32, 128)
    k = torch.zeros(1, 8, 16, 128)
    with pytest.raises(abi.OmniKVError):
        ops.decode_attn(q, k, k, torch.zeros(1, dtype=torch.int32))


def test_product_package_does_not_import_the_oracle():
    for f in (ROOT / "omnikv_b200").rglob("*.py"):
        text = f.read_text()
        assert "import oracle" not in text and "from oracle" not in text, f


def test_cache_refuses_to_overflow_its_reserve():
    from omnikv_b200.modeling import OmniKVMultiStageCache
    c = OmniKVMultiStageCache([0, 2], 2, 0, False)
    c.prefill_len, c.reserve, c._seen_tokens = 100, 4, 103
    c.check_room(1)
    with pytest.raises(RuntimeError, match="KV cache is full"):
        c.check_room(2)


def test_paged_oracle_consistency():
    """The paged-pool oracle: keeping every token equals dense attention; kept positions are ascending and
    end with the forced recent ones."""
    import torch
    from oracle import lightllm_oracle as lo

    g = torch.Generator().manual_seed(0)
    KVH, H, d, n = 2, 4, 128, 300
    pool = torch.randn(512, 2 * KVH, d, generator=g)
    table = torch.zeros(3, 400, dtype=torch.int32)
    table[2, :n] = torch.randperm(512, generator=g)[:n].to(torch.int32)
    q = torch.randn(1, H, d, generator=g)
    req, lens = torch.tensor([2]), [n]
    dense = lo.paged_decode_attention(q, pool[:, :KVH], pool[:, KVH:], table, req, lens)
    pos_all = lo.select_positions(q, pool[:, :KVH], table, req, lens, num_imp_tokens=2048)
    assert torch.equal(pos_all[0], torch.arange(n))
    again = lo.selected_decode_attention(q, pool[:, :KVH], pool[:, KVH:], table, req, pos_all)
    assert torch.allclose(dense, again, atol=1e-6)
    pos = lo.select_positions(q, pool[:, :KVH], table, req, lens, num_imp_tokens=64, keep_recent=5)[0]
    assert pos.numel() == 64 and torch.equal(pos[-5:], torch.arange(n - 5, n))
    assert torch.equal(pos, torch.sort(pos).values)


def test_index_tracer_roundtrip(tmp_path):
    """The recorder's pickle has the reference's layout and its reader returns the four parts."""
    import torch
    from omnikv_b200 import tensor_tools as tt

    tr = tt.SelectedIndexTracer(desc="cpu", directory=str(tmp_path / "logs"))
    tr.append_spec_layer(torch.tensor([[1, 5, 9]]), torch.tensor([[0.5, 0.25, 2.0]]), 100, 8)
    tr.append_spec_layer(torch.tensor([[2, 5, 7]]), torch.tensor([[1.5, 0.25, 0.1]]), 100, 8)
    tr.append(torch.tensor([3]), torch.tensor([0.1]))
    tr.append_prefill(torch.tensor([[4]]), torch.tensor([[0.3]]), 8)
    tr.append_out(("pred", "truth"))
    with pytest.raises(AssertionError):
        tr.append_spec_layer(torch.tensor([1]), torch.tensor([1.0]), 100, 8)
    tr.save_idx()
    assert tr.num_samples == 1
    idx, out, layers_idx, prefill_res = tt.read_idx_tracer(tr.save_path)
    assert out == [("pred", "truth")]
    assert [r["idx"].tolist() for r in layers_idx[0][8]] == [[[1, 5, 9]], [[2, 5, 7]]]
    assert layers_idx[0][8][0]["prefill_len"] == 100
    assert idx[0][0]["idx"].tolist() == [3] and prefill_res[0]["idx"].tolist() == [[4]]
    prev = tt.set_tracer(tr)
    assert tt.idx_tracer is tr and tt.set_tracer(prev) is tr and tt.idx_tracer is prev


def test_rope_parameters_match_reference():
    """inv_freq and attention scaling of every rope_type against what the reference's ROPE_INIT_FUNCTIONS returned
    (fixture), and dynamic-NTK scaling followed through a conversation that outgrows the trained length, falls
    back under it and grows again, against the reference's rotary module after each forward."""
    import numpy as np
    import torch

    import inputs as gi
    from omnikv_b200.modeling import LlamaCompressorConfig
    from omnikv_b200.modeling.omnikv import OmniKVRotaryEmbedding, rope_parameters
    gold = np.load(G / "rope.npz")
    meta = {m["name"]: m for m in json.loads((G / "rope.json").read_text())["cases"]}
    for case in gi.ROPE_CASES:
        cfg = LlamaCompressorConfig(**{k: v for k, v in case.items() if k != "name"})
        inv, att = rope_parameters(cfg)
        np.testing.assert_allclose(inv.numpy(), gold[f"{case['name']}/inv_freq"], rtol=2e-6, atol=0, err_msg=case["name"])
        assert att == pytest.approx(meta[case["name"]]["attention_scaling"], rel=1e-12), case["name"]
    d = gi.ROPE_DYNAMIC_SEQ
    cfg = LlamaCompressorConfig(**{k: v for k, v in d.items() if k != "forwards"})
    emb = OmniKVRotaryEmbedding(cfg)
    for i, (first, n) in enumerate(d["forwards"]):
        pos = torch.arange(first, first + n)[None, :]
        emb.advance(pos, prefill=n > 1)
        np.testing.assert_allclose(emb.inv_freq.numpy(), gold[f"dynamic_seq/{i}/inv_freq"], rtol=2e-6, atol=0, err_msg=str(i))
        cos, _ = emb(torch.zeros(1, dtype=torch.float32), pos)
        np.testing.assert_allclose(cos[0, -1].numpy(), gold[f"dynamic_seq/{i}/cos_last"], atol=2e-4, rtol=0)


def test_attention_split_counts_on_a_148_sm_device(monkeypatch):
    """The split-count model of decode attention (host logic): bounds and the cases it was tuned on."""
    from omnikv_b200 import ops
    monkeypatch.setattr(ops, "sm_count", lambda device: 148)
    dev = torch.device("cpu")
    # one sequence: two CTAs per SM, never more splits than SMs
    assert ops.default_splits(1, 8, 131073, dev) == 37
    assert ops.default_splits(1, 2, 131073, dev) == 148
    assert ops.default_splits(1, 1, 131073, dev) == 148
    # the selected rows of a batch's sparse layers: few splits (fixed cost per CTA), more when the batch is small
    assert ops.default_splits(16, 8, 2112, dev) == 2
    assert ops.default_splits(8, 1, 4391, dev) > ops.default_splits(16, 8, 2112, dev)
    # ragged long batches: two waves of equal CTAs
    assert ops.default_splits(16, 8, 32832, dev) == 5
    # never below one, never less than 128 rows per split
    for B, KVH, rows in [(1, 8, 1), (1, 8, 100), (1, 8, 300), (4, 8, 200), (64, 8, 129), (3, 1, 7000)]:
        s = ops.default_splits(B, KVH, rows, dev)
        assert 1 <= s <= max(1, (rows + 127) // 128), (B, KVH, rows, s)
