"""The LightLLM plug point over a paged KV pool, against the CPU oracle of the fork's semantics."""
from types import SimpleNamespace

import pytest
import torch

from oracle import lightllm_oracle as lo

pytestmark = pytest.mark.gpu


def _state(B, lens, H, KVH, d, dtype, seed, n_requests=6, max_seq=None, pool_tokens=None):
    """A shuffled pool: every request's tokens sit at random, non-contiguous pool rows."""
    g = torch.Generator().manual_seed(seed)
    max_seq = max_seq or (max(lens) + 16)
    pool_tokens = pool_tokens or (sum(lens) + 64)
    pool = torch.randn(pool_tokens, 2 * KVH, d, generator=g).to(dtype)
    perm = torch.randperm(pool_tokens, generator=g).to(torch.int32)
    table = torch.zeros(n_requests, max_seq, dtype=torch.int32)
    req_ids = torch.randperm(n_requests, generator=g)[:B].to(torch.int32)
    used = 0
    for b in range(B):
        table[req_ids[b], : lens[b]] = perm[used : used + lens[b]]
        used += lens[b]
    q = torch.randn(B, H * d, generator=g).to(dtype)
    # make a few keys stand out so that the selection is not a coin toss under bf16 rounding
    qm = q.view(B, H, d).float().mean(1)
    for b in range(B):
        hot = torch.randperm(lens[b], generator=g)[: max(4, lens[b] // 50)]
        rows = table[req_ids[b], hot].long()
        pool[rows, :KVH] += (3.0 * qm[b] / qm[b].norm()).to(dtype)
    imp = torch.zeros(8, n_requests, 2048 + 300, dtype=torch.int32)
    cuda = lambda t: t.cuda()  # noqa: E731
    req_manager = SimpleNamespace(req_to_token_indexs=cuda(table), req_to_imp_token_indexs=cuda(imp))
    st = SimpleNamespace(batch_size=B, max_len_in_batch=max(lens), b_seq_len=cuda(torch.tensor(lens, dtype=torch.int32)),
                         b_req_idx=cuda(req_ids), req_manager=req_manager, is_prefill=False, imp_seq_len=None,
                         max_imp_len_batch=0)
    return st, q, pool, table, req_ids


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float16, 2e-2), (torch.float32, 1e-4)])
@pytest.mark.parametrize("lens", [[3000], [5000, 777, 2049], [100]])
def test_dense_paged_attention(dtype, tol, lens):
    from omnikv_b200.lightllm_adapter import token_decode_attention_flash_decoding as attn
    H, KVH, d = 8, 2, 128
    st, q, pool, table, req = _state(len(lens), lens, H, KVH, d, dtype, seed=5)
    pool_d = pool.cuda()
    o = attn(q.cuda(), st, H, d, pool_d[:, :KVH], pool_d[:, KVH:])
    ref = lo.paged_decode_attention(q.view(-1, H, d), pool[:, :KVH], pool[:, KVH:], table, req, lens)
    assert o.shape == q.shape and o.dtype == dtype
    assert (o.float().cpu().view(-1, H, d) - ref).abs().max().item() < tol
    assert st.imp_seq_len is None


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-4)])
@pytest.mark.parametrize("lens,keep_recent", [([6000], 0), ([4100, 1500, 2048], 0), ([6000, 300], 8)])
def test_select_then_sparse(dtype, tol, lens, keep_recent):
    """A filter layer call followed by a later layer's call: same output as dense attention on the filter
    layer, selected rows recorded per request, and attention over exactly those rows afterwards."""
    from omnikv_b200.lightllm_adapter import token_decode_attention_flash_decoding as attn
    H, KVH, d, B = 8, 2, 128, len(lens)
    st, q, pool, table, req = _state(B, lens, H, KVH, d, dtype, seed=9)
    pool_d = pool.cuda()
    out = torch.empty(B, H * d, dtype=dtype, device="cuda")
    o = attn(q.cuda(), st, H, d, pool_d[:, :KVH], pool_d[:, KVH:], out=out, do_select=True, tp_rank=1,
             keep_recent=keep_recent)
    assert o is out
    q3 = q.view(B, H, d)
    ref = lo.paged_decode_attention(q3, pool[:, :KVH], pool[:, KVH:], table, req, lens)
    assert (o.float().cpu().view(B, H, d) - ref).abs().max().item() < tol
    want = lo.select_positions(q3, pool[:, :KVH], table, req, lens, 2048, keep_recent)
    counts = st.imp_seq_len.cpu().tolist()
    imp = st.req_manager.req_to_imp_token_indexs.cpu()
    assert st.max_imp_len_batch == min(2048, max(lens))
    got_pos = []
    for b in range(B):
        assert counts[b] == min(2048, lens[b]) == want[b].numel()
        rows = imp[1, int(req[b]), : counts[b]]
        inv = {int(r): p for p, r in enumerate(table[int(req[b]), : lens[b]].tolist())}
        pos = torch.tensor([inv[int(r)] for r in rows.tolist()])
        assert torch.equal(pos, torch.sort(pos).values)  # ascending positions
        got_pos.append(pos)
        if dtype == torch.float32:
            assert torch.equal(pos, want[b])
        else:  # 16-bit products: the sets may differ only at the k-th score boundary
            same = len(set(pos.tolist()) & set(want[b].tolist()))
            assert same >= counts[b] - max(2, counts[b] // 100)
    assert imp[0].abs().sum().item() == 0  # only this rank's table was written

    # a later layer: attention over the recorded rows of ITS pool (another layer's KV, same paging)
    g = torch.Generator().manual_seed(77)
    pool2 = torch.randn(pool.shape, generator=g).to(dtype)
    q2 = torch.randn(B, H * d, generator=g).to(dtype)
    pool2_d = pool2.cuda()
    o2 = attn(q2.cuda(), st, H, d, pool2_d[:, :KVH], pool2_d[:, KVH:], tp_rank=1)
    ref2 = lo.selected_decode_attention(q2.view(B, H, d), pool2[:, :KVH], pool2[:, KVH:], table, req, got_pos)
    assert (o2.float().cpu().view(B, H, d) - ref2).abs().max().item() < tol


def test_refuses_prefill_and_bad_types():
    from omnikv_b200.lightllm_adapter import token_decode_attention_flash_decoding as attn
    H, KVH, d = 8, 2, 128
    st, q, pool, table, req = _state(1, [256], H, KVH, d, torch.bfloat16, seed=1)
    pool_d = pool.cuda()
    st.is_prefill = True
    with pytest.raises(AssertionError):
        attn(q.cuda(), st, H, d, pool_d[:, :KVH], pool_d[:, KVH:])
    st.is_prefill = False
    st.b_seq_len = st.b_seq_len.long()
    with pytest.raises(TypeError):
        attn(q.cuda(), st, H, d, pool_d[:, :KVH], pool_d[:, KVH:])


def test_adapter_matches_the_forks_triton_kernels():
    """The adapter (fp32 pool, through the C ABI) on the inputs of tests/golden/lightllm.npz, whose outputs come from
    the fork's own Triton kernels: the selecting call's output, the recorded rows (the fork's top-2048 set, up to a
    band at the threshold), a later layer's attention over those rows, and the plain ragged call."""
    import json
    from pathlib import Path

    import numpy as np

    import inputs as gi
    from omnikv_b200.lightllm_adapter import token_decode_attention_flash_decoding as attn
    from parity import band_check
    G = Path(__file__).resolve().parent / "golden"
    gold = np.load(G / "lightllm.npz")
    c, x = gi.LIGHTLLM, gi.lightllm_inputs()
    meta = json.loads((G / "lightllm.json").read_text())
    assert abs(meta["inputs_checksum"] - gi.checksum(list(x.values()))) < 1e-6 * abs(meta["inputs_checksum"])
    H, KVH, d, k = c["H"], c["KVH"], c["d"], c["k"]
    t = {n: torch.from_numpy(v).cuda() for n, v in x.items()}
    req, L = c["select"]["req"], c["select"]["L"]

    def state(reqs, lens):
        imp = torch.zeros(2, c["n_requests"], k + 64, dtype=torch.int32, device="cuda")
        rm = SimpleNamespace(req_to_token_indexs=t["table"], req_to_imp_token_indexs=imp)
        return SimpleNamespace(batch_size=len(reqs), max_len_in_batch=max(lens),
                               b_seq_len=torch.tensor(lens, dtype=torch.int32, device="cuda"),
                               b_req_idx=torch.tensor(reqs, dtype=torch.int32, device="cuda"), req_manager=rm,
                               is_prefill=False, imp_seq_len=None, max_imp_len_batch=0)

    pool, pool2 = t["pool"], t["pool2"]
    st = state([req], [L])
    o = attn(t["q_sel"].reshape(1, H * d), st, H, d, pool[:, :KVH], pool[:, KVH:], do_select=True, tp_rank=0)
    assert np.abs(o.float().cpu().numpy().reshape(1, H, d) - gold["sel_out"]).max() <= 1e-4
    n_imp = int(st.imp_seq_len[0].item())
    assert n_imp == k == st.max_imp_len_batch
    rows = st.req_manager.req_to_imp_token_indexs[0, req, :n_imp].cpu()
    inv = {int(r): p for p, r in enumerate(x["table"][req, :L].tolist())}
    got = torch.tensor(sorted(inv[int(r)] for r in rows.tolist()))
    # the fixture's scores are raw logits (magnitude up to 40): 1e-3 there is the 1e-4 band of the scaled scores
    band_check(torch.from_numpy(gold["score_max"]), k, got.tolist(), gold["sel_pos_sorted"].tolist(), 1e-3,
               "rows recorded by the selecting call")
    o2 = attn(t["q_sparse"].reshape(1, H * d), st, H, d, pool2[:, :KVH], pool2[:, KVH:], tp_rank=0)
    if torch.equal(got, torch.from_numpy(gold["sel_pos_sorted"]).long()):  # same rows: same attention
        assert np.abs(o2.float().cpu().numpy().reshape(1, H, d) - gold["sparse_out"]).max() <= 1e-4
    st3 = state(c["dense"]["reqs"], c["dense"]["lens"])
    o3 = attn(t["q_dense"].reshape(-1, H * d), st3, H, d, pool[:, :KVH], pool[:, KVH:])
    assert np.abs(o3.float().cpu().numpy().reshape(-1, H, d) - gold["dense_out"]).max() <= 1e-4
