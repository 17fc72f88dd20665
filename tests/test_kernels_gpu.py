"""Parity of the CUDA kernels (called through the C ABI) against the CPU oracle.

Tolerances (from the task's acceptance rules): top-k indices bit-exact on an identical fp32
score tensor; selected sets equal wherever the k-th score gap exceeds 1e-4; attention outputs
within 2e-2 absolute for bf16/fp16 and 1e-4 for fp32.
"""
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import inputs as gi
import oracle

pytestmark = pytest.mark.gpu

G = Path(__file__).resolve().parent / "golden"
ATOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def ops():
    from omnikv_b200 import ops as _ops
    return _ops


def dev_i32(x):
    return torch.tensor(x, dtype=torch.int32, device="cuda")


def make_kv(B, KVH, L, d, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(B, KVH, L, d, generator=g).to(dtype)
    v = torch.randn(B, KVH, L, d, generator=g).to(dtype)
    return k, v


def make_q(B, H, d, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, H, d, generator=g) * scale).to(dtype)


# ------------------------------------------------------------------------------------------
# dense decode attention (+ fused score planes)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("B,H,KVH,lens,splits", [
    (1, 32, 8, [1], 1), (1, 32, 8, [63], 3), (1, 32, 8, [64], 1), (1, 32, 8, [65], 2), (1, 32, 8, [1000], 5),
    (3, 32, 8, [4097, 17, 2500], 7), (2, 16, 2, [777, 1], 4), (2, 8, 8, [300, 299], 3), (1, 32, 8, [20000], 37),
])
def test_dense_attention_and_scores(dtype, B, H, KVH, lens, splits):
    d, L = 128, max(lens) + 5
    k, v = make_kv(B, KVH, L, d, dtype, 1)
    q = make_q(B, H, d, dtype, 2, 1.5)
    len_a = dev_i32(lens)
    score_len = dev_i32([max(0, n - 2) for n in lens])  # e.g. the prompt is 2 tokens shorter
    planes = torch.full((KVH, B, L), float("nan"), dtype=torch.float32, device="cuda")
    out = ops().decode_attn(q.cuda(), k.cuda(), v.cuda(), len_a, score_out=planes, score_len=score_len,
                            n_splits=splits)
    out2 = ops().decode_attn(q.cuda(), k.cuda(), v.cuda(), len_a, n_splits=splits)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)  # the score output does not change the attention result
    for b, n in enumerate(lens):
        want = oracle.dense_attention(q[b:b + 1], k[b:b + 1, :, :n], v[b:b + 1, :, :n])
        err = (out[b:b + 1].float().cpu() - want).abs().max().item()
        assert err <= ATOL[dtype], (b, n, err)
        sl = max(0, n - 2)
        if sl:
            s_want = oracle.score_last(q[b:b + 1], k[b:b + 1], sl)[0]
            s_got = planes[:, b, :sl].max(dim=0).values.cpu()
            assert (s_got - s_want).abs().max().item() <= 2e-5 * max(1.0, s_want.abs().max().item())
        assert torch.isnan(planes[:, b, sl:]).all()  # nothing is written past score_len


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_score_only_mode_matches_fused(dtype):
    B, H, KVH, d, L = 2, 32, 8, 128, 3000
    k, v = make_kv(B, KVH, L, d, dtype, 3)
    q = make_q(B, H, d, dtype, 4)
    lens = dev_i32([3000, 1234])
    fused = torch.zeros(KVH, B, L, dtype=torch.float32, device="cuda")
    ops().decode_attn(q.cuda(), k.cuda(), v.cuda(), lens, score_out=fused, score_len=lens, n_splits=6)
    only = torch.zeros(KVH, B, L, dtype=torch.float32, device="cuda")
    ops().score_last(q.cuda(), k.cuda(), lens, score_out=only, n_splits=9)
    torch.cuda.synchronize()
    assert torch.equal(fused, only)


# ------------------------------------------------------------------------------------------
# sparse decode attention: selected rows + tail
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("B,P,ks,tails,splits", [
    (1, 5000, [335], [1], 4), (1, 5000, [1], [0], 1), (2, 3000, [200, 64], [7, 130], 3), (1, 70000, [4690], [128], 37),
    (3, 1000, [1000, 0, 999], [3, 5, 0], 5),
    # long lists with one split (direct output, no merge) and with two; ragged: a short and an empty list beside a long one
    (2, 6000, [3000, 2100], [5, 64], 1), (3, 6000, [3000, 70, 0], [5, 1, 0], 2), (1, 4000, [2112], [0], 1),
])
@pytest.mark.parametrize("layout", ["planes", "pairs"])
def test_sparse_attention(dtype, B, P, ks, tails, splits, layout):
    H, KVH, d = 32, 8, 128
    cap = P + 256
    k, v = make_kv(B, KVH, cap, d, dtype, 5)
    if layout == "pairs":  # the token-major layout of a sparse layer: the V row of a position right behind its K row
        kv = torch.stack([k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3)], dim=3).contiguous()  # [B, rows, KVH, K|V, d]
        k, v = kv[:, :, :, 0].permute(0, 2, 1, 3), kv[:, :, :, 1].permute(0, 2, 1, 3)
    q = make_q(B, H, d, dtype, 6, 1.5)
    g = torch.Generator().manual_seed(7)
    kmax = max(max(ks), 1)
    idx = torch.zeros(B, kmax, dtype=torch.int64)
    for b in range(B):
        idx[b, :ks[b]] = torch.sort(torch.randperm(P, generator=g)[:ks[b]]).values
    if layout == "pairs":
        kvc = kv.cuda()
        kc, vc = kvc[:, :, :, 0].permute(0, 2, 1, 3), kvc[:, :, :, 1].permute(0, 2, 1, 3)
    else:
        kc, vc = k.cuda(), v.cuda()
    out = ops().decode_attn(q.cuda(), kc, vc, dev_i32(ks), idx=idx.to(torch.int32).cuda(),
                            k_tail=kc, v_tail=vc, tail_start=dev_i32([P] * B), tail_len=dev_i32(tails),
                            n_splits=splits)
    torch.cuda.synchronize()
    for b in range(B):
        if ks[b] + tails[b] == 0:
            assert out[b].float().abs().max().item() == 0.0
            continue
        want = oracle.sparse_attention(q[b:b + 1], k[b:b + 1, :, :P], v[b:b + 1, :, :P], idx[b:b + 1, :ks[b]],
                                       k[b:b + 1, :, P:P + tails[b]], v[b:b + 1, :, P:P + tails[b]])
        err = (out[b:b + 1].float().cpu() - want).abs().max().item()
        assert err <= ATOL[dtype], (b, err)


# ------------------------------------------------------------------------------------------
# top-k
# ------------------------------------------------------------------------------------------
def _check_topk(scores, lens, ks, idx, count, append=None):
    """Bit-exact against the oracle's rule (stable: lowest position wins among equal scores)."""
    idx, count = idx.cpu(), count.cpu()
    for b in range(scores.shape[0]):
        n = lens[b]
        kk = min(ks[b], n)
        app = append[b] if append else 0
        assert count[b].item() == kk + app
        want = oracle.topk_ascending(scores[b:b + 1, :n], kk)[0] if kk else torch.zeros(0, dtype=torch.int64)
        got = idx[b, :kk].long()
        assert torch.equal(got, want), (b, n, kk)
        if app:
            assert torch.equal(idx[b, kk:kk + app].long(), torch.arange(n, n + app))


@pytest.mark.parametrize("L", [1, 2, 17, 255, 4096, 8193, 40000, 131072])
def test_topk_random(L):
    g = torch.Generator().manual_seed(L)
    B = 3
    s = torch.randn(B, L, generator=g)
    lens = [L, max(1, L // 2), max(1, L - 1)]
    for ks in ([1, 1, 1], [L, L, L], [L + 5, 3, max(1, L - 1)], [max(1, int(0.067 * L))] * 3, [0, 1, 2]):
        idx, cnt = ops().topk(s.cuda(), dev_i32(lens), dev_i32(ks))
        torch.cuda.synchronize()
        _check_topk(s, lens, ks, idx, cnt)


def test_topk_ties_planes_append_and_specials():
    g = torch.Generator().manual_seed(11)
    B, L, P = 4, 20000, 8
    planes = (torch.randn(P, B, L, generator=g) * 3).round() / 4  # heavy ties
    planes[0, 1, 5] = float("inf")
    planes[3, 1, 7] = float("-inf")
    planes[:, 2, :] = 1.25  # all equal: the first k positions win
    s = planes.max(dim=0).values
    lens, ks, app = [L, L - 3, 777, 19999], [1340, 5, 100, 19999], [0, 15, 3, 1]
    idx = torch.full((B, L + 32), -1, dtype=torch.int32, device="cuda")
    idx, cnt = ops().topk(planes.cuda(), dev_i32(lens), dev_i32(ks), append_n=dev_i32(app), idx_out=idx, max_len=L)
    torch.cuda.synchronize()
    _check_topk(s, lens, ks, idx, cnt, app)
    assert torch.equal(idx[2, :100].cpu().long(), torch.arange(100))


@pytest.mark.parametrize("L", [1000, 1025, 2500, 5000, 9000, 16384, 16385, 60000])
def test_topk_single_sequence_cluster_sizes(L):
    """One sequence gets slices of 1024 keys: clusters of 1, 2, 4, 8 and 16 CTAs, with heavy ties across the slices."""
    g = torch.Generator().manual_seed(100 + L)
    planes = (torch.randn(2, 1, L, generator=g) * 2).round() / 2
    s = planes.max(dim=0).values
    for n, k, app in ([L, max(1, int(0.067 * L)), 0], [L - 1, L - 1, 2], [L, 1, 0], [max(1, L - 517), 700, 5]):
        idx = torch.full((1, L + 16), -1, dtype=torch.int32, device="cuda")
        idx, cnt = ops().topk(planes.cuda(), dev_i32([n]), dev_i32([k]), append_n=dev_i32([app]), idx_out=idx, max_len=L)
        torch.cuda.synchronize()
        _check_topk(s, [n], [k], idx, cnt, [app])


def test_topk_nan_ranks_first():
    s = torch.randn(1, 1000)
    s[0, 123] = float("nan")
    idx, cnt = ops().topk(s.cuda(), dev_i32([1000]), dev_i32([1]))
    assert idx[0, 0].item() == 123


def test_topk_long_context_not_resident():
    # 450 000 keys: the slice of a CTA no longer fits shared memory, keys go through the workspace
    L = 450000
    g = torch.Generator().manual_seed(5)
    s = torch.randn(1, L, generator=g)
    k = int(0.067 * L)
    idx, cnt = ops().topk(s.cuda(), dev_i32([L]), dev_i32([k]))
    torch.cuda.synchronize()
    _check_topk(s, [L], [k], idx, cnt)


def test_topk_batch16_ragged():
    g = torch.Generator().manual_seed(6)
    B = 16
    lens = torch.randint(16384, 32769, (B,), generator=g).tolist()
    s = torch.randn(B, 32768, generator=g)
    ks = [2048] * B
    idx, cnt = ops().topk(s.cuda(), dev_i32(lens), dev_i32(ks))
    torch.cuda.synchronize()
    _check_topk(s, lens, ks, idx, cnt)


# ------------------------------------------------------------------------------------------
# window selectors
# ------------------------------------------------------------------------------------------
def _band_check(s_ref, got_idx, k, band):
    """Sets equal, or differing only on positions whose reference score lies within `band` of the k-th."""
    want = oracle.topk_ascending(s_ref[None], k)[0]
    diff = set(got_idx.tolist()) ^ set(want.tolist())
    kth = torch.sort(s_ref, descending=True).values[k - 1].item()
    assert all(abs(s_ref[i].item() - kth) <= band for i in diff), len(diff)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("selector", ["uniform", "exp", "softmax_before_last"])
@pytest.mark.parametrize("B,H,KVH,W,lens", [(1, 32, 8, 16, [3000]), (2, 32, 8, 5, [777, 64]), (1, 8, 2, 1, [130]),
                                             (2, 16, 2, 16, [1, 4100])])
def test_score_window(dtype, selector, B, H, KVH, W, lens):
    d, L = 128, max(lens) + 3
    g = torch.Generator().manual_seed(13)
    k = torch.randn(B, KVH, L, d, generator=g).to(dtype)
    qw = (torch.randn(B, H, W, d, generator=g) * 1.2).to(dtype)
    got = ops().score_window(qw.cuda(), k.cuda(), dev_i32(lens), selector, max_len=max(lens))
    planes = torch.zeros(B, W, max(lens), dtype=torch.float32, device="cuda")
    ops().score_window(qw.cuda(), k.cuda(), dev_i32(lens), selector, max_len=max(lens), planes_out=planes)
    folded = ops().window_fold(planes, dev_i32(lens), selector, max_len=max(lens))
    torch.cuda.synchronize()
    for b, n in enumerate(lens):
        want = oracle.score_window(qw[b:b + 1], k[b:b + 1], n, selector)[0]
        tol = 1e-5 * max(1.0, want.max().item()) + 1e-6
        assert (got[b, :n].cpu() - want).abs().max().item() <= tol
        assert (folded[b, :n].cpu() - want).abs().max().item() <= tol


# ------------------------------------------------------------------------------------------
# the single-layer operator case against the fixture produced by the reference itself
# ------------------------------------------------------------------------------------------
def test_operator_case_against_reference_fixture():
    o = json.loads((G / "operator_cfg1.json").read_text())
    gold = np.load(G / "operator_cfg1.npz")
    x = gi.operator_inputs()
    assert gi.checksum([x[n] for n in ("q", "k", "k2", "v2", "k_new", "v_new")]) == pytest.approx(o["input_checksum"], rel=1e-12)
    L, k = o["L"], o["k"]
    q = torch.from_numpy(x["q"]).cuda()
    kf = torch.from_numpy(x["k"]).cuda()
    q_last = q[:, :, -1, :].contiguous()
    n = dev_i32([L])
    planes = ops().score_last(q_last, kf, n)
    idx, cnt = ops().topk(planes, n, dev_i32([k]))
    torch.cuda.synchronize()
    assert cnt.item() == k
    s_ref = oracle.score_last(torch.from_numpy(x["q"])[:, :, -1], torch.from_numpy(x["k"]), L)[0]
    got = idx[0, :k].cpu().long()
    if not np.array_equal(got.numpy(), gold["idx"][0].astype(np.int64)):
        _band_check(s_ref, got, k, 1e-4)
    # second layer: prompt rows of (k2, v2) at the REFERENCE's indices + the current token's row
    cap = L + 8
    k2 = torch.zeros(1, 8, cap, 128)
    v2 = torch.zeros(1, 8, cap, 128)
    k2[:, :, :L], v2[:, :, :L] = torch.from_numpy(x["k2"]), torch.from_numpy(x["v2"])
    k2, v2 = k2.cuda(), v2.cuda()
    ops().kv_append(torch.from_numpy(x["k_new"])[:, :, 0].cuda(), torch.from_numpy(x["v_new"])[:, :, 0].cuda(), k2, v2, n)
    ref_idx = torch.from_numpy(gold["idx"].astype(np.int32)).cuda()
    out = ops().decode_attn(q_last, k2, v2, dev_i32([k]), idx=ref_idx, k_tail=k2, v_tail=v2, tail_start=n,
                            tail_len=dev_i32([1]))
    torch.cuda.synchronize()
    assert np.abs(out.cpu().numpy() - gold["out"]).max() <= 1e-4
    # window selectors on the same inputs
    for sel in ("uniform", "exp"):
        s = ops().score_window(q.contiguous(), kf, n, sel, max_len=L)
        idx_w, _ = ops().topk(s, n, dev_i32([k]))
        torch.cuda.synchronize()
        s_ref = oracle.score_window(torch.from_numpy(x["q"]), torch.from_numpy(x["k"]), L, sel)[0]
        got = idx_w[0, :k].cpu().long()
        if not np.array_equal(got.numpy(), gold[f"idx_{sel}"][0].astype(np.int64)):
            _band_check(s_ref, got, k, 1e-6)


# ------------------------------------------------------------------------------------------
# full-size (128K, bf16) run: oracle comparison + size-independent properties
# ------------------------------------------------------------------------------------------
def test_full_size_128k_bf16():
    B, H, KVH, d, L, k = 1, 32, 8, 128, 131072, 8781
    g = torch.Generator().manual_seed(21)
    kc = torch.randn(B, KVH, L + 128, d, generator=g).to(torch.bfloat16)
    vc = torch.randn(B, KVH, L + 128, d, generator=g).to(torch.bfloat16)
    q = (torch.randn(B, H, d, generator=g) * 1.5).to(torch.bfloat16)
    kg, vg, qg = kc.cuda(), vc.cuda(), q.cuda()
    n_prompt, n_all = dev_i32([L]), dev_i32([L + 1])
    planes = torch.empty(KVH, B, L, dtype=torch.float32, device="cuda")
    out = ops().decode_attn(qg, kg, vg, n_all, score_out=planes, score_len=n_prompt)
    idx, cnt = ops().topk(planes, n_prompt, dev_i32([k]))
    out_sparse = ops().decode_attn(qg, kg, vg, cnt, idx=idx, k_tail=kg, v_tail=vg, tail_start=n_prompt,
                                   tail_len=dev_i32([1]))
    torch.cuda.synchronize()
    assert cnt.item() == k
    sel = idx[0, :k].cpu().long()
    assert torch.all(sel[1:] > sel[:-1]) and sel[0] >= 0 and sel[-1] < L  # ascending, in range, unique
    # oracle
    want = oracle.dense_attention(q, kc[:, :, :L + 1], vc[:, :, :L + 1])
    assert (out.float().cpu() - want).abs().max().item() <= 2e-2
    s_ref = oracle.score_last(q, kc, L)[0]
    assert (planes.max(dim=0).values[0].cpu() - s_ref).abs().max().item() <= 1e-4
    _band_check(s_ref, sel, k, 1e-4)
    want_sparse = oracle.sparse_attention(q, kc[:, :, :L], vc[:, :, :L], sel[None], kc[:, :, L:L + 1], vc[:, :, L:L + 1])
    assert (out_sparse.float().cpu() - want_sparse).abs().max().item() <= 2e-2
    # property: selecting every row (k = L) reproduces the dense result
    idx_all, cnt_all = ops().topk(planes, n_prompt, dev_i32([L]))
    out_all = ops().decode_attn(qg, kg, vg, cnt_all, idx=idx_all, k_tail=kg, v_tail=vg, tail_start=n_prompt,
                                tail_len=dev_i32([1]))
    torch.cuda.synchronize()
    assert torch.equal(idx_all[0].cpu().long(), torch.arange(L))
    assert (out_all.float() - out.float()).abs().max().item() <= 4e-3
    # property: the result does not depend on the split count beyond rounding
    out_s3 = ops().decode_attn(qg, kg, vg, n_all, n_splits=3)
    assert (out_s3.float() - out.float()).abs().max().item() <= 4e-3


# ------------------------------------------------------------------------------------------
# KV append and the host-link gather
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_kv_append(dtype):
    B, KVH, d, cap = 3, 8, 128, 50
    kc = torch.zeros(B, KVH, cap, d, dtype=dtype, device="cuda")
    vc = torch.zeros_like(kc)
    kn = torch.randn(B, KVH, d, device="cuda").to(dtype)
    vn = torch.randn(B, KVH, d, device="cuda").to(dtype)
    pos = [0, 49, 17]
    ops().kv_append(kn, vn, kc, vc, dev_i32(pos))
    torch.cuda.synchronize()
    for b, p in enumerate(pos):
        assert torch.equal(kc[b, :, p], kn[b]) and torch.equal(vc[b, :, p], vn[b])
    assert kc.float().abs().sum().item() == pytest.approx(kn.float().abs().sum().item(), rel=1e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_offload_gather(dtype):
    tokens, layers, KVH, d, cap, n = 5000, 3, 8, 128, 400, 335
    g = torch.Generator().manual_seed(3)
    host = torch.randn(tokens, layers, 2, KVH, d, generator=g).to(dtype).pin_memory()
    idx = torch.sort(torch.randperm(tokens, generator=g)[:n]).values
    staged = torch.zeros(layers, 2, KVH, cap, d, dtype=dtype, device="cuda")
    idx_dev = torch.zeros(cap, dtype=torch.int32, device="cuda")
    idx_dev[:n] = idx.to(torch.int32).cuda()
    ops().offload_gather(host, idx_dev, dev_i32([n]), staged)
    torch.cuda.synchronize()
    want = host[idx].permute(1, 2, 3, 0, 4)  # [layers, 2, KVH, n, d]
    assert torch.equal(staged[:, :, :, :n].cpu(), want)
    assert staged[:, :, :, n:].float().abs().sum().item() == 0.0


# ------------------------------------------------------------------------------------------
# fused batch-1 decode kernels (weight streaming with TMA bulk copies) at Llama-3-8B shapes
# ------------------------------------------------------------------------------------------
def _close(got, ref, rel=1e-2, absol=1e-2):
    err = (got.float().cpu() - ref.float().cpu()).abs()
    lim = rel * ref.float().cpu().abs() + absol
    assert bool((err <= lim).all()), (err.max().item(), (err - lim).max().item())


def _rms(x, w, eps):
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean() + eps) * w.float()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hidden,H,KVH", [(4096, 32, 8), (512, 4, 1), (8192, 8, 1)])
def test_fused_qkv_rope_append(dtype, hidden, H, KVH):
    g = torch.Generator(device="cuda").manual_seed(1)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")  # noqa: E731
    h = rn(hidden).to(dtype)
    nw = (1 + 0.1 * rn(hidden)).to(dtype)
    w = (rn((H + 2 * KVH) * 128, hidden) / hidden ** 0.5).to(dtype)
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))).cuda()
    pos = 70001
    cap = 16
    kc = torch.zeros(KVH, cap, 128, dtype=dtype, device="cuda")
    vc = torch.zeros(KVH, cap, 128, dtype=dtype, device="cuda")
    q = torch.zeros(H * 128, dtype=dtype, device="cuda")
    ops().decode_qkv(h, nw, 1e-5, w, H, KVH, inv_freq, dev_i32([pos]), q, kc, vc, dev_i32([5]))
    ops().check_status("cuda")
    x = _rms(h, nw, 1e-5)
    y = (w.float() @ x).view(H + 2 * KVH, 128)
    ang = pos * inv_freq
    cos, sin = torch.cat([ang.cos(), ang.cos()]), torch.cat([ang.sin(), ang.sin()])
    rot = lambda t: t * cos + torch.cat([-t[:, 64:], t[:, :64]], dim=1) * sin  # noqa: E731
    _close(q.view(H, 128), rot(y[:H]))
    _close(kc[:, 5], rot(y[H:H + KVH]))
    _close(vc[:, 5], y[H + KVH:])
    assert kc[:, :5].abs().sum().item() == 0 and kc[:, 6:].abs().sum().item() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("N,K", [(4096, 4096), (4096, 14336), (512, 1024), (4096, 7168), (4096, 3584), (4096, 1792),
                                 (8192, 8192), (4096, 2048), (4096, 512)])
def test_fused_gemv_residual(dtype, N, K):
    g = torch.Generator(device="cuda").manual_seed(2)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")  # noqa: E731
    w = (rn(N, K) / K ** 0.5).to(dtype)
    x, r = rn(K).to(dtype), rn(N).to(dtype)
    out = torch.empty(N, dtype=dtype, device="cuda")
    ops().decode_gemv_residual(w, x, r, out)
    ref = w.float() @ x.float()
    _close(out, ref + r.float())
    ops().decode_gemv_residual(w, x, None, out)
    _close(out, ref)
    h = r.clone()
    ops().decode_gemv_residual(w, x, h, h)  # in place
    ops().check_status("cuda")
    _close(h, ref + r.float())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hidden,inter", [(4096, 14336), (512, 1024), (4096, 1792), (8192, 3584)])
def test_fused_gate_up(dtype, hidden, inter):
    g = torch.Generator(device="cuda").manual_seed(3)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")  # noqa: E731
    h, nw = rn(hidden).to(dtype), (1 + 0.1 * rn(hidden)).to(dtype)
    w = (rn(2 * inter, hidden) / hidden ** 0.5).to(dtype)
    act = torch.empty(inter, dtype=dtype, device="cuda")
    ops().decode_gate_up(h, nw, 1e-5, w, act)
    ops().check_status("cuda")
    y = w.float() @ _rms(h, nw, 1e-5)
    _close(act, torch.nn.functional.silu(y[:inter]) * y[inter:])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hidden,vocab,off", [(4096, 128256, 0), (512, 1000, 0), (4096, 16032, 32064)])
def test_fused_logits_argmax(dtype, hidden, vocab, off):
    g = torch.Generator(device="cuda").manual_seed(4)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")  # noqa: E731
    h, nw = rn(hidden).to(dtype), (1 + 0.1 * rn(hidden)).to(dtype)
    w = (rn(vocab, hidden) / hidden ** 0.5).to(dtype)
    logits = torch.empty(vocab, dtype=torch.float32, device="cuda")
    best = torch.zeros(1, dtype=torch.int64, device="cuda")
    tok = torch.zeros(1, dtype=torch.int64, device="cuda")
    for _ in range(2):  # the scratch word is re-initialised by every call
        ops().decode_logits(h, nw, 1e-5, w, off, logits, best, tok)
    ops().check_status("cuda")
    ref = w.float() @ _rms(h, nw, 1e-5)
    assert (logits - ref).abs().max().item() <= 2e-3
    assert tok.item() == off + int(logits.argmax().item())
    # ties: the lowest index wins
    w[7] = w[3]
    ops().decode_logits(h, nw, 1e-5, w, off, logits, best, tok)
    big = logits.max().item()
    h2 = h.clone()
    w[3] = w[7] = (w[int(logits.argmax().item())].float() * 1.5).to(dtype)
    ops().decode_logits(h2, nw, 1e-5, w, off, logits, best, tok)
    if logits[3].item() == logits.max().item():
        assert tok.item() == off + 3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hidden,inter,H,KVH,vocab", [(4096, 14336, 32, 8, 128256), (512, 1024, 4, 1, 1000)])
def test_decode_chain_equals_single_calls(dtype, hidden, inter, H, KVH, vocab):
    """The cooperative multi-phase launch computes exactly what the four single-phase calls compute
    (same per-row arithmetic), with the activations crossing its grid-wide barriers."""
    assert ops().decode_chain_supported(dtype, hidden, inter, H)
    g = torch.Generator(device="cuda").manual_seed(9)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")  # noqa: E731
    h0, attn = rn(hidden).to(dtype), rn(hidden).to(dtype)
    nw1, nw2 = (1 + 0.1 * rn(hidden)).to(dtype), (1 + 0.1 * rn(hidden)).to(dtype)
    w_o = (rn(hidden, hidden) / hidden ** 0.5).to(dtype)
    w_gu = (rn(2 * inter, hidden) / hidden ** 0.5).to(dtype)
    w_d = (rn(hidden, inter) / inter ** 0.5).to(dtype)
    w_qkv = (rn((H + 2 * KVH) * 128, hidden) / hidden ** 0.5).to(dtype)
    w_head = (rn(vocab, hidden) / hidden ** 0.5).to(dtype)
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))).cuda()
    rope_pos, cpos = dev_i32([131080]), dev_i32([3])

    def fresh():
        return dict(h=h0.clone(), act=torch.zeros(inter, dtype=dtype, device="cuda"),
                    q=torch.zeros(H * 128, dtype=dtype, device="cuda"), kc=torch.zeros(KVH, 8, 128, dtype=dtype, device="cuda"),
                    vc=torch.zeros(KVH, 8, 128, dtype=dtype, device="cuda"),
                    logits=torch.zeros(vocab, dtype=torch.float32, device="cuda"),
                    best=torch.zeros(1, dtype=torch.int64, device="cuda"), tok=torch.zeros(1, dtype=torch.int64, device="cuda"))

    for tail in ("qkv", "logits"):
        a, b = fresh(), fresh()
        # single calls
        ops().decode_gemv_residual(w_o, attn, a["h"], a["h"])
        ops().decode_gate_up(a["h"], nw1, 1e-5, w_gu, a["act"])
        ops().decode_gemv_residual(w_d, a["act"], a["h"], a["h"])
        if tail == "qkv":
            ops().decode_qkv(a["h"], nw2, 1e-5, w_qkv, H, KVH, inv_freq, rope_pos, a["q"], a["kc"], a["vc"], cpos)
        else:
            ops().decode_logits(a["h"], nw2, 1e-5, w_head, 0, a["logits"], a["best"], a["tok"])
        # one chained launch, three times (the grid barrier word must be reusable); static chunk assignment
        # first, then dynamic scheduling from zeroed counters
        for rep in range(3):
            b = fresh()
            kw = dict(eps=1e-5, H=H, KVH=KVH, inter=inter, w_o=w_o, attn_out=attn, post_norm_w=nw1, w_gate_up=w_gu,
                      w_down=w_d, act=b["act"],
                      chunk_counters=None if rep == 0 else torch.zeros(4, dtype=torch.int32, device="cuda"))
            if tail == "qkv":
                kw.update(in_norm_w=nw2, w_qkv=w_qkv, inv_freq=inv_freq, rope_pos=rope_pos, q_out=b["q"],
                          k_cache_seq=b["kc"], v_cache_seq=b["vc"], cache_pos=cpos)
            else:
                kw.update(final_norm_w=nw2, w_head=w_head, logits=b["logits"], best=b["best"], token_out=b["tok"])
            ops().decode_chain(b["h"], **kw)
            ops().check_status("cuda")
            for name in a:
                assert torch.equal(a[name], b[name]), (tail, rep, name)
    # a lone QKV phase (the first launch of a step)
    a, b = fresh(), fresh()
    ops().decode_qkv(a["h"], nw2, 1e-5, w_qkv, H, KVH, inv_freq, rope_pos, a["q"], a["kc"], a["vc"], cpos)
    ops().decode_chain(b["h"], eps=1e-5, H=H, KVH=KVH, inter=inter, in_norm_w=nw2, w_qkv=w_qkv, inv_freq=inv_freq,
                       rope_pos=rope_pos, q_out=b["q"], k_cache_seq=b["kc"], v_cache_seq=b["vc"], cache_pos=cpos)
    ops().check_status("cuda")
    assert torch.equal(a["q"], b["q"]) and torch.equal(a["kc"], b["kc"]) and torch.equal(a["vc"], b["vc"])


@pytest.mark.parametrize("thr", ["0.4", "0.7", "0.95"])
def test_idx_commit_follows_reference_rule(thr):
    """omnikv_idx_commit on the fixture's drifting index sequence: the same kept/replaced decisions as the
    reference's OmniKVLazyCache.set_out_idx, overlap counts equal to the oracle's score times |new|."""
    meta = json.loads((Path(__file__).resolve().parent / "golden" / "lazy_rule.json").read_text())
    gold = meta["results"][thr]
    seq = gi.lazy_rule_inputs()
    k = seq[0].shape[1]
    cap = k + 20
    live = torch.zeros(1, cap, dtype=torch.int32, device="cuda")
    live_n, applied, gather_n, overlap = (torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(4))
    rule = oracle.OracleLazyRule(float(thr))
    for s, idx in enumerate(seq):
        new = torch.zeros(1, cap, dtype=torch.int32, device="cuda")
        new[0, :k] = torch.from_numpy(idx[0]).to(torch.int32)
        n = dev_i32([k])
        ops().idx_commit(new, n, live, live_n, float(thr), applied, gather_n, overlap)
        taken, score = rule.offer(torch.from_numpy(idx), 1)
        assert bool(applied.item()) == gold["applied"][s] == taken
        assert gather_n.item() == (k if taken else 0)
        if s > 0:
            assert overlap.item() == round(score * k)
        assert live_n.item() == k
        assert torch.equal(live[0, :k].cpu().long(), rule.live[1][0])


def test_idx_commit_batch_and_edges():
    """Per-sequence decisions in a batch, ragged counts, an empty list in use, identical lists (overlap 1 > any
    threshold below 1: kept), and argument checks."""
    cap = 64
    new = torch.zeros(3, cap, dtype=torch.int32, device="cuda")
    live = torch.zeros(3, cap, dtype=torch.int32, device="cuda")
    new[0, :5] = torch.tensor([1, 3, 5, 7, 9]); live[0, :5] = torch.tensor([1, 3, 5, 7, 9])       # identical
    new[1, :4] = torch.tensor([2, 4, 6, 8]); live[1, :6] = torch.tensor([0, 1, 2, 3, 5, 7])        # 1 of 4 shared
    new[2, :3] = torch.tensor([10, 20, 30])                                                         # nothing in use
    n = dev_i32([5, 4, 3]); m = dev_i32([5, 6, 0])
    applied, gather_n, overlap = (torch.full((3,), -1, dtype=torch.int32, device="cuda") for _ in range(3))
    ops().idx_commit(new, n, live, m, 0.5, applied, gather_n, overlap)
    assert applied.tolist() == [0, 1, 1] and gather_n.tolist() == [0, 4, 3] and overlap.tolist() == [5, 1, 0]
    assert m.tolist() == [5, 4, 3]
    assert live[1, :4].tolist() == [2, 4, 6, 8] and live[2, :3].tolist() == [10, 20, 30]
    assert live[0, :5].tolist() == [1, 3, 5, 7, 9]
    # exactly at the threshold is NOT above it: replaced (2 of 4 shared, threshold 0.5)
    new[1, :4] = torch.tensor([2, 4, 60, 80])
    ops().idx_commit(new, n, live, m, 0.5, applied, gather_n, overlap)
    assert applied.tolist()[1] == 1 and overlap.tolist()[1] == 2
    with pytest.raises(Exception):
        ops().idx_commit(new, n, new, m, 0.5, applied)
    with pytest.raises(Exception):
        ops().idx_commit(new.long(), n, live, m, 0.5, applied)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float16, 4e-3), (torch.float32, 2e-6)])
@pytest.mark.parametrize("B,H,KVH", [(1, 32, 8), (5, 8, 2), (16, 4, 1)])
def test_rope_append(dtype, tol, B, H, KVH):
    """omnikv_rope_append against the rotate_half formula: rotated q, rotated k and plain v land in
    q_out and in row cache_pos[b] of a strided cache; other rows stay untouched; a negative position skips."""
    g = torch.Generator(device="cuda").manual_seed(21)
    d, cap = 128, 12
    qkv = torch.randn(B, (H + 2 * KVH) * d, generator=g, device="cuda").to(dtype)
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).cuda()
    rope_pos = torch.randint(0, 200000, (B,), generator=g, device="cuda", dtype=torch.int32)
    cache_pos = torch.randint(0, cap, (B,), generator=g, device="cuda", dtype=torch.int32)
    if B > 1:
        cache_pos[1] = -1
    kv = torch.full((B, KVH, cap, 2, d), 7.0, device="cuda").to(dtype)   # K|V rows interleaved, as the caches
    kc, vc = kv[:, :, :, 0, :], kv[:, :, :, 1, :]
    q = torch.zeros(B, H, d, device="cuda", dtype=dtype)
    ops().rope_append(qkv, H, KVH, inv_freq, rope_pos, q, kc, vc, cache_pos)
    x = qkv.double().view(B, H + 2 * KVH, d)
    # the angle is an fp32 product, as in the reference's rotary embedding; cos/sin of it in fp64
    ang = (rope_pos.float()[:, None] * inv_freq[None, :]).double()
    cos, sin = torch.cat([ang.cos(), ang.cos()], 1)[:, None, :], torch.cat([ang.sin(), ang.sin()], 1)[:, None, :]
    rot = x * cos + torch.cat([-x[..., 64:], x[..., :64]], -1) * sin
    assert (q.double() - rot[:, :H]).abs().max().item() < tol * 4
    for b in range(B):
        p = int(cache_pos[b])
        if p < 0:
            assert (kv[b].float() == 7.0).all()
            continue
        assert (kc[b, :, p].double() - rot[b, H:H + KVH]).abs().max().item() < tol * 4
        assert torch.equal(vc[b, :, p], qkv[b].view(H + 2 * KVH, d)[H + KVH:])
        mask = torch.ones(cap, dtype=torch.bool, device="cuda")
        mask[p] = False
        assert (kv[b][:, mask].float() == 7.0).all()
    with pytest.raises(Exception):
        ops().rope_append(qkv[:, :-128], H, KVH, inv_freq, rope_pos, q, kc, vc, cache_pos)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-6)])
def test_silu_mul(dtype, tol):
    g = torch.Generator(device="cuda").manual_seed(22)
    gu = (3 * torch.randn(7, 2 * 1000, generator=g, device="cuda")).to(dtype)
    act = ops().silu_mul(gu)
    ref = torch.nn.functional.silu(gu[:, :1000].double()) * gu[:, 1000:].double()
    assert act.shape == (7, 1000) and act.dtype == dtype
    assert ((act.double() - ref).abs() / (1 + ref.abs())).max().item() < tol
    with pytest.raises(Exception):
        ops().silu_mul(gu[:, :-1])


def test_ragged_batch_splits_cover_every_row():
    """Chunks are sized by the longest sequence of the batch: short sequences use fewer splits.  Any split
    count gives the oracle's attention for every sequence (lengths from 1 row to several chunks)."""
    g = torch.Generator(device="cuda").manual_seed(23)
    B, H, KVH, d, cap = 6, 8, 2, 128, 3000
    lens = [1, 63, 64, 65, 1500, 2999]
    q = torch.randn(B, H, d, generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn(B, KVH, cap, d, generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn(B, KVH, cap, d, generator=g, device="cuda").to(torch.bfloat16)
    n = dev_i32(lens)
    for s in (1, 2, 5, 11, 24):
        o = ops().decode_attn(q, k, v, n, n_splits=s)
        for b in range(B):
            ref = oracle.dense_attention(q[b:b + 1].cpu(), k[b:b + 1, :, :lens[b]].cpu(), v[b:b + 1, :, :lens[b]].cpu())
            assert (o[b:b + 1].float().cpu() - ref).abs().max().item() < 2e-2, (s, b)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,L,cap", [(1, 5000, 5000), (1, 4097, 6000), (3, 700, 1024), (2, 64, 64)])
def test_dense_attn_tensor_map_tiles_equal_cp_async(dtype, B, L, cap):
    """The two ways a dense layer's tiles reach shared memory -- TMA tensor-map boxes with a 128-byte swizzle when the
    cache's capacity is stated, 16-byte cp.async copies into padded rows otherwise -- feed the same arithmetic:
    outputs and score planes are bit-identical, also with garbage (NaN) in the cache rows past the sequence."""
    g = torch.Generator(device="cuda").manual_seed(31)
    H, KVH, d = 8, 2, 128
    kv = torch.randn(B, KVH, cap, 2, d, generator=g, device="cuda").to(dtype)
    lens = [L - 3 * b for b in range(B)]
    for b in range(B):
        kv[b, :, lens[b]:] = float("nan")   # rows the kernel may fetch but must not use
    kc, vc = kv[:, :, :, 0, :], kv[:, :, :, 1, :]
    q = torch.randn(B, H, d, generator=g, device="cuda").to(dtype)
    n = dev_i32(lens)
    outs = []
    for cap_known in (True, False):
        planes = torch.zeros(KVH, B, cap, dtype=torch.float32, device="cuda")
        o = ops().decode_attn(q, kc, vc, n, score_out=planes, score_len=n, state_capacity=cap_known, n_splits=3)
        outs.append((o, planes))
    ops().check_status("cuda")
    assert torch.isfinite(outs[0][0].float()).all()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    ref = oracle.dense_attention(q[:1].cpu(), kc[:1, :, :lens[0]].cpu(), vc[:1, :, :lens[0]].cpu())
    assert (outs[0][0][:1].float().cpu() - ref).abs().max().item() < 2e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("L,splits,with_score", [(20000, 148, False), (20000, 64, True), (300, 64, False), (9000, 100, False)])
def test_dense_attention_with_many_splits_merged_together(dtype, L, splits, with_score):
    """A dense layer whose splits fit on the GPU at once (one or two KV heads per rank, as under tensor parallelism):
    the splits wait for one another and every CTA merges a slice of the output.  Same result as the merge by the last
    CTA (a few splits) up to the order of fp32 sums, right against the oracle, the same on a second call (the
    counters are left at zero), also when most splits are empty."""
    g = torch.Generator(device="cuda").manual_seed(41)
    B, H, KVH, d = 1, 8, 2, 128
    kv = torch.randn(B, KVH, L + 64, 2, d, generator=g, device="cuda").to(dtype)
    kc, vc = kv[:, :, :, 0, :], kv[:, :, :, 1, :]
    q = (torch.randn(B, H, d, generator=g, device="cuda") * 1.5).to(dtype)
    n = dev_i32([L])
    planes = torch.zeros(KVH, B, L + 64, dtype=torch.float32, device="cuda") if with_score else None
    kw = dict(score_out=planes, score_len=n) if with_score else {}
    many = ops().decode_attn(q, kc, vc, n, state_capacity=True, n_splits=splits, **kw)
    again = ops().decode_attn(q, kc, vc, n, state_capacity=True, n_splits=splits, **kw)
    few = ops().decode_attn(q, kc, vc, n, state_capacity=True, n_splits=4, **kw)
    ops().check_status("cuda")
    assert torch.equal(many, again)
    assert (many.float() - few.float()).abs().max().item() <= 4e-3
    ref = oracle.dense_attention(q.cpu(), kc[:, :, :L].cpu(), vc[:, :, :L].cpu())
    assert (many.float().cpu() - ref).abs().max().item() < 2e-2


def _causal_reference(q, k, v, q_pos0, scale):
    """fp32 definition: query i sees keys j <= q_pos0 + i.  q [B,H,Sq,d], k/v [B,KVH,Skv,d] -> [B,Sq,H,d]."""
    B, H, Sq, d = q.shape
    KVH, Skv = k.shape[1], k.shape[2]
    G = H // KVH
    qf, kf, vf = q.float(), k.float().repeat_interleave(G, dim=1), v.float().repeat_interleave(G, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    pos = q_pos0 + torch.arange(Sq, device=q.device)[:, None]
    s = s.masked_fill(torch.arange(Skv, device=q.device)[None, :] > pos, float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), vf).transpose(1, 2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,KVH,Sq,Skv,q_pos0", [
    (1, 8, 2, 128, 128, 0),      # one tile, diagonal mask only
    (1, 8, 2, 300, 300, 0),      # ragged last query block and key tile
    (2, 4, 1, 1000, 1000, 0),    # batch, eight key tiles, one KV head for four query heads
    (1, 4, 4, 200, 520, 320),    # a chunk of queries behind 320 cached keys
    (1, 32, 8, 2048, 2048, 0),   # Llama-3-8B head counts
    (1, 2, 1, 130, 130, 0),      # a second query tile of two rows
    (1, 2, 2, 600, 4000, 3400),  # a chunk deep inside a long cache: many key tiles before the diagonal
])
@pytest.mark.parametrize("variant", [0, 1])
def test_prefill_attention_matches_definition(dtype, B, H, KVH, Sq, Skv, q_pos0, variant):
    """tcgen05 prefill attention through the C ABI against the fp32 definition (2e-2 absolute for 16-bit inputs:
    P is rounded to 16 bits before the second product, as in flash attention)."""
    g = torch.Generator().manual_seed(Sq * 7 + H)
    q = torch.randn(B, H, Sq, 128, generator=g).to(dtype).cuda()
    k = torch.randn(B, KVH, Skv, 128, generator=g).to(dtype).cuda()
    v = torch.randn(B, KVH, Skv, 128, generator=g).to(dtype).cuda()
    scale = 1.0 / math.sqrt(128)
    out = ops().prefill_attn(q, k, v, q_pos0=q_pos0, variant=variant)
    ops().check_status(q.device)
    ref = _causal_reference(q, k, v, q_pos0, scale)
    assert out.shape == (B, Sq, H, 128)
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2, err


def test_prefill_attention_reads_strided_views():
    """k and v as views of one fused projection output (row stride of the whole projection), peaked logits."""
    B, H, KVH, S = 1, 8, 2, 700
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(B, S, (H + 2 * KVH) * 128, generator=g).to(torch.bfloat16).cuda()
    q = (qkv[..., :H * 128].view(B, S, H, 128).transpose(1, 2) * 3).contiguous()
    k = qkv[..., H * 128:(H + KVH) * 128].view(B, S, KVH, 128).transpose(1, 2)
    v = qkv[..., (H + KVH) * 128:].view(B, S, KVH, 128).transpose(1, 2)
    out = ops().prefill_attn(q, k, v)
    ops().check_status(q.device)
    ref = _causal_reference(q, k, v, 0, 1.0 / math.sqrt(128))
    assert (out.float() - ref).abs().max().item() <= 2e-2


def test_prefill_attention_rejects_bad_arguments():
    q = torch.zeros(1, 4, 64, 128, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(1, 2, 32, 128, dtype=torch.bfloat16, device="cuda")
    from omnikv_b200.abi import OmniKVError
    with pytest.raises(OmniKVError):
        ops().prefill_attn(q, k, k)  # fewer keys than queries
    with pytest.raises(OmniKVError):
        ops().prefill_attn(q.float(), k.float().repeat(1, 1, 2, 1), k.float().repeat(1, 1, 2, 1))  # fp32


def _linear_reference(x, w, norm_w, eps, epilogue, residual):
    xf = x.float()
    if norm_w is not None:
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * norm_w.float()
    y = xf @ w.float().t()
    if epilogue == "residual":
        y = y + residual.float()
    if epilogue == "swiglu":
        inter = w.shape[0] // 2
        y = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
    return y


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n,rows,K,epilogue,norm", [
    (16, 6144, 4096, "store", True),        # fused QKV projection of the 8B shape behind the input norm
    (16, 4096, 4096, "residual", False),    # output projection + residual
    (16, 28672, 4096, "swiglu", True),      # gate/up behind the post-attention norm
    (16, 4096, 14336, "residual", False),   # down projection + residual: K in eight slices
    (5, 1000, 1024, "store_f32", True),     # rows that do not fill the last block, fp32 logits
    (8, 3584, 8192, "swiglu", True),        # one GPU's share of the 70B gate/up at batch 8
    (1, 256, 64, "store", False),           # one token, one K chunk
    (3, 520, 200, "residual", True),        # K that is not a multiple of 64
])
def test_batched_linear_matches_definition(dtype, n, rows, K, epilogue, norm):
    """tcgen05 weight-streaming projection through the C ABI against fp32 torch: 2e-2 relative to max(1, |y|)."""
    g = torch.Generator().manual_seed(rows + K + n)
    x = torch.randn(n, K, generator=g).to(dtype).cuda()
    w = (torch.randn(rows, K, generator=g) * K ** -0.5).to(dtype).cuda()
    norm_w = (1 + 0.1 * torch.randn(K, generator=g)).to(dtype).cuda() if norm else None
    cols = rows // 2 if epilogue == "swiglu" else rows
    residual = torch.randn(n, cols, generator=g).to(dtype).cuda() if epilogue == "residual" else None
    ref = _linear_reference(x, w, norm_w, 1e-5, epilogue, residual)
    out = ops().batched_linear(x, w, epilogue=epilogue, norm_w=norm_w, eps=1e-5, residual=residual)
    ops().check_status(x.device)
    assert out.shape == (n, cols)
    err = ((out.float() - ref).abs() / ref.abs().clamp(min=1.0)).max().item()
    assert err <= (2e-2 if epilogue != "store_f32" else 1e-2), err
    # the same call again: the workspace counters were left at zero, and sums do not depend on scheduling
    out2 = ops().batched_linear(x, w, epilogue=epilogue, norm_w=norm_w, eps=1e-5, residual=residual)
    assert torch.equal(out, out2)


def test_batched_linear_residual_in_place():
    g = torch.Generator().manual_seed(9)
    x = torch.randn(16, 4096, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(4096, 4096, generator=g) / 64).to(torch.bfloat16).cuda()
    h = torch.randn(16, 4096, generator=g).to(torch.bfloat16).cuda()
    ref = _linear_reference(x, w, None, 0.0, "residual", h)
    ops().batched_linear(x, w, epilogue="residual", residual=h, out=h)
    assert ((h.float() - ref).abs() / ref.abs().clamp(min=1.0)).max().item() <= 2e-2


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float16, 4e-3), (torch.float32, 2e-6)])
@pytest.mark.parametrize("n,hidden,with_delta", [(16, 4096, True), (3, 512, True), (8, 8192, False), (1, 1000, True)])
def test_add_rms_norm(dtype, tol, n, hidden, with_delta):
    g = torch.Generator().manual_seed(hidden + n)
    h = torch.randn(n, hidden, generator=g).to(dtype).cuda()
    delta = torch.randn(n, hidden, generator=g).to(dtype).cuda() if with_delta else None
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype).cuda()
    want_h = (h + delta) if with_delta else h.clone()
    xf = want_h.float()
    want = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    out = ops().add_rms_norm(h, delta, w, 1e-5)
    assert torch.equal(h, want_h)  # the residual stream is updated in place, rounded once
    assert ((out.float() - want).abs() / want.abs().clamp(min=1.0)).max().item() <= tol


def test_prefill_attention_random_shapes():
    """Forty seeded random shapes (batch, grouped heads, chunk lengths that leave partial tiles, chunks at an offset
    inside a longer cache, K/V as strided views) through both prompt-attention kernels against the fp32 definition."""
    rng = np.random.default_rng(77)
    for it in range(40):
        B = int(rng.integers(1, 3))
        KVH = int(rng.choice([1, 2, 4]))
        H = KVH * int(rng.choice([1, 2, 4]))
        Sq = int(rng.integers(1, 700))
        q_pos0 = int(rng.choice([0, 0, int(rng.integers(0, 900))]))
        Skv = q_pos0 + Sq + int(rng.choice([0, 0, int(rng.integers(0, 300))]))
        dtype = torch.bfloat16 if it % 2 == 0 else torch.float16
        g = torch.Generator().manual_seed(1000 + it)
        q = (torch.randn(B, H, Sq, 128, generator=g) * 1.5).to(dtype).cuda()
        if it % 3 == 0:  # K and V side by side in one buffer (row stride of two rows)
            kv = torch.randn(B, KVH, Skv, 2, 128, generator=g).to(dtype).cuda()
            k, v = kv[:, :, :, 0], kv[:, :, :, 1]
        else:
            k = torch.randn(B, KVH, Skv, 128, generator=g).to(dtype).cuda()
            v = torch.randn(B, KVH, Skv, 128, generator=g).to(dtype).cuda()
        ref = _causal_reference(q, k, v, q_pos0, 1.0 / math.sqrt(128))
        for variant in (0, 1):
            out = ops().prefill_attn(q, k, v, q_pos0=q_pos0, variant=variant)
            err = (out.float() - ref).abs().max().item()
            assert err <= 2e-2, (it, variant, B, H, KVH, Sq, Skv, q_pos0, err)
    ops().check_status("cuda")


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float16, 4e-3), (torch.float32, 2e-6)])
def test_rope_window(dtype, tol):
    """Window queries from the q projection: every slot rotated at its sequence's current position, laid out
    [B, H, W, d]; against the rotate_half formula in fp32."""
    B, W, H, d = 3, 16, 8, 128
    g = torch.Generator().manual_seed(12)
    qlin = torch.randn(B, W, H * d, generator=g).to(dtype).cuda()
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).cuda()
    pos = dev_i32([5, 4099, 131071])
    out = ops().rope_window(qlin, H, inv_freq, pos)
    x = qlin.float().view(B, W, H, d).transpose(1, 2)  # [B, H, W, d]
    ang = pos.float()[:, None] * inv_freq[None, :]     # [B, 64]
    cos = torch.cat([ang.cos(), ang.cos()], -1)[:, None, None, :]
    sin = torch.cat([ang.sin(), ang.sin()], -1)[:, None, None, :]
    rot = torch.cat([-x[..., 64:], x[..., :64]], -1)
    want = x * cos + rot * sin
    assert out.shape == (B, H, W, d)
    assert (out.float() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())
