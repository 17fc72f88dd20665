"""KV-head tensor parallelism, host-side logic on CPU ranks (gloo, world size 2): the MAX all-reduce of
per-rank score planes reproduces the selector's max over ALL heads bit for bit, sharded projections sum to
the unsharded result, sharded logits gather back in vocabulary order."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from omnikv_b200 import parallel
    tp = parallel.init(world, rank, None, backend="gloo")
    try:
        g = torch.Generator().manual_seed(0)  # the same tensors on every rank
        B, H, KVH, d, L, k = 2, 8, 4, 16, 300, 40
        q = torch.randn(B, H, d, generator=g)
        kc = torch.randn(B, KVH, L, d, generator=g)
        G = H // KVH
        lo, hi = tp.shard(KVH)
        # what a rank's attention kernel writes: one plane per LOCAL KV head (max over that head's query heads)
        planes = torch.stack([oracle.score_last(q[:, h * G:(h + 1) * G], kc[:, h:h + 1], L) for h in range(lo, hi)])
        tp.all_reduce_max(planes)                       # plane j <- max over ranks of their j-th local head
        score = planes.max(dim=0).values                # what omnikv_topk does with n_planes = local KV heads
        # reference value: the same per-head planes, all of them on one rank (MAX is order independent, so the
        # exchange must reproduce this bit for bit), and the oracle's one-shot score up to matmul rounding
        every = torch.stack([oracle.score_last(q[:, h * G:(h + 1) * G], kc[:, h:h + 1], L) for h in range(KVH)])
        want = every.max(dim=0).values
        ok_score = torch.equal(score, want) and torch.allclose(want, oracle.score_last(q, kc, L), atol=1e-5)
        idx = oracle.topk_ascending(score, k)
        gathered = [torch.empty_like(idx) for _ in range(world)]
        dist.all_gather(gathered, idx)
        ok_idx = all(torch.equal(t, gathered[0]) for t in gathered) and torch.equal(idx, oracle.topk_ascending(want, k))
        # row-parallel output projection: partial products sum to the full one
        w = torch.randn(32, H * d, generator=g)
        attn = torch.randn(B, H * d, generator=g)
        clo, chi = tp.shard(H * d)
        part = attn[:, clo:chi] @ w[:, clo:chi].T
        tp.all_reduce_sum(part)
        ok_sum = torch.allclose(part, attn @ w.T, atol=1e-4)
        # vocabulary-sharded logits
        wl = torch.randn(64, 32, generator=g)
        x = torch.randn(B, 32, generator=g)
        vlo, vhi = tp.shard(64)
        ok_gather = torch.equal(tp.all_gather_last(x @ wl[vlo:vhi].T), x @ wl.T)
        ret[rank] = (ok_score, ok_idx, ok_sum, ok_gather)
    finally:
        dist.destroy_process_group()


def test_tp_exchange_semantics_world2():
    world, port = 2, _free_port()
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: (True, True, True, True), 1: (True, True, True, True)}


def test_shard_rejects_uneven_split():
    from omnikv_b200.parallel import TPGroup
    assert TPGroup(4, 1).shard(8) == (2, 4)
    with pytest.raises(ValueError):
        TPGroup(3, 0).shard(8)
