"""The package's decode kernels behind the plug point of the reference's LightLLM fork.

The fork replaces LightLLM's decode attention with ``token_decode_attention_flash_decoding(q, infer_state,
q_head_num, head_dim, cache_k, cache_v, out, alloc_tensor_func, do_select, world_size, tp_rank)``
(omnikv-lightllm/lightllm/models/llama_omnikv/triton_kernel/flash_decoding.py:7-19, called from
layer_infer/transformer_layer_infer.py:567-598).  This module offers a function of that name and signature
over the same data structures:

* the KV pool of a layer is ``kv_buffer[layer] [tokens, 2*KVH/tp, d]`` (common/mem_manager.py:102-104);
  ``cache_k`` / ``cache_v`` are its two halves along dim 1 (transformer_layer_infer.py:574-579);
* ``infer_state.req_manager.req_to_token_indexs [requests, max_seq] int32`` maps (request, position) to a
  pool row, ``req_to_imp_token_indexs [8, requests, 2048 + 300] int32`` holds, per TP rank, the pool rows of
  the selected tokens (common/req_manager.py:12-17);
* ``infer_state.b_req_idx``, ``b_seq_len`` (int32 ``[B]``), ``batch_size``, ``max_len_in_batch``,
  ``is_prefill``; the function sets ``imp_seq_len`` and ``max_imp_len_batch`` on a filter layer
  (flash_decoding.py:39-40,94-97) and reads them on the layers after it (:176-177).

What the calls do:

* ``do_select=True`` (a filter layer): dense attention over the request's pages and, from the same pass over
  K, the selection score ``max over the rank's heads of q.k/sqrt(d)`` (:61-75); the ``min(2048, len)`` best
  positions (:79-83) are translated to pool rows and stored in ``req_to_imp_token_indexs[tp_rank, req]``
  (:85-93).  One attention launch and one top-k launch replace stage 1 with scores, ``max(dim=1)``,
  ``torch.topk`` and ``index_select``.
* ``do_select=False`` after a filter layer: attention over the selected pool rows only.  The fork stages
  these rows through a host copy with placeholder indices that its author marks as not correct and
  efficiency-only (:98-112, :181-187); here the kernel reads the selected rows in place through the index
  table, so no copy exists and the result is the attention over exactly the selected tokens.
* ``do_select=False`` before any filter layer: dense attention over the request's pages (:169-202).

Differences from the fork, all deliberate: batches larger than one select per sequence (the fork asserts
``batch_size == 1``, :77); the stored rows are in ascending position order, not in score order (attention does
not depend on the order); ``score_group`` optionally MAX-reduces the scores over the tensor-parallel ranks so
that every rank selects the same tokens (the fork selects per rank from its local heads, :76); ``keep_recent``
optionally forces the newest tokens into the selection.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from . import ops

NUM_IMP_TOKENS = 2048  # flash_decoding.py:79


def _pool_view(cache: torch.Tensor, B: int) -> torch.Tensor:
    """``[tokens, KVH, d]`` pool half -> the kernels' ``[B, KVH, rows, d]`` with a zero batch stride."""
    if cache.dim() != 3 or cache.stride(2) != 1:
        raise ValueError("cache_k / cache_v must be [tokens, kv_heads, head_dim] with contiguous head vectors")
    return cache.permute(1, 0, 2).unsqueeze(0).expand(B, -1, -1, -1)


def _const_i32(infer_state, name: str, value: int, B: int, device) -> torch.Tensor:
    """A device ``[B]`` int32 constant, kept on the infer state so that a layer loop allocates it once."""
    key = f"_omnikv_{name}_{value}_{B}"
    t = getattr(infer_state, key, None)
    if t is None or t.device != device:
        t = torch.full((B,), value, dtype=torch.int32, device=device)
        setattr(infer_state, key, t)
    return t


def token_decode_attention_flash_decoding(
    q: torch.Tensor,
    infer_state,
    q_head_num: int,
    head_dim: int,
    cache_k: torch.Tensor,
    cache_v: torch.Tensor,
    out: Optional[torch.Tensor] = None,
    alloc_tensor_func: Callable = torch.empty,
    do_select: bool = False,
    world_size: int = 1,
    tp_rank: int = 0,
    *,
    num_imp_tokens: int = NUM_IMP_TOKENS,
    keep_recent: int = 0,
    score_group=None,
) -> torch.Tensor:
    if getattr(infer_state, "is_prefill", False):
        raise AssertionError("decode only")  # flash_decoding.py:32
    B = int(infer_state.batch_size)
    max_len = int(infer_state.max_len_in_batch)
    req_mgr = infer_state.req_manager
    table = req_mgr.req_to_token_indexs
    b_req_idx, b_seq_len = infer_state.b_req_idx, infer_state.b_seq_len
    if b_req_idx.dim() != 1:
        raise AssertionError("b_req_idx must be one-dimensional")  # :38
    if table.dtype != torch.int32 or b_req_idx.dtype != torch.int32 or b_seq_len.dtype != torch.int32:
        raise TypeError("req_to_token_indexs, b_req_idx and b_seq_len must be int32")
    o_tensor = alloc_tensor_func(q.shape, dtype=q.dtype, device=q.device) if out is None else out
    q3, o3 = q.view(B, q_head_num, head_dim), o_tensor.view(B, q_head_num, head_dim)
    k4, v4 = _pool_view(cache_k, B), _pool_view(cache_v, B)
    kvh = cache_k.shape[1]

    if do_select:
        imp = req_mgr.req_to_imp_token_indexs
        n_imp = min(int(num_imp_tokens), max_len)
        if imp.shape[-1] < n_imp:
            raise ValueError("req_to_imp_token_indexs is narrower than the number of selected tokens")
        if not 0 <= keep_recent < n_imp:
            raise ValueError("keep_recent must be smaller than the number of selected tokens")
        stride = (max_len + 7) // 8 * 8
        planes = alloc_tensor_func((kvh, B, stride), dtype=torch.float32, device=q.device)
        ops.decode_attn(q3, k4, v4, b_seq_len, idx=table, idx_row=b_req_idx, out=o3, score_out=planes,
                        score_len=b_seq_len, max_rows=max_len)
        if score_group is not None and world_size > 1:
            torch.distributed.all_reduce(planes, op=torch.distributed.ReduceOp.MAX, group=score_group)
        k_dev = _const_i32(infer_state, "k", n_imp - keep_recent, B, q.device)
        pos = alloc_tensor_func((B, n_imp), dtype=torch.int32, device=q.device)
        count = torch.empty_like(b_seq_len)
        if keep_recent:
            # candidates: all but the newest keep_recent tokens, which are appended after the top-k
            cand = torch.clamp(b_seq_len - keep_recent, min=0)
            ops.topk(planes, cand, k_dev, append_n=b_seq_len - cand, idx_out=pos, count_out=count, max_len=max_len)
        else:
            ops.topk(planes, b_seq_len, k_dev, idx_out=pos, count_out=count, max_len=max_len)
        # positions -> pool rows, stored in this rank's table of selected rows (:85-93)
        lin = b_req_idx.long().unsqueeze(1) * table.shape[1] + pos.long().clamp_(0, table.shape[1] - 1)
        rows = table.reshape(-1)[lin]
        imp[tp_rank].index_put_((b_req_idx.long().unsqueeze(1), torch.arange(n_imp, device=q.device).unsqueeze(0)), rows)
        infer_state.imp_seq_len = count
        infer_state.max_imp_len_batch = n_imp
        return o_tensor

    if getattr(infer_state, "imp_seq_len", None) is not None:
        ops.decode_attn(q3, k4, v4, infer_state.imp_seq_len, idx=req_mgr.req_to_imp_token_indexs[tp_rank],
                        idx_row=b_req_idx, out=o3, max_rows=int(infer_state.max_imp_len_batch))
    else:
        ops.decode_attn(q3, k4, v4, b_seq_len, idx=table, idx_row=b_req_idx, out=o3, max_rows=max_len)
    return o_tensor
