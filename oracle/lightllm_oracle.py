"""CPU restatement of the decode attention of the reference's LightLLM fork, for parity tests.

TEST INFRASTRUCTURE ONLY: imported by tests/ (never by the package).

Follows omnikv-lightllm/lightllm/models/llama_omnikv/triton_kernel/flash_decoding.py: a request's tokens
live in pool rows ``req_to_token_indexs[req, :len]`` of ``kv_buffer[layer] [tokens, 2*KVH, d]``
(common/req_manager.py:12-17, common/mem_manager.py:102-104).  A filter layer (``do_select``) attends over
all of them and scores every position with the max over the rank's query heads of the RAW logit (the stage-1
kernel stores q . k before the softmax scale, flash_decoding_stage1.py:203-207; :61-75 take the max over heads),
keeps the ``min(2048, len)`` best (:79-83) and records their pool rows (:85-93); later layers attend over the
recorded rows.  The fork's own staging of those rows is a placeholder its author marks as not correct (:98-112),
so "attention over exactly the selected tokens" is the stage-1 / stage-2 kernels run over the recorded rows.

PINNED by tests/golden/lightllm.npz: the fork's own Triton kernels (flash_decoding_stage1.py,
flash_decoding_stage2.py), loaded by path and run on CPU tensors by Triton's interpreter
(tests/golden/make_golden.py::make_lightllm_fixture): outputs of the selecting and of the plain call, the
per-position scores, the top-2048 choice, the attention over the chosen rows (tests/test_oracle_golden.py).
"""
from __future__ import annotations

from typing import List, Tuple

import torch

from .omnikv_oracle import dense_attention, score_last, topk_ascending


def gather_request(pool_k: torch.Tensor, pool_v: torch.Tensor, rows: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Pool halves ``[tokens, KVH, d]`` and a list of pool rows -> ``[1, KVH, n, d]`` K and V."""
    k = pool_k[rows.long()].permute(1, 0, 2)[None]
    v = pool_v[rows.long()].permute(1, 0, 2)[None]
    return k, v


def paged_decode_attention(q, pool_k, pool_v, table, b_req_idx, b_seq_len) -> torch.Tensor:
    """Dense decode attention per request over its pages (flash_decoding.py:189-214).  q ``[B, H, d]``."""
    outs = []
    for b in range(q.shape[0]):
        rows = table[int(b_req_idx[b]), : int(b_seq_len[b])]
        k, v = gather_request(pool_k, pool_v, rows)
        outs.append(dense_attention(q[b : b + 1], k, v))
    return torch.cat(outs, dim=0)


def fork_scores(q, pool_k, table, b_req_idx, b_seq_len) -> List[torch.Tensor]:
    """Per request the score the fork selects by: max over the query heads of the raw logit q . k of every
    position (what flash_decode_stage1_with_score leaves in Attn_Score, maxed over dim 1 at flash_decoding.py:75)."""
    res = []
    for b in range(q.shape[0]):
        n = int(b_seq_len[b])
        rows = table[int(b_req_idx[b]), :n]
        k = pool_k[rows.long()].permute(1, 0, 2)  # [KVH, n, d]
        G = q.shape[1] // k.shape[0]
        logits = torch.einsum("hd,hnd->hn", q[b].float(), k.float().repeat_interleave(G, dim=0))
        res.append(logits.max(dim=0).values)
    return res


def select_positions(q, pool_k, table, b_req_idx, b_seq_len, num_imp_tokens: int = 2048,
                     keep_recent: int = 0) -> List[torch.Tensor]:
    """Positions (ascending) each request keeps: top ``min(num_imp_tokens, len)`` of the raw-logit score
    (flash_decoding.py:75-83); with ``keep_recent`` the newest tokens are kept unconditionally and the top-k
    runs over the older ones."""
    res = []
    for b in range(q.shape[0]):
        n = int(b_seq_len[b])
        rows = table[int(b_req_idx[b]), :n]
        k = pool_k[rows.long()].permute(1, 0, 2)[None]
        cand = max(0, n - keep_recent)
        kk = min(num_imp_tokens - keep_recent, cand)
        s = score_last(q[b : b + 1], k, cand)
        top = topk_ascending(s, kk)[0] if kk > 0 else torch.zeros(0, dtype=torch.long)
        res.append(torch.cat([top, torch.arange(cand, n)]))
    return res


def selected_decode_attention(q, pool_k, pool_v, table, b_req_idx, positions: List[torch.Tensor]) -> torch.Tensor:
    """Decode attention over the selected tokens only."""
    outs = []
    for b in range(q.shape[0]):
        rows = table[int(b_req_idx[b])][positions[b]]
        k, v = gather_request(pool_k, pool_v, rows)
        outs.append(dense_attention(q[b : b + 1], k, v))
    return torch.cat(outs, dim=0)
