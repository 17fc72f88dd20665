"""CPU restatement of OmniKV's decode-time selection path (torch CPU, fp32).

TEST INFRASTRUCTURE ONLY -- see the package docstring.  Every function names
the reference lines it follows (paths are relative to the reference project).
The code is written for clarity, not speed: it materialises what the
reference materialises (for example the K cache repeated to all query heads).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch


# ----------------------------------------------------------------------------------------------
# RoPE (transformers' Llama convention: rotate_half, cos/sin of cat(freqs, freqs))
# ----------------------------------------------------------------------------------------------
def rope_cos_sin(position_ids: torch.Tensor, head_dim: int, theta: float = 500000.0):
    """cos/sin tables ``[B, q, head_dim]`` for integer positions ``[B, q]``.

    Follows the default rotary initialisation the reference back-ports in
    modeling/patch_of_llama3_1.py:12-51 (inv_freq = theta^(-2i/d)) and the
    forward of PatchLlamaRotaryEmbedding :599-629 (fp32, cat(freqs, freqs)).
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = position_ids.to(torch.float32)[:, :, None] * inv_freq.to(position_ids.device)[None, None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate ``x [B, heads, q, d]`` with ``cos/sin [B, q', d]`` (q' broadcasts over q).

    modeling/omnikv.py:34-35 passes position_ids of shape [B, 1] while the
    window holds up to 16 queries: the single cos/sin row broadcasts, so every
    window query is rotated at the CURRENT decode position.
    """
    cos = cos.unsqueeze(1)
    sin = sin.unsqueeze(1)
    return x * cos + _rotate_half(x) * sin


def _repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    b, kvh, s, d = x.shape
    if n_rep == 1:
        return x
    return x[:, :, None].expand(b, kvh, n_rep, s, d).reshape(b, kvh * n_rep, s, d)


# ----------------------------------------------------------------------------------------------
# Filter-layer scores
# ----------------------------------------------------------------------------------------------
def score_last(q: torch.Tensor, k_cache: torch.Tensor, consider_len: int) -> torch.Tensor:
    """Raw-logit score of selector ``last``: max over ALL query heads, no softmax.

    q ``[B, H, d]`` (post-RoPE query of the current token), k_cache
    ``[B, KVH, >=consider_len, d]`` (post-RoPE keys).  Returns fp32
    ``[B, consider_len]``.  modeling/omnikv.py:37-46.
    """
    b, h, d = q.shape
    kvh = k_cache.shape[1]
    keys = _repeat_kv(k_cache[:, :, :consider_len].float(), h // kvh)
    s = torch.matmul(q.float()[:, :, None, :], keys.transpose(2, 3)) / math.sqrt(d)  # [B,H,1,L]
    return s[:, :, -1, :].max(dim=1).values


def score_window(
    qw: torch.Tensor, k_cache: torch.Tensor, consider_len: int, selector_cls: str
) -> torch.Tensor:
    """Scores of the window selectors.

    qw ``[B, H, W, d]`` (slot W-1 = current token, all rotated at the current
    position).  ``uniform``: sum over the window of (max over heads of the
    softmax over keys), modeling/omnikv.py:59-78.  ``exp``: the same with the
    recurrence ``acc = acc / 2 + m_w`` from the oldest slot, i.e. weight
    ``2^-(W-1-w)``, :81-104.  ``softmax_before_last``: the W = 1 case of
    ``uniform`` on the last slot, :49-58.
    """
    b, h, w, d = qw.shape
    kvh = k_cache.shape[1]
    keys = _repeat_kv(k_cache[:, :, :consider_len].float(), h // kvh)
    if selector_cls == "softmax_before_last":
        qw = qw[:, :, -1:, :]
        w = 1
    acc = None
    for i in range(w):
        q = qw[:, :, i : i + 1, :].float()
        a = torch.matmul(q, keys.transpose(2, 3)) / math.sqrt(d)
        a = torch.softmax(a, dim=-1)
        m = a.max(dim=1).values.sum(dim=-2)  # [B, L]
        if acc is None:
            acc = m
        elif selector_cls == "exp":
            acc = acc * 0.5 + m
        else:
            acc = acc + m
    return acc


def topk_ascending(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Positions of the k largest scores per row, returned in ascending order (int64).

    modeling/omnikv.py:47-48 (``k = min(k, L)``; torch.topk) and :109 (ascending
    sort of the indices).  torch.topk leaves ties unspecified; this restatement
    fixes the rule "among equal scores the lowest position wins" (a stable
    descending sort), which is also the CUDA kernel's rule.
    """
    k = min(int(k), scores.shape[-1])
    order = torch.sort(scores.float(), dim=-1, descending=True, stable=True).indices[..., :k]
    return torch.sort(order, dim=-1).values


def select_tokens_by_attn_universal(
    raw_attn,
    hidden_states: torch.Tensor,
    position_ids: torch.Tensor,
    past_key_value,
    num_selected_tokens: int,
    consider_len: int,
    layer_idx: Optional[int] = None,
    selector_cls: str = "last",
) -> torch.Tensor:
    """Restatement of modeling/omnikv.py:8-110 with the same signature.

    ``raw_attn`` is duck-typed exactly as in the reference: ``q_proj``,
    ``num_heads``, ``head_dim``, ``num_key_value_heads``, ``rotary_emb(x,
    position_ids) -> (cos, sin)``, ``layer_idx``.  (The reference also
    projects and rotates a key it then discards, :25,:37; that is skipped.)
    """
    bsz, q_len, _ = hidden_states.shape
    q = raw_attn.q_proj(hidden_states)
    q = q.view(bsz, q_len, raw_attn.num_heads, raw_attn.head_dim).transpose(1, 2)
    cos, sin = raw_attn.rotary_emb(q, position_ids)
    q = apply_rope(q, cos, sin)  # [B, H, W, d]
    k_cache = past_key_value.key_cache[raw_attn.layer_idx]
    if selector_cls == "last":
        s = score_last(q[:, :, -1, :], k_cache, consider_len)
    elif selector_cls in ("softmax_before_last", "uniform", "exp"):
        s = score_window(q, k_cache, consider_len, selector_cls)
    else:
        raise NotImplementedError(selector_cls)
    select_tokens_by_attn_universal.last_scores = s  # for tests that check a selection up to a score band
    return topk_ascending(s, num_selected_tokens)


def selector_k_rule(
    num_of_selected_tokens,
    prefill_len: int,
    selector_cls: str,
    window_size: int,
    decode_step: int,
) -> Tuple[int, int, int]:
    """(k, consider_len, nptw) exactly as modeling/omnikv.py:167-188 computes them.

    A float ``num_of_selected_tokens`` is a fraction of the prompt and is
    TRUNCATED (``int``), :169-171.  For the window selectors the ``nptw =
    max(0, window_size - decode_step)`` newest prompt positions still inside the
    observation window are taken out of the candidate range and out of k
    (:178,:186-188); the caller appends them after selection (:199-210).
    """
    k = num_of_selected_tokens
    if isinstance(k, float):
        k = int(k * prefill_len)
    consider_len = prefill_len
    nptw = max(0, window_size - decode_step)
    if "last" not in selector_cls:
        consider_len -= nptw
        k = max(1, k - nptw)
    else:
        nptw = 0
    return int(k), int(consider_len), int(nptw)


# ----------------------------------------------------------------------------------------------
# Layer plan and cache flow
# ----------------------------------------------------------------------------------------------
def full_attn_layers_of(do_select_layers: Sequence[int], num_hidden_layers: int) -> List[int]:
    """modeling/omnikv.py:322-331: every layer before the first filter layer, the
    filter layers, and the sentinel ``num_hidden_layers``."""
    sel = list(do_select_layers)
    return list(range(0, sel[0])) + sel + [num_hidden_layers]


def layer_plan(full_attn_layers: Sequence[int], num_hidden_layers: int, num_wait_layers: int) -> Dict[int, Tuple[bool, int, int]]:
    """``layer -> (is_sparse, group_start, group_end)``, modeling/spec_cache.py:272-281."""
    state: Dict[int, Tuple[bool, int, int]] = {}
    full = list(full_attn_layers)
    for _l in full:
        _r = num_hidden_layers
        for i in range(_l + 1, num_hidden_layers):
            if i in full:
                _r = i
                break
        for i in range(_l, min(_r, _l + num_wait_layers + 1)):
            state[i] = (False, _l, _r)
        for i in range(min(_r, _l + num_wait_layers + 1), _r):
            state[i] = (True, _l, _r)
    return state


class OracleMultiStageCache:
    """Restatement of OmniKVMultiStageCache, modeling/spec_cache.py:253-385.

    Same attribute names and the same ``update`` / ``set_idx_on_gpu`` flow, with
    ``torch.cat`` re-copies kept.  ``real_offload`` only changes where the
    sparse layers' prompt KV lives, which on a CPU oracle is a no-op.
    """

    def __init__(self, full_attn_layers, num_hidden_layers, num_wait_load_layers=2, real_offload=True):
        self.stage = "prefill"
        self.full_attn_layers = list(full_attn_layers)
        self.num_hidden_layers = num_hidden_layers
        self.num_wait_layers = num_wait_load_layers
        self.layer_state = layer_plan(full_attn_layers, num_hidden_layers, num_wait_load_layers)
        self.device = "cpu" if real_offload else None
        self.key_cache: List[torch.Tensor] = []
        self.value_cache: List[torch.Tensor] = []
        self._seen_tokens = 0
        self.part_key: Dict[int, torch.Tensor] = {}
        self.part_value: Dict[int, torch.Tensor] = {}
        self.tail_k: Dict[int, torch.Tensor] = {}
        self.tail_v: Dict[int, torch.Tensor] = {}

    def set_idx_on_gpu(self, idx: torch.Tensor, sel_layer_idx: int) -> None:
        """:290-306 -- gather the selected prompt rows of EVERY sparse layer of the
        group that starts at ``sel_layer_idx``.  ``idx.view(-1)`` flattens the
        batch, so the reference is only meaningful at batch 1."""
        _idx = idx.reshape(-1)
        _r = self.layer_state[sel_layer_idx][2]
        for i in range(sel_layer_idx + self.num_wait_layers + 1, _r):
            self.part_key[i] = torch.index_select(self.key_cache[i], 2, _idx)
            self.part_value[i] = torch.index_select(self.value_cache[i], 2, _idx)

    def _gather_hook(self, layer_idx: int) -> None:
        pass

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        """:308-369."""
        if layer_idx == 0:
            self._seen_tokens += key_states.shape[-2]
        if self.layer_state[layer_idx][0]:
            if self.stage == "prefill":
                self.key_cache.append(key_states)
                self.value_cache.append(value_states)
                return key_states, value_states
            if layer_idx not in self.tail_k:
                self.tail_k[layer_idx] = key_states
                self.tail_v[layer_idx] = value_states
            else:
                self.tail_k[layer_idx] = torch.cat([self.tail_k[layer_idx], key_states], dim=-2)
                self.tail_v[layer_idx] = torch.cat([self.tail_v[layer_idx], value_states], dim=-2)
            self._gather_hook(layer_idx)
            return (
                torch.cat([self.part_key[layer_idx], self.tail_k[layer_idx]], dim=-2),
                torch.cat([self.part_value[layer_idx], self.tail_v[layer_idx]], dim=-2),
            )
        if len(self.key_cache) <= layer_idx:
            self.key_cache.append(key_states)
            self.value_cache.append(value_states)
        else:
            self.key_cache[layer_idx] = torch.cat([self.key_cache[layer_idx], key_states], dim=-2)
            self.value_cache[layer_idx] = torch.cat([self.value_cache[layer_idx], value_states], dim=-2)
        return self.key_cache[layer_idx], self.value_cache[layer_idx]


class OracleWOPackCache(OracleMultiStageCache):
    """Restatement of WOPackCache, modeling/spec_cache.py:388-520: the index list is
    only remembered at the filter layer (:426-429) and each sparse layer
    gathers its own rows inside ``update`` (:477-483)."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.idx = None

    def set_idx_on_gpu(self, idx, sel_layer_idx):
        self.idx = idx.reshape(-1)

    def _gather_hook(self, layer_idx):
        self.part_key[layer_idx] = torch.index_select(self.key_cache[layer_idx], 2, self.idx)
        self.part_value[layer_idx] = torch.index_select(self.value_cache[layer_idx], 2, self.idx)


def idx_iou_score(new_idx: torch.Tensor, old_idx: torch.Tensor) -> float:
    """Overlap score of two index lists, modeling/spec_cache.py:10-31: the size of the intersection (counted as
    ``|new| + |old| - |unique(cat(new, old))|``) divided by ``|new|`` -- not a true IoU, the reference's
    comment says so."""
    new_idx, old_idx = new_idx.reshape(-1), old_idx.reshape(-1)
    un = torch.cat([new_idx, old_idx]).unique().numel()
    return (new_idx.numel() + old_idx.numel() - un) / new_idx.numel()


class OracleLazyRule:
    """The re-gather rule of OmniKVLazyCache.set_out_idx, modeling/spec_cache.py:539-557: a new index list
    replaces the one in use unless its overlap score with it is ABOVE ``skip_threshold``; the first list is
    always taken."""

    def __init__(self, skip_threshold: float = 0.4):
        self.skip_threshold = skip_threshold
        self.live: Dict[int, torch.Tensor] = {}
        self.last: Dict[int, Tuple[bool, float]] = {}  # outcome of the latest offer per group

    def offer(self, idx: torch.Tensor, sid: int) -> Tuple[bool, float]:
        """Returns (taken, score against the list in use or -1.0)."""
        score = -1.0
        if sid in self.live:
            score = idx_iou_score(idx, self.live[sid])
            if score > self.skip_threshold:
                self.last[sid] = (False, score)
                return False, score
        self.live[sid] = idx.clone()
        self.last[sid] = (True, score)
        return True, score


class OracleLazyMultiStageCache(OracleMultiStageCache):
    """The multi-stage cache with the lazy rule in front of ``set_idx_on_gpu``: a filter group keeps its
    gathered rows while consecutive selections overlap enough (the rule of :539-557 applied per group)."""

    def __init__(self, *a, skip_threshold: float = 0.4, **kw):
        super().__init__(*a, **kw)
        self.rule = OracleLazyRule(skip_threshold)

    def set_idx_on_gpu(self, idx, sel_layer_idx):
        taken, _ = self.rule.offer(idx, sel_layer_idx)
        if taken:
            super().set_idx_on_gpu(idx, sel_layer_idx)


# ----------------------------------------------------------------------------------------------
# Decode attention (the third-party part of the reference path: the mathematical definition)
# ----------------------------------------------------------------------------------------------
def dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """softmax(q K^T / sqrt(d)) V for one decode token.

    q ``[B, H, d]``; k, v ``[B, KVH, n, d]`` (what ``cache.update`` returned,
    modeling/spec_cache.py:358-369 for dense layers).  GQA: query head h reads
    KV head h // (H / KVH).  fp32 throughout.  Returns ``[B, H, d]``.
    """
    b, h, d = q.shape
    kvh = k.shape[1]
    kk = _repeat_kv(k.float(), h // kvh)
    vv = _repeat_kv(v.float(), h // kvh)
    s = torch.matmul(q.float()[:, :, None, :], kk.transpose(2, 3)) / math.sqrt(d)
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vv)[:, :, 0, :]


def sparse_attention(
    q: torch.Tensor,
    k_prompt: torch.Tensor,
    v_prompt: torch.Tensor,
    idx: torch.Tensor,
    tail_k: Optional[torch.Tensor] = None,
    tail_v: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Decode attention of a sparse layer: the selected prompt rows followed by
    every decode-time row (modeling/spec_cache.py:337-356), per sequence.

    idx ``[B, k]`` int64 ascending; the selection is applied per sequence
    (the reference's ``idx.view(-1)`` is only meaningful at batch 1).
    """
    outs = []
    for b in range(q.shape[0]):
        kb = torch.index_select(k_prompt[b : b + 1], 2, idx[b])
        vb = torch.index_select(v_prompt[b : b + 1], 2, idx[b])
        if tail_k is not None and tail_k.shape[2] > 0:
            kb = torch.cat([kb, tail_k[b : b + 1]], dim=2)
            vb = torch.cat([vb, tail_v[b : b + 1]], dim=2)
        outs.append(dense_attention(q[b : b + 1], kb, vb))
    return torch.cat(outs, dim=0)
