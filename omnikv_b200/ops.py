"""Tensor-level wrappers over the C ABI: they take ``torch`` CUDA tensors, pass raw pointers,
sizes and element strides to ``libomnikv_b200.so`` and launch on the current CUDA stream.

PyTorch is used here for device memory and streams only.  Nothing in this module computes a
result on its own: if the library is missing, every call raises.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import torch

from . import abi

_DT = {torch.float32: abi.F32, torch.bfloat16: abi.BF16, torch.float16: abi.F16}
_SEL = {"softmax_before_last": abi.SEL_SOFTMAX_LAST, "uniform": abi.SEL_UNIFORM, "exp": abi.SEL_EXP}

_sm_count = {}
_workspaces = {}
_retired_workspaces = []
_launches = 0


def launch_count() -> int:
    """Kernels of this library launched so far by this process (each ABI call adds what it launches)."""
    return _launches


def _count(n: int) -> None:
    global _launches
    _launches += n


def _dev_index(device) -> int:
    """Ordinal of a CUDA device given as a tensor's device, a torch.device, a string or an int ("cuda" = current)."""
    idx = torch.device(device).index if not isinstance(device, int) else device
    return torch.cuda.current_device() if idx is None else idx


def sm_count(device) -> int:
    idx = _dev_index(device)
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise abi.OmniKVError("omnikv_b200 kernels need CUDA tensors; there is no CPU path")


def workspace(device, nbytes: int, tag: str = "default") -> torch.Tensor:
    """A cached per-device scratch tensor of at least ``nbytes`` bytes (the caller of the C ABI
    owns the workspace; this cache is that caller).  Grows on demand, and a buffer that has been handed out is
    never freed: a CUDA graph captured earlier has its address baked in and keeps replaying into it, so the
    outgrown buffer stays alive beside the larger one (a few MB per growth).  Never call it with a larger size
    for the first time while a CUDA graph is being captured."""
    key = (_dev_index(device), tag)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired_workspaces.append(ws)
        # zero-filled: the decode-attention workspace starts with arrival counters that must be zero
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def default_splits(B: int, KVH: int, max_rows: int, device) -> int:
    """Split count that fills the GPU with about two CTAs per SM, at least 128 rows per split."""
    ctas = B * KVH
    if B > 1 and max_rows <= 8192:
        # short lists of a batch (the selected rows of sparse layers): a CTA costs about seven 64-row tiles of fixed
        # time (prologue, split merge) whatever it streams, and two CTAs fit on an SM, so the count that minimises
        # waves x (tiles per CTA + 7) wins -- 2 instead of 5 for 16 sequences x 8 KV heads x 2112 rows
        slots, tiles = 2 * sm_count(device), -(-max_rows // 64)
        # (few sequences, e.g. eight with one local KV head each, want many splits: the merge of c partials costs
        # about c / 16 further tile times)
        s = min(range(1, 65), key=lambda c: (-(-ctas * c // slots)) * (-(-tiles // c) + 7 + c / 16))
    elif B > 1:  # ragged batches: chunks are sized by the longest sequence, so aim at two waves of equal CTAs
        s = -(-4 * sm_count(device) // ctas)
    else:
        # two CTAs per SM, but never more splits than SMs: the last CTA of a (sequence, KV head) merges all of them, and
        # with one local KV head (8-way tensor parallelism) 296 partials cost more than the second CTA per SM gains
        # (28.3 -> 21.6 us per dense layer of one rank's share)
        s = min((2 * sm_count(device)) // max(1, ctas), sm_count(device))
    return max(1, min(s, (max_rows + 127) // 128))


def _kv_strides(t: torch.Tensor) -> Tuple[int, int, int]:
    if t.dim() != 4 or t.stride(3) != 1:
        raise abi.OmniKVError("KV tensors must be [B, KVH, rows, d] with contiguous rows")
    return t.stride(0), t.stride(1), t.stride(2)


def decode_attn(
    q: torch.Tensor,
    k: torch.Tensor,
    v: Optional[torch.Tensor],
    len_a: torch.Tensor,
    *,
    idx: Optional[torch.Tensor] = None,
    idx_row: Optional[torch.Tensor] = None,
    k_tail: Optional[torch.Tensor] = None,
    v_tail: Optional[torch.Tensor] = None,
    tail_start: Optional[torch.Tensor] = None,
    tail_len: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    score_out: Optional[torch.Tensor] = None,
    score_len: Optional[torch.Tensor] = None,
    n_splits: Optional[int] = None,
    max_rows: Optional[int] = None,
    scale: Optional[float] = None,
    ws: Optional[torch.Tensor] = None,
    scores_only: bool = False,
    state_capacity: bool = True,
) -> Optional[torch.Tensor]:
    """``omnikv_decode_attn``.  q ``[B,H,d]``; k, v ``[B,KVH,rows,d]``; ``len_a`` int32 ``[B]`` on
    the device; ``idx`` int32 ``[B, >=len_a]`` selects rows of (k, v) (with ``idx_row`` int32 ``[B]``, batch
    entry b reads row ``idx_row[b]`` of ``idx`` -- a request table over a paged pool); the tail is
    ``tail_len[b]`` rows of (k_tail, v_tail) from ``tail_start[b]``.  ``score_out``
    ``[KVH,B,stride]`` fp32 receives the per-KV-head selector-``last`` scores of positions
    ``< score_len[b]``.  ``state_capacity=False`` withholds the cache's row capacity from the kernel (it then
    uses its cp.async variant on dense layers).  Returns ``out`` ``[B,H,d]`` (None when ``scores_only``)."""
    _need_cuda(q, k, v, len_a, idx, idx_row, k_tail, v_tail, out, score_out)
    B, H, d = q.shape
    KVH = k.shape[1]
    if q.stride(2) != 1:
        raise abi.OmniKVError("q must have contiguous head vectors")
    p = abi.AttnParams()
    p.dtype = _DT[q.dtype]
    p.B, p.H, p.KVH, p.head_dim = B, H, KVH, d
    p.scale = float(scale if scale is not None else 1.0 / math.sqrt(d))
    p.q, p.q_stride_b, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    if not scores_only:
        if out is None:
            out = torch.empty_like(q)
        if out.stride() != q.stride():
            raise abi.OmniKVError("out must have the strides of q")
        p.out = out.data_ptr()
    p.kA, p.vA = k.data_ptr(), _ptr(v)
    p.a_stride_b, p.a_stride_h, p.a_stride_row = _kv_strides(k)
    if v is not None and _kv_strides(v) != _kv_strides(k):
        raise abi.OmniKVError("k and v must share strides")
    if idx is not None:
        if idx.dtype != torch.int32 or idx.stride(-1) != 1:
            raise abi.OmniKVError("idx must be contiguous int32")
        p.idxA, p.idx_stride = idx.data_ptr(), idx.stride(0) if idx.dim() == 2 else 0
        if idx_row is not None:
            if idx_row.dtype != torch.int32 or not idx_row.is_contiguous() or idx_row.numel() != B:
                raise abi.OmniKVError("idx_row must be contiguous int32 [B]")
            p.idx_row = idx_row.data_ptr()
    elif idx_row is not None:
        raise abi.OmniKVError("idx_row needs idx")
    if len_a.dtype != torch.int32:
        raise abi.OmniKVError("len_a must be int32")
    p.lenA = len_a.data_ptr()
    if tail_len is not None:
        p.kB, p.vB = k_tail.data_ptr(), _ptr(v_tail)
        p.b_stride_b, p.b_stride_h, p.b_stride_row = _kv_strides(k_tail)
        p.startB, p.lenB = tail_start.data_ptr(), tail_len.data_ptr()
    if score_out is not None:
        if score_out.dtype != torch.float32 or score_out.dim() != 3 or score_out.shape[0] != KVH or not score_out.is_contiguous():
            raise abi.OmniKVError("score_out must be contiguous fp32 [KVH, B, stride]")
        p.score_out, p.score_stride, p.score_len = score_out.data_ptr(), score_out.stride(1), score_len.data_ptr()
    if max_rows is None:
        max_rows = k.shape[2] + (k_tail.shape[2] if k_tail is not None else 0)
    p.n_splits = int(n_splits or default_splits(B, KVH, max_rows, q.device))
    if not scores_only:
        need = abi.lib().omnikv_decode_attn_workspace_bytes(B, H, p.n_splits)
        if ws is None:
            ws = workspace(q.device, need, "attn")
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel() * ws.element_size()
    p.status = status_word(q.device).data_ptr()
    # the row capacity lets a dense 16-bit layer fetch its tiles through a TMA tensor map
    p.a_rows = k.shape[2] if state_capacity else 0
    abi.check(abi.lib().omnikv_decode_attn(C.byref(p), _stream()), "omnikv_decode_attn")
    _count(1)  # one kernel: the last CTA of every (sequence, KV head) merges the splits
    return out


def score_last(q: torch.Tensor, k: torch.Tensor, score_len: torch.Tensor, *, score_out: Optional[torch.Tensor] = None,
               n_splits: Optional[int] = None, scale: Optional[float] = None) -> torch.Tensor:
    """Selector-``last`` score planes ``[KVH, B, rows]`` (max over a KV head's query heads of the scaled
    raw logits) without the attention output: the score-only mode of ``omnikv_decode_attn``."""
    B, KVH, rows = q.shape[0], k.shape[1], k.shape[2]
    if score_out is None:
        score_out = torch.empty(KVH, B, rows, dtype=torch.float32, device=q.device)
    decode_attn(q, k, None, score_len, score_out=score_out, score_len=score_len, n_splits=n_splits, scale=scale,
                scores_only=True)
    return score_out


def topk(scores: torch.Tensor, length: torch.Tensor, k: torch.Tensor, *, append_n: Optional[torch.Tensor] = None,
         idx_out: Optional[torch.Tensor] = None, count_out: Optional[torch.Tensor] = None,
         max_len: Optional[int] = None, ws: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``omnikv_topk``.  scores fp32 ``[B, n]`` or planes ``[P, B, n]`` (max over P is taken);
    ``length``, ``k`` (and ``append_n``) int32 ``[B]`` on the device.  Returns (idx int32 ``[B, cap]``
    ascending, count int32 ``[B]``)."""
    _need_cuda(scores, length, k, append_n, idx_out, count_out)
    if scores.dtype != torch.float32 or scores.stride(-1) != 1:
        raise abi.OmniKVError("scores must be fp32 with contiguous rows")
    if scores.dim() == 2:
        n_planes, plane_stride, B, batch_stride = 1, 0, scores.shape[0], scores.stride(0)
    else:
        n_planes, plane_stride, B, batch_stride = scores.shape[0], scores.stride(0), scores.shape[1], scores.stride(1)
    if max_len is None:
        max_len = scores.shape[-1]
    if idx_out is None:
        idx_out = torch.empty(B, max_len, dtype=torch.int32, device=scores.device)
    if count_out is None:
        count_out = torch.empty(B, dtype=torch.int32, device=scores.device)
    need = abi.lib().omnikv_topk_workspace_bytes(B, max_len)
    if ws is None and max_len > 8 * 49152:
        ws = workspace(scores.device, need, "topk")
    abi.check(
        abi.lib().omnikv_topk(scores.data_ptr(), n_planes, plane_stride, batch_stride, length.data_ptr(), k.data_ptr(),
                              _ptr(append_n), B, int(max_len), idx_out.data_ptr(), idx_out.stride(0),
                              count_out.data_ptr(), _ptr(ws), 0 if ws is None else ws.numel() * ws.element_size(),
                              _stream()),
        "omnikv_topk")
    _count(1)
    return idx_out, count_out


def score_window(qw: torch.Tensor, k: torch.Tensor, consider_len: torch.Tensor, selector: str, *, max_len: int,
                 score_out: Optional[torch.Tensor] = None, planes_out: Optional[torch.Tensor] = None,
                 scale: Optional[float] = None, ws: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``omnikv_score_window``.  qw ``[B,H,W,d]`` contiguous; k ``[B,KVH,rows,d]``.  Returns fp32 scores
    ``[B, stride]`` (positions ``>= consider_len[b]`` are left untouched), or fills ``planes_out``
    ``[B,W,stride]`` with the max over the local heads when given."""
    _need_cuda(qw, k, consider_len, score_out, planes_out)
    B, H, W, d = qw.shape
    if not qw.is_contiguous():
        raise abi.OmniKVError("qw must be contiguous [B,H,W,d]")
    p = abi.WindowParams()
    p.dtype = _DT[qw.dtype]
    p.B, p.H, p.KVH, p.head_dim, p.W = B, H, k.shape[1], d, W
    p.selector = _SEL[selector]
    p.scale = float(scale if scale is not None else 1.0 / math.sqrt(d))
    p.qw, p.k = qw.data_ptr(), k.data_ptr()
    p.k_stride_b, p.k_stride_h, p.k_stride_row = _kv_strides(k)
    p.consider_len, p.max_len = consider_len.data_ptr(), int(max_len)
    if planes_out is None and score_out is None:
        score_out = torch.empty(B, max_len, dtype=torch.float32, device=qw.device)
    if score_out is not None:
        p.score_out, p.score_stride = score_out.data_ptr(), score_out.stride(0)
    if planes_out is not None:
        p.planes_out, p.score_stride = planes_out.data_ptr(), planes_out.stride(1)
    need = abi.lib().omnikv_score_window_workspace_bytes(B, H, W, int(max_len))
    if ws is None:
        ws = workspace(qw.device, need, "window")
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel() * ws.element_size()
    p.status = status_word(qw.device).data_ptr()
    abi.check(abi.lib().omnikv_score_window(C.byref(p), _stream()), "omnikv_score_window")
    _count(3)  # pass 1, statistics merge, pass 2
    return score_out if planes_out is None else planes_out


def prefill_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, q_pos0: int = 0,
                 scale: Optional[float] = None, out: Optional[torch.Tensor] = None, variant: int = 0) -> torch.Tensor:
    """``omnikv_prefill_attn``: causal attention of a block of prompt queries.  q ``[B,H,Sq,d]``, k and v
    ``[B,KVH,Skv,d]`` with ``Skv >= q_pos0 + Sq`` (any strides that are multiples of 8 elements, rows contiguous),
    16-bit.  Query ``i`` sees keys ``j <= q_pos0 + i``.  Returns ``[B, Sq, H, d]``."""
    _need_cuda(q, k, v, out)
    B, H, Sq, d = q.shape
    KVH, Skv = k.shape[1], k.shape[2]
    if q.stride(3) != 1 or k.stride(3) != 1 or v.stride(3) != 1 or k.shape != v.shape or q.dtype != k.dtype:
        raise abi.OmniKVError("prefill_attn: rows of q, k, v must be contiguous and k, v of one shape and dtype")
    if out is None:
        out = torch.empty(B, Sq, H, d, dtype=q.dtype, device=q.device)
    p = abi.PrefillParams()
    p.dtype = _DT[q.dtype]
    p.B, p.H, p.KVH, p.head_dim = B, H, KVH, d
    p.Sq, p.Skv, p.q_pos0 = Sq, Skv, int(q_pos0)
    p.scale = float(scale if scale is not None else 1.0 / math.sqrt(d))
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    p.q_stride_b, p.q_stride_h, p.q_stride_row = q.stride(0), q.stride(1), q.stride(2)
    p.k_stride_b, p.k_stride_h, p.k_stride_row = k.stride(0), k.stride(1), k.stride(2)
    p.v_stride_b, p.v_stride_h, p.v_stride_row = v.stride(0), v.stride(1), v.stride(2)
    p.o_stride_b, p.o_stride_row, p.o_stride_h = out.stride(0), out.stride(1), out.stride(2)
    p.status = status_word(q.device).data_ptr()
    p.variant = int(variant)  # 0: two query tiles per CTA (default), 1: the one-tile kernel
    abi.check(abi.lib().omnikv_prefill_attn(C.byref(p), _stream()), "omnikv_prefill_attn")
    _count(1)
    return out


_EPI = {"store": abi.EPI_STORE, "store_f32": abi.EPI_STORE_F32, "residual": abi.EPI_RESIDUAL, "swiglu": abi.EPI_SWIGLU}


def batched_linear(x: torch.Tensor, w: torch.Tensor, *, epilogue: str = "store", norm_w: Optional[torch.Tensor] = None,
                   eps: float = 1e-5, residual: Optional[torch.Tensor] = None,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``omnikv_batched_linear``: x ``[n_tokens <= 16, K]`` times w ``[rows, K]`` transposed as a weight stream on
    tcgen05, with an optional RMSNorm of x in front and the epilogue ``store`` | ``store_f32`` | ``residual`` (adds
    ``residual``; ``out`` may be the same tensor) | ``swiglu`` (w = gate rows then up rows; returns
    ``[n_tokens, rows / 2]``)."""
    _need_cuda(x, w, norm_w, residual, out)
    n, K = x.shape
    rows = w.shape[0]
    if x.stride(1) != 1 or w.stride(1) != 1 or w.shape[1] != K or w.dtype != x.dtype:
        raise abi.OmniKVError("batched_linear: x [n, K] and w [rows, K] need contiguous rows and one dtype")
    epi = _EPI[epilogue]
    cols = rows // 2 if epilogue == "swiglu" else rows
    if out is None:
        out = torch.empty(n, cols, dtype=torch.float32 if epilogue == "store_f32" else x.dtype, device=x.device)
    p = abi.BatchedLinearParams()
    p.dtype, p.n_tokens, p.w_rows, p.K = _DT[x.dtype], n, rows, K
    p.w, p.w_stride_row, p.x, p.x_stride_tok = w.data_ptr(), w.stride(0), x.data_ptr(), x.stride(0)
    p.norm_w, p.eps, p.epilogue = _ptr(norm_w), float(eps), epi
    if residual is not None:
        p.residual, p.residual_stride_tok = residual.data_ptr(), residual.stride(0)
    p.out, p.out_stride_tok = out.data_ptr(), out.stride(0)
    need = abi.lib().omnikv_batched_linear_workspace_bytes(n, rows, K, epi)
    ws = workspace(x.device, need, "batched_linear")
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel() * ws.element_size()
    p.status = status_word(x.device).data_ptr()
    abi.check(abi.lib().omnikv_batched_linear(C.byref(p), _stream()), "omnikv_batched_linear")
    _count(1)
    return out


def window_fold(planes: torch.Tensor, consider_len: torch.Tensor, selector: str, *, max_len: int,
                score_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need_cuda(planes, consider_len, score_out)
    B, W, stride = planes.shape
    if score_out is None:
        score_out = torch.empty(B, stride, dtype=torch.float32, device=planes.device)
    abi.check(abi.lib().omnikv_window_fold(planes.data_ptr(), score_out.data_ptr(), B, W, planes.stride(1),
                                           consider_len.data_ptr(), int(max_len), _SEL[selector], _stream()),
              "omnikv_window_fold")
    _count(1)
    return score_out


def kv_append(k_new: torch.Tensor, v_new: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              pos: torch.Tensor) -> None:
    """Write k_new, v_new ``[B,KVH,d]`` at row ``pos[b]`` (int32, device) of the caches ``[B,KVH,rows,d]``."""
    _need_cuda(k_new, v_new, k_cache, v_cache, pos)
    B, KVH, d = k_new.shape
    if k_new.stride() != v_new.stride() or k_new.stride(2) != 1 or _kv_strides(k_cache) != _kv_strides(v_cache):
        raise abi.OmniKVError("kv_append: k/v layouts must match")
    sb, sh, sr = _kv_strides(k_cache)
    abi.check(abi.lib().omnikv_kv_append(_DT[k_new.dtype], k_new.data_ptr(), v_new.data_ptr(), k_cache.data_ptr(),
                                         v_cache.data_ptr(), B, KVH, d, k_new.stride(0), k_new.stride(1), sb, sh, sr,
                                         pos.data_ptr(), _stream()), "omnikv_kv_append")
    _count(1)


def tp_allreduce_sum(x: torch.Tensor, exchange) -> None:
    """``omnikv_tp_allreduce_sum``: in-place SUM of the contiguous tensor ``x`` over the ranks of ``exchange`` (an
    ``abi.TpExchange`` from ``parallel.PeerExchange.at(seq)``)."""
    _need_cuda(x)
    if not x.is_contiguous():
        raise abi.OmniKVError("tp_allreduce_sum: contiguous tensor expected")
    abi.check(abi.lib().omnikv_tp_allreduce_sum(_DT[x.dtype], x.data_ptr(), x.numel(), _xref(exchange),
                                                status_word(x.device).data_ptr(), _stream()), "omnikv_tp_allreduce_sum")
    _count(1)


def tp_allreduce_max(x: torch.Tensor, exchange) -> None:
    """``omnikv_tp_allreduce_max``: in-place element-wise MAX of the contiguous fp32 tensor ``x`` over the ranks."""
    _need_cuda(x)
    if not x.is_contiguous() or x.dtype != torch.float32:
        raise abi.OmniKVError("tp_allreduce_max: contiguous fp32 tensor expected")
    abi.check(abi.lib().omnikv_tp_allreduce_max(x.data_ptr(), x.numel(), _xref(exchange),
                                                status_word(x.device).data_ptr(), _stream()), "omnikv_tp_allreduce_max")
    _count(1)


def tp_allgather(x: torch.Tensor, exchange, world: int) -> torch.Tensor:
    """``omnikv_tp_allgather``: the ranks' contiguous tensors ``x`` one behind the other, ``[world, x.numel()]``."""
    _need_cuda(x)
    if not x.is_contiguous():
        raise abi.OmniKVError("tp_allgather: contiguous tensor expected")
    out = torch.empty(world, x.numel(), dtype=x.dtype, device=x.device)
    abi.check(abi.lib().omnikv_tp_allgather(_DT[x.dtype], x.data_ptr(), x.numel(), out.data_ptr(), _xref(exchange),
                                            status_word(x.device).data_ptr(), _stream()), "omnikv_tp_allgather")
    _count(1)
    return out


def rope_append(qkv: torch.Tensor, H: int, KVH: int, inv_freq: torch.Tensor, rope_pos: torch.Tensor,
                q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cache_pos: torch.Tensor) -> None:
    """``omnikv_rope_append``.  qkv ``[B, (H+2KVH)*128]`` (rows contiguous); q_out ``[B, H, 128]``; caches
    ``[B, KVH, rows, 128]``; rope_pos, cache_pos int32 ``[B]`` on the device; inv_freq fp32 ``[64]``."""
    _need_cuda(qkv, inv_freq, rope_pos, q_out, k_cache, v_cache, cache_pos)
    B = qkv.shape[0]
    if qkv.dim() != 2 or qkv.stride(1) != 1 or qkv.shape[1] != (H + 2 * KVH) * 128:
        raise abi.OmniKVError("rope_append: qkv must be [B, (H+2KVH)*128] with contiguous rows")
    if q_out.shape != (B, H, 128) or q_out.stride(2) != 1 or q_out.stride(1) != 128 or q_out.dtype != qkv.dtype:
        raise abi.OmniKVError("rope_append: q_out must be [B, H, 128] with contiguous heads")
    if _kv_strides(k_cache) != _kv_strides(v_cache) or k_cache.dtype != qkv.dtype:
        raise abi.OmniKVError("rope_append: k/v cache layouts must match")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != 64 or rope_pos.dtype != torch.int32 or cache_pos.dtype != torch.int32:
        raise abi.OmniKVError("rope_append: inv_freq fp32 [64], positions int32")
    sb, sh, sr = _kv_strides(k_cache)
    abi.check(abi.lib().omnikv_rope_append(_DT[qkv.dtype], qkv.data_ptr(), qkv.stride(0), B, H, KVH, 128,
                                           inv_freq.data_ptr(), rope_pos.data_ptr(), q_out.data_ptr(), q_out.stride(0),
                                           k_cache.data_ptr(), v_cache.data_ptr(), sb, sh, sr, cache_pos.data_ptr(),
                                           _stream()), "omnikv_rope_append")
    _count(1)


def add_rms_norm(h: torch.Tensor, delta: Optional[torch.Tensor], norm_w: torch.Tensor, eps: float,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``omnikv_add_rms_norm``.  h ``[n, hidden]`` (updated IN PLACE: ``h += delta`` when delta is given); returns
    ``RMSNorm(h) * norm_w``."""
    _need_cuda(h, delta, norm_w, out)
    if h.dim() != 2 or h.stride(1) != 1 or (delta is not None and (delta.shape != h.shape or delta.stride(1) != 1)):
        raise abi.OmniKVError("add_rms_norm: h and delta must be [n, hidden] with contiguous rows")
    if out is None:
        out = torch.empty_like(h, memory_format=torch.contiguous_format)
    abi.check(abi.lib().omnikv_add_rms_norm(_DT[h.dtype], h.data_ptr(), h.stride(0), _ptr(delta),
                                            0 if delta is None else delta.stride(0), norm_w.data_ptr(), float(eps),
                                            out.data_ptr(), out.stride(0), h.shape[0], h.shape[1], _stream()),
              "omnikv_add_rms_norm")
    _count(1)
    return out


def rope_window(qlin: torch.Tensor, H: int, inv_freq: torch.Tensor, rope_pos: torch.Tensor) -> torch.Tensor:
    """``omnikv_rope_window``.  qlin ``[B, W, H*128]`` (rows contiguous) -> rotated queries ``[B, H, W, 128]``, every
    window slot rotated at ``rope_pos[b]`` (int32, device)."""
    _need_cuda(qlin, inv_freq, rope_pos)
    B, W, n = qlin.shape
    if qlin.stride(2) != 1 or n != H * 128:
        raise abi.OmniKVError("rope_window: qlin must be [B, W, H*128] with contiguous rows")
    out = torch.empty(B, H, W, 128, dtype=qlin.dtype, device=qlin.device)
    abi.check(abi.lib().omnikv_rope_window(_DT[qlin.dtype], qlin.data_ptr(), qlin.stride(0), qlin.stride(1), B, W, H, 128,
                                           inv_freq.data_ptr(), rope_pos.data_ptr(), out.data_ptr(), _stream()),
              "omnikv_rope_window")
    _count(1)
    return out


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``omnikv_silu_mul``.  gate_up ``[B, 2*inter]`` (rows contiguous) -> ``silu(gate) * up`` ``[B, inter]``."""
    _need_cuda(gate_up, out)
    if gate_up.dim() != 2 or gate_up.stride(1) != 1 or gate_up.shape[1] % 2:
        raise abi.OmniKVError("silu_mul: gate_up must be [B, 2*inter] with contiguous rows")
    B, inter = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty(B, inter, dtype=gate_up.dtype, device=gate_up.device)
    abi.check(abi.lib().omnikv_silu_mul(_DT[gate_up.dtype], gate_up.data_ptr(), gate_up.stride(0), out.data_ptr(),
                                        out.stride(0), B, inter, _stream()), "omnikv_silu_mul")
    _count(1)
    return out


def offload_gather(host_kv: torch.Tensor, idx: torch.Tensor, n_idx: torch.Tensor, staged: torch.Tensor,
                   *, n_ctas: Optional[int] = None) -> None:
    """``omnikv_offload_gather``.  host_kv: PINNED CPU tensor ``[tokens, layers, 2, KVH, d]``;
    idx int32 device ``[>= n]``; n_idx int32 device ``[1]``; staged device ``[layers, 2, KVH, cap, d]``."""
    if host_kv.is_cuda or not host_kv.is_pinned():
        raise abi.OmniKVError("host_kv must be a pinned CPU tensor")
    _need_cuda(idx, n_idx, staged)
    tokens, layers, two, KVH, d = host_kv.shape
    if two != 2 or not host_kv.is_contiguous() or not staged.is_contiguous():
        raise abi.OmniKVError("offload_gather: bad layout")
    cap = staged.shape[3]
    dev_ptr = host_device_pointer(host_kv)
    if n_ctas is None:
        n_ctas = 2 * sm_count(staged.device)
    abi.check(abi.lib().omnikv_offload_gather(dev_ptr, host_kv.stride(0) * host_kv.element_size(), layers, KVH, d,
                                              host_kv.element_size(), idx.data_ptr(), n_idx.data_ptr(), cap,
                                              staged.data_ptr(), int(n_ctas), _stream()), "omnikv_offload_gather")
    _count(1)


def idx_commit(new_idx: torch.Tensor, new_count: torch.Tensor, live_idx: torch.Tensor, live_count: torch.Tensor,
               skip_threshold: float, applied: torch.Tensor, gather_n: Optional[torch.Tensor] = None,
               overlap: Optional[torch.Tensor] = None) -> None:
    """``omnikv_idx_commit``: the lazy re-gather rule.  int32 device tensors: new_idx / live_idx ``[B, cap]``
    ascending, new_count / live_count / applied / gather_n / overlap ``[B]``."""
    _need_cuda(new_idx, new_count, live_idx, live_count, applied, gather_n, overlap)
    for t in (new_idx, new_count, live_idx, live_count, applied, gather_n, overlap):
        if t is not None and t.dtype != torch.int32:
            raise abi.OmniKVError("idx_commit: int32 tensors expected")
    if new_idx.dim() != 2 or live_idx.dim() != 2 or new_idx.stride(1) != 1 or live_idx.stride(1) != 1:
        raise abi.OmniKVError("idx_commit: index lists must be [B, capacity] with contiguous rows")
    B, cap = new_idx.shape[0], min(new_idx.shape[1], live_idx.shape[1])
    abi.check(abi.lib().omnikv_idx_commit(new_idx.data_ptr(), new_idx.stride(0), new_count.data_ptr(),
                                          live_idx.data_ptr(), live_idx.stride(0), live_count.data_ptr(), B, cap,
                                          float(skip_threshold), applied.data_ptr(), _ptr(gather_n), _ptr(overlap),
                                          _stream()), "omnikv_idx_commit")
    _count(1)


def host_device_pointer(t: torch.Tensor) -> int:
    """Device-visible address of a pinned host tensor.  With unified virtual addressing (every
    64-bit Linux CUDA process) a page-locked allocation made by the CUDA runtime is mapped into
    the device address space at the same address, so the host pointer is the device pointer."""
    if t.is_cuda or not t.is_pinned():
        raise abi.OmniKVError("expected a pinned CPU tensor")
    return t.data_ptr()


# ------------------------------------------------------------------------------------------------
# batch-1 decode step: fused weight-streaming kernels
# ------------------------------------------------------------------------------------------------
FUSED_K = (512, 1024, 1792, 2048, 3584, 4096, 7168, 8192, 14336)
_status = {}


_sched = {}


def sched_words(device) -> torch.Tensor:
    """Four zeroed int32 per device: the dynamic-tail counters of ``omnikv_decode_gate_up`` (self-resetting)."""
    key = _dev_index(device)
    if key not in _sched:
        _sched[key] = torch.zeros(4, dtype=torch.int32, device=device)
    return _sched[key]


def status_word(device) -> torch.Tensor:
    """The device int32 the kernels report bounded-wait failures into (stays 0)."""
    key = _dev_index(device)
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device) -> None:
    """Synchronises and raises if a kernel recorded that a bounded wait ran out."""
    code = int(status_word(device).item())
    if code:
        status_word(device).zero_()
        what = {1: "a weight copy's ring slot (producer)", 2: "a weight copy (consumer)", 3: "the grid barrier",
                4: "another rank's exchange flag", 5: "a K/V tile copy"}.get(code, "an unknown wait")
        raise abi.OmniKVError(f"a decode kernel gave up waiting for {what} (status {code}); its results are incomplete")


def rows_per_stage(K: int) -> int:
    return 8 if K <= 4096 else (4 if K <= 8192 else 2)


def fused_decode_supported(dtype, hidden: int, inter: int, n_q_rows: int, vocab_rows: int) -> bool:
    """Whether the fused decode kernels cover these (local) shapes; otherwise callers use the torch ops."""
    return (dtype in (torch.bfloat16, torch.float16) and hidden in FUSED_K and inter in FUSED_K
            and n_q_rows in FUSED_K and hidden % rows_per_stage(inter) == 0 and hidden % rows_per_stage(n_q_rows) == 0
            and inter % (rows_per_stage(hidden) // 2) == 0 and vocab_rows % rows_per_stage(hidden) == 0)


def _xref(x):
    return None if x is None else C.byref(x)


def decode_qkv(h, norm_w, eps, w_qkv, H, KVH, inv_freq, rope_pos, q_out, k_cache_seq, v_cache_seq, cache_pos,
               tp_in=None, h_out=None):
    """h ``[hidden]``; w_qkv ``[(H+2KVH)*128, hidden]``; k/v_cache_seq: one sequence's ``[KVH, rows, 128]``.
    ``tp_in`` (an ``abi.TpExchange``): h is first completed with every rank's partial sums of that exchange and
    the completed vector is stored to ``h_out`` -- a DIFFERENT buffer than ``h``, which other CTAs still read."""
    abi.check(abi.lib().omnikv_decode_qkv(_DT[h.dtype], h.data_ptr(), norm_w.data_ptr(), float(eps), w_qkv.data_ptr(),
                                          w_qkv.shape[1], H, KVH, 128, inv_freq.data_ptr(), rope_pos.data_ptr(),
                                          q_out.data_ptr(), k_cache_seq.data_ptr(), v_cache_seq.data_ptr(),
                                          k_cache_seq.stride(0), k_cache_seq.stride(1), cache_pos.data_ptr(),
                                          _xref(tp_in), _ptr(h_out),
                                          status_word(h.device).data_ptr(), _stream()), "omnikv_decode_qkv")
    _count(1)


def decode_gemv_residual(w, x, resid, out, tp_out=None):
    """out ``[N]`` = (resid or 0) + w ``[N,K]`` @ x ``[K]``; ``out`` may be ``resid``.  With ``tp_out`` the fp32
    partial sums go to every rank's exchange buffer instead and ``resid`` / ``out`` are not used."""
    abi.check(abi.lib().omnikv_decode_gemv_residual(_DT[x.dtype], w.data_ptr(), w.shape[0], w.shape[1], x.data_ptr(),
                                                    _ptr(resid), _ptr(out), _xref(tp_out),
                                                    status_word(x.device).data_ptr(), _stream()),
              "omnikv_decode_gemv_residual")
    _count(1)


def decode_gate_up(h, norm_w, eps, w_gate_up, act_out, tp_in=None, h_out=None):
    abi.check(abi.lib().omnikv_decode_gate_up(_DT[h.dtype], h.data_ptr(), norm_w.data_ptr(), float(eps),
                                              w_gate_up.data_ptr(), w_gate_up.shape[1], w_gate_up.shape[0] // 2,
                                              act_out.data_ptr(), _xref(tp_in), _ptr(h_out),
                                              sched_words(h.device).data_ptr(), status_word(h.device).data_ptr(),
                                              _stream()), "omnikv_decode_gate_up")
    _count(1)


def decode_logits(h, norm_w, eps, w_head, row_offset, logits, best, token_out=None, tp_in=None):
    abi.check(abi.lib().omnikv_decode_logits(_DT[h.dtype], h.data_ptr(), norm_w.data_ptr(), float(eps), w_head.data_ptr(),
                                             w_head.shape[1], w_head.shape[0], int(row_offset), logits.data_ptr(),
                                             best.data_ptr(), _ptr(token_out), _xref(tp_in),
                                             status_word(h.device).data_ptr(), _stream()), "omnikv_decode_logits")
    _count(2 if token_out is not None else 1)


_grid_sync = {}


def grid_sync_words(device) -> torch.Tensor:
    """Two zeroed uint32 words per device for the grid-wide barrier of ``omnikv_decode_chain``."""
    key = _dev_index(device)
    if key not in _grid_sync:
        _grid_sync[key] = torch.zeros(2, dtype=torch.int32, device=device)
    return _grid_sync[key]


def decode_chain_supported(dtype, hidden: int, inter: int, H: int) -> bool:
    return dtype in _DT and bool(abi.lib().omnikv_decode_chain_supported(_DT[dtype], hidden, inter, H))


def decode_chain(h, *, eps, H, KVH, inter, w_o=None, attn_out=None, post_norm_w=None, w_gate_up=None, w_down=None,
                 act=None, in_norm_w=None, w_qkv=None, inv_freq=None, rope_pos=None, q_out=None, k_cache_seq=None,
                 v_cache_seq=None, cache_pos=None, final_norm_w=None, w_head=None, logits=None, best=None,
                 token_out=None, chunk_counters=None, next_w=None):
    """``omnikv_decode_chain``: the weight-streaming phases between two attention calls in one cooperative
    launch.  h ``[hidden]`` is updated in place."""
    p = abi.ChainParams()
    p.dtype, p.hidden, p.inter, p.H, p.KVH, p.eps = _DT[h.dtype], h.numel(), int(inter), int(H), int(KVH), float(eps)
    p.h = h.data_ptr()
    p.w_o, p.attn_out = _ptr(w_o), _ptr(attn_out)
    p.post_norm_w, p.w_gate_up, p.w_down, p.act_scratch = _ptr(post_norm_w), _ptr(w_gate_up), _ptr(w_down), _ptr(act)
    p.in_norm_w, p.w_qkv, p.inv_freq, p.rope_pos, p.q_out = _ptr(in_norm_w), _ptr(w_qkv), _ptr(inv_freq), _ptr(rope_pos), _ptr(q_out)
    if k_cache_seq is not None:
        p.k_cache_seq, p.v_cache_seq = k_cache_seq.data_ptr(), v_cache_seq.data_ptr()
        p.kv_stride_h, p.kv_stride_row = k_cache_seq.stride(0), k_cache_seq.stride(1)
    p.cache_pos = _ptr(cache_pos)
    p.final_norm_w, p.w_head = _ptr(final_norm_w), _ptr(w_head)
    p.vocab_rows = 0 if w_head is None else w_head.shape[0]
    p.logits, p.best_scratch, p.token_out = _ptr(logits), _ptr(best), _ptr(token_out)
    p.grid_sync, p.status = grid_sync_words(h.device).data_ptr(), status_word(h.device).data_ptr()
    p.chunk_counters = _ptr(chunk_counters)
    if next_w is not None:
        p.next_w, p.next_w_bytes = next_w.data_ptr(), next_w.numel() * next_w.element_size()
    abi.check(abi.lib().omnikv_decode_chain(C.byref(p), _stream()), "omnikv_decode_chain")
    _count(2 if (w_head is not None and token_out is not None) else 1)


def decode_attn_no_alloc(q, k, v, len_a, out, *, n_splits, idx=None, k_tail=None, v_tail=None, tail_start=None,
                         tail_len=None, scale=None) -> torch.Tensor:
    """``omnikv_decode_attn_no_alloc``: decode attention that touches no allocator -- not PyTorch's, not
    CUDA's.  For callers that only hold tensors (a plugin inside a runtime that owns all device memory, a
    process with a fixed memory budget, a loop that must never reach ``cudaMalloc``): the split partials go to a 4 MiB array built
    into the library instead of a workspace tensor, and ``out`` ``[B,H,d]`` must be passed in.

    ``B * H * n_splits`` may not exceed 8034 (the array's size); beyond that an ``OmniKVError`` is raised and
    nothing is launched.  All calls on a device share that array: keep them on one stream (calls that overlap
    on the GPU race on it), and make the first call on a device outside stream capture."""
    _need_cuda(q, k, v, len_a, out, idx, k_tail, v_tail)
    B, H, d = q.shape
    need = abi.lib().omnikv_decode_attn_workspace_bytes(B, H, int(n_splits))
    if need > abi.NO_ALLOC_SCRATCH_BYTES:
        raise abi.OmniKVError(
            f"omnikv_decode_attn_no_alloc: B*H*n_splits = {B * H * int(n_splits)} needs {need} bytes of scratch, the "
            f"library's built-in scratch holds {abi.NO_ALLOC_SCRATCH_BYTES}; use fewer splits or omnikv_decode_attn")
    p = abi.AttnParams()
    p.dtype, p.B, p.H, p.KVH, p.head_dim = _DT[q.dtype], B, H, k.shape[1], d
    p.scale = float(scale if scale is not None else 1.0 / math.sqrt(d))
    p.q, p.q_stride_b, p.q_stride_h, p.out = q.data_ptr(), q.stride(0), q.stride(1), out.data_ptr()
    p.kA, p.vA = k.data_ptr(), v.data_ptr()
    p.a_stride_b, p.a_stride_h, p.a_stride_row = _kv_strides(k)
    if idx is not None:
        p.idxA, p.idx_stride = idx.data_ptr(), idx.stride(0)
    p.lenA = len_a.data_ptr()
    if tail_len is not None:
        p.kB, p.vB = k_tail.data_ptr(), v_tail.data_ptr()
        p.b_stride_b, p.b_stride_h, p.b_stride_row = _kv_strides(k_tail)
        p.startB, p.lenB = tail_start.data_ptr(), tail_len.data_ptr()
    p.n_splits = int(n_splits)
    abi.check(abi.lib().omnikv_decode_attn_no_alloc(C.byref(p), _stream()), "omnikv_decode_attn_no_alloc")
    return out
