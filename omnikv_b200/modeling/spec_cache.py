"""KV caches of the OmniKV decode path: ``OmniKVMultiStageCache`` (``cache_cls = "multi"``),
``WOPackCache`` (``"without_pack"``) and ``OmniKVLazyCache`` (``"lazy"``), mirroring
modeling/spec_cache.py:253-557 of the reference.

Same public surface -- ``from_dynamic_cache``, ``update``, ``set_idx_on_gpu``, ``stage``,
``layer_state``, ``key_cache`` / ``value_cache``, ``part_key`` / ``part_value``, ``tail_k`` /
``tail_v``, ``_seen_tokens`` -- over a different memory design:

* every layer's K/V lives in ONE preallocated buffer ``[B, KVH, capacity, d]``; the current
  token's row is written in place by ``omnikv_kv_append`` (the reference re-copies the whole cache
  with ``torch.cat`` every step, :363-369);
* lengths are int32 DEVICE arrays, so a decode step captured in a CUDA graph can be replayed;
* a sparse layer never materialises ``cat([part_key, tail_k])`` (:349-356): its attention kernel
  reads the selected prompt rows through the index list and the tail rows ``[P, P + t)`` of the
  same buffer (``attend``);
* with ``real_offload`` the sparse layers' prompt KV sits in pinned host memory, token-major and
  packed per filter group ``[P, layers, K|V, KVH, d]``; ``set_idx_on_gpu`` launches ONE gather
  kernel for the whole group on a side stream (overlapping the wait layers) that reads the
  selected tokens over the host link into staged device rows.  ``WOPackCache`` keeps one host
  buffer per layer and gathers inside each sparse layer, without overlap (:426-429, :477-483).

Batches: the reference flattens the batch of the index list (:292), which is only meaningful at
batch 1; here every sequence has its own index list, lengths and tail.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch


def full_attn_layers_of(do_select_layers: Sequence[int], num_hidden_layers: int) -> List[int]:
    """Layers before the first filter layer, the filter layers, and the sentinel (modeling/omnikv.py:322-331)."""
    sel = list(do_select_layers)
    return list(range(0, sel[0])) + sel + [num_hidden_layers]


def make_layer_state(full_attn_layers, num_hidden_layers, num_wait_layers) -> Dict[int, Tuple[bool, int, int]]:
    """``layer -> (is_sparse, group_start, group_end)`` as modeling/spec_cache.py:272-281 derives it:
    a group starts at every entry of ``full_attn_layers``; the group's first ``1 + num_wait_layers``
    layers attend densely, the rest are sparse (and offloadable)."""
    marks = sorted(set(int(x) for x in full_attn_layers))
    state: Dict[int, Tuple[bool, int, int]] = {}
    for pos, left in enumerate(marks):
        if left >= num_hidden_layers:
            continue
        right = num_hidden_layers
        for cand in marks[pos + 1:]:
            if left < cand < num_hidden_layers:
                right = cand
                break
        first_sparse = min(right, left + num_wait_layers + 1)
        for layer in range(left, right):
            state[layer] = (layer >= first_sparse, left, right)
    return state


class OmniKVMultiStageCache:
    pack_gather = True  # one gather per filter group on a side stream

    def __init__(self, full_attn_layers: List, num_hidden_layers, num_wait_load_layers=2, real_offload=True):
        self.stage = "prefill"
        self.full_attn_layers = list(full_attn_layers)
        self.num_hidden_layers = num_hidden_layers
        self.num_wait_layers = num_wait_load_layers
        self.layer_state = make_layer_state(full_attn_layers, num_hidden_layers, num_wait_load_layers)
        self.need_cat_layers: List[int] = []
        self.device = "cpu" if real_offload else None  # the reference's attribute: where sparse prompt KV lives
        self.key_cache: List[torch.Tensor] = []
        self.value_cache: List[torch.Tensor] = []
        self.part_key: Dict[int, torch.Tensor] = {}
        self.part_value: Dict[int, torch.Tensor] = {}
        self.tail_k: Dict[int, torch.Tensor] = {}
        self.tail_v: Dict[int, torch.Tensor] = {}
        self._seen_tokens = 0
        # ---- B200-side state -------------------------------------------------------------------
        self.reserve = 1024            # rows kept free behind the prompt for decode-time tokens
        self.real_offload = bool(real_offload)
        self.groups: Dict[int, List[int]] = {}   # filter layer -> its sparse layers
        for layer, (sparse, left, right) in self.layer_state.items():
            if sparse:
                self.groups.setdefault(left, []).append(layer)
        for v in self.groups.values():
            v.sort()
        self._k: Dict[int, torch.Tensor] = {}    # device buffers [B, KVH, cap, d] (offloaded layers: the tail only)
        self._v: Dict[int, torch.Tensor] = {}
        self._host: Dict[int, torch.Tensor] = {}    # pack: filter layer -> pinned [P, nl, 2, KVH, d]; no pack: layer -> [P,1,2,KVH,d]
        self._staged: Dict[int, torch.Tensor] = {}  # same keys -> device [nl, 2, KVH, kcap, d]
        self._idx: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}  # filter layer -> (idx int32 [B,kcap], count int32 [B])
        self._gather_done: Dict[int, torch.cuda.Event] = {}
        self.fused_bufs = None                       # scratch of the fused batch-1 decode kernels (q, o, act, logits)
        self.sel_state: Dict[int, Any] = {}         # filter layer -> device-side selection state (k, ranges, index buffers)
        self._side_stream: Optional[torch.cuda.Stream] = None
        self.prefill_len: Optional[int] = None      # host copy (max over the batch)
        self.prefill_len_dev: Optional[torch.Tensor] = None  # int32 [B]
        self.cur_len_dev: Optional[torch.Tensor] = None      # int32 [B]: rows valid after this step's append
        self.tail_len_dev: Optional[torch.Tensor] = None     # int32 [B]: decode-time rows
        self.pos_dev: Optional[torch.Tensor] = None          # int32 [B]: row this step's token is written to
        self.tail_pos_dev: Optional[torch.Tensor] = None     # int32 [B]: the same inside a tail-only buffer
        self.zero_dev: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------------------------------
    @staticmethod
    def from_dynamic_cache(cache, full_attn_layers: List, num_hidden_layers, num_wait_load_layers=2,
                           real_offload=True):
        """modeling/spec_cache.py:371-385.  ``cache`` may be None, an object with empty ``key_cache`` /
        ``value_cache`` lists (the usual case: the prefill then runs through this cache), or one that already holds
        a prompt -- CUDA tensors ``[B, KVH, P, d]`` for every layer: they are taken over as if that prompt had just
        been prefilled (copied into the preallocated layout; with ``real_offload`` the sparse layers' rows go to
        pinned host memory), and decoding continues from there."""
        c = OmniKVMultiStageCache(full_attn_layers, num_hidden_layers, num_wait_load_layers, real_offload)
        c._adopt(cache)
        return c

    def _adopt(self, cache):
        if cache is None:
            return
        keys = list(getattr(cache, "key_cache", None) or [])
        if not keys:
            self._seen_tokens = int(getattr(cache, "_seen_tokens", 0))
            return
        vals = list(cache.value_cache)
        if len(keys) != self.num_hidden_layers or len(vals) != self.num_hidden_layers:
            raise ValueError(f"a cache to take over must hold all {self.num_hidden_layers} layers, got {len(keys)}")
        self.stage = "prefill"
        for i, (k, v) in enumerate(zip(keys, vals)):
            if not (k.is_cuda and v.is_cuda and k.dim() == 4 and k.shape == v.shape):
                raise ValueError("a cache to take over must hold CUDA tensors [B, KVH, P, d] per layer")
            self._store_prefill(k, v, i)
        if self.real_offload:
            torch.cuda.current_stream().synchronize()  # the host copies of the sparse layers have landed

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._seen_tokens

    def is_sparse(self, layer_idx: int) -> bool:
        return self.layer_state[layer_idx][0]

    def is_offloaded(self, layer_idx: int) -> bool:
        return self.real_offload and self.layer_state[layer_idx][0]

    def _host_key(self, layer_idx: int) -> Tuple[int, int]:
        """(key of the host/staged buffer, slot of the layer inside it)."""
        if self.pack_gather:
            left = self.layer_state[layer_idx][1]
            return left, self.groups[left].index(layer_idx)
        return layer_idx, 0

    # ------------------------------------------------------------------------------------------
    # allocation
    # ------------------------------------------------------------------------------------------
    def _init_meta(self, B: int, prefill_lens: Sequence[int], device) -> None:
        self.prefill_len = int(max(prefill_lens))
        i32 = dict(dtype=torch.int32, device=device)
        self.prefill_len_dev = torch.tensor(list(prefill_lens), **i32)
        # the four counters a decode step advances live in ONE tensor, so one in-place add moves them all
        self._step_counters = torch.stack([self.prefill_len_dev, torch.zeros(B, **i32), self.prefill_len_dev - 1,
                                           torch.full((B,), -1, **i32)]).contiguous()
        self.cur_len_dev, self.tail_len_dev, self.pos_dev, self.tail_pos_dev = self._step_counters.unbind(0)
        self.zero_dev = torch.zeros(B, **i32)

    def _alloc_layer(self, layer_idx: int, B: int, KVH: int, d: int, dtype, device) -> None:
        P = self.prefill_len
        if self.is_offloaded(layer_idx):
            if B != 1:
                raise NotImplementedError("real_offload keeps one sequence's prompt KV on the host (batch 1)")
            key, slot = self._host_key(layer_idx)
            if key not in self._host:
                nl = len(self.groups[key]) if self.pack_gather else 1
                self._host[key] = torch.empty(P, nl, 2, KVH, d, dtype=dtype, pin_memory=True)
            self._k[layer_idx] = torch.zeros(B, KVH, self.reserve, d, dtype=dtype, device=device)
            self._v[layer_idx] = torch.zeros(B, KVH, self.reserve, d, dtype=dtype, device=device)
        else:
            self._k[layer_idx], self._v[layer_idx] = self._alloc_kv(layer_idx, B, KVH, P + self.reserve, d, dtype, device)
        while len(self.key_cache) <= layer_idx:
            self.key_cache.append(None)
            self.value_cache.append(None)
        if self.is_offloaded(layer_idx):
            key, slot = self._host_key(layer_idx)
            self.key_cache[layer_idx] = self._host[key][:, slot, 0].permute(1, 0, 2).unsqueeze(0)
            self.value_cache[layer_idx] = self._host[key][:, slot, 1].permute(1, 0, 2).unsqueeze(0)
        else:
            self.key_cache[layer_idx] = self._k[layer_idx]
            self.value_cache[layer_idx] = self._v[layer_idx]

    def _alloc_kv(self, layer_idx, B, KVH, cap, d, dtype, device):
        """K and V of a layer in ONE buffer, as ``[B, KVH, cap, d]`` views (rows stay 16-byte aligned and
        contiguous; the kernels take the strides).  The physical order follows how the layer reads it:

        * dense layers stream whole heads: ``[B, KVH, cap, K|V, d]`` -- a head's K and V rows interleaved, so a
          tile of 64 tokens is one contiguous 32 KB block;
        * sparse layers gather a few thousand scattered tokens: ``[B, cap, KVH, K|V, d]`` -- token-major, so all
          the K and V rows of a selected token (4 KB for 8 KV heads) sit together and a gather touches one DRAM
          page per token instead of sixteen (random 256-byte reads reach under half of the HBM bandwidth).
        """
        if self.is_sparse(layer_idx):
            kv = torch.zeros(B, cap, KVH, 2, d, dtype=dtype, device=device)
            return kv[:, :, :, 0, :].permute(0, 2, 1, 3), kv[:, :, :, 1, :].permute(0, 2, 1, 3)
        kv = torch.zeros(B, KVH, cap, 2, d, dtype=dtype, device=device)
        return kv[:, :, :, 0, :], kv[:, :, :, 1, :]

    def init_synthetic(self, B: int, KVH: int, d: int, prefill_lens: Sequence[int], dtype, device, seed: int = 0,
                       reserve: Optional[int] = None) -> "OmniKVMultiStageCache":
        """Fill the cache as a prefill of ``prefill_lens[b]`` tokens would have, with seeded N(0,1)
        rows (throughput runs: the decode step's work does not depend on the values)."""
        if reserve is not None:
            self.reserve = int(reserve)
        self._init_meta(B, prefill_lens, device)
        g = torch.Generator(device=device).manual_seed(seed)
        P = self.prefill_len
        for layer in range(self.num_hidden_layers):
            self._alloc_layer(layer, B, KVH, d, dtype, device)
            if self.is_offloaded(layer):
                key, slot = self._host_key(layer)
                step = 65536
                for s in range(0, P, step):
                    e = min(P, s + step)
                    blk = torch.randn(e - s, 2, KVH, d, generator=g, device=device, dtype=torch.float32).to(dtype)
                    self._host[key][s:e, slot].copy_(blk)
            else:
                for buf in (self._k[layer], self._v[layer]):
                    for b in range(B):
                        buf[b, :, :prefill_lens[b]].copy_(
                            torch.randn(KVH, prefill_lens[b], d, generator=g, device=device, dtype=torch.float32))
        self._seen_tokens = P
        self.stage = "decoding"
        return self

    # ------------------------------------------------------------------------------------------
    # reference API
    # ------------------------------------------------------------------------------------------
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[Dict[str, Any]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """modeling/spec_cache.py:308-369: store this call's rows and return the K, V the attention sees.

        Prefill (more than one new row): the rows are stored (sparse layers with ``real_offload``:
        in pinned host memory) and the fresh ``key_states, value_states`` are returned, so prefill
        attention is always full (:318-336).  Decode: the row is appended in place; dense layers
        return views of the cache, sparse layers return ``cat([selected rows, tail])`` built with
        torch ops -- a compatibility path for callers that run their own attention.  The layers of
        this package call ``append_kv`` + ``attend`` instead and never materialise that tensor.
        """
        B, KVH, n_new, d = key_states.shape
        if n_new > 1:
            self._store_prefill(key_states, value_states, layer_idx)
            return key_states, value_states
        if layer_idx == 0:
            self.begin_decode_step()
        self.append_kv(key_states[:, :, 0], value_states[:, :, 0], layer_idx)
        return self._compat_kv(layer_idx)

    def _store_prefill(self, key_states, value_states, layer_idx) -> None:
        B, KVH, P, d = key_states.shape
        if layer_idx == 0 or self.prefill_len_dev is None:
            self._init_meta(B, [P] * B, key_states.device)
            self._seen_tokens += P
        self._alloc_layer(layer_idx, B, KVH, d, key_states.dtype, key_states.device)
        if self.is_offloaded(layer_idx):
            key, slot = self._host_key(layer_idx)
            last = layer_idx == self.num_hidden_layers - 1  # the reference blocks on the last layer (:320-329)
            self._host[key][:, slot, 0].copy_(key_states[0].transpose(0, 1), non_blocking=not last)
            self._host[key][:, slot, 1].copy_(value_states[0].transpose(0, 1), non_blocking=not last)
        else:
            self._k[layer_idx][:, :, :P].copy_(key_states)
            self._v[layer_idx][:, :, :P].copy_(value_states)

    def begin_decode_step(self) -> None:
        """Advance the device-side counters by one token (graph-capturable).  Called once per decode
        step before layer 0 appends (the reference bumps ``_seen_tokens`` at layer 0, :315-316):
        ``update`` does it for layer 0; callers of ``append_kv`` do it themselves."""
        self.check_room(1)
        self._step_counters.add_(1)  # cur_len, tail_len, pos, tail_pos
        self._seen_tokens += 1

    def check_room(self, n_tokens: int) -> None:
        """Raise before a decode step would write past the preallocated rows (``reserve`` behind the prompt)."""
        if self.prefill_len is not None and self._seen_tokens + n_tokens > self.prefill_len + self.reserve:
            raise RuntimeError(
                f"KV cache is full: {self._seen_tokens} tokens held, room for {self.prefill_len + self.reserve}; "
                "set cache.reserve (rows kept free behind the prompt) before the prefill")

    def append_kv(self, k_new: torch.Tensor, v_new: torch.Tensor, layer_idx: int) -> None:
        """Write the current token's rows ``[B, KVH, d]`` in place (``omnikv_kv_append``)."""
        from .. import ops
        pos = self.tail_pos_dev if self.is_offloaded(layer_idx) else self.pos_dev
        ops.kv_append(k_new, v_new, self._k[layer_idx], self._v[layer_idx], pos)

    def write_target_batch(self, layer_idx: int):
        """(k buffer, v buffer, row index tensor) for the current token of every sequence: the layer's
        ``[B, KVH, rows, d]`` views and the int32 device positions (tail-relative for offloaded layers)."""
        pos = self.tail_pos_dev if self.is_offloaded(layer_idx) else self.pos_dev
        return self._k[layer_idx], self._v[layer_idx], pos

    def write_target(self, layer_idx: int):
        """(k rows, v rows, row index tensor) the current token of sequence 0 is written to: ``[KVH, rows, d]``
        views of the layer's buffer and the int32 device position (tail-relative for offloaded layers)."""
        pos = self.tail_pos_dev if self.is_offloaded(layer_idx) else self.pos_dev
        return self._k[layer_idx][0], self._v[layer_idx][0], pos

    def _compat_kv(self, layer_idx):
        n = self._seen_tokens
        P = self.prefill_len
        if not self.is_sparse(layer_idx):
            return self._k[layer_idx][:, :, :n], self._v[layer_idx][:, :, :n]
        left = self.layer_state[layer_idx][1]
        idx, count = self._idx[left]
        cnt = count.tolist()
        ks, vs = [], []
        for b in range(idx.shape[0]):
            sel = idx[b, :cnt[b]].long()
            if self.is_offloaded(layer_idx):
                pk = self.key_cache[layer_idx][b:b + 1].index_select(2, sel.cpu()).to(idx.device)
                pv = self.value_cache[layer_idx][b:b + 1].index_select(2, sel.cpu()).to(idx.device)
                tk, tv = self._k[layer_idx][b:b + 1, :, :n - P], self._v[layer_idx][b:b + 1, :, :n - P]
            else:
                pk = self._k[layer_idx][b:b + 1].index_select(2, sel)
                pv = self._v[layer_idx][b:b + 1].index_select(2, sel)
                tk, tv = self._k[layer_idx][b:b + 1, :, P:n], self._v[layer_idx][b:b + 1, :, P:n]
            ks.append(torch.cat([pk, tk], dim=2))
            vs.append(torch.cat([pv, tv], dim=2))
        self.part_key[layer_idx], self.part_value[layer_idx] = pk, pv
        self.tail_k[layer_idx], self.tail_v[layer_idx] = tk, tv
        return (ks[0], vs[0]) if len(ks) == 1 else (torch.cat(ks, 0), torch.cat(vs, 0))

    def set_idx_on_gpu(self, idx: torch.Tensor, sel_layer_idx: int) -> None:
        """modeling/spec_cache.py:290-306.  ``idx`` ``[B, k]`` ascending (int64 as the reference's
        selector returns it, or int32).  Every sparse layer of the group that ``sel_layer_idx`` opens
        uses this list until the next filter layer."""
        idx32 = idx.to(torch.int32).contiguous()
        count = torch.full((idx32.shape[0],), idx32.shape[1], dtype=torch.int32, device=idx32.device)
        self.set_idx_device(idx32, count, sel_layer_idx)

    def set_idx_device(self, idx32: torch.Tensor, count: torch.Tensor, sel_layer_idx: int) -> None:
        """Device-side form: ``idx32`` int32 ``[B, capacity]`` with ``count[b]`` valid entries (what
        ``omnikv_topk`` writes) -- no host synchronisation."""
        self._idx[sel_layer_idx] = (idx32, count)
        if self.real_offload and self.pack_gather and sel_layer_idx in self.groups:
            self._launch_gather(sel_layer_idx, sel_layer_idx)

    def _gather_count(self, sel_layer_idx: int, count: torch.Tensor) -> torch.Tensor:
        """Number of rows the host gather of this group fetches (a device int32): all selected rows."""
        return count

    # ------------------------------------------------------------------------------------------
    # offload gather
    # ------------------------------------------------------------------------------------------
    def _staged_for(self, key: int, kcap: int) -> torch.Tensor:
        host = self._host[key]
        st = self._staged.get(key)
        if st is None or st.shape[3] < kcap:
            _, nl, _, KVH, d = host.shape
            st = torch.zeros(nl, 2, KVH, kcap, d, dtype=host.dtype, device=self.cur_len_dev.device)
            self._staged[key] = st
        return st

    def _launch_gather(self, key: int, sel_layer_idx: int, side: bool = True) -> None:
        from .. import ops
        idx32, count = self._idx[sel_layer_idx]
        count = self._gather_count(sel_layer_idx, count)
        staged = self._staged_for(key, idx32.shape[1])
        if not side:
            ops.offload_gather(self._host[key], idx32[0], count, staged)
            return
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=idx32.device)
        main = torch.cuda.current_stream()
        fork = torch.cuda.Event()
        fork.record(main)
        self._side_stream.wait_event(fork)
        with torch.cuda.stream(self._side_stream):
            ops.offload_gather(self._host[key], idx32[0], count, staged)
            done = torch.cuda.Event()
            done.record(self._side_stream)
        self._gather_done[key] = done

    # ------------------------------------------------------------------------------------------
    # attention through the kernels
    # ------------------------------------------------------------------------------------------
    def attend(self, q: torch.Tensor, layer_idx: int, out: Optional[torch.Tensor] = None,
               score_out: Optional[torch.Tensor] = None, score_len: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Decode attention of ``layer_idx`` for q ``[B, H, d]`` over what the reference's ``update``
        would have returned, computed by ``omnikv_decode_attn``.  ``score_out`` (filter layers):
        per-KV-head selector-``last`` score planes for positions ``< score_len``."""
        from .. import ops
        if not self.is_sparse(layer_idx):
            return ops.decode_attn(q, self._k[layer_idx], self._v[layer_idx], self.cur_len_dev, out=out,
                                   score_out=score_out, score_len=score_len)
        left = self.layer_state[layer_idx][1]
        idx32, count = self._idx[left]
        if not self.is_offloaded(layer_idx):
            return ops.decode_attn(q, self._k[layer_idx], self._v[layer_idx], count, idx=idx32,
                                   k_tail=self._k[layer_idx], v_tail=self._v[layer_idx],
                                   tail_start=self.prefill_len_dev, tail_len=self.tail_len_dev, out=out,
                                   max_rows=idx32.shape[1] + self.reserve)
        key, slot = self._host_key(layer_idx)
        if self.pack_gather:
            done = self._gather_done.pop(key, None)
            if done is not None:
                torch.cuda.current_stream().wait_event(done)
        else:
            self._launch_gather(key, left, side=False)
        staged = self._staged[key]
        return ops.decode_attn(q, staged[slot, 0].unsqueeze(0), staged[slot, 1].unsqueeze(0), count,
                               k_tail=self._k[layer_idx], v_tail=self._v[layer_idx], tail_start=self.zero_dev,
                               tail_len=self.tail_len_dev, out=out, max_rows=staged.shape[3] + self.reserve)


class WOPackCache(OmniKVMultiStageCache):
    """``cache_cls = "without_pack"`` (modeling/spec_cache.py:388-520): the index list is only remembered
    at the filter layer and every sparse layer fetches its own rows when it runs -- no packed host
    layout, no overlap with the wait layers."""

    pack_gather = False

    @staticmethod
    def from_dynamic_cache(cache, full_attn_layers: List, num_hidden_layers, num_wait_load_layers=2,
                           real_offload=True):
        c = WOPackCache(full_attn_layers, num_hidden_layers, num_wait_load_layers, real_offload)
        c._adopt(cache)
        return c


class OmniKVLazyCache(OmniKVMultiStageCache):
    """``cache_cls = "lazy"``: the re-gather rule of the reference's OmniKVLazyCache.set_out_idx
    (modeling/spec_cache.py:523-557) on top of the multi-stage cache.  When a filter layer's new selection
    overlaps the one in use by more than ``skip_threshold`` (|new & old| / |new|, :10-31), the group keeps the
    old selection: its sparse layers attend over the same rows and, with ``real_offload``, nothing crosses the
    host link in that step.  The decision is taken on the device (``omnikv_idx_commit``), so the decode step
    stays free of host synchronisation and can be captured in a CUDA graph.

    The reference offers this class to its older single-filter model (modeling/offload_select_once.py:275-276,
    config key ``skip_threshold``, default 0.4); here it plugs into ``OmniKVMulLM`` per filter group."""

    def __init__(self, *args, skip_threshold: float = 0.4, **kw):
        super().__init__(*args, **kw)
        self.skip_threshold = float(skip_threshold)
        self._lazy: Dict[int, SimpleNamespace] = {}

    @staticmethod
    def from_dynamic_cache(cache, full_attn_layers: List, num_hidden_layers, num_wait_load_layers=2,
                           real_offload=True, skip_threshold=0.4):
        c = OmniKVLazyCache(full_attn_layers, num_hidden_layers, num_wait_load_layers, real_offload,
                            skip_threshold=skip_threshold)
        c._adopt(cache)
        return c

    def set_idx_device(self, idx32: torch.Tensor, count: torch.Tensor, sel_layer_idx: int) -> None:
        from .. import ops
        st = self._lazy.get(sel_layer_idx)
        if st is None or st.live_idx.shape != idx32.shape:
            z = lambda: torch.zeros_like(count)  # noqa: E731
            st = SimpleNamespace(live_idx=torch.zeros_like(idx32), live_count=z(), applied=z(), gather_n=z(),
                                 overlap=z(), offered=0)
            self._lazy[sel_layer_idx] = st
        ops.idx_commit(idx32, count, st.live_idx, st.live_count, self.skip_threshold, st.applied, st.gather_n,
                       st.overlap)
        st.offered += 1
        super().set_idx_device(st.live_idx, st.live_count, sel_layer_idx)

    def _gather_count(self, sel_layer_idx: int, count: torch.Tensor) -> torch.Tensor:
        return self._lazy[sel_layer_idx].gather_n

    def lazy_state(self, sel_layer_idx: int) -> Dict[str, List[int]]:
        """Outcome of the last selection offered to a filter group (synchronises): per sequence whether it
        replaced the one in use and how many entries the two shared."""
        st = self._lazy[sel_layer_idx]
        return {"applied": st.applied.tolist(), "overlap": st.overlap.tolist(), "count": st.live_count.tolist()}


def get_cache_cls(config):
    """modeling/spec_cache.py:829-837.  ``multi`` and ``without_pack`` are the classes of the decode-selection
    path; ``lazy`` adds the reference's IoU-skip rule to ``multi``.  The reference's ``default`` and ``eff``
    belong to its older models (``eff`` is broken upstream)."""
    name2cls = {"multi": OmniKVMultiStageCache, "without_pack": WOPackCache, "lazy": OmniKVLazyCache}
    name = config.get("cache_cls", "default")
    if name not in name2cls:
        raise NotImplementedError(f"cache_cls={name!r}: only 'multi', 'without_pack' and 'lazy' are implemented")
    return name2cls[name]
