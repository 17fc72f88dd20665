"""OmniKV's decode-time context selection on B200: the reference's ``modeling/omnikv.py`` API
(``select_tokens_by_attn_universal``, ``OmniKVMulLayer``, ``OmniKVMulModel``, ``OmniKVMulLM``) over
the sm_100a kernels of this package.

What is different from the reference, and why the results are the same:

* the filter layer's selector-``last`` scores are emitted by the layer's OWN decode attention
  kernel while K streams through (same q, same prompt keys as modeling/omnikv.py:24-46, which
  re-projects q and re-reads K in a separate matmul over a ``repeat_kv`` copy);
* top-k + ascending order come from one kernel (``omnikv_topk``) instead of ``topk`` + ``sort``;
* sparse layers read the selected rows through the index list (no gathered copy, no ``cat``);
* lengths, k, and the window bookkeeping live in int32 device arrays, so a decode step has no
  host synchronisation and can be captured in a CUDA graph (``OmniKVMulLM.generate_greedy``).

The Llama decoder itself (embedding, RMSNorm, projections, SwiGLU, lm_head) is plain PyTorch here:
in the reference it is third-party code (transformers' ``LlamaDecoderLayer``), not part of the path.
"""
from __future__ import annotations

import math
import time
from types import SimpleNamespace
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops, tensor_tools
from .omnikv_config import logger
from .spec_cache import OmniKVMultiStageCache, WOPackCache, full_attn_layers_of, get_cache_cls  # noqa: F401

_last_call_t = time.time()


def time_analyze() -> float:
    """Seconds since the previous call (modeling/offload_select_once.py:15-19)."""
    global _last_call_t
    now = time.time()
    out = round(now - _last_call_t, 4)
    _last_call_t = now
    return out


# ----------------------------------------------------------------------------------------------
# rotary embedding (cos/sin generation is the boundary to the HF Llama patch,
# modeling/patch_of_llama3_1.py: default, linear, dynamic-NTK and llama3 frequency rules)
# ----------------------------------------------------------------------------------------------
def _dynamic_ntk_inv_freq(theta: float, d: int, factor: float, max_pos: int, seq_len: torch.Tensor) -> torch.Tensor:
    """Dynamic-NTK frequencies for the current sequence length (a 0-dim integer tensor on any device), with the
    arithmetic of modeling/patch_of_llama3_1.py:137-142 in the same order and precision (fp32 tensor maths):
    ``seq_len`` counts only above ``max_pos``, the base grows with it, ``inv_freq = base ** -(2i/d)``."""
    seq = torch.clamp(seq_len, min=max_pos)
    base = theta * ((factor * seq / max_pos) - (factor - 1)) ** (d / (d - 2))
    expo = torch.arange(0, d, 2, dtype=torch.int64, device=seq_len.device).float() / d
    return 1.0 / (base ** expo)


def rope_parameters(config, seq_len: Optional[int] = None) -> Tuple[torch.Tensor, float]:
    """(inv_freq fp32 ``[d/2]``, attention scaling) for the ``rope_scaling`` of ``config``: the rules of
    ``ROPE_INIT_FUNCTIONS`` in modeling/patch_of_llama3_1.py -- default :12-51, linear :54-93, dynamic NTK
    :96-143, yarn :146-222, longrope :225-287, llama3 :290-330.  ``rope_type`` may also be spelled ``type``."""
    d = int(config.head_dim * getattr(config, "partial_rotary_factor", 1.0))
    base = float(config.rope_theta)
    scaling = getattr(config, "rope_scaling", None) or {}
    kind = scaling.get("rope_type", scaling.get("type", "default")) or "default"
    expo = torch.arange(0, d, 2, dtype=torch.int64).float() / d
    if kind == "default":
        return 1.0 / (base ** expo), 1.0
    if kind == "linear":
        return (1.0 / (base ** expo)) / float(scaling["factor"]), 1.0
    if kind == "dynamic":
        n = torch.tensor(int(seq_len) if seq_len is not None else 0, dtype=torch.int64)
        return _dynamic_ntk_inv_freq(base, d, float(scaling["factor"]), int(config.max_position_embeddings), n), 1.0
    if kind == "llama3":
        inv = 1.0 / (base ** expo)
        factor = scaling["factor"]
        lo, hi = scaling["low_freq_factor"], scaling["high_freq_factor"]
        old = scaling["original_max_position_embeddings"]
        low_wavelen, high_wavelen = old / lo, old / hi
        wavelen = 2 * math.pi / inv
        out = torch.where(wavelen > low_wavelen, inv / factor, inv)
        smooth = (old / wavelen - lo) / (hi - lo)
        mid = (1 - smooth) * out / factor + smooth * out
        is_mid = ~(wavelen < high_wavelen) * ~(wavelen > low_wavelen)
        return torch.where(is_mid, mid, out), 1.0
    if kind == "yarn":
        factor = scaling["factor"]
        max_pos = config.max_position_embeddings
        att = scaling.get("attention_factor")
        if att is None:
            att = 0.1 * math.log(factor) + 1.0
        beta_fast = scaling.get("beta_fast") or 32
        beta_slow = scaling.get("beta_slow") or 1

        def correction_dim(n_rot):  # the dimension that makes n_rot rotations over max_pos positions
            return (d * math.log(max_pos / (n_rot * 2 * math.pi))) / (2 * math.log(base))

        low = max(math.floor(correction_dim(beta_fast)), 0)
        high = min(math.ceil(correction_dim(beta_slow)), d - 1)
        if low == high:
            high += 0.001
        pos_freqs = base ** (torch.arange(0, d, 2).float() / d)
        extrapolation, interpolation = 1.0 / pos_freqs, 1.0 / (factor * pos_freqs)
        ramp = torch.clamp((torch.arange(d // 2, dtype=torch.float32) - low) / (high - low), 0, 1)
        keep = 1 - ramp
        return interpolation * (1 - keep) + extrapolation * keep, float(att)
    if kind == "longrope":
        factor = scaling.get("factor")
        att = scaling.get("attention_factor")
        if hasattr(config, "original_max_position_embeddings"):
            max_pos = config.original_max_position_embeddings
            expanded = config.max_position_embeddings
            factor = expanded / max_pos
        else:
            max_pos = config.max_position_embeddings
            expanded = max_pos * factor
        if att is None:
            att = 1.0 if factor <= 1.0 else math.sqrt(1 + math.log(factor) / math.log(max_pos))
        ext = torch.tensor(scaling["long_factor"] if expanded > max_pos else scaling["short_factor"], dtype=torch.float32)
        return 1.0 / (ext * base ** expo), float(att)
    raise NotImplementedError(f"rope_scaling type {kind!r}")


class OmniKVRotaryEmbedding(nn.Module):
    """cos / sin generation of the Llama patch (modeling/patch_of_llama3_1.py:545-629).  One instance serves every
    layer of a model (the reference holds an identical copy per layer).  ``inv_freq`` is a device buffer that the
    fused decode kernels read directly; for dynamic-NTK scaling it is rewritten IN PLACE, on the device, whenever
    the sequence outgrows the length it was last computed for (``advance``), so a captured decode step keeps
    following the rule when replayed."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        scaling = getattr(config, "rope_scaling", None) or {}
        self.rope_type = scaling.get("rope_type", scaling.get("type", "default")) or "default"
        inv, att = rope_parameters(config)
        self.attention_scaling = float(att)
        self.register_buffer("inv_freq", inv, persistent=False)
        self.original_inv_freq = inv.clone()
        self.original_max_seq_len = int(config.max_position_embeddings)
        self.dynamic = "dynamic" in self.rope_type
        # length inv_freq was last computed for (the reference's max_seq_len_cached), on the device
        self.register_buffer("seq_cached", torch.tensor(self.original_max_seq_len, dtype=torch.int64), persistent=False)

    @torch.no_grad()
    def advance(self, position_ids: torch.Tensor, prefill: bool = False) -> None:
        """The reference's ``_dynamic_frequency_update`` (:589-606), called once per forward before anything reads
        ``inv_freq``: growth recomputes the frequencies for ``max(position_ids) + 1``; a prefill that is back inside
        the original range after a longer sequence restores the original ones.  Decode steps run entirely on the
        device (no synchronisation); a prefill reads the cached length back once."""
        if not self.dynamic:
            return
        s = getattr(self.config, "rope_scaling")
        seq = position_ids.max().to(torch.int64) + 1
        if prefill:
            n, cached = int(seq.item()), int(self.seq_cached.item())
            if n < self.original_max_seq_len and cached > self.original_max_seq_len and n <= cached:
                self.inv_freq.copy_(self.original_inv_freq.to(self.inv_freq.device))
                self.seq_cached.fill_(self.original_max_seq_len)
                return
            if n <= cached:
                return
        torch.maximum(self.seq_cached, seq.to(self.seq_cached.device), out=self.seq_cached)
        self.inv_freq.copy_(_dynamic_ntk_inv_freq(float(self.config.rope_theta), self.inv_freq.numel() * 2,
                                                  float(s["factor"]), self.original_max_seq_len, self.seq_cached))

    @torch.no_grad()
    def forward(self, x: torch.Tensor, position_ids: torch.Tensor):
        """cos, sin ``[B, q, d]`` in x's dtype for integer positions ``[B, q]`` (computed in fp32), times the
        attention scaling of yarn / longrope (:623-624)."""
        freqs = position_ids.to(torch.float32)[:, :, None] * self.inv_freq.to(x.device)[None, None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        cos, sin = emb.cos(), emb.sin()
        if self.attention_scaling != 1.0:
            cos, sin = cos * self.attention_scaling, sin * self.attention_scaling
        return cos.to(x.dtype), sin.to(x.dtype)


class _LazyRotary:
    """(cos, sin) computed when first unpacked; ``cos, sin = obj`` works as with the tuple."""

    def __init__(self, make):
        self._make, self._value = make, None

    def __iter__(self):
        if self._value is None:
            self._value = self._make()
        return iter(self._value)


def rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rotary(x, cos, sin):
    """x ``[B, heads, q, d]``; cos/sin ``[B, q', d]`` with q' == q or 1 (broadcast)."""
    return x * cos.unsqueeze(1) + rotate_half(x) * sin.unsqueeze(1)


# ----------------------------------------------------------------------------------------------
# the selector, reference signature
# ----------------------------------------------------------------------------------------------
def select_tokens_by_attn_universal(raw_attn, hidden_states, position_ids, past_key_value, num_selected_tokens,
                                    consider_len, layer_idx=None, selector_cls="last"):
    """Drop-in for modeling/omnikv.py:8-110: returns the ascending positions ``[B, k]`` (int64) of the
    ``k = min(num_selected_tokens, consider_len)`` prompt tokens with the largest selector score.

    ``raw_attn`` is read exactly as the reference reads it (``q_proj``, ``num_heads``, ``head_dim``,
    ``num_key_value_heads``, ``rotary_emb(x, position_ids)``, ``layer_idx``); ``hidden_states`` is
    ``[B, W, hidden]`` (W = 1 for ``last``) and, as in the reference, every window query is rotated
    with the cos/sin of ``position_ids [B, 1]``.  Scores (fp32) and the top-k run in the CUDA kernels.
    """
    bsz, q_len, _ = hidden_states.shape
    if not past_key_value:
        raise AssertionError("select_tokens_by_attn_universal needs the KV cache")
    if raw_attn.config.get("pretraining_tp", -1) > 1:
        raise NotImplementedError
    q = raw_attn.q_proj(hidden_states).view(bsz, q_len, raw_attn.num_heads, raw_attn.head_dim).transpose(1, 2)
    cos, sin = raw_attn.rotary_emb(q, position_ids)
    q = apply_rotary(q, cos, sin)
    k_cache = past_key_value.key_cache[raw_attn.layer_idx]
    if not k_cache.is_cuda:
        raise ValueError("the filter layer's keys must be on the GPU (filter layers are never offloaded)")
    q = q.to(k_cache.dtype)
    dev = k_cache.device
    n_dev = torch.full((bsz,), int(consider_len), dtype=torch.int32, device=dev)
    k_dev = torch.full((bsz,), int(num_selected_tokens), dtype=torch.int32, device=dev)
    if selector_cls == "last":
        scores = ops.score_last(q[:, :, -1].contiguous(), k_cache, n_dev)
    elif selector_cls in ("softmax_before_last", "uniform", "exp"):
        scores = ops.score_window(q.contiguous(), k_cache, n_dev, selector_cls, max_len=int(consider_len))
    else:
        raise NotImplementedError
    idx, _ = ops.topk(scores, n_dev, k_dev, max_len=int(consider_len))
    return idx[:, : min(int(num_selected_tokens), int(consider_len))].long()


# ----------------------------------------------------------------------------------------------
# modules
# ----------------------------------------------------------------------------------------------
class RMSNorm(nn.Module):
    def __init__(self, hidden_size, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.variance_epsilon)


class _ProjView:
    """``q_proj`` / ``k_proj`` / ... as views of a fused weight: callable and with ``.weight``."""

    def __init__(self, owner, name, lo, hi):
        self._owner, self._name, self._lo, self._hi = owner, name, lo, hi

    @property
    def weight(self):
        return getattr(self._owner, self._name)[self._lo:self._hi]

    def __call__(self, x):
        return F.linear(x, self.weight)


class OmniKVAttention(nn.Module):
    """The ``self_attn`` object of a layer: Llama attention with fused QKV weights whose decode path
    runs in ``omnikv_decode_attn`` through the cache."""

    def __init__(self, config, layer_idx: int, tp=None, rotary_emb=None):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.tp = tp
        world = tp.world if tp is not None else 1
        self.hidden_size = config.hidden_size
        # with tensor parallelism these are the LOCAL head counts (KV heads are sharded, query heads follow)
        self.num_heads = config.num_attention_heads // world
        self.head_dim = config.head_dim
        self.num_key_value_heads = config.num_key_value_heads // world
        if self.num_key_value_heads * world != config.num_key_value_heads:
            raise ValueError("the tensor-parallel size must divide the number of KV heads")
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        nq, nkv = self.num_heads * self.head_dim, self.num_key_value_heads * self.head_dim
        self.qkv_weight = nn.Parameter(torch.empty(nq + 2 * nkv, self.hidden_size))
        self.o_weight = nn.Parameter(torch.empty(self.hidden_size, nq))
        self.q_proj = _ProjView(self, "qkv_weight", 0, nq)
        self.k_proj = _ProjView(self, "qkv_weight", nq, nq + nkv)
        self.v_proj = _ProjView(self, "qkv_weight", nq + nkv, nq + 2 * nkv)
        self.o_proj = _ProjView(self, "o_weight", 0, self.hidden_size)
        # every layer reads the model's one rotary module (same frequencies everywhere, one dynamic update per step)
        self.rotary_emb = rotary_emb if rotary_emb is not None else OmniKVRotaryEmbedding(config)

    def qkv(self, x, cos, sin):
        """x ``[B, n, hidden]`` -> rotated q ``[B,H,n,d]``, rotated k and v ``[B,KVH,n,d]``."""
        B, n, _ = x.shape
        nq, nkv = self.num_heads * self.head_dim, self.num_key_value_heads * self.head_dim
        qkv = F.linear(x, self.qkv_weight)
        q = qkv[..., :nq].view(B, n, self.num_heads, self.head_dim).transpose(1, 2)
        k = qkv[..., nq:nq + nkv].view(B, n, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        v = qkv[..., nq + nkv:].view(B, n, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        return apply_rotary(q, cos, sin), apply_rotary(k, cos, sin), v

    def forward(self, hidden_states, position_embeddings, past_key_value, score_out=None, score_len=None):
        B, n, _ = hidden_states.shape
        rope_pos = getattr(past_key_value, "rope_pos_dev", None)
        if (n == 1 and rope_pos is not None and hidden_states.is_cuda and self.head_dim == 128
                and self.rotary_emb.attention_scaling == 1.0):
            # decode: rotate q and k and append k, v to the cache in one kernel, straight from the fused projection
            tc = _tc_linear_ok(self.config, hidden_states)
            x2 = hidden_states.view(B, -1)
            qkv = ops.batched_linear(x2, self.qkv_weight) if tc else F.linear(x2, self.qkv_weight)
            q = torch.empty(B, self.num_heads, self.head_dim, dtype=qkv.dtype, device=qkv.device)
            k_buf, v_buf, pos = past_key_value.write_target_batch(self.layer_idx)
            ops.rope_append(qkv, self.num_heads, self.num_key_value_heads, self.rotary_emb.inv_freq, rope_pos, q,
                            k_buf, v_buf, pos)
            o = past_key_value.attend(q, self.layer_idx, score_out=score_out, score_len=score_len)
            if tc:
                o = ops.batched_linear(o.view(B, self.num_heads * self.head_dim), self.o_weight).view(B, 1, -1)
            else:
                o = F.linear(o.view(B, 1, self.num_heads * self.head_dim), self.o_weight)
            return self.tp.all_reduce_sum(o) if self.tp is not None else o
        cos, sin = position_embeddings
        q, k, v = self.qkv(hidden_states, cos, sin)
        if n > 1:  # prefill: full causal attention over the fresh keys (what cache.update returns)
            k, v = past_key_value.update(k, v, self.layer_idx)
            if (q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and self.head_dim == 128
                    and self.config.get("prefill_kernel", "tcgen05") == "tcgen05"):
                o = ops.prefill_attn(q, k, v).view(B, n, self.num_heads * self.head_dim)  # this package's kernel
            else:  # fp32 (parity runs) or prefill_kernel="sdpa": the library path
                o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.num_key_value_groups > 1)
                o = o.transpose(1, 2).reshape(B, n, self.num_heads * self.head_dim)
        else:
            past_key_value.append_kv(k[:, :, 0].contiguous(), v[:, :, 0].contiguous(), self.layer_idx)
            o = past_key_value.attend(q[:, :, 0].contiguous(), self.layer_idx, score_out=score_out,
                                      score_len=score_len)
            o = o.view(B, 1, self.num_heads * self.head_dim)
        o = F.linear(o, self.o_weight)
        return self.tp.all_reduce_sum(o) if self.tp is not None else o


def _tc_linear_ok(config, x, inter=64) -> bool:
    """Decode-sized activations (at most 16 tokens, 16-bit, on the GPU) and ``tcgen05_linear`` switched on: the
    projections go through ``omnikv_batched_linear`` instead of the library GEMM."""
    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and x.shape[-2] == 1 and x.numel() // x.shape[-1] <= 16
            and inter % 64 == 0 and x.shape[-1] % 8 == 0 and config.get("tcgen05_linear", False))


class OmniKVMLP(nn.Module):
    def __init__(self, config, tp=None):
        super().__init__()
        self.tp = tp
        self.config = config
        self.intermediate_size = config.intermediate_size // (tp.world if tp is not None else 1)  # local slice
        self.gate_up_weight = nn.Parameter(torch.empty(2 * self.intermediate_size, config.hidden_size))
        self.down_weight = nn.Parameter(torch.empty(config.hidden_size, self.intermediate_size))
        self.gate_proj = _ProjView(self, "gate_up_weight", 0, self.intermediate_size)
        self.up_proj = _ProjView(self, "gate_up_weight", self.intermediate_size, 2 * self.intermediate_size)
        self.down_proj = _ProjView(self, "down_weight", 0, config.hidden_size)

    def forward(self, x):
        if _tc_linear_ok(self.config, x, self.intermediate_size):  # opt-in: this package's tcgen05 weight stream
            x2 = x.reshape(-1, x.shape[-1])
            act = ops.batched_linear(x2, self.gate_up_weight, epilogue="swiglu")
            o = ops.batched_linear(act, self.down_weight).view(*x.shape[:-1], -1)
            return self.tp.all_reduce_sum(o) if self.tp is not None else o
        gu = F.linear(x, self.gate_up_weight)
        if x.is_cuda and x.shape[-2] == 1:  # decode: one kernel for silu(gate) * up
            act = ops.silu_mul(gu.view(-1, 2 * self.intermediate_size)).view(*x.shape[:-1], self.intermediate_size)
        else:
            g, u = gu[..., : self.intermediate_size], gu[..., self.intermediate_size:]
            act = F.silu(g) * u
        o = F.linear(act, self.down_weight)
        return self.tp.all_reduce_sum(o) if self.tp is not None else o


class OmniKVMulLayer(nn.Module):
    """Decoder layer with the filter-layer hook of modeling/omnikv.py:113-246."""

    def __init__(self, config, layer_idx, tp=None, rotary_emb=None):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.tp = tp
        self.self_attn = OmniKVAttention(config, layer_idx, tp, rotary_emb)
        self.mlp = OmniKVMLP(config, tp)
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.prefill_len = None
        self.cache_cls = get_cache_cls(config)
        self.sparse_in_prefill = config.get("sparse_in_prefill", False)
        self.max_len_can_hold = config.get("max_len_can_hold", 32_000)
        self.attn_seg_sz = config.get("attn_seg_sz", 8000)
        self.do_select_layers = [int(i) for i in config.get("do_select_layers").split(",")]
        self.hidden_state_window = None
        self.selector_cls = config.get("selector_cls", "softmax_before_last")
        self.window_size = config.get("window_size", 16)
        self.decode_step = 0
        self.is_filter = layer_idx in self.do_select_layers
        self._fused_cache = {}

    # -- selection state -------------------------------------------------------------------------
    def _init_selection_state(self, cache: OmniKVMultiStageCache, device) -> None:
        """k, candidate range and window bookkeeping as int32 device arrays, per sequence, following
        modeling/omnikv.py:167-188: ``k0 = int(frac * prefill_len)`` (truncation) or the integer;
        for the window selectors ``nptw = max(0, window_size - decode_step)`` newest prompt positions
        are outside the candidate range and are appended after the selection."""
        P = cache.prefill_len_dev
        B = P.shape[0]
        nsel = self.config.get("num_of_selected_tokens", 4096)
        if isinstance(nsel, float):
            # int() truncation of the fraction, per sequence; computed on the host from exact integers
            k0 = torch.tensor([int(nsel * p) for p in P.tolist()], dtype=torch.int32, device=device)
        else:
            k0 = torch.full((B,), int(nsel), dtype=torch.int32, device=device)
        kcap = int(k0.max().item()) if B else 0
        kcap = max(1, min(kcap, int(P.max().item()))) + self.window_size
        st = SimpleNamespace()
        st.k0 = k0
        st.nptw = torch.full((B,), 0 if "last" in self.selector_cls else max(0, self.window_size - 1),
                             dtype=torch.int32, device=device)
        st.k = k0.clone()
        st.consider = P.clone()
        st.idx = torch.zeros(B, kcap, dtype=torch.int32, device=device)
        st.count = torch.zeros(B, dtype=torch.int32, device=device)
        st.max_len = int(P.max().item())
        st.planes = None
        cache.sel_state[self.layer_idx] = st
        return st

    def _select(self, hidden_states, position_embeddings, cache: OmniKVMultiStageCache) -> None:
        """Window selectors: scores from ``omnikv_score_window`` on the observation window's queries."""
        st, attn = cache.sel_state[self.layer_idx], self.self_attn
        B = hidden_states.shape[0]
        if "last" in self.selector_cls:  # "softmax_before_last": the current token only, no window bookkeeping
            window_hs = hidden_states
        else:
            win = torch.cat([self.hidden_state_window, hidden_states], dim=1)[:, -self.window_size:]
            if win.shape == self.hidden_state_window.shape:
                self.hidden_state_window.copy_(win)  # same buffer every step: replayable in a CUDA graph
            else:
                self.hidden_state_window = win.contiguous()
            window_hs = self.hidden_state_window
        W = window_hs.shape[1]
        q = F.linear(window_hs, attn.q_proj.weight)
        rope_pos = getattr(cache, "rope_pos_dev", None)
        if (rope_pos is not None and q.is_cuda and attn.head_dim == 128 and attn.rotary_emb.attention_scaling == 1.0
                and self.config.get("fused_small_ops", True)):
            q = ops.rope_window(q, attn.num_heads, attn.rotary_emb.inv_freq, rope_pos)  # one launch, no rotary table
        else:
            if position_embeddings is None:
                position_embeddings = attn.rotary_emb(window_hs, cache.pos_dev[:, None])
            cos, sin = position_embeddings
            q = apply_rotary(q.view(B, W, attn.num_heads, attn.head_dim).transpose(1, 2), cos, sin).contiguous()
        torch.sub(cache.prefill_len_dev, st.nptw, out=st.consider)
        torch.clamp(st.k0 - st.nptw, min=1, out=st.k)
        if st.planes is None:
            st.planes = torch.zeros(B, st.max_len, dtype=torch.float32, device=q.device)
        if self.tp is None:
            ops.score_window(q, cache._k[self.layer_idx], st.consider, self.selector_cls, max_len=st.max_len,
                             score_out=st.planes)
        else:  # max over the local heads per window slot -> MAX over ranks -> weighted window sum
            if getattr(st, "wplanes", None) is None:
                st.wplanes = torch.zeros(B, W, st.max_len, dtype=torch.float32, device=q.device)
            ops.score_window(q, cache._k[self.layer_idx], st.consider, self.selector_cls, max_len=st.max_len,
                             planes_out=st.wplanes)
            self.tp.all_reduce_max(st.wplanes)
            ops.window_fold(st.wplanes, st.consider, self.selector_cls, max_len=st.max_len, score_out=st.planes)
        ops.topk(st.planes, st.consider, st.k, append_n=st.nptw, idx_out=st.idx, count_out=st.count,
                 max_len=st.max_len)
        torch.clamp(st.nptw - 1, min=0, out=st.nptw)
        self._trace_selection(cache, st)
        cache.set_idx_device(st.idx, st.count, self.layer_idx)

    def _trace_selection(self, cache, st) -> None:
        """Hand the selection to the index recorder, if one is active (tiny_tools/tensor_tools.py:64-74)."""
        tracer = tensor_tools.idx_tracer
        if tracer is None:
            return
        scores = st.planes if st.planes.dim() == 2 else st.planes.max(dim=0).values  # [B, L]
        kmax = int(st.count.max().item())
        idx = st.idx[:, :kmax].long()
        val = scores.gather(1, idx.clamp(max=scores.shape[1] - 1))
        tracer.append_spec_layer(idx, val, cache.prefill_len, self.layer_idx)

    # -- batch-1 decode through the fused weight-streaming kernels -----------------------------------
    def _fused_ok(self, hidden_states) -> bool:
        if hidden_states.shape[0] != 1 or hidden_states.shape[1] != 1 or not hidden_states.is_cuda:
            return False
        key = hidden_states.dtype
        ok = self._fused_cache.get(key)
        if ok is None:
            a = self.self_attn
            # the fused QKV kernel rotates with cos/sin of pos * inv_freq: no attention scaling (yarn, longrope)
            ok = self.config.get("fused_decode", True) and a.rotary_emb.attention_scaling == 1.0 and ops.fused_decode_supported(
                key, self.config.hidden_size, self.mlp.intermediate_size, a.num_heads * a.head_dim, 8)
            self._fused_cache[key] = ok
        return ok

    def _fused_bufs(self, cache, dev, dt):
        bufs = cache.fused_bufs
        if bufs is None:
            attn, mlp = self.self_attn, self.mlp
            bufs = cache.fused_bufs = SimpleNamespace(
                q=torch.empty(1, attn.num_heads, attn.head_dim, dtype=dt, device=dev),
                o=torch.empty(1, attn.num_heads, attn.head_dim, dtype=dt, device=dev),
                act=torch.empty(mlp.intermediate_size, dtype=dt, device=dev))
        return bufs

    def _decode_select_begin(self, hidden_states, cache, position_embeddings, normed=None):
        """Filter layer, before its attention: selector ``last`` hands the attention kernel the score planes to
        fill; the window selectors run their own scoring kernels on the observation window now.
        Returns (score_out, score_len)."""
        if not self.is_filter:
            return None, None
        if not self.config.get("dense_more", False):
            raise ValueError("dense_more=False is not supported")  # as modeling/omnikv.py:211-214
        dev = hidden_states.device
        st = cache.sel_state.get(self.layer_idx)
        if st is None:  # first decode step on this cache (host reads of the lengths happen once, here)
            st = self._init_selection_state(cache, dev)
        if self.selector_cls == "last":
            if st.planes is None:
                st.planes = torch.zeros(self.self_attn.num_key_value_heads, hidden_states.shape[0], st.max_len,
                                        dtype=torch.float32, device=dev)
            return st.planes, cache.prefill_len_dev
        self._select(self.input_layernorm(hidden_states) if normed is None else normed, position_embeddings, cache)
        return None, None

    def _decode_select_end(self, cache, score_out):
        """Filter layer, after its attention: top-k of the planes the attention kernel filled (selector ``last``)."""
        if not self.is_filter:
            return
        if score_out is not None:
            st = cache.sel_state[self.layer_idx]
            if self.tp is not None:  # plane j <- max over ranks of their j-th local KV head: order independent
                self.tp.all_reduce_max(st.planes)
            ops.topk(st.planes, cache.prefill_len_dev, st.k0, idx_out=st.idx, count_out=st.count, max_len=st.max_len)
            self._trace_selection(cache, st)
            cache.set_idx_device(st.idx, st.count, self.layer_idx)
        cache.stage = "decoding"
        self.decode_step += 1

    def _forward_decode_fused(self, hidden_states, cache, position_embeddings):
        """One decode token, batch 1: QKV+RoPE+append, attention (+scores, top-k on filter layers), output
        projection + residual, gate/up + SiLU, down projection + residual -- five weight/KV streaming
        launches plus the split merge.  The residual stream ``hidden_states`` is updated in place."""
        attn, mlp, tp = self.self_attn, self.mlp, self.tp
        h = hidden_states.view(-1)
        bufs = self._fused_bufs(cache, h.device, h.dtype)
        xc = tp.exchange if (tp is not None and getattr(cache, "xchg_on", False)) else None
        if xc is not None and self.is_filter and self.selector_cls != "last" and self.layer_idx > 0:
            raise NotImplementedError("window selectors read the completed hidden state before the QKV kernel "
                                      "has summed the peers' partials; use the NCCL path for them")
        score_out, score_len = self._decode_select_begin(hidden_states, cache, position_embeddings)
        k_seq, v_seq, pos = cache.write_target(self.layer_idx)
        if xc is not None:
            # Fused projection + all-reduce over peer memory: a projection's partial sums go straight to every rank
            # and the NEXT kernel adds them to the residual stream while it loads its activations, storing the
            # completed stream to the other of two buffers (the kernel's other CTAs still read the old one).  The
            # down projection's partials are consumed by the next layer's QKV kernel, or by the logits kernel.
            if getattr(bufs, "hx", None) is None:
                bufs.hx = [torch.empty_like(h), torch.empty_like(h)]
                bufs.hx_i = 0

            def next_h():
                t = bufs.hx[bufs.hx_i]
                bufs.hx_i ^= 1
                return t

            if self.layer_idx > 0:
                h_new = next_h()
                ops.decode_qkv(h, self.input_layernorm.weight, self.input_layernorm.variance_epsilon, attn.qkv_weight,
                               attn.num_heads, attn.num_key_value_heads, attn.rotary_emb.inv_freq, cache.pos_dev, bufs.q,
                               k_seq, v_seq, pos, tp_in=xc.at(2 * self.layer_idx - 1), h_out=h_new)
                h = h_new
            else:
                ops.decode_qkv(h, self.input_layernorm.weight, self.input_layernorm.variance_epsilon, attn.qkv_weight,
                               attn.num_heads, attn.num_key_value_heads, attn.rotary_emb.inv_freq, cache.pos_dev, bufs.q,
                               k_seq, v_seq, pos)
            cache.attend(bufs.q, self.layer_idx, out=bufs.o, score_out=score_out, score_len=score_len)
            self._decode_select_end(cache, score_out)
            ops.decode_gemv_residual(attn.o_weight, bufs.o.view(-1), None, None, tp_out=xc.at(2 * self.layer_idx))
            h_new = next_h()
            ops.decode_gate_up(h, self.post_attention_layernorm.weight, self.post_attention_layernorm.variance_epsilon,
                               mlp.gate_up_weight, bufs.act, tp_in=xc.at(2 * self.layer_idx), h_out=h_new)
            ops.decode_gemv_residual(mlp.down_weight, bufs.act, None, None, tp_out=xc.at(2 * self.layer_idx + 1))
            return (h_new.view(1, 1, -1),)
        ops.decode_qkv(h, self.input_layernorm.weight, self.input_layernorm.variance_epsilon, attn.qkv_weight,
                       attn.num_heads, attn.num_key_value_heads, attn.rotary_emb.inv_freq, cache.pos_dev, bufs.q,
                       k_seq, v_seq, pos)
        cache.attend(bufs.q, self.layer_idx, out=bufs.o, score_out=score_out, score_len=score_len)
        self._decode_select_end(cache, score_out)
        lead = tp is None or tp.rank == 0  # with tensor parallelism only one rank adds the residual before the SUM
        ops.decode_gemv_residual(attn.o_weight, bufs.o.view(-1), h if lead else None, h)
        if tp is not None:
            tp.all_reduce_sum(h)
        ops.decode_gate_up(h, self.post_attention_layernorm.weight, self.post_attention_layernorm.variance_epsilon,
                           mlp.gate_up_weight, bufs.act)
        ops.decode_gemv_residual(mlp.down_weight, bufs.act, h if lead else None, h)
        if tp is not None:
            tp.all_reduce_sum(h)
        return (hidden_states,)

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                output_attentions=False, use_cache=False, cache_position=None, position_embeddings=None):
        if (past_key_value is not None and not output_attentions and position_embeddings is not None
                and self._fused_ok(hidden_states)):
            if not isinstance(past_key_value, self.cache_cls):
                raise AssertionError(f"expected a {self.cache_cls.__name__}")
            out = self._forward_decode_fused(hidden_states, past_key_value, position_embeddings)
            return out + ((past_key_value,) if use_cache else ())
        residual = hidden_states
        n = hidden_states.shape[1]
        # decode through the PyTorch modules (several sequences, or the fused batch-1 kernels switched off): every
        # residual add travels with the norm behind it in one launch, so the second add of a layer is handed to
        # the next layer (or to the model's final norm) through the cache object
        small = (n == 1 and hidden_states.is_cuda and hidden_states.is_contiguous() and past_key_value is not None
                 and self.config.get("fused_small_ops", True))
        if small:
            B = hidden_states.shape[0]
            stream2d = residual.view(B, -1)
            delta = getattr(past_key_value, "pending_delta", None)
            past_key_value.pending_delta = None
            hidden_states = ops.add_rms_norm(stream2d, delta, self.input_layernorm.weight,
                                             self.input_layernorm.variance_epsilon).view(B, 1, -1)
        else:
            hidden_states = self.input_layernorm(hidden_states)
        if n > 1:
            self.prefill_len = n
            if "last" not in self.selector_cls and self.is_filter:
                self.hidden_state_window = hidden_states[:, -self.window_size:].clone()
                self.decode_step = 1
        if past_key_value is not None and not isinstance(past_key_value, self.cache_cls):
            raise AssertionError(f"expected a {self.cache_cls.__name__}")
        if position_embeddings is None:
            position_embeddings = self.self_attn.rotary_emb(hidden_states, position_ids)

        selecting = n == 1 and past_key_value is not None and self.is_filter
        score_out = score_len = None
        if selecting:
            score_out, score_len = self._decode_select_begin(residual, past_key_value, position_embeddings,
                                                             normed=hidden_states if small else None)

        hidden_states = self.self_attn(hidden_states, position_embeddings, past_key_value, score_out=score_out,
                                       score_len=score_len)
        if selecting:
            self._decode_select_end(past_key_value, score_out)
        if small:
            hidden_states = ops.add_rms_norm(stream2d, hidden_states.reshape(B, -1), self.post_attention_layernorm.weight,
                                             self.post_attention_layernorm.variance_epsilon).view(B, 1, -1)
            past_key_value.pending_delta = self.mlp(hidden_states).reshape(B, -1)
            outputs = (residual,)
            if output_attentions:
                outputs += (None,)
            if use_cache:
                outputs += (past_key_value,)
            return outputs
        hidden_states = residual + hidden_states

        residual = hidden_states
        hidden_states = self.post_attention_layernorm(hidden_states)
        if n > 4000:  # prefill: MLP in 4000-token chunks (modeling/omnikv.py:233-235)
            hidden_states = torch.cat([self.mlp(hs) for hs in torch.split(hidden_states, 4000, dim=1)], dim=1)
        else:
            hidden_states = self.mlp(hidden_states)
        hidden_states = residual + hidden_states
        outputs = (hidden_states,)
        if output_attentions:
            outputs += (None,)
        if use_cache:
            outputs += (past_key_value,)
        return outputs


class OmniKVMulModel(nn.Module):
    def __init__(self, config, tp=None):
        super().__init__()
        self.config = config
        self.tp = tp
        self.padding_idx = config.pad_token_id
        self.vocab_size = config.vocab_size
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, self.padding_idx)
        self.rotary_emb = OmniKVRotaryEmbedding(config)
        self.layers = nn.ModuleList([OmniKVMulLayer(config, i, tp, self.rotary_emb) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps)

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None,
                inputs_embeds=None, use_cache=None, output_attentions=None, output_hidden_states=None,
                return_dict=None, cache_position=None, apply_final_norm=True):
        h = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds.clone()
        B, n, _ = h.shape
        cache = past_key_values
        if self.tp is not None:
            self.tp.begin_step()
        if n == 1:
            cache.begin_decode_step()
            if position_ids is None:
                position_ids = cache.pos_dev[:, None]
                cache.rope_pos_dev = cache.pos_dev
            else:  # the caller's positions (int32 on the device) for the fused rotate-and-append kernel
                cache.rope_pos_dev = position_ids.reshape(-1).to(torch.int32).contiguous()
        elif position_ids is None:
            position_ids = torch.arange(n, device=h.device)[None, :].expand(B, n)
        self.rotary_emb.advance(position_ids, prefill=n > 1)  # dynamic-NTK scaling follows the sequence length
        # the fused batch-1 kernels rotate inside the QKV kernel and never read the table: build it on first use
        pos_emb = _LazyRotary(lambda: self.rotary_emb(h, position_ids))
        for layer in self.layers:
            h = layer(h, attention_mask=attention_mask, position_ids=position_ids, past_key_value=cache,
                      use_cache=use_cache, cache_position=cache_position, position_embeddings=pos_emb)[0]
            if n > 1:
                h = h.contiguous()
        delta = getattr(cache, "pending_delta", None) if cache is not None else None
        if delta is not None:  # the last layer's second residual add, handed on by the layer (see OmniKVMulLayer.forward)
            cache.pending_delta = None
            if apply_final_norm:
                h = ops.add_rms_norm(h.view(B, -1), delta, self.norm.weight, self.norm.variance_epsilon).view(B, 1, -1)
            else:
                h = h + delta.view_as(h)
        elif apply_final_norm:
            h = self.norm(h)
        return SimpleNamespace(last_hidden_state=h, past_key_values=cache, hidden_states=None, attentions=None)


class CausalLMOutputWithPast(SimpleNamespace):
    def __getitem__(self, i):
        return (self.logits, self.past_key_values)[i]


class OmniKVMulLM(nn.Module):
    """``model_cls = "multi"`` (modeling/omnikv.py:271-394)."""

    def __init__(self, config, tp=None):
        super().__init__()
        if (fac := config.get("rope_factor", -1)) > 0:
            config.rope_scaling = {"type": "dynamic", "factor": fac}
        config.rope_scaling_ = config.rope_scaling
        self.config = config
        self.tp = tp
        self.model = OmniKVMulModel(config, tp)
        self.vocab_size = config.vocab_size
        vocab_local = config.vocab_size // (tp.world if tp is not None else 1)  # vocabulary-sharded head
        self.lm_head = nn.Linear(config.hidden_size, vocab_local, bias=False)
        self.max_context_len = config.get("max_context_len", 50_000)
        self.cache_cls = get_cache_cls(config)
        self._graph = None

    # -- construction ----------------------------------------------------------------------------
    @torch.no_grad()
    def init_random_(self, seed: int = 0, std: float = 0.02):
        """Seeded N(0, std) weights, norm weights 1 (benchmarks run on random-init weights).

        The random stream is that of the UNSHARDED model: every matrix is drawn at its full Hugging Face shape
        (q, k, v, o, gate, up, down per layer, then the embedding and the head, in that order, in blocks of rows)
        and each rank keeps its slice -- the same slices ``load_hf_state_dict`` takes.  A tensor-parallel group
        built from one seed is therefore the same model as the single-GPU one, which is what lets a multi-GPU
        run be checked against it."""
        dev = self.lm_head.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)
        tp, cfg = self.tp, self.config

        def draw(dst, rows, cols, dim=None):
            """dst: this rank's ``[rows_local, cols_local]`` slice (dimension ``dim`` sharded) of a rows x cols matrix."""
            lo_r, hi_r = tp.shard(rows) if (tp is not None and dim == 0) else (0, rows)
            lo_c, hi_c = tp.shard(cols) if (tp is not None and dim == 1) else (0, cols)
            step = max(1, (1 << 26) // cols)
            for s0 in range(0, rows, step):
                e0 = min(rows, s0 + step)
                blk = torch.randn(e0 - s0, cols, generator=g, device=dev, dtype=torch.float32)
                a, b = max(s0, lo_r), min(e0, hi_r)
                if a < b:
                    dst[a - lo_r:b - lo_r].copy_(blk[a - s0:b - s0, lo_c:hi_c] * std)

        hid, inter, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
        nq, nkv = cfg.num_attention_heads * d, cfg.num_key_value_heads * d
        for layer in self.model.layers:
            a, mlp = layer.self_attn, layer.mlp
            draw(a.q_proj.weight, nq, hid, 0)
            draw(a.k_proj.weight, nkv, hid, 0)
            draw(a.v_proj.weight, nkv, hid, 0)
            draw(a.o_proj.weight, hid, nq, 1)
            draw(mlp.gate_proj.weight, inter, hid, 0)
            draw(mlp.up_proj.weight, inter, hid, 0)
            draw(mlp.down_proj.weight, hid, inter, 1)
            layer.input_layernorm.weight.fill_(1.0)
            layer.post_attention_layernorm.weight.fill_(1.0)
        draw(self.model.embed_tokens.weight, cfg.vocab_size, hid)
        draw(self.lm_head.weight, cfg.vocab_size, hid, 0)
        self.model.norm.weight.fill_(1.0)
        return self

    @classmethod
    def from_config(cls, config, dtype=torch.bfloat16, device="cuda", seed: Optional[int] = 0, tp=None):
        prev = torch.get_default_dtype()
        torch.set_default_dtype(dtype)
        try:
            with torch.device(device):
                m = cls(config, tp)
        finally:
            torch.set_default_dtype(prev)
        m.eval()
        if seed is not None:
            m.init_random_(seed)
        return m

    @classmethod
    def from_pretrained(cls, path, config=None, torch_dtype=torch.float16, device="cuda", **_unused):
        """Load a Hugging Face Llama checkpoint directory (``*.safetensors``) into the fused layout."""
        import glob
        import os
        from safetensors import safe_open  # optional dependency, only for real checkpoints

        from .omnikv_config import LlamaCompressorConfig
        config = config or LlamaCompressorConfig.from_pretrained(path)
        m = cls.from_config(config, dtype=torch_dtype, device=device, seed=None)
        sd = {}
        for fn in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
            with safe_open(fn, framework="pt", device="cpu") as f:
                for k in f.keys():
                    sd[k] = f.get_tensor(k)
        m.load_hf_state_dict(sd)
        return m

    @torch.no_grad()
    def load_hf_state_dict(self, sd):
        tp = self.tp

        def put(dst, src, dim=None):
            """Copy the full tensor, or this rank's slice of dimension ``dim`` when sharded."""
            if tp is not None and dim is not None:
                lo, hi = tp.shard(src.shape[dim])
                src = src.narrow(dim, lo, hi - lo)
            dst.copy_(src.to(dst.dtype))
        put(self.model.embed_tokens.weight, sd["model.embed_tokens.weight"])
        put(self.model.norm.weight, sd["model.norm.weight"])
        put(self.lm_head.weight, sd.get("lm_head.weight", sd["model.embed_tokens.weight"]), 0)
        for i, layer in enumerate(self.model.layers):
            p = f"model.layers.{i}."
            a, mlp = layer.self_attn, layer.mlp
            for name in ("q_proj", "k_proj", "v_proj"):
                put(getattr(a, name).weight, sd[p + f"self_attn.{name}.weight"], 0)
            put(a.o_proj.weight, sd[p + "self_attn.o_proj.weight"], 1)
            put(mlp.gate_proj.weight, sd[p + "mlp.gate_proj.weight"], 0)
            put(mlp.up_proj.weight, sd[p + "mlp.up_proj.weight"], 0)
            put(mlp.down_proj.weight, sd[p + "mlp.down_proj.weight"], 1)
            put(layer.input_layernorm.weight, sd[p + "input_layernorm.weight"])
            put(layer.post_attention_layernorm.weight, sd[p + "post_attention_layernorm.weight"])

    def hf_state_dict(self):
        """Weights under their Hugging Face Llama names (views of the fused tensors)."""
        sd = {"model.embed_tokens.weight": self.model.embed_tokens.weight, "model.norm.weight": self.model.norm.weight,
              "lm_head.weight": self.lm_head.weight}
        for i, layer in enumerate(self.model.layers):
            p = f"model.layers.{i}."
            for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
                sd[p + f"self_attn.{name}.weight"] = getattr(layer.self_attn, name).weight
            for name in ("gate_proj", "up_proj", "down_proj"):
                sd[p + f"mlp.{name}.weight"] = getattr(layer.mlp, name).weight
            sd[p + "input_layernorm.weight"] = layer.input_layernorm.weight
            sd[p + "post_attention_layernorm.weight"] = layer.post_attention_layernorm.weight
        return sd

    @torch.no_grad()
    def prepare_synthetic_decode(self, batch: int, seed: int = 0) -> None:
        """Throughput runs that fill the KV cache directly (no prefill): give every filter layer the state a prefill
        would have left -- for the window selectors a seeded observation window of normalised hidden states -- so
        that decoding can start."""
        dev, dt = self.lm_head.weight.device, self.lm_head.weight.dtype
        g = torch.Generator(device=dev).manual_seed(seed)
        for layer in self.model.layers:
            layer.decode_step = 0
            if layer.is_filter and "last" not in layer.selector_cls:
                layer.hidden_state_window = torch.randn(batch, layer.window_size, self.config.hidden_size, generator=g,
                                                        device=dev, dtype=torch.float32).to(dt)
                layer.decode_step = 1

    # -- cache -----------------------------------------------------------------------------------
    def new_cache(self, past_key_values=None):
        """The cache wrap of modeling/omnikv.py:315-341."""
        cache_cls_name = self.config.get("cache_cls", "default")
        if cache_cls_name not in ("multi", "without_pack", "lazy"):
            raise NotImplementedError
        do_sel_layers = [int(i) for i in self.config.get("do_select_layers").split(",")]
        kwargs = {}
        if cache_cls_name == "lazy":  # modeling/offload_select_once.py:275-276
            kwargs["skip_threshold"] = self.config.get("skip_threshold", 0.4)
        return self.cache_cls.from_dynamic_cache(
            past_key_values,
            full_attn_layers=full_attn_layers_of(do_sel_layers, self.config.num_hidden_layers),
            num_hidden_layers=self.config.num_hidden_layers,
            num_wait_load_layers=self.config.get("num_wait_load_layers", 2),
            real_offload=self.config.get("real_offload", True),
            **kwargs,
        )

    # -- reference forward -----------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None,
                inputs_embeds=None, labels=None, use_cache=None, output_attentions=None,
                output_hidden_states=None, return_dict=None, cache_position=None):
        n = input_ids.shape[1]
        if not isinstance(past_key_values, self.cache_cls):
            past_key_values = self.new_cache(past_key_values)
        past_key_values.stage = "decoding" if n == 1 else "prefill"
        outputs = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                             past_key_values=past_key_values, inputs_embeds=inputs_embeds, use_cache=use_cache,
                             cache_position=cache_position)
        hidden_states = outputs.last_hidden_state[:, -1:]
        logits = self._gather_logits(self.lm_head(hidden_states)).float()
        if labels is not None:
            raise NotImplementedError
        if n > 1:
            logger.info(f"---prefill time {round(time_analyze(), 3)}s")
        else:
            logger.info(f"---decoding time {round(time_analyze(), 3)}s")
        return CausalLMOutputWithPast(loss=None, logits=logits, past_key_values=past_key_values,
                                      hidden_states=None, attentions=None)

    # -- decode engine ---------------------------------------------------------------------------
    def _decode_step(self, tokens: torch.Tensor, cache):
        """One decode step for tokens ``[B, 1]`` (device): (fp32 logits ``[B, vocab]``, greedy next token
        ``[B, 1]`` int64).  No host synchronisation.  At batch 1 in a 16-bit dtype the final norm, the
        lm_head and the arg-max run in one fused weight-streaming kernel."""
        layer0 = self.model.layers[0]
        fused = tokens.shape[0] == 1 and layer0._fused_ok(self.model.embed_tokens.weight[:1].view(1, 1, -1))
        if fused and self.tp is None and self.config.get("chained_decode", False) and ops.decode_chain_supported(
                self.lm_head.weight.dtype, self.config.hidden_size, layer0.mlp.intermediate_size,
                layer0.self_attn.num_heads) and self.lm_head.weight.shape[0] % 8 == 0:
            return self._decode_step_chained(tokens, cache)
        tp = self.tp
        xc = tp.exchange if (fused and tp is not None and self._exchange_ok()) else None
        cache.xchg_on = xc is not None
        if xc is not None:
            xc.begin_step()
        try:
            out = self.model(input_ids=tokens, past_key_values=cache, apply_final_norm=not fused)
        finally:
            cache.xchg_on = False
        h = out.last_hidden_state[:, -1]
        if not fused:
            logits = self._gather_logits(self.lm_head(h)).float()
            return logits, logits.argmax(-1, keepdim=True)
        fb = cache.fused_bufs
        if getattr(fb, "logits", None) is None:
            fb.logits = torch.empty(1, self.lm_head.weight.shape[0], dtype=torch.float32, device=h.device)
            fb.best = torch.zeros(1, dtype=torch.int64, device=h.device)
            fb.token = torch.zeros(1, 1, dtype=torch.int64, device=h.device)
        lo = tp.shard(self.vocab_size)[0] if tp is not None else 0
        n_layers = len(self.model.layers)
        ops.decode_logits(h.reshape(-1), self.model.norm.weight, self.model.norm.variance_epsilon, self.lm_head.weight,
                          lo, fb.logits, fb.best, fb.token if tp is None else None,
                          tp_in=xc.at(2 * n_layers - 1) if xc is not None else None)
        if tp is None:
            return fb.logits, fb.token
        logits = tp.all_gather_last(fb.logits)
        return logits, logits.argmax(-1, keepdim=True)

    def _exchange_ok(self) -> bool:
        """The fused projection + all-reduce path covers selector ``last`` (the window selectors need the completed
        hidden state on the host side of the layer) and fewer than 128 layers (exchange numbers stay below 256)."""
        return (self.tp is not None and self.tp.exchange is not None and len(self.model.layers) < 128
                and self.config.get("selector_cls", "softmax_before_last") == "last"
                and self.config.get("peer_exchange", True))

    def _decode_step_chained(self, tokens, cache):
        """Batch-1 decode step as 33 cooperative weight-streaming launches interleaved with the 32 attention
        launches: [QKV of layer 0], then per layer [attention] and [output projection, MLP, next layer's QKV
        (or the final norm, lm_head and arg-max)] -- see ``omnikv_decode_chain``."""
        layers = self.model.layers
        cfg = self.config
        cache.begin_decode_step()
        self.model.rotary_emb.advance(cache.pos_dev[:, None])
        h = self.model.embed_tokens(tokens).view(-1)
        fb = layers[0]._fused_bufs(cache, h.device, h.dtype)
        if getattr(fb, "logits", None) is None:
            fb.logits = torch.empty(1, self.lm_head.weight.shape[0], dtype=torch.float32, device=h.device)
            fb.best = torch.zeros(1, dtype=torch.int64, device=h.device)
            fb.token = torch.zeros(1, 1, dtype=torch.int64, device=h.device)
            fb.counters = torch.zeros(len(layers) + 1, 4, dtype=torch.int32, device=h.device)
        fb.counters.zero_()  # chunk counters of this step's launches (dynamic scheduling)
        a0 = layers[0].self_attn
        common = dict(eps=cfg.rms_norm_eps, H=a0.num_heads, KVH=a0.num_key_value_heads, inter=layers[0].mlp.intermediate_size)

        def qkv_args(layer):
            k_seq, v_seq, pos = cache.write_target(layer.layer_idx)
            return dict(in_norm_w=layer.input_layernorm.weight, w_qkv=layer.self_attn.qkv_weight,
                        inv_freq=layer.self_attn.rotary_emb.inv_freq, rope_pos=cache.pos_dev, q_out=fb.q,
                        k_cache_seq=k_seq, v_cache_seq=v_seq, cache_pos=pos)

        ops.decode_chain(h, **common, chunk_counters=fb.counters[0], next_w=layers[0].self_attn.o_weight,
                         **qkv_args(layers[0]))
        hs = h.view(1, 1, -1)
        for i, layer in enumerate(layers):
            score_out, score_len = layer._decode_select_begin(hs, cache, None)
            cache.attend(fb.q, i, out=fb.o, score_out=score_out, score_len=score_len)
            layer._decode_select_end(cache, score_out)
            tail = (qkv_args(layers[i + 1]) if i + 1 < len(layers) else
                    dict(final_norm_w=self.model.norm.weight, w_head=self.lm_head.weight, logits=fb.logits, best=fb.best,
                         token_out=fb.token))
            ops.decode_chain(h, **common, w_o=layer.self_attn.o_weight, attn_out=fb.o,
                             post_norm_w=layer.post_attention_layernorm.weight, w_gate_up=layer.mlp.gate_up_weight,
                             w_down=layer.mlp.down_weight, act=fb.act, chunk_counters=fb.counters[i + 1],
                             next_w=layers[i + 1].self_attn.o_weight if i + 1 < len(layers) else None, **tail)
        return fb.logits, fb.token

    def _gather_logits(self, local):
        return self.tp.all_gather_last(local) if self.tp is not None else local

    @torch.no_grad()
    def generate_greedy(self, input_ids: Optional[torch.Tensor], max_new_tokens: int, cache=None,
                        first_token: Optional[torch.Tensor] = None, use_cuda_graph: bool = True,
                        warmup_steps: int = 2) -> torch.Tensor:
        """Greedy decoding.  Prefills ``input_ids`` (or continues from a filled ``cache`` with
        ``first_token`` ``[B, 1]``), then runs ``max_new_tokens - 1`` decode steps on the device
        without host synchronisation; with ``use_cuda_graph`` one step is captured and replayed.
        Returns the generated ids ``[B, max_new_tokens]``."""
        runner = DecodeRunner(self, input_ids, cache=cache, first_token=first_token, max_new_tokens=max_new_tokens,
                              use_cuda_graph=use_cuda_graph, warmup_steps=warmup_steps)
        runner.run(max_new_tokens - 1 - runner.steps_done)
        return runner.tokens(check=True)


class DecodeRunner:
    """Greedy decode loop whose state lives on the device: the last token, the output buffer and the
    step counter are device tensors, so steps chain without the host; ``use_cuda_graph`` captures one
    step (all kernels of this package launch on the capturing stream) and replays it."""

    def __init__(self, lm: OmniKVMulLM, input_ids, cache=None, first_token=None, max_new_tokens=128,
                 use_cuda_graph=True, warmup_steps=2):
        self.lm = lm
        if cache is None:
            out = lm(input_ids=input_ids)
            cache = out.past_key_values
            first_token = out.logits[:, -1].argmax(-1, keepdim=True)
        self.cache = cache
        cache.stage = "decoding"
        B = first_token.shape[0]
        dev = first_token.device
        self.token = first_token.clone().to(torch.int64)              # [B,1] the token to feed next
        self.out = torch.zeros(B, max_new_tokens, dtype=torch.int64, device=dev)
        self.out[:, 0:1] = self.token
        self.step_dev = torch.ones(1, 1, dtype=torch.int64, device=dev).expand(B, 1).contiguous()
        self.logits = None
        self.steps_done = 0
        self.max_new_tokens = max_new_tokens
        self.graph = None
        self.launches_per_step = 0
        if use_cuda_graph and tensor_tools.idx_tracer is None:  # recording reads the selection on the host
            for _ in range(min(warmup_steps, max_new_tokens - 1)):
                self._step()
                self.steps_done += 1
            if self.steps_done < max_new_tokens - 1:
                self._capture()

    def _step(self):
        n0 = ops.launch_count()
        logits, nxt = self.lm._decode_step(self.token, self.cache)
        self.launches_per_step = ops.launch_count() - n0  # kernels of this package launched by one step
        self.token.copy_(nxt)
        self.out.scatter_(1, self.step_dev, nxt)
        self.step_dev.add_(1)
        if self.logits is None:
            self.logits = torch.empty_like(logits)
        self.logits.copy_(logits)

    def _capture(self):
        torch.cuda.synchronize()
        seen = self.cache._seen_tokens
        steps = [layer.decode_step for layer in self.lm.model.layers]
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._step()
        # capture ran the host side of one step without executing it on the device
        self.cache._seen_tokens = seen
        for layer, s in zip(self.lm.model.layers, steps):
            layer.decode_step = s

    def run(self, n_steps: int) -> None:
        n_steps = max(0, min(n_steps, self.max_new_tokens - 1 - self.steps_done))
        self.cache.check_room(n_steps)
        for _ in range(n_steps):
            if self.graph is not None:
                self.graph.replay()
                self.cache._seen_tokens += 1
                for layer in self.lm.model.layers:
                    if layer.is_filter:
                        layer.decode_step += 1
            else:
                self._step()
        self.steps_done += n_steps

    def tokens(self, check: bool = False) -> torch.Tensor:
        """The ids generated so far ``[B, steps_done + 1]``.  ``check`` synchronises and raises if any kernel of
        the steps reported that one of its bounded waits ran out (an absent rank, a copy that never landed):
        tokens produced after that are not to be trusted."""
        if check:
            ops.check_status(self.out.device)
        return self.out[:, : self.steps_done + 1]
