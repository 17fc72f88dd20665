"""Model-level CPU oracle: a plain fp32 PyTorch Llama decoder that calls the oracle's selector and
cache exactly where the reference's layer does.

TEST INFRASTRUCTURE ONLY.  Follows modeling/omnikv.py:143-246 (``OmniKVMulLayer.forward``: window
capture at prefill, k / consider_len / nptw bookkeeping, selection before the attention, append of
the prompt positions still inside the window, ``set_idx_on_gpu``) and :287-394 (``OmniKVMulLM.forward``:
cache wrap, stage, last-position logits in fp32).  The attention, RMSNorm, SwiGLU and RoPE themselves
are transformers 4.41.2 code in the reference (not in its tree): here they are the textbook
definitions in fp32 -- parity UNPINNED at that boundary.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from . import omnikv_oracle as oo


class _Attn:
    """The duck-typed ``self_attn`` handed to the selector."""

    def __init__(self, wq, num_heads, num_kv_heads, head_dim, theta, layer_idx):
        self.num_heads, self.num_key_value_heads, self.head_dim, self.layer_idx = num_heads, num_kv_heads, head_dim, layer_idx
        self._wq, self._theta = wq, theta

    def q_proj(self, x):
        return F.linear(x, self._wq)

    def rotary_emb(self, x, position_ids):
        return oo.rope_cos_sin(position_ids, self.head_dim, self._theta)


def _rms(x, w, eps):
    v = x.pow(2).mean(-1, keepdim=True)
    return x * torch.rsqrt(v + eps) * w


class OracleLM:
    def __init__(self, cfg: Dict, weights: Dict[str, torch.Tensor], device="cpu"):
        """cfg: plain dict with the Llama fields and the OmniKV keys; weights: HF-named tensors (held as fp32 on
        ``device``: the CPU, or a GPU when a test checks a model too large for a CPU run -- still this fp32 code)."""
        self.cfg = cfg
        self.device = torch.device(device)
        self.w = {k: v.detach().to(self.device, torch.float32) for k, v in weights.items()}
        self.n_layers = cfg["num_hidden_layers"]
        self.H, self.KVH = cfg["num_attention_heads"], cfg["num_key_value_heads"]
        self.d = cfg.get("head_dim") or cfg["hidden_size"] // self.H
        self.sel_layers = [int(i) for i in cfg["do_select_layers"].split(",")]
        self.selector = cfg.get("selector_cls", "softmax_before_last")
        self.window = cfg.get("window_size", 16)
        self.state = [dict(prefill_len=None, window=None, decode_step=0) for _ in range(self.n_layers)]
        self.selected = {}  # (decode forward number, layer) -> idx, for the tests
        self.scores = {}    # (decode forward number, layer) -> (scores [B, consider_len], k) behind that selection

    def new_cache(self):
        name = self.cfg.get("cache_cls", "multi")
        full = oo.full_attn_layers_of(self.sel_layers, self.n_layers)
        args = (full, self.n_layers, self.cfg.get("num_wait_load_layers", 2), self.cfg.get("real_offload", True))
        if name == "lazy":
            return oo.OracleLazyMultiStageCache(*args, skip_threshold=self.cfg.get("skip_threshold", 0.4))
        return (oo.OracleMultiStageCache if name == "multi" else oo.OracleWOPackCache)(*args)

    def _layer(self, i, h, position_ids, cache, fwd_no):
        p = f"model.layers.{i}."
        w, st = self.w, self.state[i]
        resid = h
        x = _rms(h, w[p + "input_layernorm.weight"], self.cfg["rms_norm_eps"])
        B, n, _ = x.shape
        if n > 1:
            st["prefill_len"] = n
            if "last" not in self.selector and i in self.sel_layers:
                st["window"] = x[:, -self.window:]
                st["decode_step"] = 1
        consider_len = st["prefill_len"]
        k_sel = self.cfg.get("num_of_selected_tokens", 4096)
        if isinstance(k_sel, float):
            k_sel = int(k_sel * consider_len)
        attn = _Attn(w[p + "self_attn.q_proj.weight"], self.H, self.KVH, self.d, self.cfg["rope_theta"], i)
        if n == 1 and i in self.sel_layers:
            window_hs = x
            nptw = max(0, self.window - st["decode_step"])
            if "last" not in self.selector:
                st["window"] = torch.cat([st["window"], x], dim=1)[:, -self.window:]
                window_hs = st["window"]
                consider_len -= nptw
                k_sel = max(1, k_sel - nptw)
            idx = oo.select_tokens_by_attn_universal(attn, window_hs, position_ids, cache, k_sel, consider_len, i,
                                                     self.selector)
            self.scores[(fwd_no, i)] = (oo.select_tokens_by_attn_universal.last_scores, k_sel)
            if "last" not in self.selector:
                extra = torch.arange(st["prefill_len"] - nptw, st["prefill_len"], device=idx.device)[None, :].repeat(idx.shape[0], 1)
                idx = torch.cat([idx, extra], dim=1)
            self.selected[(fwd_no, i)] = idx
            cache.set_idx_on_gpu(idx, i)
            cache.stage = "decoding"
            st["decode_step"] += 1
        # attention (third-party in the reference): q/k/v projections, RoPE, cache.update, softmax(qK^T/sqrt d)V
        q = F.linear(x, w[p + "self_attn.q_proj.weight"]).view(B, n, self.H, self.d).transpose(1, 2)
        k = F.linear(x, w[p + "self_attn.k_proj.weight"]).view(B, n, self.KVH, self.d).transpose(1, 2)
        v = F.linear(x, w[p + "self_attn.v_proj.weight"]).view(B, n, self.KVH, self.d).transpose(1, 2)
        cos, sin = oo.rope_cos_sin(position_ids, self.d, self.cfg["rope_theta"])
        q, k = oo.apply_rope(q, cos, sin), oo.apply_rope(k, cos, sin)
        kk, vv = cache.update(k, v, i)
        if n > 1:
            g = self.H // self.KVH
            kr = kk[:, :, None].expand(B, self.KVH, g, n, self.d).reshape(B, self.H, n, self.d)
            vr = vv[:, :, None].expand(B, self.KVH, g, n, self.d).reshape(B, self.H, n, self.d)
            s = torch.matmul(q, kr.transpose(2, 3)) / math.sqrt(self.d)
            s = s + torch.full((n, n), float("-inf"), device=s.device).triu(1)
            o = torch.matmul(torch.softmax(s, dim=-1), vr)
        else:
            o = oo.dense_attention(q[:, :, 0], kk, vv)[:, :, None, :]
        o = o.transpose(1, 2).reshape(B, n, self.H * self.d)
        h = resid + F.linear(o, w[p + "self_attn.o_proj.weight"])
        x = _rms(h, w[p + "post_attention_layernorm.weight"], self.cfg["rms_norm_eps"])
        m = F.linear(F.silu(F.linear(x, w[p + "mlp.gate_proj.weight"])) * F.linear(x, w[p + "mlp.up_proj.weight"]),
                     w[p + "mlp.down_proj.weight"])
        return h + m

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, cache=None, position_ids: Optional[torch.Tensor] = None, fwd_no=0):
        B, n = input_ids.shape
        if cache is None:
            cache = self.new_cache()
        cache.stage = "decoding" if n == 1 else "prefill"
        if position_ids is None:
            start = cache._seen_tokens
            position_ids = torch.arange(start, start + n, device=self.device)[None, :].expand(B, n)
        h = F.embedding(input_ids.to(self.device), self.w["model.embed_tokens.weight"])
        trace = [h]  # residual stream entering every layer, then leaving the last one (kept for per-layer checks)
        for i in range(self.n_layers):
            h = self._layer(i, h, position_ids, cache, fwd_no)
            trace.append(h)
        self.hidden_trace = trace
        h = _rms(h, self.w["model.norm.weight"], self.cfg["rms_norm_eps"])
        logits = F.linear(h[:, -1:], self.w["lm_head.weight"]).float()
        return logits, cache

    @torch.no_grad()
    def forward_hidden(self, x: torch.Tensor, cache=None, fwd_no=0):
        """The decoder stack alone on input hidden states ``[B, n, hidden]`` (no embedding, no final norm):
        what the layer-hook fixture drives through the reference's ``OmniKVMulLayer.forward``."""
        B, n, _ = x.shape
        if cache is None:
            cache = self.new_cache()
        cache.stage = "decoding" if n == 1 else "prefill"
        start = cache._seen_tokens
        position_ids = torch.arange(start, start + n, device=self.device)[None, :].expand(B, n)
        h = x.to(self.device, torch.float32)
        for i in range(self.n_layers):
            h = self._layer(i, h, position_ids, cache, fwd_no)
        return h, cache
