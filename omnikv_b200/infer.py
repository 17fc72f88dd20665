"""``get_any_chat_api``: the reference's model factory (infer.py:358-373, :192-287) for ``model_cls = "multi"``.

Reads the experiment JSON, builds the config (every JSON key becomes a config attribute), loads the Llama
checkpoint named by ``model_name`` into ``OmniKVMulLM`` and returns
``(chat, tokenizer, max_context_len, {"eos_token_id": ...})`` where
``chat(prompt, generation_config=None, skip_special_tokens=False, **kw) -> str``.

What the reference delegates to third-party code -- the tokenizer, chat templates and ``generate`` of
transformers -- is kept out of this package: the tokenizer comes from ``transformers.AutoTokenizer`` when
it is installed (or is passed in), and generation is the package's own greedy / top-p loop.
Batch 1, like the reference's ``inference_bs1``.
"""
from __future__ import annotations

import json
import time
from typing import Optional

import torch

from .modeling import LlamaCompressorConfig, OmniKVMulLM
from .modeling.omnikv_config import logger


def read_config(path: str) -> dict:
    with open(path) as f:
        return json.load(f)


def _sample(logits: torch.Tensor, temperature: float, top_p: float, generator=None) -> torch.Tensor:
    """Nucleus sampling of one token per row from fp32 logits ``[B, vocab]``."""
    probs = torch.softmax(logits / max(temperature, 1e-6), dim=-1)
    sp, si = torch.sort(probs, dim=-1, descending=True)
    keep = (torch.cumsum(sp, dim=-1) - sp) < top_p
    sp = torch.where(keep, sp, torch.zeros_like(sp))
    pick = torch.multinomial(sp / sp.sum(dim=-1, keepdim=True), 1, generator=generator)
    return si.gather(-1, pick)


def get_any_chat_api(cfg_path: str, tokenizer=None, model: Optional[OmniKVMulLM] = None, device: str = "cuda:0"):
    cfg = read_config(cfg_path)
    torch.set_num_threads(cfg.get("cpu_num_threads", 12))
    model_cls = cfg["model_cls"]
    if model_cls != "multi":
        raise NotImplementedError(f"model_cls={model_cls!r}: only 'multi' (OmniKVMulLM) is implemented")
    if cfg.get("load_in_8bit") or cfg.get("load_in_4bit"):
        raise NotImplementedError("bitsandbytes quantisation is not part of this package")
    model_name = cfg["model_name"]
    if model is None:
        config = LlamaCompressorConfig.from_pretrained(model_name)
        config.set_config(**cfg)
        model = OmniKVMulLM.from_pretrained(model_name, config=config, torch_dtype=torch.float16, device=device)
    else:
        model.config.set_config(**cfg)
    config = model.config
    if tokenizer is None:
        from transformers import AutoTokenizer  # third-party, as in the reference
        tokenizer = AutoTokenizer.from_pretrained(model_name)
    if cfg.get("cot", False) and not cfg.get("use_chat_template", False):
        raise AssertionError("cot needs use_chat_template")
    eos = [config.eos_token_id] if isinstance(config.eos_token_id, int) else list(config.eos_token_id or [])

    @torch.no_grad()
    def chat(prompt, generation_config=None, skip_special_tokens=False, **kwargs):
        st = time.time()
        ids = tokenizer(prompt, return_tensors="pt")["input_ids"].to(model.lm_head.weight.device)
        gc = generation_config
        max_new = int(getattr(gc, "max_new_tokens", None) or kwargs.get("max_new_tokens", 128))
        do_sample = bool(getattr(gc, "do_sample", False))
        if not do_sample:
            out = model.generate_greedy(ids, max_new, use_cuda_graph=ids.shape[0] == 1)
        else:
            res = model(input_ids=ids)
            cache, toks = res.past_key_values, []
            for _ in range(max_new):
                tok = _sample(res.logits[:, -1], float(getattr(gc, "temperature", 1.0)), float(getattr(gc, "top_p", 1.0)))
                toks.append(tok)
                if int(tok[0, 0]) in eos:
                    break
                res = model(input_ids=tok, past_key_values=cache)
            out = torch.cat(toks, dim=1)
        row = out[0].tolist()
        for i, t in enumerate(row):  # cut at the first end-of-sequence token
            if t in eos:
                row = row[:i]
                break
        text = tokenizer.batch_decode([row], skip_special_tokens=skip_special_tokens,
                                      clean_up_tokenization_spaces=False)[0]
        logger.info(f"--- chat time: {round(time.time() - st, 3)}s")
        return text

    return chat, tokenizer, config.get("max_context_len", 100_000), {"eos_token_id": config.eos_token_id}
