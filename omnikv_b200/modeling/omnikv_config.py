"""``LlamaCompressorConfig``: the reference's config object (modeling/omnikv_config.py:10-23).

Every key of the experiment JSON (configs/example.json) is set as an attribute by
``set_config_of_compressor(**json)`` and read everywhere through ``get(key, default)``, which
WRITES THE DEFAULT BACK when the key is missing (:15-19) -- later readers then see it.  The class
does not depend on ``transformers``; it carries the Llama architecture fields itself and can read a
Hugging Face ``config.json``.
"""
from __future__ import annotations

import json
import logging
import os

logger = logging.getLogger("omnikv_b200")

_LLAMA_DEFAULTS = dict(
    vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
    num_key_value_heads=8, hidden_act="silu", max_position_embeddings=8192, rms_norm_eps=1e-5, rope_theta=500000.0,
    rope_scaling=None, pad_token_id=None, bos_token_id=128000, eos_token_id=128001, pretraining_tp=1,
    tie_word_embeddings=False, attention_bias=False, mlp_bias=False, head_dim=None,
    output_attentions=False, output_hidden_states=False, use_return_dict=True,
)


class LlamaCompressorConfig:
    model_type = "llama"

    def __init__(self, **kwargs):
        for k, v in _LLAMA_DEFAULTS.items():
            setattr(self, k, v)
        for k, v in kwargs.items():
            setattr(self, k, v)
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads

    # -- the reference's three methods -------------------------------------------------------
    def set_config_of_compressor(self, **kwargs):
        for k, v in kwargs.items():
            setattr(self, k, v)

    set_config = set_config_of_compressor  # spelling used by infer.py:200 / modeling/token_model.py:74-76

    def get(self, key, default=None):
        if not hasattr(self, key):
            setattr(self, key, default)
            logger.warning(f"{key} is not set; using and storing the default {default}")
        return getattr(self, key, default)

    def _rope_scaling_validation(self):  # the reference disables HF's validation (:21-23)
        return

    # -- loading -----------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, path, **kwargs):
        cfg_file = os.path.join(path, "config.json") if os.path.isdir(path) else path
        with open(cfg_file) as f:
            d = json.load(f)
        d.update(kwargs)
        return cls(**d)

    @classmethod
    def llama3_8b(cls, **kwargs):
        return cls(**kwargs)

    @classmethod
    def llama3_70b(cls, **kwargs):
        d = dict(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80, num_attention_heads=64,
                 num_key_value_heads=8)
        d.update(kwargs)
        return cls(**d)

    def to_dict(self):
        return dict(self.__dict__)
