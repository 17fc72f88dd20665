"""Host-side mirror of the reference's ``modeling`` package for the decode-time selection path:
the same class and function names, constructor arguments and config keys
(modeling/omnikv.py, modeling/spec_cache.py, modeling/omnikv_config.py of antgroup/OmniKV)."""
from .omnikv_config import LlamaCompressorConfig  # noqa: F401
from .spec_cache import OmniKVLazyCache, OmniKVMultiStageCache, WOPackCache, get_cache_cls  # noqa: F401
from .omnikv import OmniKVMulLayer, OmniKVMulLM, OmniKVMulModel, select_tokens_by_attn_universal  # noqa: F401
