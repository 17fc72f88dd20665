"""Import the REFERENCE's own modules (``modeling.omnikv``, ``modeling.spec_cache``) from a checkout, unchanged.

TEST INFRASTRUCTURE ONLY.  Used by the fixture generator (``tests/golden/make_golden.py``) and, when a checkout is
reachable (``OMNIKV_REFERENCE=/path/to/OmniKV``), by the CPU-baseline leg of ``bench.py`` to time the reference's
functions themselves instead of the restatement in this folder.  Nothing of the reference is copied.

The reference targets transformers 4.41.2; with a newer transformers the import needs these shims:

* its logger wants a git work tree with a ``debug_logs/`` folder as the current directory
  (tiny_tools/get_code_id.py:5-28, tiny_tools/log.py:46-49) -> a scratch repository under the temp dir is the
  current directory while importing;
* ``from transformers.models.llama.modeling_llama import *`` is expected to leak ``torch, math, nn, F, Cache,
  DynamicCache, ...`` -> those names are set on that module and its ``__all__`` widened before the import;
* ``Tensor.cuda`` is made the identity on a host without a GPU (modeling/spec_cache.py:298-303 calls it on the
  gathered rows); on a GPU host the CPU timing does the same, so that "the reference's CPU path" stays on the CPU.
"""
from __future__ import annotations

import math
import os
import subprocess
import sys
import tempfile

import torch


def reference_root() -> str | None:
    """The checkout named by OMNIKV_REFERENCE, if it is there."""
    root = os.environ.get("OMNIKV_REFERENCE")
    if root and os.path.isfile(os.path.join(root, "modeling", "omnikv.py")):
        return os.path.abspath(root)
    return None


def import_reference(ref_root: str, cuda_identity: bool = True):
    """(modeling.omnikv, modeling.spec_cache) of the checkout at ``ref_root``."""
    scratch = tempfile.mkdtemp(prefix="omnikv_ref_cwd_")
    os.makedirs(os.path.join(scratch, "debug_logs"))
    env = dict(os.environ, GIT_AUTHOR_NAME="g", GIT_AUTHOR_EMAIL="g@g", GIT_COMMITTER_NAME="g", GIT_COMMITTER_EMAIL="g@g")
    subprocess.check_call(["git", "init", "-q"], cwd=scratch)
    subprocess.check_call(["git", "commit", "-q", "--allow-empty", "-m", "scratch"], cwd=scratch, env=env)
    os.chdir(scratch)
    sys.path.insert(0, ref_root)

    import transformers  # noqa: F401
    import transformers.models.llama.modeling_llama as ml
    from typing import List, Optional, Tuple, Union
    from transformers.cache_utils import Cache, DynamicCache
    from transformers.modeling_outputs import CausalLMOutputWithPast
    from transformers.models.llama.configuration_llama import LlamaConfig

    leak = dict(
        LlamaConfig=LlamaConfig, math=math, F=torch.nn.functional, nn=torch.nn, torch=torch, Cache=Cache,
        DynamicCache=DynamicCache, CausalLMOutputWithPast=CausalLMOutputWithPast, Optional=Optional,
        Tuple=Tuple, Union=Union, List=List, CrossEntropyLoss=torch.nn.CrossEntropyLoss,
        LLAMA_ATTENTION_CLASSES={},
    )
    for k, v in leak.items():
        setattr(ml, k, v)
    ml.__all__ = [n for n in dir(ml) if not n.startswith("_")]
    if cuda_identity:
        torch.Tensor.cuda = lambda self, *a, **k: self

    import modeling.omnikv as ref_omnikv
    import modeling.spec_cache as ref_cache

    return ref_omnikv, ref_cache
