"""KV-head tensor parallelism: one process per GPU, ``torch.distributed`` over NCCL (NVLink / NVSwitch).

Each rank owns ``KVH / world`` KV heads, the ``H / world`` query heads of their groups, the matching
rows of the fused QKV weight and columns of the output projection, a slice of the MLP's intermediate
dimension and a slice of the vocabulary.  KV cache, scoring, gather and attention are per KV head and
need no communication.  The exchanges of a decode step are:

* ``all_reduce(SUM)`` of the hidden state after the output projection and after the MLP (as the
  reference's LightLLM fork, lightllm/common/basemodel/layer_infer/template/
  transformer_layer_infer_template.py:119-120, :128-129);
* ``all_reduce(MAX)`` of the filter layer's fp32 score planes before the top-k.  The reference has no
  such step -- its fork selects per rank from the local heads only
  (lightllm/models/llama_omnikv/triton_kernel/flash_decoding.py:76) -- but the selector is defined as a
  max over ALL heads, and MAX is order independent, so after it every rank holds bit-identical planes
  and runs the same deterministic top-k: no index broadcast is needed;
* ``all_gather`` of the vocabulary-sharded logits.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


class TPGroup:
    def __init__(self, world: int, rank: int, group=None):
        self.world, self.rank, self.group = world, rank, group

    def shard(self, n: int) -> Tuple[int, int]:
        """[lo, hi) of this rank's contiguous share of ``n`` items (``n`` divisible by the world size)."""
        if n % self.world:
            raise ValueError(f"{n} is not divisible by the tensor-parallel size {self.world}")
        per = n // self.world
        return self.rank * per, (self.rank + 1) * per

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def all_reduce_max(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return t

    def all_gather_last(self, t: torch.Tensor) -> torch.Tensor:
        """Concatenate the ranks' tensors along the last dimension."""
        if self.world == 1:
            return t
        parts = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)


def init(world: int, rank: int, device: Optional[torch.device] = None, backend: Optional[str] = None) -> TPGroup:
    """Join the process group described by the environment (MASTER_ADDR / MASTER_PORT, as torchrun sets
    them) and return the tensor-parallel group spanning every rank."""
    if not dist.is_initialized():
        backend = backend or ("nccl" if device is not None and device.type == "cuda" else "gloo")
        kw = {}
        if backend == "nccl":
            kw["device_id"] = device
        dist.init_process_group(backend=backend, world_size=world, rank=rank, **kw)
    return TPGroup(world, rank, None)
