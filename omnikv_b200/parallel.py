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

At batch 1 the two SUM all-reduces per layer are latency, not bandwidth (8 KB of hidden state): with
``PeerExchange`` they are fused into the weight-streaming kernels on both sides -- the projection kernel
stores its partial sums straight into every rank's peer-mapped buffer over NVLink and raises a flag, the next
kernel waits for the flags (bounded) and adds the partials while it loads its activations
(``omnikv_tp_exchange`` in the C header).  With ``enable_peer_reduce`` the score planes (MAX) and the logits
(all-gather) travel through one-hop peer-memory kernels as well; NCCL is the fallback for anything that does not fit.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


class PeerExchange:
    """Peer-mapped exchange buffers of the fused projection + all-reduce kernels (one per process)."""

    def __init__(self, world: int, rank: int, hidden: int, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm

        from . import abi
        self.world, self.rank, self.hidden = world, rank, hidden
        nbytes = abi.lib().omnikv_tp_exchange_bytes(hidden)
        self.buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        grp = group if group is not None else dist.group.WORLD
        try:
            self.handle = symm.rendezvous(self.buf, grp)
        except Exception:
            symm.enable_symm_mem_for_group(grp.group_name)
            self.handle = symm.rendezvous(self.buf, grp)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.done = torch.zeros(2, dtype=torch.int32, device=device)  # [finished CTAs, calls made]
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self._structs = {}
        dist.barrier(group=group)  # every rank's buffer is zeroed and mapped before anyone stores into it

    def begin_step(self) -> None:
        """Once per decode step on every rank (graph-capturable): flags carry the step number."""
        self.epoch.add_(1)

    def at(self, seq: int):
        """The ``omnikv_tp_exchange`` describing exchange number ``seq`` of the step."""
        from . import abi
        x = self._structs.get(seq)
        if x is None:
            x = abi.TpExchange()
            x.world, x.rank, x.seq, x.hidden = self.world, self.rank, seq, self.hidden
            for r, ptr in enumerate(self.peer_ptrs):
                x.peer_base[r] = ptr
            x.done_counter, x.epoch = self.done.data_ptr(), self.epoch.data_ptr()
            self._structs[seq] = x
        return x


class TPGroup:
    def __init__(self, world: int, rank: int, group=None):
        self.world, self.rank, self.group = world, rank, group
        self.exchange: Optional[PeerExchange] = None   # fused projection + all-reduce (batch-1 decode kernels)
        self.reducer: Optional[PeerExchange] = None    # standalone small all-reduce (batched decode)
        self.peer_reduce_calls = 0                     # all_reduce_sum calls served by the peer-memory kernel

    def enable_peer_exchange(self, hidden: int, device: torch.device) -> bool:
        """Set up the peer-mapped buffers for the fused projection + all-reduce kernels.  Returns False (and
        keeps NCCL all-reduces) when symmetric memory cannot be set up on this machine."""
        if self.world <= 1 or self.world > 8:
            return False
        try:
            self.exchange = PeerExchange(self.world, self.rank, hidden, device, self.group)
        except Exception as e:  # no peer access between the GPUs, or no symmetric-memory support
            import logging
            logging.getLogger("omnikv_b200").warning(f"peer exchange unavailable, using NCCL all-reduce: {e}")
            self.exchange = None
        ok = torch.tensor([1 if self.exchange is not None else 0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            self.exchange = None
        return self.exchange is not None

    def enable_peer_reduce(self, max_bytes: int, device: torch.device) -> bool:
        """Set up a second set of peer-mapped buffers for ``all_reduce_sum`` of tensors up to ``max_bytes`` (the
        hidden state of a batched decode step): one NVLink hop and a rank-ordered fp32 sum instead of a NCCL
        ring.  Returns False (NCCL stays) when symmetric memory cannot be set up."""
        if self.world <= 1 or self.world > 8:
            return False
        try:
            self.reducer = PeerExchange(self.world, self.rank, -(-max_bytes // 64) * 16, device, self.group)
        except Exception as e:
            import logging
            logging.getLogger("omnikv_b200").warning(f"peer all-reduce unavailable, using NCCL: {e}")
            self.reducer = None
        ok = torch.tensor([1 if self.reducer is not None else 0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            self.reducer = None
        return self.reducer is not None

    def begin_step(self) -> None:
        """Once per model forward on every rank.  The peer all-reduce numbers its calls on the device, so it has
        nothing to reset here; this is the hook where per-step state of the group would go."""

    def shard(self, n: int) -> Tuple[int, int]:
        """[lo, hi) of this rank's contiguous share of ``n`` items (``n`` divisible by the world size)."""
        if n % self.world:
            raise ValueError(f"{n} is not divisible by the tensor-parallel size {self.world}")
        per = n // self.world
        return self.rank * per, (self.rank + 1) * per

    def all_reduce_sum(self, t: torch.Tensor) -> torch.Tensor:
        if self.world <= 1:
            return t
        r = self.reducer
        nbytes = t.numel() * t.element_size()
        # every condition depends on shapes and call order only, so all ranks take the same branch
        if (r is not None and t.is_cuda and t.is_contiguous() and nbytes % 16 == 0 and nbytes <= r.hidden * 4
                and t.dtype in (torch.bfloat16, torch.float16, torch.float32)):
            from . import ops
            ops.tp_allreduce_sum(t, r.at(0))
            self.peer_reduce_calls += 1
            return t
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def _peer_fits(self, t: torch.Tensor) -> bool:
        """Whether ``t`` goes through the peer-memory kernels (depends on shapes only: all ranks agree)."""
        r = self.reducer
        nbytes = t.numel() * t.element_size()
        return (r is not None and t.is_cuda and t.is_contiguous() and nbytes % 16 == 0 and 0 < nbytes <= r.hidden * 4
                and t.dtype in (torch.bfloat16, torch.float16, torch.float32))

    def all_reduce_max(self, t: torch.Tensor) -> torch.Tensor:
        if self.world <= 1:
            return t
        if t.dtype == torch.float32 and self._peer_fits(t):
            from . import ops
            ops.tp_allreduce_max(t, self.reducer.at(0))
            self.peer_reduce_calls += 1
            return t
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return t

    def all_gather_last(self, t: torch.Tensor) -> torch.Tensor:
        """Concatenate the ranks' tensors along the last dimension."""
        if self.world == 1:
            return t
        if t.numel() == t.shape[-1] and self._peer_fits(t.contiguous()):  # one row: the ranks' rows back to back
            from . import ops
            out = ops.tp_allgather(t.contiguous(), self.reducer.at(0), self.world)
            self.peer_reduce_calls += 1
            return out.view(*t.shape[:-1], self.world * t.shape[-1])
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
