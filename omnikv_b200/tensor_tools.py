"""Recorder of the token indices the filter layers select, for choosing filter layers offline.

Mirrors the recorder of the reference (tiny_tools/tensor_tools.py:38-98: ``SelectedIndexTracer``,
``read_idx_tracer``, the module-level ``idx_tracer`` that exists when the environment variable
``SAVE_SELECTED_IDX`` is set) and writes the same pickle, so the reference's analysis scripts
(tiny_runs/ana_motivation2.py:103,137) read files made here:

    {"idx": {sample: [{"idx", "value"}, ...]}, "out": [...],
     "layers_idx": {sample: {layer: [{"idx", "value", "prefill_len"}, ...]}}, "prefill_res": {sample: {...}}}

``OmniKVMulLayer`` calls ``append_spec_layer`` after every decode-time selection while a tracer is active
(the reference wires its tracer into its older single-filter model only, modeling/offload_select_once.py:90).
Recording copies the index list to the host each step, so decode then runs without CUDA-graph capture.
"""
from __future__ import annotations

import os
import pickle
from typing import Any, Dict, List, Optional

import torch


class SelectedIndexTracer:
    def __init__(self, desc: Optional[str] = None, directory: str = "debug_logs"):
        desc = os.environ.get("SAVE_SELECTED_IDX") if desc is None else desc
        self.save_path = os.path.join(directory, f"selected_index_{desc}.pkl")
        self.idx: Dict[int, List[Dict[str, torch.Tensor]]] = {}
        self.layers_idx: Dict[int, Dict[int, List[Dict[str, Any]]]] = {}
        self.prefill_res: Dict[int, Dict[str, torch.Tensor]] = {}
        self.outs: List[Any] = []
        self.num_samples = 0

    @staticmethod
    def _host(t: torch.Tensor) -> torch.Tensor:
        return t.detach().to(device="cpu", non_blocking=True)

    def append_out(self, out) -> None:
        self.outs.append(out)

    def append(self, idx: torch.Tensor, v: torch.Tensor) -> None:
        self.idx.setdefault(self.num_samples, []).append({"idx": self._host(idx), "value": self._host(v)})

    def append_prefill(self, idx: torch.Tensor, v: torch.Tensor, layer_idx: int) -> None:
        self.prefill_res[self.num_samples] = {"idx": idx.detach().cpu(), "value": v.detach().cpu()}

    def append_spec_layer(self, idx: torch.Tensor, v: torch.Tensor, prefill_len: int, layer_idx: int) -> None:
        if idx.dim() != 2 or v.dim() != 2:
            raise AssertionError("idx and value must be [batch, k]")
        per_layer = self.layers_idx.setdefault(self.num_samples, {}).setdefault(int(layer_idx), [])
        per_layer.append({"idx": self._host(idx), "value": self._host(v), "prefill_len": prefill_len})

    def save_idx(self) -> None:
        """Write everything recorded so far and move on to the next sample."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()  # the non-blocking copies above have landed
        os.makedirs(os.path.dirname(self.save_path) or ".", exist_ok=True)
        with open(self.save_path, "wb") as f:
            pickle.dump({"idx": self.idx, "out": self.outs, "layers_idx": self.layers_idx,
                         "prefill_res": self.prefill_res}, f)
        self.num_samples += 1


def read_idx_tracer(pkl_path: str):
    """-> (idx, out, layers_idx, prefill_res), as the reference's reader."""
    with open(pkl_path, "rb") as f:
        d = pickle.load(f)
    return d["idx"], d["out"], d["layers_idx"], d["prefill_res"]


idx_tracer: Optional[SelectedIndexTracer] = SelectedIndexTracer() if os.environ.get("SAVE_SELECTED_IDX") else None


def set_tracer(tracer: Optional[SelectedIndexTracer]) -> Optional[SelectedIndexTracer]:
    """Install (or remove, with None) the active tracer; returns the previous one."""
    global idx_tracer
    prev, idx_tracer = idx_tracer, tracer
    return prev
