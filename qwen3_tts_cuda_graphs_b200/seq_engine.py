"""Step function of the sequence models: requests in slots, steps of any number of tokens, logits of chosen positions.

`SequenceEngine.step(request, tokens, want)` runs `tokens` (the request's next tokens, any count: a prompt, a portion of one,
a single decoded token) through the model from the state earlier steps left in the request's slot and returns the logits at the
positions `want` (indices into `tokens`).  A step is one op list (seq_ops.StepBuilder) on libfq3codec.so: lists are cached per
(slot, token count) and replay as CUDA graphs from their second use; positions are read on the device from the slot's counter, so
a cached list serves any position.  Generation (`generate`, serving.TokenScheduler) drives the same step and samples with the
framework's sampler (sampling.sample_logits).
"""
from __future__ import annotations

import importlib
import json
import os
from collections import OrderedDict
from typing import Dict, Iterable, List, Optional, Sequence

import torch

from . import codec as _codec
from .config import SEQUENCE_ARCHITECTURES, sequence_config_from_dict
from .seq_ops import StepBuilder
from .seq_state import SequenceStateManager, SlotState


def model_class(architecture: str):
    mod, cls = SEQUENCE_ARCHITECTURES[architecture][1].split(":")
    return getattr(importlib.import_module(f"{__package__}.{mod}"), cls)


class SequenceEngine:
    MAX_PLANS = 64

    def __init__(self, model, max_tokens: int, max_slots: int = 1, use_graphs: Optional[bool] = None):
        self.model = model
        self.device = model.device
        if self.device.type != "cuda":
            raise ValueError("sequence models run on CUDA only (no CPU fallback)")
        self.lib = _codec.load_lib()
        self.f32 = model.f32
        self.use_graphs = (os.environ.get("FQ3C_GRAPH", "1") != "0") if use_graphs is None else use_graphs
        self.states = SequenceStateManager(model.state_specs(), max_tokens, self.device, max_slots)
        self._steps: "OrderedDict[tuple, dict]" = OrderedDict()
        self._heads: "OrderedDict[tuple, dict]" = OrderedDict()

    # ---- loading ----------------------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, path: str, device="cuda", dtype: str = "bfloat16", max_tokens: int = 4096, max_slots: int = 1):
        """A directory with config.json ("architecture" picks the model class) and *.safetensors."""
        from .checkpoint import TensorDir

        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be bfloat16 or float32")
        with open(os.path.join(path, "config.json")) as f:
            raw = json.load(f)
        cfg = sequence_config_from_dict(raw)
        td = TensorDir(path)
        try:
            model = model_class(raw["architecture"])(cfg, lambda n: td.get(n) if n in td else None, device, f32=dtype == "float32")
        finally:
            td.close()
        return cls(model, max_tokens, max_slots)

    # ---- requests ---------------------------------------------------------------------------------
    def open(self, request) -> SlotState:
        return self.states.acquire(request)

    def close(self, request) -> None:
        self.states.release(request)

    # ---- plans ------------------------------------------------------------------------------------
    def _step_plan(self, slot: SlotState, M: int, taps: bool = False) -> dict:
        key = (slot.index, M, taps)
        e = self._steps.get(key)
        if e is None:
            b = StepBuilder(self.device, M, slot, self.f32)
            ids = torch.zeros(M, dtype=torch.int32, device=self.device)
            b.plan.keep.append(ids)
            layer_taps = [] if taps else None
            x = self.model.build_step(b, ids, layer_taps)
            e = {"plan": b.finish(), "ids": ids, "x": x, "taps": layer_taps}
            self._steps[key] = e
            while len(self._steps) > self.MAX_PLANS:
                old_key, old = self._steps.popitem(last=False)
                self._drop(old["plan"])
                for hk in [k for k in self._heads if k[:3] == old_key]:
                    self._drop(self._heads.pop(hk)["plan"])
        else:
            self._steps.move_to_end(key)
        return e

    def _head_plan(self, slot: SlotState, M: int, taps: bool, n_want: int, x: torch.Tensor) -> dict:
        key = (slot.index, M, taps, n_want)
        e = self._heads.get(key)
        if e is None:
            b = StepBuilder(self.device, n_want, slot, self.f32)
            want = torch.zeros(n_want, dtype=torch.int32, device=self.device)
            b.plan.keep.append(want)
            logits = self.model.build_head(b, x, want)
            e = {"plan": b.finish(), "want": want, "logits": logits}
            self._heads[key] = e
        return e

    def _drop(self, plan):
        if getattr(plan, "graph", None) is not None:
            self.lib.fq3c_graph_destroy(plan.graph)
            plan.graph = None

    # ---- the step ---------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, request, tokens: Sequence[int], want: Sequence[int] = (), layer_taps: bool = False) -> Optional[torch.Tensor]:
        """Returns logits f32 [len(want), vocab] on the device (a buffer of the cached list: copy it before the next step of the
        same shape), or None when nothing is wanted.  With layer_taps the residual stream after every layer is kept in
        `self.last_taps` (list of f32 [M, width])."""
        slot = self.states.get(request) or self.open(request)
        M = len(tokens)
        if M == 0:
            return None
        if min(tokens) < 0 or max(tokens) >= self.model.vocab:
            raise ValueError("token id outside the vocabulary")
        if any(w < 0 or w >= M for w in want):
            raise ValueError("wanted position outside the step")
        self.states.reserve(slot, M)
        e = self._step_plan(slot, M, layer_taps)
        # from pageable memory: the copy is staged before the call returns, so the host list may change at once
        e["ids"].copy_(torch.as_tensor(list(tokens), dtype=torch.int32))
        _codec.run_op_plan(self.lib, e["plan"], self.use_graphs)
        self.last_taps = e["taps"]
        if not want:
            return None
        h = self._head_plan(slot, M, layer_taps, len(want), e["x"])
        h["want"].copy_(torch.as_tensor(list(want), dtype=torch.int32))
        _codec.run_op_plan(self.lib, h["plan"], self.use_graphs)
        return h["logits"]

    # ---- generation ---------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, tokens: Sequence[int], max_new_tokens: int, *, do_sample: bool = False, temperature: float = 1.0, top_k: int = 0,
                 top_p: float = 1.0, eos_id: Optional[int] = None, seed: int = 0, prefill_chunk: int = 0, request="generate") -> List[int]:
        """Prompt (optionally in portions of `prefill_chunk` tokens), then token-by-token decoding with the framework's sampler."""
        from .sampling import sample_logits

        self.open(request)
        try:
            toks = list(tokens)
            chunk = prefill_chunk if prefill_chunk > 0 else len(toks)
            logits = None
            for lo in range(0, len(toks), chunk):
                part = toks[lo:lo + chunk]
                logits = self.step(request, part, [len(part) - 1] if lo + chunk >= len(toks) else [])
            out: List[int] = []
            for i in range(max_new_tokens):
                t = int(sample_logits(logits[0], temperature=temperature, top_k=top_k, top_p=top_p, do_sample=do_sample,
                                      seed=seed, draw_index=i, engine=False))
                out.append(t)
                if eos_id is not None and t == eos_id:
                    break
                if i + 1 < max_new_tokens:
                    logits = self.step(request, [t], [0])
            return out
        finally:
            self.close(request)

    def close_all(self):
        for e in list(self._steps.values()) + list(self._heads.values()):
            self._drop(e["plan"])
        self._steps.clear()
        self._heads.clear()
