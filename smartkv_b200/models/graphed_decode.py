"""Decode steps over the multi-sequence cache as CUDA graphs (no counterpart in the reference).

A decode step through the Hugging Face modules is about forty small kernels per layer launched from Python, plus
the cache's two; on a B200 the launches, not the kernels, set the step time.  Everything a step does on the
device is a function of device-resident state (token ids, positions, the cache's counters and per-token
arrays), and which layers reallocate in a step follows from the cache's host counters alone
(``BatchedSmartKVCache.next_step_triggers``).  So one graph per distinct set of trigger layers is captured the
first time that set occurs and replayed afterwards with new inputs.

Only ``key_attribution="keys"`` is supported (the parity mode does host arithmetic per layer).  The first steps
after a prompt run eagerly, so that every lazily created buffer exists before the first capture."""
from __future__ import annotations

from typing import Callable, Dict, Tuple

import torch

from ..core.batched_cache import BatchedSmartKVCache


class GraphedDecoder:
    """``forward(ids, pos)``: runs one decode step for token ids ``ids`` int64 [B, 1] at positions ``pos`` int64 [B, 1]
    (both static device buffers owned by the decoder) through every layer of ``cache`` in order and returns the
    step's result tensor.  ``GraphedDecoder.for_model(wrapped)`` builds that function for a ``LlamaSmartKV``."""

    def __init__(self, forward: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], cache_of: Callable[[], object],
                 eager_steps: int = 2):
        self._forward = forward
        self._cache_of = cache_of
        self.eager_steps = int(eager_steps)
        self._graphs: Dict[Tuple[int, ...], torch.cuda.CUDAGraph] = {}
        self._results: Dict[Tuple[int, ...], torch.Tensor] = {}
        self._ids = None
        self._pos = None
        self._steps_since_prompt = 0

    @classmethod
    def for_model(cls, wrapped, eager_steps: int = 2) -> "GraphedDecoder":
        state = {}

        def forward(ids, pos):
            # A 4-D mask is passed through by the model as it is, which keeps its mask construction (host scalars
            # copied to the device, not allowed under capture) out of the step; the cache's attention never reads it.
            if state.get("mask") is None or state["mask"].shape[0] != ids.shape[0]:
                dtype = next(wrapped.model.parameters()).dtype
                state["mask"] = torch.zeros((ids.shape[0], 1, 1, 1), dtype=dtype, device=ids.device)
            return wrapped(input_ids=ids, position_ids=pos, attention_mask=state["mask"], use_cache=False).logits[:, -1]

        return cls(forward, lambda: wrapped.smartkv_cache, eager_steps)

    @property
    def graphs_captured(self) -> int:
        return len(self._graphs)

    def reset(self):
        """Call after every prompt pass / cache reset."""
        self._steps_since_prompt = 0

    def step(self, tokens: torch.Tensor, position: int) -> torch.Tensor:
        """tokens int64 [B] on the device: the token every sequence feeds; ``position``: its position id.
        Returns the step's result (for a model: logits [B, vocab]) in a buffer the decoder owns; read it before
        the next call."""
        cache = self._cache_of()
        if not isinstance(cache, BatchedSmartKVCache) or cache.key_attribution != "keys":
            raise RuntimeError("GraphedDecoder needs the multi-sequence cache with key_attribution='keys'")
        B = tokens.shape[0]
        if self._ids is None or self._ids.shape[0] != B:
            self._ids = torch.zeros((B, 1), dtype=torch.int64, device=tokens.device)
            self._pos = torch.zeros((B, 1), dtype=torch.int64, device=tokens.device)
            self._graphs.clear()
            self._results.clear()
        self._ids.copy_(tokens.view(B, 1))
        self._pos.fill_(int(position))
        self._steps_since_prompt += 1
        if self._steps_since_prompt <= self.eager_steps:
            with torch.no_grad():
                return self._forward(self._ids, self._pos)
        key = cache.next_step_triggers()
        graph = self._graphs.get(key)
        if graph is None:
            # capturing runs the host side of the step (counters advance as if it had run) but nothing on the device
            torch.cuda.synchronize(tokens.device)
            graph = torch.cuda.CUDAGraph()
            cache.store.capture_updates()
            with torch.no_grad(), torch.cuda.graph(graph):
                result = self._forward(self._ids, self._pos)
            if cache.store.capture_updates() % 2:
                raise RuntimeError("a decode step of this model holds an odd number of importance updates (odd layer "
                                   "count); its steps cannot be replayed as graphs")
            self._graphs[key] = graph
            self._results[key] = result
            graph.replay()
            return result
        graph.replay()
        cache.advance_after_replay(key)
        return self._results[key]
