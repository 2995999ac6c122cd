"""Decode steps of a ``LlamaSmartKV`` model as CUDA graphs (no counterpart in the reference).

A decode step through the Hugging Face modules is about forty small kernels per layer launched from Python, plus
the cache's two; on a B200 the launches, not the kernels, set the step time.  Everything a step does on the
device is a function of device-resident state (token ids, positions, the cache's counters and per-token
arrays), and which layers reallocate in a step follows from the cache's host counters alone
(``BatchedSmartKVCache.next_step_triggers``).  So one graph per distinct set of trigger layers can be captured the
first time that set occurs and replayed afterwards with new inputs.

Only the multi-sequence cache with ``key_attribution="keys"`` is supported (the parity mode does host arithmetic
per layer).  The first steps after a prompt run eagerly, so that every lazily created buffer exists before the
first capture."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..core.batched_cache import BatchedSmartKVCache


class GraphedDecoder:
    def __init__(self, wrapped, eager_steps: int = 2):
        self.wrapped = wrapped
        self.eager_steps = int(eager_steps)
        self._graphs: Dict[Tuple[int, ...], torch.cuda.CUDAGraph] = {}
        self._logits: Dict[Tuple[int, ...], torch.Tensor] = {}
        self._ids = None
        self._pos = None
        self._zero_mask = None
        self._steps_since_prompt = 0

    def reset(self):
        """Call after every prompt pass / cache reset."""
        self._steps_since_prompt = 0

    def _forward(self):
        # A 4-D mask is passed through by the model as it is, which keeps its mask construction (host scalars copied to
        # the device, not allowed under capture) out of the step; the cache's attention never reads it.
        out = self.wrapped(input_ids=self._ids, position_ids=self._pos, attention_mask=self._zero_mask, use_cache=False)
        return out.logits[:, -1]

    def step(self, tokens: torch.Tensor, position: int) -> torch.Tensor:
        """tokens int64 [B] on the device: the token every sequence feeds; ``position``: its position id.
        Returns the logits [B, vocab] of the step (a buffer the decoder owns; read it before the next call)."""
        cache = self.wrapped.smartkv_cache
        if not isinstance(cache, BatchedSmartKVCache) or cache.key_attribution != "keys":
            raise RuntimeError("GraphedDecoder needs the multi-sequence cache with key_attribution='keys'")
        B = tokens.shape[0]
        if self._ids is None or self._ids.shape[0] != B:
            self._ids = torch.zeros((B, 1), dtype=torch.int64, device=tokens.device)
            self._pos = torch.zeros((B, 1), dtype=torch.int64, device=tokens.device)
            dtype = next(self.wrapped.model.parameters()).dtype
            self._zero_mask = torch.zeros((B, 1, 1, 1), dtype=dtype, device=tokens.device)
            self._graphs.clear()
            self._logits.clear()
        self._ids.copy_(tokens.view(B, 1))
        self._pos.fill_(int(position))
        self._steps_since_prompt += 1
        if self._steps_since_prompt <= self.eager_steps:
            with torch.no_grad():
                return self._forward()
        key = cache.next_step_triggers()
        graph = self._graphs.get(key)
        if graph is None:
            # capturing runs the host side of the step (counters advance as if it had run) but nothing on the device
            torch.cuda.synchronize(tokens.device)
            graph = torch.cuda.CUDAGraph()
            cache.store.capture_updates()
            with torch.no_grad(), torch.cuda.graph(graph):
                logits = self._forward()
            if cache.store.capture_updates() % 2:
                raise RuntimeError("a decode step of this model holds an odd number of importance updates (odd layer "
                                   "count); its steps cannot be replayed as graphs")
            self._graphs[key] = graph
            self._logits[key] = logits
            graph.replay()
            return logits
        graph.replay()
        cache.advance_after_replay(key)
        return self._logits[key]
