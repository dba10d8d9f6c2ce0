"""Greedy decode loop around `TrimKVQwen3ForCausalLM` + `TrimKVCache`, optionally as a CUDA graph.

The reference decodes through HF ``generate`` (one Python-dispatched forward per token,
examples/test_qwen3.py:51).  Here the per-token forward (all layers: gate -> RoPE -> append ->
decode attention, then LM head and argmax) can be captured once in a CUDA graph and replayed; the
eviction (`cache.compress`) stays outside the graph because the host decides when it fires.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops
from .cache_utils import TrimKVCache


class GreedyDecoder:
    """Steps a prefilled (model, cache) pair one token at a time.

    ``step(ids)``: ``ids`` is ``[B,1]`` int64 on the host (pinned) or device, or None to feed back the
    previous step's argmax without leaving the device.  Returns the device tensor holding the new ids.
    """

    def __init__(self, model, cache: TrimKVCache, use_graph: bool = True):
        self.model, self.cache, self.cfg = model, cache, model.config
        dev = model.device
        self.batch = cache._batch
        self.ids = torch.zeros(self.batch, 1, dtype=torch.int64, device=dev)
        self.next_ids = torch.zeros(self.batch, 1, dtype=torch.int64, device=dev)
        self.pos = torch.full((1,), cache.get_seq_length(), dtype=torch.int64, device=dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.use_graph = use_graph

    def _forward(self):
        cfg = self.cfg
        compress, cfg.compress_memory = cfg.compress_memory, False  # eviction is driven from step()
        try:
            out = self.model(input_ids=self.ids, past_key_values=self.cache, cache_position=self.pos,
                             logits_to_keep=1)
        finally:
            cfg.compress_memory = compress
        self.next_ids.copy_(out.logits[:, -1].argmax(-1, keepdim=True))
        self.ids.copy_(self.next_ids)
        self.pos.add_(1)

    def _counters(self):
        c = self.cache
        return (c._seen_tokens, list(c.n_seen_tokens), list(c._cache_len))

    def _restore(self, snap):
        c = self.cache
        c._seen_tokens, c.n_seen_tokens, c._cache_len = snap[0], list(snap[1]), list(snap[2])

    def capture(self):
        """Records one decode step.  Views handed to attention span the full capacity so the recorded
        launch geometry is valid for every later length; the kernels read the live lengths on the device."""
        self.cache.static_views = True
        snap = self._counters()
        self.graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        with torch.cuda.graph(self.graph):
            self._forward()
        self.launches_per_replay = ops.launch_count - before
        ops.launch_count = before
        self._restore(snap)

    def step(self, ids: Optional[torch.Tensor] = None, eager: bool = False) -> torch.Tensor:
        if ids is not None:
            self.ids.copy_(ids, non_blocking=True)
        if self.use_graph and not eager:
            if self.graph is None:
                self.capture()
            self.graph.replay()
            ops.launch_count += self.launches_per_replay
            self.cache.advance(1)
        else:
            self._forward()
        if self.cfg.compress_memory:
            self.cache.compress(
                strategy=self.cfg.compress_strategy, memory_size=self.cfg.memory_size, buffer_size=self.cfg.buffer_size,
                num_layers=self.cfg.num_hidden_layers, num_key_value_heads=self.cfg.num_key_value_heads)
        return self.next_ids
