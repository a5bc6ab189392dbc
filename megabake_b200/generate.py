"""Greedy generation on one GPU: one compiled prefill that seeds the explicit KV state, then one
compiled decode call per token.

The counterpart of the reference's ``examples/single_gpu_generate.py`` -- which has to feed the
prompt through its decode step token by token because its prefill cannot seed the decode state
(``examples/single_gpu_generate.py:3-4``).  Here ``StatefulPrefill`` writes the prompt's keys and
values into the caches that ``StatefulDecoder`` appends to.
"""

from __future__ import annotations

import torch

from .frontend import make_backend
from .hf import StatefulDecoder, StatefulPrefill


class GreedyGenerator:
    """Compiles the two wrappers once for a (batch, prompt length, capacity) and reuses them."""

    def __init__(self, model: torch.nn.Module, batch: int, prompt_tokens: int, capacity: int):
        if capacity <= prompt_tokens:
            raise ValueError("capacity must exceed the prompt length")
        self.batch, self.prompt_tokens, self.capacity = batch, prompt_tokens, capacity
        self.device = next(model.parameters()).device
        prefill = StatefulPrefill(model, capacity).eval()
        decode = StatefulDecoder(model, capacity).eval()
        self.state = prefill.make_state(batch, device=self.device)
        self.prefill_backend = make_backend(mode="prefill")
        self.decode_backend = make_backend(mode="decode")
        self._prefill = torch.compile(prefill, backend=self.prefill_backend, fullgraph=True,
                                      dynamic=False)
        self._decode = torch.compile(decode, backend=self.decode_backend, fullgraph=True,
                                     dynamic=False)

    @torch.no_grad()
    def __call__(self, input_ids: torch.Tensor, new_tokens: int) -> torch.Tensor:
        """``input_ids`` ``[batch, prompt_tokens]`` -> generated ids ``[batch, new_tokens]``."""
        if tuple(input_ids.shape) != (self.batch, self.prompt_tokens):
            raise ValueError("this generator was compiled for another prompt shape")
        if self.prompt_tokens + new_tokens > self.capacity:
            raise ValueError("the KV capacity cannot hold the prompt plus the new tokens")
        logits = self._prefill(input_ids.to(self.device), *self.state)
        token = logits[:, -1].float().argmax(-1, keepdim=True)
        produced = [token]
        position = torch.full((self.batch, 1), self.prompt_tokens, dtype=torch.int64,
                              device=self.device)
        for _ in range(new_tokens - 1):
            logits = self._decode(token, position, *self.state)
            token = logits[:, -1].float().argmax(-1, keepdim=True)
            produced.append(token)
            position = position + 1
        for backend in (self.prefill_backend, self.decode_backend):
            if backend.megabake_last_callable is not None:
                backend.megabake_last_callable.check()
        return torch.cat(produced, dim=1)
