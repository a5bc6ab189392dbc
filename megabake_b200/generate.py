"""Greedy generation on one GPU: one compiled prefill that seeds the explicit KV state, then one
compiled decode call per token -- picked on the host (``__call__``) or, with no host work per
token at all, picked on the device inside a replayed CUDA graph (``on_device``).

The counterpart of the reference's ``examples/single_gpu_generate.py`` -- which has to feed the
prompt through its decode step token by token because its prefill cannot seed the decode state
(``examples/single_gpu_generate.py:3-4``).  Here ``StatefulPrefill`` writes the prompt's keys and
values into the caches that ``StatefulDecoder`` appends to.
"""

from __future__ import annotations

import torch

from . import runtime as rt
from .engine import graphed
from .frontend import make_backend
from .hf import StatefulDecoder, StatefulPrefill


class GreedyGenerator:
    """Compiles the two wrappers once for a (batch, prompt length, capacity) and reuses them."""

    def __init__(self, model: torch.nn.Module, batch: int, prompt_tokens: int, capacity: int,
                 per_row_lengths: bool = False):
        """``per_row_lengths``: every row keeps its own valid length, so that one batch can hold
        prompts of different lengths (``prompt_lengths`` of ``__call__``); ``prompt_tokens`` is
        then the padded prompt length the prefill is compiled for."""
        if capacity <= prompt_tokens:
            raise ValueError("capacity must exceed the prompt length")
        self.batch, self.prompt_tokens, self.capacity = batch, prompt_tokens, capacity
        self.per_row_lengths = per_row_lengths
        self.device = next(model.parameters()).device
        prefill = StatefulPrefill(model, capacity).eval()
        decode = StatefulDecoder(model, capacity).eval()
        self.state = prefill.make_state(batch, device=self.device, per_row_lengths=per_row_lengths)
        self.prefill_backend = make_backend(mode="prefill")
        self.decode_backend = make_backend(mode="decode")
        self._prefill = torch.compile(prefill, backend=self.prefill_backend, fullgraph=True,
                                      dynamic=False)
        self._decode = torch.compile(decode, backend=self.decode_backend, fullgraph=True,
                                     dynamic=False)

    @torch.no_grad()
    def __call__(self, input_ids: torch.Tensor, new_tokens: int,
                 prompt_lengths: torch.Tensor | None = None) -> torch.Tensor:
        """``input_ids`` ``[batch, prompt_tokens]`` -> generated ids ``[batch, new_tokens]``.

        ``prompt_lengths`` (int ``[batch]``, needs ``per_row_lengths``): the real length of every
        row's prompt; rows are padded at the end up to ``prompt_tokens`` with any valid id.  The
        causal prefill cannot see the padding from a real position; after it the valid lengths
        are set to the real lengths, so decode overwrites the padded rows of the caches and
        never attends to them."""
        if tuple(input_ids.shape) != (self.batch, self.prompt_tokens):
            raise ValueError("this generator was compiled for another prompt shape")
        if self.prompt_tokens + new_tokens > self.capacity:
            raise ValueError("the KV capacity cannot hold the prompt plus the new tokens")
        if prompt_lengths is not None and not self.per_row_lengths:
            raise ValueError("prompt_lengths needs a generator built with per_row_lengths=True")
        logits = self._prefill(input_ids.to(self.device), *self.state)
        if prompt_lengths is None:
            token = logits[:, -1].float().argmax(-1, keepdim=True)
            position = torch.full((self.batch, 1), self.prompt_tokens, dtype=torch.int64,
                                  device=self.device)
        else:
            lengths = prompt_lengths.to(self.device, torch.int64)
            if lengths.shape != (self.batch,) or int(lengths.min()) < 1 or \
                    int(lengths.max()) > self.prompt_tokens:
                raise ValueError("prompt_lengths must hold one length in 1..prompt_tokens per row")
            rows = torch.arange(self.batch, device=self.device)
            token = logits[rows, lengths - 1].float().argmax(-1, keepdim=True)
            position = lengths[:, None].clone()
            for index in range(2, len(self.state), 3):
                self.state[index].copy_(lengths.to(torch.int32))
        produced = [token]
        for _ in range(new_tokens - 1):
            logits = self._decode(token, position, *self.state)
            token = logits[:, -1].float().argmax(-1, keepdim=True)
            produced.append(token)
            position = position + 1
        for backend in (self.prefill_backend, self.decode_backend):
            if backend.megabake_last_callable is not None:
                backend.megabake_last_callable.check()
        return torch.cat(produced, dim=1)

    # -- the multi-step loop with the pick on the device ------------------------------------
    def _build_loop(self, steps_per_graph: int):
        """Capture ``steps_per_graph`` x (decode launch, greedy pick) in one CUDA graph.  The
        pick writes the next id into the very tensor the next decode launch reads and advances
        the positions, so a replay needs nothing from the host (the reference lists this loop
        as future work, ``docs/roadmap.md:180``)."""
        if 2 * steps_per_graph + 1 > self.capacity:
            raise ValueError("the KV capacity is too small to warm this many steps up")
        self._token = torch.zeros(self.batch, 1, dtype=torch.int64, device=self.device)
        self._position = torch.zeros(self.batch, 1, dtype=torch.int64, device=self.device)
        self._picked = torch.zeros(self.batch, self.capacity, dtype=torch.int64, device=self.device)
        self._cursor = torch.zeros(self.batch, dtype=torch.int32, device=self.device)
        for index in range(2, len(self.state), 3):
            self.state[index].zero_()  # the warm-up runs of the capture start from an empty cache

        def loop(token, position, *state):
            for _ in range(steps_per_graph):
                logits = self._decode(token, position, *state)
                rt.greedy_advance(logits, token, position, self._picked, self._cursor)
            return self._picked

        self._loop = graphed(loop, self._token, self._position, *self.state)
        self._loop_steps = steps_per_graph

    @torch.no_grad()
    def on_device(self, input_ids: torch.Tensor, new_tokens: int,
                  steps_per_graph: int = 1) -> torch.Tensor:
        """Same result as ``__call__``, but every token after the prompt is picked by
        ``mb_greedy_advance`` on the device and the decode steps run as replays of one CUDA
        graph holding ``steps_per_graph`` steps; the host reads the ids once, at the end.
        ``new_tokens - 1`` must be a multiple of ``steps_per_graph``."""
        if tuple(input_ids.shape) != (self.batch, self.prompt_tokens):
            raise ValueError("this generator was compiled for another prompt shape")
        if self.prompt_tokens + new_tokens > self.capacity:
            raise ValueError("the KV capacity cannot hold the prompt plus the new tokens")
        if steps_per_graph < 1 or (new_tokens - 1) % steps_per_graph:
            raise ValueError("new_tokens - 1 must be a multiple of steps_per_graph")
        if getattr(self, "_loop_steps", None) != steps_per_graph:
            self._build_loop(steps_per_graph)
        logits = self._prefill(input_ids.to(self.device), *self.state)
        self._cursor.zero_()
        self._position.fill_(self.prompt_tokens)
        # the first pick comes from the prompt's last position; positions stay where they are
        rt.greedy_advance(logits[:, -1].contiguous(), self._token, None, self._picked,
                          self._cursor)
        for _ in range((new_tokens - 1) // steps_per_graph):
            self._loop(self._token, self._position, *self.state)
        for backend in (self.prefill_backend, self.decode_backend):
            if backend.megabake_last_callable is not None:
                backend.megabake_last_callable.check()
        if int(self._cursor.max()) != new_tokens or int(self._cursor.min()) != new_tokens:
            raise RuntimeError("the device-side loop produced an unexpected number of tokens")
        return self._picked[:, :new_tokens].clone()
