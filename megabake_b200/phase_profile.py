"""Per-phase timing of one megakernel launch from the kernel's own global-timer stamps.

The counterpart of the reference's phase profiler (``tools/phase_profile.py:104-238`` on top of
the ``MEGABAKE_PHASE_TIMER`` stamps, ``src/megabake/runtime.py:22-47``): thread 0 of every CTA
records the time at phase start, after the activation copies were started, after the body and,
where a phase ends in a grid barrier, after that barrier.  From those this module derives, per
phase, how long the critical CTA worked and how long the others waited; with flagged-cell
hand-offs (no barrier) a phase's wait shows up inside the next phase's body, as the time its
consumers spent polling.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from . import runtime as rt

EVENTS = 8  # stamps per phase and CTA (0..3 common, 4..7 body-specific)
BODY_NAMES = {rt.BODY_GEMV: "gemv", rt.BODY_ATTN_DECODE: "attention", rt.BODY_NOP: "nop"}


@dataclass
class PhaseTiming:
    index: int
    body: str
    span_us: float       # first CTA in -> last CTA out of the barrier
    prologue_us: float   # median over CTAs
    work_us: float       # median body time over CTAs
    slowest_us: float    # slowest CTA: phase start -> body done
    wait_us: float       # median time spent in the closing barrier
    release_us: float    # last arrival -> median barrier exit


def capture(decoder, launch, launches: int = 3) -> torch.Tensor:
    """Run ``launch()`` ``launches`` times with tracing on; returns the stamps of the last
    one as an int64 tensor ``[ctas, phases, 8]`` (nanoseconds)."""
    plan = decoder.plan
    phases = len(decoder.layout.phases)
    buffer = torch.zeros(plan.ctas * phases * EVENTS, dtype=torch.int64, device=decoder.device)
    plan.set_trace(buffer.data_ptr(), buffer.numel() * 8)
    try:
        for _ in range(launches):
            launch()
        torch.cuda.synchronize(decoder.device)
    finally:
        plan.set_trace(0, 0)
    return buffer.view(plan.ctas, phases, EVENTS).cpu()


def summarise(stamps: torch.Tensor, layout) -> list[PhaseTiming]:
    out = []
    t = stamps.double()
    for index, phase in enumerate(layout.phases):
        s = t[:, index]
        has_prologue = phase.body == rt.BODY_GEMV
        has_barrier = bool(phase.flags & rt.FLAG_BARRIER)
        start, pro, done = s[:, 0], (s[:, 1] if has_prologue else s[:, 0]), s[:, 2]
        leave = s[:, 3] if has_barrier else done
        out.append(PhaseTiming(
            index=index,
            body=BODY_NAMES.get(phase.body, str(phase.body)),
            span_us=float(leave.max() - start.min()) / 1e3,
            prologue_us=float((pro - start).median()) / 1e3,
            work_us=float((done - pro).median()) / 1e3,
            slowest_us=float((done - start).max()) / 1e3,
            wait_us=float((leave - done).median()) / 1e3,
            release_us=float(leave.median() - done.max()) / 1e3,
        ))
    return out


def report(timings: list[PhaseTiming], first: int = 0, count: int | None = None) -> str:
    rows = timings[first: None if count is None else first + count]
    lines = [f"{'phase':>5} {'body':10} {'span':>8} {'prologue':>9} {'work':>8} {'slowest':>8} "
             f"{'wait':>8} {'release':>8}   (microseconds)"]
    for r in rows:
        lines.append(f"{r.index:5d} {r.body:10} {r.span_us:8.2f} {r.prologue_us:9.2f} "
                     f"{r.work_us:8.2f} {r.slowest_us:8.2f} {r.wait_us:8.2f} {r.release_us:8.2f}")
    total = sum(r.span_us for r in timings)
    lines.append(f"sum of spans over {len(timings)} phases: {total:.1f} us")
    return "\n".join(lines)
