"""Error convention of the backend.

Every failure the backend can explain is raised as ``CompilerError`` carrying a
``CompilerDiagnostic`` whose ``stage`` says which step refused the work
(option validation happens earlier and raises plain ``ValueError``/``TypeError``).
The shape of both classes follows the reference's ``diagnostics.py:6-30`` so
callers that catch ``megabake.CompilerError`` and read ``.diagnostic.stage`` keep
working.  Stages used here:

``pattern-recognition``  the captured FX graph is not a decoder this backend covers
``planning``             regions could not be packed into barrier intervals
``resource-admission``   a body's shared-memory / batch / shape limit is exceeded
``input-binding``        a runtime argument differs from the captured metadata
``state-capacity``       the KV cache is full
``runtime``              the device status word reported a fault after a launch
``native-library``       the CUDA shared library is missing or misses a symbol
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class CompilerDiagnostic:
    stage: str
    message: str
    source_op_ids: tuple[str, ...] = ()
    region_ids: tuple[str, ...] = ()
    requirement: str | None = None


class CompilerError(ValueError):
    """A refusal with a diagnostic.  ``safe_for_fallback`` is kept for interface
    compatibility; this backend never falls back to another compiler."""

    def __init__(self, diagnostic: CompilerDiagnostic, *, safe_for_fallback: bool = False):
        super().__init__(diagnostic.message)
        self.diagnostic = diagnostic
        self.safe_for_fallback = safe_for_fallback

    def __str__(self) -> str:
        d = self.diagnostic
        text = f"{d.stage}: {d.message}"
        if d.source_op_ids:
            text += "; source operations: " + ", ".join(d.source_op_ids)
        if d.region_ids:
            text += "; regions: " + ", ".join(d.region_ids)
        if d.requirement:
            text += f"; requirement: {d.requirement}"
        return text


def fail(stage: str, message: str, *, requirement: str | None = None, ops: tuple[str, ...] = ()):
    """Raise a ``CompilerError`` for ``stage``."""
    raise CompilerError(
        CompilerDiagnostic(stage, message, source_op_ids=tuple(ops), requirement=requirement)
    )
