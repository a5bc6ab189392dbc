"""In-process caches of a backend and the tuning file of the planner.

``PlanCache`` keeps the reference's contract (``src/megabake/cache.py:38-58``: ``entries``,
``hits``, ``misses``, ``get_or_compile(key, compiler) -> PlanCacheResult(compiled, hit,
diagnostics)``, one lock).  What is cached here is a planned decoder invocation -- the phase
table and slot layout ``planner.plan_decode`` / ``plan_prefill`` produce -- so that a second
``torch.compile`` of the same graph (another wrapper instance, a recompilation after a guard
failure, the same model under another ``make_backend`` call site that shares the cache) skips
planning; binding to live tensors stays per callable.

``make_plan_key`` hashes everything a plan depends on (the reference hashes plan, capture context
and toolchain, ``cache.py:60-80``): the recognised program (shapes, numerics switches and the
argument position of every tensor), the mode, the device fingerprint, the native library's ABI
version and shared-memory constants, and the planner options in force.

``CaptureCache`` memoises recognition: ATen graph text + input metadata -> ``DecoderProgram``.

The tuning file (``MEGABAKE_B200_TUNING_FILE``, JSON, schema 1) carries measured planner choices
per model shape and device, after the reference's ``bodies/cuda/sm100/tuning.py:93-135``:

    {"schema": 1,
     "fingerprint": {"name": "NVIDIA B200", "multiprocessor_count": 148, "abi": 2},
     "choices": {"896:4864:151936:8": {"stage_bytes": 30720, "max_chunks": 32}}}

The key is ``hidden:intermediate:vocab:batch``; a choice may set ``stage_bytes``, ``max_chunks``,
``merge_slots`` and ``cell_limit``.  A file whose fingerprint does not match the device is an
error, as in the reference.
"""

from __future__ import annotations

import dataclasses
import hashlib
import json
import os
import threading
from collections.abc import Callable, Mapping
from dataclasses import dataclass, field
from functools import lru_cache
from pathlib import Path
from types import MappingProxyType
from typing import Any

TUNING_ENV = "MEGABAKE_B200_TUNING_FILE"
TUNABLE = ("stage_bytes", "max_chunks", "merge_slots", "cell_limit")


@dataclass(frozen=True)
class PlanCacheResult:
    compiled: Any
    hit: bool
    diagnostics: Mapping[str, Any] = MappingProxyType({})


@dataclass(frozen=True)
class PlanCacheEntry:
    key: str
    compiled: Any
    diagnostics: Mapping[str, Any] = MappingProxyType({})


def _diagnostics(layout: Any) -> Mapping[str, Any]:
    notes = getattr(layout, "notes", None)
    phases = getattr(layout, "phases", None)
    return MappingProxyType({
        "phases": len(phases) if phases is not None else None,
        "notes": tuple(notes or ()),
    })


@dataclass
class PlanCache:
    entries: dict[str, PlanCacheEntry] = field(default_factory=dict)
    hits: int = 0
    misses: int = 0

    def __post_init__(self) -> None:
        self._lock = threading.Lock()

    def get_or_compile(self, key: str, compiler: Callable[[], Any]) -> PlanCacheResult:
        with self._lock:
            entry = self.entries.get(key)
            if entry is not None:
                self.hits += 1
                return PlanCacheResult(entry.compiled, True, entry.diagnostics)
            self.misses += 1
            compiled = compiler()
            entry = PlanCacheEntry(key, compiled, _diagnostics(compiled))
            self.entries[key] = entry
            return PlanCacheResult(compiled, False, entry.diagnostics)


@dataclass
class CaptureCache:
    """Recognised programs by graph hash (the reference's capture cache memoises the prepared
    graph the same way, ``src/megabake/frontend.py:555``)."""

    entries: dict[str, Any] = field(default_factory=dict)
    hits: int = 0
    misses: int = 0

    def __post_init__(self) -> None:
        self._lock = threading.Lock()

    def get_or_recognize(self, key: str, recognizer: Callable[[], Any]):
        with self._lock:
            if key in self.entries:
                self.hits += 1
                return self.entries[key], True
            self.misses += 1
            program = recognizer()
            self.entries[key] = program
            return program, False


def graph_key(graph_module, mode: str) -> str:
    """Hash of an ATen graph: its printed code plus the metadata of every placeholder."""
    import torch

    parts = [mode, graph_module.code if hasattr(graph_module, "code") else str(graph_module.graph)]
    for node in graph_module.graph.nodes:
        if node.op != "placeholder":
            continue
        value = node.meta.get("val")
        if isinstance(value, torch.Tensor):
            parts.append(f"{node.name}:{value.dtype}:{tuple(value.shape)}:{value.device}")
        else:
            parts.append(f"{node.name}:{value!r}")
    return hashlib.sha256("\n".join(parts).encode()).hexdigest()


def _canonical(value: Any) -> Any:
    if dataclasses.is_dataclass(value) and not isinstance(value, type):
        return {f.name: _canonical(getattr(value, f.name)) for f in dataclasses.fields(value)
                if f.compare}
    if isinstance(value, Mapping):
        return {str(k): _canonical(v) for k, v in sorted(value.items(), key=lambda kv: str(kv[0]))}
    if isinstance(value, (list, tuple)):
        return [_canonical(v) for v in value]
    if isinstance(value, float):
        return repr(value)
    if value is None or isinstance(value, (str, int, bool)):
        return value
    return repr(value)


def device_fingerprint(device_index: int | None = None) -> dict[str, Any]:
    """Name, SM count and capability of a CUDA device plus the native library's ABI version.
    Without a GPU (planner unit tests) the device part is the nominal B200."""
    import torch

    from . import runtime as rt

    fingerprint: dict[str, Any] = {"abi": rt.MB_ABI_VERSION}
    if torch.cuda.is_available():
        props = torch.cuda.get_device_properties(
            torch.cuda.current_device() if device_index is None else device_index)
        fingerprint.update(name=props.name, multiprocessor_count=props.multi_processor_count,
                           capability=f"{props.major}.{props.minor}")
    else:
        fingerprint.update(name="NVIDIA B200", multiprocessor_count=148, capability="10.0")
    return fingerprint


def make_plan_key(program, options, *, device_index: int | None = None, mask=None) -> str:
    from . import runtime as rt

    lib = rt.load_library()
    payload = {
        "program": _canonical(program),
        "options": _canonical(options),
        "device": device_fingerprint(device_index),
        "library": {"abi": lib.mb_abi_version(), "stage_bytes": lib.mb_stage_bytes(rt.MODE_DECODE),
                    "fixed_smem": lib.mb_fixed_smem_bytes(rt.MODE_DECODE),
                    "max_smem": lib.mb_max_smem_bytes()},
        # a non-causal prefill plan carries its mask as a constant
        "mask": None if mask is None else hashlib.sha256(
            mask.detach().cpu().contiguous().view(-1).view(dtype=__import__("torch").uint8)
            .numpy().tobytes()).hexdigest(),
    }
    encoded = json.dumps(payload, sort_keys=True, separators=(",", ":")).encode()
    return hashlib.sha256(encoded).hexdigest()


# ---------------------------------------------------------------------------------------
# Tuning file
# ---------------------------------------------------------------------------------------
@lru_cache(maxsize=16)
def _read(path: str, mtime_ns: int, size: int) -> dict:
    del mtime_ns, size
    data = json.loads(Path(path).read_text(encoding="utf-8"))
    if not isinstance(data, dict) or data.get("schema") != 1:
        raise ValueError("megabake_b200 tuning file must use schema 1")
    if not isinstance(data.get("choices"), dict):
        raise ValueError("megabake_b200 tuning file has no choices mapping")
    return data


def shape_key(program) -> str:
    return f"{program.hidden}:{program.intermediate}:{program.vocab}:{program.batch}"


def tuned_choice(program, device_index: int | None = None) -> dict[str, int]:
    """The tuning file's choice for this model shape on this device ({} without a file or an
    entry).  Raises ``ValueError`` for a malformed file or a foreign fingerprint."""
    path = os.environ.get(TUNING_ENV)
    if not path:
        return {}
    resolved = Path(path).expanduser().resolve()
    stat = resolved.stat()
    data = _read(str(resolved), stat.st_mtime_ns, stat.st_size)
    fingerprint = device_fingerprint(device_index)
    theirs = data.get("fingerprint")
    if not isinstance(theirs, dict) or any(theirs.get(k) != fingerprint[k]
                                           for k in ("name", "multiprocessor_count", "abi")):
        raise ValueError(f"tuning file {resolved} does not match this device or library "
                         f"(file: {theirs}, here: {fingerprint})")
    choice = data["choices"].get(shape_key(program))
    if choice is None:
        return {}
    if not isinstance(choice, dict) or any(k not in TUNABLE for k in choice) or any(
            not isinstance(v, int) or v < 0 for v in choice.values()):
        raise ValueError(f"invalid tuning choice for {shape_key(program)}: {choice!r}")
    if "stage_bytes" in choice and choice["stage_bytes"] % 1024:
        raise ValueError("tuned stage_bytes must be a multiple of 1024")
    return dict(choice)
