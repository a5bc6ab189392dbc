"""``make_backend``: the ``torch.compile`` backend factory, the drop-in boundary of the package.

Same call as the reference (``src/megabake/frontend.py:552-663``):

    backend = make_backend(mode="decode")            # or "prefill"
    step = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    logits = step(input_ids, position_ids, *state)

Option names, defaults and validation messages follow ``frontend.py:359-388``.  Dynamo hands the
backend an FX graph; it is lowered to ATen with AOTAutograd and Inductor's decomposition table
(the reference's own capture, ``frontend.py:425-549``, minus the pinned post-grad passes that
only exist in its torch release) and then

* ``compile_kernel=False`` (or automatic, when the inputs are not on an sm_100 GPU): the ATen
  graph itself is returned as the forward -- the reference's "FX reference" path;
* otherwise the graph is recognised as a decoder (``recognize.py``), planned into barrier
  intervals (``planner.py``) and bound to one native plan (``engine.py``); every call is one
  cooperative megakernel launch.

Deviation demanded by the target design: ``fallback="inductor"`` is accepted as an option value
but never taken -- a graph this backend does not cover raises ``CompilerError``; there is no
Inductor, Triton or CPU execution path behind a compiled call.
"""

from __future__ import annotations

import dataclasses
import json
import time
from pathlib import Path
from types import MappingProxyType
from typing import Any, Callable, Mapping, Sequence

import torch

from .diagnostics import CompilerDiagnostic, CompilerError

SUPPORTED_CAPABILITIES = {(10, 0), (10, 3)}


def _validate_options(options: Mapping[str, Any]) -> dict[str, Any]:
    known = {"mode", "fallback", "cache", "model_name", "dump_dir", "compile_kernel", "scheduler"}
    unknown = sorted(set(options) - known)
    if unknown:
        raise TypeError(f"Unknown backend options: {', '.join(unknown)}")
    mode = options.get("mode", "prefill")
    fallback = options.get("fallback", "error")
    if mode not in {"prefill", "decode"}:
        raise ValueError(f"Unsupported mode {mode!r}; expected 'prefill' or 'decode'")
    if fallback not in {"error", "inductor"}:
        raise ValueError(f"Unsupported fallback {fallback!r}; expected 'error' or 'inductor'")
    if not isinstance(options.get("cache", True), bool):
        raise TypeError("cache must be a boolean")
    model_name = options.get("model_name", "model")
    if not isinstance(model_name, str) or not model_name:
        raise TypeError("model_name must be a non-empty string")
    dump_dir = options.get("dump_dir")
    if dump_dir is not None and not isinstance(dump_dir, (str, Path)):
        raise TypeError("dump_dir must be a path or None")
    compile_kernel = options.get("compile_kernel", None)
    if compile_kernel not in {None, True, False}:
        raise TypeError("compile_kernel must be True, False, or None for automatic")
    scheduler = options.get("scheduler", "auto")
    if scheduler not in {"phase", "region-events", "auto"}:
        raise ValueError("scheduler must be 'phase', 'region-events', or 'auto'")
    return {"mode": mode, "fallback": fallback, "cache": options.get("cache", True),
            "model_name": model_name, "dump_dir": dump_dir, "compile_kernel": compile_kernel,
            "scheduler": scheduler}


def _can_auto_compile(example_inputs: Sequence[Any]) -> bool:
    tensors = [value for value in example_inputs if isinstance(value, torch.Tensor)]
    if not tensors or any(tensor.device.type != "cuda" for tensor in tensors):
        return False
    try:
        return torch.cuda.get_device_capability(tensors[0].device) in SUPPORTED_CAPABILITIES
    except Exception:  # noqa: BLE001 - any probing failure means "do not compile"
        return False


def _reject_symbolic_shapes(graph: torch.fx.GraphModule) -> None:
    for node in graph.graph.nodes:
        value = node.meta.get("val", node.meta.get("example_value"))
        if isinstance(value, torch.Tensor) and any(not isinstance(d, int) for d in value.shape):
            raise ValueError("Symbolic tensor shape is unsupported")


@dataclasses.dataclass
class PreparedFX:
    """What capture produced: the ATen-level graph and a callable that runs it."""

    graph: torch.fx.GraphModule | None
    forward: Callable[..., Any]
    mode: str
    example_inputs: tuple
    program: Any = None  # DecoderProgram once recognised


def _microseconds(start: float) -> float:
    return (time.perf_counter() - start) * 1e6


def _phase_table(layout) -> dict:
    """The planned phase records and slot layout as plain data (``dump_dir``)."""
    from . import runtime as rt

    return {
        "mode": "prefill" if layout.mode == rt.MODE_PREFILL else "decode",
        "notes": list(layout.notes), "workspace_bytes": layout.workspace_bytes,
        "activation_bytes": layout.activation_bytes, "stage_bytes": layout.stage_bytes,
        "slots": [dataclasses.asdict(slot) for slot in layout.slots],
        "phases": [{"body": phase.body, "flags": phase.flags, "i": list(phase.i),
                    "f": [float(x) for x in phase.f], "slot": list(phase.slot)}
                   for phase in layout.phases],
    }


class _MegakernelCall:
    """Boxed callable AOTAutograd invokes with the flat graph inputs; plans and binds on the
    first real call (capture-time inputs may be fake tensors), launches on every call."""

    _boxed_call = True

    def __init__(self, program, owner, options, plan_cache, trace):
        self.program = program
        self.owner = owner
        self.options = options
        self.plan_cache = plan_cache
        self.trace = trace
        self.decoder = None

    def _plan(self, program, device_index):
        from .cache import make_plan_key
        from .planner import PlannerOptions, plan_decode, plan_prefill

        planner_options = PlannerOptions.resolve(program, device_index)

        def build():
            if program.mode == "prefill":
                return plan_prefill(program, mask=program.mask)
            return plan_decode(program, planner_options)

        if self.plan_cache is None:
            return build(), False
        key = make_plan_key(program, planner_options, device_index=device_index, mask=program.mask)
        result = self.plan_cache.get_or_compile(key, build)
        return result.compiled, result.hit

    def __call__(self, args: list) -> list:
        from .engine import BoundDecoder

        flat = list(args)
        args.clear()
        if self.decoder is None:
            program = self.program
            if program.embed_scale_arg is not None:
                scale = float(flat[program.embed_scale_arg].float().reshape(-1)[0])
                program = dataclasses.replace(program, embed_scale=scale)
            device = flat[program.input_ids].device
            started = time.perf_counter()
            layout, hit = self._plan(program, device.index)
            self.trace.append({"stage": "planning", "us": _microseconds(started),
                               "plan_cache_hit": hit, "phases": len(layout.phases)})
            started = time.perf_counter()
            self.decoder = BoundDecoder(layout, flat)
            self.trace.append({"stage": "runtime-binding", "us": _microseconds(started)})
            self.decoder.megabake_trace = self.trace
            self.owner.megabake_last_callable = self.decoder
            self.owner.megabake_last_compile_us = sum(entry["us"] for entry in self.trace)
            dump_dir = self.options["dump_dir"]
            if dump_dir is not None:
                target = Path(dump_dir)
                target.mkdir(parents=True, exist_ok=True)
                (target / f"{self.options['model_name']}.{program.mode}.phases.json").write_text(
                    json.dumps(_phase_table(layout), indent=1) + "\n")
        return [self.decoder(*flat)]


def _capture(graph: torch.fx.GraphModule, example_inputs: Sequence[Any], options: dict,
             compile_kernel: bool, owner, capture_cache=None, plan_cache=None,
             trace: list | None = None) -> PreparedFX:
    from torch._functorch.aot_autograd import aot_module_simplified
    from torch._inductor.compile_fx import make_boxed_func
    from torch._inductor.decomposition import select_decomp_table

    from . import ops  # noqa: F401  (the declared operators must be registered before tracing)

    captured: dict[str, Any] = {}
    trace = trace if trace is not None else []
    capture_started = time.perf_counter()

    def inference_compiler(aten_graph: torch.fx.GraphModule, inputs):
        captured["graph"] = aten_graph
        trace.append({"stage": "fx-capture", "us": _microseconds(capture_started),
                      "nodes": len(aten_graph.graph.nodes)})
        dump_dir = options["dump_dir"]
        if dump_dir is not None:  # the captured ATen graph, as the reference dumps it
            target = Path(dump_dir)
            target.mkdir(parents=True, exist_ok=True)
            (target / f"{options['model_name']}.{options['mode']}.aten.txt").write_text(
                aten_graph.print_readable(print_output=False) + "\n")
        if not compile_kernel:
            return make_boxed_func(aten_graph.forward)
        from .cache import graph_key
        from .recognize import recognize_decoder

        started = time.perf_counter()
        if capture_cache is not None:
            program, hit = capture_cache.get_or_recognize(
                graph_key(aten_graph, options["mode"]),
                lambda: recognize_decoder(aten_graph, options["mode"]))
        else:
            program, hit = recognize_decoder(aten_graph, options["mode"]), False
        trace.append({"stage": "semantic-lowering", "us": _microseconds(started),
                      "capture_cache_hit": hit})
        captured["program"] = program
        if dump_dir is not None:
            (Path(dump_dir) / f"{options['model_name']}.{options['mode']}.program.json").write_text(
                json.dumps({f.name: repr(getattr(program, f.name))
                            for f in dataclasses.fields(program) if f.name != "mask"}, indent=1)
                + "\n")
        return _MegakernelCall(program, owner, options, plan_cache, trace)

    with torch.no_grad():
        forward = aot_module_simplified(
            graph, example_inputs, fw_compiler=inference_compiler,
            inference_compiler=inference_compiler, decompositions=select_decomp_table(),
            keep_inference_input_mutations=True,
        )
    if "graph" not in captured:
        raise RuntimeError("AOT did not produce an FX graph")
    return PreparedFX(captured["graph"], forward, options["mode"], tuple(example_inputs),
                      captured.get("program"))


def make_backend(**options: Any) -> Callable[..., Any]:
    """Create a ``torch.compile`` backend.  Options: ``mode`` ("prefill" | "decode"),
    ``fallback`` ("error" | "inductor"; never taken), ``cache``, ``model_name``, ``dump_dir``,
    ``compile_kernel`` (True | False | None = automatic), ``scheduler``."""
    from .cache import CaptureCache, PlanCache

    validated = _validate_options(options)
    contexts: list[PreparedFX] = []
    # cache=True (the default): recognised programs and planned layouts are kept for the life of
    # the backend; cache=False: every compile recognises and plans afresh (reference
    # frontend.py:555-561)
    cache = CaptureCache() if validated["cache"] else None
    plan_cache = PlanCache() if validated["cache"] else None

    def prepare(graph: Any, example_inputs: Sequence[Any], *,
                input_kinds: Mapping[str, str] | None = None,
                parameter_names: set[str] | None = None, **_unused: Any) -> PreparedFX:
        """Capture only: the ATen-level graph and a callable that runs it through ATen (the
        reference's ``backend.megabake_prepare``, ``frontend.py:563-585``)."""
        del input_kinds, parameter_names
        _reject_symbolic_shapes(graph)
        prepared = _capture(graph, example_inputs, validated, False, backend)
        contexts.append(prepared)
        return prepared

    def backend(graph: Any, example_inputs: Sequence[Any], *,
                input_kinds: Mapping[str, str] | None = None,
                parameter_names: set[str] | None = None, **dynamo_kwargs: Any):
        if dynamo_kwargs:
            raise TypeError(f"Unsupported Dynamo backend options: {', '.join(sorted(dynamo_kwargs))}")
        if torch.is_grad_enabled() and any(
            isinstance(value, torch.Tensor) and value.requires_grad for value in example_inputs
        ):
            raise RuntimeError("MegaBake supports inference only")
        _reject_symbolic_shapes(graph)
        choice = validated["compile_kernel"]
        compile_kernel = choice is True or (choice is None and _can_auto_compile(example_inputs))
        backend.megabake_last_compiled = None
        backend.megabake_last_callable = None
        backend.megabake_last_compile_us = None
        trace: list[dict] = []
        backend.megabake_last_trace = trace if compile_kernel else None
        try:
            prepared = _capture(graph, example_inputs, validated, compile_kernel, backend,
                                cache, plan_cache, trace)
        except CompilerError as error:
            error.safe_for_fallback = False  # there is nothing to fall back to
            raise
        contexts.append(prepared)
        backend.megabake_last_prepared = prepared
        backend.megabake_last_fallback = None
        if compile_kernel:
            backend.megabake_last_compiled = prepared.program
            backend.megabake_last_compile_us = sum(entry["us"] for entry in trace)
        forward = prepared.forward
        try:
            forward.megabake_contexts = contexts
            forward.megabake_cache = cache
            forward.megabake_plan_cache = plan_cache
        except AttributeError:  # some callables refuse attributes; the backend keeps them
            pass
        return forward

    backend.megabake_cache = cache
    backend.megabake_plan_cache = plan_cache
    backend.megabake_prepare = prepare
    backend.megabake_last_compile_us = None
    backend.megabake_last_trace = None
    backend.megabake_contexts = contexts
    backend.megabake_options = MappingProxyType(validated)
    backend.megabake_last_prepared = None
    backend.megabake_last_compiled = None
    backend.megabake_last_callable = None
    backend.megabake_last_fallback = None
    backend.__name__ = "megabake_backend"
    return backend


def unsupported(stage: str, message: str) -> CompilerError:
    return CompilerError(CompilerDiagnostic(stage, message))
