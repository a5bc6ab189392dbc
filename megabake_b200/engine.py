"""Host runtime of one compiled decoder invocation: workspace, binding, launch, status.

``BoundDecoder`` is what ``make_backend`` returns for a recognised graph (and what the
benchmark drives directly).  Per call it does what the reference's bound callable does
(``src/megabake/compiler.py:881-1012``): re-validate only arguments that are new objects,
rebind static addresses if one of them moved, allocate the output, enqueue one launch on the
current stream without blocking.  Weights and KV state are borrowed from the caller's
tensors and never copied; the KV caches and valid lengths are updated in place by the
kernel.
"""

from __future__ import annotations

import threading
from typing import Sequence

import torch

from . import runtime as rt
from .diagnostics import CompilerDiagnostic, CompilerError, fail
from .planner import DYN_INPUT_IDS, DYN_LOGITS, DYN_POSITION_IDS, PlanLayout

# Runtime states launched while ``graphed`` captures; None outside a capture.
_capture_log: list["BoundDecoder"] | None = None


def _require_native_device(device: torch.device) -> None:
    if device.type != "cuda":
        fail("native-library",
             f"megabake_b200 kernels need a CUDA device, got tensors on {device}",
             requirement="an sm_100 GPU; there is no CPU execution path")
    major, minor = torch.cuda.get_device_capability(device)
    if major != 10:
        fail("resource-admission",
             f"device compute capability {major}.{minor} is not sm_100",
             requirement="NVIDIA B200 (sm_100a)")


class BoundDecoder:
    """A planned decoder step bound to live tensors."""

    def __init__(self, layout: PlanLayout, args: Sequence[torch.Tensor], *, ctas: int = 0,
                 wait_limit_ms: int = 0):
        self.layout = layout
        self.program = layout.program
        p = self.program
        ids = args[p.input_ids]
        if not isinstance(ids, torch.Tensor):
            fail("input-binding", "input_ids must be a tensor")
        self.device = ids.device
        _require_native_device(self.device)
        self._lock = threading.Lock()
        self._expected = self._metadata(args)
        with torch.cuda.device(self.device):
            self.workspace = torch.empty(max(layout.workspace_bytes, 256), dtype=torch.uint8,
                                         device=self.device)
            self._zero_workspace()
            self.plan = rt.Plan(layout.phases, n_slots=len(layout.slots), n_dynamic=3,
                                activation_bytes=layout.activation_bytes,
                                device=self.device.index or 0, mode=layout.mode, ctas=ctas,
                                stage_bytes=layout.stage_bytes, wait_limit_ms=wait_limit_ms)
            # tensors the plan itself owns: a non-causal mask, and the positions 0..T-1 of
            # every row when the captured graph held them as constants
            self._constants = {name: tensor.to(self.device)
                               for name, tensor in layout.constants.items()}
            self._positions = None
            if p.position_ids is None:
                self._positions = torch.arange(p.tokens, dtype=torch.int64,
                                               device=self.device).repeat(p.batch)
        self._static_positions = sorted({s.index for s in layout.slots if s.kind == "arg"})
        self._bound_objects: dict[int, torch.Tensor] = {}
        self._bound_pointers: dict[int, int] = {}
        self._rebind(args, force=True)
        self.launches = 0
        self.megabake_trace: list[dict] = []

    # -- binding -------------------------------------------------------------------------
    def _metadata(self, args: Sequence[torch.Tensor]):
        used = {s.index for s in self.layout.slots if s.kind == "arg"}
        used |= {self.program.input_ids}
        if self.program.position_ids is not None:
            used.add(self.program.position_ids)
        return {i: (tuple(args[i].shape), args[i].dtype, args[i].device) for i in used}

    def _zero_workspace(self) -> None:
        for offset, nbytes in self.layout.zero_ranges:
            self.workspace[offset:offset + nbytes].zero_()

    def _check_tensor(self, position: int, tensor: torch.Tensor, align: int = 16) -> None:
        shape, dtype, device = self._expected[position]
        if not isinstance(tensor, torch.Tensor):
            fail("input-binding", f"argument {position} is not a tensor")
        if tuple(tensor.shape) != shape or tensor.dtype != dtype or tensor.device != device:
            fail("input-binding",
                 f"argument {position} is {tensor.dtype} {tuple(tensor.shape)} on {tensor.device}; "
                 f"the graph was captured with {dtype} {shape} on {device}",
                 requirement="static shapes: recompile for new shapes")
        if not tensor.is_contiguous():
            fail("input-binding", f"argument {position} is not contiguous")
        if tensor.data_ptr() % align:
            fail("input-binding", f"argument {position} is not {align}-byte aligned")

    def _rebind(self, args: Sequence[torch.Tensor], force: bool = False) -> None:
        changed = force
        for position in self._static_positions:
            tensor = args[position]
            if not force and self._bound_objects.get(position) is tensor:
                continue
            self._check_tensor(position, tensor)
            pointer = tensor.data_ptr()
            if self._bound_pointers.get(position) != pointer:
                changed = True
            self._bound_objects[position] = tensor
            self._bound_pointers[position] = pointer
        if not changed:
            return
        base = self.workspace.data_ptr()
        table = []
        for spec in self.layout.slots:
            if spec.kind == "dynamic":
                table.append(0)
            elif spec.kind == "arg":
                table.append(self._bound_pointers[spec.index])
            elif spec.kind == "constant":
                table.append(self._constants[spec.name].data_ptr())
            else:
                table.append(base + spec.offset)
        self.plan.bind(table)

    # -- call ----------------------------------------------------------------------------
    def __call__(self, *args: torch.Tensor) -> torch.Tensor:
        p = self.program
        with self._lock:
            ids = args[p.input_ids]
            self._check_tensor(p.input_ids, ids, align=8)
            if p.position_ids is None:
                positions = self._positions
            else:
                positions = args[p.position_ids]
                self._check_tensor(p.position_ids, positions, align=8)
            self._rebind(args)
            logits = torch.empty((p.batch, p.tokens, p.vocab), dtype=torch.bfloat16,
                                 device=self.device)
            dynamic = [0, 0, 0]
            dynamic[DYN_INPUT_IDS] = ids.data_ptr()
            dynamic[DYN_POSITION_IDS] = positions.data_ptr()
            dynamic[DYN_LOGITS] = logits.data_ptr()
            stream = torch.cuda.current_stream(self.device).cuda_stream
            self.plan.launch(dynamic, stream)
            self.launches += 1
            if _capture_log is not None:
                _capture_log.append(self)
        return logits

    def launch_into(self, ids: torch.Tensor, positions: torch.Tensor,
                    logits: torch.Tensor) -> None:
        """Launch with caller-provided, already validated dynamic tensors (benchmark loop:
        no allocation, no checks)."""
        self.plan.launch([ids.data_ptr(), positions.data_ptr(), logits.data_ptr()],
                         torch.cuda.current_stream(self.device).cuda_stream)
        self.launches += 1

    # -- status --------------------------------------------------------------------------
    def check(self) -> rt.Status:
        """Synchronise the device and raise ``CompilerError`` if the kernel recorded a
        fault (KV cache full, token id out of range, a wait that ran out)."""
        torch.cuda.synchronize(self.device)
        try:
            return self.plan.raise_for_status()
        except CompilerError:
            self.recover()
            raise

    def recover(self) -> None:
        """Clear a recorded fault so the plan can launch again."""
        torch.cuda.synchronize(self.device)
        self.plan.reset()
        self._zero_workspace()

    def close(self) -> None:
        self.plan.close()


def ensure_no_fallback(error: CompilerError) -> CompilerError:
    """Mark an error as final: this backend has no second compiler to try."""
    error.safe_for_fallback = False
    return error


class GraphedCall:
    """One compiled call captured in a CUDA graph (reference ``compiler.py:1025-1095``).

    Later calls copy tensor arguments that are new objects into the captured ones, replay
    the graph and return the captured outputs, which the next call overwrites.
    """

    def __init__(self, function, args: tuple, warmup: int):
        global _capture_log
        import torch.utils._pytree as pytree

        self._function = function
        self._inputs, self._spec = pytree.tree_flatten(args)
        saved = [leaf.clone() if isinstance(leaf, torch.Tensor) else None for leaf in self._inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                function(*args)
            for leaf, original in zip(self._inputs, saved):
                if original is not None:
                    leaf.copy_(original)  # warm-up advanced the KV state; undo
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        del saved
        self._graph = torch.cuda.CUDAGraph()
        _capture_log = []
        try:
            with torch.cuda.graph(self._graph):
                self.output = function(*args)
            self._states = tuple(dict.fromkeys(_capture_log))
        finally:
            _capture_log = None
        if not self._states:
            raise CompilerError(CompilerDiagnostic(
                "callable-binding", "the captured call launched no megabake kernel",
                requirement="a function compiled by megabake_b200.make_backend"))

    def __call__(self, *args):
        import torch.utils._pytree as pytree

        leaves, spec = pytree.tree_flatten(args)
        if spec != self._spec:
            raise ValueError("a graphed call takes the argument structure it was captured with")
        for given, captured in zip(leaves, self._inputs):
            if given is captured:
                continue
            if not isinstance(captured, torch.Tensor):
                if given != captured:
                    raise ValueError(f"graphed call captured {captured!r}, got {given!r}")
            elif given.shape != captured.shape or given.dtype != captured.dtype:
                raise ValueError(
                    f"graphed call captured a {captured.dtype} {tuple(captured.shape)} tensor, "
                    f"got {given.dtype} {tuple(given.shape)}")
            else:
                captured.copy_(given)
        self._graph.replay()
        return self.output


def graphed(function, *args, warmup: int = 2) -> GraphedCall:
    """Capture one call of a compiled ``function`` in a CUDA graph."""
    return GraphedCall(function, args, max(warmup, 2))
