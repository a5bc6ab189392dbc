"""ctypes binding of ``libmegabake_b200.so`` and the ``Plan`` object the host drives.

This is the only module that touches the native library.  It mirrors the structs of
``include/megabake_b200.h`` field for field, loads the in-tree shared object (building
nothing itself) and fails loudly -- ``CompilerError(stage="native-library")`` -- when the
library or one of its symbols is missing: there is no other execution path.
"""

from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

from .diagnostics import CompilerDiagnostic, CompilerError

MB_ABI_VERSION = 2
MB_MAX_DYNAMIC = 8
MB_PHASE_INTS = 24
MB_PHASE_FLOATS = 4
MB_PHASE_SLOTS = 20

MODE_DECODE, MODE_PREFILL = 0, 1

(BODY_NOP, BODY_GEMV, BODY_ATTN_DECODE, BODY_EMBED_ROWS, BODY_RMSNORM_ROWS, BODY_GEMM_TC,
 BODY_ROPE_ROWS, BODY_ATTN_PREFILL) = range(8)

FLAG_BARRIER, FLAG_BUMP_LENGTH, FLAG_FENCE = 1, 2, 4
CELLS_X, CELLS_OUT, CELLS_RESIDUAL, CELLS_XSTORE, CELLS_X_WAIT = 1, 2, 4, 8, 16
PRO_NONE, PRO_RMS_LLAMA, PRO_RMS_GEMMA = 0, 1, 2
EPI_NONE, EPI_RESIDUAL, EPI_SILU_MUL, EPI_GELU_TANH_MUL = 0, 1, 2, 3

# MB_BODY_GEMV field indices
GV_I_ROWS, GV_I_K, GV_I_NSEG, GV_I_N0 = 0, 1, 2, 3
GV_I_NMAT, GV_I_PROLOGUE, GV_I_EPILOGUE, GV_I_ROW_TILE, GV_I_K_CHUNK = 6, 7, 8, 9, 10
GV_I_GATHER, GV_I_VOCAB, GV_I_STORE_X, GV_I_SPLIT_Q, GV_I_SPLIT_R = 11, 12, 13, 14, 15
GV_I_CELLS, GV_I_X_SOURCE, GV_I_RES_SOURCE = 20, 21, 22
GV_F_EPS, GV_F_EMBED_SCALE = 0, 1
GV_S_X, GV_S_NORM_W, GV_S_W0, GV_S_BIAS0, GV_S_OUT0 = 0, 1, 2, 5, 8
GV_S_W_PAIR, GV_S_RESIDUAL, GV_S_IDS, GV_S_XSTORE = 11, 12, 13, 14

# MB_BODY_ATTN_DECODE field indices
AT_I_BATCH, AT_I_HEADS, AT_I_KV_HEADS, AT_I_HEAD_DIM, AT_I_CAPACITY = 0, 1, 2, 3, 4
AT_I_INVFREQ_BF16, AT_I_MAX_CHUNKS, AT_I_MERGE_SLOTS, AT_I_EXACT_KEYS = 5, 6, 7, 8
AT_I_CELLS, AT_I_QKV_SOURCE, AT_I_LEN_COUNT = 9, 10, 11
AT_F_SCALE, AT_F_ROPE_SCALE, AT_F_Q_SCALE = 0, 1, 2
(AT_S_Q, AT_S_K, AT_S_V, AT_S_KCACHE, AT_S_VCACHE, AT_S_LEN, AT_S_POS, AT_S_INVFREQ, AT_S_OUT,
 AT_S_PARTIAL, AT_S_COUNTER) = range(11)

# prefill bodies
GV_I_SPLIT_K, GV_I_TILE_N, GV_I_OUT_TOKENS, GV_I_OUT_CAPACITY = 16, 17, 18, 19
EM_I_ROWS, EM_I_K, EM_I_VOCAB = 0, 1, 2
EM_F_SCALE = 0
EM_S_TABLE, EM_S_IDS, EM_S_OUT = 0, 1, 2
RN_I_ROWS, RN_I_K, RN_I_KIND = 0, 1, 2
RN_F_EPS = 0
RN_S_X, RN_S_W, RN_S_OUT = 0, 1, 2
RP_I_ROWS, RP_I_HEADS, RP_I_KV_HEADS, RP_I_HEAD_DIM, RP_I_INVFREQ_BF16 = 0, 1, 2, 3, 4
RP_I_K_TOKENS, RP_I_K_CAPACITY, RP_I_LEN_VALUE, RP_I_LEN_COUNT = 5, 6, 7, 8
RP_F_ROPE_SCALE, RP_F_Q_SCALE = 0, 1
RP_S_Q, RP_S_K, RP_S_POS, RP_S_INVFREQ, RP_S_LEN = 0, 1, 2, 3, 4
AP_I_BATCH, AP_I_TOKENS, AP_I_HEADS, AP_I_KV_HEADS, AP_I_HEAD_DIM = 0, 1, 2, 3, 4
AP_I_CAUSAL, AP_I_MASK_BATCH, AP_I_KV_CAPACITY = 5, 6, 7
AP_F_SCALE = 0
AP_S_Q, AP_S_K, AP_S_V, AP_S_OUT, AP_S_MASK, AP_S_VT = 0, 1, 2, 3, 4, 5

STATUS_NAMES = {
    0: "ok", 1: "barrier-timeout", 2: "pipeline-timeout", 3: "kv-overflow", 4: "token-range",
    5: "bad-phase", 6: "tensor-memory", 7: "handoff-timeout",
}


class Phase(ctypes.Structure):
    _fields_ = [
        ("body", ctypes.c_int32),
        ("flags", ctypes.c_int32),
        ("i", ctypes.c_int32 * MB_PHASE_INTS),
        ("f", ctypes.c_float * MB_PHASE_FLOATS),
        ("slot", ctypes.c_int32 * MB_PHASE_SLOTS),
    ]

    @classmethod
    def blank(cls, body: int, flags: int = 0) -> "Phase":
        phase = cls()
        phase.body = body
        phase.flags = flags
        for index in range(MB_PHASE_SLOTS):
            phase.slot[index] = -1
        return phase


class PlanDesc(ctypes.Structure):
    _fields_ = [
        ("abi_version", ctypes.c_uint32),
        ("device", ctypes.c_int32),
        ("mode", ctypes.c_int32),
        ("n_phases", ctypes.c_uint32),
        ("phases", ctypes.POINTER(Phase)),
        ("n_slots", ctypes.c_uint32),
        ("n_dynamic", ctypes.c_uint32),
        ("activation_bytes", ctypes.c_uint32),
        ("ctas", ctypes.c_uint32),
        ("stage_bytes", ctypes.c_uint32),
        ("wait_limit_ms", ctypes.c_uint32),
        ("reserved", ctypes.c_uint32 * 2),
    ]


class PlanInfo(ctypes.Structure):
    _fields_ = [
        ("ctas", ctypes.c_int32),
        ("threads", ctypes.c_int32),
        ("smem_bytes", ctypes.c_int32),
        ("stages", ctypes.c_int32),
        ("barriers", ctypes.c_int32),
        ("sm_count", ctypes.c_int32),
        ("launches", ctypes.c_int32),
        ("reserved", ctypes.c_int32 * 1),
    ]


class AttentionArgs(ctypes.Structure):
    """``mb_attention_args`` of the allocation-free attention entry point."""

    _fields_ = [
        ("batch", ctypes.c_int32), ("heads", ctypes.c_int32), ("kv_heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32), ("capacity", ctypes.c_int32),
        ("inv_freq_is_bf16", ctypes.c_int32),
        ("rope_scale", ctypes.c_float), ("query_scale", ctypes.c_float),
        ("query", ctypes.c_uint64), ("key", ctypes.c_uint64), ("value", ctypes.c_uint64),
        ("key_cache", ctypes.c_uint64), ("value_cache", ctypes.c_uint64),
        ("valid_length", ctypes.c_uint64), ("position_ids", ctypes.c_uint64),
        ("inv_freq", ctypes.c_uint64), ("out", ctypes.c_uint64), ("status", ctypes.c_uint64),
    ]


class GreedyArgs(ctypes.Structure):
    """``mb_greedy_args`` of the on-device greedy pick."""

    _fields_ = [
        ("rows", ctypes.c_int32), ("vocab", ctypes.c_int32), ("out_capacity", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("logits", ctypes.c_uint64), ("input_ids", ctypes.c_uint64),
        ("position_ids", ctypes.c_uint64), ("out_tokens", ctypes.c_uint64),
        ("cursor", ctypes.c_uint64),
    ]


class Status(ctypes.Structure):
    _fields_ = [
        ("code", ctypes.c_int32),
        ("phase", ctypes.c_int32),
        ("detail", ctypes.c_int32),
        ("calls", ctypes.c_int32),
    ]


# The in-tree build, unless MEGABAKE_B200_LIBRARY names another build of the same ABI (a debug
# build, or two builds compared in one session).
LIBRARY_PATH = Path(os.environ.get("MEGABAKE_B200_LIBRARY") or
                    Path(__file__).resolve().parent / "_lib" / "libmegabake_b200.so")

# Every symbol include/megabake_b200.h declares; the loader checks all of them.
EXPORTS = (
    "mb_plan_create", "mb_plan_query", "mb_plan_bind", "mb_plan_launch", "mb_plan_status",
    "mb_plan_reset", "mb_plan_set_trace", "mb_plan_destroy", "mb_strerror", "mb_status_string", "mb_last_cuda_error",
    "mb_abi_version", "mb_fixed_smem_bytes", "mb_stage_bytes", "mb_max_smem_bytes",
    "mb_attention_decode_static", "mb_greedy_advance",
)

_library = None
_library_lock = threading.Lock()


def _native_error(message: str, requirement: str | None = None) -> CompilerError:
    return CompilerError(CompilerDiagnostic("native-library", message, requirement=requirement))


def load_library(path: Path | None = None) -> ctypes.CDLL:
    """Load (once) and type the native library; never builds and never falls back."""
    global _library
    with _library_lock:
        if _library is not None and path is None:
            return _library
        target = Path(path) if path is not None else LIBRARY_PATH
        if not target.exists():
            raise _native_error(
                f"{target} is missing",
                "build it with `python -m megabake_b200.build` (needs nvcc); there is no "
                "fallback execution path",
            )
        try:
            lib = ctypes.CDLL(str(target))
        except OSError as error:
            raise _native_error(f"cannot load {target}: {error}") from error
        missing = [name for name in EXPORTS if not hasattr(lib, name)]
        if missing:
            raise _native_error(f"{target} lacks symbols: {', '.join(missing)}")
        plan_p = ctypes.c_void_p
        lib.mb_plan_create.argtypes = [ctypes.POINTER(PlanDesc), ctypes.POINTER(plan_p)]
        lib.mb_plan_query.argtypes = [plan_p, ctypes.POINTER(PlanInfo)]
        lib.mb_plan_bind.argtypes = [plan_p, ctypes.POINTER(ctypes.c_uint64), ctypes.c_size_t]
        lib.mb_plan_launch.argtypes = [plan_p, ctypes.POINTER(ctypes.c_uint64), ctypes.c_size_t,
                                       ctypes.c_void_p]
        lib.mb_plan_status.argtypes = [plan_p, ctypes.POINTER(Status)]
        lib.mb_plan_reset.argtypes = [plan_p]
        lib.mb_plan_set_trace.argtypes = [plan_p, ctypes.c_uint64, ctypes.c_size_t]
        lib.mb_plan_destroy.argtypes = [plan_p]
        lib.mb_plan_destroy.restype = None
        for name in ("mb_plan_create", "mb_plan_query", "mb_plan_bind", "mb_plan_launch",
                     "mb_plan_status", "mb_plan_reset", "mb_plan_set_trace", "mb_abi_version",
                     "mb_max_smem_bytes"):
            getattr(lib, name).restype = ctypes.c_int
        for name in ("mb_fixed_smem_bytes", "mb_stage_bytes"):
            getattr(lib, name).argtypes = [ctypes.c_int]
            getattr(lib, name).restype = ctypes.c_int
        for name in ("mb_strerror", "mb_status_string"):
            getattr(lib, name).argtypes = [ctypes.c_int]
            getattr(lib, name).restype = ctypes.c_char_p
        lib.mb_last_cuda_error.restype = ctypes.c_char_p
        lib.mb_attention_decode_static.argtypes = [ctypes.POINTER(AttentionArgs), ctypes.c_void_p]
        lib.mb_attention_decode_static.restype = ctypes.c_int
        lib.mb_greedy_advance.argtypes = [ctypes.POINTER(GreedyArgs), ctypes.c_void_p]
        lib.mb_greedy_advance.restype = ctypes.c_int
        if lib.mb_abi_version() != MB_ABI_VERSION:
            raise _native_error(
                f"{target} speaks ABI {lib.mb_abi_version()}, the host expects {MB_ABI_VERSION}"
            )
        if path is None:
            _library = lib
        return lib


def _check(lib: ctypes.CDLL, code: int, stage: str, what: str) -> None:
    if code == 0:
        return
    message = f"{what}: {lib.mb_strerror(code).decode()}"
    detail = lib.mb_last_cuda_error().decode()
    if code == 2 and detail:
        message += f" [{detail}]"
    raise CompilerError(CompilerDiagnostic(stage, message))


def greedy_advance(logits, input_ids, position_ids=None, out_tokens=None, cursor=None,
                   stream: int | None = None) -> None:
    """Enqueue ``mb_greedy_advance``: per row of ``logits`` (``[rows, 1, vocab]`` or
    ``[rows, vocab]`` bf16) write the greedy pick into ``input_ids`` (int64 ``[rows, 1]``),
    add one to ``position_ids`` and append the pick to ``out_tokens[row, cursor[row]]``.
    Non-blocking, on ``stream`` (default: torch's current stream); the tensors are the
    caller's and must stay alive until the stream has run the kernel."""
    import torch

    lib = load_library()
    rows, vocab = logits.shape[0], logits.shape[-1]
    if logits.dtype != torch.bfloat16 or not logits.is_contiguous() or logits.numel() != rows * vocab:
        raise CompilerError(CompilerDiagnostic(
            "input-binding", "greedy_advance needs contiguous bf16 logits of one position per row"))
    for name, tensor, dtype in (("input_ids", input_ids, torch.int64),
                                ("position_ids", position_ids, torch.int64),
                                ("out_tokens", out_tokens, torch.int64),
                                ("cursor", cursor, torch.int32)):
        if tensor is None:
            continue
        if tensor.dtype != dtype or not tensor.is_contiguous() or tensor.device != logits.device:
            raise CompilerError(CompilerDiagnostic(
                "input-binding", f"greedy_advance: {name} must be a contiguous {dtype} tensor on "
                                 f"{logits.device}"))
        if name != "out_tokens" and tensor.numel() != rows:
            raise CompilerError(CompilerDiagnostic(
                "input-binding", f"greedy_advance: {name} must hold one element per row"))
    if (out_tokens is None) != (cursor is None):
        raise CompilerError(CompilerDiagnostic(
            "input-binding", "greedy_advance: out_tokens and cursor come together"))
    args = GreedyArgs()
    args.rows, args.vocab = rows, vocab
    args.out_capacity = 0 if out_tokens is None else out_tokens.shape[-1]
    args.logits, args.input_ids = logits.data_ptr(), input_ids.data_ptr()
    args.position_ids = 0 if position_ids is None else position_ids.data_ptr()
    args.out_tokens = 0 if out_tokens is None else out_tokens.data_ptr()
    args.cursor = 0 if cursor is None else cursor.data_ptr()
    if stream is None:
        stream = torch.cuda.current_stream(logits.device).cuda_stream
    with torch.cuda.device(logits.device):
        _check(lib, lib.mb_greedy_advance(ctypes.byref(args), ctypes.c_void_p(stream)),
               "runtime", "mb_greedy_advance")


class Plan:
    """One native plan: phase table + address table + launch.  Not re-entrant; the owner
    serialises calls (``BoundDecoder`` holds a lock)."""

    def __init__(self, phases: list[Phase], *, n_slots: int, n_dynamic: int,
                 activation_bytes: int, device: int, mode: int = MODE_DECODE, ctas: int = 0,
                 stage_bytes: int = 0, wait_limit_ms: int = 0):
        self._lib = load_library()
        self._handle = ctypes.c_void_p()
        self.n_slots = n_slots
        self.n_dynamic = n_dynamic
        array = (Phase * len(phases))(*phases)
        desc = PlanDesc()
        desc.abi_version = MB_ABI_VERSION
        desc.device = device
        desc.mode = mode
        desc.n_phases = len(phases)
        desc.phases = array
        desc.n_slots = n_slots
        desc.n_dynamic = n_dynamic
        desc.activation_bytes = activation_bytes
        desc.ctas = ctas
        desc.stage_bytes = stage_bytes
        desc.wait_limit_ms = wait_limit_ms
        code = self._lib.mb_plan_create(ctypes.byref(desc), ctypes.byref(self._handle))
        _check(self._lib, code, "resource-admission" if code in (3, 4) else "planning",
               "mb_plan_create")
        info = PlanInfo()
        _check(self._lib, self._lib.mb_plan_query(self._handle, ctypes.byref(info)), "planning",
               "mb_plan_query")
        self.ctas, self.threads, self.smem_bytes = info.ctas, info.threads, info.smem_bytes
        self.stages, self.barriers, self.sm_count = info.stages, info.barriers, info.sm_count
        self.launches = info.launches     # kernel launches per launch() call
        self._dynamic = (ctypes.c_uint64 * MB_MAX_DYNAMIC)()

    def bind(self, addresses: list[int]) -> None:
        array = (ctypes.c_uint64 * len(addresses))(*addresses)
        _check(self._lib, self._lib.mb_plan_bind(self._handle, array, len(addresses)),
               "runtime-binding", "mb_plan_bind")

    def launch(self, dynamic: list[int], stream: int) -> None:
        for index, address in enumerate(dynamic):
            self._dynamic[index] = address
        code = self._lib.mb_plan_launch(self._handle, self._dynamic, len(dynamic),
                                        ctypes.c_void_p(stream))
        if code:
            _check(self._lib, code, "runtime", "mb_plan_launch")

    def status(self) -> Status:
        out = Status()
        _check(self._lib, self._lib.mb_plan_status(self._handle, ctypes.byref(out)), "runtime",
               "mb_plan_status")
        return out

    def raise_for_status(self) -> Status:
        """Read the device status word (the caller synchronised already) and raise
        ``CompilerError`` for a recorded fault."""
        status = self.status()
        if status.code != 0:
            name = STATUS_NAMES.get(status.code, str(status.code))
            text = self._lib.mb_status_string(status.code).decode()
            stage = "state-capacity" if status.code == 3 else "runtime"
            raise CompilerError(CompilerDiagnostic(
                stage,
                f"device status {name}: {text} (phase {status.phase}, detail {status.detail})",
            ))
        return status

    def set_trace(self, device_address: int, nbytes: int) -> None:
        """Point the kernel's per-phase timer stamps at a device buffer of
        ``ctas * n_phases * 8`` uint64 (0 switches tracing off)."""
        _check(self._lib, self._lib.mb_plan_set_trace(self._handle, device_address, nbytes),
               "runtime-binding", "mb_plan_set_trace")

    def reset(self) -> None:
        _check(self._lib, self._lib.mb_plan_reset(self._handle), "runtime", "mb_plan_reset")

    def close(self) -> None:
        if self._handle:
            self._lib.mb_plan_destroy(self._handle)
            self._handle = ctypes.c_void_p()

    def __del__(self):  # pragma: no cover - interpreter shutdown order
        try:
            self.close()
        except Exception:
            pass
