"""CPU-side checks: the shared library loads and exports every symbol the header declares,
the ctypes mirrors match the C structs, and the planner's tables are well formed."""

import ctypes
import re
from pathlib import Path

import pytest

from megabake_b200 import models, planner
from megabake_b200 import runtime as rt
from megabake_b200.diagnostics import CompilerError

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "megabake_b200.h").read_text()


def test_library_exports_every_declared_symbol():
    lib = rt.load_library()
    declared = set(re.findall(r"\b(mb_[a-z_]+)\s*\(", HEADER))
    assert declared, "no declarations found in the header"
    assert declared == set(rt.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.mb_abi_version() == rt.MB_ABI_VERSION


def test_struct_mirrors_match_header():
    ints = int(re.search(r"#define MB_PHASE_INTS (\d+)", HEADER).group(1))
    floats = int(re.search(r"#define MB_PHASE_FLOATS (\d+)", HEADER).group(1))
    slots = int(re.search(r"#define MB_PHASE_SLOTS (\d+)", HEADER).group(1))
    assert (ints, floats, slots) == (rt.MB_PHASE_INTS, rt.MB_PHASE_FLOATS, rt.MB_PHASE_SLOTS)
    assert ctypes.sizeof(rt.Phase) == 4 * (2 + ints + floats + slots)
    for name, value in re.findall(r"#define (MB_(?:GV|AT)_[A-Z]_[A-Z0-9_]+) (\d+)", HEADER):
        mirror = name[3:]
        assert getattr(rt, mirror) == int(value), name


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(CompilerError) as info:
        rt.load_library(tmp_path / "absent.so")
    assert info.value.diagnostic.stage == "native-library"
    assert "no fallback" in str(info.value)


@pytest.mark.parametrize("name", ["smollm-135m", "qwen2-0.5b", "llama-3.2-1b", "smollm-1.7b"])
@pytest.mark.parametrize("batch", [1, 8])
def test_decode_plan_tables(name, batch):
    spec = models.get_spec(name)
    layout = planner.plan_decode(models.direct_program(spec, batch, 8192 + 33))
    lib = rt.load_library()
    stage = lib.mb_stage_bytes(rt.MODE_DECODE)
    assert len(layout.phases) == 5 * spec.layers + 1
    assert layout.intervals == 1  # activations travel as flagged cells: only the closing barrier
    writers = {}  # workspace slot -> phase that last wrote its cells
    last_read = {}  # workspace slot -> last phase that read its cells

    def written(slot, index):
        # the kernel keeps CTAs within two phases of one another: a cell buffer may be rewritten
        # from the third phase after its last reader on
        assert slot not in last_read or index - last_read[slot] >= 3, (slot, index, last_read[slot])
        writers[slot] = index

    for index, phase in enumerate(layout.phases):
        assert not phase.flags & rt.FLAG_BARRIER
        if phase.body == rt.BODY_GEMV:
            tile, chunk, nmat = phase.i[rt.GV_I_ROW_TILE], phase.i[rt.GV_I_K_CHUNK], phase.i[rt.GV_I_NMAT]
            assert tile in (8, 16) and chunk % 32 == 0 and chunk <= phase.i[rt.GV_I_K]
            assert tile == 8 or (nmat == 1 and chunk == phase.i[rt.GV_I_K] <= 1024)
            assert tile * nmat * (chunk * 2 + 64) <= stage
            assert batch * (phase.i[rt.GV_I_K] + 32) * 2 <= layout.activation_bytes
            cells = phase.i[rt.GV_I_CELLS]
            # every operand written earlier in the launch names the phase that really wrote it
            if index > 0:
                assert cells & rt.CELLS_X_WAIT
                assert writers[phase.slot[rt.GV_S_X]] == phase.i[rt.GV_I_X_SOURCE] < index
                last_read[phase.slot[rt.GV_S_X]] = index
                if not cells & rt.CELLS_X:  # plain x: its producer fenced
                    assert layout.phases[phase.i[rt.GV_I_X_SOURCE]].flags & rt.FLAG_FENCE
                    assert batch * phase.i[rt.GV_I_K] * 4 > planner.CELL_LIMIT_BYTES
            if phase.slot[rt.GV_S_RESIDUAL] >= 0:
                assert phase.slot[rt.GV_S_RESIDUAL] != phase.slot[rt.GV_S_OUT0]
                last_read[phase.slot[rt.GV_S_RESIDUAL]] = index
                if cells & rt.CELLS_RESIDUAL:
                    assert writers[phase.slot[rt.GV_S_RESIDUAL]] == phase.i[rt.GV_I_RES_SOURCE] < index
                else:
                    assert layout.phases[writers[phase.slot[rt.GV_S_RESIDUAL]]].flags & rt.FLAG_FENCE
            if phase.slot[rt.GV_S_XSTORE] >= 0:
                written(phase.slot[rt.GV_S_XSTORE], index)
            if index < len(layout.phases) - 1:
                assert bool(cells & rt.CELLS_OUT) != bool(phase.flags & rt.FLAG_FENCE) or index == 0
                for seg in range(phase.i[rt.GV_I_NSEG]):
                    written(phase.slot[rt.GV_S_OUT0 + seg], index)
            else:
                assert not cells & rt.CELLS_OUT  # the logits are plain
        elif phase.body == rt.BODY_ATTN_DECODE:
            assert phase.flags & rt.FLAG_BUMP_LENGTH
            assert phase.i[rt.AT_I_CELLS] & rt.CELLS_X
            assert bool(phase.i[rt.AT_I_CELLS] & rt.CELLS_OUT) != bool(phase.flags & rt.FLAG_FENCE)
            for s in (rt.AT_S_Q, rt.AT_S_K, rt.AT_S_V):
                assert writers[phase.slot[s]] == phase.i[rt.AT_I_QKV_SOURCE] == index - 1
                last_read[phase.slot[s]] = index
            written(phase.slot[rt.AT_S_OUT], index)
        for slot in phase.slot:
            assert -1 <= slot < len(layout.slots)
    kinds = [s.kind for s in layout.slots]
    assert kinds[:3] == ["dynamic"] * 3 and "dynamic" not in kinds[3:]
    # every weight of the model is bound exactly once
    args = [s.index for s in layout.slots if s.kind == "arg"]
    assert len(args) == len(set(args))
    fixed = lib.mb_fixed_smem_bytes(rt.MODE_DECODE)
    assert fixed + layout.activation_bytes + 2 * stage <= lib.mb_max_smem_bytes()


def test_geometry_whole_rows_when_they_fit():
    stage = rt.load_library().mb_stage_bytes(rt.MODE_DECODE)
    # a 2048-wide matrix travels as whole 4 KB rows, paired with another it is cut in two
    assert planner.gemv_geometry(2048, 2048, 1, 148, stage, 64) == (8, 2048)
    assert planner.gemv_geometry(16384, 2048, 2, 148, stage, 64) == (8, 1024)
    # Qwen2's paired gate/up rows (K = 896) travel as whole rows
    assert planner.gemv_geometry(4864, 896, 2, 148, stage, 64) == (8, 896)
    # short rows of an unpaired phase: two 8-row tiles per stage
    assert planner.gemv_geometry(151936, 896, 1, 148, stage, 64) == (16, 896)
    assert planner.gemv_geometry(49152, 576, 1, 148, stage, 64) == (16, 576)
    for k in (576, 896, 1536, 2048, 4864, 8192, 16384):
        for nmat in (1, 2):
            tile, chunk = planner.gemv_geometry(4096, k, nmat, 148, stage, 64)
            assert chunk % 32 == 0 and tile * nmat * (chunk * 2 + 64) <= stage


def test_planner_refusals():
    spec = models.get_spec("tiny-llama")
    with pytest.raises(CompilerError) as info:
        planner.plan_decode(models.direct_program(spec, 9, 16))
    assert info.value.diagnostic.stage == "resource-admission"
    odd = models.get_spec("tiny-llama", head_dim=32)
    with pytest.raises(CompilerError):
        planner.plan_decode(models.direct_program(odd, 1, 16))


def test_weight_bytes_match_the_roofline_table():
    # bytes of weights one decode step reads (bf16), per the hot-path scope table
    expect = {"smollm-135m": 134_515_008, "qwen2-0.5b": 494_032_768,
              "llama-3.2-1b": 1_235_814_400, "smollm-1.7b": 1_711_376_384}
    for name, params in expect.items():
        spec = models.get_spec(name)
        assert spec.parameter_count() == params, name
