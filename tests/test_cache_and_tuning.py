"""Plan cache, capture cache, backend attributes, dump directory and the tuning file (CPU).

Mirrors what the reference's tests read from a backend (``src/megabake/frontend.py:618-661``:
``megabake_cache``, ``megabake_plan_cache``, ``megabake_last_compile_us``, ``megabake_last_trace``,
``megabake_prepare``) and its tuning-file rules (``bodies/cuda/sm100/tuning.py:93-135``)."""

import json

import pytest
import torch

from megabake_b200 import CompilerError, StatefulDecoder, make_backend, models
from megabake_b200 import cache as mb_cache
from megabake_b200 import planner


def test_plan_cache_contract_and_keys():
    spec = models.get_spec("tiny-llama")
    program = models.direct_program(spec, 2, 16)
    options = planner.PlannerOptions()
    cache = mb_cache.PlanCache()
    key = mb_cache.make_plan_key(program, options)
    first = cache.get_or_compile(key, lambda: planner.plan_decode(program, options))
    second = cache.get_or_compile(key, lambda: pytest.fail("a hit must not plan again"))
    assert (first.hit, second.hit, cache.hits, cache.misses) == (False, True, 1, 1)
    assert second.compiled is first.compiled and first.diagnostics["phases"] == 5 * spec.layers + 1
    # everything a plan depends on moves the key
    assert mb_cache.make_plan_key(models.direct_program(spec, 3, 16), options) != key
    assert mb_cache.make_plan_key(models.direct_program(spec, 2, 32), options) != key
    assert mb_cache.make_plan_key(program, planner.PlannerOptions(max_chunks=8)) != key
    assert mb_cache.make_plan_key(models.direct_program(spec, 2, 16, per_row_lengths=True),
                                  options) != key
    assert mb_cache.make_plan_key(models.direct_program(spec, 2, 16), options) == key


def test_backend_attributes_and_capture_cache(tmp_path):
    spec = models.get_spec("tiny-llama")
    model = models.build_hf_model(spec, seed=1)
    backend = make_backend(mode="decode", compile_kernel=True, dump_dir=tmp_path, model_name="tiny")
    assert backend.megabake_cache.misses == 0 and backend.megabake_plan_cache.entries == {}
    assert backend.megabake_last_compile_us is None and backend.megabake_last_trace is None
    assert callable(backend.megabake_prepare)
    assert make_backend(cache=False).megabake_plan_cache is None
    assert make_backend(cache=False).megabake_cache is None
    for attempt in range(2):  # two wrapper instances over the same model: the same ATen graph
        wrapper = StatefulDecoder(model, 8).eval()
        torch._dynamo.reset()
        compiled = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
        state = wrapper.make_state(1)
        # recognised on CPU, but there is no CPU execution path: the first call refuses
        with pytest.raises(Exception) as info, torch.no_grad():
            compiled(torch.zeros(1, 1, dtype=torch.int64), torch.zeros(1, 1, dtype=torch.int64), *state)
        assert isinstance(info.value, CompilerError) or "CompilerError" in repr(info.value) \
            or "CUDA device" in str(info.value)
        assert backend.megabake_cache.misses == 1 and backend.megabake_cache.hits == attempt
        stages = [entry["stage"] for entry in backend.megabake_last_trace]
        assert stages[:2] == ["fx-capture", "semantic-lowering"]
        assert backend.megabake_last_trace[1]["capture_cache_hit"] == bool(attempt)
        assert backend.megabake_last_compile_us > 0
        assert backend.megabake_last_compiled.hidden == spec.hidden
    assert (tmp_path / "tiny.decode.aten.txt").read_text().count("megabake.kv_attention") >= spec.layers
    program = json.loads((tmp_path / "tiny.decode.program.json").read_text())
    assert program["hidden"] == str(spec.hidden) and program["mode"] == "'decode'"


def test_prepare_returns_the_fx_reference():
    spec = models.get_spec("tiny-llama")
    wrapper = StatefulDecoder(models.build_hf_model(spec, seed=1), 8).eval()
    backend = make_backend(mode="decode", compile_kernel=False)
    torch._dynamo.reset()
    compiled = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    state = wrapper.make_state(1)
    ids, pos = torch.ones(1, 1, dtype=torch.int64), torch.zeros(1, 1, dtype=torch.int64)
    with torch.no_grad():
        compiled(ids, pos, *state)
    assert backend.megabake_last_trace is None and backend.megabake_last_compile_us is None
    prepared = backend.megabake_last_prepared
    assert prepared.graph is not None and backend.megabake_contexts[-1] is prepared


def _tuning_file(tmp_path, fingerprint, choices):
    path = tmp_path / "tuning.json"
    path.write_text(json.dumps({"schema": 1, "fingerprint": fingerprint, "choices": choices}))
    return path


def test_tuning_file_sets_planner_options(tmp_path, monkeypatch):
    spec = models.get_spec("tiny-qwen2")
    program = models.direct_program(spec, 4, 64)
    fingerprint = mb_cache.device_fingerprint()
    key = mb_cache.shape_key(program)
    assert key == f"{spec.hidden}:{spec.intermediate}:{spec.vocab}:4"
    path = _tuning_file(tmp_path, fingerprint, {key: {"stage_bytes": 20480, "max_chunks": 4}})
    monkeypatch.setenv(mb_cache.TUNING_ENV, str(path))
    options = planner.PlannerOptions.resolve(program)
    assert (options.stage_bytes, options.max_chunks) == (20480, 4)
    layout = planner.plan_decode(program)
    assert layout.stage_bytes == 20480
    assert all(p.i[6] == 4 for p in layout.phases if p.body == 2)      # MB_AT_I_MAX_CHUNKS
    # another batch size has no entry: defaults
    assert planner.PlannerOptions.resolve(models.direct_program(spec, 1, 64)).stage_bytes is None
    # the sweep variable still wins over the file
    monkeypatch.setenv("MEGABAKE_B200_STAGE_BYTES", "24576")
    assert planner.PlannerOptions.resolve(program).stage_bytes == 24576


def test_tuning_file_is_checked(tmp_path, monkeypatch):
    spec = models.get_spec("tiny-qwen2")
    program = models.direct_program(spec, 4, 64)
    good = mb_cache.device_fingerprint()
    monkeypatch.setenv(mb_cache.TUNING_ENV, str(_tuning_file(
        tmp_path, dict(good, multiprocessor_count=good["multiprocessor_count"] + 1), {})))
    with pytest.raises(ValueError, match="does not match this device"):
        mb_cache.tuned_choice(program)
    key = mb_cache.shape_key(program)
    monkeypatch.setenv(mb_cache.TUNING_ENV, str(_tuning_file(tmp_path, good, {key: {"tile": 64}})))
    with pytest.raises(ValueError, match="invalid tuning choice"):
        mb_cache.tuned_choice(program)
    bad = tmp_path / "schema.json"
    bad.write_text(json.dumps({"schema": 2, "choices": {}}))
    monkeypatch.setenv(mb_cache.TUNING_ENV, str(bad))
    with pytest.raises(ValueError, match="schema 1"):
        mb_cache.tuned_choice(program)
