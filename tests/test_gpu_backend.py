"""The drop-in path on the GPU: ``torch.compile(wrapper, backend=make_backend(mode="decode"))``
captures, recognises, plans and launches the megakernel; results against the CPU oracle and
against the same module run eagerly on the GPU.  Reads like the reference's
``tests/gpu/test_table_gemm.py:65-120`` (compiled vs eager, logits and KV state) and
``:226-270`` (CUDA-graphed decode)."""

import threading

import pytest
import torch

from megabake_b200 import DecodeStep, StatefulDecoder, graphed, make_backend, models
from megabake_b200.engine import BoundDecoder
from oracle import decoder_oracle as oracle
from oracle.adapters import oracle_config, oracle_weights
from tests.helpers import LOGIT_COSINE, LOGIT_MAX_ABS, cosine, greedy_pick_matches, logits_close, max_abs

pytestmark = pytest.mark.gpu


def _setup(name, kind, batch, capacity, seed=2):
    spec = models.get_spec(name)
    weights = models.init_weights(spec, seed)
    model = models.build_hf_model(spec, seed, device="cuda",
                                  weights={k: v.cuda() for k, v in weights.items()})
    wrapper = (DecodeStep(model, capacity) if kind == "decode_step"
               else StatefulDecoder(model, capacity)).eval()
    cfg, ow = oracle_config(spec), oracle_weights(weights, models.inv_freq_buffer(spec))
    return spec, wrapper, cfg, ow


@pytest.mark.parametrize("name,kind,batch", [
    ("tiny-llama", "stateful", 2), ("tiny-llama", "decode_step", 1), ("tiny-qwen2", "stateful", 4),
    ("tiny-gemma", "decode_step", 2), ("tiny-mha", "stateful", 8),
])
def test_compiled_decode_matches_oracle(name, kind, batch):
    capacity, calls = 12, 6
    spec, wrapper, cfg, ow = _setup(name, kind, batch, capacity)
    backend = make_backend(mode="decode")
    torch._dynamo.reset()
    step = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    state = wrapper.make_state(batch, device="cuda")
    ref_state = oracle.make_state(cfg, batch, capacity)
    generator = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for call in range(calls):
            ids = torch.randint(0, spec.vocab, (batch, 1), generator=generator)
            pos = torch.full((batch, 1), call, dtype=torch.int64)
            ref = oracle.decode_step(cfg, ow, ids, pos, ref_state)
            got = step(ids.cuda(), pos.cuda(), *state)
            torch.cuda.synchronize()
            assert got.shape == ref.shape and got.dtype == torch.bfloat16
            assert logits_close(got, ref)[0], (call, max_abs(got, ref))
            assert cosine(got, ref) >= LOGIT_COSINE
            assert greedy_pick_matches(got[:, -1], ref[:, -1])[0]
    decoder = backend.megabake_last_callable
    assert isinstance(decoder, BoundDecoder) and decoder.launches == calls  # one launch per call
    decoder.check()
    assert backend.megabake_last_compiled is not None
    for index in range(spec.layers):
        assert int(state[3 * index + 2]) == calls
        assert max_abs(state[3 * index][:, :calls], ref_state[3 * index][:, :calls]) <= 6e-2
        assert torch.equal(state[3 * index][:, calls:].cpu(), ref_state[3 * index][:, calls:])


def test_graphed_decode_replays():
    batch, capacity = 2, 16
    spec, wrapper, cfg, ow = _setup("tiny-llama", "stateful", batch, capacity)
    backend = make_backend(mode="decode")
    torch._dynamo.reset()
    step = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    state = wrapper.make_state(batch, device="cuda")
    ids = torch.zeros(batch, 1, dtype=torch.int64, device="cuda")
    pos = torch.zeros(batch, 1, dtype=torch.int64, device="cuda")
    with torch.no_grad():
        call = graphed(step, ids, pos, *state)
    assert all(int(t) == 0 for t in state[2::3])  # warm-up and capture left the state untouched
    ref_state = oracle.make_state(cfg, batch, capacity)
    generator = torch.Generator().manual_seed(9)
    for index in range(5):
        token = torch.randint(0, spec.vocab, (batch, 1), generator=generator)
        position = torch.full((batch, 1), index, dtype=torch.int64)
        ref = oracle.decode_step(cfg, ow, token, position, ref_state)
        ids.copy_(token)
        pos.copy_(position)
        got = call(ids, pos, *state)
        torch.cuda.synchronize()
        assert logits_close(got, ref)[0], max_abs(got, ref)
        assert greedy_pick_matches(got[:, -1], ref[:, -1])[0]
    assert all(int(t) == 5 for t in state[2::3])


def test_two_threads_share_one_compiled_callable():
    """Calls are serialised per bound callable; both threads must get right answers
    (reference ``tests/gpu/test_task29_transformer_block.py:118-124``)."""
    batch, capacity = 1, 64
    spec, wrapper, cfg, ow = _setup("tiny-llama", "stateful", batch, capacity)
    backend = make_backend(mode="decode")
    torch._dynamo.reset()
    step = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    state = wrapper.make_state(batch, device="cuda")
    ids = torch.full((batch, 1), 7, dtype=torch.int64, device="cuda")
    with torch.no_grad():
        step(ids, torch.zeros(batch, 1, dtype=torch.int64, device="cuda"), *state)  # compile
    torch.cuda.synchronize()
    errors = []

    def worker():
        try:
            with torch.no_grad():
                for _ in range(10):
                    length = int(state[2])
                    step(ids, torch.full((batch, 1), length, dtype=torch.int64, device="cuda"), *state)
                    torch.cuda.synchronize()
        except Exception as error:  # noqa: BLE001
            errors.append(error)

    threads = [threading.Thread(target=worker) for _ in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert int(state[2]) == 21  # every call appended exactly one key
    backend.megabake_last_callable.check()


@pytest.mark.parametrize("name,batch,tokens", [
    ("tiny-llama", 2, 40), ("tiny-qwen2", 1, 16), ("tiny-gemma", 2, 70), ("tiny-gemma256", 1, 130),
])
def test_compiled_prefill_matches_oracle(name, batch, tokens):
    """``torch.compile(PrefillLogits(model), backend=make_backend(mode="prefill"))``: capture,
    recognition (causal mask and positions as graph constants), prefill plan, launches."""
    from megabake_b200 import PrefillLogits

    spec = models.get_spec(name)
    weights = models.init_weights(spec, 2)
    model = models.build_hf_model(spec, 2, device="cuda",
                                  weights={k: v.cuda() for k, v in weights.items()})
    wrapper = PrefillLogits(model).eval()
    cfg, ow = oracle_config(spec), oracle_weights(weights, models.inv_freq_buffer(spec))
    backend = make_backend(mode="prefill")
    torch._dynamo.reset()
    step = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    ids = torch.randint(0, spec.vocab, (batch, tokens), generator=torch.Generator().manual_seed(9))
    with torch.no_grad():
        got = step(ids.cuda())
        again = step(ids.cuda())
    torch.cuda.synchronize()
    ref = oracle.prefill(cfg, ow, ids)
    assert got.shape == ref.shape and got.dtype == torch.bfloat16
    assert torch.equal(got, again)
    assert logits_close(got, ref)[0], max_abs(got, ref)
    for b in range(batch):
        assert cosine(got[b], ref[b]) >= LOGIT_COSINE
        assert greedy_pick_matches(got[b], ref[b])[0]
    decoder = backend.megabake_last_callable
    assert isinstance(decoder, BoundDecoder) and decoder.launches == 2
    decoder.check()
    assert backend.megabake_last_compiled.mode == "prefill"


def test_bucketed_prefill_serves_odd_prompt_lengths():
    """``bucketed(PrefillLogits(model), backend=make_backend(mode="prefill"))``: prompts of 9
    and 21 tokens run through the 16- and 32-token plans; logits at the real positions match the
    oracle's prefill of the unpadded prompt."""
    from megabake_b200 import PrefillLogits, bucketed

    spec = models.get_spec("tiny-qwen2")
    weights = models.init_weights(spec, 6)
    model = models.build_hf_model(spec, 6, device="cuda",
                                  weights={k: v.cuda() for k, v in weights.items()})
    cfg, ow = oracle_config(spec), oracle_weights(weights, models.inv_freq_buffer(spec))
    backend = make_backend(mode="prefill")
    torch._dynamo.reset()
    call = bucketed(PrefillLogits(model).eval(), backend=backend,
                    sequence_args={"input_ids": 1}, buckets=(16, 32))
    generator = torch.Generator().manual_seed(4)
    planned = []
    for length in (9, 21, 16):
        ids = torch.randint(0, spec.vocab, (2, length), generator=generator)
        got = call(ids.cuda())
        torch.cuda.synchronize()
        ref = oracle.prefill(cfg, ow, ids)
        assert got.shape == ref.shape
        assert logits_close(got, ref)[0], (length, max_abs(got, ref))
        for b in range(2):
            assert cosine(got[b], ref[b]) >= LOGIT_COSINE
            assert greedy_pick_matches(got[b, -1:], ref[b, -1:])[0]
        decoder = backend.megabake_last_callable
        assert isinstance(decoder, BoundDecoder)
        decoder.check()
        planned.append(decoder.program.tokens)  # the plan of the most recent capture
    assert planned == [16, 32, 32] and call.verified == {16, 32}  # the third call reused bucket 16


def test_second_compile_of_the_same_graph_hits_the_plan_cache(tmp_path):
    """Two wrapper instances over one model under one backend: the second compile finds the
    recognised program and the planned phase table in the backend's caches; ``dump_dir`` holds
    the captured graph, the program and the phase table; the trace lists the stages."""
    import json

    batch, capacity = 2, 12
    spec, wrapper, cfg, ow = _setup("tiny-qwen2", "stateful", batch, capacity)
    backend = make_backend(mode="decode", dump_dir=tmp_path, model_name="qwen")
    ids = torch.randint(0, spec.vocab, (batch, 1), generator=torch.Generator().manual_seed(1)).cuda()
    pos = torch.zeros(batch, 1, dtype=torch.int64, device="cuda")
    outputs = []
    for attempt in range(2):
        instance = StatefulDecoder(_hf_model_of(wrapper), capacity).eval()
        torch._dynamo.reset()
        step = torch.compile(instance, backend=backend, fullgraph=True, dynamic=False)
        state = instance.make_state(batch, device="cuda")
        with torch.no_grad():
            outputs.append(step(ids, pos, *state).clone())
        backend.megabake_last_callable.check()
        cache = backend.megabake_plan_cache
        assert (cache.misses, cache.hits) == (1, attempt)
        trace = backend.megabake_last_trace
        assert [entry["stage"] for entry in trace] == ["fx-capture", "semantic-lowering",
                                                       "planning", "runtime-binding"]
        assert trace[2]["plan_cache_hit"] == bool(attempt)
        assert backend.megabake_last_compile_us >= sum(entry["us"] for entry in trace[:2])
        assert backend.megabake_last_callable.megabake_trace is trace
    assert torch.equal(outputs[0], outputs[1])
    table = json.loads((tmp_path / "qwen.decode.phases.json").read_text())
    assert len(table["phases"]) == 5 * spec.layers + 1 and table["mode"] == "decode"
    assert (tmp_path / "qwen.decode.aten.txt").exists()
    assert (tmp_path / "qwen.decode.program.json").exists()
    # cache=False plans afresh every time
    fresh = make_backend(mode="decode", cache=False)
    torch._dynamo.reset()
    step = torch.compile(StatefulDecoder(_hf_model_of(wrapper), capacity).eval(), backend=fresh,
                         fullgraph=True, dynamic=False)
    with torch.no_grad():
        again = step(ids, pos, *wrapper.make_state(batch, device="cuda"))
    assert fresh.megabake_plan_cache is None and torch.equal(again, outputs[0])


def _hf_model_of(wrapper):
    """The Hugging Face causal LM a ``StatefulDecoder`` was built from."""
    class _Model(torch.nn.Module):
        def __init__(self, inner, head, config):
            super().__init__()
            self.model, self.lm_head, self.config = inner, head, config

    return _Model(wrapper.model, wrapper.lm_head, wrapper.config)


def test_grouped_state_order_matches_the_reference_llama_wrapper():
    """The state order of the reference's Llama wrapper (all K, all V, all lengths) against the
    fixture that wrapper itself produced."""
    import json
    from pathlib import Path

    import numpy as np

    from megabake_b200 import GroupedStateDecoder

    golden = Path(__file__).parent / "golden"
    meta = json.loads((golden / "index.json").read_text())["decode_tiny-llama_smollm"]
    data = np.load(golden / "decode_tiny-llama_smollm.npz")
    spec = models.get_spec(meta["model"])
    weights = models.init_weights(spec, meta["seed"])
    model = models.build_hf_model(spec, meta["seed"], device="cuda",
                                  weights={k: v.cuda() for k, v in weights.items()})
    wrapper = GroupedStateDecoder(model, meta["capacity"]).eval()
    state = wrapper.make_state(meta["batch"], device="cuda")
    count = spec.layers
    assert [tuple(t.shape) for t in state[2 * count:]] == [(1,)] * count      # lengths come last
    backend = make_backend(mode="decode")
    torch._dynamo.reset()
    step = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    tokens = torch.from_numpy(data["tokens"])
    with torch.no_grad():
        for call in range(meta["calls"]):
            pos = torch.full((meta["batch"], 1), call, dtype=torch.int64, device="cuda")
            got = step(tokens[:, call:call + 1].contiguous().cuda(), pos, *state)
            ref = torch.from_numpy(data["logits"][call].copy()).view(torch.bfloat16)
            assert logits_close(got, ref)[0], (call, max_abs(got, ref))
            assert greedy_pick_matches(got[:, -1], ref[:, -1])[0]
    backend.megabake_last_callable.check()
    for index in range(count):
        assert int(state[2 * count + index]) == meta["calls"]
        ref_k = torch.from_numpy(data[f"k{index}"].copy()).view(torch.bfloat16)
        assert max_abs(state[index].cpu(), ref_k) <= 6e-2
