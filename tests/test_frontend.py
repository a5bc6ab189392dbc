"""The ``make_backend`` boundary on CPU: option validation, the FX reference forward
(``compile_kernel=False``) against eager, and decoder recognition of every model family
through both decode wrappers.  Mirrors the reference's ``tests/unit/test_frontend.py`` and
``tests/unit/test_task28_kv_state.py:195-210`` for the parts this backend keeps."""

import pytest
import torch

import megabake_b200
from megabake_b200 import CompilerError, DecodeStep, StatefulDecoder, make_backend, models
from megabake_b200.recognize import recognize_decoder


def test_option_validation_messages():
    with pytest.raises(ValueError, match="Unsupported mode 'train'"):
        make_backend(mode="train")
    with pytest.raises(ValueError, match="Unsupported fallback"):
        make_backend(fallback="eager")
    with pytest.raises(TypeError, match="cache must be a boolean"):
        make_backend(cache=1)
    with pytest.raises(TypeError, match="model_name must be a non-empty string"):
        make_backend(model_name="")
    with pytest.raises(TypeError, match="compile_kernel must be True, False, or None"):
        make_backend(compile_kernel="yes")
    with pytest.raises(ValueError, match="scheduler must be"):
        make_backend(scheduler="fifo")
    backend = make_backend(mode="decode", fallback="inductor")
    assert backend.megabake_options["mode"] == "decode"
    assert backend.__name__ == "megabake_backend"


def test_backend_rejects_dynamo_options_and_grad_inputs():
    backend = make_backend()
    graph = torch.fx.symbolic_trace(torch.nn.Identity())
    with pytest.raises(TypeError, match="Unsupported Dynamo backend options: mystery"):
        backend(graph, [torch.zeros(1)], mystery=1)
    with pytest.raises(RuntimeError, match="inference only"):
        backend(graph, [torch.zeros(1, requires_grad=True)])


def _wrapped(name, kind, capacity=12):
    spec = models.get_spec(name)
    model = models.build_hf_model(spec, seed=4)
    wrapper = (DecodeStep(model, capacity) if kind == "decode_step"
               else StatefulDecoder(model, capacity)).eval()
    return spec, wrapper


@pytest.mark.parametrize("name,kind", [
    ("tiny-llama", "stateful"), ("tiny-llama", "decode_step"), ("tiny-qwen2", "stateful"),
    ("tiny-gemma", "decode_step"), ("tiny-mha", "stateful"),
])
def test_fx_reference_forward_matches_eager(name, kind):
    spec, wrapper = _wrapped(name, kind)
    batch = 2
    eager_state, fx_state = wrapper.make_state(batch), wrapper.make_state(batch)
    backend = make_backend(mode="decode", compile_kernel=False)
    torch._dynamo.reset()
    compiled = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    generator = torch.Generator().manual_seed(0)
    with torch.no_grad():
        for call in range(3):
            ids = torch.randint(0, spec.vocab, (batch, 1), generator=generator)
            pos = torch.full((batch, 1), call, dtype=torch.int64)
            expected = wrapper(ids, pos, *eager_state)
            got = compiled(ids, pos, *fx_state)
            assert torch.equal(got, expected)
    for a, b in zip(eager_state, fx_state):
        assert torch.equal(a, b)  # caches appended and lengths advanced identically
    assert int(fx_state[2]) == 3
    prepared = backend.megabake_last_prepared
    assert prepared.graph is not None and backend.megabake_last_compiled is None


@pytest.mark.parametrize("name,kind", [
    ("tiny-llama", "stateful"), ("tiny-llama", "decode_step"), ("tiny-llama3", "decode_step"),
    ("tiny-qwen2", "stateful"), ("tiny-qwen2", "decode_step"), ("tiny-gemma", "stateful"),
    ("tiny-gemma", "decode_step"), ("tiny-gemma256", "stateful"), ("tiny-mha", "stateful"),
])
def test_recognition_recovers_the_architecture(name, kind):
    spec, wrapper = _wrapped(name, kind, capacity=20)
    batch = 3
    backend = make_backend(mode="decode", compile_kernel=False)
    torch._dynamo.reset()
    compiled = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    with torch.no_grad():
        compiled(torch.zeros(batch, 1, dtype=torch.int64), torch.zeros(batch, 1, dtype=torch.int64),
                 *wrapper.make_state(batch))
    graph = backend.megabake_last_prepared.graph
    program = recognize_decoder(graph, "decode")
    assert (program.batch, program.hidden, program.heads, program.kv_heads, program.head_dim) == (
        batch, spec.hidden, spec.heads, spec.kv_heads, spec.head_dim)
    assert (program.intermediate, program.vocab, program.capacity) == (
        spec.intermediate, spec.vocab, 20)
    assert len(program.layers) == spec.layers
    assert program.norm == spec.norm and program.activation == spec.activation
    assert program.eps == pytest.approx(spec.eps)
    assert program.inv_freq_dtype == "bf16" and program.rope_scale == 1.0
    assert (program.embed_scale_arg is not None) == (spec.family == "gemma")
    assert (program.layers[0].q_bias is not None) == spec.qkv_bias
    assert program.lm_head_weight == program.embed_weight  # tied embeddings: one graph input
    # every layer owns its own state tensors and weights
    caches = [layer.key_cache for layer in program.layers]
    assert len(set(caches)) == spec.layers
    with pytest.raises(ValueError, match="mode='prefill'"):
        recognize_decoder(graph, "prefill")


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-llama3", "tiny-qwen2", "tiny-gemma"])
def test_prefill_recognition_and_plan(name):
    from megabake_b200 import PrefillLogits
    from megabake_b200 import runtime as rt
    from megabake_b200.planner import plan_prefill

    spec = models.get_spec(name)
    wrapper = PrefillLogits(models.build_hf_model(spec, seed=1)).eval()
    backend = make_backend(mode="prefill", compile_kernel=False)
    torch._dynamo.reset()
    compiled = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    ids = torch.randint(0, spec.vocab, (2, 10), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        logits = compiled(ids)
        assert torch.equal(logits, wrapper(ids))       # the FX forward is the eager forward
    graph = backend.megabake_last_prepared.graph
    program = recognize_decoder(graph, "prefill")
    assert (program.mode, program.batch, program.tokens) == ("prefill", 2, 10)
    assert (program.hidden, program.heads, program.kv_heads, program.head_dim) == (
        spec.hidden, spec.heads, spec.kv_heads, spec.head_dim)
    assert program.causal and program.mask is None     # the graph's mask constant is causal
    assert program.position_ids is None                # positions 0..T-1 are graph constants
    assert program.softmax_scale == pytest.approx(spec.head_dim ** -0.5)
    assert len(program.layers) == spec.layers and program.activation == spec.activation
    with pytest.raises(ValueError, match="mode='decode'"):
        recognize_decoder(graph, "decode")
    layout = plan_prefill(program)
    assert layout.mode == rt.MODE_PREFILL
    assert len(layout.phases) == 1 + 8 * spec.layers + 2
    bodies = [phase.body for phase in layout.phases]
    assert bodies[0] == rt.BODY_EMBED_ROWS and bodies[-1] == rt.BODY_GEMM_TC
    assert bodies.count(rt.BODY_ATTN_PREFILL) == spec.layers
    assert bodies.count(rt.BODY_GEMM_TC) == 4 * spec.layers + 1


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-qwen2", "tiny-gemma"])
def test_stateful_prefill_fills_the_decode_state(name):
    """The handoff operator on CPU: eager and FX forwards equal the oracle's prefill bit for
    bit, the caches hold the oracle's keys and values, and the graph is recognised and planned
    with the caches as GEMM outputs."""
    from megabake_b200 import StatefulPrefill
    from megabake_b200 import runtime as rt
    from megabake_b200.planner import plan_prefill
    from oracle import decoder_oracle as oracle
    from oracle.adapters import oracle_config, oracle_weights

    spec = models.get_spec(name)
    weights = models.init_weights(spec, 3)
    wrapper = StatefulPrefill(models.build_hf_model(spec, 3, weights=weights), 24).eval()
    ids = torch.randint(0, spec.vocab, (2, 7), generator=torch.Generator().manual_seed(1))
    cfg, ow = oracle_config(spec), oracle_weights(weights, models.inv_freq_buffer(spec))
    reference, kv = oracle.prefill(cfg, ow, ids, return_kv=True)
    backend = make_backend(mode="prefill", compile_kernel=False)
    torch._dynamo.reset()
    compiled = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    for forward in (wrapper, compiled):
        state = wrapper.make_state(2)
        with torch.no_grad():
            logits = forward(ids, *state)
        assert torch.equal(logits, reference)
        for index in range(spec.layers):
            assert torch.equal(state[3 * index][:, :7], kv[index][0])
            assert torch.equal(state[3 * index + 1][:, :7], kv[index][1])
            assert int(state[3 * index + 2]) == 7 and not state[3 * index][:, 7:].any()
    program = recognize_decoder(backend.megabake_last_prepared.graph, "prefill")
    assert program.mode == "prefill" and program.causal and program.capacity == 24
    assert all(layer.key_cache >= 0 and layer.valid_length >= 0 for layer in program.layers)
    layout = plan_prefill(program)
    qkv = [ph for ph in layout.phases if ph.body == rt.BODY_GEMM_TC and ph.i[rt.GV_I_NSEG] == 3]
    assert len(qkv) == spec.layers
    assert all(ph.i[rt.GV_I_OUT_TOKENS] == 7 and ph.i[rt.GV_I_OUT_CAPACITY] == 24 for ph in qkv)


def test_unrecognised_graph_is_refused_not_rerouted():
    class NotADecoder(torch.nn.Module):
        def forward(self, x):
            return torch.relu(x) * 2

    backend = make_backend(mode="decode", compile_kernel=True, fallback="inductor")
    torch._dynamo.reset()
    compiled = torch.compile(NotADecoder(), backend=backend, fullgraph=True, dynamic=False)
    with pytest.raises(Exception) as info:
        compiled(torch.ones(4))
    error = info.value
    while error is not None and not isinstance(error, CompilerError):
        error = error.__cause__ or error.__context__
    assert isinstance(error, CompilerError)
    assert error.diagnostic.stage == "pattern-recognition"
    assert error.safe_for_fallback is False


def test_compiled_call_needs_the_gpu():
    """With compile_kernel=True on CPU tensors the call fails loudly: no CPU path exists."""
    spec, wrapper = _wrapped("tiny-llama", "stateful")
    backend = make_backend(mode="decode", compile_kernel=True)
    torch._dynamo.reset()
    compiled = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    with pytest.raises(Exception) as info, torch.no_grad():
        compiled(torch.zeros(1, 1, dtype=torch.int64), torch.zeros(1, 1, dtype=torch.int64),
                 *wrapper.make_state(1))
    error = info.value
    while error is not None and not isinstance(error, CompilerError):
        error = error.__cause__ or error.__context__
    assert isinstance(error, CompilerError) and error.diagnostic.stage == "native-library"


def test_public_names():
    for name in megabake_b200.__all__:
        assert getattr(megabake_b200, name) is not None
