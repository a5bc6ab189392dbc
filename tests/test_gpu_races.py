"""Race, reuse and wait-limit evidence that needs no sanitizer.

* Poisoned workspace: every byte of the plan's workspace that is not declared "starts at zero",
  and the logits buffer, are filled with 0xE5 before a launch; the results must not change (the
  reference poisons its workspace the same way, ``src/megabake/compiler.py:1972-1973``,
  ``tests/gpu/test_task29_transformer_block.py:116-124``).
* Distinct buffers: the same model planned with activation buffers of its own for every layer
  against the normal plan that reuses one set: bit-identical logits and KV state (reference
  ``src/megabake/compiler.py:227-241``).  A phase that read a buffer too early or wrote it too
  late shows up as a difference.
* Wait limit: a consumer whose producer never stores (a flag nothing sets) gives up after the
  plan's limit, the kernel RETURNS ``MB_ST_HANDOFF_TIMEOUT`` through the status word, the context
  stays usable and the next plan runs.
"""

import time

import pytest
import torch

from megabake_b200 import models
from megabake_b200 import runtime as rt
from megabake_b200.engine import BoundDecoder
from megabake_b200.planner import PlannerOptions, plan_decode
from tests.helpers import PhaseRunner
from tests.test_gpu_bodies import _bf16, _gemv_phase, _ref_linear

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]


def _decoder(name, batch, capacity, options, seed=3):
    spec = models.get_spec(name)
    weights = {k: v.cuda() for k, v in models.init_weights(spec, seed).items()}
    state = models.make_state(spec, batch, capacity, "cuda")
    ids = torch.zeros(batch, 1, dtype=torch.int64, device="cuda")
    pos = torch.zeros(batch, 1, dtype=torch.int64, device="cuda")
    args = models.direct_arguments(spec, weights, models.inv_freq_buffer(spec).cuda(), ids, pos,
                                   state)
    layout = plan_decode(models.direct_program(spec, batch, capacity), options)
    return spec, BoundDecoder(layout, args), args, ids, pos, state


def _run_steps(decoder, args, ids, pos, tokens, poison=None):
    outputs = []
    for step in range(tokens.shape[1]):
        ids.copy_(tokens[:, step:step + 1])
        pos.fill_(step)
        if poison is not None:
            poison(decoder)
        logits = torch.empty(decoder.program.batch, 1, decoder.program.vocab, dtype=torch.bfloat16,
                             device="cuda")
        if poison is not None:
            logits.view(torch.uint8).fill_(0xE5)
        decoder.launch_into(ids, pos, logits)
        decoder.check()
        outputs.append(logits.clone())
    return outputs


@pytest.mark.parametrize("name,batch,cell_limit", [
    ("tiny-llama", 3, 0), ("tiny-qwen2", 8, 0), ("tiny-gemma", 2, 0), ("tiny-qwen2", 4, 1 << 20),
])
def test_poisoned_workspace_changes_nothing(name, batch, cell_limit):
    options = PlannerOptions(cell_limit=cell_limit)
    spec, clean, args, ids, pos, state = _decoder(name, batch, 16, options)
    tokens = torch.randint(0, spec.vocab, (batch, 5), generator=torch.Generator().manual_seed(2)).cuda()
    expected = _run_steps(clean, args, ids, pos, tokens)
    expected_state = [t.clone() for t in state]
    spec, dirty, args, ids, pos, state = _decoder(name, batch, 16, options)
    keep = dirty.layout.zero_ranges  # only the attention arrival counters must start at zero ...
    counters = [s for s in dirty.layout.slots if s.name == "attention_arrivals"]
    assert len(counters) == 1

    def poison(decoder):
        saved = decoder.workspace[counters[0].offset: counters[0].offset + 256].clone()
        decoder.workspace.fill_(0xE5)
        decoder.workspace[counters[0].offset: counters[0].offset + 256] = saved

    got = _run_steps(dirty, args, ids, pos, tokens, poison=poison)
    for a, b in zip(expected, got):
        assert torch.equal(a, b)
    for a, b in zip(expected_state, state):
        assert torch.equal(a, b)
    assert keep  # (the cell buffers are zeroed at creation too; poisoning them later is harmless)


@pytest.mark.parametrize("name,batch,cell_limit", [
    ("tiny-llama", 2, 0), ("tiny-qwen2", 8, 0), ("tiny-mha", 4, 1 << 20),
])
def test_distinct_buffers_give_identical_results(name, batch, cell_limit):
    shared = _decoder(name, batch, 16, PlannerOptions(cell_limit=cell_limit))
    own = _decoder(name, batch, 16, PlannerOptions(cell_limit=cell_limit, distinct_buffers=True))
    assert own[1].layout.workspace_bytes > shared[1].layout.workspace_bytes
    spec = shared[0]
    tokens = torch.randint(0, spec.vocab, (batch, 6), generator=torch.Generator().manual_seed(4)).cuda()
    a = _run_steps(*shared[1:5], tokens)
    b = _run_steps(*own[1:5], tokens)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    for x, y in zip(shared[5], own[5]):
        assert torch.equal(x, y)


def test_a_wait_that_runs_out_returns_a_status():
    """Phase 1 polls cells that phase 0 (a no-op) never writes.  With a 40 ms limit the kernel
    must come back by itself with MB_ST_HANDOFF_TIMEOUT; afterwards another plan runs normally."""
    rows, k, n = 2, 256, 512
    x_cells = torch.zeros(rows * k // 2, dtype=torch.int64, device="cuda")   # sequence numbers: 0
    w = _bf16(n, k, scale=0.05, seed=2)
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    nop = rt.Phase.blank(rt.BODY_NOP, 0)
    phase = _gemv_phase(runner, x=x_cells, segs=[(w, None, out)], k=k, rows=rows)
    phase.i[rt.GV_I_CELLS] = rt.CELLS_X
    phase.i[rt.GV_I_X_SOURCE] = 0
    started = time.perf_counter()
    plan = runner.run([nop, phase], rows * (k + 32) * 2, wait_limit_ms=40)
    elapsed = time.perf_counter() - started
    status = plan.status()
    assert status.code == 7 and status.phase == 1        # MB_ST_HANDOFF_TIMEOUT in the GEMV phase
    assert status.calls == 0                              # the launch did not complete
    assert elapsed < 5.0
    plan.reset()
    assert plan.status().code == 0
    # the context is healthy: an ordinary plan computes the right thing
    x = _bf16(rows, k, seed=1)
    good = PhaseRunner()
    plan = good.run([_gemv_phase(good, x=x, segs=[(w, None, out)], k=k, rows=rows)],
                    rows * (k + 32) * 2)
    assert plan.status().code == 0
    ref = _ref_linear(x, w)
    assert (out != ref).float().mean() < 0.05


def test_a_faulted_launch_leaves_the_state_alone():
    """A token outside the embedding table is recorded in phase 0.  Waits that are still spinning
    see the status and drain; CTAs that get through reach the end of the launch, where the valid
    lengths are advanced only if no fault was recorded: the KV state still describes the step
    before, and after ``check()`` has reset the plan the corrected call runs from there."""
    from megabake_b200 import CompilerError

    spec, decoder, args, ids, pos, state = _decoder("tiny-llama", 2, 8, PlannerOptions())
    ids.fill_(spec.vocab + 5)
    started = time.perf_counter()
    logits = torch.empty(2, 1, spec.vocab, dtype=torch.bfloat16, device="cuda")
    decoder.launch_into(ids, pos, logits)
    with pytest.raises(CompilerError):
        decoder.check()
    assert time.perf_counter() - started < 3.0
    ids.fill_(1)
    decoder.launch_into(ids, pos, logits)                 # recovered by check(): runs again
    decoder.check()
    assert int(state[2]) == 1
