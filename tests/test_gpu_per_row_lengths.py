"""Rows of one batch that hold different numbers of keys: ``valid_length`` int32 ``[batch]``.

The reference keeps one length for the whole batch (``fx_handler/hf_attention.py:194-196``) and
lists per-sequence lengths as future work (``docs/roadmap.md:178``).  The oracle's definition --
the shared-length operator applied to every row alone -- is pinned to the reference's operator by
``tests/golden/ops_per_row.npz``; here the CUDA path is compared with it: the attention body, a
whole model, and generation from prompts of different lengths.
"""

import math

import numpy as np
import pytest
import torch

from megabake_b200 import models
from megabake_b200 import planner as pl
from megabake_b200 import runtime as rt
from megabake_b200.engine import BoundDecoder
from megabake_b200.planner import PlannerOptions, plan_decode
from oracle import decoder_oracle as oracle
from oracle.adapters import oracle_config, oracle_weights
from tests.helpers import (LOGIT_COSINE, PhaseRunner, cosine, greedy_pick_matches, logits_close,
                           max_abs)
from tests.test_oracle_golden import GOLDEN, from_bits

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(600)]


def _attention_phase(runner, tensors, batch, heads, kv_heads, dim, capacity, exact_keys=128):
    q, k, v, kc, vc, lengths, pos, inv_freq, out = tensors
    group = heads // kv_heads
    max_chunks = max(1, min(64, math.ceil(capacity / 16)))
    partial = torch.zeros(batch * kv_heads * max_chunks * group * (dim + 2), dtype=torch.float32,
                          device="cuda")
    counters = torch.zeros(max(4, batch * kv_heads), dtype=torch.int32, device="cuda")
    ph = rt.Phase.blank(rt.BODY_ATTN_DECODE, rt.FLAG_BUMP_LENGTH)
    merge_slots = pl.attention_merge_slots(dim, group)
    for index, value in ((rt.AT_I_BATCH, batch), (rt.AT_I_HEADS, heads),
                         (rt.AT_I_KV_HEADS, kv_heads), (rt.AT_I_HEAD_DIM, dim),
                         (rt.AT_I_CAPACITY, capacity), (rt.AT_I_INVFREQ_BF16, 1),
                         (rt.AT_I_MAX_CHUNKS, max_chunks), (rt.AT_I_MERGE_SLOTS, merge_slots),
                         (rt.AT_I_EXACT_KEYS, min(capacity, exact_keys)),
                         (rt.AT_I_LEN_COUNT, batch)):
        ph.i[index] = value
    ph.f[rt.AT_F_SCALE] = dim ** -0.5
    ph.f[rt.AT_F_ROPE_SCALE] = 1.0
    for index, (name, tensor) in enumerate([
        ("q", q), ("k", k), ("v", v), ("kc", kc), ("vc", vc), ("len", lengths), ("pos", pos),
        ("invf", inv_freq), ("out", out), ("partial", partial), ("cnt", counters),
    ]):
        ph.slot[index] = runner.slot(name, tensor)
    return ph, pl.attention_scratch_bytes(dim, group, merge_slots), counters


@pytest.mark.parametrize("tag,heads,kv_heads", [("gqa", 4, 2), ("mqa", 8, 1)])
def test_attention_body_matches_the_reference_fixture(tag, heads, kv_heads):
    """Inputs and expected results come from the reference's operator called row by row; the
    queries and keys are used as they are (positions 0 with inv_freq 0: RoPE is the identity)."""
    data = np.load(GOLDEN / "ops_per_row.npz")
    q, k, v = (from_bits(data[f"{tag}_{n}"]) for n in ("q", "k", "v"))
    kc, vc = from_bits(data[f"{tag}_kc_in"]), from_bits(data[f"{tag}_vc_in"])
    lengths = torch.from_numpy(data[f"{tag}_len_in"]).to(torch.int32)
    batch, capacity, dim = kc.shape[0], kc.shape[1], kc.shape[3]
    dev = [t.cuda() for t in (q.reshape(batch, -1), k.reshape(batch, -1), v.reshape(batch, -1), kc,
                              vc, lengths, torch.zeros(batch, 1, dtype=torch.int64),
                              torch.zeros(dim // 2, dtype=torch.bfloat16))]
    out = torch.zeros(batch, heads * dim, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    ph, scratch, counters = _attention_phase(runner, dev + [out], batch, heads, kv_heads, dim,
                                             capacity)
    plan = runner.run([ph], scratch)
    assert plan.status().code == 0
    expected = from_bits(data[f"{tag}_out"]).reshape(batch, heads * dim)
    assert dev[5].cpu().tolist() == data[f"{tag}_len_out"].tolist()      # every row advanced by one
    assert torch.equal(dev[3].cpu(), from_bits(data[f"{tag}_kc_out"]))   # appended rows, bit for bit
    assert torch.equal(dev[4].cpu(), from_bits(data[f"{tag}_vc_out"]))
    assert max_abs(out, expected) <= 2e-2
    assert cosine(out, expected) > 0.9999
    assert int(counters.abs().sum()) == 0


@pytest.mark.parametrize("lengths", [(0, 5, 17, 39), (3, 200, 64, 1000), (127, 128, 129, 1),
                                     (2500, 0, 16, 15)])
@pytest.mark.parametrize("heads,kv_heads,dim", [(14, 2, 64), (4, 4, 64), (8, 1, 256)])
def test_attention_body_with_mixed_lengths(lengths, heads, kv_heads, dim):
    batch, capacity = len(lengths), max(lengths) + 4
    g = torch.Generator().manual_seed(sum(lengths) + heads)
    bf = torch.bfloat16
    q = torch.randn(batch, heads * dim, generator=g).to(bf)
    k = torch.randn(batch, kv_heads * dim, generator=g).to(bf)
    v = torch.randn(batch, kv_heads * dim, generator=g).to(bf)
    kc = torch.randn(batch, capacity, kv_heads, dim, generator=g).to(bf)
    vc = torch.randn(batch, capacity, kv_heads, dim, generator=g).to(bf)
    inv_freq = (1.0 / (10000 ** (torch.arange(0, dim, 2).float() / dim))).to(bf)
    length = torch.tensor(lengths, dtype=torch.int32)
    pos = length.to(torch.int64)[:, None].clone()
    cos, sin = oracle.rotary_tables(inv_freq, pos, 1.0)
    q_r = oracle.apply_rope(q.view(batch, 1, heads, dim), cos, sin)
    k_r = oracle.apply_rope(k.view(batch, 1, kv_heads, dim), cos, sin)
    kc_ref, vc_ref, len_ref = kc.clone(), vc.clone(), length.clone()
    ref = oracle.kv_attention(q_r, k_r, v.view(batch, 1, kv_heads, dim), kc_ref, vc_ref, len_ref)
    ref = ref.reshape(batch, heads * dim)
    dev = [t.cuda() for t in (q, k, v, kc, vc, length, pos, inv_freq)]
    out = torch.zeros(batch, heads * dim, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    ph, scratch, counters = _attention_phase(runner, dev + [out], batch, heads, kv_heads, dim,
                                             capacity)
    plan = runner.run([ph], scratch)
    st = plan.status()
    assert st.code == 0, (st.code, st.phase, st.detail)
    assert dev[5].cpu().tolist() == [n + 1 for n in lengths]
    for row, cached in enumerate(lengths):
        assert torch.equal(dev[4][row, cached].cpu(), vc_ref[row, cached])       # appended value
        assert max_abs(dev[3][row, cached], kc_ref[row, cached]) <= 0.04          # appended key
        assert torch.equal(dev[3][row, :cached].cpu(), kc[row, :cached])         # untouched rows
        assert torch.equal(dev[3][row, cached + 1:].cpu(), kc[row, cached + 1:])
        assert torch.equal(dev[4][row, cached + 1:].cpu(), vc[row, cached + 1:])
        assert max_abs(out[row], ref[row]) <= 2e-2, (row, max_abs(out[row], ref[row]))
        assert cosine(out[row], ref[row]) > 0.9999
    assert int(counters.abs().sum()) == 0


def test_one_full_row_faults_the_whole_call():
    batch, heads, kv_heads, dim, capacity = 2, 4, 2, 64, 8
    g = torch.Generator().manual_seed(0)
    bf = torch.bfloat16
    tensors = [torch.randn(batch, heads * dim, generator=g).to(bf),
               torch.randn(batch, kv_heads * dim, generator=g).to(bf),
               torch.randn(batch, kv_heads * dim, generator=g).to(bf),
               torch.randn(batch, capacity, kv_heads, dim, generator=g).to(bf),
               torch.randn(batch, capacity, kv_heads, dim, generator=g).to(bf),
               torch.tensor([3, 8], dtype=torch.int32), torch.zeros(batch, 1, dtype=torch.int64),
               torch.zeros(dim // 2, dtype=bf)]
    dev = [t.cuda() for t in tensors]
    out = torch.zeros(batch, heads * dim, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    ph, scratch, _ = _attention_phase(runner, dev + [out], batch, heads, kv_heads, dim, capacity)
    plan = runner.run([ph], scratch)
    st = plan.status()
    assert st.code == 3 and st.detail == 8        # MB_ST_KV_OVERFLOW, the offending length
    assert dev[5].cpu().tolist() == [3, 8]         # no row advanced
    assert torch.equal(dev[3].cpu(), tensors[3])   # caches untouched


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-qwen2", "tiny-gemma"])
def test_model_decode_with_a_length_per_row(name):
    spec = models.get_spec(name)
    batch, capacity, steps = 4, 48, 3
    lengths = [7, 0, 30, 16]
    weights = models.init_weights(spec, 6)
    inv_freq = models.inv_freq_buffer(spec)
    cfg, ow = oracle_config(spec), oracle_weights(weights, inv_freq)
    ref_state = oracle.make_state(cfg, batch, capacity, per_row_lengths=True)
    g = torch.Generator().manual_seed(9)
    for index in range(spec.layers):
        for tensor in ref_state[3 * index: 3 * index + 2]:
            for row, cached in enumerate(lengths):
                tensor[row, :cached] = torch.randn(cached, spec.kv_heads, spec.head_dim,
                                                   generator=g).to(torch.bfloat16)
        ref_state[3 * index + 2].copy_(torch.tensor(lengths, dtype=torch.int32))
    state = [t.clone().cuda() for t in ref_state]
    ids = torch.zeros(batch, 1, dtype=torch.int64, device="cuda")
    pos = torch.zeros(batch, 1, dtype=torch.int64, device="cuda")
    dev_weights = {k: v.cuda() for k, v in weights.items()}
    args = models.direct_arguments(spec, dev_weights, inv_freq.cuda(), ids, pos, state)
    program = models.direct_program(spec, batch, capacity, per_row_lengths=True)
    decoder = BoundDecoder(plan_decode(program, PlannerOptions()), args)
    token = torch.randint(0, spec.vocab, (batch, 1), generator=g)
    for step in range(steps):
        position = torch.tensor(lengths, dtype=torch.int64)[:, None] + step
        reference = oracle.decode_step(cfg, ow, token, position, ref_state)
        ids.copy_(token)
        pos.copy_(position)
        logits = decoder(*args).cpu()
        decoder.check()
        assert logits_close(logits, reference)[0], (step, max_abs(logits, reference))
        assert cosine(logits, reference) >= LOGIT_COSINE
        assert greedy_pick_matches(logits[:, -1], reference[:, -1])[0]
        token = reference[:, -1].float().argmax(-1, keepdim=True)
    for index in range(spec.layers):
        assert state[3 * index + 2].cpu().tolist() == [n + steps for n in lengths]
        for row, cached in enumerate(lengths):
            used = cached + steps
            assert max_abs(state[3 * index][row, :used], ref_state[3 * index][row, :used]) <= 6e-2
            assert torch.equal(state[3 * index][row, used:].cpu(), ref_state[3 * index][row, used:])


def test_generation_from_prompts_of_different_lengths():
    """One batch, four prompts of different lengths (padded at the end), through the compiled
    prefill and decode: every row must produce what the same prompt produces alone."""
    from megabake_b200.generate import GreedyGenerator

    spec = models.get_spec("tiny-llama")
    weights = models.init_weights(spec, 8)
    model = models.build_hf_model(spec, 8, device="cuda",
                                  weights={k: v.cuda() for k, v in weights.items()})
    cfg, ow = oracle_config(spec), oracle_weights(weights, models.inv_freq_buffer(spec))
    lengths = torch.tensor([5, 16, 9, 1])
    padded, new_tokens, capacity = 16, 6, 32
    g = torch.Generator().manual_seed(4)
    prompts = torch.randint(0, spec.vocab, (4, padded), generator=g)
    torch._dynamo.reset()
    generator = GreedyGenerator(model, 4, padded, capacity, per_row_lengths=True)
    got = generator(prompts, new_tokens, prompt_lengths=lengths).cpu()
    for row, length in enumerate(lengths.tolist()):
        alone = prompts[row:row + 1, :length]
        ref_ids, ref_logits, _ = oracle.greedy_decode(cfg, ow, alone, new_tokens - 1, capacity)
        expected = ref_ids[0, length - 1:]
        # free-running comparison: stop at the first position where the oracle itself is
        # undecided between its two best candidates (a bf16 tie decides differently)
        for step in range(new_tokens):
            if int(got[row, step]) == int(expected[step]):
                continue
            top = ref_logits[length - 1 + step][0, -1].float().topk(2).values
            assert float(top[0] - top[1]) <= 2 * 2.0 ** (math.floor(math.log2(abs(float(top[0])))) - 7), (
                row, step)
            break
