"""Prefill -> decode handoff on the GPU: ``StatefulPrefill`` (compiled with ``mode="prefill"``)
fills the explicit KV state that ``StatefulDecoder`` (``mode="decode"``) continues from.

Oracle: the CPU prefill (logits, post-RoPE keys and values of every layer) followed by CPU decode
steps over a state seeded with those keys and values.
"""

import pytest
import torch

from megabake_b200 import StatefulDecoder, StatefulPrefill, make_backend, models
from oracle import decoder_oracle as oracle
from oracle.adapters import oracle_config, oracle_weights
from tests.helpers import LOGIT_COSINE, cosine, greedy_pick_matches, logits_close, max_abs

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(600)]


@pytest.mark.parametrize("name,batch,prompt", [
    ("tiny-llama", 2, 9), ("tiny-qwen2", 1, 70), ("tiny-gemma", 2, 33), ("tiny-mha", 3, 5),
])
def test_prefill_hands_the_state_to_decode(name, batch, prompt):
    capacity, steps = prompt + 8, 5
    spec = models.get_spec(name)
    weights = models.init_weights(spec, 4)
    model = models.build_hf_model(spec, 4, device="cuda",
                                  weights={k: v.cuda() for k, v in weights.items()})
    cfg, ow = oracle_config(spec), oracle_weights(weights, models.inv_freq_buffer(spec))
    generator = torch.Generator().manual_seed(11)
    ids = torch.randint(0, spec.vocab, (batch, prompt), generator=generator)

    # ---- oracle: prefill, seed a state with its keys / values, decode on
    ref_logits, ref_kv = oracle.prefill(cfg, ow, ids, return_kv=True)
    ref_state = oracle.make_state(cfg, batch, capacity)
    for index, (k, v) in enumerate(ref_kv):
        ref_state[3 * index][:, :prompt] = k
        ref_state[3 * index + 1][:, :prompt] = v
        ref_state[3 * index + 2].fill_(prompt)

    # ---- device: one compiled prefill, then compiled decode calls over the same state tensors
    prefill = StatefulPrefill(model, capacity).eval()
    decode = StatefulDecoder(model, capacity).eval()
    state = prefill.make_state(batch, device="cuda")
    torch._dynamo.reset()
    prefill_backend, decode_backend = make_backend(mode="prefill"), make_backend(mode="decode")
    prefill_fn = torch.compile(prefill, backend=prefill_backend, fullgraph=True, dynamic=False)
    decode_fn = torch.compile(decode, backend=decode_backend, fullgraph=True, dynamic=False)
    with torch.no_grad():
        logits = prefill_fn(ids.cuda(), *state)
    prefill_backend.megabake_last_callable.check()
    assert logits_close(logits, ref_logits)[0], max_abs(logits, ref_logits)
    for b in range(batch):
        assert cosine(logits[b], ref_logits[b]) >= LOGIT_COSINE
        assert greedy_pick_matches(logits[b], ref_logits[b])[0]
    for index in range(spec.layers):
        kc, vc, length = (t.cpu() for t in state[3 * index: 3 * index + 3])
        assert int(length) == prompt
        assert max_abs(kc[:, :prompt], ref_kv[index][0]) <= 6e-2
        assert max_abs(vc[:, :prompt], ref_kv[index][1]) <= 6e-2
        assert cosine(kc[:, :prompt], ref_kv[index][0]) > 0.9999
        assert not kc[:, prompt:].any() and not vc[:, prompt:].any()   # rows past the prompt untouched

    token = ref_logits[:, -1].float().argmax(-1, keepdim=True)      # teacher-forced greedy ids
    with torch.no_grad():
        for step in range(steps):
            pos = torch.full((batch, 1), prompt + step, dtype=torch.int64)
            ref = oracle.decode_step(cfg, ow, token, pos, ref_state)
            got = decode_fn(token.cuda(), pos.cuda(), *state)
            torch.cuda.synchronize()
            assert logits_close(got, ref)[0], (step, max_abs(got, ref))
            assert cosine(got, ref) >= LOGIT_COSINE
            assert greedy_pick_matches(got[:, -1], ref[:, -1])[0]
            token = ref[:, -1].float().argmax(-1, keepdim=True)
    decode_backend.megabake_last_callable.check()
    assert int(state[2].item()) == prompt + steps


def test_greedy_generator_picks_what_the_oracle_would():
    from megabake_b200 import GreedyGenerator

    spec = models.get_spec("tiny-llama")
    weights = models.init_weights(spec, 1)
    model = models.build_hf_model(spec, 1, device="cuda",
                                  weights={k: v.cuda() for k, v in weights.items()})
    cfg, ow = oracle_config(spec), oracle_weights(weights, models.inv_freq_buffer(spec))
    batch, prompt, new = 2, 12, 6
    ids = torch.randint(0, spec.vocab, (batch, prompt), generator=torch.Generator().manual_seed(1))
    torch._dynamo.reset()
    produced = GreedyGenerator(model, batch, prompt, capacity=prompt + new + 2)(ids, new).cpu()
    assert produced.shape == (batch, new)
    # replay the produced ids through the oracle: every one must be an acceptable greedy pick of
    # the oracle's logits at its position
    everything = torch.cat([ids, produced], dim=1)
    reference = oracle.prefill(cfg, ow, everything[:, :-1])
    for step in range(new):
        at = prompt - 1 + step
        chosen = torch.full((batch, spec.vocab), -1.0)
        chosen[torch.arange(batch), produced[:, step]] = 1.0      # "logits" whose argmax is the pick
        assert greedy_pick_matches(chosen, reference[:, at])[0], step


@pytest.mark.parametrize("rows,vocab", [(1, 49152), (3, 1001), (8, 151936), (2, 7)])
def test_greedy_advance_is_argmax_with_first_index_ties(rows, vocab):
    """``mb_greedy_advance`` through the C ABI: pick = first index of the row maximum, written
    into the ids the next launch reads; positions advance; picks are logged at the cursor."""
    from megabake_b200 import runtime as rt

    generator = torch.Generator().manual_seed(rows * 1000 + vocab)
    # few distinct values, so every row has many exact ties for the maximum
    logits = torch.randint(-6, 7, (rows, 1, vocab), generator=generator).float().mul(0.125)
    logits = logits.to(torch.bfloat16)
    if vocab % 8:  # rows that do not start on a 16-byte boundary take the scalar head and tail
        assert (vocab * 2) % 16 != 0
    expected = torch.stack([(row == row.max()).nonzero()[0, 0] for row in logits[:, 0].float()])
    ids = torch.full((rows, 1), -1, dtype=torch.int64, device="cuda")
    positions = torch.arange(rows, dtype=torch.int64, device="cuda").reshape(rows, 1) + 40
    log = torch.full((rows, 2), -1, dtype=torch.int64, device="cuda")
    cursor = torch.zeros(rows, dtype=torch.int32, device="cuda")
    device_logits = logits.cuda()
    for call in range(3):  # the third pick no longer fits the log: dropped, cursor still counts
        rt.greedy_advance(device_logits, ids, positions, log, cursor)
    torch.cuda.synchronize()
    assert ids.cpu().flatten().tolist() == expected.tolist()
    assert positions.cpu().flatten().tolist() == [40 + r + 3 for r in range(rows)]
    assert log.cpu().tolist() == [[int(e), int(e)] for e in expected]
    assert cursor.cpu().tolist() == [3] * rows
    # a NaN beats every number, the first one wins (torch.argmax's rule)
    device_logits[0, 0, vocab // 2] = float("nan")
    device_logits[0, 0, vocab - 1] = float("nan")
    rt.greedy_advance(device_logits, ids)
    torch.cuda.synchronize()
    assert int(ids[0, 0]) == vocab // 2


@pytest.mark.parametrize("steps_per_graph", [1, 5])
def test_device_side_loop_reproduces_the_host_loop(steps_per_graph):
    """The multi-step loop with on-device picks (decode launch + ``mb_greedy_advance`` replayed
    as one CUDA graph) must produce the ids the host-picked loop produces, and those must be
    acceptable greedy picks of the oracle's logits."""
    from megabake_b200 import GreedyGenerator

    spec = models.get_spec("tiny-qwen2")
    weights = models.init_weights(spec, 2)
    model = models.build_hf_model(spec, 2, device="cuda",
                                  weights={k: v.cuda() for k, v in weights.items()})
    cfg, ow = oracle_config(spec), oracle_weights(weights, models.inv_freq_buffer(spec))
    batch, prompt, new = 2, 10, 11
    ids = torch.randint(0, spec.vocab, (batch, prompt), generator=torch.Generator().manual_seed(5))
    torch._dynamo.reset()
    generator = GreedyGenerator(model, batch, prompt, capacity=prompt + new + 14)
    on_host = generator(ids, new).cpu()
    on_device = generator.on_device(ids, new, steps_per_graph=steps_per_graph).cpu()
    assert on_device.shape == (batch, new) and on_device.dtype == torch.int64
    assert torch.equal(on_device, on_host)
    again = generator.on_device(ids, new, steps_per_graph=steps_per_graph).cpu()  # graph reuse
    assert torch.equal(again, on_host)
    everything = torch.cat([ids, on_device], dim=1)
    reference = oracle.prefill(cfg, ow, everything[:, :-1])
    for step in range(new):
        chosen = torch.full((batch, spec.vocab), -1.0)
        chosen[torch.arange(batch), on_device[:, step]] = 1.0
        assert greedy_pick_matches(chosen, reference[:, prompt - 1 + step])[0], step
