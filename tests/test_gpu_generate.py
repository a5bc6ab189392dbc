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
