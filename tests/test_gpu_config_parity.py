"""Parity at the real shapes of the benchmark configurations: the CUDA path (through the C ABI)
against the CPU oracle on the same seeded weights, the same token ids and the *same* KV tensors.

Decode configurations with thousands of cached keys start from seeded random cache rows (the
reference's own long-context tests do the same, ``tests/gpu/test_table_gemm.py:159-162``; a CPU
prefill of 4,096-8,192 keys would take minutes per model): the rows are drawn once, uploaded to
the GPU and handed to the oracle, then both run the same decode steps, teacher-forced with the
oracle's picks.  Checked per step: greedy ids, logits (max-abs and cosine), the appended K/V rows,
every other cache row byte-equal, the valid lengths.  Prefill of the gemma-2b shape is compared
at the last position and at a strided sample of positions.

Every case prints its error statistics (max-abs, cosine, histogram of the error in bf16 ulps of
the reference logit, rows the two-ulp tie rule decided) and, when ``MEGABAKE_B200_REPORT_DIR``
names a directory, writes them there as JSON.
"""

import json
import os
from pathlib import Path

import pytest
import torch

from megabake_b200 import models
from megabake_b200.engine import BoundDecoder
from megabake_b200.planner import PlannerOptions, plan_decode, plan_prefill
from oracle import decoder_oracle as oracle
from oracle.adapters import oracle_config, oracle_weights
from tests.helpers import (LOGIT_COSINE, cosine, greedy_pick_matches, logits_close, max_abs,
                           ulp_histogram)

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(900)]


def _report(name: str, record: dict) -> None:
    print(f"parity {name}: " + json.dumps(record))
    target = os.environ.get("MEGABAKE_B200_REPORT_DIR")
    if target:
        directory = Path(target)
        directory.mkdir(parents=True, exist_ok=True)
        (directory / f"parity_{name}.json").write_text(json.dumps(record, indent=1) + "\n")


def _random_cache(spec, batch, capacity, keys, seed):
    """Seeded N(0, 1) rows in the first ``keys`` rows of every cache, drawn on the GPU."""
    generator = torch.Generator(device="cuda").manual_seed(seed)
    state = models.make_state(spec, batch, capacity, "cuda")
    for index in range(spec.layers):
        for tensor in state[3 * index: 3 * index + 2]:
            tensor[:, :keys].normal_(0.0, 1.0, generator=generator)
        state[3 * index + 2].fill_(keys)
    return state


DECODE_CASES = [
    # name, preset, layers (None = all), batch, cached keys
    ("qwen2-0.5b-b1-k4096", "qwen2-0.5b", None, 1, 4096),
    ("qwen2-0.5b-b4-k4096", "qwen2-0.5b", None, 4, 4096),
    ("qwen2-0.5b-b8-k4096", "qwen2-0.5b", None, 8, 4096),
    ("llama-3.2-1b-b1-k512", "llama-3.2-1b", None, 1, 512),
    ("llama-3.2-1b-b1-k8192", "llama-3.2-1b", None, 1, 8192),
    ("smollm-1.7b-b1-k8192", "smollm-1.7b", None, 1, 8192),
    # batch 8 at 8,192 keys holds 12.9 GB of KV state with all 24 layers; the host copy the
    # oracle needs is kept to a sixth of that: real widths, 4 layers
    ("smollm-1.7b-b8-k8192-4layers", "smollm-1.7b", 4, 8, 8192),
]


@pytest.mark.parametrize("name,preset,layers,batch,keys", DECODE_CASES,
                         ids=[case[0] for case in DECODE_CASES])
def test_decode_config_matches_oracle(name, preset, layers, batch, keys):
    steps = 2
    spec = models.get_spec(preset) if layers is None else models.get_spec(preset, layers=layers)
    capacity = keys + steps + 6
    weights = models.init_weights(spec, seed=11)
    inv_freq = models.inv_freq_buffer(spec)
    cfg, ow = oracle_config(spec), oracle_weights(weights, inv_freq)
    dev_weights = {k: v.cuda() for k, v in weights.items()}
    state = _random_cache(spec, batch, capacity, keys, seed=23)
    before = [t.clone() for t in state]                  # device copy of the initial state
    ref_state = [t.cpu() for t in state]
    ids = torch.zeros(batch, 1, dtype=torch.int64, device="cuda")
    pos = torch.zeros(batch, 1, dtype=torch.int64, device="cuda")
    args = models.direct_arguments(spec, dev_weights, inv_freq.cuda(), ids, pos, state)
    decoder = BoundDecoder(plan_decode(models.direct_program(spec, batch, capacity),
                                       PlannerOptions()), args)
    token = torch.randint(0, spec.vocab, (batch, 1), generator=torch.Generator().manual_seed(5))
    record = {"workload": name, "steps": [], "batch": batch, "cached_keys": keys,
              "layers": spec.layers}
    with torch.no_grad():
        for step in range(steps):
            position = torch.full((batch, 1), keys + step, dtype=torch.int64)
            reference = oracle.decode_step(cfg, ow, token, position, ref_state)
            ids.copy_(token)
            pos.copy_(position)
            logits = decoder(*args)
            decoder.check()
            got = logits.cpu()
            ok, worst = logits_close(got, reference)
            similarity = cosine(got, reference)
            picks_ok, ties = greedy_pick_matches(got[:, -1], reference[:, -1])
            record["steps"].append({
                "max_abs": worst, "cosine": similarity, "tie_rule_rows": ties,
                "ulp_histogram": ulp_histogram(got, reference),
                "max_abs_logit": float(reference.float().abs().max()),
            })
            assert ok, (name, step, worst)
            assert similarity >= LOGIT_COSINE, (name, step, similarity)
            assert picks_ok, (name, step)
            token = reference[:, -1].float().argmax(-1, keepdim=True)
    used = keys + steps
    for index in range(spec.layers):
        kc, vc, ln = state[3 * index: 3 * index + 3]
        k0, v0, _ = before[3 * index: 3 * index + 3]
        rk, rv, rl = ref_state[3 * index: 3 * index + 3]
        assert int(ln) == int(rl) == used
        # rows that were cached before and rows past the appended ones: byte-equal
        assert torch.equal(kc[:, :keys], k0[:, :keys]) and torch.equal(vc[:, :keys], v0[:, :keys])
        assert torch.equal(kc[:, used:], k0[:, used:]) and torch.equal(vc[:, used:], v0[:, used:])
        new_k, new_v = kc[:, keys:used].cpu(), vc[:, keys:used].cpu()
        assert max_abs(new_k, rk[:, keys:used]) <= 6e-2
        assert max_abs(new_v, rv[:, keys:used]) <= 6e-2
        assert cosine(new_k, rk[:, keys:used]) > 0.9999
        assert cosine(new_v, rv[:, keys:used]) > 0.9999
    record["kv"] = "appended rows within 6e-2 / cosine > 0.9999, all other rows byte-equal"
    _report(name, record)
    decoder.close()


@pytest.mark.parametrize("tokens", [128, 512, 2048])
def test_gemma_2b_prefill_matches_oracle(tokens):
    spec = models.get_spec("gemma-2b")
    weights = models.init_weights(spec, seed=11)
    inv_freq = models.inv_freq_buffer(spec)
    prompt = torch.randint(0, spec.vocab, (1, tokens), generator=torch.Generator().manual_seed(tokens))
    with torch.no_grad():
        reference = oracle.prefill(oracle_config(spec), oracle_weights(weights, inv_freq), prompt)
    dev_weights = {k: v.cuda() for k, v in weights.items()}
    args = models.direct_prefill_arguments(spec, dev_weights, inv_freq.cuda(), prompt.cuda())
    bound = BoundDecoder(plan_prefill(models.direct_prefill_program(spec, 1, tokens)), args)
    logits = bound(*args)
    bound.check()
    # the last position (the one a generation loop uses) and every 64th position
    sample = sorted(set(range(0, tokens, 64)) | {tokens - 1})
    got = logits[:, sample].cpu()
    ref = reference[:, sample]
    ok, worst = logits_close(got, ref)
    record = {"workload": f"gemma-2b-prefill-t{tokens}", "positions_checked": len(sample),
              "max_abs": worst, "cosine_worst": min(cosine(got[0, i], ref[0, i])
                                                    for i in range(len(sample))),
              "ulp_histogram": ulp_histogram(got, ref),
              "max_abs_logit": float(ref.float().abs().max())}
    picks_ok, ties = greedy_pick_matches(got[0], ref[0])
    record["tie_rule_rows"] = ties
    _report(record["workload"], record)
    assert ok, worst
    assert record["cosine_worst"] >= LOGIT_COSINE, record["cosine_worst"]
    assert picks_ok
    bound.close()
