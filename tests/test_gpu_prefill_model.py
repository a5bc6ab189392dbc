"""Whole-model prefill parity: the prefill plan (tcgen05 GEMMs, prefill attention, row kernels;
through the C ABI) against the CPU oracle and against the fixtures the reference produced.

Bar: logits max-abs <= 3e-2 (two bf16 steps for large logits) and cosine >= 0.9999 per
position; the arg-max of every position equal to the oracle's unless its two best logits tie
within two bf16 steps.
"""

import json
from pathlib import Path

import numpy as np
import pytest
import torch

from megabake_b200 import models
from megabake_b200.engine import BoundDecoder
from megabake_b200.planner import plan_prefill
from oracle import decoder_oracle as oracle
from oracle.adapters import oracle_config, oracle_weights
from tests.helpers import cosine, greedy_pick_matches, logits_close

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]

GOLDEN = Path(__file__).parent / "golden"
INDEX = json.loads((GOLDEN / "index.json").read_text())


def from_bits(array) -> torch.Tensor:
    return torch.from_numpy(array.copy()).view(torch.bfloat16)


def _prefill_on_gpu(name, seed, tokens):
    spec = models.get_spec(name)
    weights = models.init_weights(spec, seed)
    inv_freq = models.inv_freq_buffer(spec)
    batch, length = tokens.shape
    layout = plan_prefill(models.direct_prefill_program(spec, batch, length))
    ids = tokens.cuda()
    args = models.direct_prefill_arguments(spec, {k: v.cuda() for k, v in weights.items()},
                                           inv_freq.cuda(), ids)
    bound = BoundDecoder(layout, args)
    logits = bound(*args)
    bound.check()
    again = bound(*args)          # a second launch of the same plan gives the same bits
    bound.check()
    assert torch.equal(logits, again)
    return spec, weights, inv_freq, logits.cpu()


def _assert_close(logits, reference):
    batch, length, vocab = reference.shape
    ok, worst = logits_close(logits, reference)
    assert ok, worst
    for b in range(batch):
        assert cosine(logits[b], reference[b]) > 0.9999
        picks, _ = greedy_pick_matches(logits[b], reference[b])
        assert picks


@pytest.mark.parametrize("name,batch,length", [
    ("tiny-llama", 1, 16), ("tiny-llama", 2, 70), ("tiny-llama3", 1, 33), ("tiny-qwen2", 2, 10),
    ("tiny-mha", 1, 130), ("tiny-gemma", 2, 12), ("tiny-gemma256", 1, 200),
])
def test_tiny_prefill_matches_oracle(name, batch, length):
    spec = models.get_spec(name)
    tokens = torch.randint(0, spec.vocab, (batch, length),
                           generator=torch.Generator().manual_seed(length))
    spec, weights, inv_freq, logits = _prefill_on_gpu(name, 3, tokens)
    reference = oracle.prefill(oracle_config(spec), oracle_weights(weights, inv_freq), tokens)
    _assert_close(logits, reference)


@pytest.mark.parametrize("key", sorted(k for k in INDEX if k.startswith("prefill_")))
def test_prefill_matches_reference_fixture(key):
    """Logits the reference's declared attention op + Hugging Face eager produced."""
    meta = INDEX[key]
    data = np.load(GOLDEN / f"{key}.npz")
    tokens = torch.from_numpy(data["tokens"])
    _, _, _, logits = _prefill_on_gpu(meta["model"], meta["seed"], tokens)
    _assert_close(logits, from_bits(data["logits"]))


def test_prefill_chained_launches_give_the_same_bits(monkeypatch):
    """Programmatic dependent launch between the phases (on for plain stream launches, off
    under graph capture) changes when a kernel's prologue runs, never what it reads."""
    spec = models.get_spec("tiny-gemma256")
    tokens = torch.randint(0, spec.vocab, (2, 150), generator=torch.Generator().manual_seed(5))
    monkeypatch.setenv("MEGABAKE_B200_PREFILL_CHAIN", "0")
    _, _, _, plain = _prefill_on_gpu("tiny-gemma256", 3, tokens)
    monkeypatch.setenv("MEGABAKE_B200_PREFILL_CHAIN", "1")
    _, _, _, chained = _prefill_on_gpu("tiny-gemma256", 3, tokens)
    assert torch.equal(plain, chained)


def test_plan_reports_its_kernel_launches(monkeypatch):
    """`mb_plan_info.launches`: one kernel per phase, plus one per attention phase whose keys are
    shared out over several CTAs (statistics launch + values launch)."""
    spec = models.get_spec("tiny-llama")
    weights = models.init_weights(spec, 1)
    layout = plan_prefill(models.direct_prefill_program(spec, 1, 300))
    ids = torch.zeros((1, 300), dtype=torch.int64, device="cuda")
    args = models.direct_prefill_arguments(spec, {k: v.cuda() for k, v in weights.items()},
                                           models.inv_freq_buffer(spec).cuda(), ids)
    monkeypatch.setenv("MEGABAKE_B200_ATTN_PARTS", "0")
    assert BoundDecoder(layout, args).plan.launches == len(layout.phases)
    monkeypatch.delenv("MEGABAKE_B200_ATTN_PARTS")
    monkeypatch.setenv("MEGABAKE_B200_ATTN_CHUNK", "2")
    assert BoundDecoder(layout, args).plan.launches == len(layout.phases) + spec.layers


def test_prefill_reports_bad_token():
    from megabake_b200.diagnostics import CompilerError

    spec = models.get_spec("tiny-llama")
    weights = models.init_weights(spec, 1)
    layout = plan_prefill(models.direct_prefill_program(spec, 1, 8))
    ids = torch.full((1, 8), spec.vocab, dtype=torch.int64, device="cuda")
    args = models.direct_prefill_arguments(spec, {k: v.cuda() for k, v in weights.items()},
                                           models.inv_freq_buffer(spec).cuda(), ids)
    bound = BoundDecoder(layout, args)
    bound(*args)
    with pytest.raises(CompilerError):
        bound.check()
    ids.zero_()
    bound(*args)                  # usable again after the fault was reported
    bound.check()
