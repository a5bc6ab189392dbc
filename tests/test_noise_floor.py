"""How far apart two CORRECT bf16 forwards are: the evidence behind the logit bounds of the GPU
parity tests.

The parity contract asks for max-abs <= 3e-2 and cosine >= 0.9999 against the eager bf16 forward.
Whether any implementation that accumulates in a different fp32 order can meet that depends on
the model's depth and on the size of its logits, so it is measured here, on the CPU, with the
oracle itself: the 32-prompt + 32-step protocol of the SmolLM-135M shape (30 layers) is run with
the eager bf16 GEMMs and again with every GEMM replaced by

* an exact one (fp64 accumulation, rounded to bf16 once) -- the best any kernel can do,
* an fp32 one (operands widened, fp32 library GEMM, rounded once),
* an fp32 one that adds the reduction up in eight blocks, left to right (a different order),

each variant teacher-forced with the eager forward's tokens.  The distances between these
forwards are the floor under which no kernel can be asked to stay; the bounds asserted by
``tests/test_gpu_decode_model.py::test_smollm_135m_protocol`` are checked against them here, so
that they are neither tighter than the floor nor looser than about twice it.
"""

import pytest
import torch

from megabake_b200 import models
from oracle import decoder_oracle as oracle
from oracle.adapters import oracle_config, oracle_weights
from tests.helpers import LOGIT_MAX_ABS, cosine, max_abs

PROMPT, STEPS, CAPACITY = 32, 32, 96


def _exact(x, weight, bias=None):
    acc = x.double() @ weight.double().t()
    return (acc if bias is None else acc + bias.double()).to(x.dtype)


def _fp32(x, weight, bias=None):
    acc = x.float() @ weight.float().t()
    return (acc if bias is None else acc + bias.float()).to(x.dtype)


def _blocked(x, weight, bias=None):
    k = x.shape[-1]
    acc = torch.zeros(*x.shape[:-1], weight.shape[0], dtype=torch.float32)
    for start in range(0, k, max(32, k // 8)):
        stop = min(k, start + max(32, k // 8))
        acc = acc + x[..., start:stop].float() @ weight[:, start:stop].float().t()
    return (acc if bias is None else acc + bias.float()).to(x.dtype)


@pytest.fixture(scope="module")
def protocol():
    torch.set_num_threads(8)
    spec = models.get_spec("smollm-135m")
    weights = models.init_weights(spec, 1)
    cfg, ow = oracle_config(spec), oracle_weights(weights, models.inv_freq_buffer(spec))
    prompt = torch.randint(0, spec.vocab, (1, PROMPT), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ids, logits, _ = oracle.greedy_decode(cfg, ow, prompt, STEPS, CAPACITY)
    tokens = torch.cat([prompt, ids[:, PROMPT - 1:-1]], dim=1)
    return cfg, ow, tokens, logits


def _variant(protocol, linear, monkeypatch):
    cfg, ow, tokens, eager = protocol
    monkeypatch.setattr(oracle, "_linear", linear)
    state = oracle.make_state(cfg, 1, CAPACITY)
    stats = []
    with torch.no_grad():
        for call in range(PROMPT + STEPS):
            pos = torch.full((1, 1), call, dtype=torch.int64)
            got = oracle.decode_step(cfg, ow, tokens[:, call:call + 1].contiguous(), pos, state)
            stats.append((max_abs(got, eager[call]), cosine(got, eager[call]),
                          float((got.float() - eager[call].float()).abs().mean())))
    return stats


@pytest.mark.parametrize("name,linear", [("exact", _exact), ("fp32", _fp32), ("blocked", _blocked)])
def test_distance_between_correct_forwards(protocol, name, linear, monkeypatch):
    stats = _variant(protocol, linear, monkeypatch)
    worst = max(s[0] for s in stats)
    worst_cos = min(s[1] for s in stats)
    cosines = sorted(s[1] for s in stats)
    mean_abs = sum(s[2] for s in stats) / len(stats)
    within = sum(s[0] <= LOGIT_MAX_ABS for s in stats)
    print(f"noise floor, {name} GEMM vs eager bf16 GEMM over {len(stats)} calls: worst max-abs "
          f"{worst:.4f}, worst cosine {worst_cos:.6f}, median cosine {cosines[len(cosines) // 2]:.6f}, "
          f"mean abs {mean_abs:.5f}, calls within 3e-2: {within}")
    # the bounds the GPU protocol test asserts (tests/test_gpu_decode_model.py) ...
    gpu_worst, gpu_mean, gpu_worst_cos, gpu_within = 0.056, 6.5e-3, 0.9997, 0.6
    # ... hold for every correct CPU variant (they are not tighter than the floor) ...
    assert worst <= gpu_worst and mean_abs <= gpu_mean and worst_cos >= gpu_worst_cos
    assert within >= gpu_within * len(stats)
    assert cosines[len(cosines) // 2] >= 0.9999
    # ... and are within about a factor of two of it (not looser than they need to be)
    if name == "exact":
        assert worst >= gpu_worst / 2, "the max-abs bound could be tightened"
        assert 1 - worst_cos >= (1 - gpu_worst_cos) / 4, "the cosine bound could be tightened"
