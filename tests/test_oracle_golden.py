"""Pins the CPU oracle to the reference: every fixture under tests/golden/ was produced by the
reference's own operators and decode wrappers (see make_golden.py); the oracle must reproduce
them bit for bit from the same seeds."""

import json
from pathlib import Path

import numpy as np
import pytest
import torch

from megabake_b200 import models
from oracle import decoder_oracle as oracle
from oracle.adapters import oracle_config, oracle_weights

GOLDEN = Path(__file__).resolve().parent / "golden"
INDEX = json.loads((GOLDEN / "index.json").read_text())


def from_bits(array: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(array.copy()).view(torch.bfloat16)


def _setup(name, seed):
    spec = models.get_spec(name)
    weights = models.init_weights(spec, seed)
    inv = models.inv_freq_buffer(spec)
    return spec, oracle_config(spec), oracle_weights(weights, inv)


DECODE_CASES = sorted(k for k in INDEX if k.startswith("decode_"))


@pytest.mark.parametrize("key", DECODE_CASES)
def test_decode_matches_reference_wrappers(key):
    meta = INDEX[key]
    data = np.load(GOLDEN / f"{key}.npz")
    spec, cfg, ow = _setup(meta["model"], meta["seed"])
    state = oracle.make_state(cfg, meta["batch"], meta["capacity"])
    tokens = torch.from_numpy(data["tokens"])
    for call in range(meta["calls"]):
        pos = torch.full((meta["batch"], 1), call, dtype=torch.int64)
        logits = oracle.decode_step(cfg, ow, tokens[:, call:call + 1].contiguous(), pos, state)
        assert torch.equal(logits, from_bits(data["logits"][call])), (key, call)
    for index in range(spec.layers):
        assert torch.equal(state[3 * index], from_bits(data[f"k{index}"]))
        assert torch.equal(state[3 * index + 1], from_bits(data[f"v{index}"]))
        assert int(state[3 * index + 2]) == int(data["lengths"][index]) == meta["calls"]


def test_config1_protocol_matches_reference():
    meta = INDEX["protocol_smollm-135m"]
    data = np.load(GOLDEN / "protocol_smollm-135m.npz")
    spec, cfg, ow = _setup(meta["model"], meta["seed"])
    prompt = torch.from_numpy(data["prompt"])
    ids, logits, state = oracle.greedy_decode(cfg, ow, prompt, meta["steps"], meta["capacity"])
    assert ids[0].tolist() == data["picks"].tolist()
    assert torch.equal(logits[-1], from_bits(data["last_logits"]))
    used = meta["prompt_len"] + meta["steps"]
    assert torch.equal(state[0][:, :used], from_bits(data["k0"]))
    assert torch.equal(state[3 * (spec.layers - 1) + 1][:, :used], from_bits(data["v_last"]))
    # the greedy steps keep a margin of several bf16 ulps, so exact-id parity is meaningful
    margins = data["top2"][meta["prompt_len"] - 1:, 0] - data["top2"][meta["prompt_len"] - 1:, 1]
    assert float(margins.min()) >= 0.1


@pytest.mark.parametrize("tag", ["gqa", "mha", "mqa"])
def test_kv_attention_matches_reference_op(tag):
    data = np.load(GOLDEN / "ops.npz")
    get = lambda name: from_bits(data[f"kv_{tag}_{name}"])  # noqa: E731
    kc, vc = get("kc_in").clone(), get("vc_in").clone()
    length = torch.tensor([int(data[f"kv_{tag}_len_in"][0])], dtype=torch.int32)
    out = oracle.kv_attention(get("q"), get("k"), get("v"), kc, vc, length)
    assert torch.equal(out, get("out"))
    assert torch.equal(kc, get("kc_out")) and torch.equal(vc, get("vc_out"))
    assert int(length) == int(data[f"kv_{tag}_len_out"][0])


@pytest.mark.parametrize("tag", ["causal", "mqa256"])
def test_prefill_attention_matches_reference_op(tag):
    data = np.load(GOLDEN / "ops.npz")
    get = lambda name: from_bits(data[f"at_{tag}_{name}"])  # noqa: E731
    q = get("q")
    out = oracle.prefill_attention(q, get("k"), get("v"), get("mask"), q.shape[-1] ** -0.5)
    assert torch.equal(out, get("out"))
    # the oracle's own causal mask is the mask the fixtures were made with
    assert torch.equal(oracle.causal_mask(q.shape[0], q.shape[1]).contiguous(), get("mask"))


@pytest.mark.parametrize("key", sorted(k for k in INDEX if k.startswith("prefill_")))
def test_prefill_matches_reference(key):
    meta = INDEX[key]
    data = np.load(GOLDEN / f"{key}.npz")
    _, cfg, ow = _setup(meta["model"], meta["seed"])
    logits = oracle.prefill(cfg, ow, torch.from_numpy(data["tokens"]))
    assert torch.equal(logits, from_bits(data["logits"]))


def test_product_operators_match_reference_ops():
    """The package's own eager definitions of the two declared operators (what runs outside a
    compiled megakernel) against the same fixtures."""
    import megabake_b200.ops  # noqa: F401  (registers torch.ops.megabake.*)

    data = np.load(GOLDEN / "ops.npz")
    for tag in ("gqa", "mha", "mqa"):
        get = lambda name: from_bits(data[f"kv_{tag}_{name}"])  # noqa: E731
        kc, vc = get("kc_in").clone(), get("vc_in").clone()
        length = torch.tensor([int(data[f"kv_{tag}_len_in"][0])], dtype=torch.int32)
        out = torch.ops.megabake.kv_attention(get("q"), get("k"), get("v"), kc, vc, length)
        assert torch.equal(out, get("out")) and torch.equal(kc, get("kc_out"))
        assert int(length) == int(data[f"kv_{tag}_len_out"][0])
    for tag in ("causal", "mqa256"):
        get = lambda name: from_bits(data[f"at_{tag}_{name}"])  # noqa: E731
        q = get("q")
        out = torch.ops.megabake.attention(q, get("k"), get("v"), get("mask"), q.shape[-1] ** -0.5)
        assert torch.equal(out, get("out"))


@pytest.mark.parametrize("tag", ["gqa", "mqa"])
def test_per_row_lengths_match_the_reference_operator_row_by_row(tag):
    """``valid_length`` of shape ``[batch]``: the fixture holds the reference's operator called on
    every row alone with that row's length; the oracle and the eager definition of
    ``megabake::kv_attention`` must reproduce outputs, caches and lengths bit for bit."""
    import megabake_b200  # noqa: F401  (registers the operator)

    data = np.load(GOLDEN / "ops_per_row.npz")
    for implementation in (oracle.kv_attention, torch.ops.megabake.kv_attention):
        q, k, v = (from_bits(data[f"{tag}_{n}"]) for n in ("q", "k", "v"))
        kc, vc = from_bits(data[f"{tag}_kc_in"]), from_bits(data[f"{tag}_vc_in"])
        lengths = torch.from_numpy(data[f"{tag}_len_in"]).to(torch.int32)
        out = implementation(q, k, v, kc, vc, lengths)
        assert torch.equal(out, from_bits(data[f"{tag}_out"]))
        assert torch.equal(kc, from_bits(data[f"{tag}_kc_out"]))
        assert torch.equal(vc, from_bits(data[f"{tag}_vc_out"]))
        assert lengths.tolist() == data[f"{tag}_len_out"].tolist()
