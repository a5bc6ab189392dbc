"""``bucketed``: variable-length calls through fixed-shape compiled callables (host logic; the
behaviours the reference's ``src/megabake/buckets.py:49-189`` defines)."""

import pytest
import torch

from megabake_b200 import PaddingDependence, bucketed, make_backend, models


class _CausalCumulative(torch.nn.Module):
    """Position t sees positions <= t only: safe to pad at the end."""

    def forward(self, input_ids, scale=None):
        values = input_ids.float().cumsum(dim=1)
        return {"running": values if scale is None else values * scale,
                "count": torch.tensor(input_ids.shape[0])}


class _SeesEverything(torch.nn.Module):
    """Every position sees the whole row: padding changes the real positions."""

    def forward(self, input_ids):
        return input_ids.float() + input_ids.float().sum(dim=1, keepdim=True)


def test_pads_to_the_smallest_bucket_and_cuts_back():
    torch._dynamo.reset()
    call = bucketed(_CausalCumulative(), backend="eager", sequence_args={"input_ids": 1},
                    buckets=(8, 4, 16, 8))
    assert call.buckets == (4, 8, 16)
    assert [call.bucket_for(n) for n in (1, 4, 5, 8, 9, 16)] == [4, 4, 8, 8, 16, 16]
    with pytest.raises(ValueError, match="exceeds the largest bucket"):
        call.bucket_for(17)
    ids = torch.arange(1, 7).reshape(1, 6).repeat(2, 1)
    out = call(ids)
    assert out["running"].shape == (2, 6)                       # cut back from bucket 8
    assert torch.equal(out["running"], ids.float().cumsum(1))
    assert int(out["count"]) == 2                               # non-sequence outputs untouched
    assert call.verified == {8}
    exact = call(torch.ones(1, 16, dtype=torch.int64))          # exactly a bucket: no padding
    assert exact["running"].shape == (1, 16) and call.verified == {8, 16}
    keyword = call(input_ids=ids, scale=torch.tensor(2.0))      # bound by name, extras passed on
    assert torch.equal(keyword["running"], 2 * ids.float().cumsum(1))


def test_refuses_callables_whose_real_positions_see_the_padding():
    torch._dynamo.reset()
    call = bucketed(_SeesEverything(), backend="eager", sequence_args={"input_ids": 1},
                    buckets=(8,))
    with pytest.raises(PaddingDependence, match="change with the padding"):
        call(torch.ones(1, 5, dtype=torch.int64))
    unchecked = bucketed(_SeesEverything(), backend="eager", sequence_args={"input_ids": 1},
                         buckets=(8,), verify=False)
    assert unchecked(torch.ones(1, 5, dtype=torch.int64)).shape == (1, 5)


def test_argument_errors():
    with pytest.raises(ValueError, match="at least one sequence argument"):
        bucketed(_CausalCumulative(), backend="eager", sequence_args={})
    with pytest.raises(ValueError, match="positive"):
        bucketed(_CausalCumulative(), backend="eager", sequence_args={"input_ids": 1},
                 buckets=(0, 4))
    call = bucketed(_CausalCumulative(), backend="eager",
                    sequence_args={"input_ids": 1, "scale": 1}, buckets=(8,))
    with pytest.raises(ValueError, match="disagree on the length"):
        call(torch.ones(1, 5, dtype=torch.int64), torch.ones(1, 4))
    with pytest.raises(ValueError, match="exceeds the largest bucket"):
        call(torch.ones(1, 9, dtype=torch.int64))


def test_prefill_wrapper_through_buckets_on_the_fx_path():
    """A tiny HF decoder behind ``PrefillLogits``: prompts of 5 and 11 tokens share the two
    buckets, logits at the real positions equal the unpadded eager logits, and every bucket is
    its own capture (``compile_kernel=False``: the FX forward, no device needed)."""
    from megabake_b200 import PrefillLogits

    spec = models.get_spec("tiny-llama")
    wrapper = PrefillLogits(models.build_hf_model(spec, seed=3)).eval()
    backend = make_backend(mode="prefill", compile_kernel=False)
    torch._dynamo.reset()
    call = bucketed(wrapper, backend=backend, sequence_args={"input_ids": 1}, buckets=(8, 16))
    generator = torch.Generator().manual_seed(2)
    for length, bucket in ((5, 8), (11, 16), (7, 8)):
        ids = torch.randint(0, spec.vocab, (2, length), generator=generator)
        logits = call(ids)
        assert logits.shape == (2, length, spec.vocab)
        with torch.no_grad():
            eager = wrapper(ids)
        assert (logits.float() - eager.float()).norm() / eager.float().norm() < 0.05
        assert bucket in call.verified
