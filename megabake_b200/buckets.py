"""Prompts of any length through a handful of fixed-shape compiled kernels.

The kernels behind ``make_backend`` are planned for static shapes.  ``bucketed`` keeps the
reference's answer to that (``src/megabake/buckets.py:49-189``, same constructor, same
``bucket_for`` / call behaviour, same ``PaddingDependence`` error): a call pads its sequence
arguments at the end up to the smallest bucket that holds them, runs the callable compiled for
that bucket (one compile per bucket, cached by Dynamo) and narrows every output that has the
bucket's length along ``output_dim`` back to the real length.

That is exact only if results at real positions cannot see the padding -- true for a causal
decoder padded after its last token.  The claim is checked on the first call of every bucket,
with the eager module as the arbiter: two different paddings must give bit-identical results at
the real positions, and padded and unpadded eager results must agree there up to the rounding
noise of differently shaped library kernels (relative L2 distance at most 5 %).

    prefill = bucketed(PrefillLogits(model), backend=make_backend(mode="prefill"),
                       sequence_args={"input_ids": 1})
    logits = prefill(ids)            # ids of any length up to 512
"""

from __future__ import annotations

import inspect
from typing import Any, Callable, Mapping, Sequence

import torch
from torch.utils import _pytree as pytree

DEFAULT_BUCKETS = (16, 32, 64, 128, 256, 512)
RELATIVE_L2_LIMIT = 0.05  # padded against unpadded eager results at the real positions


class PaddingDependence(ValueError):
    """Results at real positions move with the padding: the callable cannot be bucketed."""


def _tensor_leaves(tree: Any) -> list[torch.Tensor]:
    return [leaf for leaf in pytree.tree_leaves(tree) if isinstance(leaf, torch.Tensor)]


class bucketed:  # noqa: N801  (the reference spells it as a function-like name)
    """``module`` callable at every sequence length up to ``max(buckets)``.

    ``sequence_args``: argument name -> its sequence dimension.  ``pad_values``: argument name
    -> the value appended (0 when absent).  ``output_dim``: the dimension along which outputs
    of bucket length are narrowed back.  ``verify=False`` skips the first-call check.
    """

    def __init__(self, module: torch.nn.Module | Callable[..., Any], *, backend: Any,
                 sequence_args: Mapping[str, int],
                 pad_values: Mapping[str, int | float] | None = None,
                 buckets: Sequence[int] = DEFAULT_BUCKETS, output_dim: int = 1,
                 verify: bool = True) -> None:
        if not sequence_args:
            raise ValueError("bucketed needs at least one sequence argument")
        if not buckets or min(buckets) < 1:
            raise ValueError("buckets must be positive lengths")
        self.module = module
        self.sequence_args = dict(sequence_args)
        self.pad_values = dict(pad_values or {})
        self.buckets = tuple(sorted(set(int(b) for b in buckets)))
        self.output_dim = output_dim
        self.verify = verify
        self.verified: set[int] = set()
        target = module.forward if isinstance(module, torch.nn.Module) else module
        self._signature = inspect.signature(target)
        # every bucket is its own static shape: leave Dynamo room for one compile per bucket
        config = torch._dynamo.config
        config.recompile_limit = max(config.recompile_limit, len(self.buckets) + 1)
        self.compiled = torch.compile(module, backend=backend, fullgraph=True, dynamic=False)

    # -- bucket choice ---------------------------------------------------------------------
    def bucket_for(self, length: int) -> int:
        for bucket in self.buckets:
            if bucket >= length:
                return bucket
        raise ValueError(f"length {length} exceeds the largest bucket {self.buckets[-1]}")

    def _real_length(self, arguments: Mapping[str, Any]) -> int:
        found = {name: arguments[name].shape[dim] for name, dim in self.sequence_args.items()
                 if isinstance(arguments.get(name), torch.Tensor)}
        if not found:
            raise ValueError("no sequence argument was passed")
        if len(set(found.values())) > 1:
            raise ValueError(f"sequence arguments disagree on the length: {found}")
        return next(iter(found.values()))

    # -- padding and narrowing -------------------------------------------------------------
    def _padded(self, arguments: Mapping[str, Any], length: int, bucket: int,
                noise_seed: int | None = None) -> dict[str, Any]:
        """The arguments with every sequence tensor grown to ``bucket``.  ``noise_seed`` swaps
        the declared pad value for seeded noise (the second padding of the check)."""
        result = dict(arguments)
        if bucket == length:
            return result
        for name, dim in self.sequence_args.items():
            tensor = arguments.get(name)
            if not isinstance(tensor, torch.Tensor):
                continue
            tail_shape = list(tensor.shape)
            tail_shape[dim] = bucket - length
            if noise_seed is None:
                tail = torch.full(tail_shape, self.pad_values.get(name, 0), dtype=tensor.dtype,
                                  device=tensor.device)
            else:
                generator = torch.Generator().manual_seed(noise_seed)
                if tensor.dtype.is_floating_point:
                    tail = torch.randn(tail_shape, generator=generator).to(tensor)
                else:
                    tail = torch.randint(0, 2, tail_shape, generator=generator).to(tensor)
            result[name] = torch.cat([tensor, tail], dim=dim)
        return result

    def _narrowed(self, output: Any, length: int, bucket: int) -> Any:
        if bucket == length:
            return output
        dim = self.output_dim

        def narrow(leaf: Any) -> Any:
            if isinstance(leaf, torch.Tensor) and leaf.dim() > dim and leaf.shape[dim] == bucket:
                return leaf.narrow(dim, 0, length)
            return leaf

        return pytree.tree_map(narrow, output)

    # -- the call --------------------------------------------------------------------------
    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        arguments = dict(self._signature.bind(*args, **kwargs).arguments)
        length = self._real_length(arguments)
        bucket = self.bucket_for(length)
        with torch.no_grad():
            output = self.compiled(**self._padded(arguments, length, bucket))
        result = self._narrowed(output, length, bucket)
        if self.verify and bucket not in self.verified:
            self._check_padding(arguments, length, bucket)
            self.verified.add(bucket)
        return result

    def _check_padding(self, arguments: Mapping[str, Any], length: int, bucket: int) -> None:
        with torch.no_grad():
            declared = self._narrowed(self.module(**self._padded(arguments, length, bucket)),
                                      length, bucket)
            noisy = self._narrowed(self.module(**self._padded(arguments, length, bucket, 1)),
                                   length, bucket)
            unpadded = self.module(**arguments)
        for a, b in zip(_tensor_leaves(declared), _tensor_leaves(noisy), strict=True):
            if not torch.equal(a, b):
                raise PaddingDependence(
                    "outputs at real positions change with the padding; this callable cannot "
                    "run through padded buckets")
        for want, got in zip(_tensor_leaves(unpadded), _tensor_leaves(declared), strict=True):
            if want.shape != got.shape:
                raise PaddingDependence(f"padded output has shape {tuple(got.shape)}, unpadded "
                                        f"{tuple(want.shape)}")
            if want.is_floating_point():
                norm = want.float().norm()
                distance = (got.float() - want.float()).norm() / norm if norm > 0 else 0.0
                if distance > RELATIVE_L2_LIMIT:
                    raise PaddingDependence(f"bucket {bucket}: padded eager is "
                                            f"{float(distance):.3g} from unpadded eager")
            elif not torch.equal(want, got):
                raise PaddingDependence(f"bucket {bucket}: padded eager differs from unpadded "
                                        "eager")
