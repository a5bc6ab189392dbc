"""megabake_b200: a B200-native (sm_100a) persistent-megakernel backend for decoder inference
behind MegaBake's ``make_backend()`` / ``torch.compile`` boundary.

Public surface (names follow the reference's ``src/megabake/__init__.py:61-121`` for the
parts of it this backend keeps):

``make_backend(mode=..., ...)``     the ``torch.compile`` backend factory
``graphed(function, *args)``        CUDA-graph capture of one compiled call
``kv_attention`` / ``attention``    the declared attention operators (``torch.ops.megabake.*``)
``DecodeStep``, ``StatefulDecoder`` explicit-state decode wrappers for Hugging Face models
``GroupedStateDecoder``             the same step, state ordered all K, all V, all lengths
``PrefillLogits``                   ids -> logits prefill wrapper over ``megabake::attention``
``StatefulPrefill``                 prefill that also fills the explicit decode state
``GreedyGenerator``                 compiled prefill + decode loop over one KV state
``bucketed`` / ``PaddingDependence`` prompts of any length through a few fixed-shape compiles
``register_transformers_attention`` the ``"megabake"`` attention implementation for HF models
``CompilerError``                   every refusal, with a staged diagnostic
"""

from .diagnostics import CompilerDiagnostic, CompilerError
from .ops import attention, kv_attention

__all__ = [
    "CompilerDiagnostic", "CompilerError", "DecodeStep", "GreedyGenerator", "GroupedStateDecoder",
    "PaddingDependence",
    "PrefillLogits", "StatefulDecoder", "StatefulPrefill", "attention", "bucketed",
    "graphed", "kv_attention", "make_backend", "register_transformers_attention",
]


def __getattr__(name):
    # Heavier modules load on first use so that `import megabake_b200` stays light.
    if name == "make_backend":
        from .frontend import make_backend
        return make_backend
    if name in ("graphed", "GraphedCall", "BoundDecoder"):
        from . import engine
        return getattr(engine, name)
    if name in ("DecodeStep", "GroupedStateDecoder", "PrefillLogits", "StatefulDecoder",
                "StatefulPrefill", "register_transformers_attention"):
        from . import hf
        return getattr(hf, name)
    if name in ("bucketed", "PaddingDependence"):
        from . import buckets
        return getattr(buckets, name)
    if name == "GreedyGenerator":
        from .generate import GreedyGenerator
        return GreedyGenerator
    raise AttributeError(name)
