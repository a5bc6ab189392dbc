"""Generate the golden fixtures in this directory from the REFERENCE implementation.

Run in the build container only (needs the reference checkout; the fixtures travel, the
reference does not):

    python tests/golden/make_golden.py /path/to/reference     (or MEGABAKE_REFERENCE=/path/to/reference)
    python tests/golden/make_golden.py /path/to/reference --per-row    (only ops_per_row.npz)

It imports the reference's own operators and decode wrappers
(``src/megabake/ops/attention.py``, ``tests/fixtures.py::StatefulSmolLM``,
``benchmarks/stateful_models.py::StatefulCausalLM``) and runs them, on CPU in bf16, over seeded
random-init Hugging Face models built by ``megabake_b200.models`` (the same seeds and
generator protocol the tests use to rebuild the weights).  Stored per case: the token ids fed,
the logits of every call and the final KV state, as raw bf16 bit patterns (int16), so the
comparison in ``tests/test_oracle_golden.py`` is bit-exact.

The product package is imported through a stub parent module so that its own registration of
``megabake::kv_attention`` does not collide with the reference's.
"""

from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
import os  # noqa: E402

if not [a for a in sys.argv[1:] if not a.startswith("--")] and "MEGABAKE_REFERENCE" not in os.environ:
    raise SystemExit("usage: make_golden.py /path/to/reference (a checkout of the reference)")
REFERENCE = Path(sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("--")
                 else os.environ["MEGABAKE_REFERENCE"])

sys.dont_write_bytecode = True
sys.path.insert(0, str(REFERENCE / "src"))
stub = types.ModuleType("megabake_b200")
stub.__path__ = [str(ROOT / "megabake_b200")]
sys.modules["megabake_b200"] = stub
from megabake_b200 import models  # noqa: E402  (no ops registered by this import)

from megabake.ops.attention import attention as ref_attention  # noqa: E402
from megabake.ops.attention import kv_attention as ref_kv_attention  # noqa: E402


def _load(name: str, path: Path):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


fixtures = _load("reference_fixtures", REFERENCE / "tests" / "fixtures.py")
stateful = _load("reference_stateful_models", REFERENCE / "benchmarks" / "stateful_models.py")


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).numpy().copy()


def decode_case(name: str, wrapper_kind: str, batch: int, capacity: int, calls: int, seed: int,
                token_seed: int):
    spec = models.get_spec(name)
    model = models.build_hf_model(spec, seed)
    model.set_attn_implementation("eager")
    if wrapper_kind == "smollm":
        wrapper = fixtures.StatefulSmolLM(model).eval()
    else:
        wrapper = stateful.StatefulCausalLM(model).eval()
    shape = (batch, capacity, spec.kv_heads, spec.head_dim)
    caches = [(torch.zeros(shape, dtype=torch.bfloat16), torch.zeros(shape, dtype=torch.bfloat16),
               torch.zeros(1, dtype=torch.int32)) for _ in range(spec.layers)]
    if wrapper_kind == "smollm":  # all K, then all V, then all lengths
        state = [c[0] for c in caches] + [c[1] for c in caches] + [c[2] for c in caches]
    else:  # per layer K, V, length
        state = [t for c in caches for t in c]
    tokens = torch.randint(0, spec.vocab, (batch, calls),
                           generator=torch.Generator().manual_seed(token_seed))
    logits = []
    with torch.no_grad():
        for call in range(calls):
            pos = torch.full((batch, 1), call, dtype=torch.int64)
            logits.append(wrapper(tokens[:, call:call + 1].contiguous(), pos, *state))
    out = {
        "tokens": tokens.numpy(),
        "logits": np.stack([bits(x) for x in logits]),
        "lengths": np.array([int(c[2]) for c in caches]),
    }
    for index, (k, v, _) in enumerate(caches):
        out[f"k{index}"] = bits(k)
        out[f"v{index}"] = bits(v)
    meta = dict(model=name, wrapper=wrapper_kind, batch=batch, capacity=capacity, calls=calls,
                seed=seed, token_seed=token_seed)
    return out, meta


def protocol_case(name: str, prompt_len: int, steps: int, seed: int, token_seed: int):
    """Config-1 protocol at full size: prompt fed token by token, then greedy steps."""
    spec = models.get_spec(name)
    model = models.build_hf_model(spec, seed)
    model.set_attn_implementation("eager")
    wrapper = fixtures.StatefulSmolLM(model).eval()
    capacity = prompt_len + steps + 32
    shape = (1, capacity, spec.kv_heads, spec.head_dim)
    ks = [torch.zeros(shape, dtype=torch.bfloat16) for _ in range(spec.layers)]
    vs = [torch.zeros(shape, dtype=torch.bfloat16) for _ in range(spec.layers)]
    ls = [torch.zeros(1, dtype=torch.int32) for _ in range(spec.layers)]
    prompt = torch.randint(0, spec.vocab, (1, prompt_len),
                           generator=torch.Generator().manual_seed(token_seed))
    token = prompt[:, :1].contiguous()
    picks, top2, last = [], [], None
    with torch.no_grad():
        for call in range(prompt_len + steps):
            pos = torch.full((1, 1), call, dtype=torch.int64)
            logits = wrapper(token, pos, *ks, *vs, *ls)
            best = logits[:, -1].float().topk(2)
            picks.append(int(best.indices[0, 0]))
            top2.append(best.values[0].numpy())
            token = (prompt[:, call + 1:call + 2].contiguous() if call + 1 < prompt_len
                     else best.indices[:, :1].contiguous())
            last = logits
    out = {"prompt": prompt.numpy(), "picks": np.array(picks), "top2": np.stack(top2),
           "last_logits": bits(last), "k0": bits(ks[0][:, :prompt_len + steps]),
           "v_last": bits(vs[-1][:, :prompt_len + steps])}
    meta = dict(model=name, prompt_len=prompt_len, steps=steps, seed=seed, token_seed=token_seed,
                capacity=capacity)
    return out, meta


def op_cases():
    """The two declared operators on seeded inputs (reference eager definitions)."""
    out = {}
    g = torch.Generator().manual_seed(123)
    for tag, (batch, heads, kv_heads, dim, cached, capacity) in {
        "gqa": (2, 4, 2, 64, 5, 8), "mha": (1, 2, 2, 64, 0, 4), "mqa": (1, 8, 1, 32, 17, 20),
    }.items():
        q = torch.randn(batch, 1, heads, dim, generator=g).to(torch.bfloat16)
        k = torch.randn(batch, 1, kv_heads, dim, generator=g).to(torch.bfloat16)
        v = torch.randn(batch, 1, kv_heads, dim, generator=g).to(torch.bfloat16)
        kc = torch.randn(batch, capacity, kv_heads, dim, generator=g).to(torch.bfloat16)
        vc = torch.randn(batch, capacity, kv_heads, dim, generator=g).to(torch.bfloat16)
        length = torch.tensor([cached], dtype=torch.int32)
        for name, t in (("q", q), ("k", k), ("v", v), ("kc_in", kc), ("vc_in", vc)):
            out[f"kv_{tag}_{name}"] = bits(t)
        out[f"kv_{tag}_len_in"] = np.array([cached])
        result = ref_kv_attention(q, k, v, kc, vc, length)
        out[f"kv_{tag}_out"] = bits(result)
        out[f"kv_{tag}_kc_out"] = bits(kc)
        out[f"kv_{tag}_vc_out"] = bits(vc)
        out[f"kv_{tag}_len_out"] = np.array([int(length)])
    for tag, (batch, length, heads, kv_heads, dim) in {
        "causal": (2, 9, 4, 2, 64), "mqa256": (1, 5, 2, 1, 256),
    }.items():
        q = torch.randn(batch, length, heads, dim, generator=g).to(torch.bfloat16)
        k = torch.randn(batch, length, kv_heads, dim, generator=g).to(torch.bfloat16)
        v = torch.randn(batch, length, kv_heads, dim, generator=g).to(torch.bfloat16)
        allowed = torch.tril(torch.ones(length, length, dtype=torch.bool))
        mask = torch.where(allowed, 0.0, torch.finfo(torch.bfloat16).min).to(torch.bfloat16)
        mask = mask[None, None].expand(batch, 1, length, length).contiguous()
        for name, t in (("q", q), ("k", k), ("v", v), ("mask", mask)):
            out[f"at_{tag}_{name}"] = bits(t)
        out[f"at_{tag}_out"] = bits(ref_attention(q, k, v, mask, dim ** -0.5))
    return out


def per_row_cases():
    """``kv_attention`` over rows that hold different numbers of keys: the reference's operator
    (one length shared by the batch, ``src/megabake/ops/attention.py:52-87``) called row by row
    on batch-1 views, each row with its own length.  This pins what a per-row ``valid_length``
    of shape ``[batch]`` has to compute."""
    out = {}
    g = torch.Generator().manual_seed(321)
    for tag, (heads, kv_heads, dim, capacity, lengths) in {
        "gqa": (4, 2, 64, 40, (0, 5, 17, 39)), "mqa": (8, 1, 64, 160, (1, 130, 159)),
    }.items():
        batch = len(lengths)
        q = torch.randn(batch, 1, heads, dim, generator=g).to(torch.bfloat16)
        k = torch.randn(batch, 1, kv_heads, dim, generator=g).to(torch.bfloat16)
        v = torch.randn(batch, 1, kv_heads, dim, generator=g).to(torch.bfloat16)
        kc = torch.randn(batch, capacity, kv_heads, dim, generator=g).to(torch.bfloat16)
        vc = torch.randn(batch, capacity, kv_heads, dim, generator=g).to(torch.bfloat16)
        for name, t in (("q", q), ("k", k), ("v", v), ("kc_in", kc), ("vc_in", vc)):
            out[f"{tag}_{name}"] = bits(t)
        out[f"{tag}_len_in"] = np.array(lengths)
        rows, after = [], []
        for row, cached in enumerate(lengths):
            length = torch.tensor([cached], dtype=torch.int32)
            # batch-1 views share storage with kc / vc, so the append lands in the full caches
            rows.append(ref_kv_attention(q[row:row + 1], k[row:row + 1], v[row:row + 1],
                                         kc[row:row + 1], vc[row:row + 1], length))
            after.append(int(length))
        out[f"{tag}_out"] = bits(torch.cat(rows, dim=0))
        out[f"{tag}_kc_out"] = bits(kc)
        out[f"{tag}_vc_out"] = bits(vc)
        out[f"{tag}_len_out"] = np.array(after)
    return out


def prefill_case(name: str, batch: int, length: int, seed: int, token_seed: int):
    """Hugging Face prefill through the reference's declared attention op."""
    from megabake.fx_handler.hf_attention import register_transformers_attention

    spec = models.get_spec(name)
    model = models.build_hf_model(spec, seed)
    model.set_attn_implementation(register_transformers_attention())
    ids = torch.randint(0, spec.vocab, (batch, length),
                        generator=torch.Generator().manual_seed(token_seed))
    with torch.no_grad():
        logits = model(input_ids=ids).logits
    return ({"tokens": ids.numpy(), "logits": bits(logits)},
            dict(model=name, batch=batch, length=length, seed=seed, token_seed=token_seed))


def reference_identity() -> str:
    """What the fixtures were made from, without a path of the build machine: a hash over the
    reference files this script imports."""
    import hashlib

    digest = hashlib.sha256()
    for relative in ("src/megabake/ops/attention.py", "tests/fixtures.py",
                     "benchmarks/stateful_models.py", "src/megabake/fx_handler/hf_attention.py"):
        digest.update((REFERENCE / relative).read_bytes())
    return "sha256:" + digest.hexdigest()[:16]


def main() -> None:
    torch.manual_seed(0)
    torch.set_num_threads(8)
    import json

    if "--per-row" in sys.argv:  # only the per-row operator fixture (the others are untouched)
        np.savez_compressed(HERE / "ops_per_row.npz", **per_row_cases())
        index = json.loads((HERE / "index.json").read_text())
        index["ops_per_row"] = {"seed": 321}
        index["_versions"]["reference"] = reference_identity()
        (HERE / "index.json").write_text(json.dumps(index, indent=1, sort_keys=True))
        return
    index = {}
    decode = [
        ("tiny-llama", "smollm", 2, 12, 8, 11, 21),
        ("tiny-llama", "causal", 2, 12, 8, 11, 21),
        ("tiny-llama3", "causal", 1, 12, 8, 12, 22),
        ("tiny-qwen2", "causal", 3, 12, 8, 13, 23),
        ("tiny-mha", "smollm", 2, 12, 8, 14, 24),
        ("tiny-gemma", "causal", 2, 12, 8, 15, 25),
        ("tiny-gemma256", "causal", 1, 12, 8, 16, 26),
    ]
    for case in decode:
        arrays, meta = decode_case(*case)
        key = f"decode_{case[0]}_{case[1]}"
        np.savez_compressed(HERE / f"{key}.npz", **arrays)
        index[key] = meta
        print(key, {k: v.shape for k, v in arrays.items() if k in ("logits",)})
    arrays, meta = protocol_case("smollm-135m", 32, 32, 1, 1)
    np.savez_compressed(HERE / "protocol_smollm-135m.npz", **arrays)
    index["protocol_smollm-135m"] = meta
    print("protocol picks", arrays["picks"][:40], "top2 margin min",
          float((arrays["top2"][:, 0] - arrays["top2"][:, 1]).min()))
    np.savez_compressed(HERE / "ops.npz", **op_cases())
    index["ops"] = {"seed": 123}
    np.savez_compressed(HERE / "ops_per_row.npz", **per_row_cases())
    index["ops_per_row"] = {"seed": 321}
    for case in [("tiny-gemma", 2, 12, 15, 35), ("tiny-llama", 1, 16, 11, 31),
                 ("tiny-qwen2", 2, 10, 13, 33)]:
        arrays, meta = prefill_case(*case)
        key = f"prefill_{case[0]}"
        np.savez_compressed(HERE / f"{key}.npz", **arrays)
        index[key] = meta
    index["_versions"] = {"torch": torch.__version__,
                          "transformers": __import__("transformers").__version__,
                          "reference": reference_identity()}
    (HERE / "index.json").write_text(json.dumps(index, indent=1, sort_keys=True))


if __name__ == "__main__":
    main()
