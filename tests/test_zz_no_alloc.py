"""The allocation-free attention entry point against the plan path.

Collected last on purpose (the file name sorts after every other test file): the entry point
keeps its scratch in one array inside the library's device image, so it has to give the same
answer in a fresh process and after everything else has used the GPU.
"""

import ctypes
import math

import pytest
import torch

from megabake_b200 import planner as pl
from megabake_b200 import runtime as rt

from helpers import PhaseRunner

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(120)]

ERR_UNSUPPORTED, ERR_RESOURCE = 3, 4  # enum mb_error
STATIC_SCRATCH_BYTES = 4 << 20
STATIC_RESERVED_BYTES = 256 + 4096


def _inputs(batch, heads, kv_heads, dim, cached, capacity, seed):
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    q = torch.randn(batch, heads * dim, generator=g).to(bf)
    k = torch.randn(batch, kv_heads * dim, generator=g).to(bf)
    v = torch.randn(batch, kv_heads * dim, generator=g).to(bf)
    kc = torch.randn(batch, capacity, kv_heads, dim, generator=g).to(bf)
    vc = torch.randn(batch, capacity, kv_heads, dim, generator=g).to(bf)
    inv_freq = (1.0 / (10000 ** (torch.arange(0, dim, 2).float() / dim))).to(bf)
    pos = torch.full((batch, 1), cached, dtype=torch.int64)
    length = torch.tensor([cached], dtype=torch.int32)
    return [t.cuda() for t in (q, k, v, kc, vc, inv_freq, pos, length)]


def _static_max_chunks(batch, heads, kv_heads, dim, capacity):
    per_chunk = batch * heads * (dim + 2) * 4
    room = STATIC_SCRATCH_BYTES - STATIC_RESERVED_BYTES
    return max(1, min(32, room // per_chunk, math.ceil(capacity / 16)))


def _plan_step(tensors, batch, heads, kv_heads, dim, capacity):
    """One attention phase through mb_plan_* (the existing entry points)."""
    q, k, v, kc, vc, inv_freq, pos, length = tensors
    group = heads // kv_heads
    max_chunks = _static_max_chunks(batch, heads, kv_heads, dim, capacity)
    out = torch.zeros(batch, heads * dim, dtype=torch.bfloat16, device="cuda")
    partial = torch.zeros(batch * kv_heads * max_chunks * group * (dim + 2),
                          dtype=torch.float32, device="cuda")
    counters = torch.zeros(max(4, batch * kv_heads), dtype=torch.int32, device="cuda")
    runner = PhaseRunner()
    ph = rt.Phase.blank(rt.BODY_ATTN_DECODE, rt.FLAG_BARRIER | rt.FLAG_BUMP_LENGTH)
    merge_slots = pl.attention_merge_slots(dim, group)
    for index, value in ((rt.AT_I_BATCH, batch), (rt.AT_I_HEADS, heads),
                         (rt.AT_I_KV_HEADS, kv_heads), (rt.AT_I_HEAD_DIM, dim),
                         (rt.AT_I_CAPACITY, capacity), (rt.AT_I_INVFREQ_BF16, 1),
                         (rt.AT_I_MAX_CHUNKS, max_chunks), (rt.AT_I_MERGE_SLOTS, merge_slots),
                         (rt.AT_I_EXACT_KEYS, min(capacity, 128))):
        ph.i[index] = value
    ph.f[rt.AT_F_SCALE] = dim ** -0.5
    ph.f[rt.AT_F_ROPE_SCALE] = 1.0
    for index, (name, tensor) in enumerate([
        ("q", q), ("k", k), ("v", v), ("kc", kc), ("vc", vc), ("len", length), ("pos", pos),
        ("invf", inv_freq), ("out", out), ("partial", partial), ("cnt", counters),
    ]):
        ph.slot[index] = runner.slot(name, tensor)
    plan = runner.run([ph], pl.attention_scratch_bytes(dim, group, merge_slots))
    assert plan.status().code == 0
    return out


def _static_step(tensors, batch, heads, kv_heads, dim, capacity, status):
    q, k, v, kc, vc, inv_freq, pos, length = tensors
    out = torch.zeros(batch, heads * dim, dtype=torch.bfloat16, device="cuda")
    args = rt.AttentionArgs(
        batch=batch, heads=heads, kv_heads=kv_heads, head_dim=dim, capacity=capacity,
        inv_freq_is_bf16=1, rope_scale=1.0, query_scale=0.0,
        query=q.data_ptr(), key=k.data_ptr(), value=v.data_ptr(), key_cache=kc.data_ptr(),
        value_cache=vc.data_ptr(), valid_length=length.data_ptr(), position_ids=pos.data_ptr(),
        inv_freq=inv_freq.data_ptr(), out=out.data_ptr(), status=status.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    code = rt.load_library().mb_attention_decode_static(ctypes.byref(args), ctypes.c_void_p(stream))
    assert code == 0, rt.load_library().mb_strerror(code)
    return out


def _oracle_step(tensors, batch, heads, kv_heads, dim):
    """The CPU oracle on copies of the inputs: a second judge, independent of the kernel code
    the two entry points share."""
    from oracle import decoder_oracle as oracle

    q, k, v, kc, vc, inv_freq, pos, length = (t.cpu().clone() for t in tensors)
    cos, sin = oracle.rotary_tables(inv_freq, pos, 1.0)
    q_r = oracle.apply_rope(q.view(batch, 1, heads, dim), cos, sin)
    k_r = oracle.apply_rope(k.view(batch, 1, kv_heads, dim), cos, sin)
    out = oracle.kv_attention(q_r, k_r, v.view(batch, 1, kv_heads, dim), kc, vc, length)
    return out.reshape(batch, heads * dim), kc, vc, length


@pytest.mark.parametrize("batch,heads,kv_heads,dim,cached", [
    (2, 14, 2, 64, 700),     # split keys: partials and arrival counters in the static array
    (1, 32, 8, 64, 40),      # short context: exact softmax, no partials
    (2, 4, 2, 128, 2500),
    (1, 8, 1, 256, 300),     # 256-wide heads, eight query heads on one kv head
    (2, 4, 2, 64, 126),      # the two calls cross from the exact softmax (<= 128 keys) ...
    (2, 4, 2, 64, 127),      # ... to the split one
])
def test_static_attention_matches_plan_path_twice(batch, heads, kv_heads, dim, cached):
    capacity = cached + 8
    seed = cached + heads
    plan_side = _inputs(batch, heads, kv_heads, dim, cached, capacity, seed)
    static_side = [t.clone() for t in plan_side]
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    g = torch.Generator().manual_seed(seed + 1)
    for call in range(2):       # the second call finds whatever the first left in the array
        if call:
            for index in range(3):  # fresh q, k, v; the position moves with the length
                fresh = torch.randn(plan_side[index].shape, generator=g).to(torch.bfloat16).cuda()
                plan_side[index].copy_(fresh)
                static_side[index].copy_(fresh)
            plan_side[6].add_(1)
            static_side[6].add_(1)
        reference, ref_kc, ref_vc, ref_len = _oracle_step(static_side, batch, heads, kv_heads, dim)
        expected = _plan_step(plan_side, batch, heads, kv_heads, dim, capacity)
        got = _static_step(static_side, batch, heads, kv_heads, dim, capacity, status)
        torch.cuda.synchronize()
        # against the oracle: result within the attention tolerance of the body tests, appended
        # value row and length exact
        assert float((got.cpu().float() - reference.float()).abs().max()) <= 2e-2
        assert int(static_side[7].item()) == int(ref_len)
        assert torch.equal(static_side[4].cpu(), ref_vc)
        assert float((static_side[3].cpu().float() - ref_kc.float()).abs().max()) <= 0.04
        assert int(status.item()) == 0
        assert int(static_side[7].item()) == cached + call + 1 == int(plan_side[7].item())
        assert torch.equal(static_side[3], plan_side[3])      # key cache, appended row included
        assert torch.equal(static_side[4], plan_side[4])
        assert torch.equal(got, expected)


def test_static_attention_reports_a_full_cache():
    """valid_length == capacity: nothing may be appended.  The call is non-blocking, so the fault
    arrives through ``status``: MB_ST_KV_OVERFLOW, with the caches and the length untouched; the
    next call (room again) works."""
    batch, heads, kv_heads, dim, capacity = 2, 4, 2, 64, 24
    tensors = _inputs(batch, heads, kv_heads, dim, capacity, capacity, seed=5)
    before = [t.clone() for t in tensors]
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    _static_step(tensors, batch, heads, kv_heads, dim, capacity, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 3                       # MB_ST_KV_OVERFLOW
    assert int(tensors[7].item()) == capacity            # length untouched
    assert torch.equal(tensors[3], before[3]) and torch.equal(tensors[4], before[4])
    tensors[7].fill_(capacity - 1)
    tensors[6].fill_(capacity - 1)
    reference, _, _, _ = _oracle_step(tensors, batch, heads, kv_heads, dim)
    got = _static_step(tensors, batch, heads, kv_heads, dim, capacity, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(tensors[7].item()) == capacity
    assert float((got.cpu().float() - reference.float()).abs().max()) <= 2e-2


def test_static_attention_rejects_misaligned_arguments():
    lib = rt.load_library()
    tensors = _inputs(1, 4, 2, 64, 3, 8, seed=1)
    q, k, v, kc, vc, inv_freq, pos, length = tensors
    out = torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda")
    base = dict(batch=1, heads=4, kv_heads=2, head_dim=64, capacity=8, inv_freq_is_bf16=1,
                rope_scale=1.0, query_scale=0.0, query=q.data_ptr(), key=k.data_ptr(),
                value=v.data_ptr(), key_cache=kc.data_ptr(), value_cache=vc.data_ptr(),
                valid_length=length.data_ptr(), position_ids=pos.data_ptr(),
                inv_freq=inv_freq.data_ptr(), out=out.data_ptr(), status=0)
    for name, offset in (("position_ids", 4), ("valid_length", 2), ("query", 8), ("status", 1)):
        args = rt.AttentionArgs(**dict(base, **{name: (base[name] or length.data_ptr()) + offset}))
        assert lib.mb_attention_decode_static(ctypes.byref(args), None) == 1, name   # MB_ERR_INVALID
    torch.cuda.synchronize()


def test_static_attention_rejects_what_the_array_cannot_hold():
    lib = rt.load_library()
    dummy = torch.zeros(64, dtype=torch.int64, device="cuda")
    base = dict(inv_freq_is_bf16=1, rope_scale=1.0, query_scale=0.0,
                **{name: dummy.data_ptr() for name in (
                    "query", "key", "value", "key_cache", "value_cache", "valid_length",
                    "position_ids", "inv_freq", "out")}, status=0)
    # 2048 (row, kv head) pairs: more arrival counters than the array reserves
    args = rt.AttentionArgs(batch=2048, heads=1, kv_heads=1, head_dim=64, capacity=64, **base)
    assert lib.mb_attention_decode_static(ctypes.byref(args), None) == ERR_RESOURCE
    # one chunk of partials alone is larger than 4 MiB
    args = rt.AttentionArgs(batch=1000, heads=8, kv_heads=1, head_dim=256, capacity=64, **base)
    assert lib.mb_attention_decode_static(ctypes.byref(args), None) == ERR_RESOURCE
    args = rt.AttentionArgs(batch=1, heads=8, kv_heads=1, head_dim=96, capacity=64, **base)
    assert lib.mb_attention_decode_static(ctypes.byref(args), None) == ERR_UNSUPPORTED
    torch.cuda.synchronize()
