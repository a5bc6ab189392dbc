"""Device bodies against plain-torch references, one phase per plan, through the C ABI.

GEMV references are computed in fp64 from the bf16 operands and rounded once, the way the
reference's own Blackwell GEMM test does (``tests/gpu/test_blackwell_gemm.py:60-63``): a
bf16 library GEMM on the GPU is not accurate enough to be the yardstick.
"""

import math

import pytest
import torch

from megabake_b200 import planner as pl
from megabake_b200 import runtime as rt
from oracle import decoder_oracle as oracle
from tests.helpers import PhaseRunner, cosine, max_abs

pytestmark = pytest.mark.gpu



def _bf16(*shape, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).cuda()


def _ref_linear(x, w, b=None):
    acc = x.double() @ w.double().t()
    if b is not None:
        acc = acc + b.double()
    return acc.float().to(torch.bfloat16)


def _gemv_phase(runner, *, x, segs, k, rows, prologue=rt.PRO_NONE, norm_w=None, eps=1e-5,
                epilogue=rt.EPI_NONE, pair=None, residual=None, k_chunk=None, ctas=148):
    n_total = sum(w.shape[0] for w, _, _ in segs)
    nmat = 2 if pair is not None else 1
    stage = rt.load_library().mb_stage_bytes(rt.MODE_DECODE)
    tile, chunk = pl.gemv_geometry(n_total, k, nmat, ctas, stage, 64)
    if k_chunk is not None:
        chunk = k_chunk
    ph = rt.Phase.blank(rt.BODY_GEMV, 0)
    ph.i[rt.GV_I_ROWS] = rows
    ph.i[rt.GV_I_K] = k
    ph.i[rt.GV_I_NSEG] = len(segs)
    ph.i[rt.GV_I_NMAT] = nmat
    ph.i[rt.GV_I_PROLOGUE] = prologue
    ph.i[rt.GV_I_EPILOGUE] = epilogue
    ph.i[rt.GV_I_ROW_TILE] = tile
    ph.i[rt.GV_I_K_CHUNK] = chunk
    ph.f[rt.GV_F_EPS] = eps
    ph.slot[rt.GV_S_X] = runner.slot("x", x)
    ph.slot[rt.GV_S_NORM_W] = runner.slot("norm", norm_w)
    for i, (w, b, out) in enumerate(segs):
        ph.i[rt.GV_I_N0 + i] = w.shape[0]
        ph.slot[rt.GV_S_W0 + i] = runner.slot(f"w{i}", w)
        ph.slot[rt.GV_S_BIAS0 + i] = runner.slot(f"b{i}", b)
        ph.slot[rt.GV_S_OUT0 + i] = runner.slot(f"o{i}", out)
    ph.slot[rt.GV_S_W_PAIR] = runner.slot("pair", pair)
    ph.slot[rt.GV_S_RESIDUAL] = runner.slot("res", residual)
    return ph


@pytest.mark.parametrize("rows", [1, 3, 8])
@pytest.mark.parametrize("n,k", [(576, 576), (1152, 896), (2048, 8192), (4100, 2048), (40, 64)])
@pytest.mark.parametrize("k_chunk", [None, 32, 192])
def test_gemv_plain(rows, n, k, k_chunk):
    x = _bf16(rows, k, seed=1)
    w = _bf16(n, k, scale=0.05, seed=2)
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    if k_chunk is not None and k_chunk > k:
        pytest.skip("chunk longer than the row")
    ph = _gemv_phase(runner, x=x, segs=[(w, None, out)], k=k, rows=rows, k_chunk=k_chunk)
    plan = runner.run([ph], rows * (k + 32) * 2)
    assert plan.status().code == 0
    ref = _ref_linear(x, w)
    # fp32 accumulation in a different order: at most one bf16 ulp apart, on a few elements
    assert max_abs(out, ref) <= 2.0 ** -7 * float(ref.float().abs().max())
    assert (out != ref).float().mean() < 0.05
    assert cosine(out, ref) > 0.99999


def test_gemv_qkv_segments_bias():
    rows, k = 4, 896
    x = _bf16(rows, k, seed=3)
    ws = [_bf16(n, k, scale=0.05, seed=10 + i) for i, n in enumerate((896, 128, 128))]
    bs = [_bf16(n, scale=0.5, seed=20 + i) for i, n in enumerate((896, 128, 128))]
    outs = [torch.zeros(rows, w.shape[0], dtype=torch.bfloat16, device="cuda") for w in ws]
    runner = PhaseRunner()
    ph = _gemv_phase(runner, x=x, segs=list(zip(ws, bs, outs)), k=k, rows=rows)
    plan = runner.run([ph], (rows + 1) * (k + 32) * 2)
    assert plan.status().code == 0
    for w, b, out in zip(ws, bs, outs):
        ref = _ref_linear(x, w, b)
        assert (out != ref).float().mean() < 0.02
        assert max_abs(out, ref) <= 2.0 ** -7 * float(ref.float().abs().max())


@pytest.mark.parametrize("kind", ["llama", "gemma"])
def test_gemv_rmsnorm_prologue(kind):
    rows, k, n = 2, 2048, 3072
    x = _bf16(rows, k, seed=5)
    nw = _bf16(k, scale=0.3, seed=6)
    w = _bf16(n, k, scale=0.05, seed=7)
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    pro = rt.PRO_RMS_LLAMA if kind == "llama" else rt.PRO_RMS_GEMMA
    ph = _gemv_phase(runner, x=x, segs=[(w, None, out)], k=k, rows=rows, prologue=pro, norm_w=nw,
                     eps=1e-5)
    plan = runner.run([ph], (rows + 1) * (k + 32) * 2)
    assert plan.status().code == 0
    normed = oracle.rms_norm(x.cpu(), nw.cpu(), 1e-5, kind).cuda()
    ref = _ref_linear(normed, w)
    assert (out != ref).float().mean() < 0.03
    assert cosine(out, ref) > 0.99999


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_gemv_gated_pair(act):
    rows, k, n = 3, 576, 1536
    x = _bf16(rows, k, seed=8)
    wg = _bf16(n, k, scale=0.08, seed=9)
    wu = _bf16(n, k, scale=0.08, seed=10)
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    epi = rt.EPI_SILU_MUL if act == "silu" else rt.EPI_GELU_TANH_MUL
    ph = _gemv_phase(runner, x=x, segs=[(wg, None, out)], k=k, rows=rows, epilogue=epi, pair=wu)
    plan = runner.run([ph], (rows + 1) * (k + 32) * 2)
    assert plan.status().code == 0
    gate, up = _ref_linear(x, wg), _ref_linear(x, wu)
    ref = (oracle._activation(gate.cpu(), act) * up.cpu()).cuda()
    assert (out != ref).float().mean() < 0.05
    assert cosine(out, ref) > 0.9999


def test_gemv_residual_in_place():
    rows, k, n = 8, 1536, 576
    x = _bf16(rows, k, seed=11)
    w = _bf16(n, k, scale=0.05, seed=12)
    hidden = _bf16(rows, n, seed=13)
    before = hidden.clone()
    runner = PhaseRunner()
    ph = _gemv_phase(runner, x=x, segs=[(w, None, hidden)], k=k, rows=rows,
                     epilogue=rt.EPI_RESIDUAL, residual=hidden)
    plan = runner.run([ph], (rows + 1) * (k + 32) * 2)
    assert plan.status().code == 0
    ref = before + _ref_linear(x, w)
    assert (hidden != ref).float().mean() < 0.02
    assert cosine(hidden, ref) > 0.99999


def _attention_case(batch, heads, kv_heads, dim, cached, capacity, seed=0, q_scale=0.0):
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(batch, heads * dim, generator=g)).to(torch.bfloat16)
    k = (torch.randn(batch, kv_heads * dim, generator=g)).to(torch.bfloat16)
    v = (torch.randn(batch, kv_heads * dim, generator=g)).to(torch.bfloat16)
    kc = torch.randn(batch, capacity, kv_heads, dim, generator=g).to(torch.bfloat16)
    vc = torch.randn(batch, capacity, kv_heads, dim, generator=g).to(torch.bfloat16)
    inv_freq = (1.0 / (10000 ** (torch.arange(0, dim, 2).float() / dim))).to(torch.bfloat16)
    pos = torch.full((batch, 1), cached, dtype=torch.int64)
    pos[-1, 0] = cached + 3  # rows may sit at different positions
    length = torch.tensor([cached], dtype=torch.int32)
    return q, k, v, kc, vc, inv_freq, pos, length


@pytest.mark.parametrize("batch,heads,kv_heads,dim", [
    (1, 9, 3, 64), (2, 14, 2, 64), (1, 32, 8, 64), (2, 4, 4, 64), (1, 8, 1, 256), (2, 4, 2, 128),
])
@pytest.mark.parametrize("cached", [0, 1, 15, 16, 63, 200, 1023, 2500])
@pytest.mark.parametrize("exact", [True, False])
def test_attention_decode(batch, heads, kv_heads, dim, cached, exact):
    capacity = cached + 5
    q, k, v, kc, vc, inv_freq, pos, length = _attention_case(batch, heads, kv_heads, dim, cached,
                                                             capacity, seed=cached + heads)
    # CPU oracle
    cos, sin = oracle.rotary_tables(inv_freq, pos, 1.0)
    q_r = oracle.apply_rope(q.view(batch, 1, heads, dim), cos, sin)
    k_r = oracle.apply_rope(k.view(batch, 1, kv_heads, dim), cos, sin)
    kc_ref, vc_ref, len_ref = kc.clone(), vc.clone(), length.clone()
    ref = oracle.kv_attention(q_r, k_r, v.view(batch, 1, kv_heads, dim), kc_ref, vc_ref, len_ref)
    ref = ref.reshape(batch, heads * dim)

    group = heads // kv_heads
    dev = [t.cuda() for t in (q, k, v, kc, vc, inv_freq, pos, length)]
    qd, kd, vd, kcd, vcd, invd, posd, lend = dev
    out = torch.zeros(batch, heads * dim, dtype=torch.bfloat16, device="cuda")
    max_chunks = max(1, min(64, math.ceil(capacity / 16)))
    partial = torch.zeros(batch * kv_heads * max_chunks * group * (dim + 2),
                          dtype=torch.float32, device="cuda")
    counters = torch.zeros(max(4, batch * kv_heads), dtype=torch.int32, device="cuda")
    runner = PhaseRunner()
    ph = rt.Phase.blank(rt.BODY_ATTN_DECODE, rt.FLAG_BARRIER | rt.FLAG_BUMP_LENGTH)
    ph.i[rt.AT_I_BATCH] = batch
    ph.i[rt.AT_I_HEADS] = heads
    ph.i[rt.AT_I_KV_HEADS] = kv_heads
    ph.i[rt.AT_I_HEAD_DIM] = dim
    ph.i[rt.AT_I_CAPACITY] = capacity
    ph.i[rt.AT_I_INVFREQ_BF16] = 1
    ph.i[rt.AT_I_MAX_CHUNKS] = max_chunks
    exact_keys = pl.exact_softmax_keys(capacity) if exact else 0
    merge_slots = pl.attention_merge_slots(dim, group)
    ph.i[rt.AT_I_MERGE_SLOTS] = merge_slots
    ph.i[rt.AT_I_EXACT_KEYS] = exact_keys
    ph.f[rt.AT_F_SCALE] = dim ** -0.5
    ph.f[rt.AT_F_ROPE_SCALE] = 1.0
    for index, (name, tensor) in enumerate([
        ("q", qd), ("k", kd), ("v", vd), ("kc", kcd), ("vc", vcd), ("len", lend), ("pos", posd),
        ("invf", invd), ("out", out), ("partial", partial), ("cnt", counters),
    ]):
        ph.slot[index] = runner.slot(name, tensor)
    plan = runner.run([ph], pl.attention_scratch_bytes(dim, group, merge_slots))
    st = plan.status()
    assert st.code == 0, (st.code, st.phase, st.detail)
    assert int(lend.item()) == cached + 1
    assert int(counters.abs().sum().item()) == 0
    # appended rows: bit-exact up to the cos/sin rounding of the device math library
    assert max_abs(kcd[:, cached], kc_ref[:, cached]) <= 0.04
    assert (kcd[:, cached].cpu() != kc_ref[:, cached]).float().mean() < 0.02
    assert torch.equal(vcd[:, cached].cpu(), vc_ref[:, cached])
    # untouched rows stay byte-equal
    assert torch.equal(kcd[:, :cached].cpu(), kc[:, :cached])
    assert torch.equal(kcd[:, cached + 1:].cpu(), kc[:, cached + 1:])
    assert torch.equal(vcd[:, cached + 1:].cpu(), vc[:, cached + 1:])
    assert max_abs(out, ref) <= 2e-2, max_abs(out, ref)
    assert cosine(out, ref) > 0.9999
    if exact and cached + 1 <= exact_keys:
        # normalised probabilities rounded like the eager operator: nearly every output
        # element is bit-identical (the rest differ by fp32 summation order)
        assert (out.cpu() != ref).float().mean() < 0.15


def test_attention_overflow_sets_status():
    batch, heads, kv_heads, dim, capacity = 1, 4, 2, 64, 8
    q, k, v, kc, vc, inv_freq, pos, length = _attention_case(batch, heads, kv_heads, dim, 8,
                                                             capacity)
    dev = [t.cuda() for t in (q, k, v, kc, vc, inv_freq, pos, length)]
    qd, kd, vd, kcd, vcd, invd, posd, lend = dev
    out = torch.zeros(batch, heads * dim, dtype=torch.bfloat16, device="cuda")
    partial = torch.zeros(4096, dtype=torch.float32, device="cuda")
    counters = torch.zeros(4, dtype=torch.int32, device="cuda")
    runner = PhaseRunner()
    ph = rt.Phase.blank(rt.BODY_ATTN_DECODE, rt.FLAG_BARRIER | rt.FLAG_BUMP_LENGTH)
    for i, value in ((rt.AT_I_BATCH, batch), (rt.AT_I_HEADS, heads), (rt.AT_I_KV_HEADS, kv_heads),
                     (rt.AT_I_HEAD_DIM, dim), (rt.AT_I_CAPACITY, capacity),
                     (rt.AT_I_INVFREQ_BF16, 1), (rt.AT_I_MAX_CHUNKS, 1), (rt.AT_I_MERGE_SLOTS, 8)):
        ph.i[i] = value
    ph.f[rt.AT_F_SCALE] = dim ** -0.5
    ph.f[rt.AT_F_ROPE_SCALE] = 1.0
    for index, (name, tensor) in enumerate([
        ("q", qd), ("k", kd), ("v", vd), ("kc", kcd), ("vc", vcd), ("len", lend), ("pos", posd),
        ("invf", invd), ("out", out), ("partial", partial), ("cnt", counters),
    ]):
        ph.slot[index] = runner.slot(name, tensor)
    plan = runner.run([ph], pl.attention_scratch_bytes(dim, 2, 8))
    st = plan.status()
    assert st.code == 3 and st.detail == 8          # MB_ST_KV_OVERFLOW, the offending length
    assert int(lend.item()) == 8                     # state untouched
    assert torch.equal(kcd.cpu(), kc)
    plan.reset()
    assert plan.status().code == 0
