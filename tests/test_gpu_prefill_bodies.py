"""Prefill bodies (one kernel launch per phase) against the CPU oracle, through the C ABI."""

import pytest
import torch

from megabake_b200 import runtime as rt
from oracle import decoder_oracle as oracle
from tests.helpers import PhaseRunner, cosine, max_abs

pytestmark = [pytest.mark.gpu, pytest.mark.timeout(300)]


def _bf16(*shape, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


def _ref_linear(x, w, b=None):
    acc = x.double() @ w.double().t()
    if b is not None:
        acc = acc + b.double()
    return acc.float().to(torch.bfloat16)


def _run(runner, phases):
    plan = runner.run(phases, mode=rt.MODE_PREFILL)
    st = plan.status()
    assert st.code == 0, (st.code, st.phase, st.detail)
    return plan


def _mismatch(a, b):
    return (a.cpu() != b.cpu()).float().mean().item()


@pytest.mark.parametrize("scale", [0.0, 16.0])
def test_embed_rows(scale):
    table = _bf16(300, 256, seed=1)
    ids = torch.tensor([5, 299, 0, 17, 17, 123], dtype=torch.int64)
    out = torch.zeros(6, 256, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    ph = rt.Phase.blank(rt.BODY_EMBED_ROWS, 0)
    ph.i[rt.EM_I_ROWS], ph.i[rt.EM_I_K], ph.i[rt.EM_I_VOCAB] = 6, 256, 300
    ph.f[rt.EM_F_SCALE] = scale
    ph.slot[rt.EM_S_TABLE] = runner.slot("t", table.cuda())
    ph.slot[rt.EM_S_IDS] = runner.slot("i", ids.cuda())
    ph.slot[rt.EM_S_OUT] = runner.slot("o", out)
    _run(runner, [ph])
    ref = table[ids]
    if scale:
        ref = ref * torch.tensor(scale, dtype=torch.bfloat16)
    assert torch.equal(out.cpu(), ref)


def test_embed_rows_reports_bad_token():
    table = _bf16(10, 64, seed=1).cuda()
    ids = torch.tensor([3, 10], dtype=torch.int64).cuda()
    out = torch.zeros(2, 64, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    ph = rt.Phase.blank(rt.BODY_EMBED_ROWS, 0)
    ph.i[rt.EM_I_ROWS], ph.i[rt.EM_I_K], ph.i[rt.EM_I_VOCAB] = 2, 64, 10
    ph.slot[rt.EM_S_TABLE] = runner.slot("t", table)
    ph.slot[rt.EM_S_IDS] = runner.slot("i", ids)
    ph.slot[rt.EM_S_OUT] = runner.slot("o", out)
    plan = runner.run([ph], mode=rt.MODE_PREFILL)
    st = plan.status()
    assert st.code == 4 and st.detail == 1     # MB_ST_TOKEN_RANGE, the offending row


@pytest.mark.parametrize("kind", ["llama", "gemma"])
@pytest.mark.parametrize("rows,k", [(1, 64), (13, 576), (130, 2048)])
def test_rmsnorm_rows(kind, rows, k):
    x = _bf16(rows, k, scale=2.0, seed=2)
    w = _bf16(k, scale=0.5, seed=3)
    out = torch.zeros(rows, k, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    ph = rt.Phase.blank(rt.BODY_RMSNORM_ROWS, 0)
    ph.i[rt.RN_I_ROWS], ph.i[rt.RN_I_K] = rows, k
    ph.i[rt.RN_I_KIND] = rt.PRO_RMS_LLAMA if kind == "llama" else rt.PRO_RMS_GEMMA
    ph.f[rt.RN_F_EPS] = 1e-6
    ph.slot[rt.RN_S_X] = runner.slot("x", x.cuda())
    ph.slot[rt.RN_S_W] = runner.slot("w", w.cuda())
    ph.slot[rt.RN_S_OUT] = runner.slot("o", out)
    _run(runner, [ph])
    ref = oracle.rms_norm(x, w, 1e-6, kind)
    assert _mismatch(out, ref) < 0.01          # fp32 summation order of mean(x^2)
    assert max_abs(out, ref) <= 0.04


def _gemm_phase(runner, *, x, segs, epilogue=rt.EPI_NONE, pair=None, residual=None):
    rows, k = x.shape
    ph = rt.Phase.blank(rt.BODY_GEMM_TC, 0)
    ph.i[rt.GV_I_ROWS] = rows
    ph.i[rt.GV_I_K] = k
    ph.i[rt.GV_I_NSEG] = len(segs)
    ph.i[rt.GV_I_NMAT] = 2 if pair is not None else 1
    ph.i[rt.GV_I_EPILOGUE] = epilogue
    ph.slot[rt.GV_S_X] = runner.slot("x", x)
    for i, (w, b, out) in enumerate(segs):
        ph.i[rt.GV_I_N0 + i] = w.shape[0]
        ph.slot[rt.GV_S_W0 + i] = runner.slot(f"w{i}", w)
        ph.slot[rt.GV_S_BIAS0 + i] = runner.slot(f"b{i}", b)
        ph.slot[rt.GV_S_OUT0 + i] = runner.slot(f"o{i}", out)
    ph.slot[rt.GV_S_W_PAIR] = runner.slot("pair", pair)
    ph.slot[rt.GV_S_RESIDUAL] = runner.slot("res", residual)
    return ph


def _check_gemm(out, ref):
    # one rounding of an fp32 sum against one rounding of an fp64 sum: identical except where
    # the sum sits within fp32 noise of a bf16 rounding boundary
    assert _mismatch(out, ref) < 0.01, _mismatch(out, ref)
    assert cosine(out, ref) > 0.99999
    diff = (out.float().cpu() - ref.float()).abs()
    assert bool((diff <= ref.float().abs() * 2 ** -7 + 2e-3).all())   # at most one bf16 ulp


@pytest.mark.parametrize("rows,n,k", [
    (12, 64, 64), (128, 128, 256), (128, 2048, 2048), (130, 1000, 576), (512, 8192, 2048),
    (16, 2048, 16384),      # few tiles, long reduction: split-K
    (300, 40, 72),          # ragged in every dimension (K a multiple of 8 only)
    (2048, 4096, 512),      # enough tiles for the 256-wide variant
])
def test_gemm_plain(rows, n, k):
    x = _bf16(rows, k, seed=rows + n)
    w = _bf16(n, k, scale=k ** -0.5, seed=k)
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    ph = _gemm_phase(runner, x=x.cuda(), segs=[(w.cuda(), None, out)])
    _run(runner, [ph])
    _check_gemm(out, _ref_linear(x, w))


GEMM_VARIANTS = [
    {"MEGABAKE_B200_GEMM_PERSISTENT": "0"},                              # one tile per CTA, two CTAs per SM
    {"MEGABAKE_B200_GEMM_BN": "256", "MEGABAKE_B200_GEMM_SPLIT": "1"},   # persistent, whole reductions
    {"MEGABAKE_B200_GEMM_BN": "256", "MEGABAKE_B200_GEMM_SPLIT": "3"},   # persistent, ragged slices
    {"MEGABAKE_B200_GEMM_BN": "128", "MEGABAKE_B200_GEMM_SPLIT": "5"},
]


@pytest.mark.parametrize("env", GEMM_VARIANTS, ids=lambda e: ",".join(f"{k[19:]}={v}" for k, v in e.items()))
@pytest.mark.parametrize("rows,n,k", [(130, 1000, 576), (512, 8192, 2048), (16, 2048, 16384)])
def test_gemm_tile_and_slice_choices(monkeypatch, env, rows, n, k):
    """Every kernel and geometry the cost model can pick gives the same contraction."""
    for key, value in env.items():
        monkeypatch.setenv(key, value)
    x = _bf16(rows, k, seed=rows + n)
    w = _bf16(n, k, scale=k ** -0.5, seed=k)
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    ph = _gemm_phase(runner, x=x.cuda(), segs=[(w.cuda(), None, out)])
    plan = _run(runner, [ph])
    _check_gemm(out, _ref_linear(x, w))
    first = out.clone()
    out.zero_()
    plan.launch([], torch.cuda.current_stream().cuda_stream)   # arrival counters re-armed
    torch.cuda.synchronize()
    assert plan.status().code == 0
    assert torch.equal(out, first)


@pytest.mark.parametrize("env", GEMM_VARIANTS[2:], ids=lambda e: ",".join(f"{k[19:]}={v}" for k, v in e.items()))
def test_gemm_epilogues_on_sliced_reductions(monkeypatch, env):
    """Gated pair, bias segments and the in-place residual when the last slice to arrive runs
    the epilogue from the parked partial sums."""
    for key, value in env.items():
        monkeypatch.setenv(key, value)
    rows, n, k = 200, 1536, 576
    x = _bf16(rows, k, seed=7)
    wg, wu = _bf16(n, k, scale=k ** -0.5, seed=8), _bf16(n, k, scale=k ** -0.5, seed=9)
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    ph = _gemm_phase(runner, x=x.cuda(), segs=[(wg.cuda(), None, out)], pair=wu.cuda(),
                     epilogue=rt.EPI_GELU_TANH_MUL)
    _run(runner, [ph])
    ref = oracle._activation(_ref_linear(x, wg), "gelu_tanh") * _ref_linear(x, wu)
    assert _mismatch(out, ref) < 0.03 and cosine(out, ref) > 0.99999

    ws = [_bf16(m, k, scale=k ** -0.5, seed=10 + i) for i, m in enumerate((896, 128, 128))]
    bs = [_bf16(m, seed=20 + i) for i, m in enumerate((896, 128, 128))]
    outs = [torch.zeros(rows, m, dtype=torch.bfloat16, device="cuda") for m in (896, 128, 128)]
    runner = PhaseRunner()
    ph = _gemm_phase(runner, x=x.cuda(), segs=[(w.cuda(), b.cuda(), o) for w, b, o in zip(ws, bs, outs)])
    _run(runner, [ph])
    for w, b, o in zip(ws, bs, outs):
        _check_gemm(o, _ref_linear(x, w, b))

    w = _bf16(k, n, scale=n ** -0.5, seed=4)
    y = _bf16(rows, n, seed=6)
    hidden0 = _bf16(rows, k, seed=5)
    hidden = hidden0.clone().cuda()
    runner = PhaseRunner()
    ph = _gemm_phase(runner, x=y.cuda(), segs=[(w.cuda(), None, hidden)], residual=hidden,
                     epilogue=rt.EPI_RESIDUAL)
    _run(runner, [ph])
    ref = hidden0 + _ref_linear(y, w)
    assert _mismatch(hidden, ref) < 0.01 and cosine(hidden, ref) > 0.99999


def test_gemm_runs_twice_with_split_k():
    # the arrival counters of a split-K phase must be back at zero after a launch
    x = _bf16(16, 4096, seed=1)
    w = _bf16(256, 4096, scale=1 / 64, seed=2)
    out = torch.zeros(16, 256, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    ph = _gemm_phase(runner, x=x.cuda(), segs=[(w.cuda(), None, out)])
    plan = _run(runner, [ph])
    first = out.clone()
    out.zero_()
    plan.launch([], torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert plan.status().code == 0
    assert torch.equal(out, first)
    _check_gemm(out, _ref_linear(x, w))


def test_gemm_qkv_segments_bias():
    rows, k = 77, 896
    x = _bf16(rows, k, seed=5)
    ws = [_bf16(n, k, scale=k ** -0.5, seed=10 + i) for i, n in enumerate((896, 128, 128))]
    bs = [_bf16(n, seed=20 + i) for i, n in enumerate((896, 128, 128))]
    outs = [torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda") for n in (896, 128, 128)]
    runner = PhaseRunner()
    ph = _gemm_phase(runner, x=x.cuda(),
                     segs=[(w.cuda(), b.cuda(), o) for w, b, o in zip(ws, bs, outs)])
    _run(runner, [ph])
    for w, b, o in zip(ws, bs, outs):
        _check_gemm(o, _ref_linear(x, w, b))


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
@pytest.mark.parametrize("rows,n,k", [(50, 1536, 576), (256, 16384, 2048)])
def test_gemm_gated_pair(act, rows, n, k):
    x = _bf16(rows, k, seed=7)
    wg = _bf16(n, k, scale=k ** -0.5, seed=8)
    wu = _bf16(n, k, scale=k ** -0.5, seed=9)
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    ph = _gemm_phase(runner, x=x.cuda(), segs=[(wg.cuda(), None, out)], pair=wu.cuda(),
                     epilogue=rt.EPI_SILU_MUL if act == "silu" else rt.EPI_GELU_TANH_MUL)
    _run(runner, [ph])
    gate, up = _ref_linear(x, wg), _ref_linear(x, wu)
    ref = oracle._activation(gate, act) * up
    assert _mismatch(out, ref) < 0.03
    assert cosine(out, ref) > 0.99999


def test_gemm_residual_in_place():
    rows, n, k = 140, 576, 1536
    x = _bf16(rows, k, seed=3)
    w = _bf16(n, k, scale=k ** -0.5, seed=4)
    hidden0 = _bf16(rows, n, seed=5)
    hidden = hidden0.clone().cuda()
    runner = PhaseRunner()
    ph = _gemm_phase(runner, x=x.cuda(), segs=[(w.cuda(), None, hidden)], residual=hidden,
                     epilogue=rt.EPI_RESIDUAL)
    _run(runner, [ph])
    ref = hidden0 + _ref_linear(x, w)
    assert _mismatch(hidden, ref) < 0.01
    assert cosine(hidden, ref) > 0.99999


@pytest.mark.parametrize("rows,heads,kv_heads,dim", [(12, 4, 2, 64), (130, 8, 1, 256), (64, 32, 8, 64)])
def test_rope_rows(rows, heads, kv_heads, dim):
    q = _bf16(rows, heads * dim, seed=1)
    k = _bf16(rows, kv_heads * dim, seed=2)
    inv_freq = (1.0 / (10000 ** (torch.arange(0, dim, 2).float() / dim)))
    pos = torch.arange(rows, dtype=torch.int64)
    qd, kd = q.clone().cuda(), k.clone().cuda()
    runner = PhaseRunner()
    ph = rt.Phase.blank(rt.BODY_ROPE_ROWS, 0)
    ph.i[rt.RP_I_ROWS], ph.i[rt.RP_I_HEADS], ph.i[rt.RP_I_KV_HEADS] = rows, heads, kv_heads
    ph.i[rt.RP_I_HEAD_DIM], ph.i[rt.RP_I_INVFREQ_BF16] = dim, 0
    ph.f[rt.RP_F_ROPE_SCALE] = 1.0
    ph.slot[rt.RP_S_Q] = runner.slot("q", qd)
    ph.slot[rt.RP_S_K] = runner.slot("k", kd)
    ph.slot[rt.RP_S_POS] = runner.slot("p", pos.cuda())
    ph.slot[rt.RP_S_INVFREQ] = runner.slot("f", inv_freq.cuda())
    _run(runner, [ph])
    cos, sin = oracle.rotary_tables(inv_freq, pos[None], 1.0)
    q_ref = oracle.apply_rope(q.view(1, rows, heads, dim), cos, sin).reshape(rows, -1)
    k_ref = oracle.apply_rope(k.view(1, rows, kv_heads, dim), cos, sin).reshape(rows, -1)
    # device sincosf against the host's: a different last bit of cos/sin moves a few results
    # by one bf16 ulp
    assert _mismatch(qd, q_ref) < 0.02 and max_abs(qd, q_ref) <= 0.04
    assert _mismatch(kd, k_ref) < 0.02 and max_abs(kd, k_ref) <= 0.04


@pytest.mark.parametrize("batch,tokens,heads,kv_heads,dim", [
    (2, 12, 4, 2, 64), (1, 64, 2, 2, 64), (1, 200, 8, 1, 256), (2, 130, 4, 4, 128),
    (1, 700, 9, 3, 64), (1, 1100, 2, 1, 256),
])
@pytest.mark.parametrize("explicit_mask", [False, True])
@pytest.mark.parametrize("tensor_core", [True, False])
def test_attention_prefill(batch, tokens, heads, kv_heads, dim, explicit_mask, tensor_core):
    _attention_case(batch, tokens, heads, kv_heads, dim, explicit_mask, tensor_core)


@pytest.mark.parametrize("env", [
    {"MEGABAKE_B200_ATTN_PARTS": "0"},     # one CTA per query tile, both sweeps in one launch
    {"MEGABAKE_B200_ATTN_CHUNK": "1"},     # every key block a part of its own
    {"MEGABAKE_B200_ATTN_CHUNK": "3"},     # ragged parts
], ids=lambda e: ",".join(f"{k[19:]}={v}" for k, v in e.items()))
@pytest.mark.parametrize("explicit_mask", [False, True])
def test_attention_prefill_key_parts(monkeypatch, env, explicit_mask):
    """The keys of a query tile shared out over several CTAs (statistics launch, values launch,
    last-arriver sum of the partial outputs) against the same oracle, twice with one plan."""
    for key, value in env.items():
        monkeypatch.setenv(key, value)
    plan, out, runner = _attention_case(2, 300, 4, 2, 128, explicit_mask, True)   # runner owns the inputs
    first = out.clone()
    out.zero_()
    plan.launch([], torch.cuda.current_stream().cuda_stream)   # arrival counters re-armed
    torch.cuda.synchronize()
    assert plan.status().code == 0
    assert torch.equal(out, first)


@pytest.mark.parametrize("tensor_core", [True, False])
def test_attention_prefill_rows_without_a_visible_key(tensor_core):
    """A mask tensor of finite minima (the Hugging Face form) that hides every key from some
    rows -- the rows of a left-padded prompt: eager softmax gives them the mean of V, and so
    must the kernel (their maximum is near -3.4e38, where a careless exponent overflows)."""
    _attention_case(1, 200, 4, 2, 64, True, tensor_core, hidden_rows=(0, 5, 150))


def _attention_case(batch, tokens, heads, kv_heads, dim, explicit_mask, tensor_core, hidden_rows=()):
    q = _bf16(batch, tokens, heads, dim, seed=tokens)
    k = _bf16(batch, tokens, kv_heads, dim, seed=tokens + 1)
    v = _bf16(batch, tokens, kv_heads, dim, seed=tokens + 2)
    scale = dim ** -0.5
    mask = oracle.causal_mask(batch, tokens).contiguous()
    for hidden in hidden_rows:
        mask[:, :, hidden, :] = torch.finfo(torch.bfloat16).min
    ref = oracle.prefill_attention(q, k, v, mask, scale)          # [B*H, T, D]
    ref = ref.view(batch, heads, tokens, dim).transpose(1, 2).reshape(batch * tokens, heads * dim)
    out = torch.zeros(batch * tokens, heads * dim, dtype=torch.bfloat16, device="cuda")
    runner = PhaseRunner()
    ph = rt.Phase.blank(rt.BODY_ATTN_PREFILL, 0)
    ph.i[rt.AP_I_BATCH], ph.i[rt.AP_I_TOKENS] = batch, tokens
    ph.i[rt.AP_I_HEADS], ph.i[rt.AP_I_KV_HEADS], ph.i[rt.AP_I_HEAD_DIM] = heads, kv_heads, dim
    ph.i[rt.AP_I_CAUSAL] = 0 if explicit_mask else 1
    ph.i[rt.AP_I_MASK_BATCH] = batch
    ph.f[rt.AP_F_SCALE] = scale
    ph.slot[rt.AP_S_Q] = runner.slot("q", q.reshape(batch * tokens, -1).cuda())
    ph.slot[rt.AP_S_K] = runner.slot("k", k.reshape(batch * tokens, -1).cuda())
    ph.slot[rt.AP_S_V] = runner.slot("v", v.reshape(batch * tokens, -1).cuda())
    ph.slot[rt.AP_S_OUT] = runner.slot("o", out)
    if explicit_mask:
        ph.slot[rt.AP_S_MASK] = runner.slot("m", mask.cuda())
    if tensor_core:   # scratch for the transposed values selects the tcgen05 kernel
        padded = (tokens + 63) // 64 * 64
        ph.slot[rt.AP_S_VT] = runner.slot("vt", torch.full(
            (batch * kv_heads * dim, padded), float("nan"), dtype=torch.bfloat16, device="cuda"))
    plan = _run(runner, [ph])
    assert max_abs(out, ref) <= 2e-2, max_abs(out, ref)
    assert cosine(out, ref) > 0.9999
    # the probabilities are rounded after normalisation, as in the eager operator: nearly every
    # output element is bit-identical, the rest differ by fp32 summation order
    assert _mismatch(out, ref) < 0.1, _mismatch(out, ref)
    return plan, out, runner
