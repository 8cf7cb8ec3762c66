"""Each kernel alone against a plain float32 torch reference of the same op, at sizes other than
the engine's tiny configurations (widths and vocabularies that are no power of two, odd row
counts, head sizes in steps of 16, scattered page tables).  In the manner of
AxiomOperator/rllm's parity tests (crates/rllm-cuda/tests/common/parity.rs:130-652).
"""
import math

import numpy as np
import pytest
import torch

import plain_impl
from helpers import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from rllm_b200.csrc import ops as o
    return o


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    V, d = 311, 200
    table = rnd(V, d, seed=1).to(dtype)
    toks = torch.tensor([0, 310, 5, 5, 77], dtype=torch.int32)
    out = torch.empty(5, d, device=DEV)
    ops().embed(table.to(DEV), toks.to(DEV), out)
    assert torch.equal(out.cpu(), table.float()[toks.long()])


@pytest.mark.parametrize("d", [64, 200, 4096, 5000])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rms_norm(d, out_dtype):
    n, eps = 7, 3e-6
    x, delta, w = rnd(n, d, seed=2), rnd(n, d, seed=3), 1 + 0.1 * rnd(d, seed=4)
    ref = plain_impl.rms_norm(x + delta, w, eps)
    xd = x.to(DEV)
    out = torch.empty(n, d, dtype=out_dtype, device=DEV)
    ops().add_rms_norm(xd, delta.to(DEV), w.to(DEV), out, eps)
    tol = 1e-5 if out_dtype == torch.float32 else 5e-3
    assert rel_err(out.float().cpu(), ref) < tol
    assert torch.equal(xd.cpu(), x + delta)                      # residual stream received the sum
    # gathered rows, no write-back, no delta
    rows = torch.tensor([6, 0, 3], dtype=torch.int32)
    out2 = torch.empty(3, d, dtype=out_dtype, device=DEV)
    x2 = x.to(DEV)
    ops().add_rms_norm(x2, None, w.to(DEV), out2, eps, rows=rows.to(DEV), write_x=False)
    assert rel_err(out2.float().cpu(), plain_impl.rms_norm(x[rows.long()], w, eps)) < tol
    assert torch.equal(x2.cpu(), x)


def test_silu_mul():
    n, F = 5, 333
    gu = rnd(n, 2 * F, seed=5, scale=3.0)
    g, u = gu[:, :F], gu[:, F:]
    ref = g / (1 + torch.exp(-g)) * u
    out = torch.empty(n, F, device=DEV)
    ops().silu_mul(gu.to(DEV), out)
    assert rel_err(out.cpu(), ref) < 1e-6


@pytest.mark.parametrize("hd,H,K", [(16, 4, 2), (48, 5, 1), (128, 8, 2), (80, 3, 3)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_qk_norm_rope_store(hd, H, K, dtype):
    n, bs, pages, theta, eps = 9, 8, 6, 50000.0, 1e-5
    qkv = rnd(n, (H + 2 * K) * hd, seed=6)
    qw, kw = 1 + 0.1 * rnd(hd, seed=7), 1 + 0.1 * rnd(hd, seed=8)
    positions = torch.tensor([0, 1, 17, 300, 4095, 2, 3, 4, 5], dtype=torch.int32)
    slots = torch.tensor([40, 3, 17, 9, 8, 47, 0, 25, 31], dtype=torch.int32)
    q = qkv[:, :H * hd].view(n, H, hd)
    k = qkv[:, H * hd:(H + K) * hd].view(n, K, hd)
    v = qkv[:, (H + K) * hd:].view(n, K, hd)
    q_ref = plain_impl.rope_neox(plain_impl.rms_norm(q, qw, eps), positions.tolist(), theta)
    k_ref = plain_impl.rope_neox(plain_impl.rms_norm(k, kw, eps), positions.tolist(), theta)
    inv = 1.0 / torch.pow(torch.tensor(theta), torch.arange(0, hd, 2).float() / hd)
    kc = torch.zeros(pages, K, bs, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(n, H * hd, dtype=dtype, device=DEV)
    ops().qk_norm_rope_store(qkv.to(DEV), qw.to(DEV), kw.to(DEV), inv.to(DEV), positions.to(DEV),
                             slots.to(DEV), q_out, kc, vc, H, K, hd, bs, eps)
    # rotation angles at position 4095 differ by a few float32 ulps between sin/cos implementations
    tol = 2e-4 if dtype == torch.float32 else 1e-2
    assert rel_err(q_out.float().cpu().view(n, H, hd), q_ref) < tol
    for t in range(n):
        s = int(slots[t])
        assert rel_err(kc[s // bs, :, s % bs].float().cpu(), k_ref[t]) < tol
        assert rel_err(vc[s // bs, :, s % bs].float().cpu(), v[t]) < (1e-7 if dtype == torch.float32 else 1e-2)
    used = {int(s) for s in slots}
    for s in range(pages * bs):
        if s not in used:
            assert float(kc[s // bs, :, s % bs].abs().max()) == 0.0


@pytest.mark.parametrize("hd,H,K", [(128, 32, 8), (128, 16, 8), (128, 64, 8), (48, 5, 1), (64, 3, 2)])
def test_qk_norm_rope_store_many_tokens(hd, H, K):
    """A prompt step takes two heads per warp, a decode step
    one: the same tokens through both give the same bits, and both agree with the plain formulas."""
    o = ops()
    n, bs, theta, eps = 200, 16, 1e6, 1e-6
    pages = -(-n // bs) + 1
    qkv = rnd(n, (H + 2 * K) * hd, seed=16)
    qw, kw = 1 + 0.1 * rnd(hd, seed=17), 1 + 0.1 * rnd(hd, seed=18)
    g = torch.Generator().manual_seed(19)
    positions = torch.randint(0, 5000, (n,), generator=g, dtype=torch.int32)
    slots = torch.randperm(pages * bs, generator=g)[:n].to(torch.int32)
    inv = (1.0 / torch.pow(torch.tensor(theta), torch.arange(0, hd, 2).float() / hd)).to(DEV)
    outs = []
    for chunk in (n, 50):                       # one launch of 200 tokens; four of 50
        kc = torch.zeros(pages, K, bs, hd, dtype=torch.bfloat16, device=DEV)
        vc = torch.zeros_like(kc)
        q_out = torch.zeros(n, H * hd, dtype=torch.bfloat16, device=DEV)
        for t0 in range(0, n, chunk):
            sl = slice(t0, t0 + chunk)
            o.qk_norm_rope_store(qkv[sl].to(DEV), qw.to(DEV), kw.to(DEV), inv, positions[sl].to(DEV),
                                 slots[sl].to(DEV), q_out[sl], kc, vc, H, K, hd, bs, eps)
        outs.append((q_out.cpu(), kc.cpu(), vc.cpu()))
    for x, y in zip(*outs):
        assert torch.equal(x, y)
    q = qkv[:, :H * hd].view(n, H, hd)
    k = qkv[:, H * hd:(H + K) * hd].view(n, K, hd)
    q_ref = plain_impl.rope_neox(plain_impl.rms_norm(q, qw, eps), positions.tolist(), theta)
    k_ref = plain_impl.rope_neox(plain_impl.rms_norm(k, kw, eps), positions.tolist(), theta)
    assert rel_err(outs[0][0].float().view(n, H, hd), q_ref) < 1e-2
    for t in (0, 57, 199):
        sl = int(slots[t])
        assert rel_err(outs[0][1][sl // bs, :, sl % bs].float(), k_ref[t]) < 1e-2
    o.check_device_errors()


@pytest.mark.parametrize("hd,H,K,d,n", [(128, 8, 2, 512, 300), (64, 6, 3, 256, 1100), (128, 5, 1, 192, 257), (128, 32, 8, 1024, 1024)])
def test_qkv_norm_rope_store_fused(hd, H, K, d, n):
    """The q/k/v projection with the q/k norm, the rotary encoding and the cache write in the epilogue of
    the two-SM product, against the product followed by the kernel that does those steps alone."""
    o = ops()
    bs, theta, eps = 16, 1e6, 1e-6
    pages = -(-n // bs) + 2
    g = torch.Generator().manual_seed(31)
    h = rnd(n, d, seed=32, dtype=torch.bfloat16).to(DEV)
    w = rnd((H + 2 * K) * hd, d, seed=33, scale=0.05, dtype=torch.bfloat16).to(DEV)
    qw, kw = (1 + 0.1 * rnd(hd, seed=34)).to(DEV), (1 + 0.1 * rnd(hd, seed=35)).to(DEV)
    positions = torch.randint(0, 9000, (n,), generator=g, dtype=torch.int32).to(DEV)
    slots = torch.randperm(pages * bs, generator=g)[:n].to(torch.int32)
    slots[7] = -1                                     # a token whose keys are not kept
    slots = slots.to(DEV)
    inv = (1.0 / torch.pow(torch.tensor(theta), torch.arange(0, hd, 2).float() / hd)).to(DEV)
    table = o.rope_table(positions, inv)
    outs = []
    for fused in (False, True):
        kc = torch.zeros(pages, K, bs, hd, dtype=torch.bfloat16, device=DEV)
        vc = torch.zeros_like(kc)
        q = torch.full((n, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        if fused:
            o.qkv_norm_rope_store_fused(h, w, qw, kw, table, slots, q, kc, vc, H, K, hd, bs, eps)
        else:
            qkv = o.linear(h, w, out_dtype=torch.float32)
            o.qk_norm_rope_store(qkv, qw, kw, None, positions, slots, q, kc, vc, H, K, hd, bs, eps, cs_table=table)
        outs.append((q.float().cpu(), kc.float().cpu(), vc.float().cpu()))
    o.check_device_errors()
    for name, x, y in zip("qkv", outs[1], outs[0]):
        assert not torch.isnan(x).any()
        assert rel_err(x, y) < 1e-2, name             # one bfloat16 rounding of values that differ in the last float32 bits
        assert float((x - y).abs().mean() / y.abs().mean()) < 2e-3, name
    # a layer that reads another layer's cache writes none of its own: the queries only
    kc = torch.zeros(pages, K, bs, hd, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    q = torch.empty(n, H * hd, dtype=torch.bfloat16, device=DEV)
    o.qkv_norm_rope_store_fused(h, w, qw, kw, table, slots, q, kc, vc, H, K, hd, bs, eps, write_kv=False)
    assert torch.equal(q.float().cpu(), outs[1][0]) and float(kc.abs().max()) == 0.0 and float(vc.abs().max()) == 0.0
    # without norm weights and without a table: the plain projection, rounded
    kc = torch.zeros(pages, K, bs, hd, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    q = torch.empty(n, H * hd, dtype=torch.bfloat16, device=DEV)
    o.qkv_norm_rope_store_fused(h, w, None, None, None, slots, q, kc, vc, H, K, hd, bs, eps)
    ref = (h.float() @ w.float().t())[:, :H * hd]
    assert rel_err(q.float().cpu(), ref.cpu()) < 1e-2
    o.check_device_errors()


def paged_case(hd, H, K, bs, lens, q_lens, seed, dtype, window=0, spike=False):
    """Builds a scattered paged cache for requests of `lens` tokens whose last `q_lens` tokens are
    the step's queries; returns kernel inputs and the plain reference output."""
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    n_pages = sum(-(-L // bs) for L in lens) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    kc = torch.zeros(n_pages, K, bs, hd)
    vc = torch.zeros(n_pages, K, bs, hd)
    width = max(-(-L // bs) for L in lens)
    table = torch.zeros(R, width, dtype=torch.int32)
    qs, pos, sid, refs = [], [], [], []
    for r, (L, ql) in enumerate(zip(lens, q_lens)):
        k = torch.randn(L, K, hd, generator=g)
        v = torch.randn(L, K, hd, generator=g)
        q = torch.randn(L, H, hd, generator=g)
        if spike:
            # one far key stands out: a fault that drops or misplaces it shows at once
            far = L // 7
            k[far] *= 0.0
            k[far, :, 0] = 6.0
            q[:, :, 0] = 6.0
        k, v, q = k.to(dtype).float(), v.to(dtype).float(), q.to(dtype).float()
        for b in range(-(-L // bs)):
            page = perm.pop()
            table[r, b] = page
            m = min(bs, L - b * bs)
            kc[page, :, :m] = k[b * bs:b * bs + m].transpose(0, 1)
            vc[page, :, :m] = v[b * bs:b * bs + m].transpose(0, 1)
        full = plain_impl.attention(q, k, v, 1.0 / math.sqrt(hd), window)
        refs.append(full[L - ql:].reshape(ql, H * hd))
        qs.append(q[L - ql:].reshape(ql, H * hd))
        pos += list(range(L - ql, L))
        sid += [r] * ql
    return dict(q=torch.cat(qs).to(dtype).to(DEV), kc=kc.to(dtype).to(DEV), vc=vc.to(dtype).to(DEV),
                table=table.to(DEV), pos=torch.tensor(pos, dtype=torch.int32, device=DEV),
                sid=torch.tensor(sid, dtype=torch.int32, device=DEV), ref=torch.cat(refs),
                q_lens=q_lens, lens=lens)


@pytest.mark.parametrize("hd,H,K,bs", [(16, 4, 2, 4), (64, 6, 2, 16), (128, 8, 2, 16), (48, 5, 5, 8), (256, 2, 1, 32)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 37])
def test_paged_attention_generic(hd, H, K, bs, dtype, window):
    c = paged_case(hd, H, K, bs, lens=[300, 1, 77, 129], q_lens=[3, 1, 77, 1], seed=9, dtype=dtype,
                   window=window, spike=True)
    out = torch.empty_like(c["q"])
    ops().paged_attention_generic(c["q"], c["kc"], c["vc"], out, c["pos"], c["sid"], c["table"], H, K, hd,
                                  bs, 1.0 / math.sqrt(hd), window)
    assert rel_err(out.float().cpu(), c["ref"]) < (2e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("m,n,k", [(1, 96, 512), (3, 37, 100), (33, 130, 257), (64, 64, 64), (200, 311, 96)])
def test_gemm_plain(m, n, k):
    a, w = rnd(m, k, seed=10), rnd(n, k, seed=11)
    ref = (a.double() @ w.double().t()).float()
    out = torch.empty(m, n, device=DEV)
    ops().gemm_plain(a.to(DEV), w.to(DEV), out)
    assert rel_err(out.cpu(), ref) < 2e-6
    base = rnd(m, n, seed=12)
    acc = base.to(DEV)
    ops().gemm_plain(a.to(DEV), w.to(DEV), acc, accumulate=True)
    assert rel_err(acc.cpu(), ref + base) < 2e-6
    # a row's result does not depend on the rows around it: bit-identical alone and in the batch
    alone = torch.empty(1, n, device=DEV)
    ops().gemm_plain(a[m - 1:m].to(DEV), w.to(DEV), alone)
    assert torch.equal(alone[0], out[m - 1])


@pytest.mark.parametrize("m,n,k", [(9, 96, 512), (70, 1000, 264), (256, 384, 4096)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_lib(m, n, k, out_dtype):
    a, w = rnd(m, k, seed=13, dtype=torch.bfloat16), rnd(n, k, seed=14, dtype=torch.bfloat16)
    ref = a.float() @ w.float().t()
    out = torch.empty(m, n, dtype=out_dtype, device=DEV)
    ops().gemm_lib(a.to(DEV), w.to(DEV), out)
    assert rel_err(out.float().cpu(), ref) < (1e-5 if out_dtype == torch.float32 else 5e-3)
    if out_dtype == torch.float32:
        base = rnd(m, n, seed=15)
        acc = base.to(DEV)
        ops().gemm_lib(a.to(DEV), w.to(DEV), acc, accumulate=True)
        assert rel_err(acc.cpu(), ref + base) < 1e-5


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 17, 33, 64])
@pytest.mark.parametrize("n,k", [(96, 512), (37, 264), (4096, 4096), (1000, 12288), (50, 8)])
def test_skinny_gemm(m, n, k):
    a, w = rnd(m, k, seed=16, dtype=torch.bfloat16), rnd(n, k, seed=17, dtype=torch.bfloat16)
    ref = a.float() @ w.float().t()
    out = torch.empty(m, n, device=DEV)
    o = ops()
    o.skinny_gemm(a.to(DEV), w.to(DEV), out)
    assert rel_err(out.cpu(), ref) < 1e-5
    out16 = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    o.skinny_gemm(a.to(DEV), w.to(DEV), out16)
    assert rel_err(out16.float().cpu(), ref) < 5e-3
    base = rnd(m, n, seed=18)
    acc = base.to(DEV)
    o.skinny_gemm(a.to(DEV), w.to(DEV), acc, epilogue=o.EPI_ACCUM)
    assert rel_err(acc.cpu(), ref + base) < 1e-5
    # a request's column does not depend on its batch-mates
    alone = torch.empty(1, n, device=DEV)
    o.skinny_gemm(a[m - 1:m].to(DEV), w.to(DEV), alone)
    assert torch.equal(alone[0], out[m - 1])


@pytest.mark.parametrize("m", [1, 8, 20, 64])
@pytest.mark.parametrize("F,k", [(224, 96), (1000, 264), (12288, 4096), (37, 64)])
def test_skinny_gemm_swiglu(m, F, k):
    a = rnd(m, k, seed=19, dtype=torch.bfloat16)
    w = rnd(2 * F, k, seed=20, scale=0.2, dtype=torch.bfloat16)
    g, u = a.float() @ w[:F].float().t(), a.float() @ w[F:].float().t()
    ref = g / (1 + torch.exp(-g)) * u
    out = torch.empty(m, F, dtype=torch.bfloat16, device=DEV)
    ops().gate_up_swiglu(a.to(DEV), w.to(DEV), out)
    assert rel_err(out.float().cpu(), ref) < 5e-3
    out32 = torch.empty(m, F, device=DEV)
    ops().gate_up_swiglu(a.to(DEV), w.to(DEV), out32)
    assert rel_err(out32.cpu(), ref) < 1e-5


def test_sample_rows_matches_plain():
    rows, V = 12, 1531
    logits = rnd(rows, V, seed=21, scale=3.0)
    logits[3, 7] = logits[3].max() + 1
    logits[3, 900] = logits[3, 7]                    # tie: the lower index wins
    logits[4, 11] = float("nan")                     # NaNs never win
    o = ops()
    ids = torch.empty(rows, dtype=torch.int32, device=DEV)
    o.sample_rows(logits.to(DEV), ids)
    want = [plain_impl.sample_row(torch.nan_to_num(logits[r], nan=-1e30).numpy(), 0, 0, 1.0, 0, 0) for r in range(rows)]
    assert ids.tolist() == want
    assert ids[3].item() == 7
    clean = torch.nan_to_num(logits, nan=-1e30)
    T = torch.tensor([0.8, 1.0, 0.5, 1.3] * 3)
    tk = torch.tensor([0, 5, 0, 40] * 3, dtype=torch.int32)
    tp = torch.tensor([1.0, 1.0, 0.9, 0.7] * 3)
    seed = torch.arange(rows, dtype=torch.int64) * 7919 + 4
    ctr = torch.arange(rows, dtype=torch.int64) + 100
    o.sample_rows(clean.to(DEV), ids, T.to(DEV), tk.to(DEV), tp.to(DEV), seed.to(DEV), ctr.to(DEV))
    want = [plain_impl.sample_row(clean[r].numpy(), float(T[r]), int(tk[r]), float(tp[r]), int(seed[r]), int(ctr[r]))
            for r in range(rows)]
    same = sum(int(a == b) for a, b in zip(ids.tolist(), want))
    assert same >= rows - 1, (ids.tolist(), want)     # float rounding of log/exp may flip a near tie


def test_logit_adjust_then_sample():
    """Bias and penalties on the device: logits[row, token] += delta before the draw, as the plain sampler."""
    from rllm_b200.sampling.device import sample_rows
    from rllm_b200.sampling.params import SamplingParams
    rows, V = 5, 777
    logits = rnd(rows, V, seed=51, scale=2.0)
    top = logits.argmax(1).tolist()
    params = [SamplingParams(),                                                      # untouched
              SamplingParams(logit_bias=((top[1], -50.0),)),                         # greedy, its best token banned
              SamplingParams(presence_penalty=60.0),                                 # greedy, penalised by counts
              SamplingParams(temperature=0.9, top_k=30, seed=5, frequency_penalty=1.5, logit_bias=((11, 3.0), (11, 1.0))),
              SamplingParams(temperature=1.1, top_p=0.8, seed=6)]
    counts = [None, None, {top[2]: 1}, {7: 3, 11: 2}, None]
    dev = logits.to(DEV)
    ids = sample_rows(dev, params, [0, 1, 2, 3, 4], counts).tolist()
    want = [plain_impl.sample_row(logits[r].numpy(), p.temperature, p.top_k, p.top_p, p.seed, r,
                                  adjust=p.adjustments(counts[r]).items()) for r, p in enumerate(params)]
    assert ids == want
    assert ids[0] == top[0] and ids[1] != top[1] and ids[2] != top[2]
    # the adjusted rows were changed in place, the others not
    after = dev.cpu()
    assert torch.equal(after[0], logits[0]) and torch.equal(after[4], logits[4])
    assert abs(float(after[3, 11] - logits[3, 11]) - (4.0 - 3.0)) < 1e-5 and abs(float(after[3, 7] - logits[3, 7]) + 4.5) < 1e-5


def test_sample_rows_frequencies():
    """Draws follow softmax(logits / T) (crates/rllm-core/src/sample.rs:133-161)."""
    V, N = 6, 20000
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 1.5, -3.0]]).repeat(N, 1)
    ids = torch.empty(N, dtype=torch.int32, device=DEV)
    T = torch.full((N,), 0.7)
    ops().sample_rows(logits.to(DEV), ids, T.to(DEV), torch.zeros(N, dtype=torch.int32, device=DEV),
                      torch.ones(N, device=DEV), torch.full((N,), 5, dtype=torch.int64, device=DEV),
                      torch.arange(N, dtype=torch.int64, device=DEV))
    freq = torch.bincount(ids.cpu().long(), minlength=V).float() / N
    p = torch.softmax(logits[0] / 0.7, 0)
    assert float((freq - p).abs().max()) < 0.015


class FakeCtx:
    """The part of a StepContext the attention dispatcher reads."""

    def __init__(self, case):
        self.n_requests = len(case["lens"])
        self.q_lens = list(case["q_lens"])
        self.start_pos = [L - q for L, q in zip(case["lens"], case["q_lens"])]
        self.positions, self.seq_ids = case["pos"], case["sid"]
        cu = [0]
        for q in self.q_lens:
            cu.append(cu[-1] + q)
        self.cu_q = torch.tensor(cu, dtype=torch.int32, device=DEV)
        self.plans = {}


@pytest.mark.parametrize("hd,H,K,bs", [(64, 4, 1, 16), (64, 6, 2, 4), (128, 8, 2, 16), (128, 5, 5, 8),
                                       (128, 8, 1, 32), (64, 40, 2, 16), (128, 3, 1, 1)])
@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("lens,q_lens", [
    ([300, 1, 77, 129], [1, 1, 1, 1]),             # pure decode, several splits
    ([300, 2, 77, 129], [3, 2, 1, 4]),             # short portions: decode shape, several tokens per tile
    ([300, 64, 77, 200], [300, 9, 77, 65]),        # prefill shape, whole prompts and portions
    ([520, 5, 90, 130], [130, 1, 17, 2]),          # mixed: both shapes in one step
])
@pytest.mark.parametrize("decode_rows", [8, 16])
def test_paged_flash_attention(hd, H, K, bs, window, lens, q_lens, decode_rows, monkeypatch):
    c = paged_case(hd, H, K, bs, lens=lens, q_lens=q_lens, seed=23, dtype=torch.bfloat16, window=window,
                   spike=True)
    out = torch.full_like(c["q"], float("nan"))
    ctx = FakeCtx(c)
    monkeypatch.setattr(ops(), "DECODE_ROWS", decode_rows)           # both decode kernels: keys as the M side (8 rows), 16 rows
    ops().paged_attention(c["q"], c["kc"], c["vc"], out, ctx, c["table"], H, K, hd, bs, 1.0 / math.sqrt(hd), window)
    assert ctx.plans, "the tensor-core path was not taken"
    assert torch.isfinite(out.float()).all()
    # the probabilities are rounded to bfloat16 before P.V: errors of a few bfloat16 ulps of the output
    assert rel_err(out.float().cpu(), c["ref"]) < 1.5e-2
    plain = torch.empty_like(c["q"])
    ops().paged_attention_generic(c["q"], c["kc"], c["vc"], plain, c["pos"], c["sid"], c["table"], H, K, hd,
                                  bs, 1.0 / math.sqrt(hd), window)
    assert rel_err(out.float().cpu(), plain.float().cpu()) < 1.5e-2


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (65, 40, 8), (200, 300, 264), (1000, 1111, 1096), (2048, 512, 4096)])
def test_gemm_tc(m, n, k):
    """The tcgen05 / TMA product: tiles that are cut by every edge (m, n and k tails)."""
    o = ops()
    a, w = rnd(m, k, seed=24, dtype=torch.bfloat16), rnd(n, k, seed=25, scale=0.1, dtype=torch.bfloat16)
    ref = a.float() @ w.float().t()
    out = torch.full((m, n), float("nan"), device=DEV)
    o.gemm_tc(a.to(DEV), w.to(DEV), out)
    torch.cuda.synchronize()
    o.check_device_errors()
    assert rel_err(out.cpu(), ref) < 1e-5
    out16 = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(a.to(DEV), w.to(DEV), out16)
    assert rel_err(out16.float().cpu(), ref) < 5e-3
    base = rnd(m, n, seed=26)
    acc = base.to(DEV)
    o.gemm_tc(a.to(DEV), w.to(DEV), acc, epilogue=o.EPI_ACCUM)
    assert rel_err(acc.cpu(), ref + base) < 1e-5
    plain = torch.empty(m, n, device=DEV)
    o.gemm_plain(a.to(DEV), w.to(DEV), plain)
    assert rel_err(out.cpu(), plain.cpu()) < 1e-5
    o.check_device_errors()


@pytest.mark.parametrize("m,F,k", [(65, 224, 96), (300, 1000, 264), (1024, 3072, 1024)])
def test_gemm_tc_swiglu(m, F, k):
    o = ops()
    a = rnd(m, k, seed=27, dtype=torch.bfloat16)
    w = rnd(2 * F, k, seed=28, scale=0.2, dtype=torch.bfloat16)
    g, u = a.float() @ w[:F].float().t(), a.float() @ w[F:].float().t()
    ref = g / (1 + torch.exp(-g)) * u
    out = torch.full((m, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.gate_up_swiglu(a.to(DEV), w.to(DEV), out)
    assert rel_err(out.float().cpu(), ref) < 5e-3
    out32 = torch.full((m, F), float("nan"), device=DEV)
    o.gemm_tc(a.to(DEV), w.to(DEV), out32, epilogue=o.EPI_SWIGLU, up_row_offset=F)
    assert rel_err(out32.cpu(), ref) < 1e-5
    o.check_device_errors()


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (65, 40, 8), (200, 300, 264), (1000, 1111, 1096), (2048, 512, 4096),
                                   (300, 700, 136), (4096, 1024, 128)])
def test_gemm_tc2(m, n, k):
    """The product with two SMs per tile (tcgen05.mma.cta_group::2): tiles cut by every edge, K that
    ends inside a stage of 128 and inside a block of 64, more tiles than pairs (both accumulator
    buffers in turn)."""
    o = ops()
    a, w = rnd(m, k, seed=24, dtype=torch.bfloat16), rnd(n, k, seed=25, scale=0.1, dtype=torch.bfloat16)
    ref = a.float() @ w.float().t()
    for _ in range(2):
        out = torch.full((m, n), float("nan"), device=DEV)
        o.gemm_tc2(a.to(DEV), w.to(DEV), out)
        torch.cuda.synchronize()
        o.check_device_errors()
        assert rel_err(out.cpu(), ref) < 1e-5
    out16 = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.gemm_tc2(a.to(DEV), w.to(DEV), out16)
    assert rel_err(out16.float().cpu(), ref) < 5e-3
    base = rnd(m, n, seed=26)
    acc = base.to(DEV)
    o.gemm_tc2(a.to(DEV), w.to(DEV), acc, epilogue=o.EPI_ACCUM)
    assert rel_err(acc.cpu(), ref + base) < 1e-5
    one = torch.empty(m, n, device=DEV)
    o.gemm_tc(a.to(DEV), w.to(DEV), one)
    assert rel_err(out.cpu(), one.cpu()) < 1e-6          # the one-CTA kernel adds in the same order
    o.check_device_errors()


@pytest.mark.parametrize("m,F,k", [(65, 224, 96), (300, 1000, 264), (1024, 3072, 1024), (2048, 1536, 512)])
def test_gemm_tc2_swiglu(m, F, k):
    o = ops()
    a = rnd(m, k, seed=27, dtype=torch.bfloat16)
    w = rnd(2 * F, k, seed=28, scale=0.2, dtype=torch.bfloat16)
    g, u = a.float() @ w[:F].float().t(), a.float() @ w[F:].float().t()
    ref = g / (1 + torch.exp(-g)) * u
    out = torch.full((m, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.gemm_tc2(a.to(DEV), w.to(DEV), out, epilogue=o.EPI_SWIGLU, up_row_offset=F)
    assert rel_err(out.float().cpu(), ref) < 5e-3
    out32 = torch.full((m, F), float("nan"), device=DEV)
    o.gemm_tc2(a.to(DEV), w.to(DEV), out32, epilogue=o.EPI_SWIGLU, up_row_offset=F)
    assert rel_err(out32.cpu(), ref) < 1e-5
    o.check_device_errors()


@pytest.mark.parametrize("m", [1, 8, 17, 32, 33, 64])
@pytest.mark.parametrize("n,k,splits", [(96, 512, None), (37, 264, 1), (4096, 4096, None), (1000, 1096, 3), (300, 8, 1),
                                        (130, 2048, 4), (640, 4096, 8), (200, 1024, 2)])
def test_skinny_gemm_tc(m, n, k, splits):
    """The swapped tcgen05 product: weights as the streamed operand, with and without split K (2, 4
    and 8 CTAs of a cluster share the additions and the writes; 3 leaves them to the leader)."""
    o = ops()
    a, w = rnd(m, k, seed=29, dtype=torch.bfloat16), rnd(n, k, seed=30, scale=0.1, dtype=torch.bfloat16)
    ref = a.float() @ w.float().t()
    for _ in range(2):                               # twice: the tile counters must have been reset
        out = torch.full((m, n), float("nan"), device=DEV)
        o.skinny_gemm_tc(a.to(DEV), w.to(DEV), out, n_splits=splits)
        assert rel_err(out.cpu(), ref) < 1e-5
    out16 = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.skinny_gemm_tc(a.to(DEV), w.to(DEV), out16, n_splits=splits)
    assert rel_err(out16.float().cpu(), ref) < 5e-3
    base = rnd(m, n, seed=31)
    acc = base.to(DEV)
    o.skinny_gemm_tc(a.to(DEV), w.to(DEV), acc, epilogue=o.EPI_ACCUM, n_splits=splits)
    assert rel_err(acc.cpu(), ref + base) < 1e-5
    # a request's column does not depend on its batch-mates
    alone = torch.empty(1, n, device=DEV)
    o.skinny_gemm_tc(a[m - 1:m].to(DEV), w.to(DEV), alone, n_splits=splits)
    assert torch.equal(alone[0], out[m - 1])
    o.check_device_errors()


@pytest.mark.parametrize("m", [2, 20, 64])
@pytest.mark.parametrize("F,k,splits", [(224, 96, 1), (1000, 264, 2), (12288, 4096, None), (37, 64, 1)])
def test_skinny_gemm_tc_swiglu(m, F, k, splits):
    o = ops()
    a = rnd(m, k, seed=32, dtype=torch.bfloat16)
    w = rnd(2 * F, k, seed=33, scale=0.2, dtype=torch.bfloat16)
    g, u = a.float() @ w[:F].float().t(), a.float() @ w[F:].float().t()
    ref = g / (1 + torch.exp(-g)) * u
    out = torch.full((m, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.skinny_gemm_tc(a.to(DEV), w.to(DEV), out, epilogue=o.EPI_SWIGLU, up_row_offset=F, n_splits=splits)
    assert rel_err(out.float().cpu(), ref) < 5e-3
    out32 = torch.full((m, F), float("nan"), device=DEV)
    o.skinny_gemm_tc(a.to(DEV), w.to(DEV), out32, epilogue=o.EPI_SWIGLU, up_row_offset=F, n_splits=splits)
    assert rel_err(out32.cpu(), ref) < 1e-5
    o.check_device_errors()


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n,k,grid,stages", [(96, 512, None, None), (37, 64, 3, 3), (4096, 4096, None, None),
                                             (1000, 1216, 148, 5), (6144, 1024, 444, 3), (520, 12288, 148, 10),
                                             (8, 192, None, None), (2500, 320, 7, 5)])
def test_gemv_stream(m, n, k, grid, stages):
    """The persistent TMA-fed product for decode steps: every stage shape (shares of 1, 2 and more
    granules), shares that end inside a stage, rows that are no multiple of 8, k that is no multiple
    of a stage, one and two batch tiles."""
    o = ops()
    a, w = rnd(m, k, seed=41, dtype=torch.bfloat16), rnd(n, k, seed=42, scale=0.1, dtype=torch.bfloat16)
    ref = a.float() @ w.float().t()
    for _ in range(2):
        out = torch.full((m, n), float("nan"), device=DEV)
        o.gemv_stream(a.to(DEV), w.to(DEV), out, grid=grid, stages=stages)
        assert rel_err(out.cpu(), ref) < 1e-5
    out16 = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.gemv_stream(a.to(DEV), w.to(DEV), out16, grid=grid, stages=stages)
    assert rel_err(out16.float().cpu(), ref) < 5e-3
    base = rnd(m, n, seed=43)
    acc = base.to(DEV)
    o.gemv_stream(a.to(DEV), w.to(DEV), acc, epilogue=o.EPI_ACCUM, grid=grid, stages=stages)
    assert rel_err(acc.cpu(), ref + base) < 1e-5
    # a request's column does not depend on its batch-mates, nor on the grid
    alone = torch.empty(1, n, device=DEV)
    o.gemv_stream(a[m - 1:m].to(DEV), w.to(DEV), alone, grid=grid, stages=stages)
    assert torch.equal(alone[0], out[m - 1])
    other = torch.empty(m, n, device=DEV)
    o.gemv_stream(a.to(DEV), w.to(DEV), other, grid=5, stages=3)
    assert torch.equal(other, out)
    o.check_device_errors()


@pytest.mark.parametrize("m", [2, 8, 13])
@pytest.mark.parametrize("F,k,grid,stages", [(224, 128, None, None), (1000, 320, 148, 5), (12288, 4096, None, None),
                                             (37, 64, 2, 3), (3072, 1024, 444, 3)])
def test_gemv_stream_swiglu(m, F, k, grid, stages):
    o = ops()
    a = rnd(m, k, seed=44, dtype=torch.bfloat16)
    w = rnd(2 * F, k, seed=45, scale=0.2, dtype=torch.bfloat16)
    g, u = a.float() @ w[:F].float().t(), a.float() @ w[F:].float().t()
    ref = g / (1 + torch.exp(-g)) * u
    out = torch.full((m, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.gemv_stream(a.to(DEV), w.to(DEV), out, epilogue=o.EPI_SWIGLU, up_row_offset=F, grid=grid, stages=stages)
    assert rel_err(out.float().cpu(), ref) < 5e-3
    out32 = torch.full((m, F), float("nan"), device=DEV)
    o.gemv_stream(a.to(DEV), w.to(DEV), out32, epilogue=o.EPI_SWIGLU, up_row_offset=F, grid=grid, stages=stages)
    assert rel_err(out32.cpu(), ref) < 1e-5
    o.check_device_errors()


@pytest.mark.parametrize("m", [1, 5, 8, 13])
@pytest.mark.parametrize("d,k,F,grid", [(1024, 512, 768, None), (4096, 4096, 12288, None), (320, 192, 100, 7),
                                        (960, 64, 520, 148)])
def test_gemv_stream_deferred_norm(m, d, k, F, grid):
    """An RMSNorm between two products without a kernel of its own: the accumulating product also
    writes bfloat16(x * norm weight) and the rows' sums of squares in per-CTA partial sums, the
    product behind it (plain, and fused gate/up) divides its result rows by the rms.  Against
    rmsnorm(x) . W^T computed plainly; the partial sums against the sum of squares of the rows."""
    o = ops()
    eps = 1e-5
    a = rnd(m, k, seed=51, dtype=torch.bfloat16)
    w_before = rnd(d, k, seed=52, scale=0.1, dtype=torch.bfloat16)
    base = rnd(m, d, seed=53)
    norm_w = 1.0 + rnd(d, seed=54, scale=0.1)
    w_after = rnd(2 * F, d, seed=55, scale=0.1, dtype=torch.bfloat16)
    x = base + a.float() @ w_before.float().t()                      # the residual stream after the first product
    resid = base.to(DEV)
    rows = o.gemv_stream(a.to(DEV), w_before.to(DEV), resid, epilogue=o.EPI_ACCUM, grid=grid,
                         then_norm=(norm_w.to(DEV), eps))
    assert isinstance(rows, o.NormedRows) and rows.shape == (m, d) and rows.d == d
    assert rel_err(resid.cpu(), x) < 1e-5
    assert rel_err(rows.xw.float().cpu(), x * norm_w) < 5e-3         # one bfloat16 rounding
    ssq = rows.ssq[:rows.n_parts].sum(0).cpu()
    assert rel_err(ssq[:m], (x * x).sum(-1)) < 1e-5
    assert (ssq[m:] == 0).all()
    # what the norm kernel followed by the product would give, from the same bfloat16 xw
    r = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / d + eps)
    h = rows.xw.float().cpu() * r
    ref = h @ w_after[:F].float().t()
    out = torch.full((m, F), float("nan"), device=DEV)
    o.gemv_stream(rows, w_after[:F].contiguous().to(DEV), out, grid=grid)
    assert rel_err(out.cpu(), ref) < 2e-5
    g, u = ref, h @ w_after[F:].float().t()
    act = torch.full((m, F), float("nan"), device=DEV)
    o.gemv_stream(rows, w_after.to(DEV), act, epilogue=o.EPI_SWIGLU, up_row_offset=F, grid=grid)
    assert rel_err(act.cpu(), g / (1 + torch.exp(-g)) * u) < 2e-5
    # against the norm itself (no bfloat16 hand-over in the plain formula): one rounding apart
    plain = (x * r * norm_w) @ w_after[:F].float().t()
    assert rel_err(out.cpu(), plain) < 5e-3
    # a row's result does not depend on its batch-mates
    if m > 1:
        resid1 = base[m - 1:].to(DEV)
        rows1 = o.gemv_stream(a[m - 1:].to(DEV), w_before.to(DEV), resid1, epilogue=o.EPI_ACCUM, grid=grid,
                              then_norm=(norm_w.to(DEV), eps))
        out1 = torch.empty(1, F, device=DEV)
        o.gemv_stream(rows1, w_after[:F].contiguous().to(DEV), out1, grid=grid)
        assert torch.equal(out1[0], out[m - 1])
    o.check_device_errors()


@pytest.mark.parametrize("m", [17, 32, 40, 64])
@pytest.mark.parametrize("d,k,F,splits", [(1024, 512, 768, None), (4096, 4096, 12288, None), (320, 192, 100, 1),
                                          (960, 512, 520, 3), (600, 1024, 136, 2), (520, 2048, 72, 8)])
def test_skinny_gemm_tc_deferred_norm(m, d, k, F, splits):
    """The same contract on the tcgen05 weight-streaming kernel (17 to 64 rows): every way its
    epilogue is shared by a cluster (1 CTA; 2, 4, 8 CTAs that each write a share of the rows; 3 CTAs
    whose leader writes all), widths that are no multiple of the 128-row tile."""
    o = ops()
    eps = 1e-5
    a = rnd(m, k, seed=61, dtype=torch.bfloat16)
    w_before = rnd(d, k, seed=62, scale=0.1, dtype=torch.bfloat16)
    base = rnd(m, d, seed=63)
    norm_w = 1.0 + rnd(d, seed=64, scale=0.1)
    w_after = rnd(2 * F, d, seed=65, scale=0.1, dtype=torch.bfloat16)
    x = base + a.float() @ w_before.float().t()
    resid = base.to(DEV)
    rows = o.skinny_gemm_tc(a.to(DEV), w_before.to(DEV), resid, epilogue=o.EPI_ACCUM, n_splits=splits,
                            then_norm=(norm_w.to(DEV), eps))
    assert isinstance(rows, o.NormedRows) and rows.shape == (m, d) and rows.d == d and rows.cols == 64
    assert rel_err(resid.cpu(), x) < 1e-5
    assert rel_err(rows.xw.float().cpu(), x * norm_w) < 5e-3         # one bfloat16 rounding
    ssq = rows.ssq[:rows.n_parts].sum(0).cpu()
    assert rel_err(ssq[:m], (x * x).sum(-1)) < 1e-5
    assert (ssq[m:(32 if m <= 32 else 64)] == 0).all()
    r = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / d + eps)
    h = rows.xw.float().cpu() * r
    ref = h @ w_after[:F].float().t()
    for dt, tol in ((torch.float32, 2e-5), (torch.bfloat16, 5e-3)):
        out = torch.full((m, F), float("nan"), device=DEV, dtype=dt)
        o.skinny_gemm_tc(rows, w_after[:F].contiguous().to(DEV), out, n_splits=splits)
        assert rel_err(out.float().cpu(), ref) < tol
        g, u = ref, h @ w_after[F:].float().t()
        act = torch.full((m, F), float("nan"), device=DEV, dtype=dt)
        o.skinny_gemm_tc(rows, w_after.to(DEV), act, epilogue=o.EPI_SWIGLU, up_row_offset=F)
        assert rel_err(act.float().cpu(), g / (1 + torch.exp(-g)) * u) < tol
    out = torch.full((m, F), float("nan"), device=DEV)
    o.skinny_gemm_tc(rows, w_after[:F].contiguous().to(DEV), out, n_splits=splits)
    plain = (x * r * norm_w) @ w_after[:F].float().t()
    assert rel_err(out.cpu(), plain) < 5e-3
    # through the dispatch: linear and gate_up_swiglu take the rows to the kernel that made them
    out2 = o.linear(rows, w_after[:F].contiguous().to(DEV), out_dtype=torch.float32)
    assert rel_err(out2.cpu(), ref) < 2e-5
    # a row's result does not depend on its batch-mates
    resid1 = base[m - 1:].to(DEV)
    rows1 = o.skinny_gemm_tc(a[m - 1:].to(DEV), w_before.to(DEV), resid1, epilogue=o.EPI_ACCUM, n_splits=splits,
                             then_norm=(norm_w.to(DEV), eps))
    out1 = torch.empty(1, F, device=DEV)
    o.skinny_gemm_tc(rows1, w_after[:F].contiguous().to(DEV), out1, n_splits=splits)
    assert torch.equal(out1[0], out[m - 1])
    o.check_device_errors()


def test_defers_norm_rule():
    """A norm between two products is deferred whenever both can run on a few-row kernel: bfloat16
    matrices with rows of a multiple of 8 elements, at most 64 batch rows."""
    o = ops()
    w_o = torch.empty(4096, 4096, dtype=torch.bfloat16, device=DEV)
    w_gu = torch.empty(2 * 12288, 4096, dtype=torch.bfloat16, device=DEV)
    for m, want in ((1, True), (8, True), (9, True), (16, True), (17, True), (64, True), (65, False), (0, False)):
        assert o.defers_norm(m, w_o, w_gu, True) == want, m
    small = torch.empty(256, 128, dtype=torch.bfloat16, device=DEV)
    assert o.defers_norm(32, small, small)
    assert not o.defers_norm(8, small, torch.empty(64, 100, dtype=torch.bfloat16, device=DEV))      # rows of 100 elements
    assert not o.defers_norm(8, small.float(), small)


@pytest.mark.parametrize("m", [1, 3, 8, 13, 16, 17, 40, 64])
@pytest.mark.parametrize("d,k,F", [(320, 192, 100), (1024, 2048, 3072), (72, 40, 56)])
def test_skinny_gemm_deferred_norm(m, d, k, F):
    """The same contract on the mma.sync kernel of short-lived CTAs (small matrices, any row count
    up to 64): parts of 16 columns up to 16 rows, of 64 above."""
    o = ops()
    eps = 1e-5
    a = rnd(m, k, seed=71, dtype=torch.bfloat16)
    w_before = rnd(d, k, seed=72, scale=0.1, dtype=torch.bfloat16)
    base = rnd(m, d, seed=73)
    norm_w = 1.0 + rnd(d, seed=74, scale=0.1)
    w_after = rnd(2 * F, d, seed=75, scale=0.1, dtype=torch.bfloat16)
    x = base + a.float() @ w_before.float().t()
    resid = base.to(DEV)
    rows = o.skinny_gemm(a.to(DEV), w_before.to(DEV), resid, epilogue=o.EPI_ACCUM, then_norm=(norm_w.to(DEV), eps))
    assert isinstance(rows, o.NormedRows) and rows.shape == (m, d) and rows.cols == (16 if m <= 16 else 64)
    assert rows.n_parts == -(-d // 16)
    assert rel_err(resid.cpu(), x) < 1e-5
    assert rel_err(rows.xw.float().cpu(), x * norm_w) < 5e-3
    ssq = rows.ssq[:rows.n_parts].sum(0).cpu()
    assert rel_err(ssq[:m], (x * x).sum(-1)) < 1e-5
    r = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / d + eps)
    h = rows.xw.float().cpu() * r
    ref = h @ w_after[:F].float().t()
    out = torch.full((m, F), float("nan"), device=DEV)
    o.skinny_gemm(rows, w_after[:F].contiguous().to(DEV), out)
    assert rel_err(out.cpu(), ref) < 2e-5
    g, u = ref, h @ w_after[F:].float().t()
    act = torch.full((m, F), float("nan"), device=DEV, dtype=torch.bfloat16)
    o.skinny_gemm(rows, w_after.to(DEV), act, epilogue=o.EPI_SWIGLU, up_row_offset=F)
    assert rel_err(act.float().cpu(), g / (1 + torch.exp(-g)) * u) < 5e-3
    # a row's result does not depend on its batch-mates
    resid1 = base[m - 1:].to(DEV)
    rows1 = o.skinny_gemm(a[m - 1:].to(DEV), w_before.to(DEV), resid1, epilogue=o.EPI_ACCUM,
                          then_norm=(norm_w.to(DEV), eps))
    out1 = torch.empty(1, F, device=DEV)
    o.skinny_gemm(rows1, w_after[:F].contiguous().to(DEV), out1)
    assert torch.equal(out1[0], out[m - 1])
    o.check_device_errors()


@pytest.mark.parametrize("m", [2, 8, 12, 16, 24, 64])
def test_deferred_norm_across_kernels(m):
    """Any of the three few-row kernels may prepare a norm and any may finish it: the parts they
    leave differ only in their width (16 or 64 columns), which every reader is told."""
    o = ops()
    eps, d, k, F = 1e-6, 1024, 512, 640
    a = rnd(m, k, seed=81, dtype=torch.bfloat16)
    w_before = rnd(d, k, seed=82, scale=0.1, dtype=torch.bfloat16).to(DEV)
    base = rnd(m, d, seed=83)
    norm_w = (1.0 + rnd(d, seed=84, scale=0.1)).to(DEV)
    w_after = rnd(F, d, seed=85, scale=0.1, dtype=torch.bfloat16).to(DEV)
    x = base + a.float() @ w_before.float().cpu().t()
    r = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / d + eps)
    kernels = {"skinny": o.skinny_gemm, "swap": o.skinny_gemm_tc}
    if m <= 16:
        kernels["stream"] = o.gemv_stream
    for pname, producer in kernels.items():
        resid = base.to(DEV)
        rows = producer(a.to(DEV), w_before, resid, epilogue=o.EPI_ACCUM, then_norm=(norm_w, eps))
        ref = (rows.xw.float().cpu() * r) @ w_after.float().cpu().t()
        for cname, consumer in kernels.items():
            out = torch.full((m, F), float("nan"), device=DEV)
            consumer(rows, w_after, out)
            assert rel_err(out.cpu(), ref) < 2e-5, (pname, cname)
    o.check_device_errors()


def test_gemv_stream_lm_head_size():
    """The largest matrix of the decode step (vocabulary 151,936 x 4,096): 444 CTAs, dozens of chunks each."""
    o = ops()
    m, n, k = 8, 151936, 4096
    a, w = rnd(m, k, seed=46, dtype=torch.bfloat16), rnd(n, k, seed=47, scale=0.05, dtype=torch.bfloat16)
    ref = a.float() @ w.float().t()
    out = torch.full((m, n), float("nan"), device=DEV)
    o.gemv_stream(a.to(DEV), w.to(DEV), out)
    assert rel_err(out.cpu(), ref) < 1e-5
    again = torch.full((m, n), float("nan"), device=DEV)
    o.gemv_stream(a.to(DEV), w.to(DEV), again)
    assert torch.equal(again, out)
    o.check_device_errors()


def test_opbench_times_a_product():
    """The single-kernel timer runs its graph of back-to-back launches and reports a positive time."""
    from rllm_b200.csrc import opbench
    us, gbs = opbench.time_product("skinny_gemm_tc", 24, 1024, 2048, "accum", launches=8)
    assert us > 0 and gbs > 0
    us, gbs = opbench.time_product("gemv_stream", 8, 4096, 2048, "swiglu", launches=8)
    assert us > 0 and gbs > 0
