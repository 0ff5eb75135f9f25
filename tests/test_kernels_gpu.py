"""Each kernel alone against a plain PyTorch 32-bit reference of the same operation, at
sizes other than the engine's tiny models: widths and vocabularies that are no power of two,
head sizes in steps of 16, group sizes 1 to 8, pages of 8, 16 and 24 tokens, windows, and
inputs made so that a single far key decides the result."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def native():
    from atom_b200 import native as n
    n.lib()
    return n


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def _tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2)


# ----------------------------------------------------------------------------- small kernels


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V,H,T", [(389, 96, 7), (1000, 200, 33), (151, 4104, 3), (77, 100, 5), (301, 4096, 9), (64, 12288, 2)])
def test_embedding(native, dtype, V, H, T):
    table = _rand((V, H), dtype, 1)
    ids = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(2)).to(torch.int32).to(DEV)
    out = torch.empty((T, H), dtype=torch.float32, device=DEV)
    native.embedding(out, table, ids)
    assert torch.equal(out, table.float()[ids.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,T,eps", [(96, 5, 1e-5), (1000, 17, 1e-6), (4104, 3, 3e-6)])
def test_add_rmsnorm(native, dtype, H, T, eps):
    res = _rand((T, H), torch.float32, 3)
    delta = _rand((T, H), dtype, 4)
    w = (_rand((H,), torch.float32, 5) * 0.1 + 1).to(dtype)
    r0 = res.clone()
    out = torch.empty((T, H), dtype=dtype, device=DEV)
    native.add_rmsnorm(out, res, delta, w, eps)
    r = r0 + delta.float()
    want = r * torch.rsqrt((r * r).mean(-1, keepdim=True) + eps) * w.float()
    assert torch.allclose(res, r, rtol=0, atol=0)
    torch.testing.assert_close(out.float(), want.to(dtype).float(), **_tol(dtype))
    # picked rows: normalised densely, the residual stays as it is
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    res2 = r0.clone()
    out2 = torch.empty((2, H), dtype=dtype, device=DEV)
    native.add_rmsnorm(out2, res2, delta, w, eps, rows, 2)
    assert torch.equal(res2, r0)
    torch.testing.assert_close(out2.float(), want[[T - 1, 0]].to(dtype).float(), **_tol(dtype))
    # no delta
    res3 = r0.clone()
    native.add_rmsnorm(out, res3, None, w, eps)
    want3 = r0 * torch.rsqrt((r0 * r0).mean(-1, keepdim=True) + eps) * w.float()
    torch.testing.assert_close(out.float(), want3.to(dtype).float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("I,T", [(160, 5), (1001, 9), (12288, 2)])
def test_silu_mul(native, dtype, I, T):
    gu = _rand((T, 2 * I), dtype, 6, 2.0)
    out = torch.empty((T, I), dtype=dtype, device=DEV)
    native.silu_mul(out, gu)
    g, u = gu.float()[:, :I], gu.float()[:, I:]
    torch.testing.assert_close(out.float(), (g * torch.sigmoid(g) * u).to(dtype).float(), **_tol(dtype))


@pytest.mark.parametrize("M,N,K", [(1, 389, 96), (37, 130, 257), (129, 64, 1000)])
def test_gemm_f32_is_true_32_bit(native, M, N, K):
    a, w = _rand((M, K), torch.float32, 7), _rand((N, K), torch.float32, 8)
    bias = _rand((N,), torch.float32, 9)
    out = torch.empty((M, N), dtype=torch.float32, device=DEV)
    native.gemm_f32(out, a, w, bias)
    want = (a.double() @ w.double().T + bias.double())
    # a reduced-precision matrix mode (10-bit mantissa) would be off by ~1e-2 here
    assert (out.double() - want).abs().max().item() < 1e-4 * math.sqrt(K / 96)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(1, 392, 96), (37, 136, 264), (300, 1000, 512)])
def test_gemm_bf16(native, out_dtype, M, N, K):
    a, w = _rand((M, K), torch.bfloat16, 10), _rand((N, K), torch.bfloat16, 11)
    out = torch.empty((M, N), dtype=out_dtype, device=DEV)
    native.gemm_bf16(out, a, w)
    want = a.float() @ w.float().T
    torch.testing.assert_close(out.float(), want.to(out_dtype).float(), rtol=1e-2, atol=1e-2 * math.sqrt(K / 96))


# ----------------------------------------------------------------------------- rope + cache write


def _rope_table(max_pos, rd, theta):
    inv = 1.0 / (theta ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    return torch.cat([ang.cos(), ang.sin()], 1).contiguous().to(DEV)


def _ref_qknorm_rope(qkv, nh, nkv, hd, qw, kw, eps, table, rd, positions):
    T = qkv.shape[0]
    x = qkv.float().view(T, nh + 2 * nkv, hd)
    q, k, v = x[:, :nh], x[:, nh:nh + nkv], x[:, nh + nkv:]

    def norm(t, w):
        if w is None:
            return t
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * w.float()

    def rope(t):
        cs = table[positions.long()]
        c, s = cs[:, None, :rd // 2], cs[:, None, rd // 2:]
        x1, x2 = t[..., :rd // 2], t[..., rd // 2:rd]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, t[..., rd:]], -1)

    return rope(norm(q, qw)), rope(norm(k, kw)), v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rd,page,use_norm", [(4, 2, 16, 16, 16, True), (5, 5, 48, 48, 8, True),
                                                          (8, 1, 128, 64, 24, False), (6, 2, 80, 80, 16, True),
                                                          (32, 8, 128, 128, 16, True), (7, 7, 64, 64, 8, False),
                                                          (6, 2, 256, 256, 16, True), (3, 1, 128, 0, 16, True)])
@pytest.mark.parametrize("q_lens,starts", [([3, 1, 19], [5, 40, 0]), ([90, 1, 70], [3, 127, 0])])
def test_qknorm_rope_kvwrite(native, dtype, nh, nkv, hd, rd, page, use_norm, q_lens, starts):
    S, T = len(q_lens), sum(q_lens)
    max_pos, eps, theta = 128, 1e-5, 10000.0
    table = _rope_table(max_pos, rd, theta)
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, q_lens)]).to(torch.int32).to(DEV)
    sot = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).to(torch.int32).to(DEV)
    P = -(-max_pos // page)
    n_pages = S * P + 4
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(12))[: S * P].view(S, P)
    bt = perm.to(torch.int32).to(DEV)
    qkv = _rand((T, (nh + 2 * nkv) * hd), dtype, 13)
    qw = (_rand((hd,), torch.float32, 14) * 0.1 + 1).to(dtype) if use_norm else None
    kw = (_rand((hd,), torch.float32, 15) * 0.1 + 1).to(dtype) if use_norm else None
    kp = torch.zeros((n_pages, nkv, page, hd), dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    rq, rk, rv = _ref_qknorm_rope(qkv, nh, nkv, hd, qw, kw, eps, table, rd, pos)
    native.qknorm_rope_kvwrite(qkv, nh, nkv, hd, qw, kw, eps, table, rd, pos, sot, bt, page, kp, vp, status)
    assert int(status.item()) == 0
    got_q = qkv.float().view(T, nh + 2 * nkv, hd)[:, :nh]
    torch.testing.assert_close(got_q, rq.to(dtype).float(), **_tol(dtype))
    written = torch.zeros((n_pages, page), dtype=torch.bool)
    for t in range(T):
        s, p = int(sot[t]), int(pos[t])
        pg = int(bt[s, p // page])
        written[pg, p % page] = True
        torch.testing.assert_close(kp[pg, :, p % page].float(), rk[t].to(dtype).float(), **_tol(dtype))
        assert torch.equal(vp[pg, :, p % page].float(), rv[t].to(dtype).float())
    # nothing else was touched
    untouched = ~written.to(DEV)
    assert float(kp.float().abs().sum(dim=(1, 3))[untouched].sum()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,T", [(3, 1, 16, 5), (5, 5, 48, 33), (32, 8, 128, 4), (6, 2, 200, 7)])
def test_qk_headnorm(native, dtype, nh, nkv, hd, T):
    """Per-head RMSNorm of the q and k heads in place; v heads and padding rows are not touched."""
    eps = 3e-6
    qkv = _rand((T, (nh + 2 * nkv) * hd), dtype, 31)
    before = qkv.clone()
    qw = (_rand((hd,), torch.float32, 32) * 0.1 + 1).to(dtype)
    kw = (_rand((hd,), torch.float32, 33) * 0.1 + 1).to(dtype)
    sot = torch.zeros(T, dtype=torch.int32, device=DEV)
    sot[T - 1] = -1                                   # a padding row
    native.qk_headnorm(qkv, nh, nkv, hd, qw, kw, eps, sot)
    x = before.double().view(T, nh + 2 * nkv, hd)
    w = torch.cat([qw.double().expand(nh, hd), kw.double().expand(nkv, hd)])
    want = x.clone()
    want[:, :nh + nkv] = x[:, :nh + nkv] * torch.rsqrt(x[:, :nh + nkv].pow(2).mean(-1, keepdim=True) + eps) * w
    want[T - 1] = x[T - 1]
    got = qkv.view(T, nh + 2 * nkv, hd)
    torch.testing.assert_close(got.float(), want.to(dtype).float(), **_tol(dtype))
    assert torch.equal(got[:, nh + nkv:], before.view(T, nh + 2 * nkv, hd)[:, nh + nkv:])
    assert torch.equal(got[T - 1], before.view(T, nh + 2 * nkv, hd)[T - 1])


# ----------------------------------------------------------------------------- attention


def _paged_case(q_lens, ctx_lens, nh, nkv, hd, page, dtype, seed, n_extra_pages=7, holes=None):
    """Random q and a paged cache with shuffled pages.  Returns the kernel inputs and dense
    per-request keys/values for the reference."""
    S, T = len(q_lens), sum(q_lens)
    P = max(-(-c // page) for c in ctx_lens)
    n_pages = sum(-(-c // page) for c in ctx_lens) + n_extra_pages
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g).tolist()
    bt = torch.full((S, P), -1, dtype=torch.int32)
    kp = torch.randn((n_pages, nkv, page, hd), generator=g).to(dtype)     # stale values on unused pages
    vp = torch.randn((n_pages, nkv, page, hd), generator=g).to(dtype)
    dense = []
    for s, c in enumerate(ctx_lens):
        k = torch.randn((c, nkv, hd), generator=g).to(dtype)
        v = torch.randn((c, nkv, hd), generator=g).to(dtype)
        dense.append((k, v))
        for lp in range(-(-c // page)):
            pg = perm.pop()
            bt[s, lp] = pg
            n = min(page, c - lp * page)
            kp[pg, :, :n] = k[lp * page: lp * page + n].transpose(0, 1)
            vp[pg, :, :n] = v[lp * page: lp * page + n].transpose(0, 1)
    q = torch.randn((T, nh, hd), generator=g).to(dtype)
    return q, kp, vp, bt, dense


def _ref_attention(q, dense, q_lens, ctx_lens, nh, nkv, scale, window):
    outs = []
    t0 = 0
    G = nh // nkv
    for s, (n, c) in enumerate(zip(q_lens, ctx_lens)):
        k, v = dense[s][0].double(), dense[s][1].double()
        qs = q[t0:t0 + n].double()
        pos = torch.arange(c - n, c)
        j = torch.arange(c)
        mask = j[None, :] <= pos[:, None]
        if window:
            mask &= j[None, :] > pos[:, None] - window
        o = torch.empty((n, nh, q.shape[-1]), dtype=torch.float64)
        for h in range(nh):
            sc = (qs[:, h] @ k[:, h // G].T) * scale
            sc = sc.masked_fill(~mask, float("-inf"))
            o[:, h] = torch.softmax(sc, -1) @ v[:, h // G]
        outs.append(o)
        t0 += n
    return torch.cat(outs).float()


def _run_attention(native, kind, q, kp, vp, bt, q_lens, ctx_lens, nh, nkv, hd, scale, window, force_splits=None):
    T, S = sum(q_lens), len(q_lens)
    dev = lambda x: x.to(DEV)
    qd, kpd, vpd, btd = dev(q.reshape(T, nh * hd).contiguous()), dev(kp), dev(vp), dev(bt.contiguous())
    cu = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32, device=DEV)
    ctx = torch.tensor(ctx_lens, dtype=torch.int32, device=DEV)
    pos = torch.cat([torch.arange(c - n, c) for n, c in zip(q_lens, ctx_lens)]).to(torch.int32).to(DEV)
    sot = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).to(torch.int32).to(DEV)
    out = torch.full((T, nh * hd), float("nan"), dtype=q.dtype, device=DEV)
    if kind == "generic":
        native.paged_attention_generic(out, qd, nh * hd, kpd, vpd, btd, pos, sot, T, nh, nkv, hd, scale, window)
    else:
        long_rows = native.LONG_ROWS if (kind == "flash_tc" and native.flash_has_tc(hd)) else 0
        plan = native.flash_plan(q_lens, nh // nkv, nkv, max(ctx_lens), long_rows=long_rows)
        if kind == "flash_tc":
            assert plan[3] > 0, "the case has no request long enough for the tcgen05 kernel"
        if force_splits:
            plan = (plan[0], plan[1], force_splits) + tuple(plan[3:])
        scratch = None
        if plan[2] > 1:
            scratch = torch.empty(native.flash_scratch_elems(T, nh, hd, plan[2]), dtype=torch.float32, device=DEV)
        native.flash_attention(out, qd, nh * hd, kpd, vpd, btd, cu, ctx, sot, T, S, nh, nkv, hd, scale,
                               window, plan, scratch)
    torch.cuda.synchronize()
    return out.float().cpu().view(T, nh, hd)


ATTN_CASES = [
    # nh, nkv, hd, page, window, q_lens, ctx_lens
    (4, 2, 16, 16, 0, [1, 7, 33], [1, 7, 33]),
    (8, 2, 32, 8, 0, [1, 2, 13, 1, 70], [100, 37, 64, 9, 70]),
    (5, 5, 48, 16, 24, [1, 40, 3], [77, 120, 31]),
    (8, 1, 64, 24, 0, [2, 1, 90], [50, 300, 91]),
    (32, 8, 128, 16, 0, [1, 1, 200, 5], [700, 129, 333, 64]),
    (6, 3, 80, 16, 50, [1, 130], [260, 130]),
    (16, 2, 256, 16, 0, [1, 35], [97, 35]),
]


@pytest.mark.parametrize("case", ATTN_CASES, ids=lambda c: f"nh{c[0]}kv{c[1]}hd{c[2]}pg{c[3]}w{c[4]}")
@pytest.mark.parametrize("kind,dtype", [("generic", torch.float32), ("generic", torch.bfloat16),
                                        ("flash", torch.bfloat16)])
def test_paged_attention(native, case, kind, dtype):
    nh, nkv, hd, page, window, q_lens, ctx_lens = case
    q, kp, vp, bt, dense = _paged_case(q_lens, ctx_lens, nh, nkv, hd, page, dtype, seed=hd + page)
    scale = hd ** -0.5
    want = _ref_attention(q, dense, q_lens, ctx_lens, nh, nkv, scale, window)
    got = _run_attention(native, kind, q, kp, vp, bt, q_lens, ctx_lens, nh, nkv, hd, scale, window)
    assert torch.isfinite(got).all()
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    err = (got - want).abs().max().item()
    assert err <= tol, f"max abs error {err:.3e}"


TC_CASES = [
    # nh, nkv, page, q_lens, ctx_lens  (head size 128; at least one request with >= 128 packed rows)
    (32, 8, 16, [1, 1, 200, 5], [700, 129, 333, 64]),
    (4, 4, 16, [300], [500]),                 # group 1, a portion that continues a cached prefix
    (8, 1, 24, [33, 64], [33, 200]),          # group 8, pages of 24 tokens
    (6, 2, 16, [129, 1, 43, 2048 // 16], [129, 1000, 300, 128]),
    (16, 4, 8, [520], [520]),                 # several key tiles, rows not a multiple of 128
    # two query tiles per CTA (pages of 8, 16, ... tokens, a group size that divides 128):
    (8, 1, 32, [16, 33, 64], [16, 400, 64]),  # group 8: 128, 264 and 512 packed rows; the second tile empty, 8 rows, full
    (4, 4, 128, [129, 257], [129, 900]),      # group 1: the second tile sees one key tile more than the first; pages of 128
    (8, 2, 16, [32, 1, 64, 96], [32, 77, 1000, 96]),   # several requests, exactly 128 / 256 / 384 rows, a long prefix
    (2, 1, 64, [700], [1500]),                # group 2, 1400 rows, prefix of 800 keys
]


@pytest.mark.parametrize("case", TC_CASES, ids=lambda c: f"nh{c[0]}kv{c[1]}pg{c[2]}")
def test_tcgen05_attention(native, case):
    nh, nkv, page, q_lens, ctx_lens = case
    hd = 128
    q, kp, vp, bt, dense = _paged_case(q_lens, ctx_lens, nh, nkv, hd, page, torch.bfloat16, seed=nh + page)
    scale = hd ** -0.5
    want = _ref_attention(q, dense, q_lens, ctx_lens, nh, nkv, scale, 0)
    got = _run_attention(native, "flash_tc", q, kp, vp, bt, q_lens, ctx_lens, nh, nkv, hd, scale, 0)
    native.check_error_flags()
    assert torch.isfinite(got).all()
    err = (got - want).abs().max().item()
    assert err <= 2e-2, f"max abs error {err:.3e}"


@pytest.mark.parametrize("far", [0, 127, 128, 300, 511])
def test_tcgen05_one_far_key_decides(native, far):
    """As test_one_far_key_decides, for a long portion on the tcgen05 kernel: the key that
    stands out lies at a tile's edge, in the first tile, in a middle one."""
    nh, nkv, hd, page = 8, 2, 128, 16
    q_lens, ctx_lens = [80], [592]
    q, kp, vp, bt, dense = _paged_case(q_lens, ctx_lens, nh, nkv, hd, page, torch.bfloat16, seed=far)
    row = 37                                    # a token in the middle of the portion
    qv = q[row, 5].float()
    key = (qv / qv.norm() * 6.0).to(torch.bfloat16)
    k0, v0 = dense[0]
    k0[far, 1] = key                            # query head 5 reads kv head 1
    kp[int(bt[0, far // page]), 1, far % page] = key
    got = _run_attention(native, "flash_tc", q, kp, vp, bt, q_lens, ctx_lens, nh, nkv, hd, 1.0, 0)
    native.check_error_flags()
    torch.testing.assert_close(got[row, 5], v0[far, 1].float(), rtol=2e-2, atol=2e-2)
    want = _ref_attention(q, dense, q_lens, ctx_lens, nh, nkv, 1.0, 0)
    assert (got - want).abs().max().item() <= 3e-2


TMA_DECODE_CASES = [
    # nh, nkv, hd, page, window, q_lens, ctx_lens, splits  (head size a multiple of 64, pages of 8, 16, ... tokens:
    # short requests take their pages as TMA boxes)
    (32, 8, 128, 16, 0, [1] * 6, [2100, 1, 63, 64, 65, 1000], 1),
    (32, 8, 128, 16, 0, [1] * 6, [2100, 1, 63, 64, 65, 1000], 5),
    (8, 4, 64, 8, 100, [1, 2, 4, 8, 3], [300, 130, 77, 8, 259], 3),      # 2 to 16 packed rows, a window
    (4, 2, 256, 32, 0, [1, 3, 8], [500, 35, 260], 2),                    # pieces of 16 keys of 32-token pages
    (6, 2, 192, 64, 0, [1, 5, 2], [333, 70, 129], 1),                    # three 64-column halves
    (8, 2, 128, 128, 0, [1, 4, 1], [700, 300, 129], 4),                  # pages larger than a tile
    (8, 4, 128, 16, 0, [1] * 40, [40 + 13 * i for i in range(40)], 1),   # more CTAs than SMs: two CTAs an SM
    (8, 4, 128, 16, 0, [1] * 40, [40 + 13 * i for i in range(40)], 3),
    (64, 8, 128, 16, 0, [1] * 5, [4096, 17, 300, 1, 1031], 4),           # group 8 (the 32B sizes): 8 packed rows
    (64, 8, 128, 16, 0, [2, 1, 2], [900, 64, 33], 2),                    # group 8, two tokens: 16 packed rows
    (32, 2, 128, 16, 0, [1] * 4, [700, 16, 129, 2000], 3),               # group 16: 16 packed rows from one token
]


@pytest.mark.parametrize("case", TMA_DECODE_CASES, ids=lambda c: f"nh{c[0]}kv{c[1]}hd{c[2]}pg{c[3]}w{c[4]}s{c[7]}n{len(c[5])}")
def test_flash_decode_tma(native, case):
    nh, nkv, hd, page, window, q_lens, ctx_lens, splits = case
    q, kp, vp, bt, dense = _paged_case(q_lens, ctx_lens, nh, nkv, hd, page, torch.bfloat16, seed=hd + page + splits)
    scale = hd ** -0.5
    want = _ref_attention(q, dense, q_lens, ctx_lens, nh, nkv, scale, window)
    got = _run_attention(native, "flash", q, kp, vp, bt, q_lens, ctx_lens, nh, nkv, hd, scale, window,
                         force_splits=splits)
    native.check_error_flags()
    assert torch.isfinite(got).all()
    err = (got - want).abs().max().item()
    assert err <= 2e-2, f"max abs error {err:.3e}"


@pytest.mark.parametrize("far", [0, 15, 16, 31, 32, 63, 64, 1023, 1024, 1999])
@pytest.mark.parametrize("splits", [1, 4])
def test_flash_decode_tma_one_far_key_decides(native, far, splits):
    """One key among two thousand decides the output: at a box's, a tile's, a ring's and a split's edge."""
    nh, nkv, hd, page = 8, 2, 128, 16
    q_lens, ctx_lens = [1, 1], [2000, 700]
    q, kp, vp, bt, dense = _paged_case(q_lens, ctx_lens, nh, nkv, hd, page, torch.bfloat16, seed=far)
    qv = q[0, 5].float()
    key = (qv / qv.norm() * 6.0).to(torch.bfloat16)
    k0, v0 = dense[0]
    k0[far, 1] = key                            # query head 5 reads kv head 1
    kp[int(bt[0, far // page]), 1, far % page] = key
    got = _run_attention(native, "flash", q, kp, vp, bt, q_lens, ctx_lens, nh, nkv, hd, 1.0, 0, force_splits=splits)
    native.check_error_flags()
    torch.testing.assert_close(got[0, 5], v0[far, 1].float(), rtol=2e-2, atol=2e-2)
    want = _ref_attention(q, dense, q_lens, ctx_lens, nh, nkv, 1.0, 0)
    assert (got - want).abs().max().item() <= 3e-2


ROTATING_CASES = [
    # nh, nkv, hd, rotary_dim, page, window, use_norm, ctx_lens (the new token is each request's last)
    (32, 8, 128, 128, 16, 0, True, [700, 1, 129, 16, 4097, 33]),
    (8, 1, 128, 64, 8, 0, False, [50, 300, 9]),
    (4, 2, 64, 64, 32, 24, True, [77, 120, 31, 2]),
    (16, 2, 256, 256, 16, 0, True, [97, 35]),
    (6, 2, 192, 96, 16, 0, True, [260, 17]),
]


@pytest.mark.parametrize("case", ROTATING_CASES, ids=lambda c: f"nh{c[0]}kv{c[1]}hd{c[2]}rd{c[3]}pg{c[4]}w{c[5]}")
@pytest.mark.parametrize("splits", [1, 3])
def test_decode_attention_that_rotates_and_stores_its_new_tokens(native, case, splits):
    """A decode step hands the raw projection [q | k | v] to the attention kernel, which normalises and
    rotates the heads, stores the new key and value in the token's page and attends over the pages and the new
    token.  The output is the float64 attention over the dense keys with the rotated new key at the end,
    the page holds the rotated key and the value, no other place of the cache changes, and the result agrees
    with the two kernels it replaces.  New tokens at a page's first and last place, a request of one token."""
    nh, nkv, hd, rd, page, window, use_norm, ctx_lens = case
    S = len(ctx_lens)
    q_lens = [1] * S
    eps, theta, scale = 1e-5, 10000.0, hd ** -0.5
    _, kp, vp, bt, dense = _paged_case(q_lens, ctx_lens, nh, nkv, hd, page, torch.bfloat16, seed=hd + page + splits)
    assert native.flash_rotating_supports(hd, page, kp.shape[0], nh, nkv, rd)
    table = _rope_table(max(ctx_lens) + 1, rd, theta)
    pos = torch.tensor([c - 1 for c in ctx_lens], dtype=torch.int32, device=DEV)
    qkv = _rand((S, (nh + 2 * nkv) * hd), torch.bfloat16, 77)
    wdt = torch.bfloat16 if hd == 128 else torch.float32                     # (norm weights of either type)
    qw = (_rand((hd,), torch.float32, 14) * 0.1 + 1).to(wdt) if use_norm else None
    kw = (_rand((hd,), torch.float32, 15) * 0.1 + 1).to(wdt) if use_norm else None
    rq, rk, rv = _ref_qknorm_rope(qkv, nh, nkv, hd, qw, kw, eps, table, rd, pos)
    rq, rk, rv = rq.bfloat16().cpu(), rk.bfloat16().cpu(), rv.bfloat16().cpu()
    # the reference sees the rotated new key and the value at each request's last position
    dense_new = []
    for s, (k, v) in enumerate(dense):
        k, v = k.clone(), v.clone()
        k[-1], v[-1] = rk[s], rv[s]
        dense_new.append((k, v))
    want = _ref_attention(rq.view(S, nh, hd), dense_new, q_lens, ctx_lens, nh, nkv, scale, window)
    kpd, vpd, btd = kp.to(DEV), vp.to(DEV), bt.contiguous().to(DEV)
    kp0, vp0 = kpd.clone(), vpd.clone()
    cu = torch.arange(S + 1, dtype=torch.int32, device=DEV)
    ctx = torch.tensor(ctx_lens, dtype=torch.int32, device=DEV)
    sot = torch.arange(S, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((S, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    scratch = torch.empty(max(1, native.flash_scratch_elems(S, nh, hd, splits)), dtype=torch.float32, device=DEV)
    raw = qkv.clone()
    native.flash_attention_rotating(out, qkv, kpd, vpd, btd, cu, ctx, sot, S, S, nh, nkv, hd, scale, window, splits,
                                    scratch, table, rd, pos, qw, kw, eps, True, status)
    native.check_error_flags()
    assert int(status.item()) == 0 and torch.equal(qkv, raw)          # (the projection is left as it was)
    got = out.float().cpu().view(S, nh, hd)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() <= 2e-2
    touched = torch.zeros(kpd.shape[0], page, dtype=torch.bool)
    for s, c in enumerate(ctx_lens):
        pg, slot = int(bt[s, (c - 1) // page]), (c - 1) % page
        touched[pg, slot] = True
        torch.testing.assert_close(kpd[pg, :, slot].float().cpu(), rk[s].float(), rtol=1.6e-2, atol=1.6e-2)
        assert torch.equal(vpd[pg, :, slot].cpu(), rv[s])
    same = ~touched.to(DEV)[:, None, :, None].expand_as(kpd)
    assert torch.equal(kpd[same], kp0[same]) and torch.equal(vpd[same], vp0[same])
    # the two kernels it replaces, from the same raw projection and the old cache
    q2, k2, v2 = raw.clone(), kp0.clone(), vp0.clone()
    native.qknorm_rope_kvwrite(q2, nh, nkv, hd, qw, kw, eps, table, rd, pos, sot, btd, page, k2, v2, status)
    plan = (0, True, splits)
    out2 = torch.empty_like(out)
    native.flash_attention(out2, q2, q2.shape[1], k2, v2, btd, cu, ctx, sot, S, S, nh, nkv, hd, scale, window, plan,
                           scratch)
    assert (out2.float() - out.float()).abs().max().item() <= 1e-2
    assert (k2.float() - kpd.float()).abs().max().item() <= 1.6e-2 and torch.equal(v2, vpd)


def test_decode_attention_that_rotates_reports_a_token_without_a_page(native):
    """The new token's position has no page in the block table: nothing is stored, the status word is set."""
    nh, nkv, hd, page = 8, 2, 128, 16
    ctx_lens = [40, 17]
    _, kp, vp, bt, _ = _paged_case([1, 1], ctx_lens, nh, nkv, hd, page, torch.bfloat16, seed=5)
    bt[1, 1] = -1
    kpd, vpd, btd = kp.to(DEV), vp.to(DEV), bt.contiguous().to(DEV)
    kp0 = kpd.clone()
    table = _rope_table(64, hd, 10000.0)
    qkv = _rand((2, (nh + 2 * nkv) * hd), torch.bfloat16, 78)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty((2, nh * hd), dtype=torch.bfloat16, device=DEV)
    native.flash_attention_rotating(out, qkv, kpd, vpd, btd, torch.arange(3, dtype=torch.int32, device=DEV),
                                    torch.tensor(ctx_lens, dtype=torch.int32, device=DEV),
                                    torch.arange(2, dtype=torch.int32, device=DEV), 2, 2, nh, nkv, hd, hd ** -0.5, 0, 1,
                                    None, table, hd, torch.tensor([39, 16], dtype=torch.int32, device=DEV), None, None,
                                    0.0, True, status)
    native.check_error_flags()
    assert int(status.item()) == 1
    pg0 = int(bt[0, 2])
    changed = (kpd != kp0).flatten(1).any(1).nonzero().flatten().tolist()
    assert changed == [pg0]


@pytest.mark.parametrize("splits", [2, 3, 7])
def test_flash_decode_splits_agree(native, splits):
    nh, nkv, hd, page = 8, 2, 64, 16
    q_lens, ctx_lens = [1, 1, 2, 1], [1000, 65, 513, 3]
    q, kp, vp, bt, dense = _paged_case(q_lens, ctx_lens, nh, nkv, hd, page, torch.bfloat16, seed=5)
    want = _ref_attention(q, dense, q_lens, ctx_lens, nh, nkv, hd ** -0.5, 0)
    got = _run_attention(native, "flash", q, kp, vp, bt, q_lens, ctx_lens, nh, nkv, hd, hd ** -0.5, 0,
                         force_splits=splits)
    assert (got - want).abs().max().item() <= 2e-2


@pytest.mark.parametrize("kind,dtype", [("generic", torch.float32), ("flash", torch.bfloat16)])
@pytest.mark.parametrize("far", [0, 17, 255, 256, 600])
def test_one_far_key_decides(native, kind, dtype, far):
    """One key among hundreds gets a score that stands out: the output must be its value.
    A kernel that skips, repeats or misplaces a key (a page's edge, a tile's edge, a split's
    edge) returns an average of values instead."""
    nh, nkv, hd, page = 4, 2, 32, 16
    q_lens, ctx_lens = [1, 3], [800, 801]
    q, kp, vp, bt, dense = _paged_case(q_lens, ctx_lens, nh, nkv, hd, page, dtype, seed=far)
    # put a key equal to 6*q/|q| at position `far` of request 0, kv head 0, for query head 1
    qv = q[0, 1].float()
    key = (qv / qv.norm() * 6.0).to(dtype)
    k0, v0 = dense[0]
    k0[far, 0] = key
    pg = int(bt[0, far // page])
    kp[pg, 0, far % page] = key
    scale = 4.0          # score = 4 * 6 * |q| ~ 24 * 5.6: every other key is e^-100 away
    got = _run_attention(native, kind, q, kp, vp, bt, q_lens, ctx_lens, nh, nkv, hd, scale, 0)
    torch.testing.assert_close(got[0, 1], v0[far, 0].float(), rtol=2e-2, atol=2e-2)
    want = _ref_attention(q, dense, q_lens, ctx_lens, nh, nkv, scale, 0)
    assert (got - want).abs().max().item() <= (3e-2 if dtype == torch.bfloat16 else 1e-4)


def test_window_edge(native):
    """The key exactly `window` back is out, the one after it is in."""
    nh, nkv, hd, page, window = 2, 1, 32, 8, 40
    q_lens, ctx_lens = [1], [200]
    for kind, dtype in (("generic", torch.float32), ("flash", torch.bfloat16)):
        q, kp, vp, bt, dense = _paged_case(q_lens, ctx_lens, nh, nkv, hd, page, dtype, seed=3)
        qv = q[0, 0].float()
        key = (qv / qv.norm() * 6.0).to(dtype)
        pos = 199
        for j, inside in ((pos - window, False), (pos - window + 1, True)):
            k0 = dense[0][0].clone()
            kp2 = kp.clone()
            k0[j, 0] = key
            kp2[int(bt[0, j // page]), 0, j % page] = key
            got = _run_attention(native, kind, q, kp2, vp, bt, q_lens, ctx_lens, nh, nkv, hd, 4.0, window)
            hit = torch.allclose(got[0, 0], dense[0][1][j, 0].float(), rtol=3e-2, atol=3e-2)
            assert hit == inside, f"{kind}: key at distance {pos - j} inside={inside}"


def test_freed_pages_are_not_read(native):
    """Pages that a window has passed are marked -1 in the block table; the kernels must not
    follow them."""
    nh, nkv, hd, page, window = 4, 2, 64, 16, 32
    q_lens, ctx_lens = [1, 20], [300, 150]
    for kind, dtype in (("generic", torch.float32), ("flash", torch.bfloat16)):
        q, kp, vp, bt, dense = _paged_case(q_lens, ctx_lens, nh, nkv, hd, page, dtype, seed=8)
        bt2 = bt.clone()
        bt2[0, : (300 - 1 - window + 1) // page] = -1
        bt2[1, : (150 - 20 - window + 1) // page] = -1
        want = _ref_attention(q, dense, q_lens, ctx_lens, nh, nkv, hd ** -0.5, window)
        got = _run_attention(native, kind, q, kp, vp, bt2, q_lens, ctx_lens, nh, nkv, hd, hd ** -0.5, window)
        assert (got - want).abs().max().item() <= (2e-2 if dtype == torch.bfloat16 else 2e-5)


def test_flash_refuses_other_head_sizes(native):
    assert not native.flash_supports(40, torch.bfloat16)
    assert not native.flash_supports(272, torch.bfloat16)
    assert not native.flash_supports(64, torch.float32)


# ----------------------------------------------------------------------------- sampling


def test_sampler_greedy_and_distribution():
    from atom_b200.sampling.params import SamplingParams
    from atom_b200.sampling.sampler import Sampler

    V = 389
    logits = _rand((6, V), torch.float32, 21, 2.0)
    logits[2, 7] = logits[2, 300] = 50.0           # a tie: the lowest index wins
    sm = Sampler(DEV)
    ids = sm.sample(logits, [SamplingParams(temperature=0.0)] * 6, [0] * 6, [0] * 6).tolist()
    assert ids == logits.argmax(-1).tolist() and ids[2] == 7
    # the empirical distribution of temperature sampling follows softmax(logits / T)
    V2, n = 11, 4000
    row = torch.tensor([[2.0, 1.0, 0.5, 0.0, -1.0, 1.5, -3.0, 0.2, 0.1, -0.5, 0.7]], device=DEV)
    rows = row.repeat(n, 1).contiguous()
    T = 0.8
    ids = sm.sample(rows, [SamplingParams(temperature=T)] * n, [1234] * n, list(range(n))).cpu().numpy()
    p = torch.softmax(row[0] / T, -1).cpu().numpy()
    counts = np.bincount(ids, minlength=V2)
    chi2 = float(((counts - n * p) ** 2 / (n * p)).sum())
    assert chi2 < 40.0, f"chi-square {chi2:.1f} over 10 degrees of freedom"
    # the draw depends on (seed, index) only, not on the row's place in the batch
    a = sm.sample(rows[:5], [SamplingParams(temperature=T)] * 5, [9] * 5, [0, 1, 2, 3, 4]).tolist()
    b = sm.sample(rows[:5], [SamplingParams(temperature=T)] * 5, [9] * 5, [4, 3, 2, 1, 0]).tolist()
    assert a == b[::-1]


# ----------------------------------------------------------------------------- few-row matrix product (rows of W shared out)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(1, 389, 64), (3, 130, 320), (8, 4096, 4096), (9, 1000, 576), (16, 77, 1024),
                                   (7, 301, 192), (4, 200, 448), (13, 9600, 2112), (2, 2500, 512), (5, 151, 12288),
                                   (8, 10007, 128), (6, 151936, 64)])
def test_gemm_rows(native, out_dtype, M, N, K):
    """Fewer rows of W than CTAs, one sub-slab, several sub-slabs of a height that is no multiple of 16,
    a last sub-slab that is shorter, k of one chunk and of many stages; both token tiles."""
    a, w = _rand((M, K), torch.bfloat16, 30), _rand((N, K), torch.bfloat16, 31)
    bias = _rand((N,), torch.bfloat16 if N % 4 == 1 else torch.float32, 32) if N % 2 else None
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    assert native.gemm_rows_supports(M, N, K, K)
    native.gemm_rows(a, w, out, bias)
    native.check_error_flags()
    want = a.float() @ w.float().T + (bias.float() if bias is not None else 0)
    torch.testing.assert_close(out.float(), want.to(out_dtype).float(), rtol=1e-2, atol=1e-2 * math.sqrt(K / 96))


@pytest.mark.parametrize("M,I,K", [(1, 160, 128), (7, 1001, 320), (8, 12288, 4096), (12, 112, 64), (16, 333, 1024),
                                   (3, 5000, 192)])
def test_gemm_rows_gated(native, M, I, K):
    a, w = _rand((M, K), torch.bfloat16, 33), _rand((2 * I, K), torch.bfloat16, 34, 0.3)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    native.gemm_rows(a, w, out, gated=True)
    native.check_error_flags()
    gu = a.double() @ w.double().T
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    torch.testing.assert_close(out.double(), want, rtol=2e-2, atol=2e-2 * math.sqrt(K / 96))


def test_gemm_rows_strided_input_and_output(native):
    """X and the output may be column ranges of wider arrays (the leading dimensions are passed on)."""
    M, N, K = 5, 700, 256
    big_a = _rand((M, K + 64), torch.bfloat16, 50)
    w = _rand((N, K), torch.bfloat16, 51)
    big_out = torch.full((M, N + 24), float("nan"), dtype=torch.float32, device=DEV)
    native.gemm_rows(big_a[:, 64:], w, big_out[:, 8:8 + N])
    native.check_error_flags()
    torch.testing.assert_close(big_out[:, 8:8 + N], big_a[:, 64:].float() @ w.float().T, rtol=2e-3, atol=5e-3)
    assert torch.isnan(big_out[:, :8]).all() and torch.isnan(big_out[:, 8 + N:]).all()


def test_gemm_rows_do_not_depend_on_the_batch(native):
    """A row's result does not depend on the rows beside it: bit-equal whatever the number of rows."""
    N, K = 520, 1088
    a, w = _rand((16, K), torch.bfloat16, 35), _rand((N, K), torch.bfloat16, 36)
    outs = {}
    for m in (1, 5, 8, 9, 16):
        outs[m] = torch.empty((m, N), dtype=torch.float32, device=DEV)
        native.gemm_rows(a[:m], w, outs[m])
    native.check_error_flags()
    for m in (1, 5, 8, 9):
        assert torch.equal(outs[m], outs[16][:m])
    torch.testing.assert_close(outs[16], a.float() @ w.float().T, rtol=2e-3, atol=5e-3)


# ----------------------------------------------------------------------------- many-row product on pairs of CTAs (tcgen05)


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (1, 8, 8), (300, 544, 448), (129, 1000, 200), (2048, 4096, 4096),
                                   (777, 5000, 72), (4100, 520, 1024), (5000, 20000, 64)])
def test_gemm_pairs(native, M, N, K):
    """One tile and less than one, rows and columns that end inside a tile, a k that ends inside a block of 64,
    more tiles than the device holds pairs of CTAs (several rounds, the last in halves)."""
    a, w = _rand((M, K), torch.bfloat16, 60), _rand((N, K), torch.bfloat16, 61)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert native.gemm_pairs_supports(M, N, K, K, N)
    native.gemm_pairs(a, w, out)
    native.check_error_flags()
    want = a.float() @ w.float().T
    torch.testing.assert_close(out.float(), want.bfloat16().float(), rtol=1e-2, atol=1e-2 * math.sqrt(K / 96))


@pytest.mark.parametrize("M,I,K", [(256, 256, 128), (5, 112, 64), (1030, 1001 * 8, 320), (2048, 12288, 4096),
                                   (333, 160, 192), (3000, 9728, 2560)])
def test_gemm_pairs_gated(native, M, I, K):
    """The activation in the epilogue: gate and up sums of an output lie in the same half of a tile."""
    a, w = _rand((M, K), torch.bfloat16, 62), _rand((2 * I, K), torch.bfloat16, 63, 0.3)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    native.gemm_pairs(a, w, out, gated=True)
    native.check_error_flags()
    gu = a.double() @ w.double().T
    want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    torch.testing.assert_close(out.double(), want, rtol=2e-2, atol=2e-2 * math.sqrt(K / 96))


def test_gemm_pairs_strided_and_batch_independent(native):
    """X and the output may be column ranges of wider arrays, nothing beside the output is written, and a
    row's result does not depend on the rows beside it."""
    M, N, K = 700, 392, 256
    big_a = _rand((M, K + 64), torch.bfloat16, 64)
    w = _rand((N, K), torch.bfloat16, 65)
    big_out = torch.full((M, N + 24), float("nan"), dtype=torch.bfloat16, device=DEV)
    native.gemm_pairs(big_a[:, 64:], w, big_out[:, 8:8 + N])
    native.check_error_flags()
    want = (big_a[:, 64:].float() @ w.float().T).bfloat16().float()
    torch.testing.assert_close(big_out[:, 8:8 + N].float(), want, rtol=1e-2, atol=2e-2)
    assert torch.isnan(big_out[:, :8]).all() and torch.isnan(big_out[:, 8 + N:]).all()
    part = torch.empty((130, N), dtype=torch.bfloat16, device=DEV)
    native.gemm_pairs(big_a[300:430, 64:], w, part)
    native.check_error_flags()
    assert torch.equal(part, big_out[300:430, 8:8 + N])


def test_gemm_pairs_refuses_what_it_cannot_take(native):
    assert not native.gemm_pairs_supports(64, 100, 64, 64, 100)      # columns: a multiple of 8
    assert not native.gemm_pairs_supports(64, 96, 60, 60, 96)        # k: a multiple of 8
    assert not native.gemm_pairs_supports(64, 96, 64, 68, 96)        # rows of x 16 bytes apart
    a, w = _rand((64, 60), torch.bfloat16, 66), _rand((96, 60), torch.bfloat16, 67)
    with pytest.raises(RuntimeError):
        native.gemm_pairs(a, w, torch.empty((64, 96), dtype=torch.bfloat16, device=DEV))


@pytest.mark.parametrize("M,H,I,wdtype", [(8, 4096, 12288, torch.bfloat16), (3, 320, 960, torch.float32),
                                          (1, 64, 192, torch.float32), (11, 1088, 2112, torch.bfloat16)])
def test_gemm_rows_norm_without_a_pass_of_its_own(native, M, H, I, wdtype):
    """A product in residual mode followed by a product that multiplies its rows by rstd is the residual
    add, the RMSNorm and the product of the plain formulas:  r += a Wo^T;  y = RMSNorm(r; w) W2^T.
    Checked against float64 for a plain second product with a bias and for a gated one; the residual
    stream itself must be the exact 32-bit sum of the old residual and the product."""
    eps = 1e-5
    G = native.gemm_rows_grid()
    a = _rand((M, I), torch.bfloat16, 60)
    wo = _rand((H, I), torch.bfloat16, 61, I ** -0.5)
    res0 = _rand((M, H), torch.float32, 62)
    nw = (_rand((H,), torch.float32, 63) * 0.2 + 1).to(wdtype)
    w2 = _rand((2 * I, H), torch.bfloat16, 64, H ** -0.5)
    bias = _rand((2 * I,), torch.float32, 65)
    res = res0.clone()
    xw = torch.full((M, H), float("nan"), dtype=torch.bfloat16, device=DEV)
    ssq = torch.full((G, 16), float("nan"), dtype=torch.float32, device=DEV)
    native.gemm_rows(a, wo, residual=res, norm_w=nw, xout=xw, ssq_out=ssq)
    plain = torch.full((M, 2 * I), float("nan"), dtype=torch.float32, device=DEV)
    gated = torch.full((M, I), float("nan"), dtype=torch.float32, device=DEV)
    native.gemm_rows(xw, w2, plain, bias, ssq_in=ssq, norm_size=H, norm_eps=eps)
    native.gemm_rows(xw, w2, gated, gated=True, ssq_in=ssq, norm_size=H, norm_eps=eps)
    native.check_error_flags()
    r = res0.double() + a.double() @ wo.double().T
    torch.testing.assert_close(res.double(), r, rtol=1e-5, atol=2e-5 * math.sqrt(I / 96))
    torch.testing.assert_close(ssq[:, :M].double().sum(0), res.double().pow(2).sum(-1), rtol=1e-5, atol=1e-5)
    assert (ssq[:, M:] == 0).all()
    y = r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + eps) * nw.double()
    full = y @ w2.double().T
    torch.testing.assert_close(plain.double(), full + bias.double(), rtol=1e-2, atol=1.5e-2 * math.sqrt(H / 96))
    torch.testing.assert_close(gated.double(), torch.nn.functional.silu(full[:, :I]) * full[:, I:],
                               rtol=2e-2, atol=2e-2 * math.sqrt(H / 96))


def test_gemm_rows_refuses_other_sizes(native):
    assert not native.gemm_rows_supports(17, 64, 64, 64)
    assert not native.gemm_rows_supports(4, 64, 96, 96)      # K no multiple of 64
    assert not native.gemm_rows_supports(4, 64, 64, 100)     # leading dimension no multiple of 8
    assert not native.gemm_rows_supports(4, 64, 32, 32)


# ----------------------------------------------------------------------------- both sides of every launch choice


@pytest.mark.parametrize("name,value", [("pdl", 0), ("decode_tma", 0), ("decode_ktw", 16), ("decode_ktw", 32)])
def test_forced_launch_choices_give_the_same_results(native, name, value):
    """The launch code chooses between kernels and tilings by itself (dependent launch, the TMA decode kernel
    and its warp tile); ``set_option`` forces a
    side.  Each forced side is checked against the dense references, so no path runs only at sizes the
    default happens to send there."""
    try:
        native.set_option(name, value)
        # decode attention: 16 packed rows, several splits, a request shorter than a page
        nh, nkv, hd, page = 16, 4, 128, 16
        q_lens, ctx_lens = [1, 2, 1, 1], [1000, 130, 7, 2049]
        q, kp, vp, bt, dense = _paged_case(q_lens, ctx_lens, nh, nkv, hd, page, torch.bfloat16, seed=91)
        want = _ref_attention(q, dense, q_lens, ctx_lens, nh, nkv, hd ** -0.5, 0)
        got = _run_attention(native, "flash", q, kp, vp, bt, q_lens, ctx_lens, nh, nkv, hd, hd ** -0.5, 0,
                             force_splits=3)
        assert (got - want).abs().max().item() <= 2e-2
        # the streaming product under the same launch mode: plain with bias, and gated
        for M, N, K, gated in ((8, 4096, 12288, False), (3, 1000, 576, False), (5, 2048, 1024, True)):
            a = _rand((M, K), torch.bfloat16, 92)
            w = _rand(((2 if gated else 1) * N, K), torch.bfloat16, 93, 0.3)
            bias = None if gated else _rand((N,), torch.bfloat16, 94)
            out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
            native.gemm_rows(a, w, out, bias, gated=gated)
            acc = a.double() @ w.double().T
            ref = torch.nn.functional.silu(acc[:, :N]) * acc[:, N:] if gated else acc + bias.double()
            torch.testing.assert_close(out.double(), ref, rtol=1e-2, atol=2e-2 * math.sqrt(K / 96))
        # a small kernel chain under the same launch mode: norm, then rows gathered
        x = _rand((5, 320), torch.bfloat16, 95)
        res = _rand((5, 320), torch.float32, 96)
        wn = (_rand((320,), torch.float32, 97) * 0.1 + 1).to(torch.bfloat16)
        out = torch.empty((5, 320), dtype=torch.bfloat16, device=DEV)
        r0 = res.clone()
        native.add_rmsnorm(out, res, x, wn, 1e-6, None, 5)
        rr = r0.double() + x.double()
        ref = rr * torch.rsqrt(rr.pow(2).mean(-1, keepdim=True) + 1e-6) * wn.double()
        torch.testing.assert_close(out.double(), ref, rtol=2e-2, atol=2e-2)
        native.check_error_flags()
    finally:
        native.reset_options()
