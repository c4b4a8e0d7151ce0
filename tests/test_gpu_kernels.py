"""sm_100a kernels against the plain-PyTorch fp32 restatements of the same ops."""
import math

import pytest
import torch

from picotron_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["pair", "pair_direct_store", "single"])
def C(request):
    """The extension with GEMMs on CTA pairs (cta_group::2; TMA-store epilogue, then per-thread stores) and on single CTAs."""
    from picotron_b200.ops import _ext
    ext = _ext.load()
    ext.set_gemm_pair(request.param != "single")
    ext.set_gemm_tma_epilogue(request.param == "pair")
    yield ext
    ext.set_gemm_pair(True)
    ext.set_gemm_tma_epilogue(True)


def _status_ok(C):
    torch.cuda.synchronize()
    assert C.kernel_status() == 0


def bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


def _rel(got, want):
    """Relative Frobenius error. bf16 inputs and one bf16 rounding of the output give ~2e-3; a dropped k-block of a small-K
    GEMM, which the element-wise tolerance below lets pass, gives 1/sqrt(number of k-blocks) or more."""
    return float((got.float() - want).norm() / (want.norm() + 1e-20))


GEMM_SHAPES = [(128, 256, 64), (128, 256, 256), (256, 512, 320), (200, 328, 136), (64, 64, 64), (1024, 2048, 512),
               (384, 1536, 2048), (1000, 1096, 1000), (2048, 2560, 1024)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_forward_layout(C, M, N, K):
    x, w = bf(M, K, seed=1), bf(N, K, seed=2)
    y = C.gemm(x, w, False, False)
    _status_ok(C)
    want = x.float() @ w.float().t()
    torch.testing.assert_close(y.float(), want, rtol=2e-2, atol=2e-2 * math.sqrt(K))
    assert _rel(y, want) < 4e-3


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_dgrad_layout(C, M, N, K):
    dy, w = bf(M, K, seed=3), bf(K, N, seed=4)          # D[M,N] = dy[M,K] @ w[K,N]
    y = C.gemm(dy, w, False, True)
    _status_ok(C)
    want = dy.float() @ w.float()
    torch.testing.assert_close(y.float(), want, rtol=2e-2, atol=2e-2 * math.sqrt(K))
    assert _rel(y, want) < 4e-3


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_wgrad_layout_and_fp32_accumulate(C, M, N, K):
    a, b = bf(K, M, seed=5), bf(K, N, seed=6)            # D[M,N] = a^T b
    want = a.float().t() @ b.float()
    y = C.gemm(a, b, True, True)
    _status_ok(C)
    torch.testing.assert_close(y.float(), want, rtol=2e-2, atol=2e-2 * math.sqrt(K))
    assert _rel(y, want) < 4e-3
    acc = torch.full((M, N), 0.5, device="cuda", dtype=torch.float32)
    C.gemm(a, b, True, True, acc, True)
    C.gemm(a, b, True, True, acc, True)
    _status_ok(C)
    torch.testing.assert_close(acc, 0.5 + 2 * want, rtol=1e-3, atol=1e-3 * math.sqrt(K))
    assert _rel(acc - 0.5, 2 * want) < 1e-4                   # fp32 accumulation: only the bf16 inputs round


@pytest.mark.parametrize("T,I,K", [(256, 128, 64), (300, 384, 320), (1024, 2048, 512), (4096, 1024, 2048)])
def test_gemm_with_swiglu_epilogue(T, I, K):
    """gate/up GEMM whose epilogue also writes silu(gate) * up, against the two separate kernels and fp32 math."""
    from picotron_b200.ops import _ext
    C = _ext.load()
    C.set_gemm_pair(True)
    C.set_gemm_tma_epilogue(True)
    x, w = bf(T, K, seed=21), bf(2 * I, K, seed=22, scale=0.5)
    r = C.gemm_swiglu(x, w)
    assert r, "the fused kernel should cover this shape"
    gu, h = r
    _status_ok(C)
    gu_ref = C.gemm(x, w, False, False)
    torch.testing.assert_close(gu.float(), gu_ref.float(), rtol=0, atol=0)            # same accumulators, same rounding
    torch.testing.assert_close(gu.float(), x.float() @ w.float().t(), rtol=2e-2, atol=2e-2 * math.sqrt(K))
    torch.testing.assert_close(h.float(), ref.swiglu_fwd(gu).float(), rtol=2e-2, atol=2e-2)
    assert C.gemm_swiglu(x, bf(2 * 72, K, seed=23)) == []                             # I % 128 != 0: not covered


@pytest.mark.parametrize("T,V,K,vocab_start", [(256, 512, 64, 0), (300, 1000, 192, 0), (2048, 49152, 2048, 0), (512, 4096, 256, 4096),
                                               (32, 48, 256, 0), (200, 1000, 64, 1000)])
def test_lm_head_gemm_with_cross_entropy_statistics_epilogue(T, V, K, vocab_start):
    """Logits GEMM whose epilogue produces row max / sum-exp / target logit, against the separate statistics kernel (which
    reads the same stored logits) and against fp32 math."""
    from picotron_b200.ops import _ext
    C = _ext.load()
    C.set_gemm_pair(True)
    C.set_gemm_tma_epilogue(True)
    x, w = bf(T, K, seed=61), bf(V, K, seed=62, scale=0.3)
    g = torch.Generator(device="cuda").manual_seed(63)
    targets = torch.randint(0, 2 * V if vocab_start else V, (T,), device="cuda", generator=g)   # some outside this shard
    r = C.gemm_ce_stats(x, w, targets, vocab_start)
    assert r, "the fused kernel should cover this shape"
    logits, rowmax, sumexp, tgt = r
    _status_ok(C)
    plain = C.gemm(x, w, False, False)
    torch.testing.assert_close(logits.float(), plain.float(), rtol=0, atol=0)
    m2, s2, t2 = C.ce_stats(plain, targets, vocab_start)
    torch.testing.assert_close(rowmax, m2, rtol=0, atol=0)
    torch.testing.assert_close(sumexp, s2, rtol=2e-3, atol=1e-3)
    torch.testing.assert_close(tgt, t2, rtol=0, atol=0)
    lse_ref = torch.logsumexp(x.float() @ w.float().t(), dim=-1)
    torch.testing.assert_close(rowmax + torch.log(sumexp), lse_ref, rtol=1e-2, atol=3e-2)


@pytest.mark.parametrize("T,N,K", [(256, 256, 64), (300, 328, 320), (1024, 2048, 512), (4096, 2048, 8192), (200, 72, 136)])
def test_gemm_with_residual_add_epilogue(T, N, K):
    """Projection + residual add from one GEMM (the epilogue fetches the residual tile) against GEMM followed by the add."""
    from picotron_b200.ops import _ext
    C = _ext.load()
    C.set_gemm_pair(True)
    C.set_gemm_tma_epilogue(True)
    x, w, res = bf(T, K, seed=41), bf(N, K, seed=42, scale=0.5), bf(T, N, seed=43, scale=4.0)
    got = C.gemm_add(x, w, res)
    assert got is not None, "the fused kernel should cover this shape"
    _status_ok(C)
    want = x.float() @ w.float().t() + res.float()
    torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=2e-2 * math.sqrt(K))
    assert _rel(got, want) < 4e-3
    two_step = C.add(res, C.gemm(x, w, False, False))
    assert _rel(got, want) <= _rel(two_step, want) + 1e-4       # one rounding instead of two


@pytest.mark.parametrize("T,I,H", [(256, 256, 64), (300, 320, 192), (1024, 2048, 512), (4096, 8192, 2048), (512, 5504, 1024)])
def test_dgrad_gemm_with_swiglu_backward_epilogue(T, I, H):
    """Down-projection dgrad whose epilogue applies the SwiGLU backward, against dgrad GEMM + activation-backward kernel
    and against fp32 math."""
    from picotron_b200.ops import _ext
    C = _ext.load()
    C.set_gemm_pair(True)
    C.set_gemm_tma_epilogue(True)
    dy, w, gu = bf(T, H, seed=51), bf(H, I, seed=52, scale=0.5), bf(T, 2 * I, seed=53, scale=1.5)
    got = C.gemm_dgrad_swiglu_bwd(dy, w, gu)
    assert got is not None, "the fused kernel should cover this shape"
    _status_ok(C)
    da = dy.float() @ w.float()
    g, u = gu[:, :I].float(), gu[:, I:].float()
    sig = torch.sigmoid(g)
    want = torch.cat([da * u * sig * (1 + g * (1 - sig)), da * g * sig], dim=1)
    assert _rel(got, want) < 6e-3
    two_step = C.swiglu_bwd(gu, C.gemm(dy, w, False, True))
    assert _rel(got, want) <= _rel(two_step, want) + 1e-4       # da is not rounded to bf16 on the way
    torch.testing.assert_close(got.float(), two_step.float(), rtol=5e-2, atol=5e-2 * math.sqrt(H))
    assert C.gemm_dgrad_swiglu_bwd(dy, bf(H, 72, seed=54), bf(T, 144, seed=55)) is None      # I % 64 != 0: not covered


@pytest.mark.parametrize("B,S,hq,hkv,d,K", [(2, 128, 4, 2, 64, 256), (1, 200, 3, 1, 64, 192), (2, 128, 4, 2, 128, 256),
                                            (4, 1024, 32, 32, 64, 512), (1, 96, 5, 5, 128, 128)])
def test_gemm_with_rope_epilogue(B, S, hq, hkv, d, K):
    """qkv GEMM whose epilogue rotates the q and k heads, against GEMM followed by the RoPE kernel / fp32 restatement."""
    from picotron_b200.ops import _ext
    C = _ext.load()
    C.set_gemm_pair(True)
    C.set_gemm_tma_epilogue(True)
    N = (hq + 2 * hkv) * d
    x, w = bf(B * S, K, seed=31), bf(N, K, seed=32, scale=0.5)
    cos, sin = ref.rope_tables(S, d, 10000.0, device="cuda")
    got = C.gemm_rope(x, w, cos, sin, hq + hkv, d, S)
    assert got is not None
    _status_ok(C)
    plain = C.gemm(x, w, False, False)
    want = ref.rope_((x.float() @ w.float().t()), cos, sin, hq + hkv, d, S)          # fp32 throughout
    torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=2e-2 * math.sqrt(K))
    torch.testing.assert_close(got[:, (hq + hkv) * d:].float(), plain[:, (hq + hkv) * d:].float(), rtol=0, atol=0)   # v untouched
    two_step = plain.clone()
    C.rope_(two_step, cos, sin, hq + hkv, d, S, False)
    torch.testing.assert_close(got.float(), two_step.float(), rtol=2e-2, atol=0.25)   # one rounding instead of two


@pytest.mark.parametrize("group_m", [1, 3, 8, 64])
def test_gemm_tile_numbering_group_sizes(group_m):
    """Every group size of the tile numbering visits each output tile exactly once (ragged shapes included)."""
    from picotron_b200.ops import _ext
    C = _ext.load()
    C.set_gemm_pair(True)
    keep = C.get_gemm_group_m()
    C.set_gemm_group_m(group_m)
    try:
        for M, N, K in [(2816, 1280, 192), (1000, 1096, 320), (256, 4096, 128)]:
            x, w = bf(M, K, seed=41), bf(N, K, seed=42)
            y = C.gemm(x, w, False, False)
            _status_ok(C)
            torch.testing.assert_close(y.float(), x.float() @ w.float().t(), rtol=2e-2, atol=2e-2 * math.sqrt(K))
    finally:
        C.set_gemm_group_m(keep)


def test_gemm_strided_rows_and_out_slice(C):
    big = bf(512, 1024, seed=7)
    x = big[:, 256:512]                                    # row stride 1024, 256 columns
    w = bf(384, 256, seed=8)
    out = torch.zeros(600, 384, device="cuda", dtype=torch.bfloat16)
    C.gemm(x, w, False, False, out[40:552], False)
    _status_ok(C)
    torch.testing.assert_close(out[40:552].float(), x.float() @ w.float().t(), rtol=2e-2, atol=0.4)
    assert float(out[:40].abs().sum()) == 0 and float(out[552:].abs().sum()) == 0


@pytest.mark.parametrize("T,H", [(7, 64), (300, 2048), (129, 4096)])
def test_rmsnorm_fwd_bwd(C, T, H):
    x, d, w = bf(T, H, seed=1), bf(T, H, seed=2), (1 + 0.1 * bf(H, seed=3).float()).to(torch.bfloat16)
    y, rstd = C.rmsnorm_fwd(x, w, 1e-5)
    y_ref, rstd_ref = ref.rmsnorm_fwd(x, w, 1e-5)
    torch.testing.assert_close(y.float(), y_ref.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(rstd, rstd_ref, rtol=1e-4, atol=1e-5)
    xn, y2, rstd2 = C.add_rmsnorm_fwd(x, d, w, 1e-5)
    xn_ref, y2_ref, rstd2_ref = ref.add_rmsnorm_fwd(x, d, w, 1e-5)
    torch.testing.assert_close(xn.float(), xn_ref.float(), rtol=0, atol=0)
    torch.testing.assert_close(y2.float(), y2_ref.float(), rtol=1e-2, atol=2e-2)
    dy, dres = bf(T, H, seed=4), bf(T, H, seed=5)
    dx, dw = C.rmsnorm_bwd(dy, x, w, rstd, dres)
    dx_ref, dw_ref = ref.rmsnorm_bwd(dy, x, w, rstd_ref, dres)
    torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=2e-2, atol=3e-2)
    torch.testing.assert_close(dw, dw_ref, rtol=1e-3, atol=1e-2 * math.sqrt(T))
    dx0, _ = C.rmsnorm_bwd(dy, x, w, rstd, None)
    torch.testing.assert_close(dx0.float(), ref.rmsnorm_bwd(dy, x, w, rstd_ref)[0].float(), rtol=2e-2, atol=3e-2)


@pytest.mark.parametrize("T,H", [(513, 2048), (64, 768), (33, 256), (40, 4096), (9, 320)])
def test_rmsnorm_bwd_accumulates_into_fp32_destination(C, T, H):
    """dw added in place to an fp32 vector (a gradient-bucket slice), also when that slice is not 16-byte aligned."""
    x, dy, dres = bf(T, H, seed=1), bf(T, H, seed=2), bf(T, H, seed=3)
    w = (1 + 0.1 * bf(H, seed=4).float()).to(torch.bfloat16)
    _, rstd = C.rmsnorm_fwd(x, w, 1e-5)
    dx_ref, dw_ref = ref.rmsnorm_bwd(dy, x, w, rstd, dres)
    store = torch.full((H + 4,), 0.5, device="cuda", dtype=torch.float32)
    for off in (0, 1):
        acc = store[off:off + H]
        acc.fill_(0.5)
        dx, out = C.rmsnorm_bwd(dy, x, w, rstd, dres, acc)
        dx, out = C.rmsnorm_bwd(dy, x, w, rstd, dres, acc)
        _status_ok(C)
        assert out.data_ptr() == acc.data_ptr()
        torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=2e-2, atol=3e-2)
        torch.testing.assert_close(acc, 0.5 + 2 * dw_ref, rtol=1e-3, atol=2e-2 * math.sqrt(T))


@pytest.mark.parametrize("d,hq,hkv", [(64, 4, 2), (128, 2, 2), (64, 32, 8), (128, 16, 5), (32, 4, 4)])
def test_rope_inplace_and_inverse(C, d, hq, hkv):
    B, S = 2, 48
    qkv = bf(B * S, (hq + 2 * hkv) * d, seed=1)
    cos, sin = ref.rope_tables(S, d, 10000.0, device="cuda")
    want = ref.rope_(qkv.clone(), cos, sin, hq + hkv, d, S)
    got = qkv.clone()
    C.rope_(got, cos, sin, hq + hkv, d, S, False)
    torch.testing.assert_close(got.float(), want.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(got[:, (hq + hkv) * d:], qkv[:, (hq + hkv) * d:], rtol=0, atol=0)   # v untouched
    C.rope_(got, cos, sin, hq + hkv, d, S, True)
    torch.testing.assert_close(got.float(), qkv.float(), rtol=2e-2, atol=3e-2)


def test_swiglu(C):
    gu, da = bf(100, 2 * 512, seed=1), bf(100, 512, seed=2)
    torch.testing.assert_close(C.swiglu_fwd(gu).float(), ref.swiglu_fwd(gu).float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(C.swiglu_bwd(gu, da).float(), ref.swiglu_bwd(gu, da).float(), rtol=2e-2, atol=2e-2)


def test_embedding_fwd_bwd_with_vocab_shard(C):
    V, H, T = 300, 128, 500
    w = bf(V, H, seed=1)
    ids = torch.randint(0, 2 * V, (T,), device="cuda")
    out = C.embedding_fwd(ids, w, 100)
    torch.testing.assert_close(out.float(), ref.embedding_fwd(ids, w, 100).float(), rtol=0, atol=0)
    dy = bf(T, H, seed=2)
    dw = torch.zeros(V, H, device="cuda")
    C.embedding_bwd(ids, dy, dw, 100)
    want = torch.zeros(V, H, device="cuda")
    ref.embedding_bwd(ids, dy, want, 100)
    torch.testing.assert_close(dw, want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("V,start", [(1000, 0), (4096, 4096), (50257, 0)])
def test_cross_entropy_stats_and_grad(C, V, start):
    T = 64
    logits = bf(T, V, scale=3.0, seed=1)
    tgt = torch.randint(0, max(V, start + V), (T,), device="cuda")
    rm, se, tl = C.ce_stats(logits, tgt, start)
    rm_r, se_r, tl_r = ref.ce_stats(logits, tgt, start)
    torch.testing.assert_close(rm, rm_r, rtol=0, atol=0)
    torch.testing.assert_close(se, se_r, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(tl, tl_r, rtol=0, atol=0)
    lse = rm_r + torch.log(se_r)
    want = ref.ce_grad_(logits.clone(), tgt, lse, 0.25, start)
    got = logits.clone()
    C.ce_grad_(got, tgt, lse, 0.25, start)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=1e-4)


def test_accumulate_add_merge(C):
    acc = torch.randn(1000 * 8 + 3, device="cuda")
    g = bf(1000 * 8 + 3, seed=1)
    want = acc + g.float()
    C.accumulate_(acc, g)
    torch.testing.assert_close(acc, want)
    a, b = bf(33, 200, seed=2), bf(33, 200, seed=3)
    torch.testing.assert_close(C.add(a, b).float(), (a.float() + b.float()).to(torch.bfloat16).float())
    B, S, h, d = 2, 20, 3, 64
    out, lse = torch.randn(B, S, h, d, device="cuda"), torch.randn(B, h, S, device="cuda")
    bo, bl = bf(B, S, h, d, seed=4), torch.randn(B, h, S, device="cuda")
    o_ref, l_ref = ref.merge_attention_(out.clone(), lse.clone(), bo, bl)
    C.merge_attention_(out, lse, bo, bl)
    torch.testing.assert_close(out, o_ref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(lse, l_ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("master", [True, False])
def test_adamw_multi_tensor(C, master):
    torch.manual_seed(0)
    shapes = [(300, 64), (17,), (70000,), (128, 256)] * 8
    params = [torch.randn(*s, device="cuda").to(torch.bfloat16) for s in shapes]
    grads = [torch.randn(*s, device="cuda") for s in shapes]
    ms = [torch.zeros(*s, device="cuda") for s in shapes]
    vs = [torch.zeros(*s, device="cuda") for s in shapes]
    masters = [p.float().clone() if master else None for p in params]
    rp, rm, rv = [p.clone() for p in params], [m.clone() for m in ms], [v.clone() for v in vs]
    rmw = [m.clone() if m is not None else None for m in masters]
    for step in (1, 2):
        C.adamw_multi_(params, grads, ms, vs, masters, step, 1e-2, 0.9, 0.999, 1e-8, 0.01)
        ref.adamw_step_(rp, grads, rm, rv, rmw, step, 1e-2, 0.9, 0.999, 1e-8, 0.01)
    for a, b in zip(params, rp):
        torch.testing.assert_close(a.float(), b.float(), rtol=1e-2, atol=1e-2)
    for a, b in zip(ms, rm):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-6)
    if master:
        for a, b in zip(masters, rmw):
            torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)
