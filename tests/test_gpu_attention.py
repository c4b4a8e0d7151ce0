"""tcgen05 flash attention (forward and backward) against the fp32 PyTorch restatement."""
import math

import pytest
import torch

from picotron_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C():
    from picotron_b200.ops import _ext
    return _ext.load()


def rnd(*shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


CASES = [
    # B, Sq, Sk, hq, hkv, d, causal
    (2, 256, 256, 4, 2, 64, True),
    (1, 128, 128, 2, 2, 64, True),
    (2, 300, 300, 4, 4, 64, True),      # ragged tail
    (1, 1024, 1024, 4, 1, 64, True),
    (1, 16, 16, 2, 1, 64, True),        # tiny (the multi-GPU tests use such sizes)
    (2, 256, 256, 2, 1, 128, True),
    (1, 200, 200, 2, 2, 128, True),
    (1, 128, 384, 4, 2, 64, False),     # full attention, Sq != Sk (ring blocks from earlier ranks)
    (1, 200, 136, 2, 2, 128, False),
]


@pytest.mark.parametrize("B,Sq,Sk,hq,hkv,d,causal", CASES)
def test_attention_forward(C, B, Sq, Sk, hq, hkv, d, causal):
    q, k, v = rnd(B, Sq, hq, d, seed=1), rnd(B, Sk, hkv, d, seed=2), rnd(B, Sk, hkv, d, seed=3)
    scale = 1.0 / math.sqrt(d)
    o, lse = C.attention_fwd(q, k, v, causal, scale)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    o_ref, lse_ref = ref.attention_fwd(q, k, v, causal, scale)
    torch.testing.assert_close(lse, lse_ref, rtol=1e-3, atol=2e-3)
    torch.testing.assert_close(o.float(), o_ref.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("B,Sq,Sk,hq,hkv,d,causal", CASES)
def test_attention_backward(C, B, Sq, Sk, hq, hkv, d, causal):
    q, k, v = rnd(B, Sq, hq, d, seed=1), rnd(B, Sk, hkv, d, seed=2), rnd(B, Sk, hkv, d, seed=3)
    do = rnd(B, Sq, hq, d, seed=4)
    scale = 1.0 / math.sqrt(d)
    o_ref, lse_ref = ref.attention_fwd(q, k, v, causal, scale)
    dq_r, dk_r, dv_r = ref.attention_bwd(do, q, k, v, o_ref, lse_ref, causal, scale)
    dq, dk, dv = C.attention_bwd(do, q, k, v, o_ref, lse_ref, causal, scale)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    for name, got, want in (("dq", dq, dq_r), ("dk", dk, dk_r), ("dv", dv, dv_r)):
        err = float((got.float() - want).norm() / (want.norm() + 1e-12))
        assert err < 2e-2, f"{name}: relative error {err:.4f}"
        torch.testing.assert_close(got.float(), want, rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("B,S,hq,hkv,d", [(2, 256, 4, 2, 64), (1, 300, 4, 4, 64), (2, 256, 2, 1, 128), (3, 128, 2, 2, 64)])
def test_attention_backward_with_inverse_rope_on_dq_dk(C, B, S, hq, hkv, d):
    """dq / dk un-rotated inside the backward (dq in the fp32->bf16 conversion, dk in the epilogue) vs the RoPE kernel."""
    q, k, v = rnd(B, S, hq, d, seed=1), rnd(B, S, hkv, d, seed=2), rnd(B, S, hkv, d, seed=3)
    do = rnd(B, S, hq, d, seed=4)
    scale = 1.0 / math.sqrt(d)
    o_ref, lse_ref = ref.attention_fwd(q, k, v, True, scale)
    dq_r, dk_r, dv_r = ref.attention_bwd(do, q, k, v, o_ref, lse_ref, True, scale)
    cos, sin = ref.rope_tables(S + 40, d, 10000.0, device="cuda")        # a table longer than the sequence
    want_q = ref.rope_(dq_r.reshape(B * S, hq * d).clone(), cos, sin, hq, d, S, True).view(B, S, hq, d)
    want_k = ref.rope_(dk_r.reshape(B * S, hkv * d).clone(), cos, sin, hkv, d, S, True).view(B, S, hkv, d)
    dq, dk, dv = C.attention_bwd(do, q, k, v, o_ref, lse_ref, True, scale, None, None, cos, sin)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    for name, got, want in (("dq", dq, want_q), ("dk", dk, want_k), ("dv", dv, dv_r)):
        err = float((got.float() - want.float()).norm() / (want.float().norm() + 1e-12))
        assert err < 2e-2, f"{name}: relative error {err:.4f}"


def test_phase_profiling_variant_gives_the_same_results_and_counts_cycles(C):
    B, S, hq, hkv, d = 2, 512, 4, 2, 64
    q, k, v, do = rnd(B, S, hq, d, seed=1), rnd(B, S, hkv, d, seed=2), rnd(B, S, hkv, d, seed=3), rnd(B, S, hq, d, seed=4)
    scale = 1.0 / math.sqrt(d)
    o, lse = C.attention_fwd(q, k, v, True, scale)
    dq, dk, dv = C.attention_bwd(do, q, k, v, o, lse, True, scale)
    counters = torch.zeros(16, dtype=torch.int64, device="cuda")
    C.attention_set_profile(counters)
    try:
        o2, lse2 = C.attention_fwd(q, k, v, True, scale)
        dq2, dk2, dv2 = C.attention_bwd(do, q, k, v, o, lse, True, scale)
        torch.cuda.synchronize()
    finally:
        C.attention_set_profile(None)
    assert C.kernel_status() == 0
    # a separately compiled instantiation: same algorithm, fp32 sums may be associated differently by a few ulp
    torch.testing.assert_close(o2.float(), o.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(lse2, lse, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(dk2.float(), dk.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(dv2.float(), dv.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(dq2.float(), dq.float(), rtol=1e-2, atol=1e-2)
    c = counters.tolist()
    ctas_fwd, ctas_bwd = B * hq * (S // 128), B * hkv * (S // 128)
    assert c[13] == ctas_fwd and c[6] == ctas_bwd
    assert c[11] == B * hq * sum(range(1, S // 128 + 1))                              # causal: 1 + 2 + ... key blocks
    assert min(c[8], c[10], c[1], c[3]) > 0
    before = counters.clone()
    C.attention_fwd(q, k, v, True, scale)                                             # switched off: nothing is added
    torch.cuda.synchronize()
    assert torch.equal(counters, before)


def test_attention_on_packed_qkv_views_with_outs_and_delta(C):
    B, S, hq, hkv, d = 2, 256, 4, 2, 64
    T = B * S
    qkv = rnd(T, (hq + 2 * hkv) * d, seed=5)
    q = qkv[:, : hq * d].view(B, S, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].view(B, S, hkv, d)
    v = qkv[:, (hq + hkv) * d:].view(B, S, hkv, d)
    scale = 1.0 / math.sqrt(d)
    o, lse = C.attention_fwd(q, k, v, True, scale)
    o_ref, lse_ref = ref.attention_fwd(q, k, v, True, scale)
    torch.testing.assert_close(o.float(), o_ref.float(), rtol=2e-2, atol=2e-2)
    do = rnd(B, S, hq, d, seed=6)
    dqkv = torch.zeros_like(qkv)
    dq = dqkv[:, : hq * d].view(B, S, hq, d)
    dk = dqkv[:, hq * d:(hq + hkv) * d].view(B, S, hkv, d)
    dv = dqkv[:, (hq + hkv) * d:].view(B, S, hkv, d)
    delta = (do.float() * o.float()).sum(-1).permute(0, 2, 1).contiguous()
    C.attention_bwd(do, q, k, v, o, lse, True, scale, delta, [dq, dk, dv])
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    dq_r, dk_r, dv_r = ref.attention_bwd(do, q, k, v, o_ref, lse_ref, True, scale)
    for got, want in ((dq, dq_r), (dk, dk_r), (dv, dv_r)):
        assert float((got.float() - want).norm() / want.norm()) < 2e-2
