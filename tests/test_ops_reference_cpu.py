"""The fp32 restatements in ``ops/reference.py`` are the oracle of every GPU kernel test and the CPU execution path.
Here they are themselves checked, against PyTorch's autograd and built-ins, on random shapes (native GQA included)."""
import pytest
import torch
import torch.nn.functional as F

from picotron_b200.ops import reference as R

torch.manual_seed(0)


def _close(a, b, tol=2e-5):
    torch.testing.assert_close(a.double(), b.double(), rtol=tol, atol=tol)


@pytest.mark.parametrize("T,H", [(7, 16), (33, 96)])
def test_rmsnorm_forward_and_backward_match_autograd(T, H):
    x = torch.randn(T, H, requires_grad=True)
    w = torch.randn(H, requires_grad=True)
    res = torch.randn(T, H)
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w
    dy = torch.randn(T, H)
    y.backward(dy)
    got_y, rstd = R.rmsnorm_fwd(x.detach(), w.detach(), 1e-5)
    dx, dw = R.rmsnorm_bwd(dy, x.detach(), w.detach(), rstd, dres=res)
    _close(got_y, y.detach())
    _close(dx, x.grad + res)
    _close(dw, w.grad)
    x_new, y2, _ = R.add_rmsnorm_fwd(x.detach(), res, w.detach(), 1e-5)
    _close(x_new, x.detach() + res)
    _close(y2, R.rmsnorm_fwd(x.detach() + res, w.detach(), 1e-5)[0])


@pytest.mark.parametrize("B,Sq,Sk,hq,hkv,d,causal", [(2, 8, 8, 4, 2, 16, True), (1, 12, 12, 6, 6, 8, True),
                                                     (2, 5, 9, 4, 1, 8, False)])
def test_attention_forward_and_backward_match_sdpa_with_expanded_kv_heads(B, Sq, Sk, hq, hkv, d, causal):
    q = torch.randn(B, Sq, hq, d, requires_grad=True)
    k = torch.randn(B, Sk, hkv, d, requires_grad=True)
    v = torch.randn(B, Sk, hkv, d, requires_grad=True)
    scale = d ** -0.5
    ke, ve = k.repeat_interleave(hq // hkv, dim=2), v.repeat_interleave(hq // hkv, dim=2)
    want = F.scaled_dot_product_attention(q.transpose(1, 2), ke.transpose(1, 2), ve.transpose(1, 2), is_causal=causal,
                                          scale=scale).transpose(1, 2)
    do = torch.randn_like(want)
    want.backward(do)
    o, lse = R.attention_fwd(q.detach(), k.detach(), v.detach(), causal, scale)
    _close(o, want.detach())
    dq, dk, dv = R.attention_bwd(do, q.detach(), k.detach(), v.detach(), o, lse, causal, scale)
    _close(dq, q.grad, 1e-4)
    _close(dk, k.grad, 1e-4)                                  # summed over the query heads of each KV group
    _close(dv, v.grad, 1e-4)
    # log-sum-exp is the one of the scaled, masked scores
    s = torch.einsum("bqhd,bkhd->bhqk", q.detach(), ke.detach()) * scale
    if causal:
        s = s.masked_fill(torch.ones(Sq, Sk, dtype=torch.bool).triu(1), float("-inf"))
    _close(lse, torch.logsumexp(s, -1))


def test_merging_attention_over_two_key_blocks_equals_attention_over_their_union():
    B, S, hq, hkv, d = 2, 6, 4, 2, 8
    q, k, v = torch.randn(B, S, hq, d), torch.randn(B, 10, hkv, d), torch.randn(B, 10, hkv, d)
    scale = d ** -0.5
    full, full_lse = R.attention_fwd(q, k, v, False, scale)
    o1, l1 = R.attention_fwd(q, k[:, :4], v[:, :4], False, scale)
    o2, l2 = R.attention_fwd(q, k[:, 4:], v[:, 4:], False, scale)
    out, lse = o1.float().clone(), l1.clone()
    R.merge_attention_(out, lse, o2, l2)
    _close(out, full)
    _close(lse, full_lse)


def test_rope_is_the_half_split_rotation_and_its_inverse_undoes_it():
    B, S, heads, d = 2, 8, 3, 16
    cos, sin = R.rope_tables(S, d, 10000.0)
    x = torch.randn(B * S, heads * d)
    rotated = R.rope_(x.clone(), cos, sin, 2, d, S)                       # the first two heads rotate, the third stays
    xh = x.view(B, S, heads, d)
    c = torch.cat([cos, cos], -1).view(1, S, 1, d)
    s = torch.cat([sin, sin], -1).view(1, S, 1, d)
    rotate_half = torch.cat([-xh[..., d // 2:], xh[..., :d // 2]], -1)
    want = (xh * c + rotate_half * s)
    got = rotated.view(B, S, heads, d)
    _close(got[:, :, :2], want[:, :, :2])
    assert torch.equal(got[:, :, 2], xh[:, :, 2])
    _close(R.rope_(rotated.clone(), cos, sin, 2, d, S, inverse=True), x)


def test_swiglu_forward_and_backward_match_autograd():
    gu = torch.randn(9, 24, requires_grad=True)
    a = F.silu(gu[:, :12]) * gu[:, 12:]
    da = torch.randn(9, 12)
    a.backward(da)
    _close(R.swiglu_fwd(gu.detach()), a.detach())
    _close(R.swiglu_bwd(gu.detach(), da), gu.grad)


@pytest.mark.parametrize("shards", [1, 3])
def test_cross_entropy_statistics_and_gradient_match_autograd_also_when_the_vocabulary_is_sharded(shards):
    T, V = 11, 30
    logits = torch.randn(T, V, requires_grad=True)
    targets = torch.randint(0, V, (T,))
    loss = F.cross_entropy(logits, targets, reduction="mean")
    loss.backward()
    per = V // shards
    stats = [R.ce_stats(logits.detach()[:, i * per:(i + 1) * per], targets, i * per) for i in range(shards)]
    gmax = torch.stack([s[0] for s in stats]).max(0).values
    sumexp = sum(s[1] * torch.exp(s[0] - gmax) for s in stats)
    tgt = sum(s[2] for s in stats)
    lse = gmax + torch.log(sumexp)
    _close((lse - tgt).mean(), loss.detach())
    grads = [R.ce_grad_(logits.detach()[:, i * per:(i + 1) * per].clone(), targets, lse, 1.0 / T, i * per) for i in range(shards)]
    _close(torch.cat(grads, -1), logits.grad)


def test_embedding_shards_sum_to_the_lookup_and_scatter_their_own_rows_back():
    V, H = 12, 5
    w = torch.randn(V, H, requires_grad=True)
    ids = torch.randint(0, V, (3, 7))
    out = F.embedding(ids, w)
    dy = torch.randn(3, 7, H)
    out.backward(dy)
    parts = [R.embedding_fwd(ids, w.detach()[i * 4:(i + 1) * 4], i * 4) for i in range(3)]
    _close(sum(parts), out.detach().reshape(-1, H))
    for i in range(3):
        dw = torch.zeros(4, H)
        R.embedding_bwd(ids, dy, dw, i * 4)
        _close(dw, w.grad[i * 4:(i + 1) * 4])


def test_adamw_restatement_follows_torch_adamw_over_several_steps():
    p = torch.nn.Parameter(torch.randn(6, 4))
    opt = torch.optim.AdamW([p], lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    mine, m, v = p.detach().clone(), torch.zeros(6, 4), torch.zeros(6, 4)
    for step in range(1, 6):
        g = torch.randn(6, 4)
        p.grad = g.clone()
        opt.step()
        R.adamw_step_([mine], [g], [m], [v], [None], step, 3e-3, 0.9, 0.95, 1e-8, 0.1)
        _close(mine, p.detach(), 1e-6)
    # bf16 parameter with an fp32 master copy: the master follows the fp32 run, the parameter is its rounding
    master = mine.clone()
    pb = mine.to(torch.bfloat16)
    g = torch.randn(6, 4)
    p.grad = g.clone()
    opt.step()
    R.adamw_step_([pb], [g], [m], [v], [master], 6, 3e-3, 0.9, 0.95, 1e-8, 0.1)
    _close(master, p.detach(), 1e-6)
    assert torch.equal(pb, master.to(torch.bfloat16))
