import torch

from picotron_b200.config import ModelConfig
from picotron_b200.models.llama import Llama
from picotron_b200.optim import FusedAdamW
from picotron_b200.parallel.data_parallel import DataParallelBucket

import oracle


def tiny_cfg(**kw):
    base = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, vocab_size=97, max_position_embeddings=16)
    base.update(kw)
    return ModelConfig(**base)


def test_fused_layer_matches_autograd_oracle():
    torch.manual_seed(0)
    cfg = tiny_cfg()
    m = Llama(cfg)
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    tgt = torch.randint(0, cfg.vocab_size, (2, 16))
    loss = m(ids, target_ids=tgt)
    loss.backward()
    ref_loss, ref_grads = oracle.loss_and_grads(dict(m.named_parameters()), cfg, ids, tgt)
    torch.testing.assert_close(loss.detach(), ref_loss, rtol=1e-5, atol=1e-6)
    for n, p in m.named_parameters():
        torch.testing.assert_close(p.grad, ref_grads[n], rtol=1e-4, atol=1e-6, msg=lambda s, n=n: f"{n}: {s}")
    logits = m(ids)
    torch.testing.assert_close(logits, oracle.llama_forward(dict(m.named_parameters()), cfg, ids), rtol=1e-5, atol=1e-5)


def test_mha_and_chunked_head():
    torch.manual_seed(1)
    cfg = tiny_cfg(num_key_value_heads=4)
    m = Llama(cfg)
    m.ce_chunk_tokens = 5  # ragged chunks
    ids = torch.randint(0, cfg.vocab_size, (3, 16))
    tgt = torch.randint(0, cfg.vocab_size, (3, 16))
    loss = m(ids, target_ids=tgt, loss_scale=0.5)
    loss.backward()
    ref_loss, ref_grads = oracle.loss_and_grads(dict(m.named_parameters()), cfg, ids, tgt)
    torch.testing.assert_close(loss.detach(), 0.5 * ref_loss, rtol=1e-5, atol=1e-6)
    for n, p in m.named_parameters():
        torch.testing.assert_close(p.grad, 0.5 * ref_grads[n], rtol=1e-4, atol=1e-6)


def test_bucket_accumulation_over_micro_batches_and_adamw():
    torch.manual_seed(2)
    cfg = tiny_cfg()
    m = Llama(cfg)
    params0 = {n: p.detach().clone() for n, p in m.named_parameters()}
    w = DataParallelBucket(m, bucket_cap_mb=1)
    n_mb = 3
    ids = torch.randint(0, cfg.vocab_size, (n_mb, 2, 16))
    tgt = torch.randint(0, cfg.vocab_size, (n_mb, 2, 16))
    for i in range(n_mb):
        w.require_backward_grad_sync = i == n_mb - 1
        w(ids[i], target_ids=tgt[i], loss_scale=1.0 / n_mb).backward()
    _, ref_grads = oracle.loss_and_grads(params0, cfg, ids.view(-1, 16), tgt.view(-1, 16))
    for n, p in m.named_parameters():
        assert p.grad is None
        torch.testing.assert_close(p.main_grad, ref_grads[n], rtol=1e-4, atol=1e-6)
    # packed groups stay adjacent in the buckets
    a = m.decoder_layers[0].attention
    assert a.q_proj.weight.main_grad.data_ptr() + a.q_proj.weight.main_grad.numel() * 4 == a.k_proj.weight.main_grad.data_ptr()

    opt = FusedAdamW(w.parameters(), lr=1e-2, master_weights=False)
    ref_params = [p.detach().clone().requires_grad_(True) for p in params0.values()]
    ref_opt = torch.optim.AdamW(ref_params, lr=1e-2)
    for rp, (n, p) in zip(ref_params, m.named_parameters()):
        rp.grad = p.main_grad.clone()  # identical inputs: the first Adam step is ~lr*sign(g), ill-conditioned near 0
    opt.step()
    ref_opt.step()
    for rp, (n, p) in zip(ref_params, m.named_parameters()):
        torch.testing.assert_close(p.detach(), rp.detach(), rtol=1e-4, atol=2e-5)
    w.reset()
    assert all(float(p.main_grad.abs().sum()) == 0.0 for p in m.parameters())


def test_state_dict_names_follow_reference_layout():
    m = Llama(tiny_cfg(num_hidden_layers=1))
    assert sorted(m.state_dict().keys()) == sorted([
        "embedding.weight", "decoder_layers.0.input_layernorm.weight",
        "decoder_layers.0.post_attention_layernorm.weight", "decoder_layers.0.attention.q_proj.weight",
        "decoder_layers.0.attention.k_proj.weight", "decoder_layers.0.attention.v_proj.weight",
        "decoder_layers.0.attention.out_proj.weight", "decoder_layers.0.mlp.gate_proj.weight",
        "decoder_layers.0.mlp.up_proj.weight", "decoder_layers.0.mlp.down_proj.weight",
        "final_norm.weight", "final_proj.weight"])


def test_packing_survives_module_to():
    torch.manual_seed(3)
    cfg = tiny_cfg(num_hidden_layers=1)
    m = Llama(cfg)
    ids = torch.randint(0, cfg.vocab_size, (1, 16))
    y0 = m(ids)
    m.to(torch.float64)
    y1 = m(ids)
    torch.testing.assert_close(y0.double(), y1, rtol=1e-4, atol=1e-4)
    layer = m.decoder_layers[0]
    assert layer.packed_qkv().data_ptr() == layer.attention.q_proj.weight.data_ptr()


def test_checked_mode_names_the_op_that_produced_non_finite_values():
    import pytest
    from picotron_b200 import ops
    ops.enable_checked_mode(True)
    try:
        x = torch.randn(4, 8)
        w = torch.randn(16, 8)
        assert ops.linear_fwd(x, w).shape == (4, 16)                 # a healthy op passes through unchanged
        bad = w.clone()
        bad[3, 2] = float("nan")
        with pytest.raises(FloatingPointError, match="ops.linear_fwd"):
            ops.linear_fwd(x, bad)
    finally:
        ops.enable_checked_mode(False)
    assert torch.isnan(ops.linear_fwd(x, bad)).any()                 # unchecked again


def test_reference_named_model_symbols_exist_and_agree():
    """``picotron.model`` names of the reference: both RMSNorm classes, the flash-attention wrapper, the RoPE helpers."""
    import torch.nn.functional as F
    from picotron_b200.model import (LlamaRMSNorm, TritonRMSNorm, apply_rotary_pos_emb, flash_attention, get_cos_sin)
    fused, eager = TritonRMSNorm(32, eps=1e-5), LlamaRMSNorm(32, eps=1e-5)
    x = torch.randn(2, 5, 32)
    torch.testing.assert_close(fused(x), eager(x), rtol=1e-5, atol=1e-6)         # fp32: the rounding orders coincide
    q, k, v = torch.randn(1, 4, 16, 8), torch.randn(1, 2, 16, 8), torch.randn(1, 2, 16, 8)
    want = F.scaled_dot_product_attention(q, k.repeat_interleave(2, 1), v.repeat_interleave(2, 1), is_causal=True)
    torch.testing.assert_close(flash_attention(q, k, v, True), want.permute(0, 2, 1, 3), rtol=1e-5, atol=1e-5)
    cos, sin = get_cos_sin(16, 8, base=10000.0)
    assert cos.shape == (16, 8) and torch.equal(cos[:, :4], cos[:, 4:])
    r = apply_rotary_pos_emb(q, cos, sin)
    torch.testing.assert_close(r.norm(dim=-1), q.norm(dim=-1), rtol=1e-5, atol=1e-5)   # a rotation keeps the norm


def test_fused_head_loss_without_grad_leaves_the_gradient_buckets_alone():
    """An evaluation forward (no_grad) must not add the LM-head weight gradient to the fp32 bucket; with grad it does, and
    the activation gradient follows the incoming gradient of the loss."""
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.config import ModelConfig
    from picotron_b200.models.llama import Llama
    from picotron_b200.parallel.data_parallel import DataParallelBucket
    pgm.reset()
    cfg = ModelConfig(hidden_size=32, intermediate_size=64, vocab_size=64, num_hidden_layers=1, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=16)
    torch.manual_seed(0)
    model = DataParallelBucket(Llama(cfg))
    ids = torch.randint(0, 64, (2, 16))
    tgt = torch.randint(0, 64, (2, 16))
    head = model.module.final_proj.weight
    with torch.no_grad():
        eval_loss = model(input_ids=ids, target_ids=tgt)
    assert float(head.main_grad.abs().max()) == 0.0
    assert not eval_loss.requires_grad
    loss = model(input_ids=ids, target_ids=tgt)
    torch.testing.assert_close(loss.detach(), eval_loss)
    loss.backward()
    g1 = model.module.embedding.weight.main_grad.clone()
    assert float(head.main_grad.abs().max()) > 0.0
    model.reset()
    (2.0 * model(input_ids=ids, target_ids=tgt)).backward()      # dh follows grad_out (dW keeps the forward-time scale)
    torch.testing.assert_close(model.module.embedding.weight.main_grad, 2.0 * g1, rtol=1e-5, atol=1e-7)


def test_rope_scaling_matches_the_hugging_face_frequencies_and_defaults_to_plain_rope():
    import math
    from picotron_b200.ops.reference import rope_tables, scaled_rope_frequencies
    scaling = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 8192}
    d, base = 64, 500000.0
    inv = 1.0 / (base ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
    ours = scaled_rope_frequencies(inv, scaling)
    try:
        from transformers import LlamaConfig
        from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
        cfg = LlamaConfig(hidden_size=2048, num_attention_heads=32, max_position_embeddings=131072, rope_theta=base,
                          rope_scaling=dict(scaling))
        theirs, factor = ROPE_INIT_FUNCTIONS["llama3"](cfg, "cpu")
        assert factor == 1.0
        torch.testing.assert_close(ours, theirs, rtol=1e-6, atol=0)
    except ImportError:
        pass
    # the three regimes: short wavelengths untouched, long ones divided by the factor, a blended band between
    wavelen = 2 * math.pi / inv
    assert torch.equal(ours[wavelen < 2048], inv[wavelen < 2048])
    torch.testing.assert_close(ours[wavelen > 8192], inv[wavelen > 8192] / 32.0)
    band = (wavelen >= 2048) & (wavelen <= 8192)
    assert band.any() and bool(((ours[band] <= inv[band]) & (ours[band] >= inv[band] / 32.0)).all())
    torch.testing.assert_close(scaled_rope_frequencies(inv, {"type": "linear", "factor": 4.0}), inv / 4.0)
    plain = rope_tables(128, d, base)
    assert torch.equal(rope_tables(128, d, base, scaling=None)[0], plain[0])
    assert not torch.equal(rope_tables(128, d, base, scaling=scaling)[0], plain[0])
    # the model picks the field up from its config
    from picotron_b200 import process_group_manager as pgm
    from picotron_b200.config import ModelConfig
    from picotron_b200.models.llama import Llama
    pgm.reset()
    kw = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=1, num_key_value_heads=1,
              vocab_size=32, max_position_embeddings=64, rope_theta=base)
    a, b = Llama(ModelConfig(**kw)), Llama(ModelConfig(**kw, rope_scaling=scaling))
    assert not torch.equal(a.decoder_layers[0].cos, b.decoder_layers[0].cos)
