"""The fused model on the GPU (bf16, CUDA kernels) against the same model on CPU (fp32, PyTorch restatements)."""
import pytest
import torch

from picotron_b200.config import ModelConfig
from picotron_b200.models.llama import Llama
from picotron_b200.optim import FusedAdamW
from picotron_b200.parallel.data_parallel import DataParallelBucket

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("hq,hkv,d", [(8, 8, 64), (8, 2, 64), (4, 2, 128)])
def test_model_loss_and_grads_match_cpu_fp32(hq, hkv, d):
    from picotron_b200.ops import _ext
    C = _ext.load()
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=hq * d, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=hq,
                      num_key_value_heads=hkv, vocab_size=1024, max_position_embeddings=256)
    cpu = Llama(cfg, init="normal")
    gpu = Llama(cfg, init="normal")
    gpu.load_state_dict(cpu.state_dict())
    gpu = gpu.to(torch.bfloat16).cuda()
    with torch.no_grad():                      # same (bf16-rounded) weights on both sides
        for pc, pg in zip(cpu.parameters(), gpu.parameters()):
            pc.copy_(pg.float().cpu())
    wg = DataParallelBucket(gpu)
    ids = torch.randint(0, cfg.vocab_size, (2, 256))
    tgt = torch.randint(0, cfg.vocab_size, (2, 256))
    n0 = C.launch_count()
    loss_g = wg(input_ids=ids.cuda(), target_ids=tgt.cuda())
    loss_g.backward()
    torch.cuda.synchronize()
    assert C.launch_count() > n0, "the CUDA kernels did not run"
    assert C.kernel_status() == 0
    loss_c = cpu(ids, target_ids=tgt)
    loss_c.backward()
    assert abs(loss_g.item() - loss_c.item()) < 3e-2, (loss_g.item(), loss_c.item())
    for (n, pc), pg in zip(cpu.named_parameters(), gpu.parameters()):
        g, r = pg.main_grad.float().cpu(), pc.grad
        err = (g - r).norm() / (r.norm() + 1e-12)
        assert err < 5e-2, f"{n}: relative gradient error {err:.4f}"
    opt = FusedAdamW(wg.parameters(), lr=1e-3)
    before = [p.detach().clone() for p in gpu.parameters()]
    opt.step()
    wg.reset()
    torch.cuda.synchronize()
    assert any(not torch.equal(a, b) for a, b in zip(before, gpu.parameters()))
    assert all(torch.isfinite(p).all() for p in gpu.parameters())
