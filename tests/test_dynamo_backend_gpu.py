"""torch.compile(backend="b200k") on the GPU: the compiled module must run the b200k kernels for
its linear layers and its attention and match eager PyTorch within the path's tolerance."""

import pytest
import torch
import torch.nn.functional as F

import iree_turbine_b200 as tb
from iree_turbine_b200 import dynamo_backend as db

pytestmark = pytest.mark.gpu
DEV = "cuda"


class Block(torch.nn.Module):
    def __init__(self, dim=512, heads=4):
        super().__init__()
        self.heads = heads
        self.qkv = torch.nn.Linear(dim, 3 * dim, bias=False)
        self.proj = torch.nn.Linear(dim, dim, bias=True)

    def forward(self, x, causal: bool):
        b, s, d = x.shape
        qkv = self.qkv(x.reshape(b * s, d)).reshape(b, s, 3, self.heads, d // self.heads)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        o = F.scaled_dot_product_attention(q, k, v, is_causal=causal)
        return self.proj(o.transpose(1, 2).reshape(b * s, d)).reshape(b, s, d)


@pytest.mark.parametrize("causal", [False, True])
def test_compiled_block_matches_eager(causal):
    torch.manual_seed(0)
    m = Block().to(DEV).half().eval()
    x = (torch.randn(2, 256, 512, device=DEV) * 0.5).half()
    with torch.no_grad():
        ref = m(x, causal)
        torch._dynamo.reset()
        db.backend.last_replaced = 0
        out = torch.compile(m, backend="b200k")(x, causal)
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    assert db.backend.last_replaced >= 3, "qkv mm, attention and proj addmm should all have been routed"
    torch.testing.assert_close(out.float(), ref.float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("head_dim", [128, 64])
def test_compiled_training_step_routes_attention_forward_and_backward(head_dim):
    """A training step through torch.compile: the forward graph's fused attention (whose log-sum-exp is saved)
    and the backward graph's attention-backward node both run on the b200k kernels; gradients match eager."""
    import copy

    torch.manual_seed(1)
    m = Block(dim=4 * head_dim, heads=4).to(DEV).to(torch.bfloat16)
    ref_m = copy.deepcopy(m)
    x = (torch.randn(2, 256, 4 * head_dim, device=DEV) * 0.5).to(torch.bfloat16)
    ref = ref_m(x, True)
    ref.float().square().mean().backward()
    torch._dynamo.reset()
    db.backend.last_replaced = db.backend.last_replaced_backward = 0
    out = torch.compile(m, backend="b200k")(x, True)
    out.float().square().mean().backward()
    torch.cuda.synchronize()
    assert tb.device_status() == 0
    assert db.backend.last_replaced >= 3
    assert db.backend.last_replaced_backward >= 1, "the backward graph's attention node should have been routed"
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)
    for (name, p), (_, pr) in zip(m.named_parameters(), ref_m.named_parameters()):
        scale = pr.grad.float().abs().max().item()
        err = (p.grad.float() - pr.grad.float()).abs().max().item()
        assert err <= 3e-2 * max(scale, 1e-6), (name, err, scale)
