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
