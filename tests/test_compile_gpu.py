"""forge_b200.compile on a GPU: a model compiled with the INT8 backends gives bit for bit the
output of the same model converted by forge_b200.quant.quantize (reference mechanism:
python/forge/compile/backend.py:20-49, there for the FP32 GEMM)."""
import copy
import os
import sys

import pytest
import torch
import torch.fx as fx
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

pytestmark = pytest.mark.gpu


class Block(nn.Module):
    def __init__(self, d=256, f=512):
        super().__init__()
        self.up = nn.Linear(d, f)
        self.down = nn.Linear(f, d, bias=False)
        self.head_w = nn.Parameter(torch.randn(48, d) * 0.05)

    def forward(self, x):
        h = F.silu(self.up(x))
        return F.linear(self.down(h) + x, self.head_w)


def _expected(model, x, sparse):
    """The same network with its layers converted by quantize(); the F.linear head by hand."""
    from forge_b200 import quant as Q
    from forge_b200.quant import _to_w8a8
    q = Q.quantize(copy.deepcopy(model), sparse=sparse, verbose=False)
    head = nn.Linear(model.head_w.shape[1], model.head_w.shape[0], bias=False).to(x.device, x.dtype)
    head.weight.data.copy_(model.head_w.data)
    head = _to_w8a8(head, sparse)
    with torch.no_grad():
        h = F.silu(q.up(x))
        return head(q.down(h) + x)


@pytest.mark.parametrize("sparse", [False, True])
def test_fx_rewrite_matches_converted_model(sparse):
    from forge_b200 import _forge_C as C
    from forge_b200 import compile as fcompile
    torch.manual_seed(5)
    model = Block().cuda().half().eval()
    x = torch.randn(3, 70, 256, device="cuda", dtype=torch.float16)
    gm = fcompile.apply_int8_patterns(fx.symbolic_trace(model), sparse=sparse)
    assert gm.forge_b200_replacements == 3
    y = gm(x)
    want = _expected(model, x, sparse)
    assert y.dtype == torch.float16 and y.shape == (3, 70, 48)
    assert torch.equal(y.view(torch.int16), want.view(torch.int16))
    # a second call reuses the prepared weights; an in-place weight update re-prepares them
    n_before = len(fcompile._prepared)
    assert torch.equal(gm(x).view(torch.int16), want.view(torch.int16))
    assert len(fcompile._prepared) == n_before
    with torch.no_grad():
        model.up.weight.mul_(0.5)
    want2 = _expected(model, x, sparse)
    assert torch.equal(gm(x).view(torch.int16), want2.view(torch.int16))
    assert C.device_status() == 0


def test_torch_compile_backend_runs_the_int8_kernels():
    import forge_b200.compile  # noqa: F401  (registers the backends)
    import torch._dynamo as dynamo
    dynamo.reset()
    torch.manual_seed(6)
    model = Block().cuda().half().eval()
    x = torch.randn(200, 256, device="cuda", dtype=torch.float16)
    fast = torch.compile(model, backend="forge_b200_int8")
    with torch.no_grad():
        y = fast(x)
        ref_fp = model(x)
    want = _expected(model, x, False)
    assert torch.equal(y.view(torch.int16), want.view(torch.int16))
    # and it is the quantized result, not the fp16 one that Dynamo would fall back to
    assert not torch.equal(y, ref_fp)
    assert torch.allclose(y.float(), ref_fp.float(), atol=0.15, rtol=0.1)


def test_fp32_model_keeps_its_dtype():
    from forge_b200 import compile as fcompile
    torch.manual_seed(7)
    lin = nn.Linear(128, 64).cuda().eval()
    x = torch.randn(33, 128, device="cuda")
    gm = fcompile.apply_int8_patterns(fx.symbolic_trace(lin))
    y = gm(x)
    assert y.dtype == torch.float32 and y.shape == (33, 64)
    assert torch.allclose(y, lin(x), atol=0.05, rtol=0.05)
