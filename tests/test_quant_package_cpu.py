"""forge_b200.quant on the CPU: the two conversion functions that mirror the reference's
forge.quant package (python/forge/quant/convert.py). Layer forwards need a GPU and are covered by
tests/test_nn_modules_gpu.py; here: signatures and the module swaps."""
import inspect

import pytest
import torch
import torch.nn as nn

from forge_b200 import quant as Q
from forge_b200.nn import QuantizedLinear, quantize_weight_per_channel


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(32, 48)
        self.block = nn.Sequential(nn.ReLU(), nn.Linear(48, 16, bias=False))
        self.emb = nn.Embedding(10, 4)

    def forward(self, x):
        return self.block(self.a(x))


def test_quantize_keeps_the_reference_parameter_order():
    names = list(inspect.signature(Q.quantize).parameters)
    assert names[:6] == ["model", "calibration_data", "num_calibration_batches", "scheme", "inplace", "forward_fn"]
    assert hasattr(Q, "finalize_qat")


@pytest.mark.parametrize("scheme", ["dynamic_int8", "static_int8", "weight_only_int8"])
def test_quantize_swaps_linears_on_a_copy(scheme):
    torch.manual_seed(0)
    net = Net()
    seen = []
    data = [torch.randn(4, 32) for _ in range(5)]
    # forward_fn is used instead of model(batch), so no GPU layer runs here
    out = Q.quantize(net, data, 3, scheme, forward_fn=lambda m, b: seen.append(tuple(b.shape)), verbose=False)
    assert isinstance(net.a, nn.Linear) and out is not net
    assert isinstance(out.a, QuantizedLinear) and isinstance(out.block[1], QuantizedLinear)
    assert isinstance(out.emb, nn.Embedding) and out.block[1].bias is None
    wq, ws = quantize_weight_per_channel(net.a.weight.data)
    assert torch.equal(out.a.w_int8, wq) and torch.equal(out.a.w_scale.data, ws)
    assert torch.equal(out.a.bias.data, net.a.bias.data.half())
    assert len(seen) == (3 if scheme == "static_int8" else 0)
    with pytest.raises(ValueError):
        Q.quantize(net, scheme="int4", verbose=False)


class FakeQuantStub(nn.Module):
    """Stands in for the reference's FakeQuantize module: finalize_qat only looks at the wrapper's shape."""

    def forward(self, x):
        return x


class WrappedLinear(nn.Module):
    """Same attribute layout as the reference's QAT wrapper (python/forge/quant/convert.py:123-160)."""

    def __init__(self, linear):
        super().__init__()
        self.linear = linear
        self.weight_fq = FakeQuantStub()
        self.input_fq = FakeQuantStub()

    def forward(self, x):
        return nn.functional.linear(self.input_fq(x), self.weight_fq(self.linear.weight), self.linear.bias)


def test_finalize_qat_converts_wrappers_recognised_by_their_shape():
    torch.manual_seed(2)
    net = Net()
    net.a = WrappedLinear(net.a)
    net.block[1] = WrappedLinear(net.block[1])
    with torch.no_grad():
        net.a.linear.weight.mul_(0.5)             # "training" changed the weight
    trained = net.a.linear.weight.data.clone()
    final = Q.finalize_qat(net, verbose=False)
    assert isinstance(final.a, QuantizedLinear) and isinstance(final.block[1], QuantizedLinear)
    assert isinstance(final.emb, nn.Embedding)
    wq, ws = quantize_weight_per_channel(trained)
    assert torch.equal(final.a.w_int8, wq) and torch.equal(final.a.w_scale.data, ws)
    # a module that merely has a `linear` attribute is left alone
    other = nn.Sequential(nn.Linear(8, 8))
    other.linear = nn.Linear(8, 8)
    assert isinstance(Q.finalize_qat(other, verbose=False).linear, nn.Linear)
