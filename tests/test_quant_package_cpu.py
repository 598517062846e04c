"""forge_b200.quant on the CPU: the conversion and QAT helpers that mirror the reference's
forge.quant package (python/forge/quant/{convert,fake_quantize,observers}.py). Layer forwards need a
GPU and are covered by tests/test_nn_modules_gpu.py; here: signatures, observers, the fake-quantize
arithmetic and its straight-through gradient, and the module swaps."""
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
    for fn in ("prepare_qat", "enable_calibration", "enable_qat", "finalize_qat", "MinMaxObserver",
               "PercentileObserver", "FakeQuantize"):
        assert hasattr(Q, fn)


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


def test_min_max_observer_scales():
    obs = Q.MinMaxObserver()
    obs(torch.tensor([-3.0, 1.0]))
    obs(torch.tensor([0.5, 2.0]))
    assert float(obs.compute_scale()) == pytest.approx(3.0 / 127.0) and int(obs.num_batches) == 2
    pc = Q.MinMaxObserver(per_channel=True, ch_axis=0)
    pc(torch.tensor([[1.0, -4.0], [0.5, 0.25]]))
    pc(torch.tensor([[2.0, 0.0], [-1.0, 0.0]]))
    assert torch.allclose(pc.compute_scale(), torch.tensor([4.0, 1.0]) / 127.0)
    obs.reset()
    obs(torch.zeros(3))
    assert float(obs.compute_scale()) == pytest.approx(1e-8)     # the floor


def test_percentile_observer_clips_outliers():
    torch.manual_seed(1)
    x = torch.randn(100000)
    x[0] = 1000.0
    mm, pct = Q.MinMaxObserver(), Q.PercentileObserver(percentile=99.9)
    mm(x)
    pct(x)
    assert float(pct.compute_scale()) < 0.1 * float(mm.compute_scale())
    pct.reset()
    assert float(pct.compute_scale()) == 1.0


def test_fake_quantize_rounds_and_passes_gradients_inside_the_range():
    fq = Q.FakeQuantize()
    x = torch.tensor([-1.27, -0.5049, 0.0, 0.004, 0.5, 1.27], requires_grad=True)
    assert torch.equal(fq(x), x)                 # observe only
    fq.quantize()
    scale = float(fq.scale)
    assert scale == pytest.approx(0.01)
    y = fq(x)
    assert torch.allclose(y, torch.round(x.detach() / scale).clamp(-127, 127) * scale)
    big = torch.tensor([5.0, -5.0, 0.3], requires_grad=True)
    fq(big).sum().backward()
    assert big.grad.tolist() == [0.0, 0.0, 1.0]  # clipped values get no gradient
    fq.calibrate()
    assert torch.equal(fq(x), x)


def test_qat_round_trip_ends_in_w8a8_layers():
    torch.manual_seed(2)
    net = Net()
    qat = Q.prepare_qat(net)
    assert isinstance(net.a, nn.Linear) and qat.a.in_features == 32 and qat.block[1].out_features == 16
    Q.enable_calibration(qat)
    x = torch.randn(8, 32)
    ref = net(x)
    assert torch.allclose(qat(x), ref)           # calibration mode changes nothing
    Q.enable_qat(qat)
    y = qat(x)
    assert not torch.equal(y, ref) and (y - ref).abs().max() < 0.1
    y.sum().backward()                            # straight-through: the float weights get gradients
    assert qat.a.linear.weight.grad is not None and qat.a.linear.weight.grad.abs().sum() > 0
    with torch.no_grad():
        qat.a.linear.weight.mul_(0.5)             # "training" changed the weight
    final = Q.finalize_qat(qat, verbose=False)
    assert isinstance(final.a, QuantizedLinear) and isinstance(final.block[1], QuantizedLinear)
    wq, ws = quantize_weight_per_channel(net.a.weight.data * 0.5)
    assert torch.equal(final.a.w_int8, wq) and torch.equal(final.a.w_scale.data, ws)
