"""Model conversion onto the forge_b200 INT8 layers: the counterpart of the reference's
`forge.quant` package for the layers on this path.

  quantize(model, ...)                      post-training conversion (python/forge/quant/convert.py:19-98):
                                            every `nn.Linear` becomes a `QuantizedLinear` holding its
                                            per-channel INT8 weight - or a `SparseLinear` with sparse=True
                                            where the shape allows 2:4. Same parameter order as the
                                            reference, so `quantize(model, dataloader)` keeps working.
  prepare_qat / enable_calibration /        quantization-aware training (convert.py:123-237,
  enable_qat / finalize_qat                 fake_quantize.py, observers.py): fake-quantize wrappers with
                                            a straight-through backward, then conversion of the trained
                                            wrappers to `QuantizedLinear`.
  MinMaxObserver, PercentileObserver,       the statistics modules behind the wrappers.
  FakeQuantize

As in the reference every scheme ends in the same dynamic per-token layer (the reference's
"static_int8" only runs the calibration batches through the converted model; its layers have no
static activation scale either). `nn.Embedding` and every other module are left untouched: the
reference's FP embedding replacement is not on this path.
"""
import copy

import torch
import torch.nn as nn

from .nn import QuantizedLinear, SparseLinear

_SCHEMES = ("dynamic_int8", "static_int8", "weight_only_int8")


def _set_child(model, dotted, new_module):
    parent = model
    *path, leaf = dotted.split(".")
    for part in path:
        parent = getattr(parent, part)
    setattr(parent, leaf, new_module)


def _run_calibration(model, data, num_batches, forward_fn, device):
    """convert.py:101-120: up to num_batches batches through the model, first element of tuple batches."""
    model.eval()
    with torch.no_grad():
        for i, batch in enumerate(data):
            if i >= num_batches:
                break
            if isinstance(batch, (tuple, list)):
                batch = batch[0]
            batch = batch.to(device)
            if forward_fn is not None:
                forward_fn(model, batch)
            else:
                model(batch)


def _to_w8a8(linear, sparse):
    dev = linear.weight.device
    has_bias = linear.bias is not None
    use_sparse = (sparse and dev.type == "cuda" and linear.in_features % 64 == 0 and linear.out_features % 16 == 0)
    new = (SparseLinear if use_sparse else QuantizedLinear)(linear.in_features, linear.out_features, bias=has_bias).to(dev)
    if use_sparse:
        new.from_dense_weight(linear.weight.data)
    else:
        new.quantize_weight(linear.weight.data)
    if has_bias:
        new.bias.data.copy_(linear.bias.data.to(torch.float16))
    return new


def quantize(model, calibration_data=None, num_calibration_batches=100, scheme="dynamic_int8", inplace=False,
             forward_fn=None, *, sparse=False, verbose=True):
    """Returns `model` with its `nn.Linear` layers replaced by W8A8 layers.

    Parameters up to `forward_fn` are the reference's (convert.py:19-26). Additive, keyword only:
    sparse=True prunes each weight 2:4 by magnitude and uses `SparseLinear` where the layer is on a
    GPU, in_features % 64 == 0 and out_features % 16 == 0 (other layers stay dense INT8);
    verbose=False silences the one-line report.
    """
    if scheme not in _SCHEMES:
        raise ValueError(f"unknown scheme {scheme!r}; expected one of {_SCHEMES}")
    if not inplace:
        model = copy.deepcopy(model)
    swaps = [(name, _to_w8a8(m, sparse)) for name, m in model.named_modules() if isinstance(m, nn.Linear)]
    for name, new in swaps:
        _set_child(model, name, new)
    if scheme == "static_int8" and calibration_data is not None:
        first = next(model.parameters(), None)
        device = first.device if first is not None else torch.device("cpu")
        _run_calibration(model, calibration_data, num_calibration_batches, forward_fn, device)
    if verbose:
        n_sparse = sum(isinstance(m, SparseLinear) for _, m in swaps)
        print(f"forge_b200.quant: converted {len(swaps) - n_sparse} Linear -> QuantizedLinear, "
              f"{n_sparse} Linear -> SparseLinear")
    return model


# ------------------------------------------------------------------------------------------------
# Observers (python/forge/quant/observers.py)

class MinMaxObserver(nn.Module):
    """Running minimum / maximum of everything it sees, per tensor or per slice of `ch_axis`;
    symmetric INT8 scale = max(|min|, |max|) / 127, floored at 1e-8 (observers.py:6-58)."""

    def __init__(self, per_channel=False, ch_axis=0):
        super().__init__()
        self.per_channel, self.ch_axis = per_channel, ch_axis
        self.register_buffer("min_val", torch.tensor(float("inf")))
        self.register_buffer("max_val", torch.tensor(float("-inf")))
        self.register_buffer("num_batches", torch.tensor(0, dtype=torch.long))

    @torch.no_grad()
    def forward(self, x):
        if self.per_channel:
            other = [d for d in range(x.ndim) if d != self.ch_axis]
            lo = x.amin(dim=other) if other else x
            hi = x.amax(dim=other) if other else x
            if int(self.num_batches) == 0:
                self.min_val, self.max_val = lo.clone(), hi.clone()
            else:
                self.min_val, self.max_val = torch.minimum(self.min_val, lo), torch.maximum(self.max_val, hi)
        else:
            self.min_val = torch.minimum(self.min_val, x.min())
            self.max_val = torch.maximum(self.max_val, x.max())
        self.num_batches += 1
        return x

    def compute_scale(self):
        return (torch.maximum(self.min_val.abs(), self.max_val.abs()) / 127.0).clamp(min=1e-8)

    def reset(self):
        dev = self.min_val.device
        self.min_val = torch.tensor(float("inf"), device=dev)
        self.max_val = torch.tensor(float("-inf"), device=dev)
        self.num_batches.zero_()


class PercentileObserver(nn.Module):
    """Histogram of the observed values over the range of the first batch; the scale clips at the
    given percentile on both sides (observers.py:61-128)."""

    def __init__(self, percentile=99.99, num_bins=2048):
        super().__init__()
        self.percentile, self.num_bins = percentile, num_bins
        self.register_buffer("histogram", torch.zeros(num_bins))
        self.register_buffer("bin_edges", torch.zeros(num_bins + 1))
        self.register_buffer("min_val", torch.tensor(float("inf")))
        self.register_buffer("max_val", torch.tensor(float("-inf")))
        self.register_buffer("num_batches", torch.tensor(0, dtype=torch.long))
        self._have_edges = False

    @torch.no_grad()
    def forward(self, x):
        flat = x.float().flatten()
        lo, hi = flat.min(), flat.max()
        self.min_val, self.max_val = torch.minimum(self.min_val, lo), torch.maximum(self.max_val, hi)
        if not self._have_edges:
            self.bin_edges = torch.linspace(lo.item(), hi.item(), self.num_bins + 1, device=x.device)
            self._have_edges = True
        self.histogram += torch.histc(flat, bins=self.num_bins, min=self.bin_edges[0].item(),
                                      max=self.bin_edges[-1].item()).to(self.histogram.device)
        self.num_batches += 1
        return x

    def compute_scale(self):
        total = self.histogram.sum()
        if total == 0:
            return torch.tensor(1.0)
        cdf = self.histogram.cumsum(dim=0) / total
        q = self.percentile / 100.0
        above = (cdf >= q).nonzero(as_tuple=True)[0]
        clip = self.bin_edges[above[0] + 1].abs() if len(above) else self.max_val.abs()
        below = (cdf >= 1.0 - q).nonzero(as_tuple=True)[0]
        if len(below):
            clip = torch.maximum(clip, self.bin_edges[below[0]].abs())
        return (clip / 127.0).clamp(min=1e-8)

    def reset(self):
        self.histogram.zero_()
        self.min_val.fill_(float("inf"))
        self.max_val.fill_(float("-inf"))
        self.num_batches.zero_()
        self._have_edges = False


# ------------------------------------------------------------------------------------------------
# Fake quantization (python/forge/quant/fake_quantize.py)

class _RoundClampSTE(torch.autograd.Function):
    """x -> clamp(round(x / scale), -127, 127) * scale; the gradient passes where |x| <= 127 * scale."""

    @staticmethod
    def forward(ctx, x, scale):
        ctx.save_for_backward((x.abs() <= scale * 127).to(x.dtype))
        return (x * (1.0 / scale)).round().clamp(-127, 127) * scale

    @staticmethod
    def backward(ctx, grad):
        (inside,) = ctx.saved_tensors
        return grad * inside, None


class FakeQuantize(nn.Module):
    """Observes always; once `quantize()` has been called also simulates symmetric INT8 rounding with
    a straight-through backward (fake_quantize.py:14-67). `calibrate()` goes back to observe-only."""

    def __init__(self, observer=None, per_channel=False, ch_axis=0):
        super().__init__()
        self.observer = observer if observer is not None else MinMaxObserver(per_channel, ch_axis)
        self.per_channel, self.ch_axis = per_channel, ch_axis
        self.enabled = False
        self.register_buffer("scale", torch.tensor(1.0))
        self._calibrated = False

    def calibrate(self):
        self.enabled = False

    def quantize(self):
        if not self._calibrated:
            self.update_scale()
        self.enabled = True

    def update_scale(self):
        self.scale = self.observer.compute_scale()
        self._calibrated = True

    def forward(self, x):
        self.observer(x)
        if not self.enabled:
            return x
        scale = self.scale
        if self.per_channel and scale.ndim == 1 and x.ndim > 1:
            shape = [1] * x.ndim
            shape[self.ch_axis] = -1
            scale = scale.view(shape)
        return _RoundClampSTE.apply(x, scale)


# ------------------------------------------------------------------------------------------------
# Quantization-aware training (python/forge/quant/convert.py:123-237)

class _QATLinearWrapper(nn.Module):
    """An `nn.Linear` with fake quantization of its input (per tensor) and weight (per output channel)."""

    def __init__(self, linear):
        super().__init__()
        self.linear = linear
        self.weight_fq = FakeQuantize(MinMaxObserver(per_channel=True, ch_axis=0), per_channel=True, ch_axis=0)
        self.input_fq = FakeQuantize(MinMaxObserver(per_channel=False))

    def forward(self, x):
        return nn.functional.linear(self.input_fq(x), self.weight_fq(self.linear.weight), self.linear.bias)

    def calibrate(self):
        self.weight_fq.calibrate()
        self.input_fq.calibrate()

    def enable_qat(self):
        self.weight_fq.quantize()
        self.input_fq.quantize()

    @property
    def in_features(self):
        return self.linear.in_features

    @property
    def out_features(self):
        return self.linear.out_features


def prepare_qat(model, inplace=False):
    """Wraps every `nn.Linear` so that training sees INT8 rounding noise on inputs and weights."""
    if not inplace:
        model = copy.deepcopy(model)
    for name, module in list(model.named_modules()):
        if isinstance(module, nn.Linear):
            _set_child(model, name, _QATLinearWrapper(module))
    return model


def enable_calibration(model):
    """All fake-quantize modules observe only."""
    for m in model.modules():
        if isinstance(m, (FakeQuantize, _QATLinearWrapper)):
            m.calibrate()


def enable_qat(model):
    """All fake-quantize modules round (scales taken from their observers on first use)."""
    for m in model.modules():
        if isinstance(m, FakeQuantize):
            m.quantize()
        elif isinstance(m, _QATLinearWrapper):
            m.enable_qat()


def finalize_qat(model, *, sparse=False, verbose=True):
    """Replaces the trained wrappers by W8A8 layers built from their (trained) float weights
    (convert.py:205-237). Additive: sparse=True as in `quantize`."""
    swaps = [(name, _to_w8a8(m.linear, sparse)) for name, m in model.named_modules()
             if isinstance(m, _QATLinearWrapper)]
    for name, new in swaps:
        _set_child(model, name, new)
    if verbose:
        print(f"forge_b200.quant: finalized {len(swaps)} QAT layers")
    return model
