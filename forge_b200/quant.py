"""Model conversion onto the forge_b200 INT8 layers: the two functions of the reference's
`forge.quant` package that create layers of this path.

  quantize(model, ...)     post-training conversion (python/forge/quant/convert.py:19-98): every
                           `nn.Linear` becomes a `QuantizedLinear` holding its per-channel INT8
                           weight - or a `SparseLinear` with sparse=True where the shape allows 2:4.
                           Same parameter order as the reference, so `quantize(model, dataloader)`
                           keeps working.
  finalize_qat(model)      the last step of quantization-aware training (convert.py:205-237): the
                           trained fake-quantize wrappers become `QuantizedLinear` / `SparseLinear`.

The observers, fake-quantize modules and `prepare_qat` / `enable_qat` of the reference are plain
PyTorch and do not touch the kernels; they are used as they are (python/forge/quant/
{observers,fake_quantize}.py) and are not restated here. `finalize_qat` recognises the
reference's wrapper by its shape - a module with a `linear` (`nn.Linear`), a `weight_fq` and an
`input_fq` attribute - so it works on a model prepared by the reference package.

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


def _is_qat_wrapper(m):
    """The reference's QAT wrapper (convert.py:123-160), recognised structurally."""
    return isinstance(getattr(m, "linear", None), nn.Linear) and hasattr(m, "weight_fq") and hasattr(m, "input_fq")


def finalize_qat(model, *, sparse=False, verbose=True):
    """Replaces trained fake-quantize wrappers by W8A8 layers built from their (trained) float
    weights (convert.py:205-237). Additive: sparse=True as in `quantize`."""
    swaps = [(name, _to_w8a8(m.linear, sparse)) for name, m in model.named_modules() if _is_qat_wrapper(m)]
    for name, new in swaps:
        _set_child(model, name, new)
    if verbose:
        print(f"forge_b200.quant: finalized {len(swaps)} QAT layers")
    return model
