"""Model conversion onto the forge_b200 INT8 layers.

Counterpart of the reference's `forge.quant.quantize` for the layers on this path
(python/forge/quant/convert.py:19-98): walks the module tree and swaps every `nn.Linear` for a
`QuantizedLinear` holding its per-channel INT8 weight, or for a `SparseLinear` when
`sparse=True` and the shape allows it. Only the dynamic per-token scheme exists here (it is the
one the kernels implement); `nn.Embedding` and every other module are left untouched.
"""
import copy

import torch
import torch.nn as nn

from .nn import QuantizedLinear, SparseLinear


def _set_child(model, dotted, new_module):
    parent = model
    *path, leaf = dotted.split(".")
    for part in path:
        parent = getattr(parent, part)
    setattr(parent, leaf, new_module)


def quantize(model, scheme="dynamic_int8", inplace=False, sparse=False, verbose=True):
    """Returns `model` with its `nn.Linear` layers replaced by W8A8 layers.

    sparse=True prunes each weight 2:4 by magnitude and uses `SparseLinear` where
    in_features % 64 == 0 and out_features % 16 == 0 (other layers stay dense INT8).
    """
    if scheme != "dynamic_int8":
        raise ValueError("forge_b200 implements the dynamic per-token INT8 scheme only")
    if not inplace:
        model = copy.deepcopy(model)
    swaps = []
    for name, module in model.named_modules():
        if not isinstance(module, nn.Linear):
            continue
        dev = module.weight.device
        has_bias = module.bias is not None
        use_sparse = sparse and module.in_features % 64 == 0 and module.out_features % 16 == 0
        cls = SparseLinear if use_sparse else QuantizedLinear
        new = cls(module.in_features, module.out_features, bias=has_bias).to(dev)
        if use_sparse:
            new.from_dense_weight(module.weight.data)
        else:
            new.quantize_weight(module.weight.data)
        if has_bias:
            new.bias.data.copy_(module.bias.data.to(torch.float16))
        swaps.append((name, new))
    for name, new in swaps:
        _set_child(model, name, new)
    if verbose:
        n_sparse = sum(isinstance(m, SparseLinear) for _, m in swaps)
        print(f"forge_b200.quant: converted {len(swaps) - n_sparse} Linear -> QuantizedLinear, "
              f"{n_sparse} Linear -> SparseLinear")
    return model
