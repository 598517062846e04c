"""`torch.compile` front end for the W8A8 path: rewrites the linear layers of a traced graph into
calls of the INT8 kernels.

The reference's compile package (python/forge/compile/backend.py:20-49, patterns.py:62-128)
registers a Dynamo backend that walks the FX graph and replaces `nn.Linear` modules and
`F.linear` calls by its FP32 GEMM; everything else in the graph keeps running as ordinary
PyTorch ops. This module is the same mechanism pointed at the INT8 layers of this library:

    import forge_b200.compile                                   # registers the backends
    fast = torch.compile(model, backend="forge_b200_int8")      # dense W8A8
    fast = torch.compile(model, backend="forge_b200_int8_sparse")   # 2:4 where the shape allows

`apply_int8_patterns(gm)` is the rewrite itself for callers that trace with `torch.fx` directly.
Dynamo only captures the graph; the work runs in `w8a8_linear`, which prepares each weight once
(per-channel quantisation, and 2:4 prune + compress + pack for the sparse backend, one kernel on
the weight's device) and then calls the same `QuantizedLinear` / `SparseLinear` forward as a model
converted by `forge_b200.quant.quantize`. Inference only, like the reference's backend: the
rewritten call has no autograd formula.
"""
import weakref

import torch
import torch.fx as fx
import torch.nn as nn
import torch.nn.functional as F

from .nn import QuantizedLinear, SparseLinear

# prepared layers, keyed by the identity of the weight tensor they were made from
_prepared = {}


def _sparse_ok(weight):
    return weight.is_cuda and weight.shape[1] % 64 == 0 and weight.shape[0] % 16 == 0


def prepared_layer(weight, bias, sparse):
    """The W8A8 layer for `weight` (N, K), built on first use and rebuilt when the weight is
    modified in place (its version counter moves) or replaced."""
    key = (id(weight), bool(sparse))
    hit = _prepared.get(key)
    if hit is not None:
        ref, version, layer = hit
        if ref() is weight and version == weight._version:
            return layer
    n, k = weight.shape
    use_sparse = sparse and _sparse_ok(weight)
    layer = (SparseLinear if use_sparse else QuantizedLinear)(k, n, bias=bias is not None).to(weight.device)
    with torch.no_grad():
        if use_sparse:
            layer.from_dense_weight(weight)
        else:
            layer.quantize_weight(weight)
        if bias is not None:
            layer.bias.data.copy_(bias.detach().to(torch.float16))
    layer.requires_grad_(False)
    _prepared[key] = (weakref.ref(weight, lambda _r, key=key: _prepared.pop(key, None)), weight._version, layer)
    return layer


def w8a8_linear(x, weight, bias=None, sparse=False):
    """`F.linear(x, weight, bias)` on the INT8 path; the result has x's dtype."""
    layer = prepared_layer(weight, bias, sparse)
    with torch.no_grad():
        return layer(x).to(x.dtype)


def _is_linear_module(node, modules):
    return node.op == "call_module" and type(modules.get(node.target)) is nn.Linear


def apply_int8_patterns(gm, sparse=False):
    """Replace every `nn.Linear` module call and every `F.linear` call of `gm` by `w8a8_linear`.
    Returns `gm` (rewritten in place); `gm.forge_b200_replacements` holds the count."""
    graph = gm.graph
    modules = dict(gm.named_modules())
    count = 0
    for node in list(graph.nodes):
        if not node.users:
            continue
        if _is_linear_module(node, modules):
            with graph.inserting_before(node):
                w = graph.get_attr(node.target + ".weight")
                b = graph.get_attr(node.target + ".bias") if modules[node.target].bias is not None else None
                new = graph.call_function(w8a8_linear, args=(node.args[0], w, b, sparse))
        elif node.op == "call_function" and node.target is F.linear:
            args = list(node.args)
            bias = args[2] if len(args) > 2 else node.kwargs.get("bias")
            x = args[0] if args else node.kwargs["input"]
            w = args[1] if len(args) > 1 else node.kwargs["weight"]
            with graph.inserting_before(node):
                new = graph.call_function(w8a8_linear, args=(x, w, bias, sparse))
        else:
            continue
        node.replace_all_uses_with(new)
        graph.erase_node(node)
        count += 1
    if count:
        graph.lint()
        gm.recompile()
    gm.forge_b200_replacements = count
    return gm


def _backend(sparse):
    def compiler(gm: fx.GraphModule, example_inputs):
        return apply_int8_patterns(gm, sparse=sparse)
    return compiler


forge_b200_int8 = _backend(False)
forge_b200_int8_sparse = _backend(True)

try:
    import torch._dynamo as _dynamo
    _dynamo.register_backend(name="forge_b200_int8", compiler_fn=forge_b200_int8)
    _dynamo.register_backend(name="forge_b200_int8_sparse", compiler_fn=forge_b200_int8_sparse)
except ImportError:   # a torch build without Dynamo: the FX entry point still works
    pass
