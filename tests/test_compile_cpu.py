"""Graph rewriting of forge_b200.compile (the INT8 counterpart of the reference's
python/forge/compile/patterns.py:62-128): which nodes are replaced. No kernel runs here."""
import os
import sys

import torch
import torch.fx as fx
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from forge_b200 import compile as fcompile  # noqa: E402


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(64, 128)
        self.b = nn.Linear(128, 32, bias=False)
        self.extra_w = nn.Parameter(torch.randn(16, 32))
        self.norm = nn.LayerNorm(128)

    def forward(self, x):
        h = self.norm(torch.relu(self.a(x)))
        return F.linear(self.b(h), self.extra_w)


def test_every_linear_becomes_a_w8a8_call_and_nothing_else_changes():
    gm = fx.symbolic_trace(Net())
    out = fcompile.apply_int8_patterns(gm, sparse=True)
    assert out is gm and gm.forge_b200_replacements == 3
    calls = [n for n in gm.graph.nodes if n.op == "call_function" and n.target is fcompile.w8a8_linear]
    assert len(calls) == 3
    assert all(c.args[3] is True for c in calls)
    # the module calls kept their weight / bias as get_attr nodes; the bias-free layer passes None
    assert calls[0].args[1].op == "get_attr" and calls[0].args[1].target == "a.weight"
    assert calls[0].args[2].target == "a.bias" and calls[1].args[2] is None
    assert not any(n.op == "call_function" and n.target is F.linear for n in gm.graph.nodes)
    mods = dict(gm.named_modules())
    assert not any(n.op == "call_module" and isinstance(mods[n.target], nn.Linear) for n in gm.graph.nodes)
    # LayerNorm and relu are untouched
    assert sum(1 for n in gm.graph.nodes if n.op == "call_module") == 1


def test_graph_without_linears_is_left_alone():
    class Plain(nn.Module):
        def forward(self, x):
            return torch.relu(x) + 1

    gm = fx.symbolic_trace(Plain())
    code = gm.code
    fcompile.apply_int8_patterns(gm)
    assert gm.forge_b200_replacements == 0 and gm.code == code


def test_backends_are_registered():
    import torch._dynamo as dynamo
    names = dynamo.list_backends(exclude_tags=())
    assert "forge_b200_int8" in names and "forge_b200_int8_sparse" in names
