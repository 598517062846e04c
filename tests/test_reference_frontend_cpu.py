"""The reference's own Python front end, unchanged, on top of this library's binding module.

The reference's layers do `from forge import _forge_C as _C` (python/forge/nn/linear.py:10). Here
a two-entry stand-in package `forge` is put into sys.modules whose `_forge_C` is
`forge_b200._forge_C`, and the reference's linear.py / quant/*.py are loaded from the reference
source tree with importlib, byte for byte as they are. Checked without a GPU:

  - every call the reference modules make into `_C` binds to the signature of the function of the
    same name in forge_b200._forge_C (a recorder stands in for the GPU work and validates the
    argument list, dtypes and shapes);
  - the reference's QuantizedLinear / SparseLinear and forge_b200.nn's have interchangeable
    state_dicts (same keys, dtypes, shapes; strict loading both ways) and the same weight
    quantisation, bit for bit;
  - forge_b200.quant.finalize_qat converts a model prepared by the reference's prepare_qat.

The numerics of the functions behind those calls are covered by the GPU tests of
forge_b200._forge_C. The reference tree is read where it lies and is not needed on a GPU box:
without it this file skips."""
import importlib.util
import inspect
import os
import sys
import types

import pytest
import torch
import torch.nn as nn

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
import build as oracle_build  # noqa: E402

from forge_b200 import _forge_C as real_C  # noqa: E402
from forge_b200 import nn as fb_nn  # noqa: E402
from forge_b200 import quant as fb_quant  # noqa: E402

REF_PY = os.path.join(oracle_build.REFERENCE_ROOT, "python", "forge")
pytestmark = pytest.mark.skipif(not os.path.exists(os.path.join(REF_PY, "nn", "linear.py")),
                                reason="reference source tree not present")


class Recorder:
    """Stands in for forge_b200._forge_C on a machine without a GPU: every call is bound against the
    real function's signature (a TypeError here = the reference's call would not fit), recorded, and
    answered with a tensor of the documented shape and dtype."""

    def __init__(self):
        self.calls = []

    def __getattr__(self, name):
        real = getattr(real_C, name)          # AttributeError if this library lacks the binding

        def fake(*args, **kwargs):
            bound = inspect.signature(real).bind(*args, **kwargs)
            bound.apply_defaults()
            self.calls.append((name, bound.arguments))
            a = bound.arguments
            if name == "int8_linear":
                return torch.zeros((a["x"].shape[0], a["w_int8"].shape[0]), dtype=torch.float16)
            if name == "sparse_int8_linear":
                return torch.zeros((a["x"].shape[0], a["W_comp"].shape[0]), dtype=torch.float16)
            return None
        return fake


@pytest.fixture()
def reference_forge():
    """The reference's linear.py and quant package loaded under the names they expect."""
    saved = {k: v for k, v in sys.modules.items() if k == "forge" or k.startswith("forge.")}
    for k in saved:
        del sys.modules[k]
    rec = Recorder()
    pkg = types.ModuleType("forge")
    pkg.__path__ = []
    pkg._forge_C = rec
    sys.modules["forge"] = pkg
    sys.modules["forge._forge_C"] = rec

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(REF_PY, rel))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod

    linear = load("forge.nn.linear", os.path.join("nn", "linear.py"))
    fnn = types.ModuleType("forge.nn")
    fnn.__path__ = []
    fnn.QuantizedLinear, fnn.SparseLinear, fnn.Linear = linear.QuantizedLinear, linear.SparseLinear, linear.Linear
    fnn.Embedding = nn.Embedding            # convert.py only instantiates it for nn.Embedding layers
    sys.modules["forge.nn"] = fnn
    pkg.nn = fnn
    qpkg = types.ModuleType("forge.quant")
    qpkg.__path__ = []
    sys.modules["forge.quant"] = qpkg
    load("forge.quant.observers", os.path.join("quant", "observers.py"))
    load("forge.quant.fake_quantize", os.path.join("quant", "fake_quantize.py"))
    convert = load("forge.quant.convert", os.path.join("quant", "convert.py"))
    try:
        yield types.SimpleNamespace(linear=linear, convert=convert, rec=rec)
    finally:
        for k in [k for k in sys.modules if k == "forge" or k.startswith("forge.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_reference_quantized_linear_calls_fit_and_state_dicts_interchange(reference_forge):
    ref = reference_forge
    torch.manual_seed(0)
    w = torch.randn(24, 48) * 0.05
    theirs = ref.linear.QuantizedLinear(48, 24, bias=True)
    ours = fb_nn.QuantizedLinear(48, 24, bias=True)
    theirs.quantize_weight(w)
    ours.quantize_weight(w)
    assert torch.equal(theirs.w_int8, ours.w_int8) and torch.equal(theirs.w_scale, ours.w_scale)
    sd_t, sd_o = theirs.state_dict(), ours.state_dict()
    assert list(sd_t) == list(sd_o)
    for k in sd_t:
        assert sd_t[k].dtype == sd_o[k].dtype and sd_t[k].shape == sd_o[k].shape
    ours.load_state_dict(sd_t, strict=True)
    theirs.load_state_dict(sd_o, strict=True)
    # the reference forward: its call into _C binds to this library's int8_linear
    x = torch.randn(5, 48).to(torch.float16)
    y = theirs(x)
    assert y.shape == (5, 24) and y.dtype == torch.float16
    name, a = ref.rec.calls[-1]
    assert name == "int8_linear"
    assert a["x"] is x and a["w_int8"].dtype == torch.int8 and a["w_scale"].dtype == torch.float16
    assert a["scratch_a_int8"].shape == (5, 48) and a["scratch_a_int8"].dtype == torch.int8
    assert a["scratch_a_scale"].shape == (5,) and a["scratch_a_scale"].dtype == torch.float32


def test_reference_sparse_linear_calls_fit_and_state_dicts_interchange(reference_forge):
    ref = reference_forge
    theirs = ref.linear.SparseLinear(128, 32, bias=False)
    ours = fb_nn.SparseLinear(128, 32, bias=False)
    sd_t, sd_o = theirs.state_dict(), ours.state_dict()
    assert list(sd_t) == list(sd_o)
    for k in sd_t:
        assert sd_t[k].dtype == sd_o[k].dtype and sd_t[k].shape == sd_o[k].shape
    ours.load_state_dict(sd_t, strict=True)
    theirs.load_state_dict(sd_o, strict=True)
    x = torch.randn(3, 128).to(torch.float16)
    y = theirs(x)
    assert y.shape == (3, 32)
    name, a = ref.rec.calls[-1]
    assert name == "sparse_int8_linear"
    assert a["w_meta"].dtype == torch.int32 and a["W_comp"].shape == (32, 64)
    assert a["splitk_workspace"] is None and a["split_k"] == 0 and a["bias"] is None   # linear.py:186-189
    # the two packing calls of from_dense_weight (linear.py:243-244) exist with the argument lists it uses
    for fn, n_args in (("prune_compress_24", 5), ("pack_metadata", 4)):
        assert len(inspect.signature(getattr(real_C, fn)).parameters) == n_args


def test_reference_quantize_and_qat_round_trip_end_in_interchangeable_layers(reference_forge, capsys):
    ref = reference_forge
    torch.manual_seed(1)
    net = nn.Sequential(nn.Linear(32, 64), nn.ReLU(), nn.Linear(64, 16, bias=False))
    q_ref = ref.convert.quantize(net)
    q_ours = fb_quant.quantize(net, verbose=False)
    for a, b in zip(q_ref.state_dict().items(), q_ours.state_dict().items()):
        assert a[0] == b[0] and torch.equal(a[1], b[1])
    # a model prepared by the reference's QAT wrapper is finalized by this library's finalize_qat
    qat = ref.convert.prepare_qat(net)
    assert type(qat[0]).__name__ == "_QATLinearWrapper"
    final = fb_quant.finalize_qat(qat, verbose=False)
    assert isinstance(final[0], fb_nn.QuantizedLinear) and isinstance(final[2], fb_nn.QuantizedLinear)
    for a, b in zip(final.state_dict().items(), q_ours.state_dict().items()):
        assert a[0] == b[0] and torch.equal(a[1], b[1])
    capsys.readouterr()
