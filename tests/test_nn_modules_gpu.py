"""The drop-in modules (forge_b200.nn / forge_b200.quant) on a GPU: conversion of a small
nn.Module, state_dict round trip with the reference's buffer names and dtypes, agreement with
the C-ABI calls they wrap (bit-exact) and with the fp16 model (loosely: it is a quantised model)."""
import io

import numpy as np
import pytest
import torch
import torch.nn as nn

import oracle_lib as O
from forge_b200 import _forge_C as C
from forge_b200.nn import QuantizedLinear, SparseLinear, quantize_weight_per_channel
from forge_b200.quant import quantize

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class TinyMLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.up = nn.Linear(256, 512)
        self.act = nn.SiLU()
        self.down = nn.Linear(512, 256, bias=False)

    def forward(self, x):
        return self.down(self.act(self.up(x)))


def test_quantized_linear_matches_cabi_and_oracle():
    torch.manual_seed(0)
    lin = nn.Linear(384, 272).to(DEV).half()
    q = QuantizedLinear(384, 272).to(DEV)
    q.quantize_weight(lin.weight.data)
    q.bias.data.copy_(lin.bias.data)
    x = torch.randn(5, 7, 384, device=DEV, dtype=torch.float16)      # extra leading dimension
    y = q(x)
    assert y.shape == (5, 7, 272)
    x2 = x.reshape(-1, 384)
    xq, xs = C.fused_quantize_activation(x2, 35, 384)
    want = O.dequantize_bias(O.gemm_s32(xq.cpu().numpy(), q.w_int8.cpu().numpy()), xs.cpu().numpy(),
                             q.w_scale.detach().cpu().numpy(), q.bias.detach().cpu().numpy(), gemm_epilogue=True)
    assert np.array_equal(y.reshape(-1, 272).detach().cpu().numpy().view(np.uint16), want.view(np.uint16))
    # close to the fp16 layer it replaces
    ref = lin(x)
    assert (y - ref).abs().max() < 0.05 * ref.abs().max() + 0.05
    # weight recipe: absmax/127, round half even, clamp +-127
    wq, ws = quantize_weight_per_channel(lin.weight.data.cpu())
    assert torch.equal(wq.to(DEV), q.w_int8) and int(wq.abs().max()) == 127


def test_backward_of_quantized_linear_runs():
    q = QuantizedLinear(128, 64).to(DEV)
    q.quantize_weight(torch.randn(64, 128))
    x = torch.randn(16, 128, device=DEV, dtype=torch.float16, requires_grad=True)
    q(x).float().sum().backward()
    assert x.grad is not None and x.grad.shape == x.shape and q.bias.grad.shape == (64,)


def test_sparse_linear_and_state_dict_round_trip():
    torch.manual_seed(1)
    w = torch.randn(208, 192)
    s = SparseLinear(192, 208).to(DEV)
    s.from_dense_weight(w)
    sd = s.state_dict()
    assert set(sd) == {"W_comp", "w_meta", "w_scale", "bias"}
    assert sd["W_comp"].dtype == torch.int8 and sd["W_comp"].shape == (208, 96)
    assert sd["w_meta"].dtype == torch.int32 and sd["w_meta"].shape == (208, 6)
    assert sd["w_scale"].dtype == torch.float16
    # compressed form equals the oracle's prune/compress/pack of the quantised weight
    wq, _ = quantize_weight_per_channel(w)        # on the CPU: IEEE arithmetic
    comp, raw = O.prune_compress_24(wq.numpy())
    assert np.array_equal(sd["W_comp"].cpu().numpy(), comp)
    assert np.array_equal(sd["w_meta"].cpu().numpy().view(np.uint32), O.pack_metadata(raw, 208, 192))
    buf = io.BytesIO()
    torch.save(sd, buf)
    buf.seek(0)
    s2 = SparseLinear(192, 208).to(DEV)
    s2.load_state_dict(torch.load(buf))
    x = torch.randn(37, 192, device=DEV, dtype=torch.float16)
    assert torch.equal(s(x), s2(x))
    qd = QuantizedLinear(192, 208).state_dict()
    assert set(qd) == {"w_int8", "w_scale", "bias"} and qd["w_int8"].dtype == torch.int8


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("N,K", [(208, 192), (33, 64), (1000, 4096)])
def test_one_pass_weight_preparation_equals_the_torch_recipe(dtype, N, K):
    """forge_prepare_weight against the reference's recipe (torch per-channel quantisation, then
    prune_compress_24 + pack_metadata), bit for bit."""
    g = torch.Generator().manual_seed(N + K)
    w = (torch.randn((N, K), generator=g) * 0.02).to(dtype)
    w[0] = 0                      # an all-zero channel exercises the 1e-8 floor
    w[1, :8] = w[1, 8]            # ties inside groups
    # the recipe with IEEE arithmetic = torch on the CPU (torch's CUDA kernels replace the division
    # by the scalar 127 with a multiplication by its reciprocal, which moves some scales by one ulp)
    wq, ws = quantize_weight_per_channel(w)
    wq, ws = wq.to(DEV), ws.to(DEV)
    q_dense, _, _, s_dense = C.prepare_weight(w.to(DEV), sparse=False)
    assert torch.equal(q_dense, wq) and torch.equal(s_dense.view(torch.int16), ws.view(torch.int16))
    _, comp, meta, s_sparse = C.prepare_weight(w.to(DEV), sparse=True)
    comp_cpu, raw_cpu = O.prune_compress_24(wq.cpu().numpy())
    assert np.array_equal(comp.cpu().numpy(), comp_cpu)
    assert np.array_equal(meta.cpu().numpy().view(np.uint32), O.pack_metadata(raw_cpu, N, K))
    assert torch.equal(s_sparse.view(torch.int16), ws.view(torch.int16))


@pytest.mark.parametrize("sparse", [False, True])
def test_quantize_converts_a_model(sparse):
    torch.manual_seed(2)
    model = TinyMLP().to(DEV).half()
    qmodel = quantize(model, sparse=sparse, verbose=False)
    kinds = {type(m).__name__ for m in qmodel.modules()}
    assert "Linear" not in kinds and (("SparseLinear" in kinds) == sparse)
    assert isinstance(model.up, nn.Linear), "the input model must be left untouched"
    x = torch.randn(64, 256, device=DEV, dtype=torch.float16)
    y, ref = qmodel(x), model(x)
    assert y.shape == ref.shape and torch.isfinite(y).all()
    if not sparse:
        assert (y - ref).abs().max() < 0.1 * ref.abs().max() + 0.05


def _make_pair():
    torch.manual_seed(3)
    w = torch.randn(256, 512)
    dense = QuantizedLinear(512, 256).to(DEV)
    dense.quantize_weight(w)
    sparse = SparseLinear(512, 256).to(DEV)
    sparse.from_dense_weight(w)
    dense.bias.data.normal_(0, 0.01)
    sparse.bias.data.copy_(dense.bias.data)
    return dense, sparse


def test_modules_capture_into_a_cuda_graph():
    """After one warm-up call (scratch allocated, kernels configured) the forward of both modules is a
    fixed sequence of launches on the current stream: it captures into a CUDA graph and the replay on
    new input values gives the eager result."""
    dense, sparse = _make_pair()
    for mod in (dense, sparse):
        mod.eval()
        x = torch.randn(48, 512, device=DEV, dtype=torch.float16)
        with torch.no_grad():
            mod(x)                                   # warm-up
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    y = mod(x)
            torch.cuda.current_stream().wait_stream(side)
            x.copy_(torch.randn(48, 512, device=DEV, dtype=torch.float16) * 3)
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(y, mod(x))
    assert C.device_status() == 0


def test_modules_accept_non_contiguous_and_wider_dtypes():
    dense, sparse = _make_pair()
    big = torch.randn(40, 1024, device=DEV, dtype=torch.float16)
    strided = big[:, ::2]                            # every other column: row stride 1024, element stride 2
    transposed = torch.randn(512, 40, device=DEV, dtype=torch.float16).t()
    with torch.no_grad():
        for mod in (dense, sparse):
            assert torch.equal(mod(strided), mod(strided.contiguous()))
            assert torch.equal(mod(transposed), mod(transposed.contiguous()))
            x32 = torch.randn(8, 512, device=DEV)    # fp32 input is converted to fp16 first
            assert torch.equal(mod(x32), mod(x32.half()))


def test_scratch_buffers_follow_the_batch_size():
    dense, sparse = _make_pair()
    with torch.no_grad():
        for mod in (dense, sparse):
            outs = {}
            for m in (4, 64, 16, 200, 4):            # grows, shrinks, grows past the first allocation
                x = torch.randn(m, 512, device=DEV, dtype=torch.float16)
                outs[m] = (x, mod(x).clone())
            fresh_dense, fresh_sparse = _make_pair()
            fresh = fresh_dense if isinstance(mod, QuantizedLinear) else fresh_sparse
            for m, (x, y) in outs.items():
                assert torch.equal(fresh(x), y)


class _FakeQuantWrapped(nn.Module):
    """The attribute layout of the reference's QAT wrapper (python/forge/quant/convert.py:123-160): a float
    `linear` plus `weight_fq` / `input_fq` modules; finalize_qat recognises it by that shape."""

    def __init__(self, linear):
        super().__init__()
        self.linear, self.weight_fq, self.input_fq = linear, nn.Identity(), nn.Identity()

    def forward(self, x):
        return nn.functional.linear(self.input_fq(x), self.weight_fq(self.linear.weight), self.linear.bias)


def test_static_scheme_calibration_and_qat_finalization_on_the_gpu():
    """quantize(model, data, scheme="static_int8") runs the calibration batches through the converted
    model (the reference's call shape), and finalize_qat turns fake-quantize wrappers around trained
    float layers into layers whose output equals a direct conversion of the same float weights."""
    from forge_b200 import quant as Q
    torch.manual_seed(4)
    model = TinyMLP().to(DEV).half()
    data = [torch.randn(8, 256, device=DEV, dtype=torch.float16) for _ in range(3)]
    q_static = Q.quantize(model, data, 2, "static_int8", verbose=False)
    q_dyn = Q.quantize(model, verbose=False)
    x = torch.randn(16, 256, device=DEV, dtype=torch.float16)
    with torch.no_grad():
        assert torch.equal(q_static(x), q_dyn(x))
    import copy
    qat = copy.deepcopy(model).float()
    for name, child in list(qat.named_children()):
        if isinstance(child, nn.Linear):
            setattr(qat, name, _FakeQuantWrapped(child))
    qat(x.float()).sum().backward()
    final = Q.finalize_qat(qat, verbose=False)
    with torch.no_grad():
        assert torch.equal(final(x), q_dyn(x))


@pytest.mark.parametrize("in_features", [48, 100])
def test_quantize_accepts_any_in_features_on_the_gpu(in_features):
    """The reference's quantize_weight takes any K (python/forge/nn/linear.py:167-173); widths that are not
    a multiple of 32 take the torch recipe on the device instead of the one-pass kernel, and the layer then
    runs on the ragged-shape GEMM path."""
    from forge_b200 import quant as Q
    torch.manual_seed(in_features)
    net = nn.Sequential(nn.Linear(in_features, 24)).to(DEV)
    q = Q.quantize(net, verbose=False)
    assert isinstance(q[0], QuantizedLinear)
    wq, ws = quantize_weight_per_channel(net[0].weight.data)           # the recipe, on the weight's device
    assert torch.equal(q[0].w_int8, wq) and torch.equal(q[0].w_scale.data, ws)
    wq_cpu, _ = quantize_weight_per_channel(net[0].weight.data.cpu())  # CPU arithmetic: at most one step apart
    assert (q[0].w_int8.cpu().int() - wq_cpu.int()).abs().max() <= 1
    x = torch.randn(9, in_features, device=DEV, dtype=torch.float16)
    with torch.no_grad():
        y = q(x)
    torch.cuda.synchronize()
    xq, xs = C.fused_quantize_activation(x, 9, in_features)
    want = O.dequantize_bias(O.gemm_s32(xq.cpu().numpy(), q[0].w_int8.cpu().numpy()), xs.cpu().numpy(),
                             q[0].w_scale.data.cpu().numpy(), q[0].bias.data.cpu().numpy(), gemm_epilogue=True)
    assert np.array_equal(y.cpu().numpy().view(np.uint16), want.view(np.uint16))
