"""forge_int8_linear_static - the W8A8 linear layer with its scratch inside the library.

Some callers of this library cannot hand over scratch buffers: plug-ins under a host framework
whose allocator owns all GPU memory, or serving loops where a cudaMalloc (which synchronises the
device) is not acceptable. For them the library offers one entry point that allocates nothing
and keeps the int8 activations and token scales in a fixed device array of its own.

This test drives that entry point through the C ABI, twice in a row with different inputs (the
second call must not see anything the first left in the shared array), and requires the output
to equal forge_int8_linear's bit for bit - the same tolerance the other GEMM tests use. It also
checks that over-sized requests are refused. The file sorts last so that a run that stops at the
first failure has already executed every other test."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from forge_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOO_LARGE = 6   # FORGE_B200_TOO_LARGE


def _case(M, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((M, K), generator=g) * (1 + seed % 3)).to(torch.float16).to(DEV)
    w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8).to(DEV)
    w_s = (torch.rand(N, generator=g) * 0.02 + 0.001).to(torch.float16).to(DEV)
    bias = (torch.randn(N, generator=g) * 0.01).to(torch.float16).to(DEV)
    return x, w, w_s, bias


def _reference_linear(x, w, w_s, bias):
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=torch.float16, device=DEV)
    sa = torch.empty((M, K), dtype=torch.int8, device=DEV)
    ss = torch.empty((M,), dtype=torch.float32, device=DEV)
    _lib.call("forge_int8_linear", x.data_ptr(), w.data_ptr(), w_s.data_ptr(), bias.data_ptr(), out.data_ptr(),
              M, K, N, sa.data_ptr(), ss.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return out


def test_static_scratch_linear_matches_int8_linear_twice_in_a_row():
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    # two calls back to back on one stream; the second is smaller, so stale bytes of the first
    # remain in the array beyond what it uses
    for (M, K, N, seed) in [(1024, 4096, 1536, 1), (300, 1024, 528, 2)]:
        x, w, w_s, bias = _case(M, K, N, seed)
        out = torch.full((M, N), 0x7B7B, dtype=torch.int16, device=DEV).view(torch.float16)
        st = lib.forge_int8_linear_static(x.data_ptr(), w.data_ptr(), w_s.data_ptr(), bias.data_ptr(),
                                          out.data_ptr(), M, K, N, stream)
        assert st == 0, lib.forge_b200_status_string(st)
        want = _reference_linear(x, w, w_s, bias)
        torch.cuda.synchronize()
        assert lib.forge_b200_device_status(1) == 0
        assert torch.equal(out.view(torch.int16), want.view(torch.int16))


def test_static_scratch_linear_against_the_cpu_oracle():
    """Independent of forge_int8_linear: the CPU oracle's chain on the same input. The quantized
    values never leave the library here, so the oracle's own quantizer is used; it may differ from
    the GPU's by one int8 step where x / scale falls next to a rounding boundary (IEEE divide against
    the kernels' approximate one), which moves an output by at most (sum of |w|) * scales."""
    lib = _lib.load()
    M, K, N = 96, 512, 160
    x, w, w_s, bias = _case(M, K, N, 4)
    out = torch.empty((M, N), dtype=torch.float16, device=DEV)
    st = lib.forge_int8_linear_static(x.data_ptr(), w.data_ptr(), w_s.data_ptr(), bias.data_ptr(), out.data_ptr(),
                                      M, K, N, torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert lib.forge_b200_device_status(1) == 0
    q, s = O.quantize(x.cpu().numpy())
    want = O.dequantize_bias(O.gemm_s32(q, w.cpu().numpy()), s, w_s.cpu().numpy(), bias.cpu().numpy(),
                             gemm_epilogue=True).astype(np.float32)
    got = out.cpu().numpy().astype(np.float32)
    # bound of one flipped int8 step per activation element: |w|_1 * act_scale * w_scale (+ fp16 rounding)
    slack = (np.abs(w.cpu().numpy().astype(np.float32)).sum(axis=1)[None, :] * s[:, None] *
             w_s.cpu().numpy().astype(np.float32)[None, :])
    assert np.all(np.abs(got - want) <= slack + 2e-3 * np.abs(want) + 1e-3)
    # and in practice almost every output is identical
    assert np.mean(out.cpu().numpy().view(np.uint16) == O.dequantize_bias(
        O.gemm_s32(q, w.cpu().numpy()), s, w_s.cpu().numpy(), bias.cpu().numpy(), gemm_epilogue=True).view(np.uint16)) > 0.9


def test_static_scratch_linear_rejects_oversized_requests():
    lib = _lib.load()
    x, w, w_s, bias = _case(8, 64, 16, 3)
    out = torch.empty((8, 16), dtype=torch.float16, device=DEV)
    args = (x.data_ptr(), w.data_ptr(), w_s.data_ptr(), bias.data_ptr(), out.data_ptr())
    assert lib.forge_int8_linear_static(*args, 4097, 4096, 16, 0) == TOO_LARGE     # M*K > 16 Mi
    assert lib.forge_int8_linear_static(*args, 16385, 64, 16, 0) == TOO_LARGE      # M > 16384
    assert lib.forge_int8_linear_static(*args, 0, 64, 16, 0) == 0                  # empty: no-op
