"""GPU parity at the full sizes of the benchmark configurations, through the C ABI.

  W8A8 linear, 4096 tokens x 4096 -> 4096: FP16 activations ~N(0,1) with 1 % of the input channels
      scaled x20 (outlier columns), per-channel INT8 weights from ~N(0,0.02) floats, FP16 bias.
  W8A8 gated MLP block, 8192 tokens, 4096 -> 14336 -> 4096, dense and 2:4-sparse weights.
  One rank's share of the sharded 2:4-sparse layer: 8192 of the 65536 tokens, K = 8192, N = 28672.

Checks that do not depend on the size: the quantizer output is compared in full against the
standalone quantizer (and the reference's kernel); GEMM outputs are compared in full, bit for bit,
against the reference's own kernels (src/gemm/int8_dense.cu:213-232, src/gemm/int8_sparse.cu:1005-1043)
and on sampled token rows against the CPU oracle (exact int32 accumulation + the GEMM epilogue's
operation order). The gated block uses the stage checks of test_gated_mlp_gpu.py: h within 1 fp16
ulp of the fp64 composition, everything downstream of the GPU's own h bit-exact."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from forge_b200 import _forge_C as C
from forge_b200 import _lib
from forge_b200.nn import quantize_weight_per_channel

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _status_ok():
    torch.cuda.synchronize()
    assert C.device_status() == 0, "a kernel reported a timed-out wait"


def _sample_rows(M, n=8, seed=0):
    rows = sorted(set([0, 1, M // 2 - 1, M // 2, M - 2, M - 1] +
                      np.random.default_rng(seed).integers(0, M, n).tolist()))
    return rows


def _compress(W):
    N, K = W.shape
    comp = torch.empty((N, K // 2), dtype=torch.int8, device=DEV)
    raw = torch.empty((N * (K // 4),), dtype=torch.uint8, device=DEV)
    meta = torch.empty((N, K // 32), dtype=torch.int32, device=DEV)
    C.prune_compress_24(W, comp, raw, N, K)
    C.pack_metadata(raw, meta, N, K)
    return comp, meta


def test_w8a8_linear_4096_with_outlier_channels():
    M = K = N = 4096
    g = torch.Generator(device=DEV).manual_seed(2)
    x = torch.randn((M, K), generator=g, device=DEV)
    cols = torch.randperm(K, generator=torch.Generator().manual_seed(7))[:K // 100 + 1]   # 41 outlier columns
    assert len(cols) == 41
    x[:, cols.to(DEV)] *= 20.0
    x = x.to(torch.float16)
    w_int8, w_scale = quantize_weight_per_channel(torch.randn((N, K), generator=g, device=DEV) * 0.02)
    bias = (torch.randn(N, generator=g, device=DEV) * 0.01).to(torch.float16)
    sa = torch.empty((M, K), dtype=torch.int8, device=DEV)
    ss = torch.empty((M,), dtype=torch.float32, device=DEV)
    out = C.int8_linear(x, w_int8, w_scale, bias, sa, ss)
    _status_ok()
    # the quantized activations are what the standalone quantizer gives, and they use the full int8 range
    q, s = C.fused_quantize_activation(x, M, K)
    assert torch.equal(q, sa) and torch.equal(s, ss)
    assert int(sa.abs().max()) == 127
    # sampled rows against the CPU oracle (exact s32 GEMM + the GEMM epilogue's association)
    rows = _sample_rows(M, 24)
    acc = O.gemm_s32(sa[rows].cpu().numpy(), w_int8.cpu().numpy())
    want = O.dequantize_bias(acc, ss[rows].cpu().numpy(), w_scale.cpu().numpy(), bias.cpu().numpy(), gemm_epilogue=True)
    assert np.array_equal(out[rows].cpu().numpy().view(np.uint16), want.view(np.uint16))
    # the CPU quantizer restatement agrees to one int8 step (its divide is IEEE, the kernels' is approximate)
    q_cpu, s_cpu = O.quantize(x[rows].cpu().numpy())
    assert np.abs(q_cpu.astype(np.int32) - sa[rows].cpu().numpy().astype(np.int32)).max() <= 1
    np.testing.assert_allclose(ss[rows].cpu().numpy(), s_cpu, rtol=1e-6)
    # the whole output, scratch included, bit for bit against the reference's int8_linear
    if O.require_ref():
        ref = torch.empty_like(out)
        sa2, ss2 = torch.empty_like(sa), torch.empty_like(ss)
        O.ref().ref_int8_linear(x.data_ptr(), w_int8.data_ptr(), w_scale.data_ptr(), bias.data_ptr(), ref.data_ptr(),
                                M, K, N, sa2.data_ptr(), ss2.data_ptr(), O.cur_stream())
        torch.cuda.synchronize()
        assert torch.equal(sa, sa2) and torch.equal(ss, ss2)
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16))


@pytest.mark.parametrize("sparse", [False, True])
def test_gated_mlp_block_8192_tokens_full_size(sparse):
    lib = _lib.load()
    M, d_model, d_ffn = 8192, 4096, 14336
    g = torch.Generator(device=DEV).manual_seed(41)
    x = torch.randn((M, d_model), generator=g, device=DEV).to(torch.float16)

    def weight(n, k):
        wq, ws = quantize_weight_per_channel(torch.randn((n, k), generator=g, device=DEV) * 0.02)
        return wq, ws, (torch.randn(n, generator=g, device=DEV) * 0.05).to(torch.float16)

    (Wg, sg, bg), (Wu, su, bu), (Wd, sd, bd) = weight(d_ffn, d_model), weight(d_ffn, d_model), weight(d_model, d_ffn)
    nbytes = lib.forge_w8a8_gated_mlp_workspace_bytes(M, d_model, d_ffn)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    out = torch.full((M, d_model), 0x7B7B, dtype=torch.int16, device=DEV).view(torch.float16)
    scales_biases = [t.data_ptr() for t in (sg, su, sd, bg, bu, bd)]
    if sparse:
        (cg, mg), (cu, mu), (cd, md) = _compress(Wg), _compress(Wu), _compress(Wd)
        _lib.call("forge_sparse_w8a8_gated_mlp", x.data_ptr(), cg.data_ptr(), mg.data_ptr(), cu.data_ptr(),
                  mu.data_ptr(), cd.data_ptr(), md.data_ptr(), *scales_biases, out.data_ptr(), M, d_model, d_ffn,
                  ws.data_ptr(), 0)
        Wg_e, Wu_e, Wd_e = (O.prune_24_dense(w.cpu().numpy()) for w in (Wg, Wu, Wd))
    else:
        _lib.call("forge_w8a8_gated_mlp", x.data_ptr(), Wg.data_ptr(), Wu.data_ptr(), Wd.data_ptr(), *scales_biases,
                  out.data_ptr(), M, d_model, d_ffn, ws.data_ptr(), 0)
        Wg_e, Wu_e, Wd_e = (w.cpu().numpy() for w in (Wg, Wu, Wd))
    _status_ok()
    pad = lambda n: (n + 255) & ~255
    o = 0
    xq = ws[o:o + M * d_model].view(torch.int8).view(M, d_model); o += pad(M * d_model)
    xs = ws[o:o + 4 * M].view(torch.float32); o += pad(4 * M)
    h = ws[o:o + 2 * M * d_ffn].view(torch.float16).view(M, d_ffn); o += pad(2 * M * d_ffn)
    hq = ws[o:o + M * d_ffn].view(torch.int8).view(M, d_ffn); o += pad(M * d_ffn)
    hs = ws[o:o + 4 * M].view(torch.float32); o += pad(4 * M)
    assert o == nbytes
    # stages 1 and 3 in full: both quantizations are the standalone quantizer's, bit for bit
    q1, s1 = C.fused_quantize_activation(x, M, d_model)
    assert torch.equal(q1, xq) and torch.equal(s1, xs)
    q2, s2 = C.fused_quantize_activation(h, M, d_ffn)
    assert torch.equal(q2, hq) and torch.equal(s2, hs)
    # stages 2 and 4 on sampled token rows
    rows = _sample_rows(M, 4, seed=3)
    xq_r, xs_r = xq[rows].cpu().numpy(), xs[rows].cpu().numpy()
    want_h = O.gated_epilogue(O.gemm_s32(xq_r, Wg_e), O.gemm_s32(xq_r, Wu_e), xs_r, sg.cpu().numpy(),
                              su.cpu().numpy(), bg.cpu().numpy(), bu.cpu().numpy())
    assert O.half_ulp_distance(h[rows].cpu().numpy(), want_h).max() <= 1     # tolerance: 1 fp16 ulp
    want_out = O.dequantize_bias(O.gemm_s32(hq[rows].cpu().numpy(), Wd_e), hs[rows].cpu().numpy(), sd.cpu().numpy(),
                                 bd.cpu().numpy(), gemm_epilogue=True)
    assert np.array_equal(out[rows].cpu().numpy().view(np.uint16), want_out.view(np.uint16))
    # a second call on the same inputs reproduces every byte of the output
    out2 = torch.empty_like(out)
    args = (cg, mg, cu, mu, cd, md) if sparse else (Wg, Wu, Wd)
    _lib.call("forge_sparse_w8a8_gated_mlp" if sparse else "forge_w8a8_gated_mlp", x.data_ptr(),
              *[t.data_ptr() for t in args], *scales_biases, out2.data_ptr(), M, d_model, d_ffn, ws.data_ptr(), 0)
    _status_ok()
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))


def test_one_rank_share_of_the_sharded_sparse_layer():
    """8192 of the 65536 token rows (what one of eight ranks computes under token-row sharding),
    K = 8192, N = 28672, 2:4-pruned uniform int8 weights."""
    M, K, N = 8192, 8192, 28672
    g = torch.Generator(device=DEV).manual_seed(55)
    W = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8, device=DEV)
    comp, meta = _compress(W)
    w_scale = (torch.rand(N, generator=g, device=DEV) * 0.01 + 0.001).to(torch.float16)
    bias = (torch.randn(N, generator=g, device=DEV) * 0.05).to(torch.float16)
    x = torch.randn((M, K), generator=g, device=DEV).to(torch.float16)
    sq = torch.empty((M, K), dtype=torch.int8, device=DEV)
    ss = torch.empty((M,), dtype=torch.float32, device=DEV)
    out = C.sparse_int8_linear(x, comp, meta, w_scale, bias, sq, ss)
    _status_ok()
    rows = _sample_rows(M, 2, seed=5)
    W_pruned = O.prune_24_dense(W.cpu().numpy())
    del W
    acc = O.gemm_s32(sq[rows].cpu().numpy(), W_pruned)
    want = O.dequantize_bias(acc, ss[rows].cpu().numpy(), w_scale.cpu().numpy(), bias.cpu().numpy(), gemm_epilogue=True)
    assert np.array_equal(out[rows].cpu().numpy().view(np.uint16), want.view(np.uint16))
    # column checksum of the raw accumulators over all 8192 rows, exact in int64
    acc_gpu = C.sparse_int8_gemm_s32(comp, sq, meta)
    _status_ok()
    col_sum = acc_gpu.sum(dim=0, dtype=torch.int64)
    del acc_gpu
    x_sum = sq.sum(dim=0, dtype=torch.int64).double()
    want_sum = (torch.from_numpy(W_pruned).to(DEV).double() @ x_sum).round().long()
    assert torch.equal(col_sum, want_sum)
    if O.require_ref():
        ref = torch.empty_like(out)
        sq2, ss2 = torch.empty_like(sq), torch.empty_like(ss)
        # split_k = 1 and no workspace: the reference's deterministic path
        O.ref().ref_sparse_int8_linear(x.data_ptr(), comp.data_ptr(), meta.data_ptr(), w_scale.data_ptr(),
                                       bias.data_ptr(), ref.data_ptr(), M, K, N, sq2.data_ptr(), ss2.data_ptr(), 0, 1,
                                       O.cur_stream(), -1)
        torch.cuda.synchronize()
        assert torch.equal(sq, sq2) and torch.equal(ss, ss2)
        assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
