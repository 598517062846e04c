"""GPU parity of the gated-MLP path (W8A8 Llama-style MLP block: per-token quantize -> INT8 GEMM gate & up
-> dequant + SiLU(gate)*up fused in the epilogue -> re-quantize -> INT8 GEMM down -> dequant),
dense and 2:4-sparse, through the C ABI.

The reference has no gated epilogue, so the oracle is the composition defined in
oracle/forge_oracle.c: g and u are dequantised in fp32 exactly as the GEMM epilogue does (bit
reproducible on the CPU), SiLU(g)*u is evaluated in double and rounded once to fp16. The GPU
evaluates SiLU in fp32 with approximate exp/divide, so h is required to be within 1 fp16 ulp of
that; everything downstream of the GPU's own h (re-quantize, down GEMM, dequant) is required to be
bit-exact, and the sparse kernels must agree bit for bit with the dense kernel run on the
zero-filled pruned weights."""

import numpy as np
import pytest
import torch

import oracle_lib as O
from forge_b200 import _forge_C as C
from forge_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _weights(N, K, g, dev=True):
    W = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    s = (torch.rand(N, generator=g) * 0.004 + 0.0005).to(torch.float16)
    b = (torch.randn(N, generator=g) * 0.05).to(torch.float16)
    return W, s, b


def _compress(W):
    N, K = W.shape
    comp = torch.empty((N, K // 2), dtype=torch.int8, device=DEV)
    raw = torch.empty((N * (K // 4),), dtype=torch.uint8, device=DEV)
    meta = torch.empty((N, K // 32), dtype=torch.int32, device=DEV)
    C.prune_compress_24(W.to(DEV), comp, raw, N, K)
    C.pack_metadata(raw, meta, N, K)
    return comp, meta


def _status_ok():
    torch.cuda.synchronize()
    assert C.device_status() == 0


def _gated_dense(xq, xs, Wg, Wu, sg, su, bg, bu):
    M, K = xq.shape
    N = Wg.shape[0]
    h = torch.full((M, N), 0x7B7B, dtype=torch.int16, device=DEV).view(torch.float16)
    _lib.call("forge_int8_gated_gemm", xq.data_ptr(), Wg.data_ptr(), Wu.data_ptr(), xs.data_ptr(), sg.data_ptr(),
              su.data_ptr(), 0 if bg is None else bg.data_ptr(), 0 if bu is None else bu.data_ptr(), h.data_ptr(),
              M, K, N, 0)
    return h


def _gated_sparse(xq, xs, cg, mg, cu, mu, sg, su, bg, bu):
    M, K = xq.shape
    N = cg.shape[0]
    h = torch.full((M, N), 0x7B7B, dtype=torch.int16, device=DEV).view(torch.float16)
    _lib.call("forge_sparse_int8_gated_gemm", cg.data_ptr(), mg.data_ptr(), cu.data_ptr(), mu.data_ptr(),
              xq.data_ptr(), xs.data_ptr(), sg.data_ptr(), su.data_ptr(), 0 if bg is None else bg.data_ptr(),
              0 if bu is None else bu.data_ptr(), h.data_ptr(), M, K, N, 0)
    return h


@pytest.mark.parametrize("M,K,N", [(256, 512, 384), (300, 640, 272), (37, 256, 200), (1024, 1024, 1024),
                                   (2050, 512, 400)])
@pytest.mark.parametrize("with_bias", [True, False])
def test_gated_gemm_dense_and_sparse(M, K, N, with_bias):
    g = torch.Generator().manual_seed(5 + M + K + N)
    xq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    xs = (torch.rand(M, generator=g) * 0.02 + 0.001).float()
    Wg, sg, bg = _weights(N, K, g)
    Wu, su, bu = _weights(N, K, g)
    if not with_bias:
        bg = bu = None
    d = lambda t: None if t is None else t.to(DEV)
    dxq, dxs, dsg, dsu, dbg, dbu = d(xq), d(xs), d(sg), d(su), d(bg), d(bu)
    # dense
    h = _gated_dense(dxq, dxs, d(Wg), d(Wu), dsg, dsu, dbg, dbu)
    _status_ok()
    want = O.gated_epilogue(O.gemm_s32(xq.numpy(), Wg.numpy()), O.gemm_s32(xq.numpy(), Wu.numpy()), xs.numpy(),
                            sg.numpy(), su.numpy(), None if bg is None else bg.numpy(),
                            None if bu is None else bu.numpy())
    assert O.half_ulp_distance(h.cpu().numpy(), want).max() <= 1
    # the CTA-pair form of the gated kernel (tile id 512) must give the same bits as the single-CTA one
    _lib.load().forge_b200_set_dense_tile(512)
    try:
        h_pair = _gated_dense(dxq, dxs, d(Wg), d(Wu), dsg, dsu, dbg, dbu)
        _status_ok()
    finally:
        _lib.load().forge_b200_set_dense_tile(0)
    assert torch.equal(h_pair.view(torch.int16), h.view(torch.int16))
    # sparse: vs the oracle on the pruned weights, and bit-identical to the dense kernel on them
    cg, mg = _compress(Wg)
    cu, mu = _compress(Wu)
    Wg_p, Wu_p = O.prune_24_dense(Wg.numpy()), O.prune_24_dense(Wu.numpy())
    for knob in ([0, 128, 1224] if M >= 256 else [0, 32]):
        _lib.load().forge_b200_set_sparse_tile(knob)
        try:
            hs = _gated_sparse(dxq, dxs, cg, mg, cu, mu, dsg, dsu, dbg, dbu)
            _status_ok()
        finally:
            _lib.load().forge_b200_set_sparse_tile(0)
        want_s = O.gated_epilogue(O.gemm_s32(xq.numpy(), Wg_p), O.gemm_s32(xq.numpy(), Wu_p), xs.numpy(), sg.numpy(),
                                  su.numpy(), None if bg is None else bg.numpy(), None if bu is None else bu.numpy())
        assert O.half_ulp_distance(hs.cpu().numpy(), want_s).max() <= 1, f"knob {knob}"
        h_dense_pruned = _gated_dense(dxq, dxs, torch.from_numpy(Wg_p).to(DEV), torch.from_numpy(Wu_p).to(DEV), dsg,
                                      dsu, dbg, dbu)
        _status_ok()
        assert torch.equal(hs.view(torch.int16), h_dense_pruned.view(torch.int16)), f"knob {knob}"


@pytest.mark.parametrize("sparse", [False, True])
@pytest.mark.parametrize("M,d_model,d_ffn", [(512, 1024, 2816), (1100, 512, 1408)])
def test_gated_mlp_block(sparse, M, d_model, d_ffn):
    lib = _lib.load()
    g = torch.Generator().manual_seed(9 + M + d_ffn)
    x = torch.randn((M, d_model), generator=g).to(torch.float16).to(DEV)
    Wg, sg, bg = _weights(d_ffn, d_model, g)
    Wu, su, bu = _weights(d_ffn, d_model, g)
    Wd, sd, bd = _weights(d_model, d_ffn, g)
    dev = [t.to(DEV) for t in (Wg, Wu, Wd, sg, su, sd, bg, bu, bd)]
    nbytes = lib.forge_w8a8_gated_mlp_workspace_bytes(M, d_model, d_ffn)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    out = torch.full((M, d_model), 0x7B7B, dtype=torch.int16, device=DEV).view(torch.float16)
    if sparse:
        (cg, mg), (cu, mu), (cd, md) = _compress(Wg), _compress(Wu), _compress(Wd)
        _lib.call("forge_sparse_w8a8_gated_mlp", x.data_ptr(), cg.data_ptr(), mg.data_ptr(), cu.data_ptr(),
                  mu.data_ptr(), cd.data_ptr(), md.data_ptr(), *[t.data_ptr() for t in dev[3:]], out.data_ptr(), M,
                  d_model, d_ffn, ws.data_ptr(), 0)
        Wg_e, Wu_e, Wd_e = (O.prune_24_dense(w.numpy()) for w in (Wg, Wu, Wd))
    else:
        _lib.call("forge_w8a8_gated_mlp", x.data_ptr(), *[t.data_ptr() for t in dev], out.data_ptr(), M, d_model,
                  d_ffn, ws.data_ptr(), 0)
        Wg_e, Wu_e, Wd_e = Wg.numpy(), Wu.numpy(), Wd.numpy()
    _status_ok()
    # carve the workspace as the header documents
    pad = lambda n: (n + 255) & ~255
    o = 0
    xq = ws[o:o + M * d_model].view(torch.int8).view(M, d_model); o += pad(M * d_model)
    xs = ws[o:o + 4 * M].view(torch.float32); o += pad(4 * M)
    h = ws[o:o + 2 * M * d_ffn].view(torch.float16).view(M, d_ffn); o += pad(2 * M * d_ffn)
    hq = ws[o:o + M * d_ffn].view(torch.int8).view(M, d_ffn); o += pad(M * d_ffn)
    hs = ws[o:o + 4 * M].view(torch.float32); o += pad(4 * M)
    assert o == nbytes
    # stage 1: x quantized exactly as the standalone quantizer does
    q1, s1 = C.fused_quantize_activation(x, M, d_model)
    assert torch.equal(q1, xq) and torch.equal(s1, xs)
    # stage 2: h within 1 fp16 ulp of the composition oracle
    want_h = O.gated_epilogue(O.gemm_s32(xq.cpu().numpy(), Wg_e), O.gemm_s32(xq.cpu().numpy(), Wu_e), xs.cpu().numpy(),
                              sg.numpy(), su.numpy(), bg.numpy(), bu.numpy())
    assert O.half_ulp_distance(h.cpu().numpy(), want_h).max() <= 1
    # stages 3-4: bit-exact downstream of the GPU's own h
    q2, s2 = C.fused_quantize_activation(h, M, d_ffn)
    assert torch.equal(q2, hq) and torch.equal(s2, hs)
    want_out = O.dequantize_bias(O.gemm_s32(hq.cpu().numpy(), Wd_e), hs.cpu().numpy(), sd.numpy(), bd.numpy(),
                                 gemm_epilogue=True)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want_out.view(np.uint16))
