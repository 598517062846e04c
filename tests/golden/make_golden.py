"""Generates tests/golden/reference_vectors.npz and tests/golden/reference_conv_vectors.npz: small
seeded inputs together with the outputs of the REFERENCE's own CUDA kernels
(oracle/_ref/libforge_ref.so, built from the reference sources for sm_100a by oracle/build.py).
Needs a GPU:

    python tests/golden/make_golden.py [output.npz [conv_output.npz]]

The committed .npz pins the CPU oracle in the CPU-only test run (tests/test_oracle_cpu.py).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as O  # noqa: E402


def main(out_path):
    dev = "cuda:0"
    g = torch.Generator().manual_seed(20240601)
    out = {}

    def rand_i8(*shape):
        return torch.randint(-127, 128, shape, generator=g, dtype=torch.int8)

    # quantize: vector path, ragged two-pass path, multi-vector rows
    for name, (M, K) in {"q0": (32, 256), "q1": (9, 100), "q2": (16, 2056), "q3": (3, 8200)}.items():
        x = (torch.rand((M, K), generator=g) * 6 - 3).to(torch.float16)
        if name == "q0":
            x[3] = 0  # an all-zero row exercises the 1e-8 floor
        q, s = O.ref_quantize(x.to(dev))
        out[name + "_x"], out[name + "_q"], out[name + "_s"] = x.numpy(), q.cpu().numpy(), s.cpu().numpy()

    # dequant + bias
    M, N = 16, 64
    acc = torch.randint(-50000, 50001, (M, N), generator=g, dtype=torch.int32)
    a_s = (torch.rand(M, generator=g) * 0.049 + 0.001).float()
    w_s = (torch.rand(N, generator=g) * 0.049 + 0.001).to(torch.float16)
    bias = (torch.rand(N, generator=g) - 0.5).to(torch.float16)
    out["d_acc"], out["d_as"], out["d_ws"], out["d_bias"] = acc.numpy(), a_s.numpy(), w_s.numpy(), bias.numpy()
    out["d_out_bias"] = O.ref_dequantize_bias(acc.to(dev), a_s.to(dev), w_s.to(dev), bias.to(dev)).cpu().numpy()
    out["d_out_nobias"] = O.ref_dequantize_bias(acc.to(dev), a_s.to(dev), w_s.to(dev), None).cpu().numpy()

    # prune + compress + pack
    w = rand_i8(32, 128)
    w[0, :8] = torch.tensor([5, -5, 5, 5, 0, 0, 0, 0], dtype=torch.int8)  # ties
    comp, raw, packed = O.ref_prune_pack(w.to(dev))
    out["p_w"], out["p_comp"], out["p_raw"] = w.numpy(), comp.cpu().numpy(), raw.cpu().numpy()
    out["p_packed"] = packed.cpu().numpy().view(np.uint32)

    # dense GEMM + dequant (reference wmma kernel), shape of tests/test_int8_dense_gemm.cu
    M, K, N = 32, 128, 64
    A, B = rand_i8(M, K), rand_i8(N, K)
    a_s = (torch.rand(M, generator=g) * 0.049 + 0.001).float()
    w_s = (torch.rand(N, generator=g) * 0.049 + 0.001).to(torch.float16)
    bias = (torch.rand(N, generator=g) - 0.5).to(torch.float16)
    out["g_A"], out["g_B"], out["g_as"], out["g_ws"], out["g_bias"] = (A.numpy(), B.numpy(), a_s.numpy(),
                                                                      w_s.numpy(), bias.numpy())
    out["g_out_bias"] = O.ref_int8_gemm_dequant(A.to(dev), B.to(dev), a_s.to(dev), w_s.to(dev),
                                                bias.to(dev)).cpu().numpy()
    out["g_out_nobias"] = O.ref_int8_gemm_dequant(A.to(dev), B.to(dev), a_s.to(dev), w_s.to(dev), None).cpu().numpy()

    # sparse GEMM + dequant (reference mma.sp kernel), a ragged shape of tests/test_int8_sparse_gemm.cu
    M, K, N = 37, 192, 208
    W, x = rand_i8(N, K), rand_i8(M, K)
    a_s = (torch.rand(M, generator=g) * 0.049 + 0.001).float()
    w_s = (torch.rand(N, generator=g) * 0.049 + 0.001).to(torch.float16)
    bias = (torch.rand(N, generator=g) - 0.5).to(torch.float16)
    comp, raw, packed = O.ref_prune_pack(W.to(dev))
    out["s_W"], out["s_x"], out["s_as"], out["s_ws"], out["s_bias"] = (W.numpy(), x.numpy(), a_s.numpy(),
                                                                      w_s.numpy(), bias.numpy())
    out["s_comp"], out["s_packed"] = comp.cpu().numpy(), packed.cpu().numpy().view(np.uint32)
    out["s_out_bias"] = O.ref_sparse_int8_gemm(comp, x.to(dev), packed, a_s.to(dev), w_s.to(dev),
                                               bias.to(dev)).cpu().numpy()
    out["s_out_nobias"] = O.ref_sparse_int8_gemm(comp, x.to(dev), packed, a_s.to(dev), w_s.to(dev), None).cpu().numpy()
    torch.cuda.synchronize()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


def conv_vectors(out_path):
    """The reference's conv pipelines on its own test shapes (tests/test_int8_conv2d.cu:206-257,
    tests/test_int8_special_conv.cu:282-284), one sample each. Besides the output, the int8 patches and
    their scales are read back from the reference's workspace ([fp16 col | int8 col | fp32 scales | ...],
    src/nn/int8_conv2d.cu:172-176), which pins every later step on the CPU exactly."""
    dev = "cuda:0"
    g = torch.Generator().manual_seed(20240602)
    out = {}
    cases = {"c0": (8, 16, 16, 16, 3, 3, 1, 1, 1, 1, 1, 1, True), "c1": (7, 32, 32, 16, 2, 2, 0, 0, 2, 2, 1, 1, True),
             "c2": (4, 12, 12, 8, 3, 3, 1, 1, 1, 1, 1, 1, False), "c3": (8, 16, 16, 8, 3, 3, 2, 2, 1, 1, 2, 2, True)}
    for name, (Ci, H, W, Co, kH, kW, pH, pW, sH, sW, dH, dW, use_bias) in cases.items():
        K = Ci * kH * kW
        x = (torch.rand((1, Ci, H, W), generator=g) * 2 - 1).to(torch.float16)
        w = torch.randint(-127, 128, (Co, K), generator=g, dtype=torch.int8)
        w_s = (torch.rand(Co, generator=g) * 0.045 + 0.005).to(torch.float16)
        bias = (torch.rand(Co, generator=g) - 0.5).to(torch.float16) if use_bias else None
        Ho, Wo = O.conv_out_size(H, pH, dH, kH, sH), O.conv_out_size(W, pW, dW, kW, sW)
        M = Ho * Wo
        ws = torch.zeros(int(O.ref().ref_int8_conv2d_workspace_size(Ci, H, W, Co, kH, kW, pH, pW, sH, sW, dH, dW)) + 16,
                         dtype=torch.uint8, device=dev)
        y = torch.empty((1, Co, Ho, Wo), dtype=torch.float16, device=dev)
        xd, wd, sd = x.to(dev), w.to(dev), w_s.to(dev)
        bd = None if bias is None else bias.to(dev)
        O.ref().ref_int8_conv2d_forward(O.tp(xd), O.tp(wd), O.tp(sd), O.tp(bd), O.tp(y), 1, Ci, H, W, Co, kH, kW, pH, pW,
                                        sH, sW, dH, dW, O.tp(ws), O.cur_stream())
        torch.cuda.synchronize()
        wsb = ws.cpu().numpy()
        out[name + "_cfg"] = np.array([Ci, H, W, Co, kH, kW, pH, pW, sH, sW, dH, dW], np.int32)
        out[name + "_x"], out[name + "_w"], out[name + "_ws"] = x.numpy(), w.numpy(), w_s.numpy()
        if bias is not None:
            out[name + "_bias"] = bias.numpy()
        out[name + "_q"] = wsb[2 * M * K:3 * M * K].view(np.int8).reshape(M, K).copy()
        out[name + "_as"] = wsb[3 * M * K:3 * M * K + 4 * M].view(np.float32).copy()
        out[name + "_y"] = y.cpu().numpy()
    # 2x2 stride-2 transposed conv
    for name, (Ci, H, W, Co, use_bias) in {"t0": (32, 16, 16, 64, True), "t1": (16, 32, 32, 16, False)}.items():
        x = (torch.rand((1, Ci, H, W), generator=g) * 2 - 1).to(torch.float16)
        w = torch.randint(-127, 128, (4 * Co, Ci), generator=g, dtype=torch.int8)
        w_s = (torch.rand(Co, generator=g) * 0.045 + 0.005).to(torch.float16)
        bias = (torch.rand(Co, generator=g) - 0.5).to(torch.float16) if use_bias else None
        y = O.ref_int8_conv_transpose2d_k2s2(x.to(dev), w.to(dev), w_s.to(dev), None if bias is None else bias.to(dev))
        out[name + "_x"], out[name + "_w"], out[name + "_ws"] = x.numpy(), w.numpy(), w_s.numpy()
        if bias is not None:
            out[name + "_bias"] = bias.numpy()
        out[name + "_y"] = y.cpu().numpy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_vectors.npz"))
    conv_vectors(sys.argv[2] if len(sys.argv) > 2 else os.path.join(HERE, "reference_conv_vectors.npz"))
