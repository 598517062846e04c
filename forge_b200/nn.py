"""Drop-in INT8 linear modules on the forge_b200 kernels.

Mirror of the reference's `forge.nn.QuantizedLinear` and `forge.nn.SparseLinear`
(python/forge/nn/linear.py:135-254): same constructor arguments, same registered buffers and
parameters with the same names, dtypes and layouts (`w_int8`, `w_scale`, `bias`; `W_comp`,
`w_meta` int32, `w_scale`, `bias`), so state_dicts written by either implementation load into
the other. Weight quantisation is the reference's recipe (per output channel, absmax / 127,
round half to even, clamp to +-127, scale stored as fp16).

Beyond the reference: inputs with more than two dimensions are flattened over the leading
dimensions, non-contiguous inputs are made contiguous, and `SparseLinear.from_dense_weight`
prunes on the module's own device instead of assuming "cuda".
"""
import torch
import torch.nn as nn

from . import _forge_C as _C


def quantize_weight_per_channel(weight_fp):
    """(N, K) float weight -> (int8 (N, K), fp16 scales (N)); linear.py:167-173."""
    w = weight_fp.detach().to(torch.float32)
    scale = w.abs().amax(dim=1).clamp(min=1e-8) / 127.0
    q = torch.clamp(torch.round(w / scale.unsqueeze(1)), -127, 127).to(torch.int8)
    return q, scale.to(torch.float16)


class _Int8LinearFn(torch.autograd.Function):
    """Forward on the INT8 tensor-core path; backward through the dequantised weight in fp16,
    as the reference does (linear.py:123-132)."""

    @staticmethod
    def forward(ctx, x, w_int8, w_scale, bias, scratch_q, scratch_s):
        out = _C.int8_linear(x, w_int8, w_scale, bias, scratch_q, scratch_s)
        ctx.save_for_backward(x, w_int8, w_scale)
        ctx.has_bias = bias is not None
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x, w_int8, w_scale = ctx.saved_tensors
        g = grad_out.to(torch.float16)
        w = w_int8.to(torch.float16) * w_scale.unsqueeze(1)
        grad_bias = g.sum(dim=0) if ctx.has_bias else None
        return g @ w, None, None, grad_bias, None, None


class _ScratchMixin:
    def _scratch(self, M, K, device):
        q = getattr(self, "_scratch_q", None)
        if q is None or q.shape[0] < M or q.shape[1] != K or q.device != device:
            self._scratch_q = torch.empty((M, K), dtype=torch.int8, device=device)
            self._scratch_s = torch.empty((M,), dtype=torch.float32, device=device)
        return self._scratch_q, self._scratch_s

    @staticmethod
    def _as_rows(x):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if x2.dtype != torch.float16:
            x2 = x2.to(torch.float16)
        return x2.contiguous(), lead


class QuantizedLinear(nn.Module, _ScratchMixin):
    """W8A8 linear layer: per-token activation quantisation + dense INT8 GEMM + dequant + bias."""

    def __init__(self, in_features, out_features, bias=True):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("w_int8", torch.zeros(out_features, in_features, dtype=torch.int8))
        self.w_scale = nn.Parameter(torch.ones(out_features, dtype=torch.float16))
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, dtype=torch.float16))
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        x2, lead = self._as_rows(x)
        q, s = self._scratch(x2.shape[0], x2.shape[1], x2.device)
        y = _Int8LinearFn.apply(x2, self.w_int8, self.w_scale, self.bias, q, s)
        return y.reshape(*lead, self.out_features)

    @torch.no_grad()
    def quantize_weight(self, weight_fp):
        if self.w_int8.is_cuda and weight_fp.shape[1] % 32 == 0:
            # one kernel on the module's device (IEEE arithmetic: bit-identical to torch on the CPU)
            q, _, _, scale = _C.prepare_weight(weight_fp.detach().to(self.w_int8.device), sparse=False)
        else:
            # any in_features, as the reference accepts (linear.py:167-173); the kernel walks 32-wide runs
            q, scale = quantize_weight_per_channel(weight_fp.detach().to(self.w_int8.device))
        self.w_int8.copy_(q)
        self.w_scale.data.copy_(scale)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


class SparseLinear(nn.Module, _ScratchMixin):
    """W8A8 linear layer with a 2:4 structured-sparse weight (inference only)."""

    def __init__(self, in_features, out_features, bias=True):
        super().__init__()
        if in_features % 64 != 0 or out_features % 16 != 0:
            raise ValueError("SparseLinear needs in_features % 64 == 0 and out_features % 16 == 0")
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("W_comp", torch.zeros(out_features, in_features // 2, dtype=torch.int8))
        self.register_buffer("w_meta", torch.zeros(out_features, in_features // 32, dtype=torch.int32))
        self.w_scale = nn.Parameter(torch.ones(out_features, dtype=torch.float16))
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, dtype=torch.float16))
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        x2, lead = self._as_rows(x)
        q, s = self._scratch(x2.shape[0], x2.shape[1], x2.device)
        y = _C.sparse_int8_linear(x2, self.W_comp, self.w_meta, self.w_scale.detach(),
                                  None if self.bias is None else self.bias.detach(), q, s, None, 0)
        return y.reshape(*lead, self.out_features)

    @torch.no_grad()
    def from_dense_weight(self, weight_fp):
        """Quantise, prune 2:4 by magnitude, compress and pack (linear.py:234-249)."""
        dev = self.W_comp.device
        if dev.type != "cuda":
            raise RuntimeError("move the module to a CUDA device before from_dense_weight()")
        # one kernel: per-channel quantisation + 2:4 prune + compress + metadata pack
        _, comp, meta, scale = _C.prepare_weight(weight_fp.detach().to(dev), sparse=True)
        self.W_comp.copy_(comp)
        self.w_meta.copy_(meta)
        self.w_scale.data.copy_(scale)

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.bias is not None}, sparse=2:4")
