"""Multi-GPU sharding of the W8A8 linear layers: one process per GPU (torchrun), NCCL for the
one exchange step that exists.

The reference is single-GPU (no NCCL, MPI or peer access anywhere in its tree); this module is
an additive layer. Two modes, both bit-identical to the single-GPU result because every output element is still one exact int32 accumulation followed by the same
fp32 epilogue:

  rows     token rows are split across ranks, weights replicated. No communication at all: each
           rank quantizes and multiplies its own rows. This is the mode that scales linearly.
  columns  output channels (weight rows) are split across ranks, activations replicated; each
           rank computes out[:, n0:n1] and every rank ends up with the full (M, N) output. The
           exchange moves (g-1)/g * 2*M*N bytes into every GPU, so it is link-bound, not
           compute-bound. Two implementations:
             fused  (default on GPUs) every rank's output buffer is mapped into every process
                    (symmetric memory, else CUDA IPC) and the GEMM epilogue stores each tile
                    straight into all g buffers - the all-gather is done by the kernel's own
                    peer stores, tile by tile, overlapped with the tensor-core work.
             nccl   rows are processed in chunks; the slice of chunk i is all-gathered with NCCL
                    while the GEMM of chunk i+1 runs, then interleaved into place by a copy.

The local compute is the C ABI of libforge_b200 (no fallback). `local_linear` can be injected so
that the partition / gather / interleave logic is testable with gloo on CPUs.
"""
from dataclasses import dataclass

import torch
import torch.distributed as dist


def partition(total, world, rank):
    """Balanced contiguous partition of `total` items: (start, count) of `rank`'s share."""
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


@dataclass
class SparseWeights:
    """One 2:4-sparse INT8 weight: compressed values (N, K/2) int8, metadata (N, K/32) int32,
    fp16 per-channel scales (N) and optional fp16 bias (N) - the buffers of the reference's
    SparseLinear module (python/forge/nn/linear.py:207-217)."""
    W_comp: torch.Tensor
    w_meta: torch.Tensor
    w_scale: torch.Tensor
    bias: torch.Tensor = None

    def rows(self, start, count):
        b = None if self.bias is None else self.bias[start:start + count]
        return SparseWeights(self.W_comp[start:start + count], self.w_meta[start:start + count],
                             self.w_scale[start:start + count], b)


def _forge_sparse_linear(x, w):
    """x (m, K) fp16 on this rank's GPU -> (m, n) fp16 through libforge_b200."""
    from . import _forge_C as C
    m, k = x.shape
    scratch_q = torch.empty((m, k), dtype=torch.int8, device=x.device)
    scratch_s = torch.empty((m,), dtype=torch.float32, device=x.device)
    return C.sparse_int8_linear(x, w.W_comp, w.w_meta, w.w_scale, w.bias, scratch_q, scratch_s)


def map_peer_buffers(tensor, group=None):
    """Maps `tensor` (same shape on every rank, one per GPU) into every process of `group`.
    Returns (pointers, keepalive, buffer): pointers[r] is rank r's buffer as seen from this process
    and `buffer` is this rank's own tensor to use from now on (a fresh symmetric-memory allocation
    when that route is taken). Tries torch's symmetric memory first, then CUDA IPC through torch's
    storage sharing; the ranks agree on the route with one all-reduce, so that no rank enters a
    collective the others skipped."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    buf = hdl = None
    try:
        import torch.distributed._symmetric_memory as symm_mem
        buf = symm_mem.empty(tensor.shape, dtype=tensor.dtype, device=tensor.device)
        ok = 1
    except Exception:   # no symmetric-memory support in this build / on this device
        ok = 0
    agreed = torch.tensor([ok], dtype=torch.int32, device=tensor.device)
    dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
    if int(agreed.item()) == 1:
        hdl = symm_mem.rendezvous(buf, group if group is not None else dist.group.WORLD)
        return [int(p) for p in hdl.buffer_ptrs], (buf, hdl), buf
    info = tensor.untyped_storage()._share_cuda_()
    infos = [None] * world
    dist.all_gather_object(infos, info, group=group)
    keep, ptrs = [], []
    for r in range(world):
        if r == rank:
            ptrs.append(tensor.data_ptr())
            continue
        st = torch.UntypedStorage._new_shared_cuda(*infos[r])
        keep.append(st)
        ptrs.append(st.data_ptr() + tensor.storage_offset() * tensor.element_size())
    return ptrs, keep, tensor


class ShardedSparseLinear:
    """2:4-sparse W8A8 linear layer sharded over the ranks of `group`.

    mode "rows":    `weights` is the full weight on every rank; forward(x_local) takes this
                    rank's token rows and returns their outputs (no collective).
    mode "columns": `weights` is the full weight; the constructor keeps only this rank's output
                    channels. forward(x) takes all tokens (replicated) and returns the full
                    (M, N) output on every rank.

    With exchange="fused" the returned tensor is a view of a persistent buffer that the other ranks
    write into: it is valid until the next forward() of this layer (clone it to keep it - a
    residual connection or a saved activation must). The buffer is sized for the largest M seen so
    far; smaller batches use its leading rows, so changing batch sizes does not redo the mapping.
    exchange="nccl" returns a fresh tensor every call.
    """

    def __init__(self, weights, mode, group=None, chunks=4, local_linear=None, exchange="auto"):
        if mode not in ("rows", "columns"):
            raise ValueError("mode must be 'rows' or 'columns'")
        self.mode = mode
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.chunks = max(1, chunks)
        self.local_linear = local_linear or _forge_sparse_linear
        # "fused": all-gather by the GEMM epilogue's peer stores; "nccl": chunked NCCL all-gather
        self.exchange = exchange
        if exchange == "auto":
            self.exchange = "fused" if (local_linear is None and weights.W_comp.is_cuda) else "nccl"
        self._peer = None   # (rows, pointers, keepalive, out tensor, sync scalar)
        self._comm_stream = None
        self.N = weights.W_comp.shape[0]
        if mode == "columns":
            if self.N % self.world != 0:
                raise ValueError(f"output channels ({self.N}) must divide evenly over {self.world} ranks")
            n0, n = partition(self.N, self.world, self.rank)
            self.weights = weights.rows(n0, n)
        else:
            self.weights = weights

    def rows_of(self, M):
        """(start, count) of the token rows this rank owns in mode 'rows'."""
        return partition(M, self.world, self.rank)

    def forward(self, x):
        if self.mode == "rows" or self.world == 1:
            return self.local_linear(x, self.weights)
        M = x.shape[0]
        n_local = self.N // self.world
        if self.exchange == "fused":
            return self._forward_fused(x)
        out = torch.empty((M, self.N), dtype=torch.float16, device=x.device)
        use_streams = x.is_cuda
        if use_streams and self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=x.device)
        comm_stream = self._comm_stream
        pending = []
        for c in range(self.chunks):
            r0, rows = partition(M, self.chunks, c)
            if rows == 0:
                continue
            y = self.local_linear(x[r0:r0 + rows], self.weights)          # (rows, n_local)
            if use_streams:
                ev = torch.cuda.Event()
                ev.record()
                with torch.cuda.stream(comm_stream):
                    comm_stream.wait_event(ev)
                    # allocated on the stream that uses it, so the caching allocator cannot hand the
                    # block to the compute stream while the gather or the copy is still running
                    flat = torch.empty((self.world * rows, n_local), dtype=torch.float16, device=x.device)
                    dist.all_gather_into_tensor(flat, y.contiguous(), group=self.group)
                    # interleave: out[r0+i, w*n_local + j] = flat[w*rows + i, j]
                    out[r0:r0 + rows].view(rows, self.world, n_local).copy_(
                        flat.view(self.world, rows, n_local).permute(1, 0, 2))
                    done = torch.cuda.Event()
                    done.record()
                y.record_stream(comm_stream)
                out.record_stream(comm_stream)
                pending.append(done)
            else:
                # concatenated along dim 0 by the collective; viewed as (rank, row, column) afterwards
                flat = torch.empty((self.world * rows, n_local), dtype=torch.float16, device=x.device)
                dist.all_gather_into_tensor(flat, y.contiguous(), group=self.group)
                out[r0:r0 + rows].view(rows, self.world, n_local).copy_(
                    flat.view(self.world, rows, n_local).permute(1, 0, 2))
        for ev in pending:
            torch.cuda.current_stream().wait_event(ev)
        return out

    def _forward_fused(self, x):
        """Quantize locally, then one GEMM launch whose epilogue writes this rank's columns into
        every rank's output buffer. Stream-ordered all-reduces of one scalar fence the exchange:
        nobody overwrites a buffer a peer may still read, nobody reads before all have written."""
        import ctypes
        from . import _forge_C as C
        from . import _lib
        M, K = x.shape
        n_local = self.N // self.world
        # every rank sees the same M (the activations are replicated), so all ranks re-map together
        if self._peer is None or self._peer[0] < M:
            self._peer = None   # drop the old mapping before making a larger one
            out = torch.empty((M, self.N), dtype=torch.float16, device=x.device)
            ptrs, keep, out = map_peer_buffers(out, self.group)
            self._peer = (M, ptrs, keep, out, torch.zeros(1, device=x.device))
        _, ptrs, _, out, token = self._peer
        out = out[:M]
        xq, xs = C.fused_quantize_activation(x, M, K)
        col0_bytes = self.rank * n_local * 2
        arr = (ctypes.c_void_p * self.world)(*[p + col0_bytes for p in ptrs])
        dist.all_reduce(token, group=self.group)          # every rank is done with the previous contents
        w = self.weights
        _lib.call("forge_sparse_int8_gemm_multi", w.W_comp.data_ptr(), xq.data_ptr(), w.w_meta.data_ptr(),
                  xs.data_ptr(), w.w_scale.data_ptr(), 0 if w.bias is None else w.bias.data_ptr(), arr, self.world,
                  self.N, M, K, n_local, torch.cuda.current_stream().cuda_stream)
        dist.all_reduce(token, group=self.group)          # every rank's stores have landed
        return out

    __call__ = forward
