"""Row-sharded aggregation layer: one process per GPU, torch.distributed for the exchange.

Rank r owns rows [bounds[r], bounds[r+1]) of A, of C and of dC (nnz-balanced blocks from
``shard_bounds``), and rows [feat_bounds[r], feat_bounds[r+1]) of H and of dH.  Rows of C depend on
the same rows of A and on all of H, so the layer has two exchange steps and nothing else:

  forward            all-gather H  (every rank broadcasts its rows into the others' own memory),
                     then the local product  C_own = A_own · H
  backward, features local product  P = A_ownᵀ · dC_own  (N × K, a partial sum), then a
                     reduce-scatter: rank r receives the sum over ranks of rows feat_bounds[r:r+2] of P
  backward, weights  local SDDMM(dC_own, H) on the H gathered by the forward pass; no exchange

The shards differ in size, so the two collectives are one broadcast (or reduce) per rank, issued
asynchronously and waited for together; NCCL runs them as one group.  Remote rows always land in
this GPU's own memory before a kernel reads them.  The reference is single-GPU
(test/test_all.cpp:27-109); this has no counterpart there.

The products themselves come from a ``local`` object.  ``GpuLocal`` is the product implementation
(the C ABI's layer handle on CUDA tensors).  Tests of the exchange logic on CPU ranks pass their own.
"""
import torch
import torch.distributed as dist

from . import Context, Layer


class GpuLocal:
    """The products of one rank's shard through ``hpspmm_layer_*`` on CUDA tensors."""

    def __init__(self, row_ptr, col_idx, vals, M_own, N, max_K, device):
        for t, dt in ((row_ptr, torch.int32), (col_idx, torch.int32), (vals, torch.float32)):
            if not t.is_cuda or t.dtype != dt or not t.is_contiguous():
                raise RuntimeError("hpspmm: shard arrays must be contiguous CUDA tensors (int32, int32, float32)")
        self.device = device
        self.M_own, self.N, self.nnz = int(M_own), int(N), int(vals.numel())
        self._keep = (row_ptr, col_idx, vals)
        self.ctx = Context(device.index)
        with torch.cuda.device(device):
            self.layer = Layer(self.ctx, self.M_own, self.N, self.nnz, row_ptr.data_ptr(), col_idx.data_ptr(),
                               vals.data_ptr(), max_K, torch.cuda.current_stream().cuda_stream)

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def forward(self, H):
        C = torch.empty((self.M_own, H.shape[1]), dtype=torch.float32, device=self.device)
        self.layer.forward(H.shape[1], H.data_ptr(), C.data_ptr(), self._stream())
        return C

    def backward_features(self, dC, out):
        self.layer.backward_features(dC.shape[1], dC.data_ptr(), out.data_ptr(), self._stream())
        return out

    def backward_weights(self, dC, H):
        dA = torch.empty((self.nnz,), dtype=torch.float32, device=self.device)
        self.layer.backward_weights(dC.shape[1], dC.data_ptr(), H.data_ptr(), dA.data_ptr(), self._stream())
        return dA

    def close(self):
        self.layer.close()
        self.ctx.close()


class ShardedLayer:
    def __init__(self, local, N, feat_bounds, rank, world, device=None, group=None):
        if len(feat_bounds) != world + 1 or int(feat_bounds[0]) != 0 or int(feat_bounds[-1]) != N:
            raise ValueError("feat_bounds must hold world + 1 ascending row indices from 0 to N")
        self.local, self.N, self.rank, self.world = local, int(N), rank, world
        self.feat_bounds = [int(b) for b in feat_bounds]
        self.device = device if device is not None else torch.device("cpu")
        self.group = group
        self._H = None        # gathered H of the last forward pass
        self._P = None        # partial N × K product of the last backward pass

    def _rows(self, r):
        return slice(self.feat_bounds[r], self.feat_bounds[r + 1])

    def _buffer(self, name, K):
        buf = getattr(self, name)
        if buf is None or buf.shape[1] != K:
            buf = torch.empty((self.N, K), dtype=torch.float32, device=self.device)
            setattr(self, name, buf)
        return buf

    def gather_features(self, H_own):
        """All-gather of the feature shards into this rank's own N × K buffer."""
        K = H_own.shape[1]
        if H_own.shape[0] != self.feat_bounds[self.rank + 1] - self.feat_bounds[self.rank]:
            raise ValueError("H_own does not have this rank's number of rows")
        H = self._buffer("_H", K)
        H[self._rows(self.rank)].copy_(H_own)
        work = []
        for r in range(self.world):
            part = H[self._rows(r)]
            if part.numel():
                work.append(dist.broadcast(part, src=self._global(r), group=self.group, async_op=True))
        for w in work:
            w.wait()
        return H

    def _global(self, r):
        return r if self.group is None else dist.get_global_rank(self.group, r)

    def forward(self, H_own):
        return self.local.forward(self.gather_features(H_own))

    def backward_features(self, dC_own):
        K = dC_own.shape[1]
        P = self.local.backward_features(dC_own, self._buffer("_P", K))
        work = []
        for r in range(self.world):
            part = P[self._rows(r)]
            if part.numel():
                work.append(dist.reduce(part, dst=self._global(r), op=dist.ReduceOp.SUM, group=self.group,
                                        async_op=True))
        for w in work:
            w.wait()
        return P[self._rows(self.rank)].clone()

    def backward_weights(self, dC_own):
        if self._H is None or self._H.shape[1] != dC_own.shape[1]:
            raise RuntimeError("backward_weights needs the H gathered by a forward pass of the same width")
        return self.local.backward_weights(dC_own, self._H)
