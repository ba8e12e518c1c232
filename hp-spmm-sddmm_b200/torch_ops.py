"""PyTorch front-end of the aggregation layer: autograd over the C ABI, no PyTorch arithmetic.

    layer = TorchLayer(row_ptr, col_idx, vals, M, N, max_K)   # CUDA tensors, int32 / int32 / float32
    C = layer(H)                                              # C = A·H, differentiable in H and in vals
    C.sum().backward()                                        # dH = Aᵀ·dC (SpMM), dvals = SDDMM(dC, H)

Three operators are registered with torch.library under the namespace ``hpspmm`` (``layer_forward``,
``layer_backward_features``, ``layer_backward_weights``), with shape functions for tracing and an
autograd formula that chains them, so the layer can sit inside a compiled or exported module.  Every
operator calls ``hpspmm_layer_*`` of libhpspmm.so on the current CUDA stream of the input's device; a
CPU tensor is rejected (there is no fallback).  PyTorch supplies memory, streams and the autograd
tape only.

The reference has no framework binding; this is the caller either side of its products
(test/test_all.cpp:63-107 issues them one at a time from a C++ driver).
"""
import itertools
import threading

import torch

from . import Context, Layer

_layers = {}
_ids = itertools.count(1)
_lock = threading.Lock()   # guards the registry of layers


def _entry(layer_id):
    try:
        return _layers[layer_id]
    except KeyError:
        raise RuntimeError("hpspmm: unknown or closed layer id %d" % layer_id) from None


def _require_cuda_f32(t, rows, what):
    if not t.is_cuda:
        raise RuntimeError("hpspmm: %s must be a CUDA tensor (there is no CPU path)" % what)
    if t.dtype != torch.float32 or t.dim() != 2 or t.shape[0] != rows:
        raise RuntimeError("hpspmm: %s must be float32 of shape [%d, K], got %s %s"
                           % (what, rows, t.dtype, tuple(t.shape)))
    return t.contiguous()


def _sync_values(e, vals):
    """Re-gathers the transpose's values when the weight tensor moved or was written in place."""
    key = (vals.data_ptr(), vals._version)
    if key != e["vals_key"]:
        e["vals_ref"] = vals            # keeps the borrowed device array alive
        e["layer"].update_values(vals.data_ptr(), torch.cuda.current_stream(vals.device).cuda_stream)
        e["vals_key"] = key


@torch.library.custom_op("hpspmm::layer_forward", mutates_args=())
def layer_forward(H: torch.Tensor, vals: torch.Tensor, layer_id: int) -> torch.Tensor:
    e = _entry(layer_id)
    H = _require_cuda_f32(H, e["N"], "H")
    K = H.shape[1]
    with torch.cuda.device(H.device):
        vals = vals.detach().contiguous()
        _sync_values(e, vals)
        C = torch.empty((e["M"], K), dtype=torch.float32, device=H.device)
        e["layer"].forward(K, H.data_ptr(), C.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return C


@layer_forward.register_fake
def _(H, vals, layer_id):
    return H.new_empty((_entry(layer_id)["M"], H.shape[1]))


@torch.library.custom_op("hpspmm::layer_backward_features", mutates_args=())
def layer_backward_features(dC: torch.Tensor, vals: torch.Tensor, layer_id: int) -> torch.Tensor:
    e = _entry(layer_id)
    dC = _require_cuda_f32(dC, e["M"], "dC")
    K = dC.shape[1]
    with torch.cuda.device(dC.device):
        _sync_values(e, vals.detach().contiguous())
        dH = torch.empty((e["N"], K), dtype=torch.float32, device=dC.device)
        e["layer"].backward_features(K, dC.data_ptr(), dH.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return dH


@layer_backward_features.register_fake
def _(dC, vals, layer_id):
    return dC.new_empty((_entry(layer_id)["N"], dC.shape[1]))


@torch.library.custom_op("hpspmm::layer_backward_weights", mutates_args=())
def layer_backward_weights(dC: torch.Tensor, H: torch.Tensor, layer_id: int) -> torch.Tensor:
    e = _entry(layer_id)
    dC = _require_cuda_f32(dC, e["M"], "dC")
    H = _require_cuda_f32(H, e["N"], "H")
    K = dC.shape[1]
    if H.shape[1] != K:
        raise RuntimeError("hpspmm: dC and H differ in width")
    with torch.cuda.device(dC.device):
        dA = torch.empty((e["nnz"],), dtype=torch.float32, device=dC.device)
        e["layer"].backward_weights(K, dC.data_ptr(), H.data_ptr(), dA.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream)
    return dA


@layer_backward_weights.register_fake
def _(dC, H, layer_id):
    return dC.new_empty((_entry(layer_id)["nnz"],))


def _setup_context(ctx, inputs, output):
    H, vals, layer_id = inputs
    ctx.layer_id = layer_id
    ctx.save_for_backward(H, vals)


def _backward(ctx, dC):
    H, vals = ctx.saved_tensors
    dH = dvals = None
    if ctx.needs_input_grad[0]:
        dH = layer_backward_features(dC, vals, ctx.layer_id)
    if ctx.needs_input_grad[1]:
        dvals = layer_backward_weights(dC, H, ctx.layer_id)
    return dH, dvals, None


layer_forward.register_autograd(_backward, setup_context=_setup_context)


class TorchLayer:
    """A sparse operand A (CSR on one GPU) as a differentiable map H -> A·H."""

    def __init__(self, row_ptr, col_idx, vals, M, N, max_K):
        for t, dt, what in ((row_ptr, torch.int32, "row_ptr"), (col_idx, torch.int32, "col_idx"),
                            (vals, torch.float32, "vals")):
            if not t.is_cuda or t.dtype != dt or not t.is_contiguous():
                raise RuntimeError("hpspmm: %s must be a contiguous CUDA %s tensor" % (what, dt))
        if row_ptr.numel() != M + 1 or col_idx.numel() != vals.numel():
            raise RuntimeError("hpspmm: CSR arrays disagree with M or with each other")
        self.M, self.N, self.nnz, self.max_K = int(M), int(N), int(vals.numel()), int(max_K)
        self.row_ptr, self.col_idx, self.vals = row_ptr, col_idx, vals
        dev = row_ptr.device
        # One context per layer.  A context owns scratch and a flag that plan building uses (also lazily, on
        # the first product of a new width class), and calls that share a context must not overlap on the
        # GPU: with a context of their own, two layers driven from different streams or threads cannot meet
        # there.  Products of ONE layer still must not overlap with each other.
        ctx = Context(dev.index if dev.index is not None else torch.cuda.current_device())
        with torch.cuda.device(dev):
            v = vals.detach()
            layer = Layer(ctx, self.M, self.N, self.nnz, row_ptr.data_ptr(), col_idx.data_ptr(), v.data_ptr(),
                          self.max_K, torch.cuda.current_stream().cuda_stream)
        with _lock:
            self.layer_id = next(_ids)
            _layers[self.layer_id] = {"layer": layer, "ctx": ctx, "M": self.M, "N": self.N, "nnz": self.nnz,
                                      "vals_key": (v.data_ptr(), v._version), "vals_ref": v,
                                      "keep": (row_ptr, col_idx)}

    def __call__(self, H, vals=None):
        return layer_forward(H, self.vals if vals is None else vals, self.layer_id)

    def close(self):
        with _lock:
            e = _layers.pop(self.layer_id, None)
        if e:
            e["layer"].close()
            e["ctx"].close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
