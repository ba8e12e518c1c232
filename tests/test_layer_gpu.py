"""The aggregation layer (forward SpMM, transposed SpMM, SDDMM behind one handle) against the CPU oracle,
through the C ABI and through the PyTorch autograd front-end (needs a B200)."""
import ctypes
import importlib

import numpy as np
import pytest

from helpers import check_against_f64

pytestmark = pytest.mark.gpu


def _rect_graph(pkg, M, N, seed):
    """Rectangular CSR with a few heavy rows, empty rows and unreferenced columns."""
    g = pkg.gen_uniform_degree(M, N, 0, 24, seed=seed, vals_kind=pkg.VALS_UPM1)
    return g


@pytest.mark.parametrize("K", [32, 64, 128, 20])
@pytest.mark.parametrize("kind", ["rmat", "rect"])
def test_layer_products_match_oracle(gpu_ctx, pkg, oracle, K, kind):
    ctx = gpu_ctx
    g = pkg.gen_rmat(12, 16, seed=11) if kind == "rmat" else _rect_graph(pkg, 3000, 1777, 12)
    M, N, nnz = g["M"], g["N"], g["nnz"]
    H = pkg.host_fill_uniform(N * K, 11, 1, -1.0, 1.0).reshape(N, K)
    dC = pkg.host_fill_uniform(M * K, 11, 2, -1.0, 1.0).reshape(M, K)
    d_rp, d_ci, d_v = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"])
    d_H, d_dC = ctx.upload(H), ctx.upload(dC)
    d_C, d_dH, d_dA = ctx.alloc((M, K), np.float32), ctx.alloc((N, K), np.float32), ctx.alloc((nnz,), np.float32)
    layer = pkg.Layer(ctx, M, N, nnz, d_rp, d_ci, d_v, 128)
    info = layer.info()
    assert (info["M"], info["N"], info["nnz"], info["max_K"]) == (M, N, nnz, 128) and info["owned_bytes"] > 0

    # the transpose the layer owns is the oracle's, bit for bit
    rpt, cit, vt, perm = oracle.csr_transpose(M, N, g["row_ptr"], g["col_idx"], g["vals"])
    p_rpt, p_cit, p_vt, p_perm = layer.transposed()

    def read(ptr, count, dtype):
        out = np.empty(count, dtype=dtype)
        ctx.memcpy_d2h(out, ptr)
        ctx.stream_sync()
        return out

    assert np.array_equal(read(p_rpt, N + 1, np.int32), rpt)
    assert np.array_equal(read(p_cit, nnz, np.int32), cit)
    assert np.array_equal(read(p_vt, nnz, np.float32), vt)
    assert np.array_equal(read(p_perm, nnz, np.int32), perm)

    layer.forward(K, d_H, d_C)
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], H)
    check_against_f64(d_C.to_host(), ref, abs_sum, "layer forward")

    layer.backward_features(K, d_dC, d_dH)
    ref, abs_sum = oracle.spmm_f64(rpt, cit, vt, dC)
    check_against_f64(d_dH.to_host(), ref, abs_sum, "layer backward (features)")

    layer.backward_weights(K, d_dC, d_H, d_dA)
    ref, abs_sum = oracle.sddmm_f64(g["row_ptr"], g["col_idx"], dC, H)
    check_against_f64(d_dA.to_host(), ref, abs_sum, "layer backward (weights)")

    # new edge weights reach both A and its transpose
    v2 = pkg.host_fill_uniform(nnz, 11, 3, -2.0, 2.0)
    d_v2 = ctx.upload(v2)
    layer.update_values(d_v2)
    layer.forward(K, d_H, d_C)
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], v2, H)
    check_against_f64(d_C.to_host(), ref, abs_sum, "layer forward, new weights")
    layer.backward_features(K, d_dC, d_dH)
    ref, abs_sum = oracle.spmm_f64(rpt, cit, v2[perm], dC)
    check_against_f64(d_dH.to_host(), ref, abs_sum, "layer backward, new weights")

    layer.close()
    for b in (d_rp, d_ci, d_v, d_v2, d_H, d_dC, d_C, d_dH, d_dA):
        b.free()


def test_layer_argument_errors(gpu_ctx, pkg):
    ctx = gpu_ctx
    g = pkg.gen_uniform_degree(64, 64, 1, 4, seed=3)
    d_rp, d_ci, d_v = ctx.upload(g["row_ptr"]), ctx.upload(g["col_idx"]), ctx.upload(g["vals"])
    layer = pkg.Layer(ctx, 64, 64, g["nnz"], d_rp, d_ci, d_v, 32)
    d_H, d_C = ctx.alloc((64, 64), np.float32), ctx.alloc((64, 64), np.float32)
    with pytest.raises(pkg.HpspmmError) as ei:
        layer.forward(64, d_H, d_C)             # wider than max_K
    assert ei.value.status == pkg.ERR_INVALID
    with pytest.raises(pkg.HpspmmError):
        pkg.Layer(ctx, 64, 64, g["nnz"], None, d_ci, d_v, 32)
    lib = ctx.lib
    assert lib.hpspmm_layer_forward(ctx.handle, None, 32, ctypes.c_void_p(d_H.ptr), ctypes.c_void_p(d_C.ptr),
                                    None) == pkg.ERR_INVALID
    assert lib.hpspmm_layer_destroy(ctx.handle, None) == 0
    layer.close()
    for b in (d_rp, d_ci, d_v, d_H, d_C):
        b.free()


def test_empty_layer(gpu_ctx, pkg):
    ctx = gpu_ctx
    rp = np.zeros(9, dtype=np.int32)
    d_rp = ctx.upload(rp)
    layer = pkg.Layer(ctx, 8, 5, 0, d_rp, None, None, 32)
    d_H, d_C, d_dH = ctx.alloc((5, 32), np.float32), ctx.alloc((8, 32), np.float32), ctx.alloc((5, 32), np.float32)
    ctx.fill(d_C, 8 * 32, 7.0)
    ctx.fill(d_dH, 5 * 32, 7.0)
    layer.forward(32, d_H, d_C)
    layer.backward_features(32, d_C, d_dH)
    assert not d_C.to_host().any() and not d_dH.to_host().any()
    layer.close()
    for b in (d_rp, d_H, d_C, d_dH):
        b.free()


@pytest.mark.parametrize("K", [64, 48])
def test_torch_autograd_front_end(pkg, oracle, K):
    torch = pytest.importorskip("torch")
    ops = importlib.import_module(pkg.__name__ + ".torch_ops")
    dev = torch.device("cuda", 0)
    g = pkg.gen_rmat(11, 16, seed=21)
    M, N, nnz = g["M"], g["N"], g["nnz"]
    H_h = pkg.host_fill_uniform(N * K, 21, 1, -1.0, 1.0).reshape(N, K)
    G_h = pkg.host_fill_uniform(M * K, 21, 2, -1.0, 1.0).reshape(M, K)
    rp, ci = torch.from_numpy(g["row_ptr"]).to(dev), torch.from_numpy(g["col_idx"]).to(dev)
    vals = torch.from_numpy(g["vals"]).to(dev).requires_grad_(True)
    H = torch.from_numpy(H_h).to(dev).requires_grad_(True)
    G = torch.from_numpy(G_h).to(dev)
    layer = ops.TorchLayer(rp, ci, vals, M, N, max_K=128)

    C = layer(H)
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], H_h)
    check_against_f64(C.detach().cpu().numpy(), ref, abs_sum, "torch forward")
    (C * G).sum().backward()
    rpt, cit, vt, perm = oracle.csr_transpose(M, N, g["row_ptr"], g["col_idx"], g["vals"])
    ref, abs_sum = oracle.spmm_f64(rpt, cit, vt, G_h)
    check_against_f64(H.grad.cpu().numpy(), ref, abs_sum, "torch dH")
    ref, abs_sum = oracle.sddmm_f64(g["row_ptr"], g["col_idx"], G_h, H_h)
    check_against_f64(vals.grad.cpu().numpy(), ref, abs_sum, "torch dvals")

    # an in-place step on the weights (what an optimiser does) reaches the next forward and backward
    with torch.no_grad():
        vals.mul_(-0.5)
    H.grad = None
    C2 = layer(H)
    v2 = (g["vals"] * np.float32(-0.5)).astype(np.float32)
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], v2, H_h)
    check_against_f64(C2.detach().cpu().numpy(), ref, abs_sum, "torch forward after step")
    (C2 * G).sum().backward()
    ref, abs_sum = oracle.spmm_f64(rpt, cit, v2[perm], G_h)
    check_against_f64(H.grad.cpu().numpy(), ref, abs_sum, "torch dH after step")

    # registration: schema and shape function agree with the real operator
    torch.library.opcheck(ops.layer_forward, (H.detach(), vals.detach(), layer.layer_id),
                          test_utils=("test_schema", "test_faketensor"))

    # no CPU path
    with pytest.raises(RuntimeError, match="CUDA"):
        layer(H.detach().cpu())
    layer.close()
    with pytest.raises(RuntimeError, match="unknown or closed"):
        layer(H)
