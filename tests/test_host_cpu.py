"""Host-side parts of the library and the C-ABI surface, without a GPU."""
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.load_library()
    header = open(os.path.join(ROOT, "include", "hpspmm.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = re.findall(r"HPSPMM_API\s+[\w\s\*]+?\b(hpspmm_\w+)\s*\(", header)
    assert len(declared) >= 45
    for name in declared:
        assert hasattr(lib, name), "library does not export " + name
        assert name in pkg.PROTOTYPES, "binding lacks " + name
    assert sorted(set(declared)) == sorted(pkg.PROTOTYPES)


def test_status_strings(pkg):
    lib = pkg.load_library()
    assert lib.hpspmm_status_string(0) == b"ok"
    assert b"CSR" in lib.hpspmm_status_string(pkg.ERR_BAD_CSR)
    assert lib.hpspmm_version().startswith(b"hpspmm")


def test_cfg1_generator_shape_and_determinism(pkg):
    g = pkg.gen_uniform_degree(4096, 4096, 1, 32, seed=1, vals_kind=pkg.VALS_UPM1)
    h = pkg.gen_uniform_degree(4096, 4096, 1, 32, seed=1, vals_kind=pkg.VALS_UPM1)
    for k in ("row_ptr", "col_idx", "vals"):
        assert np.array_equal(g[k], h[k])
    deg = np.diff(g["row_ptr"])
    assert deg.min() >= 1 and deg.max() <= 32 and 60_000 < g["nnz"] < 75_000
    for r in range(0, 4096, 97):
        cols = g["col_idx"][g["row_ptr"][r]:g["row_ptr"][r + 1]]
        assert np.all(np.diff(cols) > 0) and cols.min() >= 0 and cols.max() < 4096
    assert g["vals"].min() >= -1 and g["vals"].max() < 1 and abs(g["vals"].mean()) < 0.02
    other = pkg.gen_uniform_degree(4096, 4096, 1, 32, seed=2, vals_kind=pkg.VALS_UPM1)
    assert not np.array_equal(other["col_idx"][:100], g["col_idx"][:100])


def test_rmat_generator_properties(pkg):
    import scipy.sparse as sp
    g = pkg.gen_rmat(12, 16, seed=2)
    n = 1 << 12
    assert g["M"] == n and g["N"] == n and g["row_ptr"][-1] == g["nnz"]
    A = sp.csr_matrix((np.ones(g["nnz"]), g["col_idx"], g["row_ptr"]), shape=(n, n))
    assert (A != A.T).nnz == 0                      # symmetric pattern
    assert A.has_sorted_indices or np.all(np.diff(g["col_idx"][:g["row_ptr"][1]]) > 0)
    for r in range(0, n, 53):
        cols = g["col_idx"][g["row_ptr"][r]:g["row_ptr"][r + 1]]
        assert np.all(np.diff(cols) > 0)            # sorted, no duplicates
    deg = np.diff(g["row_ptr"])
    assert deg.max() > 20 * max(deg.mean(), 1)      # power-law skew
    assert g["nnz"] <= 16 * n and g["nnz"] > 8 * n
    assert g["vals"].min() >= 0 and g["vals"].max() < 1


def test_erdos_renyi_generator(pkg):
    g = pkg.gen_erdos_renyi(20000, 20000, 50.0, seed=3)
    deg = np.diff(g["row_ptr"])
    assert abs(deg.mean() - 50) < 0.5 and abs(deg.var() - 50) < 3   # Poisson
    cols = g["col_idx"][g["row_ptr"][17]:g["row_ptr"][18]]
    assert np.all(np.diff(cols) > 0)


def test_host_fill_uniform(pkg):
    a = pkg.host_fill_uniform(10000, 5, 9, -1.0, 1.0)
    b = pkg.host_fill_uniform(10000, 5, 9, -1.0, 1.0)
    assert np.array_equal(a, b) and a.min() >= -1 and a.max() < 1 and abs(a.mean()) < 0.03
    assert not np.array_equal(a, pkg.host_fill_uniform(10000, 5, 10, -1.0, 1.0))
    # a prefix of a longer stream is the same stream
    assert np.array_equal(a[:100], pkg.host_fill_uniform(100, 5, 9, -1.0, 1.0))


def test_shard_bounds_match_oracle(pkg, oracle):
    g = pkg.gen_rmat(12, 16, seed=4)
    for G in (1, 2, 4, 8, 7):
        got = pkg.shard_bounds(g["row_ptr"], G)
        assert np.array_equal(got, oracle.shard_bounds(g["row_ptr"], G))   # bit exact
        sizes = [g["row_ptr"][got[i + 1]] - g["row_ptr"][got[i]] for i in range(G)]
        assert sum(sizes) == g["nnz"]
        assert max(sizes) - min(sizes) <= 2 * np.diff(g["row_ptr"]).max()


def test_shard_csr_rebases(pkg):
    g = pkg.gen_uniform_degree(1000, 1000, 0, 9, seed=5)
    b = pkg.shard_bounds(g["row_ptr"], 4)
    pieces = []
    for i in range(4):
        rp, ci, v = pkg.shard_csr(g["row_ptr"], g["col_idx"], g["vals"], int(b[i]), int(b[i + 1]))
        assert rp[0] == 0 and rp[-1] == len(ci) == len(v)
        assert np.array_equal(np.diff(rp), np.diff(g["row_ptr"][b[i]:b[i + 1] + 1]))
        pieces.append(ci)
    assert np.array_equal(np.concatenate(pieces), g["col_idx"])


def test_smtx_reader(pkg, tmp_path):
    g = pkg.gen_uniform_degree(50, 40, 0, 7, seed=6)
    p = tmp_path / "g.smtx"
    with open(p, "w") as f:
        f.write("%d, %d, %d\n" % (g["M"], g["N"], g["nnz"]))
        f.write(" ".join(map(str, g["row_ptr"])) + "\n")
        f.write(" ".join(map(str, g["col_idx"])) + "\n")
    h = pkg.read_smtx(str(p))
    assert (h["M"], h["N"], h["nnz"]) == (g["M"], g["N"], g["nnz"])
    assert np.array_equal(h["row_ptr"], g["row_ptr"]) and np.array_equal(h["col_idx"], g["col_idx"])
    assert np.all(h["vals"] == 1.0)   # the reference's loader sets every value to 1.0
    bad = tmp_path / "bad.smtx"
    bad.write_text("3,3,2\n0 1 2\n0\n")
    with pytest.raises(pkg.HpspmmError):
        pkg.read_smtx(str(bad))


def test_metric_matches_oracle(pkg, oracle):
    assert pkg.gflops(123456, 64, 0.37) == oracle.gflops(123456, 64, 0.37)
    g = pkg.gen_rmat(10, 8, seed=1)
    lib = pkg.load_library()
    assert lib.hpspmm_row_length_cv(g["M"], g["row_ptr"].ctypes.data) == pytest.approx(
        oracle.row_length_cv(g["row_ptr"]), rel=1e-12)
    assert pkg.spmm_algorithmic_bytes(10, 20, 32, 100) == 4 * 11 + 800 + 4 * 32 * 20 + 4 * 32 * 10


def test_context_needs_a_gpu_or_fails_loudly(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    with pytest.raises(pkg.HpspmmError):
        pkg.Context(0)


def test_torch_front_end_registers_and_has_no_cpu_path(pkg):
    """The autograd front-end imports without a GPU, registers its three operators, and refuses CPU tensors."""
    import importlib
    import torch
    ops = importlib.import_module(pkg.__name__ + ".torch_ops")
    for name in ("layer_forward", "layer_backward_features", "layer_backward_weights"):
        assert hasattr(torch.ops.hpspmm, name)
    rp = torch.zeros(5, dtype=torch.int32)
    ci = torch.zeros(0, dtype=torch.int32)
    v = torch.zeros(0, dtype=torch.float32)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.TorchLayer(rp, ci, v, 4, 4, 32)
    with pytest.raises(RuntimeError, match="unknown or closed"):
        ops.layer_forward(torch.zeros(4, 32), v, 12345)
    # the shape functions need no device
    ops._layers[-1] = {"M": 7, "N": 4, "nnz": 9}
    try:
        with torch._subclasses.fake_tensor.FakeTensorMode():
            H = torch.empty(4, 32)
            assert ops.layer_forward(H, torch.empty(9), -1).shape == (7, 32)
            assert ops.layer_backward_features(torch.empty(7, 32), torch.empty(9), -1).shape == (4, 32)
            assert ops.layer_backward_weights(torch.empty(7, 32), H, -1).shape == (9,)
    finally:
        del ops._layers[-1]


def test_row_order_reader(pkg, tmp_path):
    """One line of M row ids (the reference's .cugraph_reorder file); anything but a permutation is refused."""
    rng = np.random.default_rng(5)
    order = rng.permutation(1000).astype(np.int32)
    good = tmp_path / "g.cugraph_reorder"
    good.write_text(" ".join(str(int(x)) for x in order) + "\n")
    assert np.array_equal(pkg.read_row_order(str(good), 1000), order)
    for name, text in (("dup", "0 1 1 3"), ("range", "0 1 2 4"), ("short", "0 1 2"), ("neg", "0 -1 2 3")):
        bad = tmp_path / name
        bad.write_text(text + "\n")
        with pytest.raises(pkg.HpspmmError):
            pkg.read_row_order(str(bad), 4)
    with pytest.raises(pkg.HpspmmError):
        pkg.read_row_order(str(tmp_path / "missing"), 4)


def test_numpy_restatement_of_the_generator_matches_the_library(pkg):
    """tests/helpers.uniform_rows regenerates rows of a device-filled operand on the host; it must equal the
    library's own host generator bit for bit."""
    from helpers import uniform_at, uniform_rows
    for seed, stream, lo, hi in ((2, 132, -1.0, 1.0), (9, 7, 0.0, 1.0), (4, 128, -0.5, 2.5)):
        want = pkg.host_fill_uniform(5000, seed, stream, lo, hi)
        assert np.array_equal(uniform_at(seed, stream, np.arange(5000), lo, hi), want)
    K = 128
    full = pkg.host_fill_uniform(300 * K, 4, 128, -1.0, 1.0).reshape(300, K)
    rows = np.array([0, 17, 299, 17])
    assert np.array_equal(uniform_rows(4, 128, rows, K, -1.0, 1.0), full[rows])
    # far beyond 2^31 elements: compare with a window generated by the library at that offset
    big = np.array([2 ** 31 + 5, 2 ** 32 + 1, 17_499_999 * 128 + 127], dtype=np.uint64)
    got = uniform_at(9, 1, big, -1.0, 1.0)
    assert got.dtype == np.float32 and np.all((got >= -1.0) & (got < 1.0))
