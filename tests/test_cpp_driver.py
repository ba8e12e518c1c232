"""The C++ mirror of the reference's call surface (include/spmm/**) and its bench driver."""
import importlib.util
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _builder():
    spec = importlib.util.spec_from_file_location("hpspmm_build", os.path.join(ROOT, "hp-spmm-sddmm_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_headers_and_driver_compile():
    path = _builder().build_test_all()
    assert path and os.path.exists(path)
    # without arguments the driver prints its usage and returns 2 (no GPU work)
    res = subprocess.run([path], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    assert res.returncode == 2 and "usage" in res.stderr


def test_driver_resumes_a_sweep(tmp_path):
    """A (graph, K) pair that already has a row in the CSV is skipped before any GPU work (no GPU needed)."""
    path = _builder().build_test_all()
    (tmp_path / "full_graph_res.csv").write_text(
        "rmat:12,4096,4096,60000,64,3.1,GE-SpMM: ,0.1,1,HP-SpMM ,0.1,1,HP-SpMM(COO): ,0.1,1,HP-SDDMM: ,0.1,1,"
        "CPU CSR loop: ,1,1\n")
    res = subprocess.run([path, "rmat:12", "64", "5"], cwd=tmp_path, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                         text=True, timeout=60)
    assert res.returncode == 0 and "skipped" in res.stdout
    assert len((tmp_path / "full_graph_res.csv").read_text().splitlines()) == 1


@pytest.mark.gpu
def test_driver_force_and_other_widths_are_measured(tmp_path):
    path = _builder().build_test_all()
    for args, rows in ((["rmat:10", "32", "3"], 1), (["rmat:10", "32", "3"], 1), (["rmat:10", "64", "3"], 2),
                       (["rmat:10", "32", "3", "--force"], 3)):
        res = subprocess.run([path] + args, cwd=tmp_path, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                             timeout=300)
        assert res.returncode == 0, res.stdout
        assert len((tmp_path / "full_graph_res.csv").read_text().splitlines()) == rows


@pytest.mark.gpu
@pytest.mark.parametrize("spec,K", [("cfg1", 32), ("rmat:12", 64), ("rmat:10", 128)])
def test_driver_runs_and_checks_itself(tmp_path, spec, K):
    path = _builder().build_test_all()
    res = subprocess.run([path, spec, str(K), "5"], cwd=tmp_path, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                         text=True, timeout=300)
    assert res.returncode == 0, res.stdout
    assert "PASSed" in res.stdout and "Wrong" not in res.stdout
    row = open(tmp_path / "full_graph_res.csv").read().strip().split(",")
    assert row[0] == spec and int(row[4]) == K
    assert "HP-SpMM " in row and float(row[row.index("HP-SpMM ") + 1]) > 0


@pytest.mark.gpu
def test_driver_reads_smtx(tmp_path, pkg):
    g = pkg.gen_uniform_degree(300, 300, 0, 12, seed=3)
    p = tmp_path / "g.smtx"
    with open(p, "w") as f:
        f.write("%d,%d,%d\n" % (g["M"], g["N"], g["nnz"]))
        f.write(" ".join(map(str, g["row_ptr"])) + "\n" + " ".join(map(str, g["col_idx"])) + "\n")
    path = _builder().build_test_all()
    res = subprocess.run([path, str(p), "32", "3"], cwd=tmp_path, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                         text=True, timeout=300)
    assert res.returncode == 0, res.stdout
