"""Multi-GPU row sharding on CPU: the partitioner, and a world-size-2 gloo run in which every
rank multiplies its shard with the CPU oracle and the gathered C equals the unsharded product."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, b_sharded, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    import oracle_lib
    pkg = entry.load_package()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = pkg.gen_rmat(11, 16, seed=21)
    K = 32
    bounds = pkg.shard_bounds(g["row_ptr"], world)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    rp, ci, v = pkg.shard_csr(g["row_ptr"], g["col_idx"], g["vals"], lo, hi)
    if b_sharded:
        # B is produced row-sharded with the same boundaries (a GNN layer's output): all-gather it
        mine = pkg.host_fill_uniform(g["N"] * K, 21, 1, -1.0, 1.0).reshape(g["N"], K)[lo:hi]
        sizes = [int(bounds[r + 1] - bounds[r]) for r in range(world)]
        parts = [torch.empty((s, K), dtype=torch.float32) for s in sizes]
        pad = max(sizes)
        padded = torch.zeros((pad, K), dtype=torch.float32)
        padded[:hi - lo] = torch.from_numpy(np.ascontiguousarray(mine))
        gathered = [torch.empty((pad, K), dtype=torch.float32) for _ in range(world)]
        dist.all_gather(gathered, padded)
        B = torch.cat([gathered[r][:sizes[r]] for r in range(world)]).numpy()
    else:
        B = pkg.host_fill_uniform(g["N"] * K, 21, 1, -1.0, 1.0).reshape(g["N"], K)   # replicated
    C_local = oracle_lib.spmm_f32(rp, ci, v, B)
    np.save(os.path.join(out_dir, "c_%d.npy" % rank), C_local)
    np.save(os.path.join(out_dir, "nnz_%d.npy" % rank), np.array([len(ci)]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("b_sharded", [False, True])
def test_two_rank_row_sharding_gloo(tmp_path, pkg, oracle, b_sharded):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_rank_main, args=(2, port, b_sharded, str(tmp_path)), nprocs=2, join=True)
    g = pkg.gen_rmat(11, 16, seed=21)
    B = pkg.host_fill_uniform(g["N"] * 32, 21, 1, -1.0, 1.0).reshape(g["N"], 32)
    want = oracle.spmm_f32(g["row_ptr"], g["col_idx"], g["vals"], B)
    got = np.concatenate([np.load(tmp_path / ("c_%d.npy" % r)) for r in range(2)])
    assert np.array_equal(got, want)          # row blocks are independent: bit-identical
    nnz = [int(np.load(tmp_path / ("nnz_%d.npy" % r))[0]) for r in range(2)]
    assert sum(nnz) == g["nnz"] and abs(nnz[0] - nnz[1]) <= 2 * np.diff(g["row_ptr"]).max()


class _OracleLocal:
    """Stand-in for the GPU products so that the exchange logic of ShardedLayer runs on CPU ranks."""

    def __init__(self, oracle_lib, rp, ci, v, M_own, N):
        self.o, self.rp, self.ci, self.v, self.M_own, self.N = oracle_lib, rp, ci, v, M_own, N
        self.rpt, self.cit, self.vt, _ = oracle_lib.csr_transpose(M_own, N, rp, ci, v)

    def forward(self, H):
        import torch
        return torch.from_numpy(self.o.spmm_f32(self.rp, self.ci, self.v, H.numpy()))

    def backward_features(self, dC, out):
        import torch
        out.copy_(torch.from_numpy(self.o.spmm_f32(self.rpt, self.cit, self.vt, dC.numpy())))
        return out

    def backward_weights(self, dC, H):
        import torch
        ref, _ = self.o.sddmm_f64(self.rp, self.ci, dC.numpy(), H.numpy())
        return torch.from_numpy(ref.astype(np.float32))


def _layer_rank_main(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import importlib
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    import oracle_lib
    pkg = entry.load_package()
    sharded = importlib.import_module(pkg.__name__ + ".sharded")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = pkg.gen_rmat(10, 16, seed=23)
    N, K = g["N"], 32
    bounds = pkg.shard_bounds(g["row_ptr"], world)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    rp, ci, v = pkg.shard_csr(g["row_ptr"], g["col_idx"], g["vals"], lo, hi)
    H = pkg.host_fill_uniform(N * K, 23, 1, -1.0, 1.0).reshape(N, K)
    dC = pkg.host_fill_uniform(N * K, 23, 2, -1.0, 1.0).reshape(N, K)
    layer = sharded.ShardedLayer(_OracleLocal(oracle_lib, rp, ci, v, hi - lo, N), N, bounds, rank, world)
    C_own = layer.forward(torch.from_numpy(np.ascontiguousarray(H[lo:hi])))
    dC_own = torch.from_numpy(np.ascontiguousarray(dC[lo:hi]))
    dH_own = layer.backward_features(dC_own)
    dA_own = layer.backward_weights(dC_own)
    for name, t in (("c", C_own), ("dh", dH_own), ("da", dA_own)):
        np.save(os.path.join(out_dir, "%s_%d.npy" % (name, rank)), t.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_layer_exchange_gloo(tmp_path, pkg, oracle, world):
    """Forward all-gather, backward reduce-scatter and the SDDMM on the gathered features, on CPU ranks."""
    import torch.multiprocessing as mp
    from helpers import check_against_f64
    mp.spawn(_layer_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    g = pkg.gen_rmat(10, 16, seed=23)
    N, K = g["N"], 32
    H = pkg.host_fill_uniform(N * K, 23, 1, -1.0, 1.0).reshape(N, K)
    dC = pkg.host_fill_uniform(N * K, 23, 2, -1.0, 1.0).reshape(N, K)
    cat = lambda name: np.concatenate([np.load(tmp_path / ("%s_%d.npy" % (name, r))) for r in range(world)])
    assert np.array_equal(cat("c"), oracle.spmm_f32(g["row_ptr"], g["col_idx"], g["vals"], H))
    rpt, cit, vt, _ = oracle.csr_transpose(g["M"], N, g["row_ptr"], g["col_idx"], g["vals"])
    ref, abs_sum = oracle.spmm_f64(rpt, cit, vt, dC)
    check_against_f64(cat("dh"), ref, abs_sum, "sharded dH")       # summed across ranks: order differs
    ref, abs_sum = oracle.sddmm_f64(g["row_ptr"], g["col_idx"], dC, H)
    check_against_f64(cat("da"), ref, abs_sum, "sharded dA")


def test_shards_tile_the_matrix_for_every_world_size(pkg, oracle):
    g = pkg.gen_erdos_renyi(5000, 5000, 20.0, seed=22)
    B = pkg.host_fill_uniform(5000 * 32, 22, 1, -1.0, 1.0).reshape(5000, 32)
    want = oracle.spmm_f32(g["row_ptr"], g["col_idx"], g["vals"], B)
    for G in (1, 2, 3, 4, 8):
        bounds = pkg.shard_bounds(g["row_ptr"], G)
        parts = []
        for r in range(G):
            rp, ci, v = pkg.shard_csr(g["row_ptr"], g["col_idx"], g["vals"], int(bounds[r]), int(bounds[r + 1]))
            parts.append(oracle.spmm_f32(rp, ci, v, B))
        assert np.array_equal(np.concatenate(parts), want)
        sizes = np.diff(g["row_ptr"][bounds])
        assert sizes.max() - sizes.min() <= 2 * np.diff(g["row_ptr"]).max()


def test_weighted_bounds(pkg):
    g = pkg.gen_rmat(12, 16, seed=27)
    rp, M = g["row_ptr"], g["M"]
    for G in (1, 2, 3, 8):
        assert np.array_equal(pkg.shard_bounds_weighted(rp, G, 0.0), pkg.shard_bounds(rp, G))
        for w in (0.5, 2.0, 16.0):
            b = pkg.shard_bounds_weighted(rp, G, w)
            assert b[0] == 0 and b[-1] == M and np.all(np.diff(b) >= 0)
            cost = rp[b].astype(np.float64) + w * b
            parts = np.diff(cost)
            # every block within one row's cost of the ideal share
            assert np.all(np.abs(parts - cost[-1] / G) <= np.diff(rp).max() + w + 1)
    # a heavier row weight moves the first cut (the hub rows come first in an R-MAT graph) to later rows
    assert pkg.shard_bounds_weighted(rp, 2, 8.0)[1] > pkg.shard_bounds(rp, 2)[1]
    with pytest.raises(pkg.HpspmmError):
        pkg.shard_bounds_weighted(rp, 2, -1.0)


def test_degenerate_shards(pkg):
    rp = np.array([0, 0, 0, 5, 5], dtype=np.int32)      # one non-empty row, four shards
    b = pkg.shard_bounds(rp, 4)
    assert b[0] == 0 and b[-1] == 4 and np.all(np.diff(b) >= 0)
    assert sum(int(rp[b[i + 1]] - rp[b[i]]) for i in range(4)) == 5
    empty = np.zeros(7, dtype=np.int32)
    assert list(pkg.shard_bounds(empty, 3)) == [0, 0, 0, 6]


def _leaving_rank_main(rank, world, port, out_dir):
    """Rank 1 leaves between two steps (an exception on the host, nothing in flight); rank 0's next exchange
    must end with an error after the process group's timeout instead of waiting for ever."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import datetime
    import importlib
    import time
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    import oracle_lib
    pkg = entry.load_package()
    sharded = importlib.import_module(pkg.__name__ + ".sharded")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    g = pkg.gen_rmat(9, 8, seed=29)
    N, K = g["N"], 32
    bounds = pkg.shard_bounds(g["row_ptr"], world)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    rp, ci, v = pkg.shard_csr(g["row_ptr"], g["col_idx"], g["vals"], lo, hi)
    H = pkg.host_fill_uniform(N * K, 29, 1, -1.0, 1.0).reshape(N, K)
    H_own = torch.from_numpy(np.ascontiguousarray(H[lo:hi]))
    layer = sharded.ShardedLayer(_OracleLocal(oracle_lib, rp, ci, v, hi - lo, N), N, bounds, rank, world)
    layer.forward(H_own)                       # step 1: everybody takes part
    dist.barrier()
    if rank == 1:
        open(os.path.join(out_dir, "rank1_left"), "w").close()
        os._exit(17)                           # leaves without a word, between steps
    t0 = time.time()
    try:
        layer.forward(H_own)                   # step 2: the partner is gone
        outcome = "completed"
    except Exception as exc:                   # gloo reports the lost peer or the timeout
        outcome = "error: %s" % type(exc).__name__
    with open(os.path.join(out_dir, "rank0_outcome"), "w") as fh:
        fh.write("%s after %.1f s" % (outcome, time.time() - t0))
    os._exit(0)


def test_a_rank_that_leaves_ends_the_next_exchange_with_an_error(tmp_path):
    import multiprocessing
    ctx = multiprocessing.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_leaving_rank_main, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
    alive = [p.is_alive() for p in procs]
    for p in procs:
        if p.is_alive():
            p.kill()
    assert not any(alive), "a rank hung after its partner left"
    assert (tmp_path / "rank1_left").exists() and procs[1].exitcode == 17
    outcome = (tmp_path / "rank0_outcome").read_text()
    assert outcome.startswith("error"), outcome
