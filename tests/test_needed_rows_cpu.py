"""Needed-rows exchange of the row-sharded product, on CPU ranks.

hpspmm_shard_needed_rows is pure host code; here it is checked against numpy, and then three gloo
ranks run the whole protocol the C library runs over NCCL -- counts to every owner, row lists to
every owner, the owners' packed rows back -- with the CPU oracle as the local product, and the
stacked C must equal the unsharded product bit for bit (same rows, same order of terms)."""
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


def test_needed_rows_matches_numpy(pkg):
    g = pkg.gen_rmat(12, 8, seed=5)
    for world in (1, 2, 5):
        bounds = pkg.shard_bounds(g["row_ptr"], world)
        for r in range(world):
            _, ci, _ = pkg.shard_csr(g["row_ptr"], g["col_idx"], g["vals"], int(bounds[r]), int(bounds[r + 1]))
            cc, need, off = pkg.shard_needed_rows(ci, g["N"], bounds)
            uniq = np.unique(ci)
            assert np.array_equal(need, uniq)
            assert np.array_equal(need[cc], ci)
            assert off[0] == 0 and off[-1] == len(uniq)
            for s in range(world):
                part = need[off[s]:off[s + 1]]
                assert np.all((part >= bounds[s]) & (part < bounds[s + 1]))


def test_needed_rows_edge_cases(pkg):
    lib = pkg.load_library()
    # empty shard
    cc, need, off = pkg.shard_needed_rows(np.zeros(0, np.int32), 10, np.array([0, 4, 10]))
    assert len(cc) == 0 and len(need) == 0 and list(off) == [0, 0, 0]
    # an owner with no rows at all, an owner nobody references
    cc, need, off = pkg.shard_needed_rows(np.array([9, 0, 9, 3], np.int32), 10, np.array([0, 0, 4, 8, 10]))
    assert list(need) == [0, 3, 9] and list(off) == [0, 0, 2, 2, 3] and list(cc) == [2, 0, 2, 1]
    # a column outside [0, N) is refused, not renumbered
    with pytest.raises(pkg.HpspmmError) as e:
        pkg.shard_needed_rows(np.array([1, 10], np.int32), 10, np.array([0, 10]))
    assert e.value.status == pkg.ERR_BAD_CSR
    # bounds that do not span [0, N]
    with pytest.raises(pkg.HpspmmError) as e:
        pkg.shard_needed_rows(np.array([1], np.int32), 10, np.array([0, 5, 9]))
    assert e.value.status == pkg.ERR_INVALID
    assert lib is not None


def _rank_main(rank, world, port, out_dir):
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
    g = pkg.gen_rmat(11, 16, seed=23)
    N, K = g["N"], 32
    bounds = pkg.shard_bounds(g["row_ptr"], world)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    rp, ci, v = pkg.shard_csr(g["row_ptr"], g["col_idx"], g["vals"], lo, hi)
    B_own = pkg.host_fill_uniform(N * K, 23, 1, -1.0, 1.0).reshape(N, K)[lo:hi].copy()   # this rank's rows only

    cc, need, off = pkg.shard_needed_rows(ci, N, bounds)
    want = torch.tensor([int(off[s + 1] - off[s]) for s in range(world)], dtype=torch.int64)
    all_want = [torch.zeros(world, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(all_want, want)
    send_cnt = [int(all_want[d][rank]) for d in range(world)]
    # row lists to the owners
    reqs, lists = [], {}
    for d in range(world):
        if d == rank:
            continue
        if want[d] > 0:
            reqs.append(dist.isend(torch.from_numpy(need[off[d]:off[d + 1]].copy()), d))
        if send_cnt[d] > 0:
            lists[d] = torch.empty(send_cnt[d], dtype=torch.int32)
            reqs.append(dist.irecv(lists[d], d))
    for r in reqs:
        r.wait()
    # rows back
    B_local = np.empty((len(need), K), dtype=np.float32)
    B_local[off[rank]:off[rank + 1]] = B_own[need[off[rank]:off[rank + 1]] - lo]
    reqs, bufs = [], {}
    for d in range(world):
        if d == rank:
            continue
        if send_cnt[d] > 0:
            rows = lists[d].numpy() - lo
            assert rows.min() >= 0 and rows.max() < hi - lo
            reqs.append(dist.isend(torch.from_numpy(B_own[rows].copy()), d))
        if want[d] > 0:
            bufs[d] = torch.empty((int(want[d]), K), dtype=torch.float32)
            reqs.append(dist.irecv(bufs[d], d))
    for r in reqs:
        r.wait()
    for d, t in bufs.items():
        B_local[off[d]:off[d + 1]] = t.numpy()
    C_local = oracle_lib.spmm_f32(rp, cc, v, B_local)
    np.save(os.path.join(out_dir, "c_%d.npy" % rank), C_local)
    np.save(os.path.join(out_dir, "moved_%d.npy" % rank), np.array([len(need) - int(want[rank]), N - (hi - lo)]))
    dist.barrier()
    dist.destroy_process_group()


def test_three_rank_needed_rows_exchange_gloo(tmp_path, pkg, oracle):
    import torch.multiprocessing as mp
    world = 3
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    g = pkg.gen_rmat(11, 16, seed=23)
    B = pkg.host_fill_uniform(g["N"] * 32, 23, 1, -1.0, 1.0).reshape(g["N"], 32)
    ref = oracle.spmm_f32(g["row_ptr"], g["col_idx"], g["vals"], B)
    got = np.concatenate([np.load(tmp_path / ("c_%d.npy" % r)) for r in range(world)])
    assert np.array_equal(got, ref)
    # the exchange moved fewer rows than an all-gather would have
    for r in range(world):
        needed, allgather = np.load(tmp_path / ("moved_%d.npy" % r))
        assert needed < allgather
