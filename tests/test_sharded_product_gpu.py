"""Row-sharded product through the C ABI (hpspmm_comm_* / hpspmm_shard_plan_* / hpspmm_sharded_*).

One GPU: world = 1, which still runs the whole path except NCCL (row lists, renumbered columns, packing
into the local dense operand, slots, events).  Two GPUs: two processes, the communicator id carried
through a file, the rows of B exchanged over NCCL; skipped when fewer than two GPUs are visible."""
import multiprocessing
import os
import sys
import time

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _shard(pkg, g, world, rank):
    bounds = pkg.shard_bounds(g["row_ptr"], world)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    rp, ci, v = pkg.shard_csr(g["row_ptr"], g["col_idx"], g["vals"], lo, hi)
    return bounds, lo, hi, np.ascontiguousarray(rp), np.ascontiguousarray(ci), np.ascontiguousarray(v)


@pytest.mark.parametrize("exchange", [0, 1, 2])
def test_world_one_matches_plain_product(gpu_ctx, pkg, oracle, exchange):
    from helpers import check_against_f64
    ctx = gpu_ctx
    g = pkg.gen_rmat(13, 16, seed=41)          # heavy rows, 40 % empty rows, unreferenced columns
    M, N, nnz = g["M"], g["N"], g["nnz"]
    bounds, lo, hi, rp, ci, v = _shard(pkg, g, 1, 0)
    sp = pkg.ShardedSpmm(ctx, 1, 0, None, M, N, rp, ci, bounds, 516, exchange=exchange)
    info = sp.info()
    assert info["rows_received"] == 0 and info["rows_sent"] == 0
    assert info["rows_local"] == (len(np.unique(ci)) if exchange != 1 else N)
    d_v = ctx.upload(v)
    d_rp, d_ci = ctx.upload(rp), ctx.upload(ci)
    for K in (32, 64, 128, 20, 7, 516):          # 7: no 16-byte rows; 516: rows of 2064 bytes
        B = pkg.host_fill_uniform(N * K, 41, K, -1.0, 1.0).reshape(N, K)
        d_B = ctx.upload(B)
        d_C, d_C2 = ctx.alloc((M, K), np.float32), ctx.alloc((M, K), np.float32)
        sp.spmm(K, d_v, d_B, d_C)
        ctx.spmm_csr(M, N, K, nnz, d_rp, d_ci, d_v, d_B, d_C2)
        got, plain = d_C.to_host(), d_C2.to_host()
        ref, abs_sum = oracle.spmm_f64(rp, ci, v, B)
        check_against_f64(got, ref, abs_sum, "world-1 sharded product K=%d" % K)
        # same rows, same order of entries inside a row: only the chunking of split rows may differ
        assert np.max(np.abs(got - plain) / np.maximum(abs_sum, 1e-30)) <= 1e-6
    sp.close()


def test_slots_overlap_and_reuse(gpu_ctx, pkg, oracle):
    """Three products begun together and multiplied in turn, twice over (buffers and events reused)."""
    from helpers import check_against_f64
    ctx = gpu_ctx
    g = pkg.gen_rmat(12, 16, seed=43)
    M, N = g["M"], g["N"]
    bounds, lo, hi, rp, ci, v = _shard(pkg, g, 1, 0)
    sp = pkg.ShardedSpmm(ctx, 1, 0, None, M, N, rp, ci, bounds, 128)
    d_v = ctx.upload(v)
    Ks = (32, 64, 128)
    for step in range(2):
        Bs = {K: pkg.host_fill_uniform(N * K, 43 + step, K, -1.0, 1.0).reshape(N, K) for K in Ks}
        dB = {K: ctx.upload(Bs[K]) for K in Ks}
        dC = {K: ctx.alloc((M, K), np.float32) for K in Ks}
        for slot, K in enumerate(Ks):
            sp.begin(slot, K, dB[K])
        for slot, K in enumerate(Ks):
            sp.product(slot, K, d_v, dC[K])
        for K in Ks:
            ref, abs_sum = oracle.spmm_f64(rp, ci, v, Bs[K])
            check_against_f64(dC[K].to_host(), ref, abs_sum, "slots step %d K=%d" % (step, K))
    # a product on a slot nothing was begun on is refused, and so is a second begin before the product
    with pytest.raises(pkg.HpspmmError) as e:
        sp.product(3, 32, d_v, dC[32])
    assert e.value.status == pkg.ERR_INVALID
    sp.begin(0, 32, dB[32])
    with pytest.raises(pkg.HpspmmError) as e:
        sp.begin(0, 32, dB[32])
    assert e.value.status == pkg.ERR_INVALID
    sp.product(0, 32, d_v, dC[32])
    with pytest.raises(pkg.HpspmmError):
        sp.begin(4, 32, dB[32])
    sp.close()


def test_plan_argument_errors(gpu_ctx, pkg):
    ctx = gpu_ctx
    rp = np.array([0, 1, 2], np.int32)
    ci = np.array([0, 3], np.int32)
    with pytest.raises(pkg.HpspmmError) as e:      # bounds do not end at N
        pkg.ShardedSpmm(ctx, 1, 0, None, 2, 4, rp, ci, np.array([0, 3]), 32)
    assert e.value.status == pkg.ERR_INVALID
    with pytest.raises(pkg.HpspmmError) as e:      # column outside [0, N)
        pkg.ShardedSpmm(ctx, 1, 0, None, 2, 3, rp, ci, np.array([0, 3]), 32)
    assert e.value.status == pkg.ERR_BAD_CSR
    with pytest.raises(pkg.HpspmmError) as e:      # world > 1 without a communicator id
        pkg.ShardedSpmm(ctx, 2, 0, None, 2, 4, rp, ci, np.array([0, 2, 4]), 32)
    assert e.value.status == pkg.ERR_INVALID
    # the context is still usable
    d = ctx.alloc((4,), np.float32)
    ctx.fill(d, 4, 1.0)
    assert np.all(d.to_host() == 1.0)


def _rank_main(rank, world, exchange, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    if exchange == 10:      # the push transport with one rank unable to map its peer's buffers: all fall back to NCCL
        os.environ["HPSPMM_DEBUG_FAIL_PEER_MAPPING"] = "1"
        exchange = 0
    import __graft_entry__ as entry
    pkg = entry.load_package()
    id_path = os.path.join(out_dir, "comm_id.bin")
    if rank == 0:
        with open(id_path + ".tmp", "wb") as fh:
            fh.write(pkg.comm_unique_id())
        os.replace(id_path + ".tmp", id_path)
    deadline = time.time() + 60
    while not os.path.exists(id_path):
        if time.time() > deadline:
            raise RuntimeError("communicator id never arrived")
        time.sleep(0.05)
    comm_id = open(id_path, "rb").read()
    ctx = pkg.Context(rank)
    g = pkg.gen_rmat(14, 16, seed=31)
    N = g["N"]
    bounds, lo, hi, rp, ci, v = _shard(pkg, g, world, rank)
    sp = pkg.ShardedSpmm(ctx, world, rank, comm_id, hi - lo, N, rp, ci, bounds, 128, exchange=exchange)
    d_v = ctx.upload(v)
    Ks = (32, 64, 128)
    info = sp.info()
    for step in range(4):
        dB, dC = {}, {}
        for K in Ks:
            B_own = pkg.host_fill_uniform(N * K, 31 + step, K, -1.0, 1.0).reshape(N, K)[lo:hi]
            dB[K] = ctx.upload(np.ascontiguousarray(B_own))
            dC[K] = ctx.alloc((hi - lo, K), np.float32)
        if step % 2 == 0:
            for K in Ks:                       # one call per product
                sp.spmm(K, d_v, dB[K], dC[K])
        else:
            for slot, K in enumerate(Ks):      # all exchanges first, then the products
                sp.begin(slot, K, dB[K])
            for slot, K in enumerate(Ks):
                sp.product(slot, K, d_v, dC[K])
        for K in Ks:
            np.save(os.path.join(out_dir, "c_%d_%d_%d.npy" % (step, K, rank)), dC[K].to_host())
    np.save(os.path.join(out_dir, "info_%d.npy" % rank),
            np.array([info["rows_local"], info["rows_received"], info["rows_sent"], len(np.unique(ci)), N - (hi - lo)]))
    sp.close()
    ctx.close()


@pytest.mark.parametrize("exchange", [0, 1, 2, 10])
def test_two_gpu_exchange_and_product(tmp_path, pkg, oracle, exchange):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from helpers import check_against_f64
    world = 2
    mpctx = multiprocessing.get_context("spawn")
    procs = [mpctx.Process(target=_rank_main, args=(r, world, exchange, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    for p in procs:
        if p.is_alive():
            p.kill()
            pytest.fail("a rank did not finish")
        assert p.exitcode == 0
    g = pkg.gen_rmat(14, 16, seed=31)
    N = g["N"]
    for step in range(4):                      # four steps: both buffers of every slot are used twice
        for K in (32, 64, 128):
            B = pkg.host_fill_uniform(N * K, 31 + step, K, -1.0, 1.0).reshape(N, K)
            ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], B)
            got = np.concatenate([np.load(tmp_path / ("c_%d_%d_%d.npy" % (step, K, r))) for r in range(world)])
            check_against_f64(got, ref, abs_sum, "two-GPU sharded product step %d K=%d" % (step, K))
    sent = recv = 0
    for r in range(world):
        rows_local, rows_received, rows_sent, distinct, others = np.load(tmp_path / ("info_%d.npy" % r))
        recv += rows_received
        sent += rows_sent
        if exchange != 1:
            assert rows_local == distinct and rows_received < others
        else:
            assert rows_local == N and rows_received == others
    assert sent == recv
