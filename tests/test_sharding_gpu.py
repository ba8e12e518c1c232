"""Row-sharded SpMM on two GPUs: one process per GPU, nnz-balanced row blocks of A, B either
replicated or produced row-sharded and all-gathered with NCCL; C stays row-sharded.
Skipped when fewer than two GPUs are visible."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, b_sharded, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    pkg = entry.load_package()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    g = pkg.gen_rmat(14, 16, seed=31)
    N, K = g["N"], 64
    bounds = pkg.shard_bounds(g["row_ptr"], world)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    rp, ci, v = pkg.shard_csr(g["row_ptr"], g["col_idx"], g["vals"], lo, hi)
    t_rp, t_ci, t_v = (torch.from_numpy(np.ascontiguousarray(a)).to(dev) for a in (rp, ci, v))
    B_full = torch.from_numpy(pkg.host_fill_uniform(N * K, 31, 1, -1.0, 1.0).reshape(N, K))
    if b_sharded:
        rows_b = N // world
        own = B_full[rank * rows_b:(rank + 1) * rows_b].to(dev).contiguous()
        B = torch.empty((N, K), dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(B, own)          # lands in this GPU's own memory
    else:
        B = B_full.to(dev)
    C = torch.empty((hi - lo, K), dtype=torch.float32, device=dev)
    ctx = pkg.Context(rank)
    stream = torch.cuda.current_stream().cuda_stream
    ctx.spmm_csr(hi - lo, N, K, len(ci), t_rp.data_ptr(), t_ci.data_ptr(), t_v.data_ptr(), B.data_ptr(),
                 C.data_ptr(), stream=stream)
    torch.cuda.synchronize()
    np.save(os.path.join(out_dir, "c_%d.npy" % rank), C.cpu().numpy())
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("b_sharded", [False, True])
def test_two_gpu_row_sharded_product(tmp_path, pkg, oracle, b_sharded):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from helpers import check_against_f64
    mp.spawn(_rank_main, args=(2, _free_port(), b_sharded, str(tmp_path)), nprocs=2, join=True)
    g = pkg.gen_rmat(14, 16, seed=31)
    B = pkg.host_fill_uniform(g["N"] * 64, 31, 1, -1.0, 1.0).reshape(g["N"], 64)
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], B)
    got = np.concatenate([np.load(tmp_path / ("c_%d.npy" % r)) for r in range(2)])
    check_against_f64(got, ref, abs_sum, "two-GPU sharded product")


def _layer_rank_main(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import importlib
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    pkg = entry.load_package()
    sharded = importlib.import_module(pkg.__name__ + ".sharded")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    g = pkg.gen_rmat(14, 16, seed=33)
    N, K = g["N"], 64
    bounds = pkg.shard_bounds(g["row_ptr"], world)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    rp, ci, v = pkg.shard_csr(g["row_ptr"], g["col_idx"], g["vals"], lo, hi)
    t_rp, t_ci, t_v = (torch.from_numpy(np.ascontiguousarray(a)).to(dev) for a in (rp, ci, v))
    H = pkg.host_fill_uniform(N * K, 33, 1, -1.0, 1.0).reshape(N, K)
    dC = pkg.host_fill_uniform(N * K, 33, 2, -1.0, 1.0).reshape(N, K)
    local = sharded.GpuLocal(t_rp, t_ci, t_v, hi - lo, N, 128, dev)
    layer = sharded.ShardedLayer(local, N, bounds, rank, world, device=dev)
    C_own = layer.forward(torch.from_numpy(np.ascontiguousarray(H[lo:hi])).to(dev))
    dC_own = torch.from_numpy(np.ascontiguousarray(dC[lo:hi])).to(dev)
    dH_own = layer.backward_features(dC_own)
    dA_own = layer.backward_weights(dC_own)
    torch.cuda.synchronize()
    for name, t in (("c", C_own), ("dh", dH_own), ("da", dA_own)):
        np.save(os.path.join(out_dir, "%s_%d.npy" % (name, rank)), t.cpu().numpy())
    dist.barrier()
    local.close()
    dist.destroy_process_group()


def test_two_gpu_sharded_layer(tmp_path, pkg, oracle):
    """Forward (all-gather + SpMM), backward in the features (transposed SpMM + reduce-scatter) and in the
    weights (SDDMM on the gathered features) of a layer sharded over two GPUs."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from helpers import check_against_f64
    mp.spawn(_layer_rank_main, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    g = pkg.gen_rmat(14, 16, seed=33)
    N, K = g["N"], 64
    H = pkg.host_fill_uniform(N * K, 33, 1, -1.0, 1.0).reshape(N, K)
    dC = pkg.host_fill_uniform(N * K, 33, 2, -1.0, 1.0).reshape(N, K)
    cat = lambda name: np.concatenate([np.load(tmp_path / ("%s_%d.npy" % (name, r))) for r in range(2)])
    ref, abs_sum = oracle.spmm_f64(g["row_ptr"], g["col_idx"], g["vals"], H)
    check_against_f64(cat("c"), ref, abs_sum, "two-GPU layer forward")
    rpt, cit, vt, _ = oracle.csr_transpose(g["M"], N, g["row_ptr"], g["col_idx"], g["vals"])
    ref, abs_sum = oracle.spmm_f64(rpt, cit, vt, dC)
    check_against_f64(cat("dh"), ref, abs_sum, "two-GPU layer dH")
    ref, abs_sum = oracle.sddmm_f64(g["row_ptr"], g["col_idx"], dC, H)
    check_against_f64(cat("da"), ref, abs_sum, "two-GPU layer dA")
