"""Shared helpers for the parity tests: error metrics and device round trips via the C ABI."""
import numpy as np

# Tolerances (required: max relative error 1e-4, FP32 summation-order differences only).
# Measured over the whole GPU suite the backward error |got - ref| / sum|terms| peaks at 1.9e-7 (SpMM, rows
# of 40 K entries summed in chunks) and 4.5e-8 (SDDMM): FP32 rounding, 6e-8 per operation, grows with the
# logarithm of the row length when partial sums are combined pairwise.  BACKWARD_TOL = 2e-6 leaves a factor
# of ten for other graphs and rejects a dropped term that weighs 2e-6 of its row or more.
# The relative error of an element is its backward error times its condition number sum|terms| / |ref|, so a
# relative bound only makes sense up to some condition number: with the cut at 1000 (|ref| >= 1e-3 sum|terms|)
# the uniform-sparse full-size case (157 M elements, B in U(-1,1) cancelling) measured 1.07e-4 -- plain FP32
# rounding already passes 1e-4 there, whatever the kernel; at 400 the same run stays under 5e-5.
REL_TOL = 1e-4             # elementwise on well-conditioned elements, and normwise
BACKWARD_TOL = 2e-6        # |got - ref| / sum|terms|, every element
WELL_CONDITIONED = 2.5e-3  # an element is well conditioned if |ref| >= this * sum|terms| (condition number <= 400)


def check_against_f64(got, ref64, abs_sum, what=""):
    """Asserts the three error bounds; returns them for reporting."""
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == ref64.shape, (got.shape, ref64.shape)
    assert np.all(np.isfinite(got)), what + ": non-finite output"
    diff = np.abs(got - ref64)
    if diff.size == 0:
        return 0.0, 0.0, 0.0
    floor = np.maximum(abs_sum, 1e-30)
    backward = float(np.max(diff / floor))
    well = np.abs(ref64) >= WELL_CONDITIONED * floor
    rel = float(np.max(diff[well] / np.abs(ref64[well]))) if np.any(well) else 0.0
    denom = float(np.max(np.abs(ref64)))
    normwise = float(np.max(diff)) / denom if denom > 0 else float(np.max(diff))
    # elements whose every term is zero must be exactly zero
    assert np.all(got[abs_sum == 0] == 0), what + ": structural zero not zero"
    assert backward <= BACKWARD_TOL, "%s: backward error %g" % (what, backward)
    assert rel <= REL_TOL, "%s: relative error %g" % (what, rel)
    assert normwise <= REL_TOL, "%s: normwise error %g" % (what, normwise)
    return backward, rel, normwise


def csr_from_rows(rows, N, rng=None, vals=None):
    """rows: list of column lists -> (row_ptr, col_idx, vals)"""
    row_ptr = np.zeros(len(rows) + 1, dtype=np.int32)
    for i, r in enumerate(rows):
        row_ptr[i + 1] = row_ptr[i] + len(r)
    col_idx = np.array([c for r in rows for c in r], dtype=np.int32).reshape(-1)
    if vals is None:
        rng = rng or np.random.default_rng(0)
        vals = rng.uniform(-1, 1, size=len(col_idx)).astype(np.float32)
    return row_ptr, col_idx, np.asarray(vals, dtype=np.float32)


def random_csr(M, N, degrees, seed):
    """CSR with the given per-row degrees, distinct sorted random columns, values U(-1,1)."""
    rng = np.random.default_rng(seed)
    rows = []
    for d in degrees:
        d = int(min(d, N))
        if d == 0:
            rows.append([])
        elif d * 4 > N:
            rows.append(np.sort(rng.choice(N, size=d, replace=False)).tolist())
        else:
            s = set()
            while len(s) < d:
                s.update(rng.integers(0, N, size=d - len(s)).tolist())
            rows.append(sorted(s))
    return csr_from_rows(rows, N, rng)


GUARD = 256  # floats of canary on each side of an output


def guarded_output(ctx, shape, fill=np.float32(-777.25)):
    """Device output with canary bands; returns (buffer, pointer to payload, checker)."""
    n = int(np.prod(shape))
    total = n + 2 * GUARD
    buf = ctx.alloc((total,), np.float32)
    ctx.fill(buf, total, float(fill))
    payload = buf.ptr + GUARD * 4

    def read():
        host = buf.to_host()
        assert np.all(host[:GUARD] == fill), "write before the output buffer"
        assert np.all(host[GUARD + n:] == fill), "write past the output buffer"
        return host[GUARD:GUARD + n].reshape(shape).copy()

    return buf, payload, read


def gpu_spmm(ctx, pkg, row_ptr, col_idx, vals, B, N=None, opts=None, use_plan=False, guard=True,
             plan_cols=True):
    M = len(row_ptr) - 1
    N = B.shape[0] if N is None else N
    K = B.shape[1]
    nnz = len(col_idx)
    d_rp, d_ci, d_v, d_B = ctx.upload(row_ptr), ctx.upload(col_idx), ctx.upload(vals), ctx.upload(B)
    buf, c_ptr, read = guarded_output(ctx, (M, K))
    plan = None
    if use_plan:
        plan = ctx.plan_create(M, nnz, d_rp, K, opts, N=N, col_idx=d_ci if plan_cols else None)
    ctx.spmm_csr(M, N, K, nnz, d_rp, d_ci, d_v, d_B, c_ptr, plan=plan, opts=opts)
    ctx.stream_sync()
    C = read()
    if plan:
        ctx.plan_destroy(plan)
    for b in (d_rp, d_ci, d_v, d_B, buf):
        b.free()
    return C


# ---- the library's counter-based generator, restated in numpy (csrc/hpspmm_internal.h) -----------------
_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix64(z):
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def uniform_at(seed, stream_id, indices, lo, hi):
    """Elements `indices` of the stream hpspmm_fill_uniform_f32(seed, stream_id, lo, hi) produces, as float32:
    rows of a dense operand can be regenerated on the host without holding the operand."""
    with np.errstate(over="ignore"):
        idx = np.asarray(indices, dtype=np.uint64)
        k = _mix64(np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15) + np.uint64(stream_id) + np.uint64(0x632BE59BD9B4E019))
        bits = _mix64(k + idx * np.uint64(0x9E3779B97F4A7C15))
    u = (bits >> np.uint64(40)).astype(np.float64) * (1.0 / 16777216.0)
    # the library computes fmaf(span, u, lo) in FP32: one rounding of the exact value, as here
    span = np.float64(np.float32(hi) - np.float32(lo))
    return (span * u + np.float64(np.float32(lo))).astype(np.float32)


def uniform_rows(seed, stream_id, rows, K, lo, hi):
    """Rows `rows` of the N x K matrix filled by hpspmm_fill_uniform_f32 (element i = row * K + column)."""
    rows = np.asarray(rows, dtype=np.uint64)
    idx = rows[:, None] * np.uint64(K) + np.arange(K, dtype=np.uint64)[None, :]
    return uniform_at(seed, stream_id, idx, lo, hi)
