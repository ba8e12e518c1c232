"""The load-path probes (needs a B200): the per-lane gather probe runs, and the TMA gather4 probe delivers
exactly the rows its index stream names (checked through the sum of everything its consumers read)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _replayed_rows(n, table_rows):
    """Row read by gather i = 0..n-1: the probes' multiplicative hash in 32-bit arithmetic."""
    i = np.arange(n, dtype=np.uint64)
    h = (i * np.uint64(2654435761)) & np.uint64(0xFFFFFFFF)
    h2 = ((h ^ (h >> np.uint64(15))) * np.uint64(2246822519)) & np.uint64(0xFFFFFFFF)
    return (h2 * np.uint64(table_rows)) >> np.uint64(32)


def test_gather_probe_reports_a_rate(gpu_ctx):
    gbs, ms = gpu_ctx.probe_gather(256, 100_000, 1 << 20, pattern=1, repeats=2)
    assert gbs > 100.0 and ms > 0.0


@pytest.mark.parametrize("row_bytes", [128, 256, 512])
@pytest.mark.parametrize("ctas_per_sm", [1, 3])
def test_tma_gather_probe_reads_the_named_rows(gpu_ctx, row_bytes, ctas_per_sm):
    table_rows = 50_021
    gbs, ms, checksum, done = gpu_ctx.probe_tma_gather(row_bytes, table_rows, 300_000, ctas_per_sm, repeats=2)
    assert gbs > 100.0 and ms > 0.0
    assert done >= 300_000 and done % (16384 // row_bytes) == 0
    rows = _replayed_rows(done, table_rows)
    assert rows.max() < table_rows
    # row r holds r mod 251 in each of its row_bytes / 4 columns; every partial sum stays below 2^24
    want = float((rows % np.uint64(251)).sum()) * (row_bytes // 4)
    assert checksum == want


def test_tma_gather_probe_rejects_bad_arguments(gpu_ctx, pkg):
    with pytest.raises(pkg.HpspmmError):
        gpu_ctx.probe_tma_gather(100, 1000, 1000)
    with pytest.raises(pkg.HpspmmError):
        gpu_ctx.probe_tma_gather(128, 1000, 1000, ctas_per_sm=7)
