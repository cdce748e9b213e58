import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device")


ACHIEVED = {}  # test family -> [worst max-norm relative error, worst element-wise relative error, comparisons]


def record_error(family, max_norm_rel, elem_rel):
    """Keeps the worst achieved errors per test family; written as JSON to the path in $YITU_PARITY_REPORT (if set)
    at the end of the session, so the tolerance that the tests state can be read beside the error that the kernels
    actually reach."""
    cur = ACHIEVED.setdefault(family, [0.0, 0.0, 0])
    cur[0], cur[1], cur[2] = max(cur[0], float(max_norm_rel)), max(cur[1], float(elem_rel)), cur[2] + 1


def pytest_sessionfinish(session, exitstatus):
    path = os.environ.get("YITU_PARITY_REPORT")
    if ACHIEVED and path:
        import json
        with open(path, "w") as f:
            json.dump({k: {"max_norm_rel": v[0], "elementwise_rel_where_ref_ge_1pct_of_max": v[1], "comparisons": v[2]}
                       for k, v in sorted(ACHIEVED.items())}, f, indent=1)


def assert_close(got, ref, rtol=1e-5, what=""):
    """fp32 parity bar of the aggregation kernels: |got - ref| <= rtol * (|ref| + max|ref|).

    The max|ref| term covers entries that are small through cancellation: a sum of n terms of size s carries
    a reduction-order error ~ eps*sqrt(n)*s whatever the sum's own size.  The achieved errors are recorded per
    test family (first word of `what`): max|got-ref| / max|ref|, and the worst element-wise relative error over
    the entries with |ref| >= 1 % of max|ref| (below that, cancellation makes a relative figure meaningless)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, "%s shape %s vs %s" % (what, got.shape, ref.shape)
    if ref.size == 0:
        return
    assert np.isfinite(got).all(), "%s: non-finite values" % what
    scale = np.abs(ref).max()
    if scale > 0:
        big = np.abs(ref) >= 0.01 * scale
        record_error((what.split() or ["?"])[0], np.abs(got - ref).max() / scale,
                     (np.abs(got - ref)[big] / np.abs(ref)[big]).max())
    err = np.abs(got - ref) - rtol * (np.abs(ref) + scale)
    worst = err.max()
    assert worst <= 0, "%s: max excess %.3e (max|ref|=%.3e, max abs err %.3e)" % (
        what, worst, scale, np.abs(got - ref).max())


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


def random_csr(rng, n_rows, n_cols, density=0.02, hubs=0, hub_deg=0, empty_rows=True):
    """Random CSR by destination with sorted unique columns; a few hub rows if asked."""
    rows = []
    for r in range(n_rows):
        if hubs and r % max(1, n_rows // hubs) == 1:
            k = min(n_cols, hub_deg)
        else:
            k = rng.binomial(n_cols, density)
            if empty_rows and r % 7 == 3:
                k = 0
        rows.append(np.sort(rng.choice(n_cols, size=k, replace=False)).astype(np.int32))
    indptr = np.zeros(n_rows + 1, dtype=np.int32)
    indptr[1:] = np.cumsum([len(r) for r in rows])
    indices = np.concatenate(rows) if rows else np.zeros(0, dtype=np.int32)
    return indptr, indices.astype(np.int32)
