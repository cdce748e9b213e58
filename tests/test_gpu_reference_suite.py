"""The reference's own kernel test file, run unmodified over the drop-in.

`make -C oracle ref_py` stages the reference's YiTu_GNN/YiTu_H/xgnn_h/*.py and test/test_kernel.py, as they lie, into
the git-ignored oracle/_ref/py.  Here yitu_b200.install_as_reference_modules() registers the drop-in under the name
`graph_ext`, the reference's OWN xgnn_h package (its sparse.py, bundle.py, block.py, convert.py) is imported on top of
it, and the reference's checks run as written: dense-math identities of gspmm, fused gsddmm (with and without
segments), the bundled GEMMs, stitch_csr + segmented softmax, and the horizontally fused pair, each forward and
backward at the reference's own tolerance (test_kernel.py:25,97,187,236,362).  Skipped where the staging is absent."""
import importlib
import os
import random
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAGED = os.path.join(ROOT, "oracle", "_ref", "py")


@pytest.fixture(scope="module")
def reference_checks():
    if not os.path.exists(os.path.join(STAGED, "test_kernel.py")):
        pytest.skip("the reference's test file is not staged (make -C oracle ref_py)")
    import yitu_b200
    yitu_b200.install_as_reference_modules()
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "xgnn_h" or k.startswith("xgnn_h.")}
    sys.path.insert(0, STAGED)
    try:
        mod = importlib.import_module("test_kernel")
        import xgnn_h
        assert os.path.dirname(xgnn_h.__file__) == os.path.join(STAGED, "xgnn_h"), "must be the reference's package"
        import graph_ext
        assert graph_ext.__name__ == "yitu_b200.graph_ext", "the reference's wrappers must sit on the drop-in"
        yield mod
    finally:
        sys.path.remove(STAGED)
        for k in [k for k in sys.modules if k == "xgnn_h" or k.startswith("xgnn_h.") or k == "test_kernel"]:
            del sys.modules[k]
        sys.modules.update(saved)


@pytest.mark.parametrize("check", ["check_gspmm", "check_gsddmm", "check_bundle", "check_stitch", "check_hfuse"])
def test_reference_check(reference_checks, check):
    random.seed(20 + len(check))
    torch.manual_seed(20 + len(check))
    for _ in range(1 if check == "check_hfuse" else 3):
        getattr(reference_checks, check)()
