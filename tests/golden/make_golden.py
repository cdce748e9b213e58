"""Generates tests/golden/*.json from the REFERENCE's own CPU-executable code for this path.

Run where the reference checkout is mounted (its path in $YITU_REFERENCE):

    make -C oracle ref            # compiles ccsrc/kernel/YiTu_GNN.cpp as it lies into oracle/_ref/
    python tests/golden/make_golden.py

Sources of truth
  build_part   the compiled reference function (ccsrc/kernel/YiTu_GNN.cpp:203-245), called through its pybind
               module; only this host function is invoked (the CUDA entry points of that file are unresolved)
  stitch_csr   the reference's pure-Python xgnn_h/block.py:36-67, loaded straight from the checkout
  to_csr       the reference's xgnn_h/convert.py:30-47 (the CSR convention its kernel tests use)

The fixtures are small integer vectors; the tests compare the CPU checker and the library's host routines
against them bit for bit.
"""
import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REFERENCE = os.environ.get("YITU_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")  # beside the repository


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def random_indptr(rng, n, max_deg, zero_last=False):
    deg = rng.integers(0, max_deg + 1, size=n)
    deg[rng.random(n) < 0.2] = 0
    if zero_last:
        deg[-1] = 0
    return np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)


def golden_build_part():
    sys.setdlopenflags(os.RTLD_LAZY)  # the CUDA launchers of the reference file stay unresolved
    sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
    import yitu_ref_ccsrc as ref
    rng = np.random.default_rng(2024)
    cases = [([0, 3, 3, 8, 9], 2), ([0, 3, 3, 8, 8], 2), ([0], 4), ([0, 0, 0], 3), ([0, 5], 5), ([0, 5], 32),
             ([0, 64, 65, 65, 200], 32),
             # pointers above 2^24 are rounded by the float32 storage of the reference
             ([0, 16777217, 33554435], 16777216)]
    for i in range(12):
        n = int(rng.integers(1, 60))
        cases.append((random_indptr(rng, n, int(rng.integers(1, 90)), zero_last=(i % 3 == 0)).tolist(),
                      int(rng.choice([1, 2, 3, 8, 32]))))
    out = []
    for indptr, ps in cases:
        part_ptr, part2node = ref.build_part(ps, torch.IntTensor(indptr))
        assert part_ptr.dtype == torch.float32 and part2node.dtype == torch.float32
        out.append({"part_size": ps, "indptr": indptr, "part_ptr": part_ptr.tolist(), "part2node": part2node.tolist()})
    return out


def golden_stitch_and_csr():
    block = _load(os.path.join(REFERENCE, "YiTu_GNN/YiTu_H/xgnn_h/block.py"), "ref_block")
    convert = _load(os.path.join(REFERENCE, "YiTu_GNN/YiTu_H/xgnn_h/convert.py"), "ref_convert")
    gen = torch.Generator().manual_seed(11)
    stitch, csr = [], []
    for case in range(6):
        n_rows = int(torch.randint(1, 20, (1,), generator=gen))
        blocks, desc = [], []
        for b in range(int(torch.randint(1, 5, (1,), generator=gen))):
            n_cols = int(torch.randint(1, 25, (1,), generator=gen))
            dense = (torch.rand(n_rows, n_cols, generator=gen) < 0.25).float()
            (indptr, indices), _ = convert.to_csr(dense)
            csr.append({"dense": dense.int().tolist(), "indptr": indptr.tolist(), "indices": indices.tolist()})
            blocks.append(block.Block(size=[n_rows, n_cols], adj=[indptr, indices]))
            desc.append({"n_cols": n_cols, "indptr": indptr.tolist(), "indices": indices.tolist()})
        st = block.stitch_csr(blocks)
        stitch.append({"n_rows": n_rows, "blocks": desc, "size": list(st.size), "indptr": st.adj_sparse[0].tolist(),
                       "indices": st.adj_sparse[1].tolist()})
    return stitch, csr


def main():
    bp = golden_build_part()
    stitch, csr = golden_stitch_and_csr()
    for name, obj in (("build_part", bp), ("stitch_csr", stitch), ("to_csr", csr)):
        with open(os.path.join(HERE, name + ".json"), "w") as f:
            json.dump(obj, f, separators=(",", ":"))
        print(name, len(obj), "cases")


if __name__ == "__main__":
    main()
