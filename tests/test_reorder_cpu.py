"""The CPU restatement of the community reordering: it must return a permutation, leave the graph isomorphic, be
reproducible, and put planted communities back into contiguous id ranges after their ids were shuffled."""
import numpy as np


def planted_graph(rng, n, community, degree, p_intra):
    """Edges mostly inside blocks of `community` consecutive ids, then the ids are shuffled."""
    m = n * degree
    src = rng.integers(0, n, size=m)
    inside = rng.random(m) < p_intra
    dst = np.where(inside, (src // community) * community + rng.integers(0, community, size=m), rng.integers(0, n, size=m))
    shuffle = rng.permutation(n)
    return shuffle[src].astype(np.int32), shuffle[dst].astype(np.int32), shuffle


def test_reorder_is_a_permutation_and_reproducible(oracle):
    rng = np.random.default_rng(0)
    n = 3000
    src, dst = rng.integers(0, n, 20000), rng.integers(0, n, 20000)
    a, levels, top = oracle.reorder_communities(n, src, dst)
    b, _, _ = oracle.reorder_communities(n, src, dst)
    assert np.array_equal(a, b)
    assert np.array_equal(np.sort(a), np.arange(n))
    assert 1 <= levels <= 32 and 1 <= top < n
    # the relabelled edge multiset is the image of the original one
    inv = np.empty(n, dtype=np.int64)
    inv[a] = np.arange(n)
    assert np.array_equal(inv[a[src]], src) and np.array_equal(inv[a[dst]], dst)


def test_reorder_edge_cases(oracle):
    ident, levels, top = oracle.reorder_communities(6, [], [])
    assert ident.tolist() == list(range(6)) and levels == 0 and top == 6
    ident, levels, _ = oracle.reorder_communities(4, [2, 2, 0], [2, 2, 0])  # self-loops only
    assert ident.tolist() == [0, 1, 2, 3] and levels == 0
    # two triangles joined by nothing, ids interleaved: each triangle ends up in one id range
    src = np.array([0, 2, 4, 1, 3, 5])
    dst = np.array([2, 4, 0, 3, 5, 1])
    new_id, _, top = oracle.reorder_communities(6, src, dst)
    assert top == 2
    assert sorted(new_id[[0, 2, 4]].tolist()) in ([0, 1, 2], [3, 4, 5])
    assert sorted(new_id[[1, 3, 5]].tolist()) in ([0, 1, 2], [3, 4, 5])
    # max_levels caps the hierarchy
    rng = np.random.default_rng(1)
    s, d = rng.integers(0, 500, 4000), rng.integers(0, 500, 4000)
    _, levels, _ = oracle.reorder_communities(500, s, d, max_levels=2)
    assert levels == 2


def test_reorder_recovers_planted_communities(oracle):
    rng = np.random.default_rng(2)
    n, community = 1 << 14, 128
    src, dst, _ = planted_graph(rng, n, community, 12, 0.9)
    near_before = (np.abs(src.astype(np.int64) - dst) < 4 * community).mean()
    new_id, levels, top = oracle.reorder_communities(n, src, dst)
    s2, d2 = new_id[src].astype(np.int64), new_id[dst].astype(np.int64)
    near_after = (np.abs(s2 - d2) < 4 * community).mean()
    assert near_before < 0.1 and near_after > 0.6, (near_before, near_after)
    assert np.abs(s2 - d2).mean() < 0.3 * np.abs(src.astype(np.int64) - dst).mean()
    assert levels >= 3 and top <= n // community
