"""The oracle's blocked-ELL helpers (format of GenerateUniformBlockedELLIndex, GEMM/include/bm_test_utils.h:48-70). No GPU."""
import numpy as np


def test_bell_indices_are_ascending_unique_and_in_range(oracle):
    vals, ind = oracle.make_bell_uniform(700, 2000, 5, 0, seed=3)
    assert vals.shape == (700, 5 * 128) and ind.shape == (6, 5) and ind.dtype == np.int32
    assert (np.diff(ind, axis=1) > 0).all() and ind.min() >= 0 and ind.max() < 16
    # every block column is drawn sooner or later (uniform subset per block row)
    seen = set()
    for s in range(40):
        seen |= set(oracle.make_bell_uniform(128, 2000, 5, 0, seed=s)[1].ravel().tolist())
    assert seen == set(range(16))


def test_bell_to_dense_places_blocks_and_drops_padding(oracle):
    m, k = 200, 300                                     # ragged block row and a block column cut by K
    vals = oracle.fill_normal(m * 256, 0, 1.0, 8).reshape(m, 256) | 1          # no zero bytes, no NaN
    ind = np.array([[0, 2], [-1, 1]], dtype=np.int32)
    d = oracle.bell_to_dense(vals, ind, k)
    assert d.shape == (m, k)
    assert np.array_equal(d[:128, 0:128], vals[:128, 0:128])
    assert np.array_equal(d[:128, 256:300], vals[:128, 128:128 + 44])       # block column 2 is cut at K
    assert not d[:128, 128:256].any()
    assert not d[128:, 0:128].any() and not d[128:, 256:].any()             # the padding block is dropped
    assert np.array_equal(d[128:, 128:256], vals[128:, 128:256])
    # the dense matrix and the block list give the same product
    x = oracle.fill_normal(k, 0, 1.0, 4).reshape(1, k)
    full, _ = oracle.gemm_f64(d, 0, x, 0)
    dec = oracle.decode(vals, 0).astype(np.float64)
    xs = oracle.decode(x, 0).astype(np.float64)[0]
    want = np.zeros(m)
    for r in range(2):
        for j, c in enumerate(ind[r]):
            if c < 0:
                continue
            w = min(128, k - c * 128)
            rows = slice(r * 128, min(m, (r + 1) * 128))
            want[rows] += dec[rows, j * 128:j * 128 + w] @ xs[c * 128:c * 128 + w]
    assert np.allclose(full[:, 0], want, rtol=1e-12, atol=1e-12)
