"""Host restatement of the device top-k selection loop (k_router_topk in lev_moe.cu) for the case
the GPU tests must not provoke: non-finite router scores.  Every probability is then NaN, no
`v > best` comparison succeeds and the running index keeps its sentinel; the kernel records the
condition and selects the rank itself with weight zero instead of following the sentinel."""
import numpy as np

SENTINEL = 0x7FFFFFFF


def select(scores: np.ndarray, top_k: int):
    experts = scores.size
    with np.errstate(invalid="ignore", over="ignore"):
        m = np.float32(-np.inf)
        for s in scores:
            m = np.fmax(m, s)  # fmaxf ignores NaN like the device intrinsic
        p = np.exp((scores - m).astype(np.float64))
        p = p / p.sum()
    flagged = False
    idx, sel = [], []
    for k in range(top_k):
        best, bi = -1.0, SENTINEL
        for i in range(experts):
            if p[i] > best:
                best, bi = p[i], i
        if bi >= experts:
            flagged = True
            bi = k if k < experts else 0
            best = 0.0
        idx.append(bi)
        sel.append(best)
        p[bi] = -1.0
    total = sum(sel)
    w = [np.float32(v / total) if total > 0.0 else np.float32(0.0) for v in sel]
    return idx, w, flagged


def test_finite_scores_select_the_largest_first_lowest_index_on_ties():
    s = np.array([0.5, 2.0, 2.0, -1.0, 0.25], np.float32)
    idx, w, flagged = select(s, 3)
    assert idx == [1, 2, 0] and not flagged
    assert abs(sum(w) - 1.0) < 1e-6


def test_nan_scores_never_leave_the_expert_range():
    for bad in (np.nan, np.inf, -np.inf):
        s = np.full(16, 0.1, np.float32)
        s[5] = bad
        idx, w, flagged = select(s, 8)
        assert all(0 <= i < 16 for i in idx)
        if bad is np.nan or bad == np.inf:
            # inf - inf and NaN poison every probability
            assert flagged and all(v == 0.0 for v in w)
