"""lev_matvec_static_scratch, the entry point for callers that cannot
allocate device memory at call time (fixed-budget decode loops, processes
whose allocator owns the whole GPU).  It must give what lev_matvec gives, on
repeated calls, although its work buffers are one shared static array that
keeps the previous call's contents."""
import numpy as np
import pytest
import torch

import leviathan_b200 as lev
from leviathan_b200 import quant as Q
from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,rows,cols,n_cols", [("q4_k", 96, 4096, 1), ("q4_0", 300, 2816, 2), ("q4_k", 35, 768, 4)])
def test_static_scratch_matches_the_allocating_entry_point_twice(name, rows, cols, n_cols):
    t = H.TYPES[name]
    ctx = lev.Context(0)
    w = H.quantized(t, 71, rows, cols)
    wh = ctx.upload(w, t, rows, cols)
    for call in range(2):  # second call meets the first call's leftovers in the array
        x = torch.from_numpy(Q.normal(80 + call, (n_cols, cols), 1.0)).cuda()
        ref = ctx.matvec(wh, x, schedule=lev.SCHEDULE_STREAM).cpu().numpy()
        got = ctx.matvec_static_scratch(wh, x).cpu().numpy()
        for c in range(n_cols):
            assert O.max_rel_err(got[c], ref[c].astype(np.float64)) < H.REPORT_TOL, (name, call, c)
            assert O.max_rel_err(got[c], O.matvec_f64(t, w, rows, cols, x[c].cpu().numpy())) < H.REPORT_TOL
    wh.free()
    ctx.close()


def test_static_scratch_refuses_what_does_not_fit_or_is_not_served():
    ctx = lev.Context(0)
    lib = ctx.lib
    assert lib.lev_static_scratch_bytes() == 4 << 20
    # an odd row offset is not served by the stream schedule
    w6 = H.quantized(Q.GGML_Q6_K, 3, 32, 256)
    h6 = ctx.upload(w6, Q.GGML_Q6_K, 32, 256)
    with pytest.raises(lev.LevError) as e:
        ctx.matvec_static_scratch(h6, torch.zeros(256, device="cuda"), row0=3, rows=16)
    assert e.value.name == "unsupported"
    h6.free()
    # eight columns of a million-wide row need 33 MB of split-activation tables
    cols = 1 << 20
    big = torch.zeros(16 * (cols // 256) * 144, dtype=torch.uint8, device="cuda")
    hb = ctx.upload(big, Q.GGML_Q4_K, 16, cols)
    with pytest.raises(lev.LevError) as e:
        ctx.matvec_static_scratch(hb, torch.zeros((8, cols), device="cuda"))
    assert e.value.name == "exceedsModelWorkload" and "static scratch" in e.value.message
    hb.free()
    ctx.close()
