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


# the first three shapes are served by the one-launch kernel (tables in shared memory, no work
# buffer); five and eight columns, and one tensor whose tables outgrow shared memory, run the
# prepare + stream pair with their tables in the static device array
CASES = [("q4_k", 96, 4096, 1, False), ("q4_0", 300, 2816, 2, False), ("q4_k", 35, 768, 4, False),
         ("q4_k", 96, 4096, 8, True), ("q6_k", 64, 2816 // 256 * 256, 5, True), ("q4_0", 300, 2816, 8, True),
         ("q4_k", 48, 65536, 4, True)]


@pytest.mark.parametrize("name,rows,cols,n_cols,uses_array", CASES)
def test_static_scratch_matches_the_allocating_entry_point_twice(name, rows, cols, n_cols, uses_array):
    t = H.TYPES[name]
    ctx = lev.Context(0)
    w = H.quantized(t, 71, rows, cols)
    wh = ctx.upload(w, t, rows, cols)
    # a second tensor of another shape: its call leaves different tables in the array in between
    rows2, cols2, n2 = 80, 1024, 8 if uses_array else 2
    w2 = H.quantized(t, 72, rows2, cols2)
    wh2 = ctx.upload(w2, t, rows2, cols2)
    for call in range(2):  # the second call meets what the calls before it left in the array
        x = torch.from_numpy(Q.normal(80 + call, (n_cols, cols), 1.0)).cuda()
        ref = ctx.matvec(wh, x, schedule=lev.SCHEDULE_STREAM).cpu().numpy()
        l0 = ctx.launch_count()
        got = ctx.matvec_static_scratch(wh, x).cpu().numpy()
        launches = ctx.launch_count() - l0
        assert launches == (2 if uses_array else 1), (name, launches)  # prepare + stream, or the one-launch kernel
        for c in range(n_cols):
            assert O.max_rel_err(got[c], ref[c].astype(np.float64)) < H.REPORT_TOL, (name, call, c)
            assert O.max_rel_err(got[c], O.matvec_f64(t, w, rows, cols, x[c].cpu().numpy())) < H.REPORT_TOL
        x2 = torch.from_numpy(Q.normal(90 + call, (n2, cols2), 1.0)).cuda()
        got2 = ctx.matvec_static_scratch(wh2, x2).cpu().numpy()
        for c in range(n2):
            assert O.max_rel_err(got2[c], O.matvec_f64(t, w2, rows2, cols2, x2[c].cpu().numpy())) < H.REPORT_TOL
    # a row window of the first tensor
    if rows >= 48:
        x = torch.from_numpy(Q.normal(99, (n_cols, cols), 1.0)).cuda()
        got = ctx.matvec_static_scratch(wh, x, row0=16, rows=32).cpu().numpy()
        full = O.matvec_f64(t, w, rows, cols, x[0].cpu().numpy())
        assert O.max_rel_err(got[0], full[16:48]) < H.REPORT_TOL
    wh.free()
    wh2.free()
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
