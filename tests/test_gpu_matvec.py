"""Parity of the CUDA decode path with the oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import leviathan_b200 as lev
from leviathan_b200 import quant as Q
from oracle import oracle as O
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = lev.Context(0)
    yield c
    c.close()


SHAPES = {
    "q4_0": [(35, 33 * 32), (128, 256), (64, 4096), (512, 704), (300, 2816)],
    "q4_k": [(35, 3 * 256), (16, 1024), (96, 4096), (17, 256)],
    "q6_k": [(35, 3 * 256), (64, 512), (48, 12288 // 4), (9, 256)],
}


@pytest.mark.parametrize("name", ["q4_0", "q4_k", "q6_k"])
@pytest.mark.parametrize("source", ["encoded", "random_bytes"])
def test_dequantize_is_bit_exact(ctx, name, source):
    t = H.TYPES[name]
    for i, (rows, cols) in enumerate(SHAPES[name]):
        w = H.quantized(t, 100 + i, rows, cols) if source == "encoded" else H.random_blocks(t, 200 + i, rows, cols)
        wh = ctx.upload(w, t, rows, cols)
        got = ctx.dequantize(wh)
        ref = O.dequantize_rows(t, w, rows, cols)
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), (name, rows, cols)
        # a row window addresses a sub-tensor of the resident buffer
        if rows > 4:
            part = ctx.dequantize(wh, row0=3, rows=rows - 4)
            assert np.array_equal(part.view(np.uint32), ref[3:rows - 1].view(np.uint32))
        wh.free()


def _schedules(ctx, wh, x):
    out = [lev.SCHEDULE_PLAIN]
    try:
        ctx.matvec(wh, x, schedule=lev.SCHEDULE_STREAM)
        out.append(lev.SCHEDULE_STREAM)
    except lev.LevError as e:
        assert e.name == "unsupported"
    return out


@pytest.mark.parametrize("name", ["q4_0", "q4_k", "q6_k"])
@pytest.mark.parametrize("n_cols", [1, 2, 3, 4, 8])
def test_matvec_matches_f64_oracle(ctx, name, n_cols):
    t = H.TYPES[name]
    for i, (rows, cols) in enumerate(SHAPES[name]):
        for source in ("encoded", "random_bytes"):
            w = H.quantized(t, 300 + i, rows, cols) if source == "encoded" else H.random_blocks(t, 400 + i, rows, cols)
            x = Q.normal(500 + i, (n_cols, cols), 1.0)
            wh = ctx.upload(w, t, rows, cols)
            xd = torch.from_numpy(x).cuda()
            for sched in _schedules(ctx, wh, xd):
                buf, view = H.guarded(n_cols * rows)
                y = ctx.matvec(wh, xd, out=view.view(n_cols, rows), schedule=sched, check_finite=True)
                torch.cuda.synchronize()
                assert H.guards_intact(buf, n_cols * rows)
                y = y.cpu().numpy()
                for c in range(n_cols):
                    ref = O.matvec_f64(t, w, rows, cols, x[c])
                    err = O.max_rel_err(y[c], ref)
                    # random block bytes give rows whose terms are ~1e2 and
                    # cancel: f32 accumulation noise alone (the CPU f32 form
                    # shows it too) sits near 1e-4 there, so those rows are
                    # held to the pass bar and the encoded ones to the
                    # reference's own 1e-4 gate
                    tol = H.REPORT_TOL if source == "encoded" else H.PASS_TOL
                    assert err < tol, (name, rows, cols, source, sched, c, err)
                # the same call twice gives the same bits
                y2 = ctx.matvec(wh, xd, schedule=sched).cpu().numpy()
                assert np.array_equal(y.view(np.uint32), y2.view(np.uint32))
            wh.free()


@pytest.mark.parametrize("name", ["q4_0", "q4_k", "q6_k"])
def test_columns_are_independent_of_batching(ctx, name):
    """Column c of an n-column call equals the 1-column call on x[c]."""
    t = H.TYPES[name]
    rows, cols = SHAPES[name][0]
    w = H.quantized(t, 31, rows, cols)
    x = torch.from_numpy(Q.normal(32, (8, cols), 1.0)).cuda()
    wh = ctx.upload(w, t, rows, cols)
    for sched in _schedules(ctx, wh, x):
        y8 = ctx.matvec(wh, x, schedule=sched).cpu().numpy()
        for c in (0, 5, 7):
            y1 = ctx.matvec(wh, x[c], schedule=sched).cpu().numpy()
            assert O.max_rel_err(y1, y8[c].astype(np.float64)) < 1e-6
    wh.free()


@pytest.mark.parametrize("name", ["q4_0", "q4_k", "q6_k"])
def test_adversarial_activations(ctx, name):
    t = H.TYPES[name]
    rows, cols = SHAPES[name][2]
    w = H.random_blocks(t, 77, rows, cols)
    wh = ctx.upload(w, t, rows, cols)
    for kind in ("sinusoid", "alternating", "onehot"):
        x = Q.adversarial_activations(kind, cols)
        ref = O.matvec_f64(t, w, rows, cols, x)
        for sched in _schedules(ctx, wh, torch.from_numpy(x).cuda()):
            y = ctx.matvec(wh, torch.from_numpy(x).cuda(), schedule=sched).cpu().numpy()
            assert O.max_rel_err(y, ref) < H.PASS_TOL, (name, kind, sched)
    wh.free()


def test_row_window_addresses_a_sub_tensor(ctx):
    t = Q.GGML_Q4_0
    rows, cols = 8 * 48, 704  # 8 stacked expert slices of 48 rows
    w = H.quantized(t, 9, rows, cols)
    x = Q.normal(10, (cols,), 1.0)
    wh = ctx.upload(w, t, rows, cols)
    xd = torch.from_numpy(x).cuda()
    full = O.matvec_f64(t, w, rows, cols, x)
    for e in (0, 3, 7):
        for sched in _schedules(ctx, wh, xd):
            y = ctx.matvec(wh, xd, row0=e * 48, rows=48, schedule=sched).cpu().numpy()
            assert O.max_rel_err(y, full[e * 48:(e + 1) * 48]) < H.REPORT_TOL
    wh.free()


def test_known_answer_blocks_on_the_gpu(ctx):
    # Q6_K exact -315 (Sources/leviathan-tests/main.swift:1087-1123)
    block = np.zeros(210, np.uint8)
    block[208], block[209] = 0x00, 0x3C
    block[192], block[193], block[196], block[200], block[204] = 3, 0xFD, 2, 3, 2
    block[0], block[128], block[64], block[160] = 0x21, 0x03, 0x21, 0x01
    x = np.zeros(256, np.float32)
    x[0], x[16], x[64], x[128], x[192] = 1, -1, 2, -2, 4
    y, ev = ctx.q6_k_matvec_reporting(block, 1, 256, x)
    assert y[0] == -315.0 and ev["command_status"] == "completed" and ev["device_name"]
    # Q4_0 two rows (main.swift:728-738)
    w = np.array([0x00, 0x3C] + [0] * 16 + [0x00, 0xBC] + [0] * 16, np.uint8)
    xs = O.seeded_input_swift(32, 7)
    y, _ = ctx.q4_0_matvec_reporting(w, 2, 32, xs)
    s = float(xs.astype(np.float64).sum())
    assert abs(y[0] + 8 * s) < 1e-3 and abs(y[1] - 8 * s) < 1e-3
    # Q4_K hand block (rust/crates/lev-cpu/src/lib.rs:437-464): rows of 0 / 1
    blk = np.zeros(144, np.uint8)
    blk[0:2], blk[2:4] = [0x00, 0x3C], [0x00, 0x38]
    blk[4:16] = O.q4_k_pack_scale_min([1] * 8, [2] * 8)
    blk[16:] = 0x21
    y, _ = ctx.q4_k_matvec_reporting(blk, 1, 256, np.ones(256, np.float32))
    assert y[0] == 128.0


def test_reference_generator_gate_on_the_gpu(ctx):
    """Sources/leviathan-tests/main.swift:748-773 (Q4_0 128x256 seeds 99/101)."""
    r = O.SplitMix64(99)
    out = bytearray()
    for _ in range(128 * 8):
        scale = np.float16(np.float32(r.uniform_swift()) * np.float32(2) - np.float32(1))
        bits = int(scale.view(np.uint16))
        out += bytes([bits & 0xFF, bits >> 8])
        for _ in range(16):
            out.append(r.next() & 0xFF)
    w = np.frombuffer(bytes(out), np.uint8)
    x = O.seeded_input_swift(256, 101)
    y, ev = ctx.q4_0_matvec_reporting(w, 128, 256, x)
    oracle = O.q4_0_matvec_f32(w, 128, 256, x)
    assert np.max(np.abs(y - oracle) / np.maximum(1, np.abs(oracle))) < 1e-4
    assert ev["out_dim"] == 128 and ev["in_dim"] == 256 and ev["gpu_us"] > 0


def test_host_side_rejections(ctx):
    """One negative per status, before any device work
    (Sources/leviathan-tests/main.swift:778-796)."""
    z = np.zeros(8 * 18, np.uint8)
    with pytest.raises(lev.LevError) as e:
        ctx.q4_0_matvec_reporting(np.zeros(0, np.uint8), 8, 33, np.zeros(0, np.float32))
    assert e.value.name == "badDimensions" and "inDim 33, outDim 8" in e.value.message
    with pytest.raises(lev.LevError) as e:
        ctx.q4_0_matvec_reporting(np.zeros(0, np.uint8), 8, 32, np.zeros(0, np.float32))
    assert e.value.name == "badDimensions" and "weights are 0 bytes, geometry needs 144" in e.value.message
    with pytest.raises(lev.LevError) as e:
        ctx.q4_0_matvec_reporting(z, 8, 32, np.zeros(3, np.float32))
    assert e.value.name == "wrongInputCount"
    bad = np.zeros(32, np.float32)
    bad[1] = np.inf
    with pytest.raises(lev.LevError) as e:
        ctx.q4_0_matvec_reporting(z, 8, 32, bad)
    assert e.value.name == "nonFiniteInput"
    inf_scale = z.copy()
    inf_scale[1] = 0x7C
    with pytest.raises(lev.LevError) as e:
        ctx.q4_0_matvec_reporting(inf_scale, 8, 32, np.zeros(32, np.float32))
    assert e.value.name == "nonFiniteScale"
    with pytest.raises(lev.LevError) as e:
        ctx.upload(z, 99, 8, 32)
    assert e.value.name == "badArgument"
    with pytest.raises(lev.LevError) as e:
        ctx.upload(z, Q.GGML_Q4_0, 8, (1 << 22) + 32)
    assert e.value.name == "badDimensions"
    wh = ctx.upload(z, Q.GGML_Q4_0, 8, 32)
    x = torch.zeros(32, device="cuda")
    with pytest.raises(lev.LevError) as e:
        ctx.matvec(wh, x, row0=4, rows=8)
    assert e.value.name == "badDimensions"
    with pytest.raises(lev.LevError) as e:
        ctx.matvec(wh, x, out=torch.zeros(1, 4, device="cuda"))
    assert e.value.name == "badDimensions"
    with pytest.raises(lev.LevError) as e:
        ctx.matvec(wh, torch.zeros(9, 32, device="cuda"))
    assert e.value.name == "badDimensions"
    both = torch.zeros(64, device="cuda")
    with pytest.raises(lev.LevError) as e:
        ctx.matvec(wh, both[:32], out=both[24:32].view(1, 8))
    assert e.value.name == "badArgument"
    nanx = torch.zeros(32, device="cuda")
    nanx[5] = float("nan")
    with pytest.raises(lev.LevError) as e:
        ctx.matvec(wh, nanx, check_finite=True)
    assert e.value.name == "nonFiniteInput"
    # the context stays usable after every rejection
    assert ctx.matvec(wh, x).shape == (8,)
    wh.free()


def test_hardware_profile(ctx):
    p = ctx.hardware_profile()
    assert p["cc_major"] == 10 and p["sm_count"] > 100 and p["warp_width"] == 32
    assert p["free_memory"] > 0 and "B200" in p["device_name"]


@pytest.mark.parametrize("name,rows,cols", [("q4_k", 2400, 4096), ("q6_k", 1040, 12288), ("q4_0", 4096, 4096)])
def test_bench_sized_rows_and_row_windows(ctx, name, rows, cols):
    """Shapes with the bench's K (every SM gets tiles, warps share tiles, the ring refills),
    a row count that is not a multiple of the tile height, and a 16-aligned row window."""
    t = H.TYPES[name]
    w = H.quantized(t, 900, rows, cols)
    x = Q.normal(901, (1, cols), 1.0)
    wh = ctx.upload(w, t, rows, cols)
    xd = torch.from_numpy(x).cuda()
    ref = O.matvec_f64(t, w, rows, cols, x[0])
    y = ctx.matvec(wh, xd, schedule=lev.SCHEDULE_STREAM).cpu().numpy()
    assert O.max_rel_err(y[0], ref) < H.REPORT_TOL
    # the same call again gives the same bits (fixed summation order)
    y2 = ctx.matvec(wh, xd, schedule=lev.SCHEDULE_STREAM).cpu().numpy()
    assert np.array_equal(y.view(np.uint32), y2.view(np.uint32))
    n_win = min(1000, rows - 160 - 7)
    win = ctx.matvec(wh, xd, row0=160, rows=n_win, schedule=lev.SCHEDULE_STREAM).cpu().numpy()
    assert O.max_rel_err(win[0], ref[160:160 + n_win]) < H.REPORT_TOL
    wh.free()


def test_host_call_writes_page_locked_outputs_directly(ctx):
    """LEV_FLAG_HOST_IO with a pinned (device-mapped) output buffer skips the device->host copy;
    pageable buffers take the staged path.  Both give the same bits."""
    t = H.TYPES["q4_k"]
    rows, cols = 512, 1024
    w = H.quantized(t, 910, rows, cols)
    x = Q.normal(911, (1, cols), 1.0)
    wh = ctx.upload(w, t, rows, cols)
    pinned = torch.empty((1, rows), dtype=torch.float32).pin_memory()
    ctx.matvec(wh, x, out=pinned.numpy())
    pageable = np.empty((1, rows), np.float32)
    ctx.matvec(wh, x, out=pageable)
    assert np.array_equal(pinned.numpy().view(np.uint32), pageable.view(np.uint32))
    assert O.max_rel_err(pageable[0], O.matvec_f64(t, w, rows, cols, x[0])) < H.REPORT_TOL
    wh.free()


def test_installed_op_serves_matching_tensors(ctx):
    """lev_op_serves is the analogue of q4GeneratedServesTensor
    (Sources/LeviathanCore/Gemma4.swift:989-1012): an installed op spec serves a resident
    tensor whose quant, inDim and row count match."""
    import json

    doc = {"schema": 1, "op": "q4_k.matvec", "semantics": "dot(W_row, x)", "inDim": 1024, "outDim": 512,
           "layout": "row-major-q4_k-blocks", "quant": "q4_k", "accumulate": "f32", "inputPrecision": "f32"}
    op = ctx.op_install(json.dumps(doc))
    w = H.quantized(H.TYPES["q4_k"], 920, 512, 1024)
    good = ctx.upload(w, H.TYPES["q4_k"], 512, 1024)
    other = ctx.upload(H.quantized(H.TYPES["q4_0"], 921, 512, 1024), H.TYPES["q4_0"], 512, 1024)
    assert ctx.op_serves(op, good, 512)
    assert not ctx.op_serves(op, good, 256)
    assert not ctx.op_serves(op, other, 512)
    ctx.op_uninstall(op)
    good.free()
    other.free()


@pytest.mark.parametrize("name,rows_list,cols", [("q4_k", (1040, 512, 96), 1024), ("q6_k", (64, 80), 768),
                                                 ("q4_0", (300, 300), 2816)])
@pytest.mark.parametrize("n_cols", [1, 3])
def test_matvec_multi_matches_single_calls(ctx, name, rows_list, cols, n_cols):
    """lev_matvec_multi: several tensors against the same activations in one launch give each
    tensor's own result (vs the f64 oracle, and close to the single-tensor call)."""
    t = H.TYPES[name]
    ws = [H.quantized(t, 700 + i, r, cols) for i, r in enumerate(rows_list)]
    hs = [ctx.upload(w, t, r, cols) for w, r in zip(ws, rows_list)]
    x = Q.normal(710, (n_cols, cols), 1.0)
    xd = torch.from_numpy(x).cuda()
    outs = ctx.matvec_multi(hs, xd, check_finite=True)
    torch.cuda.synchronize()
    for w, r, h, o in zip(ws, rows_list, hs, outs):
        o = o.cpu().numpy()
        single = ctx.matvec(h, xd, schedule=lev.SCHEDULE_STREAM).cpu().numpy()
        for c in range(n_cols):
            assert O.max_rel_err(o[c], O.matvec_f64(t, w, r, cols, x[c])) < H.REPORT_TOL
            assert O.max_rel_err(o[c], single[c].astype(np.float64)) < 1e-5
    # host buffers
    houts = ctx.matvec_multi(hs, x)
    for o, ho in zip(outs, houts):
        assert np.array_equal(o.cpu().numpy().view(np.uint32), ho.view(np.uint32))
    # tensors that do not share a format fall back to one launch per tensor
    if name == "q4_k":
        other = ctx.upload(H.quantized(H.TYPES["q4_0"], 720, 64, cols), H.TYPES["q4_0"], 64, cols)
        mixed = ctx.matvec_multi([hs[0], other], xd)
        assert np.array_equal(mixed[0].cpu().numpy().view(np.uint32), outs[0].cpu().numpy().view(np.uint32)) or \
            O.max_rel_err(mixed[0].cpu().numpy()[0], outs[0].cpu().numpy()[0].astype(np.float64)) < 1e-5
        other.free()
    with pytest.raises(lev.LevError) as e:
        ctx.matvec_multi(hs, xd[:, :-32].contiguous())
    assert e.value.name == "wrongInputCount"
    for h in hs:
        h.free()


def test_release_of_the_gguf_order_copy(ctx):
    """A decode-only host keeps a tensor once: after lev_weights_release_gguf the stream schedule gives
    the same bits as before, and the entry points that read GGUF-order bytes refuse the tensor."""
    t = H.TYPES["q4_k"]
    rows, cols = 96, 1024
    w = H.quantized(t, 77, rows, cols)
    wh = ctx.upload(w, t, rows, cols)
    x = torch.from_numpy(Q.normal(78, (2, cols), 1.0)).cuda()
    before1 = ctx.matvec(wh, x[0], schedule=lev.SCHEDULE_STREAM).clone()
    before2 = ctx.matvec(wh, x, schedule=lev.SCHEDULE_STREAM).clone()
    wh.release_gguf()
    wh.release_gguf()  # idempotent
    assert torch.equal(ctx.matvec(wh, x[0], schedule=lev.SCHEDULE_STREAM).view(torch.int32), before1.view(torch.int32))
    assert torch.equal(ctx.matvec(wh, x, schedule=lev.SCHEDULE_STREAM).view(torch.int32), before2.view(torch.int32))
    with pytest.raises(lev.LevError) as e:
        ctx.matvec(wh, x[0], schedule=lev.SCHEDULE_PLAIN)
    assert e.value.name == "unsupported"
    with pytest.raises(lev.LevError) as e:
        ctx.dequantize(wh)
    assert e.value.name == "unsupported"
    wh.free()
