"""Python host layer over the C ABI: contexts, resident weights and the
operators of the quantized-weight hot path.

numpy arrays are host buffers (the call copies in and out and synchronizes,
LEV_FLAG_HOST_IO); torch CUDA tensors are device buffers (the call is
asynchronous on the context's stream).  torch is used for device memory and
streams only; every operation runs in libleviathan_cuda.so.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L


class LevError(RuntimeError):
    """A non-zero lev_status; `.name` is the reference's error-case name."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{L.STATUS.get(status, status)}: {message}")
        self.status = status
        self.name = L.STATUS.get(status, str(status))
        self.message = message


def _is_torch(a) -> bool:
    return type(a).__module__.startswith("torch")


def _ptr(a):
    if a is None:
        return None
    if _is_torch(a):
        return a.data_ptr()
    return a.ctypes.data


class Weights:
    def __init__(self, ctx: "Context", handle, ggml_type: int, rows: int, cols: int, gguf_bytes: int):
        self.ctx, self.handle = ctx, handle
        self.ggml_type, self.rows, self.cols, self.gguf_bytes = ggml_type, rows, cols, gguf_bytes

    def release_gguf(self):
        """lev_weights_release_gguf: drop the GGUF-order copy (decode-only use: the stream schedule keeps
        the repacked bytes); dequantize, the plain schedule and prefill then refuse this tensor."""
        self.ctx._check(self.ctx.lib.lev_weights_release_gguf(self.ctx.handle, self.handle))

    def free(self):
        if self.handle:
            self.ctx.lib.lev_weights_free(self.ctx.handle, self.handle)
            self.handle = None


class MoEWeights:
    def __init__(self, ctx: "Context", handle, experts, hidden, inter, local_first, local_count):
        self.ctx, self.handle = ctx, handle
        self.experts, self.hidden, self.inter = experts, hidden, inter
        self.local_first, self.local_count = local_first, local_count

    def release_gguf(self):
        """lev_moe_weights_release_gguf: keep only the repacked copy of the experts (decode-sized calls)."""
        self.ctx._check(self.ctx.lib.lev_moe_weights_release_gguf(self.ctx.handle, self.handle))

    def free(self):
        if self.handle:
            self.ctx.lib.lev_moe_weights_free(self.ctx.handle, self.handle)
            self.handle = None


class Context:
    """One device, one stream (lev_ctx).  Not thread-safe."""

    def __init__(self, device: int = 0, follow_torch_stream: bool = True):
        """follow_torch_stream: before every call that is given torch tensors,
        issue on torch's current stream for this device, so the usual torch
        ordering rules hold between this library's kernels and torch's."""
        self.follow_torch_stream = follow_torch_stream
        self._stream_seen = None
        self.lib = L.load()
        h = C.c_void_p()
        st = self.lib.lev_cuda_init(device, C.byref(h))
        if st != L.OK:
            raise LevError(st, f"lev_cuda_init(device={device})")
        self.handle = h
        self.device = device

    # -- plumbing --
    def _check(self, st: int):
        if st != L.OK:
            raise LevError(st, self.lib.lev_last_error(self.handle).decode(errors="replace"))

    def close(self):
        if self.handle:
            self.lib.lev_cuda_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def hardware_profile(self) -> dict:
        p = L.HwProfile()
        self._check(self.lib.lev_cuda_hardware_profile(self.handle, C.byref(p)))
        return {k: (getattr(p, k).decode() if k == "device_name" else getattr(p, k)) for k, _ in p._fields_}

    def set_stream(self, cuda_stream: int | None):
        """cuda_stream: a cudaStream_t value; 0 means the legacy default
        stream (passed as cudaStreamLegacy), None the context's own stream."""
        if cuda_stream == 0:
            cuda_stream = 1  # cudaStreamLegacy
        self._check(self.lib.lev_cuda_set_stream(self.handle, cuda_stream))

    def use_torch_stream(self):
        import torch

        self.set_stream(torch.cuda.current_stream(self.device).cuda_stream)

    def synchronize(self):
        self._check(self.lib.lev_cuda_synchronize(self.handle))

    def launch_count(self) -> int:
        return self.lib.lev_cuda_launch_count(self.handle)

    def last_evidence(self) -> dict:
        e = L.Evidence()
        self._check(self.lib.lev_cuda_last_evidence(self.handle, C.byref(e)))
        return {k: (getattr(e, k).decode() if k.endswith("_name") else getattr(e, k)) for k, _ in e._fields_}

    def _flags(self, host: bool, check_finite: bool) -> int:
        if not host and self.follow_torch_stream:
            import torch

            s = torch.cuda.current_stream(self.device).cuda_stream
            if s != self._stream_seen:
                self.set_stream(s)
                self._stream_seen = s
        return (L.FLAG_HOST_IO if host else 0) | (L.FLAG_CHECK_FINITE if check_finite else 0)

    def _empty_like_io(self, like, shape, dtype_np, dtype_torch_name):
        if _is_torch(like):
            import torch

            return torch.empty(shape, dtype=getattr(torch, dtype_torch_name), device=like.device)
        return np.empty(shape, dtype_np)

    # -- weights --
    def upload(self, blocks, ggml_type: int, rows: int, cols: int) -> Weights:
        """lev_weights_upload: raw GGUF block bytes (numpy uint8 or torch uint8 CUDA)."""
        on_dev = _is_torch(blocks) and blocks.is_cuda
        if not _is_torch(blocks):
            blocks = np.ascontiguousarray(blocks, np.uint8)
            n = blocks.size
        else:
            blocks = blocks.contiguous()
            n = blocks.numel()
        if on_dev:
            self._flags(False, False)
        h = C.c_void_p()
        self._check(self.lib.lev_weights_upload(self.handle, _ptr(blocks), n, ggml_type, rows, cols,
                                                1 if on_dev else 0, C.byref(h)))
        return Weights(self, h, ggml_type, rows, cols, n)

    def dequantize(self, w: Weights, row0: int = 0, rows: int | None = None, device_out=None):
        rows = w.rows - row0 if rows is None else rows
        if device_out is not None:
            self._flags(False, False)
            self._check(self.lib.lev_dequantize(self.handle, w.handle, row0, rows, _ptr(device_out), 0))
            return device_out
        out = np.empty((max(rows, 0), w.cols), np.float32)
        self._check(self.lib.lev_dequantize(self.handle, w.handle, row0, rows, _ptr(out), L.FLAG_HOST_IO))
        return out

    # -- decode matvec --
    def matvec(self, w: Weights, x, row0: int = 0, rows: int | None = None, out=None,
               schedule: int = L.SCHEDULE_AUTO, check_finite: bool = False):
        """y[c][r] = W[row0+r] . x[c]; x is [cols] or [n_cols][cols]."""
        rows = w.rows - row0 if rows is None else rows
        host = not _is_torch(x)
        if host:
            x = np.ascontiguousarray(x, np.float32)
            x_count = x.size
        else:
            x = x.contiguous()
            x_count = x.numel()
        one_d = x.ndim == 1
        n_cols = 1 if one_d else x.shape[0]
        if out is None:
            out = self._empty_like_io(x, (n_cols, max(rows, 0)), np.float32, "float32")
        cap = out.size if host else out.numel()
        self._check(self.lib.lev_matvec(self.handle, w.handle, row0, rows, _ptr(x), x_count, n_cols, _ptr(out), cap,
                                        schedule, self._flags(host, check_finite)))
        return out[0] if one_d else out

    def matvec_multi(self, ws, x, outs=None, check_finite: bool = False):
        """Several resident tensors against the same activations (one launch when they share
        format and inDim).  Returns one [n_cols][rows_i] array per tensor."""
        host = not _is_torch(x)
        x = np.ascontiguousarray(x, np.float32) if host else x.contiguous()
        one_d = x.ndim == 1
        n_cols = 1 if one_d else x.shape[0]
        n = len(ws)
        if outs is None:
            outs = [self._empty_like_io(x, (n_cols, w.rows), np.float32, "float32") for w in ws]
        wp = (C.c_void_p * n)(*[w.handle for w in ws])
        yp = (C.c_void_p * n)(*[_ptr(o) for o in outs])
        cap = (C.c_int64 * n)(*[int(o.size if host else o.numel()) for o in outs])
        count = int(x.size if host else x.numel())
        self._check(self.lib.lev_matvec_multi(self.handle, n, wp, _ptr(x), count, n_cols, yp, cap, self._flags(host, check_finite)))
        return outs

    def matvec_static_scratch(self, w: Weights, x, row0: int = 0, rows: int | None = None, out=None):
        """lev_matvec_static_scratch: the stream-schedule matvec that allocates
        nothing (torch CUDA tensors only); see include/leviathan_cuda.h."""
        import torch

        rows = w.rows - row0 if rows is None else rows
        x = x.contiguous()
        one_d = x.ndim == 1
        n_cols = 1 if one_d else x.shape[0]
        if out is None:
            out = torch.empty((n_cols, max(rows, 0)), dtype=torch.float32, device=x.device)
        self._flags(False, False)
        self._check(self.lib.lev_matvec_static_scratch(self.handle, w.handle, row0, rows, _ptr(x), x.numel(), n_cols,
                                                       _ptr(out), out.numel()))
        return out[0] if one_d else out

    # -- the steps either side of a matvec (torch CUDA tensors only) --
    def rmsnorm(self, x, weight=None, eps: float = 1e-6, out=None, want_inverse: bool = False):
        """lev_rmsnorm over the rows of x [vectors][n]; out may be x."""
        import torch

        x2 = x.reshape(1, -1) if x.ndim == 1 else x
        out = torch.empty_like(x2) if out is None else out
        inv = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device) if want_inverse else None
        self._flags(False, False)
        self._check(self.lib.lev_rmsnorm(self.handle, _ptr(x2), x2.shape[0], x2.shape[1], _ptr(weight), eps, _ptr(out), _ptr(inv)))
        out = out.reshape(x.shape)
        return (out, inv) if want_inverse else out

    def rmsnorm_cached(self, x, inverse, weight=None, out=None):
        import torch

        x2 = x.reshape(1, -1) if x.ndim == 1 else x
        out = torch.empty_like(x2) if out is None else out
        self._flags(False, False)
        self._check(self.lib.lev_rmsnorm_cached(self.handle, _ptr(x2), x2.shape[0], x2.shape[1], _ptr(weight), _ptr(inverse), _ptr(out)))
        return out.reshape(x.shape)

    def gelu_up(self, gate_up, out=None):
        """lev_gelu_up: rows are [gate | up]; returns [vectors][inter]."""
        import torch

        gu = gate_up.reshape(1, -1) if gate_up.ndim == 1 else gate_up
        inter = gu.shape[1] // 2
        out = torch.empty((gu.shape[0], inter), dtype=torch.float32, device=gu.device) if out is None else out
        self._flags(False, False)
        self._check(self.lib.lev_gelu_up(self.handle, _ptr(gu), gu.shape[0], inter, _ptr(out)))
        return out[0] if gate_up.ndim == 1 else out

    def axpy(self, alpha: float, x, r, out=None):
        """lev_axpy: out = r + alpha * x (out may be r)."""
        import torch

        out = torch.empty_like(r) if out is None else out
        self._flags(False, False)
        self._check(self.lib.lev_axpy(self.handle, alpha, _ptr(x), _ptr(r), x.numel(), _ptr(out)))
        return out

    def qkv_norm_rope(self, qkv, q_heads: int, kv_heads: int, head_dim: int, q_weight=None, k_weight=None, eps: float = 1e-6,
                      inv_freq=None, pos=None):
        """lev_qkv_norm_rope, in place on qkv [n_cols][(q_heads + 2 * kv_heads) * head_dim]."""
        self._flags(False, False)
        self._check(self.lib.lev_qkv_norm_rope(self.handle, _ptr(qkv), qkv.shape[0], q_heads, kv_heads, head_dim, _ptr(q_weight),
                                               _ptr(k_weight), eps, _ptr(inv_freq), _ptr(pos)))
        return qkv

    def qkv_norm_rope_append(self, qkv, q_heads: int, cache: "PagedKV", slot, pos, q_weight=None, k_weight=None,
                             eps: float = 1e-6, inv_freq=None):
        """lev_qkv_norm_rope_append: as qkv_norm_rope, and k / v also go to the cache at (slot, pos)."""
        self._flags(False, False)
        self._check(self.lib.lev_qkv_norm_rope_append(self.handle, _ptr(qkv), qkv.shape[0], q_heads, cache.layout.head_dim, _ptr(q_weight),
                                                      _ptr(k_weight), eps, _ptr(inv_freq), _ptr(pos), C.byref(cache.layout),
                                                      _ptr(cache.k), _ptr(cache.v), _ptr(cache.table), _ptr(slot)))
        return qkv

    def qkv_norm_rope_append_split(self, q, k, v, q_heads: int, cache: "PagedKV", slot, pos, q_weight=None, k_weight=None,
                                   eps: float = 1e-6, inv_freq=None):
        """lev_qkv_norm_rope_append_split: q [n][q_heads * head_dim], k, v [n][kv_heads * head_dim] as three matrices."""
        self._flags(False, False)
        self._check(self.lib.lev_qkv_norm_rope_append_split(self.handle, _ptr(q), _ptr(k), _ptr(v), q.shape[0], q_heads, cache.layout.head_dim,
                                                            _ptr(q_weight), _ptr(k_weight), eps, _ptr(inv_freq), _ptr(pos),
                                                            C.byref(cache.layout), _ptr(cache.k), _ptr(cache.v), _ptr(cache.table), _ptr(slot)))
        return q, k, v

    def argmax(self, x, want_margin: bool = False):
        """lev_argmax over the rows of x [vectors][n]: int32 indices (and best - second best)."""
        import torch

        x2 = (x.reshape(1, -1) if x.ndim == 1 else x).contiguous()
        idx = torch.empty(x2.shape[0], dtype=torch.int32, device=x.device)
        mar = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device) if want_margin else None
        self._flags(False, False)
        self._check(self.lib.lev_argmax(self.handle, _ptr(x2), x2.shape[0], x2.shape[1], _ptr(idx), _ptr(mar)))
        return (idx, mar) if want_margin else idx

    def argmax_into(self, x, out_index):
        """lev_argmax writing into an existing int32 tensor (the token ids of the next step)."""
        self._flags(False, False)
        self._check(self.lib.lev_argmax(self.handle, _ptr(x), x.shape[0], x.shape[1], _ptr(out_index), None))
        return out_index

    def embed_rows(self, w: Weights, tokens, scale: float = 1.0, out=None):
        """lev_embed_rows: out[t] = row tokens[t] of w, decoded, times scale; tokens is an int32 device tensor."""
        import torch

        n = tokens.numel()
        out = torch.empty((n, w.cols), dtype=torch.float32, device=tokens.device) if out is None else out
        self._flags(False, False)
        self._check(self.lib.lev_embed_rows(self.handle, w.handle, _ptr(tokens), n, scale, _ptr(out)))
        return out

    def softcap(self, x, cap: float):
        """lev_softcap: x = cap * tanh(x / cap), in place."""
        self._flags(False, False)
        self._check(self.lib.lev_softcap(self.handle, _ptr(x), x.numel(), cap))
        return x

    @staticmethod
    def _fusion(prologue, norm_weight, eps, residual, alpha):
        code = {None: L.PROLOGUE_NONE, "rmsnorm": L.PROLOGUE_RMSNORM, "gelu_up": L.PROLOGUE_GELU_UP}[prologue]
        return L.Fusion(code, _ptr(norm_weight), eps, _ptr(residual), alpha)

    def matvec_fused(self, w: Weights, x, prologue=None, norm_weight=None, eps: float = 1e-6, residual=None,
                     alpha: float = 1.0, row0: int = 0, rows: int | None = None, out=None):
        """lev_matvec_fused: out = residual + alpha * W prologue(x); prologue None, "rmsnorm" or
        "gelu_up" (x rows are then [gate | up]).  out may be residual."""
        import torch

        rows = w.rows - row0 if rows is None else rows
        x = x.contiguous()
        one_d = x.ndim == 1
        n_cols = 1 if one_d else x.shape[0]
        if out is None:
            out = torch.empty((n_cols, max(rows, 0)), dtype=torch.float32, device=x.device)
        f = self._fusion(prologue, norm_weight, eps, residual, alpha)
        self._flags(False, False)
        self._check(self.lib.lev_matvec_fused(self.handle, w.handle, row0, rows, _ptr(x), x.numel(), n_cols, C.byref(f),
                                              _ptr(out), out.numel()))
        return out[0] if one_d and out.ndim == 2 else out

    def matvec_multi_fused(self, ws, x, prologue=None, norm_weight=None, eps: float = 1e-6, outs=None):
        """lev_matvec_multi_fused: several tensors behind one prologue."""
        import torch

        x = x.contiguous()
        n_cols = 1 if x.ndim == 1 else x.shape[0]
        n = len(ws)
        if outs is None:
            outs = [torch.empty((n_cols, w.rows), dtype=torch.float32, device=x.device) for w in ws]
        wp = (C.c_void_p * n)(*[w.handle for w in ws])
        yp = (C.c_void_p * n)(*[_ptr(o) for o in outs])
        cap = (C.c_int64 * n)(*[int(o.numel()) for o in outs])
        f = self._fusion(prologue, norm_weight, eps, None, 1.0)
        self._flags(False, False)
        self._check(self.lib.lev_matvec_multi_fused(self.handle, n, wp, _ptr(x), x.numel(), n_cols, C.byref(f), yp, cap))
        return outs

    def matvec_chain(self, ops, check_finite: bool = False):
        """lev_matvec_chain: a list of one-column products in one submission.  Each op is a dict with
        keys w (Weights), x, out (all torch CUDA tensors, or all numpy arrays for the host-buffer form),
        and optionally row0, rows, prologue, norm_weight, eps, residual, alpha, depends.  Returns the
        list of outputs."""
        self.chain_submit(self.chain_prepare(ops, check_finite))
        return [o["out"] for o in ops]

    def chain_submit(self, prepared):
        """Submits a list built by chain_prepare: the bare C call, for loops that reuse the same buffers."""
        n, arr, flags, host, _keep = prepared
        if not host:
            self._flags(False, False)
        self._check(self.lib.lev_matvec_chain(self.handle, n, arr, flags))

    def chain_prepare(self, ops, check_finite: bool = False):
        """The lev_chain_op array of a list (see matvec_chain), built once; the buffers it names must stay alive."""
        n = len(ops)
        arr = (L.ChainOp * n)()
        host = n > 0 and not _is_torch(ops[0]["x"])
        for i, o in enumerate(ops):
            w = o["w"]
            row0 = o.get("row0", 0)
            rows = o.get("rows", w.rows - row0)
            x, out = o["x"], o["out"]
            if host:
                assert x.dtype == np.float32 and x.flags["C_CONTIGUOUS"] and out.flags["C_CONTIGUOUS"]
            else:
                assert x.is_contiguous() and out.is_contiguous()
            f = self._fusion(o.get("prologue"), o.get("norm_weight"), o.get("eps", 1e-6), o.get("residual"), o.get("alpha", 1.0))
            arr[i] = L.ChainOp(w.handle, row0, rows, _ptr(x), _ptr(out), int(bool(o.get("depends", False))), f)
        flags = self._flags(host, check_finite)
        return n, arr, flags, host, [(o["x"], o["out"], o.get("residual"), o.get("norm_weight")) for o in ops]

    # -- decode attention over a paged KV cache (torch CUDA tensors only) --
    def kv_append(self, cache: "PagedKV", slot, pos, k, v):
        """lev_kv_append: k, v f32 [n_cols][kv_heads][head_dim] to position pos[c] of sequence slot[c]."""
        k, v = k.contiguous(), v.contiguous()  # held until the launch is queued
        self._flags(False, False)
        self._check(self.lib.lev_kv_append(self.handle, C.byref(cache.layout), _ptr(cache.k), _ptr(cache.v), _ptr(cache.table),
                                           _ptr(slot), _ptr(pos), int(slot.numel()), _ptr(k), _ptr(v)))

    def attn_decode(self, cache: "PagedKV", slot, pos, q, window: int = 0, scale: float = 1.0, out=None):
        """lev_attn_decode: q f32 [n_cols][q_heads][head_dim] -> out of the same shape."""
        import torch

        q = q.contiguous()
        out = torch.empty_like(q) if out is None else out
        self._flags(False, False)
        self._check(self.lib.lev_attn_decode(self.handle, C.byref(cache.layout), _ptr(cache.k), _ptr(cache.v), _ptr(cache.table),
                                             _ptr(slot), _ptr(pos), q.shape[0], q.shape[1], _ptr(q), window, scale, _ptr(out)))
        return out

    def attn_decode_fused_rows(self, cache: "PagedKV", slot, pos, qkv, q_heads: int, window: int = 0, scale: float = 1.0, out=None):
        """lev_attn_decode_ld: the queries are the leading q_heads * head_dim elements of each row of qkv
        [n_cols][(q_heads + 2 kv_heads) * head_dim], the fused projection output -> out [n_cols][q_heads][head_dim]."""
        import torch

        assert qkv.is_contiguous() and qkv.ndim == 2
        hd = cache.layout.head_dim
        out = torch.empty((qkv.shape[0], q_heads, hd), device=qkv.device) if out is None else out
        self._flags(False, False)
        self._check(self.lib.lev_attn_decode_ld(self.handle, C.byref(cache.layout), _ptr(cache.k), _ptr(cache.v), _ptr(cache.table),
                                                _ptr(slot), _ptr(pos), qkv.shape[0], q_heads, _ptr(qkv), qkv.shape[1], window, scale,
                                                _ptr(out)))
        return out

    def _matvec_host(self, fn, blocks, out_dim, in_dim, x):
        blocks = np.ascontiguousarray(blocks, np.uint8)
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty(max(out_dim, 0), np.float32)
        ev = L.Evidence()
        self._check(fn(self.handle, _ptr(blocks), blocks.size, out_dim, in_dim, _ptr(x), x.size, _ptr(y), C.byref(ev)))
        evidence = {k: (getattr(ev, k).decode() if k.endswith("_name") else getattr(ev, k)) for k, _ in ev._fields_}
        evidence["command_status"] = "completed" if ev.status == 0 else L.STATUS.get(ev.status, "?")
        return y, evidence

    def q4_0_matvec_reporting(self, blocks, out_dim, in_dim, x):
        """Q4MetalBackend.matvecReporting (Sources/LeviathanCore/Q4.swift:165-167)."""
        return self._matvec_host(self.lib.lev_q4_0_matvec_host, blocks, out_dim, in_dim, x)

    def q6_k_matvec_reporting(self, blocks, out_dim, in_dim, x):
        """Q6MetalBackend.matvecReporting (Sources/LeviathanCore/Q6.swift:199-201)."""
        return self._matvec_host(self.lib.lev_q6_k_matvec_host, blocks, out_dim, in_dim, x)

    def q4_k_matvec_reporting(self, blocks, out_dim, in_dim, x):
        """VulkanContext::run_matvec for Q4_K (rust/crates/lev-vulkan/src/lib.rs:571-582)."""
        return self._matvec_host(self.lib.lev_q4_k_matvec_host, blocks, out_dim, in_dim, x)

    # -- prefill --
    def act_bf16(self, x, out=None):
        import torch

        out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) if out is None else out
        self._flags(False, False)
        self._check(self.lib.lev_act_bf16(self.handle, _ptr(x.contiguous()), x.numel(), _ptr(out)))
        return out

    def gemm_prefill(self, w: Weights, x_bf16, out=None):
        """Y[t][r] = sum_k bf16(W[r][k]) X[t][k]; X torch bf16 CUDA [tokens][cols]."""
        import torch

        x_bf16 = x_bf16.contiguous()
        tokens = x_bf16.shape[0]
        if out is None:
            out = torch.empty((tokens, w.rows), dtype=torch.float32, device=x_bf16.device)
        self._flags(False, False)
        self._check(self.lib.lev_gemm_prefill(self.handle, w.handle, _ptr(x_bf16), tokens, _ptr(out), 0))
        return out

    # -- MoE --
    def moe_upload(self, router_w, gate_up, down, experts, hidden, inter, local_first=0, local_count=None) -> MoEWeights:
        local_count = experts if local_count is None else local_count
        on_dev = _is_torch(gate_up) and gate_up.is_cuda
        if not on_dev:
            router_w = np.ascontiguousarray(router_w, np.float32)
            gate_up = np.ascontiguousarray(gate_up, np.uint8)
            down = np.ascontiguousarray(down, np.uint8)
            gb, db = gate_up.size, down.size
        else:
            router_w, gate_up, down = router_w.contiguous(), gate_up.contiguous(), down.contiguous()
            gb, db = gate_up.numel(), down.numel()
        if on_dev:
            self._flags(False, False)
        h = C.c_void_p()
        self._check(self.lib.lev_moe_weights_upload(self.handle, _ptr(router_w), _ptr(gate_up), gb, _ptr(down), db,
                                                    experts, hidden, inter, local_first, local_count,
                                                    1 if on_dev else 0, C.byref(h)))
        return MoEWeights(self, h, experts, hidden, inter, local_first, local_count)

    def moe_route(self, mw: MoEWeights, x, top_k: int, want_scores: bool = False, check_finite: bool = False):
        host = not _is_torch(x)
        x = np.ascontiguousarray(x, np.float32) if host else x.contiguous()
        tokens = x.shape[0]
        idx = self._empty_like_io(x, (tokens, top_k), np.int32, "int32")
        wts = self._empty_like_io(x, (tokens, top_k), np.float32, "float32")
        scores = self._empty_like_io(x, (tokens, mw.experts), np.float32, "float32") if want_scores else None
        self._check(self.lib.lev_moe_route(self.handle, mw.handle, _ptr(x), tokens, top_k, _ptr(idx), _ptr(wts),
                                           _ptr(scores), self._flags(host, check_finite)))
        return (idx, wts, scores) if want_scores else (idx, wts)

    def moe_group(self, idx, experts: int):
        host = not _is_torch(idx)
        idx = np.ascontiguousarray(idx, np.int32) if host else idx.contiguous()
        tokens, top_k = idx.shape
        counts = self._empty_like_io(idx, (experts,), np.int32, "int32")
        offsets = self._empty_like_io(idx, (experts + 1,), np.int32, "int32")
        perm = self._empty_like_io(idx, (tokens * top_k,), np.int32, "int32")
        self._check(self.lib.lev_moe_group(self.handle, _ptr(idx), tokens, top_k, experts, _ptr(counts), _ptr(offsets),
                                           _ptr(perm), self._flags(host, False)))
        return counts, offsets, perm

    def moe_experts(self, mw: MoEWeights, x, idx, want_act: bool = False):
        host = not _is_torch(x)
        x = np.ascontiguousarray(x, np.float32) if host else x.contiguous()
        idx = np.ascontiguousarray(idx, np.int32) if host else idx.contiguous()
        tokens, top_k = idx.shape
        y = self._empty_like_io(x, (tokens, top_k, mw.hidden), np.float32, "float32")
        act = self._empty_like_io(x, (tokens, top_k, mw.inter), np.float32, "float32") if want_act else None
        self._check(self.lib.lev_moe_experts(self.handle, mw.handle, _ptr(x), tokens, top_k, _ptr(idx), _ptr(y),
                                             _ptr(act), self._flags(host, False)))
        return (y, act) if want_act else y

    def moe_combine(self, y_slots, weights):
        host = not _is_torch(y_slots)
        y_slots = np.ascontiguousarray(y_slots, np.float32) if host else y_slots.contiguous()
        weights = np.ascontiguousarray(weights, np.float32) if host else weights.contiguous()
        tokens, top_k, hidden = y_slots.shape
        out = self._empty_like_io(y_slots, (tokens, hidden), np.float32, "float32")
        self._check(self.lib.lev_moe_combine(self.handle, _ptr(y_slots), _ptr(weights), tokens, top_k, hidden, _ptr(out),
                                             self._flags(host, False)))
        return out

    def moe_layer(self, mw: MoEWeights, x, top_k: int, out=None, want_routing: bool = False, check_finite: bool = False,
                  expert_parallel: bool = False):
        host = not _is_torch(x)
        x = np.ascontiguousarray(x, np.float32) if host else x.contiguous()
        tokens = x.shape[0]
        if out is None:
            out = self._empty_like_io(x, (tokens, mw.hidden), np.float32, "float32")
        idx = self._empty_like_io(x, (tokens, top_k), np.int32, "int32") if want_routing else None
        wts = self._empty_like_io(x, (tokens, top_k), np.float32, "float32") if want_routing else None
        fn = self.lib.lev_moe_layer_ep if expert_parallel else self.lib.lev_moe_layer
        self._check(fn(self.handle, mw.handle, _ptr(x), tokens, top_k, _ptr(out), _ptr(idx), _ptr(wts),
                       self._flags(host, check_finite)))
        return (out, idx, wts) if want_routing else out

    def moe_layer_residual(self, mw: MoEWeights, x, top_k: int, residual, alpha: float = 1.0, out=None):
        """lev_moe_layer_residual: out = residual + alpha * layer(x) in the layer's own launches (torch CUDA tensors;
        out may be residual)."""
        x, residual = x.contiguous(), residual.contiguous()
        out = residual if out is None else out
        self._flags(False, False)
        self._check(self.lib.lev_moe_layer_residual(self.handle, mw.handle, _ptr(x), x.shape[0], top_k, _ptr(residual), float(alpha),
                                                    _ptr(out), 0))
        return out

    # -- op spec --
    def op_install(self, op_json: str | bytes):
        data = op_json.encode() if isinstance(op_json, str) else op_json
        h = C.c_void_p()
        self._check(self.lib.lev_op_install_json(self.handle, data, len(data), C.byref(h)))
        return h

    def op_describe(self, op) -> dict:
        kind = C.create_string_buffer(32)
        ident = C.create_string_buffer(65)
        kern = C.create_string_buffer(64)
        i, o, t, c = C.c_int64(), C.c_int64(), C.c_int(), C.c_int()
        self._check(self.lib.lev_op_describe(op, kind, C.byref(i), C.byref(o), C.byref(t), C.byref(c), ident, kern))
        return {"kind": kind.value.decode(), "in_dim": i.value, "out_dim": o.value, "ggml_type": t.value,
                "columns": c.value, "identity": ident.value.decode(), "kernel_name": kern.value.decode()}

    def op_serves(self, op, w: Weights, rows: int) -> bool:
        return bool(self.lib.lev_op_serves(op, w.handle, rows))

    def op_uninstall(self, op):
        self._check(self.lib.lev_op_uninstall(self.handle, op))

    # -- multi-GPU --
    @staticmethod
    def dist_unique_id() -> bytes:
        buf = C.create_string_buffer(L.NCCL_ID_BYTES)
        st = L.load().lev_dist_unique_id(buf)
        if st != L.OK:
            raise LevError(st, "lev_dist_unique_id")
        return buf.raw

    def dist_init(self, rank: int, world: int, unique_id: bytes):
        self._check(self.lib.lev_dist_init(self.handle, rank, world, unique_id))

    def matvec_rowsplit_allgather(self, w_local: Weights, x, world: int, out=None):
        import torch

        x = x.contiguous()
        one_d = x.ndim == 1
        n_cols = 1 if one_d else x.shape[0]
        if out is None:
            out = torch.empty((n_cols, w_local.rows * world), dtype=torch.float32, device=x.device)
        self._flags(False, False)
        self._check(self.lib.lev_matvec_rowsplit_allgather(self.handle, w_local.handle, _ptr(x), x.numel(), n_cols,
                                                           _ptr(out), out.numel(), 0))
        return out[0] if one_d else out

    def matvec_chain_rowsplit(self, ops):
        """lev_matvec_chain_rowsplit: ops like matvec_chain's (w = this rank's rows, out = the whole output)."""
        n = len(ops)
        arr = (L.ChainOp * n)()
        for i, o in enumerate(ops):
            w = o["w"]
            f = self._fusion(o.get("prologue"), o.get("norm_weight"), o.get("eps", 1e-6), None, 1.0)
            arr[i] = L.ChainOp(w.handle, 0, w.rows, _ptr(o["x"]), _ptr(o["out"]), 0, f)
        self._flags(False, False)
        self._check(self.lib.lev_matvec_chain_rowsplit(self.handle, n, arr))
        return [o["out"] for o in ops]

    def gemm_prefill_rowsplit_allgather(self, w_local: Weights, x_bf16, world: int, out=None):
        import torch

        x_bf16 = x_bf16.contiguous()
        tokens = x_bf16.shape[0]
        if out is None:
            out = torch.empty((tokens, w_local.rows * world), dtype=torch.float32, device=x_bf16.device)
        self._flags(False, False)
        self._check(self.lib.lev_gemm_prefill_rowsplit_allgather(self.handle, w_local.handle, _ptr(x_bf16), tokens,
                                                                 _ptr(out), 0))
        return out


class PagedKV:
    """Device pools and block table of one layer's paged KV cache (pools [blocks][page][kv_heads][head_dim],
    table [slots][max_blocks]; rust/crates/lev-model/src/kv.rs:36-85).  Block 0 is the scratch block every
    unused table entry points to; `ensure` hands out the others, low ids first, like BlockManager.ensure."""

    def __init__(self, blocks: int, page: int, kv_heads: int, head_dim: int, slots: int, max_blocks: int,
                 dtype: str = "f16", device: str = "cuda"):
        import torch

        td = torch.float16 if dtype == "f16" else torch.float32
        self.layout = L.KVLayout(L.KV_F16 if dtype == "f16" else L.KV_F32, page, kv_heads, head_dim, blocks, max_blocks, slots)
        self.k = torch.zeros((blocks, page, kv_heads, head_dim), dtype=td, device=device)
        self.v = torch.zeros_like(self.k)
        self.table_host = np.zeros((slots, max_blocks), np.int32)
        self.table = torch.zeros((slots, max_blocks), dtype=torch.int32, device=device)
        self.free = list(range(blocks - 1, 0, -1))
        self.owned = [[] for _ in range(slots)]
        self.page, self.max_blocks = page, max_blocks

    def ensure(self, slot: int, pos: int) -> int:
        """Make sequence `slot` own the block of `pos`; returns the flat pool position."""
        import torch

        need = pos // self.page + 1
        if need > self.max_blocks:
            raise IndexError("beyond context")
        grew = False
        while len(self.owned[slot]) < need:
            if not self.free:
                raise MemoryError("out of blocks")
            b = self.free.pop()
            self.table_host[slot, len(self.owned[slot])] = b
            self.owned[slot].append(b)
            grew = True
        if grew:
            self.table.copy_(torch.from_numpy(self.table_host))
        return self.owned[slot][pos // self.page] * self.page + pos % self.page

    def release(self, slot: int):
        import torch

        while self.owned[slot]:
            self.free.append(self.owned[slot].pop())
        self.table_host[slot] = 0
        self.table.copy_(torch.from_numpy(self.table_host))


class GGUFFile:
    """lev_gguf_*: a parsed GGUF v2/v3 container (GGUFFile in the reference,
    Sources/LeviathanCore/GGUF.swift:96-406).  `source` is a path (mapped
    read-only) or a bytes-like object (kept alive by this object).  Needs no
    device; `upload` needs a Context."""

    def __init__(self, source):
        self.lib = L.load()
        h = C.c_void_p()
        err = C.create_string_buffer(256)
        if isinstance(source, str):
            st = self.lib.lev_gguf_open(source.encode(), C.byref(h), err, len(err))
            self._keep = None
        else:
            self._keep = np.frombuffer(bytes(source), np.uint8)
            st = self.lib.lev_gguf_parse(self._keep.ctypes.data, self._keep.size, C.byref(h), err, len(err))
        if st != L.OK:
            raise LevError(st, err.value.decode(errors="replace"))
        self.handle = h
        v, nt, nk, al, off = C.c_uint32(), C.c_int64(), C.c_int64(), C.c_uint64(), C.c_uint64()
        self.lib.lev_gguf_summary(h, C.byref(v), C.byref(nt), C.byref(nk), C.byref(al), C.byref(off))
        self.version, self.tensor_count, self.metadata_count = v.value, nt.value, nk.value
        self.alignment, self.data_offset = al.value, off.value

    def close(self):
        if self.handle:
            self.lib.lev_gguf_close(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def tensor(self, key) -> dict:
        """Directory entry by index or name: name, ggml_type, dims (innermost first),
        file_offset (absolute), n_bytes.  Raises LevError('missing') when absent."""
        i = key if isinstance(key, int) else self.lib.lev_gguf_find_tensor(self.handle, key.encode())
        name, ty, nd, dims = C.c_char_p(), C.c_int(), C.c_int(), (C.c_int64 * 4)()
        off, nb = C.c_uint64(), C.c_uint64()
        st = self.lib.lev_gguf_tensor_info(self.handle, i, C.byref(name), C.byref(ty), C.byref(nd), C.byref(dims),
                                           C.byref(off), C.byref(nb))
        if st != L.OK:
            raise LevError(st, f"tensor {key!r}")
        return {"index": i, "name": name.value.decode(), "ggml_type": ty.value, "dims": list(dims)[:nd.value],
                "file_offset": off.value, "n_bytes": nb.value}

    def tensors(self) -> list:
        return [self.tensor(i) for i in range(self.tensor_count)]

    def tensor_bytes(self, key) -> np.ndarray:
        """The tensor's storage as a uint8 copy."""
        t = self.tensor(key)
        p = self.lib.lev_gguf_tensor_data(self.handle, t["index"])
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(t["n_bytes"],)).copy()

    def meta_uint(self, key: str) -> int:
        v = C.c_uint64()
        st = self.lib.lev_gguf_meta_u64(self.handle, key.encode(), C.byref(v))
        if st != L.OK:
            raise LevError(st, f"metadata {key}")
        return v.value

    def meta_float(self, key: str) -> float:
        v = C.c_double()
        st = self.lib.lev_gguf_meta_f64(self.handle, key.encode(), C.byref(v))
        if st != L.OK:
            raise LevError(st, f"metadata {key}")
        return v.value

    def meta_string(self, key: str) -> str:
        p, n = C.c_char_p(), C.c_size_t()
        st = self.lib.lev_gguf_meta_string(self.handle, key.encode(), C.byref(p), C.byref(n))
        if st != L.OK:
            raise LevError(st, f"metadata {key}")
        return C.string_at(p, n.value).decode(errors="replace")

    _SCALAR = {0: "<u1", 1: "<i1", 2: "<u2", 3: "<i2", 4: "<u4", 5: "<i4", 6: "<f4", 7: "<u1", 10: "<u8", 11: "<i8",
               12: "<f8"}

    def meta_array(self, key: str) -> list:
        """An array value as a Python list (strings, ints, floats or bools)."""
        et, n = C.c_int(), C.c_uint64()
        st = self.lib.lev_gguf_meta_array(self.handle, key.encode(), C.byref(et), C.byref(n))
        if st != L.OK:
            raise LevError(st, f"metadata {key}")
        out = []
        p, nb = C.c_void_p(), C.c_size_t()
        for i in range(n.value):
            self.lib.lev_gguf_meta_array_item(self.handle, key.encode(), i, C.byref(p), C.byref(nb))
            raw = C.string_at(p, nb.value)
            if et.value == 8:
                out.append(raw.decode(errors="replace"))
            else:
                v = np.frombuffer(raw, self._SCALAR[et.value])[0].item()
                out.append(bool(v) if et.value == 7 else v)
        return out

    def upload(self, ctx: "Context", name: str) -> Weights:
        """lev_gguf_upload: a quantized tensor straight from the mapping to the device."""
        h = C.c_void_p()
        ctx._check(self.lib.lev_gguf_upload(ctx.handle, self.handle, name.encode(), C.byref(h)))
        ty, rows, cols, nb = C.c_int(), C.c_int64(), C.c_int64(), C.c_size_t()
        self.lib.lev_weights_info(h, C.byref(ty), C.byref(rows), C.byref(cols), C.byref(nb))
        return Weights(ctx, h, ty.value, rows.value, cols.value, nb.value)

    def moe_upload(self, ctx: "Context", layer: int, local_first: int = 0, local_count: int = 0):
        """lev_gguf_moe_upload: (MoEWeights of blk.<layer>, the file's expert_used_count)."""
        h, k = C.c_void_p(), C.c_int()
        ctx._check(self.lib.lev_gguf_moe_upload(ctx.handle, self.handle, layer, local_first, local_count, C.byref(h),
                                                C.byref(k)))
        arch = self.meta_string("general.architecture")
        experts = self.meta_uint(f"{arch}.expert_count")
        hidden, inter = self.meta_uint(f"{arch}.embedding_length"), self.meta_uint(f"{arch}.expert_feed_forward_length")
        return MoEWeights(ctx, h, experts, hidden, inter, local_first, local_count or experts), k.value
