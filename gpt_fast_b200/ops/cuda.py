"""ctypes bindings of the kernel libraries: host-side checks, kernel choice,
launch on the current stream."""
import ctypes
from ctypes import c_float, c_int, c_long, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from ..csrc import build
from .types import BatchMeta, PagedKV

_DT = {torch.float32: 0, torch.bfloat16: 1}
_EPI = {"store": 0, "add": 1, "swiglu": 2, "gelu": 4, "gelu_tanh": 5, "silu": 6, "relu2": 7}
_UNARY = ("gelu", "gelu_tanh", "silu", "relu2")
_TC_UNARY = ("gelu", "relu2")             # the unary epilogues the tensor-core product has (they store bfloat16)
_PAIRING = {"interleaved": 0, "half": 1}


def _fail(msg):
    from . import KernelError
    raise KernelError(msg)


def _dt(t: torch.Tensor) -> int:
    if t.dtype not in _DT:
        _fail(f"kernels take float32 or bfloat16, got {t.dtype}")
    return _DT[t.dtype]


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, dtype=None, shape=None, name="tensor"):
    if not t.is_cuda:
        _fail(f"{name} is on {t.device}: the kernels of this library run on a CUDA device only")
    if not t.is_contiguous():
        _fail(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        _fail(f"{name} must be {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        _fail(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream of the current device as a handle for the kernels.  Asked for at every launch (a capture
    runs on a stream of its own); the short way through torch's C module costs a tenth of `current_stream()`."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def decode_slices(max_kv_len: int, page_size: int, blocks: int, sm_count: int) -> int:
    """Into how many slices a decode step cuts each sequence's cache (`blocks` = tokens x key/value heads, the
    blocks of one slice).  A simple cost model fitted to measurements on a B200 (contexts of 600 to 32,000,
    batches of 1 to 64): two blocks fit on an SM, so blocks * slices run in ceil(blocks * slices / (2 SMs))
    rounds; a round costs the pages of a slice plus about four pages' worth of fixed work per block; a slice
    keeps at least 4 pages.  The cheapest count wins, the smaller one on ties."""
    pages = -(-max(max_kv_len, 1) // page_size)
    cap = 2 * sm_count
    best, best_cost = 1, None
    for s in range(1, max(1, min(pages // 4, 48)) + 1):
        cost = -(-blocks * s // cap) * (pages / s + 4.0)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


class CudaKernels:
    """The operations of `ops`, bound to the sm_100a libraries.  A library is
    compiled and loaded when its first function is needed."""

    def __init__(self):
        if not torch.cuda.is_available():
            _fail("no CUDA device: this library has no CPU path")
        self._fn = {}
        self._sm_count = None
        self._status = None
        self.trace = None                  # a list: (label, start event, stop event) of every launch is appended
        self._label = None                 # what the next launch is called in the trace (default: the entry point)
        self._bias_cache = {}              # distance biases in the tensor-core prefill kernel's layout, by table
        self._overlap = True               # kernels may start while their predecessor drains (programmatic dependent launch)

    def _f(self, lib: str, name: str):
        key = (lib, name)
        fn = self._fn.get(key)
        if fn is None:
            handle = build.library(lib)
            if not self._overlap:
                handle.gfb_set_overlap(0)
            fn = getattr(handle, name)
            fn.restype = c_int
            self._fn[key] = fn
            fn._lib = handle
        return fn

    def set_launch_overlap(self, on: bool) -> None:
        """Whether the kernels launched from now on may start while their predecessor in the stream still drains.  Off: every
        launch waits for the one before it in the ordinary way."""
        on = bool(on)
        if on == self._overlap:
            return
        self._overlap = on
        for handle in {fn._lib for fn in self._fn.values()}:
            handle.gfb_set_overlap(1 if on else 0)

    def _call(self, lib, name, *args):
        fn = self._f(lib, name)
        trace = self.trace
        if trace is not None:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        rc = fn(*args)
        if trace is not None:
            stop.record()
            trace.append((self._label or name, start, stop))
        self._label = None
        if rc != 0:
            _fail(f"{name}: {fn._lib.gfb_last_error().decode()}")

    # -- element-wise / per-row -------------------------------------------------
    def embed(self, tokens, table, out, status, scale=1.0):
        T = tokens.shape[0]
        V, D = table.shape
        _need(tokens, torch.int32, name="tokens")
        _need(table, name="embedding table")
        _need(out, torch.float32, (T, D), "embedding output")
        self._call("core", "gfb_embed", _ptr(tokens), _ptr(table), c_int(_dt(table)), _ptr(out),
                   c_int(T), c_int(D), c_int(V), c_float(scale), _ptr(status), _stream())

    def embed_hashed(self, tokens, table, extra, out, batch, prev, buckets, mul_prev, mul_cur, scale=1.0):
        T = tokens.shape[0]
        V, D = table.shape
        _need(tokens, torch.int32, (batch.n_tokens,), "tokens")
        _need(table, name="embedding table")
        _need(extra, table.dtype, (buckets + 1, D), "hashed embedding table")
        _need(out, torch.float32, (T, D), "embedding output")
        _need(prev, torch.int32, name="previous tokens")
        self._call("embedding", "gfb_embed_hashed", _ptr(tokens), _ptr(table), _ptr(extra), c_int(_dt(table)), _ptr(out),
                   *self._batch_args(batch), _ptr(prev), c_int(D), c_int(V), c_int(buckets), c_longlong(mul_prev), c_longlong(mul_cur),
                   c_float(scale), _ptr(batch.status), _stream())

    def embed_positions(self, tokens, table, positions, out, batch, scale=1.0):
        T = tokens.shape[0]
        V, D = table.shape
        _need(tokens, torch.int32, (batch.n_tokens,), "tokens")
        _need(table, name="embedding table")
        _need(positions, table.dtype, (positions.shape[0], D), "position table")
        _need(out, torch.float32, (T, D), "embedding output")
        self._call("embedding", "gfb_embed_positions", _ptr(tokens), _ptr(table), _ptr(positions), c_int(_dt(table)), _ptr(out),
                   *self._batch_args(batch), c_int(D), c_int(V), c_int(positions.shape[0]), c_float(scale), _ptr(batch.status),
                   _stream())

    def softcap(self, x, cap):
        _need(x, torch.float32, name="logits")
        self._call("core", "gfb_softcap", _ptr(x), c_long(x.numel()), c_float(cap), _stream())

    def rmsnorm(self, x, weight, eps, out, rows=None, pending=None):
        D = x.shape[-1]
        R = out.shape[0]
        _need(x, torch.float32, name="norm input")
        _need(weight, shape=(D,), name="norm weight")
        _need(out, shape=(R, D), name="norm output")
        if rows is not None:
            _need(rows, torch.int32, (R,), "rows")
            if pending is not None:
                self.add_partials(x, pending)
                pending = None
        elif x.shape[0] != R:
            _fail(f"norm output has {R} rows, input {x.shape[0]}")
        S = 0
        if pending is not None:
            S = pending.shape[0]
            _need(pending, torch.float32, (S,) + tuple(x.shape), "pending partial sums")
        self._call("core", "gfb_rmsnorm", _ptr(x), _ptr(pending), c_int(S), c_long(x.numel()), _ptr(weight),
                   c_int(_dt(weight)), _ptr(out), c_int(_dt(out)), _ptr(rows), c_int(R), c_int(D), c_float(eps), _stream())

    def add_partials(self, x, pending):
        _need(x, torch.float32, name="sum")
        _need(pending, torch.float32, (pending.shape[0],) + tuple(x.shape), "pending partial sums")
        self._call("core", "gfb_add_partials", _ptr(x), _ptr(pending), c_int(pending.shape[0]), c_long(x.numel()), _stream())

    def rope_table(self, inv_freq, table, amplitude=1.0):
        P, half, two = table.shape
        _need(inv_freq, torch.float32, (half,), "inv_freq")
        _need(table, torch.float32, name="rotary table")
        self._call("core", "gfb_rope_table", _ptr(inv_freq), _ptr(table), c_int(P), c_int(half), c_float(amplitude), _stream())

    def _batch_args(self, b: BatchMeta):
        return (_ptr(b.cu_seqlens), _ptr(b.tok_seq), _ptr(b.slots), _ptr(b.lengths), c_int(b.n_seqs), c_int(b.n_tokens))

    def _kv_args(self, kv: PagedKV):
        return (_ptr(kv.k_pool), _ptr(kv.v_pool), _ptr(kv.page_table), c_int(kv.page_table.shape[1]),
                c_int(kv.page_size), c_int(kv.k_pool.shape[0]))

    def rope_append(self, qkv, q_out, kv, batch, table, n_head, n_kv, head_dim, pairing, append, partials=None):
        T = batch.n_tokens
        W = (n_head + 2 * n_kv) * head_dim
        if partials is not None:
            _need(partials, torch.float32, (partials.shape[0], T, W), "partial sums of qkv")
            src, n_part = partials, partials.shape[0]
        else:
            _need(qkv, shape=(T, W), name="qkv")
            src, n_part = qkv, 0
        _need(q_out, shape=(T, n_head, head_dim), name="q_out")
        qkv = q_out                                     # the element type of the outputs
        _need(table, torch.float32, name="rotary table")
        if append:
            _need(kv.k_pool, qkv.dtype, name="key pool")
            if tuple(kv.k_pool.shape[1:]) != (n_kv, kv.page_size, head_dim):
                _fail(f"key pool pages are {tuple(kv.k_pool.shape[1:])}, the layer needs {(n_kv, kv.page_size, head_dim)}")
        self._call("core", "gfb_rope_append", _ptr(src), c_int(n_part), _ptr(q_out), c_int(_dt(q_out)), *self._kv_args(kv),
                   *self._batch_args(batch), _ptr(table), c_int(table.shape[0]), c_int(n_head), c_int(n_kv),
                   c_int(head_dim), c_int(_PAIRING[pairing]), c_int(1 if append else 0), _ptr(batch.status), _stream())

    def advance_lengths(self, batch):
        self._call("core", "gfb_advance_lengths", _ptr(batch.lengths), _ptr(batch.slots), _ptr(batch.cu_seqlens),
                   c_int(batch.n_seqs), _stream())

    def add_into(self, out, y):
        _need(out, torch.float32, name="sum")
        _need(y, shape=out.shape, name="addend")
        self._call("core", "gfb_add_into", _ptr(out), _ptr(y), c_int(_dt(y)), c_long(out.numel()), _stream())

    # -- layer norm, q/k/v preparation, retention, activations ---------------------------
    def layernorm(self, x, weight, bias, eps, out, rows=None, branch=None, rms=False):
        T, D = x.shape
        _need(x, torch.float32, name="norm input")
        if out is not None:
            R = out.shape[0]
            if weight is not None:
                _need(weight, shape=(D,), name="norm weight")
            if not rms and bias is not None and weight is not None:
                _need(bias, weight.dtype, (D,), "norm bias")
            _need(out, shape=(R, D), name="norm output")
            if rows is not None:
                _need(rows, torch.int32, (R,), "rows")
            elif R != T:
                _fail(f"norm output has {R} rows, input {T}")
        else:
            R = T
        y = pw = pb = None
        S, peps, mult = 0, 0.0, 0.0
        if branch is not None:
            y, pw, pb, peps, mult = branch
            if rows is not None:
                _fail("a branch sum cannot be combined with a row gather")
            _need(pw, shape=(D,), name="branch norm weight")
            if not rms and pb is not None:
                _need(pb, pw.dtype, (D,), "branch norm bias")
            if y.dim() == 3:
                S = y.shape[0]
                _need(y, torch.float32, (S, T, D), "partial sums of the branch")
            else:
                _need(y, torch.float32, (T, D), "branch")
        elif out is None:
            return
        self._call("layernorm", "gfb_layernorm", _ptr(x), _ptr(y), c_int(S), c_long(T * D), _ptr(pw), _ptr(pb),
                   c_int(_dt(pw) if pw is not None else 0), c_float(peps), c_float(mult), _ptr(weight if out is not None else None),
                   _ptr(bias if out is not None and weight is not None else None), c_int(_dt(weight) if out is not None and weight is not None else 0), c_float(eps),
                   _ptr(out), c_int(_dt(out) if out is not None else 0), _ptr(rows), c_int(R), c_int(D), c_int(1 if rms else 0),
                   _stream())

    def layernorm_multi(self, x, branches=(), outs=(), rows=None, rms=False):
        T, D = x.shape
        _need(x, torch.float32, name="norm input")
        if len(branches) > 2 or len(outs) > 2:
            _fail("at most two branches and two outputs")
        if branches and rows is not None:
            _fail("a branch sum cannot be combined with a row gather")
        b_args, scale_dt = [], 0
        for y, scale in list(branches) + [(None, None)] * (2 - len(branches)):
            S = 0
            if y is not None:
                if y.dim() == 3:
                    S = y.shape[0]
                    _need(y, torch.float32, (S, T, D), "partial sums of a branch")
                else:
                    _need(y, torch.float32, (T, D), "branch")
                if scale is not None:
                    _need(scale, shape=(D,), name="branch factor")
                    scale_dt = _dt(scale)
            b_args += [_ptr(y), c_int(S), _ptr(scale)]
        scales = [s for _, s in branches if s is not None]
        if len(scales) == 2 and scales[0].dtype != scales[1].dtype:
            _fail("the branch factors must have one type")
        o_args, w_dt, out_dt, R = [], 0, 0, T
        for w, eps, out in list(outs) + [(None, 0.0, None)] * (2 - len(outs)):
            if out is not None:
                R = out.shape[0]
                _need(w, shape=(D,), name="norm weight")
                _need(out, shape=(R, D), name="norm output")
                w_dt, out_dt = _dt(w), _dt(out)
            o_args += [_ptr(w), c_float(eps), _ptr(out)]
        if len(outs) == 2 and (outs[0][0].dtype != outs[1][0].dtype or outs[0][2].dtype != outs[1][2].dtype
                               or outs[0][2].shape != outs[1][2].shape):
            _fail("the two outputs must agree in shape and types")
        if rows is not None:
            _need(rows, torch.int32, (R,), "rows")
        elif outs and R != T:
            _fail(f"norm output has {R} rows, input {T}")
        if not branches and not outs:
            return
        self._call("layernorm", "gfb_layernorm_multi", _ptr(x), *b_args[:3], *b_args[3:], c_int(scale_dt), c_long(T * D),
                   *o_args[:3], *o_args[3:], c_int(w_dt), c_int(out_dt), _ptr(rows), c_int(R), c_int(D), c_int(1 if rms else 0),
                   _stream())

    def latent_prepare(self, src, q_off, kv_off, q_out, kv, batch, n_head, head_dim, rot_dim, rank, norm_weight, eps, table,
                       pairing="interleaved", append=True):
        T = batch.n_tokens
        W = src.shape[1]
        _need(src, q_out.dtype, (T, W), "projection")
        if max(q_off + n_head * (head_dim + rot_dim), kv_off + rank + rot_dim) > W:
            _fail(f"queries at {q_off} and the down projection at {kv_off} do not fit rows of {W}")
        _need(q_out, shape=(T, n_head, rank + rot_dim), name="q_out")
        _need(norm_weight, shape=(rank,), name="latent norm weight")
        _need(table, torch.float32, name="rotary table")
        if table.shape[1] * 2 != rot_dim:
            _fail(f"the rotary table serves {table.shape[1] * 2} dimensions, the mixer rotates {rot_dim}")
        if append:
            _need(kv.k_pool, q_out.dtype, name="key pool")
            if tuple(kv.k_pool.shape[1:]) != (1, kv.page_size, rank + rot_dim):
                _fail(f"cache pages are {tuple(kv.k_pool.shape[1:])}, the layer needs {(1, kv.page_size, rank + rot_dim)}")
        self._call("latent", "gfb_latent_prepare", _ptr(src), c_int(_dt(src)), c_int(W), c_int(q_off), c_int(kv_off), _ptr(q_out),
                   _ptr(kv.k_pool), _ptr(kv.page_table), c_int(kv.page_table.shape[1]), c_int(kv.page_size), c_int(kv.k_pool.shape[0]),
                   *self._batch_args(batch), _ptr(table), c_int(table.shape[0]), _ptr(norm_weight), c_int(_dt(norm_weight)),
                   c_float(eps), c_int(n_head), c_int(head_dim), c_int(rot_dim), c_int(rank), c_int(_PAIRING[pairing]),
                   c_int(1 if append else 0), _ptr(batch.status), _stream())

    def headwise_linear(self, a, w, out, n_head, k, n, a_off=0, a_stride=None, out_off=0, out_stride=None, gate=None, gate_off=0):
        T = a.shape[0]
        a_stride = k if a_stride is None else a_stride
        out_stride = n if out_stride is None else out_stride
        _need(a, name="head-wise input")
        _need(out, a.dtype, name="head-wise output")
        if a.dim() != 2 or out.dim() != 2 or out.shape[0] != T:
            _fail("head-wise product: input and output are [tokens, columns]")
        _need(w, a.dtype, (n_head, k, n), "head-wise weight")
        if a_off + (n_head - 1) * a_stride + k > a.shape[1] or out_off + (n_head - 1) * out_stride + n > out.shape[1]:
            _fail("head-wise product: the heads do not fit the rows")
        if gate is not None:
            _need(gate, a.dtype, name="gate")
            if gate.shape[0] != T or gate_off + n_head * n > gate.shape[1]:
                _fail("head-wise product: the gate does not fit")
        self._call("latent", "gfb_headwise_linear", _ptr(a), c_int(_dt(a)), c_int(a.shape[1]), c_int(a_off), c_int(a_stride), _ptr(w), _ptr(out), c_int(out.shape[1]), c_int(out_off), c_int(out_stride), _ptr(gate),
                   c_int(gate.shape[1] if gate is not None else 0), c_int(gate_off), c_int(T), c_int(n_head), c_int(k), c_int(n),
                   _stream())

    @staticmethod
    def _state_args(state, state_off, need):
        _need(state, torch.float32, name="per-sequence state")
        if state.dim() != 2 or state_off < 0 or state_off + need > state.shape[1]:
            _fail(f"{need} numbers of state at column {state_off} do not fit rows of {tuple(state.shape)}")
        return c_void_p(state.data_ptr() + 4 * state_off), c_long(state.shape[1])

    def short_conv(self, src, col_off, channels, weight, bias, state, state_off, out, batch, act=True, in_bias=None):
        T = batch.n_tokens
        taps = weight.shape[1]
        _need(src, name="convolution input")
        if src.shape[0] != T or col_off + channels > src.shape[1]:
            _fail(f"{channels} channels at column {col_off} do not fit {tuple(src.shape)}")
        _need(weight, shape=(channels, taps), name="convolution weight")
        if bias is not None:
            _need(bias, weight.dtype, (channels,), "convolution bias")
        if in_bias is not None:
            _need(in_bias, weight.dtype, (channels,), "bias of the convolution's inputs")
        _need(out, torch.float32, (T, channels), "convolution output")
        sp, sld = self._state_args(state, state_off, (taps - 1) * channels)
        self._call("recurrent", "gfb_short_conv", _ptr(src), c_int(_dt(src)), c_int(src.shape[1]), c_int(col_off), c_int(channels),
                   _ptr(weight), _ptr(bias), _ptr(in_bias), c_int(_dt(weight)), c_int(taps), sp, sld, _ptr(out), *self._batch_args(batch),
                   c_int(1 if act else 0), _stream())

    def rglru(self, u, w_a, w_i, b_a, b_i, lam, decay_scale, y_src, y_off, y_bias, state, state_off, out, batch):
        T = batch.n_tokens
        C = u.shape[1]
        blocks, bw = w_a.shape[0], w_a.shape[1]
        _need(u, torch.float32, (T, C), "recurrence input")
        if blocks * bw != C:
            _fail(f"gate matrices {tuple(w_a.shape)} do not cover {C} channels")
        _need(w_a, shape=(blocks, bw, bw), name="recurrence gate matrices")
        _need(w_i, w_a.dtype, (blocks, bw, bw), "input gate matrices")
        for v, name in ((b_a, "recurrence gate bias"), (b_i, "input gate bias"), (lam, "decay parameter"), (y_bias, "gate branch bias")):
            _need(v, b_a.dtype, (C,), name)
        _need(y_src, name="gate branch")
        if y_src.dim() != 2 or y_src.shape[0] != T or y_off + C > y_src.shape[1]:
            _fail(f"{C} columns at {y_off} do not fit {tuple(y_src.shape)}")
        _need(out, shape=(T, C), name="recurrence output")
        sp, sld = self._state_args(state, state_off, C)
        fn = self._f("recurrent", "gfb_rglru_scratch_floats")
        fn.restype = c_long
        need = fn(c_int(T), c_int(batch.n_seqs), c_int(int(batch.max_q_len)), c_int(C))
        fn.restype = c_int
        scratch = torch.empty(need, dtype=torch.float32, device=u.device)
        self._call("recurrent", "gfb_rglru", _ptr(u), _ptr(w_a), _ptr(w_i), c_int(_dt(w_a)), _ptr(b_a), _ptr(b_i), _ptr(lam), _ptr(y_bias),
                   c_int(_dt(b_a)), c_float(decay_scale), _ptr(y_src), c_int(_dt(y_src)), c_int(y_src.shape[1]), c_int(y_off), sp, sld,
                   _ptr(out), c_int(_dt(out)), _ptr(scratch), *self._batch_args(batch), c_int(int(batch.max_q_len)), c_int(C), c_int(blocks),
                   _stream())

    def ssd_scan(self, x, b_off, c_off, dt_src, dt_off, dt_bias, a_log, skip, state, state_off, out, batch, n_head, head_dim,
                 n_state, n_groups):
        T = batch.n_tokens
        _need(x, torch.float32, name="scan input")
        if x.shape[0] != T or max(n_head * head_dim, b_off + n_groups * n_state, c_off + n_groups * n_state) > x.shape[1]:
            _fail(f"heads, B and C do not fit rows of {tuple(x.shape)}")
        _need(dt_src, name="step sizes")
        if dt_src.shape[0] != T or dt_off + n_head > dt_src.shape[1]:
            _fail("the step sizes do not fit their rows")
        for v, name in ((dt_bias, "dt_bias"), (a_log, "A_log")) + (((skip, "D"),) if skip is not None else ()):
            _need(v, dt_bias.dtype, (n_head,), name)
        _need(out, torch.float32, (T, n_head, head_dim), "scan output")
        sp, sld = self._state_args(state, state_off, n_head * n_state * head_dim)
        self._call("recurrent", "gfb_ssd_scan", _ptr(x), c_int(x.shape[1]), c_int(b_off), c_int(c_off), _ptr(dt_src), c_int(_dt(dt_src)),
                   c_int(dt_src.shape[1]), c_int(dt_off), _ptr(dt_bias), _ptr(a_log), _ptr(skip), c_int(_dt(dt_bias)), sp, sld,
                   _ptr(out), *self._batch_args(batch), c_int(n_head), c_int(head_dim), c_int(n_state), c_int(n_groups), _stream())

    def delta_rule(self, qkv, offsets, beta_src, beta_off, a_src, a_off, dt_bias, a_log, state, state_off, out, batch, n_head,
                   n_qk, head_dim, v_head_dim, q_scale, unit_eps=1e-6, head_decay=False):
        T = batch.n_tokens
        q_off, k_off, v_off = offsets
        _need(qkv, torch.float32, name="q, k, v")
        if qkv.shape[0] != T or max(q_off + n_qk * head_dim, k_off + n_qk * head_dim, v_off + n_head * v_head_dim) > qkv.shape[1]:
            _fail(f"q, k and v at {offsets} do not fit rows of {tuple(qkv.shape)}")
        _need(beta_src, name="beta")
        _need(a_src, torch.float32, name="decay input")
        per_head = 1 if head_decay else head_dim
        if beta_src.shape[0] != T or beta_off + n_head > beta_src.shape[1] or a_src.shape[0] != T or a_off + n_head * per_head > a_src.shape[1]:
            _fail("beta or the decay input do not fit their rows")
        _need(dt_bias, shape=(n_head * per_head,), name="dt_bias")
        _need(a_log, dt_bias.dtype, (n_head,), "A_log")
        _need(out, torch.float32, (T, n_head, v_head_dim), "delta-rule output")
        sp, sld = self._state_args(state, state_off, n_head * head_dim * v_head_dim)
        self._call("recurrent", "gfb_delta_rule", _ptr(qkv), c_int(qkv.shape[1]), c_int(q_off), c_int(k_off), c_int(v_off),
                   _ptr(beta_src), c_int(_dt(beta_src)), c_int(beta_src.shape[1]), c_int(beta_off), _ptr(a_src), c_int(a_src.shape[1]),
                   c_int(a_off), _ptr(dt_bias), _ptr(a_log), c_int(_dt(dt_bias)), sp, sld, _ptr(out), *self._batch_args(batch),
                   c_int(n_head), c_int(n_qk), c_int(head_dim), c_int(v_head_dim), c_float(q_scale), c_float(unit_eps),
                   c_int(1 if head_decay else 0), _stream())

    def gated_norm(self, y, gate, gate_off, weight, out, group, eps, act="silu", gate_first=False):
        T, C = y.shape
        _need(y, torch.float32, name="norm input")
        _need(gate, name="gate")
        _need(out, shape=(T, C), name="gated output")
        _need(weight, name="norm weight")
        if C % group or gate.shape[0] != T or gate_off + C > gate.shape[1] or (C % weight.shape[0] and weight.shape[0] % group):
            _fail(f"groups of {group}, a gate of {tuple(gate.shape)} at {gate_off} or a weight of {tuple(weight.shape)} do not fit {C} columns")
        if act not in ("silu", "sigmoid"):
            _fail(f"unknown gate activation '{act}'")
        self._call("recurrent", "gfb_gated_norm", _ptr(y), _ptr(gate), c_int(_dt(gate)), c_int(gate.shape[1]), c_int(gate_off),
                   _ptr(weight), c_int(_dt(weight)), c_int(weight.shape[0]), _ptr(out), c_int(_dt(out)), c_int(T), c_int(C // group),
                   c_int(group), c_float(eps), c_int(1 if act == "sigmoid" else 0), c_int(1 if gate_first else 0), _stream())

    def qkv_prepare(self, src, partials, offsets, q_out, kv, batch, n_head, n_kv, head_dim, v_head_dim, table=None, rot_dims=0,
                    pairing="half", q_norm=None, k_norm=None, norm_eps=0.0, k_scale=1.0, append=True, norm_whole=False,
                    norm_bare=False, norm_last=False, maps=1, q_spread=False):
        T = batch.n_tokens
        if norm_whole and (norm_bare or norm_last or maps != 1):
            _fail("a norm over the whole projection has weights, runs ahead of the rotation and knows one map per head")
        if partials is not None:
            W = partials.shape[2]
            _need(partials, torch.float32, (partials.shape[0], T, W), "partial sums of the projection")
            source, n_part = partials, partials.shape[0]
        else:
            W = src.shape[1]
            _need(src, q_out.dtype, (T, W), "projection")
            source, n_part = src, 0
        q_off, k_off, v_off = offsets
        ends = [q_off + n_head * maps * head_dim] + ([k_off + n_kv * maps * head_dim, v_off + n_kv * v_head_dim] if append else [])
        if max(ends) > W:
            _fail(f"q, k and v at {offsets} do not fit rows of {W}")
        _need(q_out, shape=(T, n_head * maps, head_dim * (maps if q_spread else 1)), name="q_out")
        if table is not None:
            _need(table, torch.float32, name="rotary table")
            if table.shape[1] * 2 != rot_dims:
                _fail(f"the rotary table serves {table.shape[1] * 2} dimensions, the mixer rotates {rot_dims}")
        w_dt = 0
        for wn, heads in ((q_norm, n_head), (k_norm, n_kv)):
            if wn is not None:
                _need(wn, shape=((heads if norm_whole else 1) * head_dim,), name="q/k norm weight")
                w_dt = _dt(wn)
        if q_norm is not None and k_norm is not None and q_norm.dtype != k_norm.dtype:
            _fail("the q and k norm weights must have one type")
        if append:
            _need(kv.k_pool, q_out.dtype, name="key pool")
            if tuple(kv.k_pool.shape[1:]) != (n_kv, kv.page_size, head_dim * maps) or tuple(kv.v_pool.shape[1:]) != (n_kv, kv.page_size, v_head_dim):
                _fail(f"cache pages are {tuple(kv.k_pool.shape[1:])} / {tuple(kv.v_pool.shape[1:])}, the layer needs "
                      f"{(n_kv, kv.page_size, head_dim * maps)} / {(n_kv, kv.page_size, v_head_dim)}")
        self._call("qkv_prepare", "gfb_qkv_prepare", _ptr(source), c_int(n_part), c_int(W), c_int(q_off), c_int(k_off), c_int(v_off),
                   _ptr(q_out), c_int(_dt(q_out)), *self._kv_args(kv), *self._batch_args(batch), _ptr(table),
                   c_int(table.shape[0] if table is not None else 0), c_int(rot_dims if table is not None else 0),
                   c_int(_PAIRING[pairing]), _ptr(q_norm), _ptr(k_norm), c_int(w_dt), c_float(norm_eps), c_float(k_scale),
                   c_int(n_head), c_int(n_kv), c_int(head_dim), c_int(v_head_dim), c_int(1 if append else 0),
                   c_int((1 if norm_whole else 0) | (2 if norm_bare else 0) | (4 if norm_last else 0) | (8 if q_spread else 0)), c_int(maps),
                   _ptr(batch.status), _stream())

    def retention(self, src, offsets, state, out, batch, n_head, head_dim, v_head_dim, decay, table=None, rot_dims=0,
                  pairing="half", k_scale=1.0):
        T = batch.n_tokens
        W = src.shape[1]
        _need(src, shape=(T, W), name="projection")
        q_off, k_off, v_off = offsets
        if max(q_off + n_head * head_dim, k_off + n_head * head_dim, v_off + n_head * v_head_dim) > W:
            _fail(f"q, k and v at {offsets} do not fit rows of {W}")
        _need(state, torch.float32, (state.shape[0], n_head, head_dim, v_head_dim), "retention state")
        _need(out, torch.float32, (T, n_head, v_head_dim), "retention output")
        _need(decay, torch.float32, (n_head,), "decay")
        if table is not None:
            _need(table, torch.float32, name="rotary table")
            if table.shape[1] * 2 != rot_dims:
                _fail(f"the rotary table serves {table.shape[1] * 2} dimensions, the mixer rotates {rot_dims}")
        # prompts of several chunks run their chunks side by side and need room for one state per chunk
        fn = self._f("retention", "gfb_retention_scratch_floats")
        fn.restype = c_long
        need = fn(c_int(T), c_int(batch.n_seqs), c_int(int(batch.max_q_len)), c_int(n_head), c_int(head_dim), c_int(v_head_dim))
        fn.restype = c_long
        scratch = torch.empty(need, dtype=torch.float32, device=src.device) if need > 0 else None
        self._call("retention", "gfb_retention", _ptr(src), c_int(_dt(src)), c_int(W), c_int(q_off), c_int(k_off), c_int(v_off),
                   _ptr(state), _ptr(out), *self._batch_args(batch), c_int(int(batch.max_q_len)), _ptr(table),
                   c_int(table.shape[0] if table is not None else 0), c_int(rot_dims if table is not None else 0),
                   c_int(_PAIRING[pairing]), _ptr(decay), c_float(k_scale), c_int(n_head), c_int(head_dim), c_int(v_head_dim),
                   _ptr(scratch), c_long(need), _ptr(batch.status), _stream())

    def retention_gate(self, o, src, gate_offset, out, n_head, v_head_dim, eps):
        T, W = src.shape
        _need(o, torch.float32, (T, n_head, v_head_dim), "retention output")
        _need(src, name="projection")
        _need(out, src.dtype, (T, n_head * v_head_dim), "gated output")
        if gate_offset + n_head * v_head_dim > W:
            _fail(f"a gate at column {gate_offset} does not fit rows of {W}")
        self._call("retention", "gfb_retention_gate", _ptr(o), _ptr(src), c_int(_dt(src)), c_int(W), c_int(gate_offset), _ptr(out),
                   c_int(T), c_int(n_head), c_int(v_head_dim), c_float(eps), _stream())

    def sigmoid_gate(self, y, gate, gate_off, group):
        T, C = y.shape
        _need(y, name="gated tensor")
        _need(gate, name="gate")
        if gate.dtype not in (y.dtype, torch.float32):
            _fail(f"a gate of {gate.dtype} on a tensor of {y.dtype}")
        if gate.dim() != 2 or gate.shape[0] != T or group < 1 or C % group or gate_off + C // group > gate.shape[1]:
            _fail(f"gates for groups of {group} of {C} columns at column {gate_off} do not fit {tuple(gate.shape)}")
        self._call("elementwise", "gfb_sigmoid_gate", _ptr(y), _ptr(gate), c_int(_dt(y)), c_int(_dt(gate)), c_int(T), c_int(C), c_int(gate.shape[1]),
                   c_int(gate_off), c_int(group), _stream())

    # -- mixture of experts ------------------------------------------------------------------
    MOE_TILE_ROWS = 64                 # rows of a tile of the sorted form on CUDA cores
    MOE_TC_TILE_ROWS = 128             # ... and on the tensor cores (the rows of one MMA)
    MOE_FEW_TOKENS = 32                # up to this many tokens a warp per output number streams the weight rows (CUDA-core forms)
    MOE_TC_FEW_TOKENS = 0              # ... where the tensor-core tiles run: they stream a chosen expert's weights once per step by TMA
    MOE_PAIR_ROWS_PER_EXPERT = 384     # (token, expert) pairs per expert from which the row tiles have 256 rows
    _EPI_GLU_CLAMP = 8

    _ROUTE_SCORES = {"sigmoid": 0, "softmax_top": 1}

    def moe_route(self, logits, correction, top, scale, idx, weights, score="sigmoid"):
        T = logits.shape[0]
        if score not in self._ROUTE_SCORES:
            _fail(f"unknown router score '{score}'")
        E = correction.shape[0]
        _need(logits, torch.float32, name="router logits")
        if logits.dim() != 2 or logits.shape[1] < E:
            _fail(f"router logits {tuple(logits.shape)} for {E} experts")
        _need(correction, name="router correction")
        _need(idx, torch.int32, (T, top), "chosen experts")
        _need(weights, torch.float32, (T, top), "expert weights")
        self._call("moe", "gfb_moe_route", _ptr(logits), c_int(logits.shape[1]), _ptr(correction), c_int(_dt(correction)), c_int(E),
                   c_int(top), c_float(scale), _ptr(idx), _ptr(weights), c_int(T), c_int(self._ROUTE_SCORES[score]), _stream())

    MOE_ROUTER_FEW_TOKENS = 64         # up to this many tokens the router's product and its choice are one launch

    def moe_router(self, h, router, correction, top, scale, idx, weights, score="sigmoid", extra=None) -> bool:
        T, D = h.shape
        E = correction.shape[0]
        n_extra = 0 if extra is None else extra.shape[1]
        if T > self.MOE_ROUTER_FEW_TOKENS or (D + E + n_extra) * 4 > 48 * 1024:
            return False
        if score not in self._ROUTE_SCORES:
            _fail(f"unknown router score '{score}'")
        if extra is not None:
            _need(extra, torch.float32, (T, n_extra), "logits of the further rows")
        _need(h, name="router input")
        _need(router, h.dtype, (router.shape[0], D), "router weights")
        if router.shape[0] < E + n_extra:
            _fail(f"router weights {tuple(router.shape)} for {E} experts and {n_extra} further rows")
        _need(correction, name="router correction")
        _need(idx, torch.int32, (T, top), "chosen experts")
        _need(weights, torch.float32, (T, top), "expert weights")
        self._call("moe", "gfb_moe_router", _ptr(h), _ptr(router), c_int(_dt(h)), _ptr(correction), c_int(_dt(correction)), c_int(E),
                   c_int(top), c_float(scale), _ptr(idx), _ptr(weights), c_int(T), c_int(D), c_int(self._ROUTE_SCORES[score]),
                   c_int(n_extra), _ptr(extra), _stream())
        return True

    def moe_experts(self, h, idx, weights, w13, w2, x, limit, alpha, shift=1.0):
        T, D = h.shape
        E, F2, _ = w13.shape
        F, top = F2 // 2, idx.shape[1]
        _need(h, name="expert input")
        _need(w13, h.dtype, (E, 2 * F, D), "gate/up weights")
        _need(w2, h.dtype, (E, D, F), "down weights")
        _need(idx, torch.int32, (T, top), "chosen experts")
        _need(weights, torch.float32, (T, top), "expert weights")
        _need(x, torch.float32, (T, D), "residual stream")
        dt = c_int(_dt(h))
        sizes = (c_int(T), c_int(top), c_int(E), c_int(F), c_int(D))
        if h.dtype == torch.bfloat16 and T > self.MOE_TC_FEW_TOKENS and D % 8 == 0 and F % 8 == 0 and E * max(2 * F, D) < 2 ** 31:
            # sorted by expert in tiles of 128 rows, both products on the tensor cores: gather the rows, gate/up with the
            # activation in the epilogue, down into 32-bit rows, then the weighted sum into the stream in pair order
            pairs = T * top
            # from about two full tiles per expert on: tiles of 256 rows for pairs of SMs (tcgen05 cta_group::2)
            # a decode step: an expert has at most T rows, so tiles of at least T rows (the columns of the swapped MMA) read
            # every chosen expert's weights exactly once
            rows = (16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else
                    self.MOE_TC_TILE_ROWS * (2 if pairs >= self.MOE_PAIR_ROWS_PER_EXPERT * E else 1))
            tiles = (pairs + min(E, pairs) * (rows - 1)) // rows
            plan = torch.empty(tiles * rows + pairs + tiles + 1, dtype=torch.int32, device=h.device)
            row_pair, pair_row = plan[:tiles * rows], plan[tiles * rows:tiles * rows + pairs]
            tile_expert, tiles_used = plan[tiles * rows + pairs:-1], plan[-1:]
            self._call("moe", "gfb_moe_plan", _ptr(idx), c_int(pairs), c_int(E), c_int(rows), _ptr(row_pair), _ptr(pair_row),
                       _ptr(tile_expert), c_int(tiles), _ptr(tiles_used), _stream())
            hs = torch.empty(tiles * rows, D, dtype=h.dtype, device=h.device)
            self._call("moe", "gfb_moe_gather_rows", _ptr(h), _ptr(row_pair), _ptr(hs), c_int(tiles * rows), c_int(top), c_int(D), _stream())
            act = torch.empty(tiles * rows, F, dtype=h.dtype, device=h.device)
            self._label = f"moe_glu_tc {2 * F}x{D}"
            self._call("gemm_tc", "gfb_gemm_tc_grouped", _ptr(hs), _ptr(w13), _ptr(act), c_int(_dt(act)), c_int(tiles * rows), c_int(rows), c_int(E),
                       c_int(2 * F), c_int(D), c_int(self._EPI_GLU_CLAMP), _ptr(tile_expert), _ptr(tiles_used), c_float(limit), c_float(alpha),
                       c_float(shift), _ptr(self.status), _stream())
            y = torch.empty(tiles * rows, D, dtype=torch.float32, device=h.device)
            self._label = f"moe_down_tc {D}x{F}"
            self._call("gemm_tc", "gfb_gemm_tc_grouped", _ptr(act), _ptr(w2), _ptr(y), c_int(_dt(y)), c_int(tiles * rows), c_int(rows), c_int(E),
                       c_int(D), c_int(F), c_int(_EPI["store"]), _ptr(tile_expert), _ptr(tiles_used), c_float(0.0), c_float(0.0), c_float(0.0),
                       _ptr(self.status), _stream())
            self._call("moe", "gfb_moe_combine_rows", _ptr(y), _ptr(pair_row), _ptr(weights), _ptr(x), c_int(T), c_int(top), c_int(D),
                       _stream())
            return
        if T <= self.MOE_FEW_TOKENS:
            act = torch.empty(T * top, F, dtype=h.dtype, device=h.device)
            self._call("moe", "gfb_moe_glu", _ptr(h), _ptr(idx), _ptr(w13), _ptr(act), dt, *sizes, c_float(limit), c_float(alpha),
                       c_float(shift), _ptr(None), _ptr(None), c_int(0), _stream())
            self._call("moe", "gfb_moe_down", _ptr(act), _ptr(idx), _ptr(weights), _ptr(w2), _ptr(x), dt, *sizes, _ptr(None), _ptr(None),
                       c_int(0), _ptr(None), _stream())
            return
        # the sorted form: pairs grouped by expert, every expert's rows padded to whole tiles
        rows = self.MOE_TILE_ROWS
        pairs = T * top
        tiles = (pairs + min(E, pairs) * (rows - 1)) // rows
        plan = torch.empty(tiles * rows + pairs + tiles, dtype=torch.int32, device=h.device)
        row_pair, pair_row, tile_expert = plan[:tiles * rows], plan[tiles * rows:tiles * rows + pairs], plan[tiles * rows + pairs:]
        self._call("moe", "gfb_moe_plan", _ptr(idx), c_int(pairs), c_int(E), c_int(rows), _ptr(row_pair), _ptr(pair_row),
                   _ptr(tile_expert), c_int(tiles), _ptr(None), _stream())
        act = torch.empty(tiles * rows, F, dtype=h.dtype, device=h.device)
        y = torch.empty(pairs, D, dtype=torch.float32, device=h.device)
        self._call("moe", "gfb_moe_glu", _ptr(h), _ptr(idx), _ptr(w13), _ptr(act), dt, *sizes, c_float(limit), c_float(alpha),
                   c_float(shift), _ptr(row_pair), _ptr(tile_expert), c_int(tiles), _stream())
        self._call("moe", "gfb_moe_down", _ptr(act), _ptr(idx), _ptr(weights), _ptr(w2), _ptr(x), dt, *sizes, _ptr(row_pair),
                   _ptr(tile_expert), c_int(tiles), _ptr(y), _stream())

    def activation(self, x, kind, out=None):
        if kind not in _UNARY:
            _fail(f"unknown activation '{kind}'")
        out = x if out is None else out
        _need(x, name="activation input")
        _need(out, x.dtype, x.shape, "activation output")
        self._call("elementwise", "gfb_activation", _ptr(x), _ptr(out), c_int(_dt(x)), c_long(x.numel()), c_int(_EPI[kind]), _stream())

    # -- matrix products -----------------------------------------------------------
    def linear(self, a, w, out, mode="store", defer=False):
        M, K = a.shape
        N = w.shape[0]
        _need(a, name="activation")
        _need(w, a.dtype, (N, K), "weight")
        No = N // 2 if mode == "swiglu" else N
        _need(out, shape=(M, No), name="product output")
        if mode == "add" and out.dtype != torch.float32:
            _fail("the residual sum is kept in float32")
        if mode != "add" and out.dtype not in (a.dtype, torch.float32):
            _fail(f"product of {a.dtype} cannot be stored as {out.dtype}")
        self._label = f"linear {N}x{K} {mode}"
        if a.dtype == torch.bfloat16 and self._tc_fits(M, N, K, mode):
            if mode in _UNARY and not (mode in _TC_UNARY and out.dtype == torch.bfloat16):
                # the other activations have no epilogue of their own in the tensor-core kernel
                self._linear_tc(a, w, out, "store")
                return self.activation(out, mode)
            return self._linear_tc(a, w, out, mode, defer=defer and mode in ("store", "add"))
        if a.dtype == torch.float32 and out.dtype != torch.float32:
            _fail("a float32 product is stored as float32")
        self._call("gemm_simt", "gfb_gemm_simt", _ptr(a), _ptr(w), _ptr(out), c_int(_dt(a)), c_int(_dt(out)),
                   c_int(M), c_int(N), c_int(K), c_int(_EPI[mode]), _stream())

    def _tc_fits(self, M, N, K, mode) -> bool:
        """The tensor-core kernel takes rows of whole 16-byte units (TMA) and stores in 16-byte vectors."""
        return K % 8 == 0 and N % (16 if mode == "swiglu" else 8) == 0

    def tc_plan(self, M, N, K, mode="store"):
        """(swap, bn, splits, stages) for the tensor-core product.  Few tokens: the weight rows fill the
        128 MMA rows and the tokens are its columns, split over K until about two blocks per SM stream
        weights; many tokens: 256 x 256 tiles on pairs of SMs (bn = 1024 names that kernel, 512 the
        one-SM persistent kernel, 128/256 one tile per block).  In between (129 to 512 tokens) a product
        that may be split over K stays in the first form, with several column tiles of 128 tokens: one or two
        row tiles of 256 x 256 leave most pairs of SMs idle unless the weight matrix is wide (measured at 256
        tokens: q/k/v 26.8 -> 15.5 us, output projection 29.4 -> 12.8, down projection 78.1 -> 31.8; the
        gate/up product with its SwiGLU cannot be split and is wide enough: 57 us on pairs, 78 us this way; so is
        the output product: 224 us on pairs, 383 us this way, hence the count of 256 x 256 tiles in the rule)."""
        if 128 < M <= 512 and mode != "swiglu" and -(-M // 256) * -(-N // 256) < self.sm_count // 2:
            blocks = -(-N // 128) * -(-M // 128)
            total_kb = -(-K // 64)
            splits = max(1, min(total_kb // 8, (2 * self.sm_count) // blocks))
            return 1, 128, splits, 3
        if M <= 128:
            bn = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
            blocks = -(-N // 128)
            total_kb = -(-K // 64)
            splits = max(1, min(total_kb // 8, (2 * self.sm_count) // blocks))
            stage = 16384 + bn * 128
            stages = max(2, min(8, (100 * 1024) // stage))
            if blocks > 4 * self.sm_count:
                stages = 3          # many rounds of blocks (the output product): four short rings per SM stream better than two long ones
            return 1, bn, splits, stages
        if N >= 256:
            # pairs of SMs on 256 x 256 tiles (bn 1024 = the cta_group::2 kernel), persistent, two
            # accumulators in tensor memory so that a tile's epilogue hides behind the next main loop
            return 0, 1024, 1, 6
        return 0, 128, 1, 6

    @property
    def sm_count(self):
        if self._sm_count is None:
            self._sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        return self._sm_count

    @property
    def status(self):
        """Error words of kernels that take no status of a step (bounded waits that ran out)."""
        if self._status is None:
            self._status = torch.zeros(4, dtype=torch.int32, device="cuda")
        return self._status

    def _linear_tc(self, a, w, out, mode, plan=None, defer=False):
        M, K = a.shape
        N = w.shape[0]
        swap, bn, splits, stages = plan or self.tc_plan(M, N, K, mode)
        ws = torch.empty(splits, M, N, dtype=torch.float32, device=a.device) if splits > 1 else None
        used = c_int(1)
        self._call("gemm_tc", "gfb_gemm_tc", _ptr(a), _ptr(w), _ptr(out), c_int(_dt(out)), c_int(M), c_int(N), c_int(K),
                   c_int(_EPI[mode]), c_int(swap), c_int(bn), c_int(splits), c_int(stages), _ptr(ws),
                   c_int(0 if defer else 1), ctypes.byref(used), _ptr(self.status), _stream())
        if defer and used.value > 1:
            return ws[:used.value]
        return None

    # -- attention ---------------------------------------------------------------------
    def spread_queries(self, dtype, n_head, n_kv, head_dim, v_head_dim, maps, page_size) -> bool:
        """Whether attention with `maps` score maps per head wants its queries spread out: q [T, H * maps, maps * head_dim] with
        query j at columns (j mod maps) * head_dim of its row and zeros elsewhere.  Against the cached row of `maps` keys
        side by side such a query meets its own key only, so every map is an ordinary head of maps * head_dim and the
        tensor-core kernels run as they are."""
        d = maps * head_dim
        return (dtype == torch.bfloat16 and maps > 1 and d == v_head_dim and d in (64, 128) and page_size == 64
                and (n_head * maps) // n_kv <= 8)

    def attention(self, q, kv, batch, out, n_head, n_kv, head_dim, scale, window=None, chunk=None, sink=None, v_head_dim=None,
                  values_in_keys=False, bias=None, slopes=None, softcap=None, keep_first=0, maps=1, diff=None):
        T = batch.n_tokens
        dv = v_head_dim or head_dim
        if maps == 2 and diff is not None and q.dim() == 3 and q.shape[2] == maps * head_dim:
            # spread queries: 2H ordinary heads over the same keys and values, then the difference of each pair of maps
            both = torch.empty(T, n_head * maps * dv, dtype=q.dtype, device=q.device)
            self.attention(q, kv, batch, both, n_head * maps, n_kv, maps * head_dim, scale, window, chunk, sink, dv, values_in_keys,
                           bias, slopes, softcap, keep_first)
            _need(out, q.dtype, (T, n_head * dv), "attention output")
            return self._call("elementwise", "gfb_diff_combine", _ptr(both), _ptr(out), c_int(_dt(out)), c_int(T), c_int(n_head), c_int(dv),
                              c_float(diff[0]), c_float(diff[1]), c_float(diff[2]), _stream())
        if maps not in (1, 2) or (maps == 2) != (diff is not None):
            _fail("two score maps per head come with (lambda, eps, out_scale), one map without")
        if keep_first and not window:
            keep_first = 0                             # without a window every earlier position is visible anyway
        _need(q, shape=(T, n_head * maps, head_dim), name="q")
        _need(out, q.dtype, (T, n_head * dv), "attention output")
        _need(kv.k_pool, q.dtype, name="key pool")
        if sink is not None:
            _need(sink, torch.float32, (n_head,), "sink")
        if bias is not None:
            _need(bias, torch.float32, (bias.shape[0], n_head), "distance bias table")
        if slopes is not None:
            _need(slopes, torch.float32, (n_head,), "distance slopes")
        biased = bias is not None or slopes is not None
        capped = bool(softcap) or bool(keep_first)                    # the tensor-core kernels have these at head sizes 64 and 128
        special = capped or maps != 1
        plain = chunk is None and sink is None and not biased and not special
        if (values_in_keys and not biased and not special and q.dtype == torch.bfloat16 and n_kv == 1 and chunk is None and sink is None
                and not window and head_dim % 16 == 0 and dv % 16 == 0 and dv <= 512 and dv < head_dim and kv.page_size % 32 == 0
                and (64 + 2 * 32) * (head_dim + 8) * 2 <= 220 * 1024):
            # a latent that all heads share: the tensor-core kernel that fetches every cached row once per 64 (token, head)
            # pairs of a sequence (a decode step's heads are the rows of one MMA)
            splits, scratch = 1, None
            if batch.max_q_len == 1:
                # a decode step: slices of at least 128 cached rows, as many as keep about four blocks per SM busy
                splits = max(1, min(16, -(-int(batch.max_kv_len) // 32) // 4))
                while splits > 1 and batch.n_seqs * -(-n_head // 64) * splits > 4 * self.sm_count:
                    splits //= 2
                if splits > 1:
                    scratch = torch.empty(T * n_head * splits * (dv + 2), dtype=torch.float32, device=q.device)
            return self._call("latent", "gfb_latent_attention", _ptr(q), _ptr(out), _ptr(kv.k_pool), _ptr(kv.page_table),
                              c_int(kv.page_table.shape[1]), c_int(kv.page_size), c_int(kv.k_pool.shape[0]), *self._batch_args(batch),
                              c_int(int(batch.max_q_len)), c_int(n_head), c_int(head_dim), c_int(dv), c_float(scale), c_int(splits),
                              _ptr(scratch), _ptr(batch.status), _stream())
        if (not values_in_keys and maps == 1 and dv == head_dim and q.dtype == torch.bfloat16 and kv.page_size == 64 and n_head // n_kv <= 8
                and (head_dim in (64, 128) or (plain and head_dim % 8 == 0 and head_dim <= 256)) and (not (biased or capped) or scale > 0)
                and not (keep_first and (biased or sink is not None))):
            # the tensor-core kernels; a block mask, a sink, a distance bias, a soft cap or kept first positions only at the
            # head sizes they are built for
            return self._attention_bf16(q, kv, batch, out, n_head, n_kv, head_dim, scale, window, chunk=chunk, sink=sink,
                                        bias=bias, slopes=slopes, softcap=softcap, keep_first=keep_first)
        self._call("attention_generic", "gfb_attention_generic", _ptr(q), _ptr(out), c_int(_dt(q)),
                   *self._kv_args(kv), *self._batch_args(batch), c_int(n_head), c_int(n_kv), c_int(head_dim), c_int(dv),
                   c_float(scale), c_int(window or 0), c_int(chunk or 0), _ptr(sink), c_int(1 if values_in_keys else 0),
                   _ptr(bias), c_int(bias.shape[0] if bias is not None else 0), _ptr(slopes), c_float(softcap or 0.0),
                   c_int(int(keep_first)), c_int(maps), c_float(diff[0] if diff else 0.0), c_float(diff[1] if diff else 0.0),
                   c_float(diff[2] if diff else 1.0), _ptr(batch.status), _stream())

    def decode_slices(self, max_kv_len, page_size, blocks) -> int:
        return decode_slices(max_kv_len, page_size, blocks, self.sm_count)

    # entries of a distance array ahead of the table (all the far value) and behind distance 0 (keys behind the query)
    BIAS_FAR_ENTRIES, BIAS_BEHIND_ENTRIES = 128, 384

    def _distance_arrays(self, bias, slopes, scale):
        """A distance bias in the form the tensor-core prefill kernel reads, made once per table and kept: everything divided
        by the score scale (the kernel adds it to the raw score); the table [rows, H] as four copies [4, H, len] of a
        per-head array in which entry `top` - n holds distance n (distances beyond the table the last row's value, entries
        beyond `top` zeros), copy s moved down by s entries so that 16-byte loads from any entry are aligned in one copy."""
        key = (bias.data_ptr() if bias is not None else 0, slopes.data_ptr() if slopes is not None else 0, float(scale))
        hit = self._bias_cache.get(key)
        if hit is not None and hit[0] is bias and hit[1] is slopes:
            return hit[2:]
        arrays, length, top = None, 0, 0
        if bias is not None:
            rows = bias.shape[0]
            top = rows - 1 + self.BIAS_FAR_ENTRIES
            length = -(-(top + 1 + self.BIAS_BEHIND_ENTRIES) // 4) * 4
            n = top - torch.arange(length + 3, device=bias.device)                        # the distance of every entry
            one = (bias / scale)[n.clamp(0, rows - 1)] * (n >= 0).unsqueeze(1)            # [len + 3, H]
            arrays = torch.stack([one[s:s + length].t() for s in range(4)]).contiguous()  # [4, H, len]
        per_head = None if slopes is None else (slopes / scale).contiguous()
        if len(self._bias_cache) > 256:
            self._bias_cache.clear()
        self._bias_cache[key] = (bias, slopes, arrays, length, top, per_head)
        return arrays, length, top, per_head

    def _attention_bf16(self, q, kv, batch, out, n_head, n_kv, head_dim, scale, window, splits=None, prefill=None, tiles=0,
                        max_blocks=0, chunk=None, sink=None, bias=None, slopes=None, softcap=None, keep_first=0):
        T = batch.n_tokens
        capped = bool(softcap) or bool(keep_first)
        if prefill is None:
            prefill = splits is None and batch.max_q_len > 1 and head_dim in (64, 128)
        if prefill and head_dim in (64, 128) and n_head // n_kv <= 8:
            if capped:
                arrays, length, top, per_head = self._distance_arrays(bias, slopes, scale) if (bias is not None or slopes is not None) else (None, 0, 0, None)
                # kept first positions are merged into the rows behind the windowed attention, which leaves each row's log-sum-exp
                lse = torch.empty(T * n_head, dtype=torch.float32, device=q.device) if keep_first else None
                self._call("attention_tc", "gfb_attn_prefill_tc_capped", _ptr(q), _ptr(out), *self._kv_args(kv), *self._batch_args(batch),
                           c_int(n_head), c_int(n_kv), c_int(head_dim), c_float(scale), c_int(window or 0), c_int(chunk or 0),
                           _ptr(sink), _ptr(arrays), c_int(length), c_int(top), _ptr(per_head), c_float(softcap or 0.0),
                           c_int(int(keep_first or 0)), _ptr(lse), c_int(tiles), c_int(max_blocks), _ptr(batch.status), _stream())
                return
            if bias is not None or slopes is not None:
                arrays, length, top, per_head = self._distance_arrays(bias, slopes, scale)
                self._call("attention_tc", "gfb_attn_prefill_tc_biased", _ptr(q), _ptr(out), *self._kv_args(kv), *self._batch_args(batch),
                           c_int(n_head), c_int(n_kv), c_int(head_dim), c_float(scale), c_int(window or 0), c_int(chunk or 0),
                           _ptr(sink), _ptr(arrays), c_int(length), c_int(top), _ptr(per_head), c_int(tiles), c_int(max_blocks),
                           _ptr(batch.status), _stream())
                return
            self._call("attention_tc", "gfb_attn_prefill_tc_masked", _ptr(q), _ptr(out), *self._kv_args(kv), *self._batch_args(batch),
                       c_int(n_head), c_int(n_kv), c_int(head_dim), c_float(scale), c_int(window or 0), c_int(chunk or 0), _ptr(sink),
                       c_int(tiles), c_int(max_blocks), _ptr(batch.status), _stream())
            return
        if splits is None:
            splits = 1
            if batch.max_q_len == 1:
                # a query reads at most its own block of `chunk` positions (and the page that block starts in)
                reach = batch.max_kv_len if not chunk else min(batch.max_kv_len, chunk + kv.page_size)
                if window and capped:
                    reach = min(reach, window + kv.page_size)   # the window's slices; the kept first positions have their own
                splits = self.decode_slices(reach, kv.page_size, T * n_kv)
            if keep_first:
                splits += 1                                 # the kept first positions are a slice of their own, the grid's last
        scratch = None
        if splits > 1:
            scratch = torch.empty(T * n_head * splits * (head_dim + 2), dtype=torch.float32, device=q.device)
        if capped:
            self._call("attention_bf16", "gfb_attn_decode_capped", _ptr(q), _ptr(out), *self._kv_args(kv), *self._batch_args(batch),
                       c_int(n_head), c_int(n_kv), c_int(head_dim), c_float(scale), c_int(window or 0), c_int(chunk or 0), _ptr(sink),
                       _ptr(bias), c_int(bias.shape[0] if bias is not None else 0), _ptr(slopes), c_float(softcap or 0.0),
                       c_int(int(keep_first or 0)), c_int(splits), _ptr(scratch), _ptr(batch.status), _stream())
            return
        if bias is not None or slopes is not None:
            self._call("attention_bf16", "gfb_attn_decode_biased", _ptr(q), _ptr(out), *self._kv_args(kv), *self._batch_args(batch),
                       c_int(n_head), c_int(n_kv), c_int(head_dim), c_float(scale), c_int(window or 0), c_int(chunk or 0), _ptr(sink),
                       _ptr(bias), c_int(bias.shape[0] if bias is not None else 0), _ptr(slopes), c_int(splits), _ptr(scratch),
                       _ptr(batch.status), _stream())
            return
        self._call("attention_bf16", "gfb_attn_decode_masked", _ptr(q), _ptr(out), *self._kv_args(kv), *self._batch_args(batch),
                   c_int(n_head), c_int(n_kv), c_int(head_dim), c_float(scale), c_int(window or 0), c_int(chunk or 0), _ptr(sink),
                   c_int(splits), _ptr(scratch), _ptr(batch.status), _stream())

    def rope_append_attention(self, qkv, partials, kv, batch, table, out, n_head, n_kv, head_dim, pairing, append,
                              scale, window=None, lengths_early=None) -> bool:
        """Rotary encoding, cache append and attention of a decode step in one launch, where the kernel for
        it fits (bfloat16, one token per sequence, head_dim 64 or 128, pages of 64, at most 8 query heads per
        key/value head).  Returns False, having done nothing, where it does not.  lengths_early (tests only):
        what the kernel's read of the lengths ahead of its dependency wait is to see."""
        T = batch.n_tokens
        if not (out.dtype == torch.bfloat16 and batch.max_q_len == 1 and head_dim in (64, 128) and kv.page_size == 64
                and n_head // n_kv <= 8):
            return False
        W = (n_head + 2 * n_kv) * head_dim
        if partials is not None:
            _need(partials, torch.float32, (partials.shape[0], T, W), "partial sums of qkv")
            src, n_part = partials, partials.shape[0]
        else:
            _need(qkv, torch.bfloat16, (T, W), "qkv")
            src, n_part = qkv, 0
        _need(out, torch.bfloat16, (T, n_head * head_dim), "attention output")
        _need(table, torch.float32, name="rotary table")
        _need(kv.k_pool, torch.bfloat16, name="key pool")
        if tuple(kv.k_pool.shape[1:]) != (n_kv, kv.page_size, head_dim):
            _fail(f"key pool pages are {tuple(kv.k_pool.shape[1:])}, the layer needs {(n_kv, kv.page_size, head_dim)}")
        splits = self.decode_slices(batch.max_kv_len, kv.page_size, T * n_kv)
        scratch = None
        if splits > 1:
            scratch = torch.empty(T * n_head * splits * (head_dim + 2), dtype=torch.float32, device=out.device)
        self._call("attention_bf16", "gfb_attn_decode_rope", _ptr(src), c_int(n_part), _ptr(out), *self._kv_args(kv),
                   *self._batch_args(batch), _ptr(table), c_int(table.shape[0]), c_int(n_head), c_int(n_kv), c_int(head_dim),
                   c_int(_PAIRING[pairing]), c_int(1 if append else 0), c_float(scale), c_int(window or 0), c_int(splits),
                   _ptr(scratch), _ptr(batch.status), _ptr(lengths_early), c_int(int(batch.max_kv_len)), _stream())
        return True

    # -- sampling --------------------------------------------------------------------------
    def argmax(self, logits, out):
        B, V = logits.shape
        _need(logits, torch.float32, name="logits")
        _need(out, torch.int32, (B,), "token output")
        self._call("sampling", "gfb_argmax", _ptr(logits), _ptr(out), c_int(B), c_int(V), _stream())

    def sample(self, logits, out, temperature, top_k, seed, request_ids=None, token_index=None, index_map=None,
               noise_out=None, seed_dev=None):
        B, V = logits.shape
        _need(logits, torch.float32, name="logits")
        _need(out, torch.int32, (B,), "token output")
        if request_ids is not None:
            _need(request_ids, torch.int64, (B,), "request ids")
        if token_index is not None:
            _need(token_index, torch.int32, name="token index")
        if index_map is not None:
            _need(index_map, torch.int32, (B,), "index map")
        elif token_index is not None and token_index.shape[0] < B:
            _fail("token index has fewer entries than logits has rows")
        if noise_out is not None:
            _need(noise_out, torch.float32, (B, V), "noise output")
        self._call("sampling", "gfb_sample", _ptr(logits), _ptr(out), c_int(B), c_int(V), c_float(temperature),
                   c_int(int(top_k) if top_k else 0), c_ulonglong(seed & (2 ** 64 - 1)), _ptr(seed_dev), _ptr(request_ids),
                   _ptr(token_index), _ptr(index_map), _ptr(noise_out), _stream())
