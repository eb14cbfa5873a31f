"""The operations a model step is made of, each one a hand-written sm_100a
kernel (sources under `csrc/`).

Parts call the functions of this module; the functions check shapes and
types on the host, pick the kernel that fits (tensor-core kernels for aligned
bfloat16 shapes, the generic kernels otherwise and for 32-bit) and launch it
on the current CUDA stream.  There is no CPU or library fallback: if the
kernel libraries cannot be built or the tensors are not on a CUDA device, the
call raises.  `kernels()` returns the object that implements the operations;
tests may put a stand-in there with `use_kernels` to exercise the host-side
logic without a GPU.
"""
from contextlib import contextmanager
from typing import Optional

import torch

from .types import BatchMeta, PagedKV

STATUS_WORDS = 4
_STATUS_TEXT = {
    1: "token id out of range (token index {a}, id {b})",
    2: "position beyond the cache or the rotary table (token index {a}, position {b})",
    3: "a device-side wait ran out (wait {a}, block {b})",
    4: "page table has no page there (slot {a}, page index {b})",
}

_kernels = None


class KernelError(RuntimeError):
    pass


def kernels():
    global _kernels
    if _kernels is None:
        from .cuda import CudaKernels
        _kernels = CudaKernels()
    return _kernels


def use_kernels(obj):
    """Replace the kernel object (a test seam); returns the previous one."""
    global _kernels
    prev, _kernels = _kernels, obj
    return prev


@contextmanager
def trace():
    """Time every kernel launch made inside the block: yields a list that receives (label, start event,
    stop event) per launch; `trace_times` turns it into milliseconds.  The events sit between the
    launches, so kernels no longer overlap their neighbours: the times say where a step's work is, not
    how long the step takes in a CUDA graph.  Not for use under stream capture."""
    k = kernels()
    prev, k.trace = k.trace, []
    try:
        yield k.trace
    finally:
        k.trace = prev


def trace_times(records):
    """[(label, milliseconds)] of a finished trace, in launch order (synchronises)."""
    torch.cuda.synchronize()
    return [(label, start.elapsed_time(stop)) for label, start, stop in records]


def set_launch_overlap(on: bool) -> None:
    """Whether kernels launched from now on may start while their predecessor in the stream still drains (the default), or
    run strictly one after the other.  A model asks for the second through `ModelSpec.launch_overlap = False`."""
    k = kernels()
    if hasattr(k, "set_launch_overlap"):
        k.set_launch_overlap(on)


def new_status(device) -> torch.Tensor:
    return torch.zeros(STATUS_WORDS, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor) -> None:
    """Read the device-side error words (this synchronises) and raise if a
    kernel reported something; the words are cleared afterwards."""
    own = getattr(_kernels, "_status", None)
    if own is not None and own is not status:
        check_status(own)
    s = status.tolist()
    if s[0] != 0:
        status.zero_()
        text = _STATUS_TEXT.get(s[0], "device error code {c}").format(a=s[1], b=s[2], c=s[0])
        raise KernelError(f"a kernel reported: {text}")


# ---- the operations ---------------------------------------------------------------

def embed(tokens, table, out, status, scale: float = 1.0):
    """out[t] = table[tokens[t]] * scale widened to 32-bit.  tokens int32 [T]; table
    [V, D]; out float32 [T, D]."""
    return kernels().embed(tokens, table, out, status, scale)


def embed_positions(tokens, table, positions, out, batch: BatchMeta, scale: float = 1.0):
    """out[t] = table[tokens[t]] * scale + positions[p_t], p_t the token's place in its sequence.  positions [P, D] of the
    table's type; out float32 [T, D]."""
    return kernels().embed_positions(tokens, table, positions, out, batch, scale)


def embed_hashed(tokens, table, extra, out, batch: BatchMeta, prev, buckets: int, mul_prev: int, mul_cur: int, scale: float = 1.0):
    """out[t] = table[tokens[t]] * scale + extra[(previous token * mul_prev + tokens[t] * mul_cur) mod buckets], with
    extra's row `buckets` for a sequence's first token.  extra [buckets + 1, D]; prev int32 [n_slots] is per-sequence
    state: the token before a step's first one is read from it, and every sequence's last token of the step is
    written to it afterwards."""
    return kernels().embed_hashed(tokens, table, extra, out, batch, prev, buckets, mul_prev, mul_cur, scale)


def softcap(x, cap: float):
    """x (float32, in place) = cap * tanh(x / cap)."""
    return kernels().softcap(x, cap)


def rmsnorm(x, weight, eps: float, out, rows=None, pending=None):
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * weight.  x float32
    [T, D]; weight [D] (bfloat16 or float32); out [R, D]; rows int32 [R] or None.
    pending (float32 [S, T, D], only without rows): partial sums still owed to x;
    the kernel first completes x += sum_s pending[s] (written back), then norms."""
    return kernels().rmsnorm(x, weight, eps, out, rows, pending)


def layernorm(x, weight, bias, eps: float, out, rows=None, branch=None, rms: bool = False):
    """Layer norm with weight and bias (bias None: none), (v - mean) / sqrt(mean((v - mean)^2) + eps) * weight + bias,
    statistics in 32-bit.  x float32 [T, D]; out [R, D] in the compute type, or None; rows int32 [R] or None.
    branch = (y, weight, bias, eps, mult), only without rows: the kernel first completes
    x += mult * norm(y) with that norm's parameters (written back), y being a float32 [T, D] tensor or partial sums
    [S, T, D] of it, and then norms the new x into `out` (if given).  rms=True: the root-mean-square form, no mean
    and no bias, for both norms.  weight=None with an `out`: no norm at all, out = the (new) x in the compute type."""
    return kernels().layernorm(x, weight, bias, eps, out, rows, branch, rms)


def layernorm_multi(x, branches=(), outs=(), rows=None, rms: bool = False):
    """One row, one mean and variance, several norms.  x float32 [T, D].  branches: up to two (y, scale): first
    x += scale * y (written back), y a float32 [T, D] tensor or partial sums [S, T, D] added in ascending order,
    scale a per-column factor [D] or None.  outs: up to two (weight, eps, out): out [R, D] = (x - mean) / sqrt(var +
    eps) * weight in the compute type.  rows int32 [R] gathers input rows (not together with branches).  rms=True:
    the root-mean-square form (no mean)."""
    return kernels().layernorm_multi(x, branches, outs, rows, rms)


def latent_prepare(src, q_off: int, kv_off: int, q_out, kv: PagedKV, batch: BatchMeta, n_head: int, head_dim: int,
                   rot_dim: int, rank: int, norm_weight, eps: float, table, pairing: str = "interleaved", append: bool = True):
    """Latent attention's per-token work.  src [T, W] holds, at column q_off, n_head heads of (head_dim unrotated +
    rot_dim rotated) query numbers and, at kv_off, rank + rot_dim numbers of the down projection.  The first rank of
    those, divided by their root mean square (eps inside the root) and times norm_weight, are the latent; the last
    rot_dim are rotated by the token's position (table float32 [P, rot_dim/2, 2]).  Both go to the token's place in
    the cache as ONE key row of rank + rot_dim numbers (one key head; the value pool is not used).  Every head's
    rotated query part is turned too and written to q_out[t, h, rank:], q_out being [T, n_head, rank + rot_dim]."""
    return kernels().latent_prepare(src, q_off, kv_off, q_out, kv, batch, n_head, head_dim, rot_dim, rank, norm_weight, eps,
                                    table, pairing, append)


def headwise_linear(a, w, out, n_head: int, k: int, n: int, a_off: int = 0, a_stride: Optional[int] = None, out_off: int = 0,
                    out_stride: Optional[int] = None, gate=None, gate_off: int = 0):
    """A product with a weight per head: out[t, h, :] = a[t, h, :] W_h.  a [T, Wa]: head h's k inputs start at column
    a_off + h * a_stride; out [T, Wo]: its n outputs at out_off + h * out_stride; w [n_head, k, n].  gate [T, Wg] (or
    None): the result is multiplied by sigmoid(gate[t, gate_off + h * n + j])."""
    return kernels().headwise_linear(a, w, out, n_head, k, n, a_off, a_stride, out_off, out_stride, gate, gate_off)


def short_conv(src, col_off: int, channels: int, weight, bias, state, state_off: int, out, batch: BatchMeta, act: bool = True,
               in_bias=None):
    """Causal convolution over time per channel, then SiLU (act).  src [T, W]: the channels start at column col_off;
    weight [channels, taps], whose last column meets the current token; bias [channels] or None; out float32 [T,
    channels].  state float32 [n_slots, S]: from column state_off, the (taps - 1) * channels latest inputs of each
    sequence, oldest first (zeros at a sequence's start); read for the tokens at a step's start and advanced.
    in_bias [channels]: added to every input ahead of the taps (a projection's bias; the zeros before a sequence's start
    stay zeros, and the state keeps the sums)."""
    if in_bias is None:
        return kernels().short_conv(src, col_off, channels, weight, bias, state, state_off, out, batch, act)
    return kernels().short_conv(src, col_off, channels, weight, bias, state, state_off, out, batch, act, in_bias=in_bias)


def rglru(u, w_a, w_i, b_a, b_i, lam, decay_scale: float, y_src, y_off: int, y_bias, state, state_off: int, out, batch: BatchMeta):
    """A gated linear recurrence per channel, token after token.  The C channels are `blocks` equal parts; per part b
    r = sigmoid(u_b Wa_b + ba_b), i = sigmoid(u_b Wi_b + bi_b);  a = exp(-decay_scale r softplus(lam));
    S <- a S + sqrt(1 - a^2) i u;  out = S * gelu_tanh(y + y_bias).
    u float32 [T, C]; w_a, w_i [blocks, C / blocks (in), C / blocks (out)]; b_a, b_i, lam, y_bias [C] of one type;
    y = y_src[:, y_off : y_off + C]; state float32 [n_slots, S] holds S (C numbers per sequence) from column state_off;
    out [T, C] in the compute type.  Gates, decay and state are 32-bit."""
    return kernels().rglru(u, w_a, w_i, b_a, b_i, lam, decay_scale, y_src, y_off, y_bias, state, state_off, out, batch)


def ssd_scan(x, b_off: int, c_off: int, dt_src, dt_off: int, dt_bias, a_log, skip, state, state_off: int, out,
             batch: BatchMeta, n_head: int, head_dim: int, n_state: int, n_groups: int):
    """Selective state space, token after token: per head h (group g = h // (n_head / n_groups))
    dt = softplus(dt_raw + dt_bias[h]);  S <- exp(-exp(a_log[h]) dt) S + dt B_g x_h^T;  y = S^T C_g + skip[h] x_h.
    x float32 [T, W]: heads of head_dim at column 0, B groups of n_state at b_off, C at c_off; dt_raw = dt_src[:, dt_off
    + h]; state float32 [n_slots, S] holds [n_head, n_state, head_dim] per sequence from column state_off; out float32
    [T, n_head, head_dim]."""
    return kernels().ssd_scan(x, b_off, c_off, dt_src, dt_off, dt_bias, a_log, skip, state, state_off, out, batch, n_head,
                              head_dim, n_state, n_groups)


def delta_rule(qkv, offsets, beta_src, beta_off: int, a_src, a_off: int, dt_bias, a_log, state, state_off: int, out,
               batch: BatchMeta, n_head: int, n_qk: int, head_dim: int, v_head_dim: int, q_scale: float, unit_eps: float = 1e-6,
               head_decay: bool = False):
    """Gated delta rule, token after token: per head h (query/key head j = h // (n_head / n_qk)), with q and k divided
    by sqrt(sum of squares + unit_eps) (q also times q_scale), beta = sigmoid(beta_src[:, beta_off + h]) and
    g = exp(-exp(a_log[h]) softplus(a_src[:, a_off + h * head_dim + i] + dt_bias[h * head_dim + i])):
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
    qkv float32 [T, W] with q, k, v at the column offsets `offsets`; a_src float32; state float32 [n_slots, S] holds
    [n_head, head_dim, v_head_dim] per sequence from column state_off; out float32 [T, n_head, v_head_dim].
    qkv and a_src are the caller's scratch: the kernels overwrite q and k by their unit vectors and the decay inputs by the
    decays.  head_decay: one decay per head and token, g = exp(-exp(a_log[h]) softplus(a_src[:, a_off + h] + dt_bias[h])),
    dt_bias being [n_head]."""
    if not head_decay:
        return kernels().delta_rule(qkv, offsets, beta_src, beta_off, a_src, a_off, dt_bias, a_log, state, state_off, out, batch,
                                    n_head, n_qk, head_dim, v_head_dim, q_scale, unit_eps)
    return kernels().delta_rule(qkv, offsets, beta_src, beta_off, a_src, a_off, dt_bias, a_log, state, state_off, out, batch,
                                n_head, n_qk, head_dim, v_head_dim, q_scale, unit_eps, head_decay=True)


def gated_norm(y, gate, gate_off: int, weight, out, group: int, eps: float, act: str = "silu", gate_first: bool = False):
    """Root-mean-square norm over groups of `group` columns with a gate: v = y (times act(gate) first if gate_first),
    out = v / sqrt(mean(v^2) + eps) * weight[column mod len(weight)] (times act(gate) here otherwise).  y float32
    [T, C]; gate [T, Wg] from column gate_off; act 'silu' or 'sigmoid'; out [T, C] in the compute type."""
    return kernels().gated_norm(y, gate, gate_off, weight, out, group, eps, act, gate_first)


def qkv_prepare(src, partials, offsets, q_out, kv: PagedKV, batch: BatchMeta, n_head: int, n_kv: int, head_dim: int,
                v_head_dim: int, table=None, rot_dims: int = 0, pairing: str = "half", q_norm=None, k_norm=None,
                norm_eps: float = 0.0, k_scale: float = 1.0, append: bool = True, norm_whole: bool = False,
                norm_bare: bool = False, norm_last: bool = False, maps: int = 1, q_spread: bool = False):
    """From a projection's row to attention's inputs.  src [T, W] holds q (H heads of head_dim), k (G heads of
    head_dim) and v (G heads of v_head_dim) at the column offsets `offsets` = (q, k, v); with `partials` (float32
    [S, T, W]) src is their sum.  Per head, in this order: root-mean-square norm of q and k with the weights
    q_norm / k_norm [head_dim] (None: none), rotation of the first rot_dims dimensions by the token's position from
    `table` (None: none), k times k_scale.  q goes to q_out [T, H, head_dim], k and v to the token's place in the
    cache (unless append is False).  norm_whole: the norm's mean square runs over all heads of q (of k) at once and the
    weights are [H * head_dim] and [G * head_dim].  norm_bare: q and k are divided by their root mean square per head
    without a weight.  norm_last: the per-head norm follows the rotation.  maps > 1: every query head and every key head
    is `maps` vectors of head_dim side by side, each normed and rotated like a head; q_out is [T, H * maps, head_dim]
    and a cached key row holds maps * head_dim numbers.  q_spread (see `spread_queries`): q_out is [T, H * maps,
    maps * head_dim], zeroed by the caller, and query j goes to columns (j mod maps) * head_dim of its row."""
    if q_spread:
        return kernels().qkv_prepare(src, partials, offsets, q_out, kv, batch, n_head, n_kv, head_dim, v_head_dim, table,
                                     rot_dims, pairing, q_norm, k_norm, norm_eps, k_scale, append, norm_whole=norm_whole,
                                     norm_bare=norm_bare, norm_last=norm_last, maps=maps, q_spread=True)
    if norm_bare or norm_last or maps != 1:
        return kernels().qkv_prepare(src, partials, offsets, q_out, kv, batch, n_head, n_kv, head_dim, v_head_dim, table,
                                     rot_dims, pairing, q_norm, k_norm, norm_eps, k_scale, append, norm_whole=norm_whole,
                                     norm_bare=norm_bare, norm_last=norm_last, maps=maps)
    if not norm_whole:
        return kernels().qkv_prepare(src, partials, offsets, q_out, kv, batch, n_head, n_kv, head_dim, v_head_dim, table,
                                     rot_dims, pairing, q_norm, k_norm, norm_eps, k_scale, append)
    return kernels().qkv_prepare(src, partials, offsets, q_out, kv, batch, n_head, n_kv, head_dim, v_head_dim, table,
                                 rot_dims, pairing, q_norm, k_norm, norm_eps, k_scale, append, norm_whole=True)


def spread_queries(dtype, n_head: int, n_kv: int, head_dim: int, v_head_dim: int, maps: int, page_size: int) -> bool:
    """Whether `attention` with `maps` score maps per head wants its queries spread out (`qkv_prepare(q_spread=True)`):
    q [T, H * maps, maps * head_dim] with query j at columns (j mod maps) * head_dim of its row and zeros elsewhere, so that
    against a cached row of `maps` keys side by side it meets its own key only.  The kernels decide: where their fast
    attention takes heads of maps * head_dim, every map runs as an ordinary head."""
    ask = getattr(kernels(), "spread_queries", None)
    return bool(ask and ask(dtype, n_head, n_kv, head_dim, v_head_dim, maps, page_size))


def retention(src, offsets, state, out, batch: BatchMeta, n_head: int, head_dim: int, v_head_dim: int, decay, table=None,
              rot_dims: int = 0, pairing: str = "half", k_scale: float = 1.0):
    """Retention over the tokens of a step: per head S = decay * S + k v^T, o = S^T q, token after token, with q and k
    rotated on their first rot_dims dimensions and k times k_scale.  src [T, W] holds q, k (H heads of head_dim) and v
    (H heads of v_head_dim) at the column offsets `offsets`; state float32 [n_slots, H, head_dim, v_head_dim] is the
    sequences' carried S (read and written at the batch's slots); decay float32 [H]; out float32 [T, H, v_head_dim]."""
    return kernels().retention(src, offsets, state, out, batch, n_head, head_dim, v_head_dim, decay, table, rot_dims, pairing, k_scale)


def retention_gate(o, src, gate_offset: int, out, n_head: int, v_head_dim: int, eps: float):
    """out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * silu(gate[t, h, :]) with the gate at column
    gate_offset of src [T, W]; o float32 [T, H, dv]; out [T, H*dv] in the compute type."""
    return kernels().retention_gate(o, src, gate_offset, out, n_head, v_head_dim, eps)


def sigmoid_gate(y, gate, gate_off: int, group: int):
    """y[t, c] *= sigmoid(gate[t, gate_off + c // group]), in place: one gate per `group` columns of y [T, C]; gate
    [T, Wg] of y's type or float32."""
    return kernels().sigmoid_gate(y, gate, gate_off, group)


def moe_route(logits, correction, top: int, scale: float, idx, weights, score: str = "sigmoid"):
    """Choice of experts.  logits float32 [T, >= E] (the first E columns count, E = len(correction)): s = sigmoid(logits);
    the `top` experts with the largest s + correction (lowest index on ties) go to idx int32 [T, top], and
    weights float32 [T, top] = their s / (sum of the chosen s + 1e-20) * scale.  score 'softmax_top': the `top` largest
    logits (+ correction) are chosen and weights = softmax over the chosen logits * scale."""
    if score == "sigmoid":
        return kernels().moe_route(logits, correction, top, scale, idx, weights)
    return kernels().moe_route(logits, correction, top, scale, idx, weights, score=score)


def moe_router(h, router, correction, top: int, scale: float, idx, weights, score: str = "sigmoid", n_extra: int = 0):
    """Router logits z = h router^T (32-bit) and `moe_route` on them.  h [T, D]; router [>= E + n_extra, D] (rows beyond
    those are padding).  A set of kernels may do both in one launch (`moe_router` returning True); otherwise the
    product and the choice run one after the other.  n_extra: that many rows behind the experts' are further 32-bit
    products of the same input (a gate, say); returns (tensor float32 [T, >= n_extra], first column) where their logits
    are, or None."""
    k = kernels()
    fused = getattr(k, "moe_router", None)
    E = correction.shape[0]
    if fused is not None:
        if score == "sigmoid" and n_extra == 0:
            if fused(h, router, correction, top, scale, idx, weights):
                return None
        else:
            extra = torch.empty(h.shape[0], n_extra, dtype=torch.float32, device=h.device) if n_extra else None
            if fused(h, router, correction, top, scale, idx, weights, score=score, extra=extra):
                return None if extra is None else (extra, 0)
    z = torch.empty(h.shape[0], router.shape[0], dtype=torch.float32, device=h.device)
    linear(h, router, z)
    moe_route(z, correction, top, scale, idx, weights, score)
    return (z, E) if n_extra else None


def moe_experts(h, idx, weights, w13, w2, x, limit: float, alpha: float, shift: float = 1.0):
    """x float32 [T, D] += sum_r weights[t, r] * W2_e (g * sigmoid(alpha g) * (u + shift)), e = idx[t, r],
    g = min(gate_e h, limit), u = clamp(up_e h, -limit, limit) (limit <= 0: no clamps).  w13 [E, 2F, D]: rows alternate
    gate, up; w2 [E, D, F]; h [T, D] of the weights' type."""
    return kernels().moe_experts(h, idx, weights, w13, w2, x, limit, alpha, shift)


def activation(x, kind: str, out=None):
    """out (default: in place) = f(x) with f 'gelu' (exact, erf), 'gelu_tanh', 'silu' or 'relu2' (max(x, 0)^2)."""
    return kernels().activation(x, kind, out)


def linear(a, w, out, mode: str = "store", defer: bool = False):
    """a [M, K] times w [N, K] transposed.  mode 'store': out [M, N] = product;
    'add': out float32 [M, N] += product (the residual sum, in 32-bit);
    'swiglu': w's rows alternate gate, up and out [M, N/2] = silu(gate) * up;
    'gelu' (exact, erf), 'gelu_tanh', 'silu', 'relu2': out [M, N] = f(product).

    defer=True (modes 'store' and 'add'): if the kernel splits the sum over K it
    may return the partial sums (float32 [S, M, N]) INSTEAD of finishing `out`;
    the caller hands them to the kernel that consumes the result (`rmsnorm`'s
    `pending`, `rope_append`'s `partials`, or `add_partials`).  Returns None when
    `out` is complete."""
    return kernels().linear(a, w, out, mode, defer)


def add_partials(x, pending):
    """x (float32 [T, D]) += sum_s pending[s] in ascending s."""
    return kernels().add_partials(x, pending)


def rope_table(inv_freq, table, amplitude: float = 1.0):
    """table[p, i] = amplitude * (cos, sin)(p * inv_freq[i]) in 32-bit.  table float32 [P, d/2, 2]."""
    if amplitude == 1.0:
        return kernels().rope_table(inv_freq, table)
    return kernels().rope_table(inv_freq, table, amplitude)


def rope_append(qkv, q_out, kv: PagedKV, batch: BatchMeta, table, n_head: int, n_kv: int, head_dim: int,
                pairing: str = "interleaved", append: bool = True, partials=None):
    """Rotate the q and k heads of qkv [T, (H+2G)d] by each token's position;
    q goes to q_out [T, H, d]; k and v go to the token's place in the cache
    (unless append is False).  With partials (float32 [S, T, (H+2G)d], the
    deferred result of `linear`) qkv is their sum and the `qkv` argument is not read."""
    return kernels().rope_append(qkv, q_out, kv, batch, table, n_head, n_kv, head_dim, pairing, append, partials)


def attention(q, kv: PagedKV, batch: BatchMeta, out, n_head: int, n_kv: int, head_dim: int, scale: float,
              window: Optional[int] = None, chunk: Optional[int] = None, sink=None, v_head_dim: Optional[int] = None,
              values_in_keys: bool = False, bias=None, slopes=None, softcap: Optional[float] = None, keep_first: int = 0,
              maps: int = 1, diff=None):
    """Causal grouped-query attention of q [T, H, d] over the cache (which
    already holds this step's keys and values); out [T, H*dv].  chunk: a query sees only the keys of its own block
    of `chunk` positions (counted from the sequence's first position).  sink (float32 [H]): exp(sink_h) joins the
    softmax denominator of head h, with no value.  v_head_dim: the values' head size if it differs from d.
    values_in_keys: a key's first v_head_dim numbers are also its value (the value pool is not read).
    bias (float32 [L, H]): bias[min(n, L - 1), h] is added to the scaled score of a key n positions back.
    slopes (float32 [H]): slopes[h] * n is taken off it.
    softcap: the scaled score s becomes softcap * tanh(s / softcap).  keep_first (with a window): the sequence's first
    keep_first positions stay visible beyond the window.  maps = 2 with diff = (lambda, eps, out_scale): q is [T, H * 2, d],
    a cached key row holds two keys; each (query, key) pair is a softmax of its own over the same values, and the head's
    output is (o_1 - lambda o_2) / sqrt(mean((o_1 - lambda o_2)^2) + eps) * out_scale.  q may come spread out
    ([T, H * 2, 2 d], see `spread_queries`)."""
    if softcap or keep_first or maps != 1:
        return kernels().attention(q, kv, batch, out, n_head, n_kv, head_dim, scale, window, chunk, sink, v_head_dim or head_dim,
                                   values_in_keys=values_in_keys, bias=bias, slopes=slopes, softcap=softcap, keep_first=keep_first,
                                   maps=maps, diff=diff)
    if bias is not None or slopes is not None:
        return kernels().attention(q, kv, batch, out, n_head, n_kv, head_dim, scale, window, chunk, sink, v_head_dim or head_dim,
                                   values_in_keys=values_in_keys, bias=bias, slopes=slopes)
    if values_in_keys:
        return kernels().attention(q, kv, batch, out, n_head, n_kv, head_dim, scale, window, chunk, sink, v_head_dim or head_dim,
                                   values_in_keys=True)
    if chunk is None and sink is None and v_head_dim in (None, head_dim):
        return kernels().attention(q, kv, batch, out, n_head, n_kv, head_dim, scale, window)
    return kernels().attention(q, kv, batch, out, n_head, n_kv, head_dim, scale, window, chunk, sink, v_head_dim or head_dim)


def rope_append_attention(qkv, partials, kv: PagedKV, batch: BatchMeta, table, out, n_head: int, n_kv: int, head_dim: int,
                          pairing: str, append: bool, scale: float, window: Optional[int] = None):
    """`rope_append` followed by `attention`: qkv [T, (H+2G)d] (or its deferred partial sums) -> out [T, H*d].
    Where a kernel does both in one launch (a decode step in bfloat16) that kernel runs; q then never goes
    through memory."""
    k = kernels()
    fused = getattr(k, "rope_append_attention", None)
    if fused is not None and fused(qkv, partials, kv, batch, table, out, n_head, n_kv, head_dim, pairing, append, scale, window):
        return
    q = torch.empty(batch.n_tokens, n_head, head_dim, dtype=out.dtype, device=out.device)
    k.rope_append(qkv, q, kv, batch, table, n_head, n_kv, head_dim, pairing, append, partials)
    k.attention(q, kv, batch, out, n_head, n_kv, head_dim, scale, window)


def advance_lengths(batch: BatchMeta):
    """lengths[slot] += number of new tokens, for every sequence of the batch."""
    return kernels().advance_lengths(batch)


def add_into(out, y):
    """out (float32) += y."""
    return kernels().add_into(out, y)


def argmax(logits, out):
    """out[b] = index of the largest logits[b, :], lowest index on ties."""
    return kernels().argmax(logits, out)


def sample(logits, out, temperature: float, top_k: Optional[int], seed: int, request_ids=None, token_index=None,
           index_map=None, noise_out=None, seed_dev=None):
    """Temperature / top-k / exponential-race draw per row of float32 logits.
    The noise of row b is keyed by (seed, request_ids[b], token_index[index_map[b]
    or b], vocabulary index), so it does not depend on the row's place in the batch.
    seed_dev (int64 [1] on the device) overrides `seed`: a captured graph can then be replayed with another seed."""
    return kernels().sample(logits, out, temperature, top_k, seed, request_ids, token_index, index_map, noise_out, seed_dev)
