"""Plain PyTorch/NumPy statement of every operation in `gpt_fast_b200.ops`.

Two uses.  (1) Each kernel's reference: the GPU tests call a kernel and the
function of the same name here on the same inputs and compare.  (2) A
stand-in for the kernels (`ops.use_kernels(PlainOps())`), so that the host-side
logic of the library (cache, step function, generation loop, replay) can be
exercised on a machine without a GPU.  It is test code: the library itself has
no CPU path.

Accumulations are done in float64, so that the reference is tighter than the
32-bit kernels it judges.
"""
import math

import numpy as np
import torch


def token_positions(batch):
    """Absolute position of every packed token, as the kernels derive it."""
    seq = batch.tok_seq.long()
    slots = batch.slots.long()[seq]
    start = batch.lengths.long()[slots]
    t = torch.arange(batch.n_tokens, device=seq.device)
    return start + (t - batch.cu_seqlens.long()[seq]), slots


# ---- Philox4x32-10, as in csrc/sampling.cu ---------------------------------------
_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint64) & _MASK for c in (c0, c1, c2, c3))
    k0, k1 = int(k0) & 0xFFFFFFFF, int(k1) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = _M0 * c0, _M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK
        hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK
        c0, c1, c2, c3 = hi1 ^ c1 ^ np.uint64(k0), lo1, hi0 ^ c3 ^ np.uint64(k1), lo0
        k0, k1 = (k0 + _W0) & 0xFFFFFFFF, (k1 + _W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def race_noise(seed, request, token_index, V):
    """Exp(1) noise of one row: -log(u), u = ((r >> 9) + 0.5) / 2^23, float32."""
    i = np.arange(V, dtype=np.uint64)
    req = int(request) & (2 ** 64 - 1)
    seed = int(seed) & (2 ** 64 - 1)
    r0, _, _, _ = philox4x32_10(i, np.uint64(int(token_index) & 0xFFFFFFFF), np.uint64(req & 0xFFFFFFFF),
                                np.uint64(req >> 32), seed & 0xFFFFFFFF, seed >> 32)
    u = ((r0 >> np.uint64(9)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)
    return -np.log(u, dtype=np.float32)


class PlainOps:
    # -- element-wise / per-row ---------------------------------------------------
    def softcap(self, x, cap):
        x.copy_((cap * torch.tanh(x.double() / cap)).float())

    def embed(self, tokens, table, out, status, scale=1.0):
        ids = tokens.long()
        bad = (ids < 0) | (ids >= table.shape[0])
        if bad.any():
            t = int(bad.nonzero()[0])
            if status[0] == 0:
                status[0], status[1], status[2] = 1, t, int(ids[t])
        out.copy_(table[ids.clamp(0, table.shape[0] - 1)].float() * scale)
        out[bad] = 0

    def embed_positions(self, tokens, table, positions, out, batch, scale=1.0):
        pos, _ = token_positions(batch)
        if int(pos.max()) >= positions.shape[0]:
            raise IndexError("position beyond the position table")
        out.copy_((table[tokens.long()].double() * scale + positions[pos].double()).float())

    def sigmoid_gate(self, y, gate, gate_off, group):
        C = y.shape[1]
        g = torch.sigmoid(gate[:, gate_off:gate_off + C // group].double()).repeat_interleave(group, dim=1)
        y.copy_((y.double() * g).to(y.dtype))

    # -- mixture of experts ---------------------------------------------------------------------
    def moe_route(self, logits, correction, top, scale, idx, weights, score="sigmoid"):
        E = correction.shape[0]
        s = torch.sigmoid(logits[:, :E].float()) if score == "sigmoid" else logits[:, :E].float()
        choice = s + correction.float()
        for t in range(s.shape[0]):
            order = sorted(range(E), key=lambda e: (-float(choice[t, e]), e))[:top]
            picked = s[t, order]
            idx[t] = torch.tensor(order, dtype=idx.dtype)
            if score == "sigmoid":
                weights[t] = picked / (picked.sum() + 1e-20) * scale
            else:
                weights[t] = torch.softmax(picked.double(), -1).float() * scale

    def moe_experts(self, h, idx, weights, w13, w2, x, limit, alpha, shift=1.0):
        hd = h.double()
        for t in range(h.shape[0]):
            acc = torch.zeros(x.shape[1], dtype=torch.float64)
            for r in range(idx.shape[1]):
                e = int(idx[t, r])
                z = w13[e].double() @ hd[t]
                g, u = z[0::2], z[1::2]
                if limit > 0:
                    g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
                a = (g * torch.sigmoid(alpha * g) * (u + shift)).to(h.dtype).double()
                acc += float(weights[t, r]) * (w2[e].double() @ a)
            x[t] = (x[t].double() + acc).float()

    def rmsnorm(self, x, weight, eps, out, rows=None, pending=None):
        if pending is not None:
            self.add_partials(x, pending)
        xr = (x if rows is None else x[rows.long()]).double()
        n = xr * torch.rsqrt((xr * xr).mean(-1, keepdim=True) + eps)
        out.copy_((n * weight.double()).to(out.dtype))

    def layernorm(self, x, weight, bias, eps, out, rows=None, branch=None, rms=False):
        def norm(v, w, b, e):
            v = v.double()
            if w is None:
                return v
            if rms:
                return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + e) * w.double()
            dev = v - v.mean(-1, keepdim=True)
            return dev * torch.rsqrt((dev * dev).mean(-1, keepdim=True) + e) * w.double() + (0 if b is None else b.double())
        if branch is not None:
            y, pw, pb, peps, mult = branch
            if y.dim() == 3:
                y = y.double().sum(0)
            x.copy_((x.double() + mult * norm(y, pw, pb, peps)).float())
        if out is not None:
            xr = x if rows is None else x[rows.long()]
            out.copy_(norm(xr, weight, bias, eps).to(out.dtype))

    # -- a hashed bigram embedding, one row with several norms ------------------------------
    def embed_hashed(self, tokens, table, extra, out, batch, prev, buckets, mul_prev, mul_cur, scale=1.0):
        ids = tokens.long()
        pos, slots = token_positions(batch)
        seq = batch.tok_seq.long()
        first_of_step = torch.arange(batch.n_tokens) == batch.cu_seqlens.long()[seq]
        before = torch.where(first_of_step, prev.long()[slots], torch.roll(ids, 1))
        rows = torch.where(pos == 0, torch.tensor(buckets), (before * mul_prev + ids * mul_cur) % buckets)
        out.copy_((table[ids].double() * scale + extra[rows].double()).float())
        last = batch.cu_seqlens.long()[1:] - 1
        prev[batch.slots.long()] = tokens[last]

    def layernorm_multi(self, x, branches=(), outs=(), rows=None, rms=False):
        for y, scale in branches:
            y = y.double().sum(0) if y.dim() == 3 else y.double()
            x.copy_((x.double() + (y if scale is None else y * scale.double())).float())
        for w, eps, out in outs:
            v = (x if rows is None else x[rows.long()]).double()
            dev = v if rms else v - v.mean(-1, keepdim=True)
            out.copy_((dev * torch.rsqrt((dev * dev).mean(-1, keepdim=True) + eps) * w.double()).to(out.dtype))

    # -- latent attention ---------------------------------------------------------------------
    def latent_prepare(self, src, q_off, kv_off, q_out, kv, batch, n_head, head_dim, rot_dim, rank, norm_weight, eps, table,
                       pairing="interleaved", append=True):
        T, H, d, r = batch.n_tokens, n_head, head_dim, rot_dim
        x = src.double()
        pos, slots = token_positions(batch)
        cs = table[pos].double()
        q = x[:, q_off:q_off + H * (d + r)].reshape(T, H, d + r)[..., d:]
        q_out[..., rank:] = self._rotate_front(q, cs, r, pairing).to(q_out.dtype)
        if append:
            lat = x[:, kv_off:kv_off + rank]
            c = lat * torch.rsqrt((lat * lat).mean(-1, keepdim=True) + eps) * norm_weight.double()
            kr = self._rotate_front(x[:, kv_off + rank:kv_off + rank + r].reshape(T, 1, r), cs, r, pairing)[:, 0]
            page = kv.page_table.long()[slots, pos // kv.page_size]
            if int(page.min()) < 0:
                raise IndexError("token lands on a page the slot does not hold")
            kv.k_pool[page, 0, pos % kv.page_size] = torch.cat([c, kr], -1).to(kv.k_pool.dtype)

    def headwise_linear(self, a, w, out, n_head, k, n, a_off=0, a_stride=None, out_off=0, out_stride=None, gate=None, gate_off=0):
        a_stride = k if a_stride is None else a_stride
        out_stride = n if out_stride is None else out_stride
        for h in range(n_head):
            x = a[:, a_off + h * a_stride:a_off + h * a_stride + k].double()
            y = x @ w[h].double()
            if gate is not None:
                y = y * torch.sigmoid(gate[:, gate_off + h * n:gate_off + (h + 1) * n].double())
            out[:, out_off + h * out_stride:out_off + h * out_stride + n] = y.to(out.dtype)

    # -- recurrent mixers -----------------------------------------------------------------------
    def short_conv(self, src, col_off, channels, weight, bias, state, state_off, out, batch, act=True, in_bias=None):
        taps, C = weight.shape[1], channels
        w = weight.double()
        x = src[:, col_off:col_off + C].double()
        if in_bias is not None:
            x = x + in_bias.double()
        cu = batch.cu_seqlens.tolist()
        for s in range(batch.n_seqs):
            slot = int(batch.slots[s])
            old = state[slot, state_off:state_off + (taps - 1) * C].double().view(taps - 1, C) if taps > 1 else x.new_zeros(0, C)
            seq = torch.cat([old, x[cu[s]:cu[s + 1]]])
            n = cu[s + 1] - cu[s]
            y = torch.zeros(n, C, dtype=torch.float64)
            for j in range(taps):
                y += seq[j:j + n] * w[:, j]
            if bias is not None:
                y += bias.double()
            out[cu[s]:cu[s + 1]] = (y / (1 + torch.exp(-y)) if act else y).float()
            if taps > 1:                                           # one tap carries nothing
                state[slot, state_off:state_off + (taps - 1) * C] = seq[n:].reshape(-1).float()

    def rglru(self, u, w_a, w_i, b_a, b_i, lam, decay_scale, y_src, y_off, y_bias, state, state_off, out, batch):
        T, C = u.shape
        blocks, bw = w_a.shape[0], w_a.shape[1]
        ub = u.double().view(T, blocks, bw)
        r = torch.sigmoid(torch.einsum("tbi,bio->tbo", ub, w_a.double()).reshape(T, C) + b_a.double())
        g = torch.sigmoid(torch.einsum("tbi,bio->tbo", ub, w_i.double()).reshape(T, C) + b_i.double())
        log_a = -decay_scale * r * torch.nn.functional.softplus(lam.double())
        a, b = torch.exp(log_a), torch.sqrt(-torch.expm1(2 * log_a)) * g * u.double()
        z = y_src[:, y_off:y_off + C].double() + y_bias.double()
        gate = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
        cu = batch.cu_seqlens.tolist()
        for s in range(batch.n_seqs):
            slot = int(batch.slots[s])
            S = state[slot, state_off:state_off + C].double()
            for t in range(cu[s], cu[s + 1]):
                S = a[t] * S + b[t]
                out[t] = (S * gate[t]).to(out.dtype)
            state[slot, state_off:state_off + C] = S.float()

    def ssd_scan(self, x, b_off, c_off, dt_src, dt_off, dt_bias, a_log, skip, state, state_off, out, batch, n_head, head_dim,
                 n_state, n_groups):
        H, P, N, G = n_head, head_dim, n_state, n_groups
        T = batch.n_tokens
        xd = x.double()
        X = xd[:, :H * P].reshape(T, H, P)
        B = xd[:, b_off:b_off + G * N].reshape(T, G, N).repeat_interleave(H // G, dim=1)
        C = xd[:, c_off:c_off + G * N].reshape(T, G, N).repeat_interleave(H // G, dim=1)
        dt = torch.nn.functional.softplus(dt_src[:, dt_off:dt_off + H].double() + dt_bias.double())
        decay = torch.exp(-torch.exp(a_log.double()) * dt)
        _, slots = token_positions(batch)
        for t in range(T):
            slot = int(slots[t])
            S = state[slot, state_off:state_off + H * N * P].double().view(H, N, P)
            S = decay[t][:, None, None] * S + (dt[t][:, None] * B[t])[:, :, None] * X[t][:, None, :]
            state[slot, state_off:state_off + H * N * P] = S.reshape(-1).float()
            y = torch.einsum("hnp,hn->hp", S, C[t])
            if skip is not None:
                y = y + skip.double()[:, None] * X[t]
            out[t] = y.float()

    def delta_rule(self, qkv, offsets, beta_src, beta_off, a_src, a_off, dt_bias, a_log, state, state_off, out, batch, n_head,
                   n_qk, head_dim, v_head_dim, q_scale, unit_eps=1e-6, head_decay=False):
        H, J, d, dv = n_head, n_qk, head_dim, v_head_dim
        T = batch.n_tokens
        x = qkv.double()
        qo, ko, vo = offsets
        q = x[:, qo:qo + J * d].reshape(T, J, d)
        k = x[:, ko:ko + J * d].reshape(T, J, d)
        v = x[:, vo:vo + H * dv].reshape(T, H, dv)
        q = (q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) * q_scale).repeat_interleave(H // J, dim=1)
        k = (k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)).repeat_interleave(H // J, dim=1)
        beta = torch.sigmoid(beta_src[:, beta_off:beta_off + H].double())
        if head_decay:
            a = (a_src[:, a_off:a_off + H].double() + dt_bias.double())[:, :, None].expand(T, H, d)
        else:
            a = (a_src[:, a_off:a_off + H * d].double() + dt_bias.double()).view(T, H, d)
        g = torch.exp(-torch.exp(a_log.double())[None, :, None] * torch.nn.functional.softplus(a))
        _, slots = token_positions(batch)
        for t in range(T):
            slot = int(slots[t])
            S = g[t][:, :, None] * state[slot, state_off:state_off + H * d * dv].double().view(H, d, dv)
            u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
            S = S + k[t][:, :, None] * u[:, None, :]
            state[slot, state_off:state_off + H * d * dv] = S.reshape(-1).float()
            out[t] = torch.einsum("hdv,hd->hv", S, q[t]).float()

    def gated_norm(self, y, gate, gate_off, weight, out, group, eps, act="silu", gate_first=False):
        T, C = y.shape
        z = gate[:, gate_off:gate_off + C].double()
        a = torch.sigmoid(z) if act == "sigmoid" else z * torch.sigmoid(z)
        v = y.double() * a if gate_first else y.double()
        v = v.view(T, C // group, group)
        v = (v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)).view(T, C) * weight.double().repeat(C // weight.shape[0])
        out.copy_((v if gate_first else v * a).to(out.dtype))

    @staticmethod
    def _rotate_front(v, cs, rot_dims, pairing):
        """v [T, heads, d] (float64), cs [T, rot_dims/2, 2]: rotate the leading rot_dims dimensions."""
        half = rot_dims // 2
        c, s = cs[:, None, :, 0], cs[:, None, :, 1]
        out = v.clone()
        if pairing == "interleaved":
            a, b = v[..., 0:rot_dims:2], v[..., 1:rot_dims:2]
            out[..., 0:rot_dims:2], out[..., 1:rot_dims:2] = a * c - b * s, b * c + a * s
        else:
            a, b = v[..., :half], v[..., half:rot_dims]
            out[..., :half], out[..., half:rot_dims] = a * c - b * s, b * c + a * s
        return out

    def qkv_prepare(self, src, partials, offsets, q_out, kv, batch, n_head, n_kv, head_dim, v_head_dim, table=None, rot_dims=0,
                    pairing="half", q_norm=None, k_norm=None, norm_eps=0.0, k_scale=1.0, append=True, norm_whole=False,
                    norm_bare=False, norm_last=False, maps=1):
        H, G, d, dv = n_head * maps, n_kv * maps, head_dim, v_head_dim
        T = batch.n_tokens
        x = (partials.double().sum(0) if partials is not None else src.double())
        qo, ko, vo = offsets
        q = x[:, qo:qo + H * d].reshape(T, H, d)
        if append:
            k = x[:, ko:ko + G * d].reshape(T, G, d)
            v = x[:, vo:vo + n_kv * dv].reshape(T, n_kv, dv)
        else:                                                  # only q is made: the row may hold no keys or values at all
            k, k_norm = x.new_zeros(T, G, d), None
        pos, slots = token_positions(batch)
        if norm_whole:
            if q_norm is not None:
                q = q * torch.rsqrt((q * q).mean((-2, -1), keepdim=True) + norm_eps) * q_norm.double().view(H, d)
            if k_norm is not None:
                k = k * torch.rsqrt((k * k).mean((-2, -1), keepdim=True) + norm_eps) * k_norm.double().view(G, d)
            q_norm = k_norm = None

        def head_norm(v, w):
            if w is None and not norm_bare:
                return v
            v = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + norm_eps)
            return v if w is None else v * w.double()
        if not norm_last and not norm_whole:
            q, k = head_norm(q, q_norm), head_norm(k, k_norm) if append else k
        if table is not None:
            cs = table[pos].double()
            q, k = self._rotate_front(q, cs, rot_dims, pairing), self._rotate_front(k, cs, rot_dims, pairing)
        if norm_last and not norm_whole:
            q, k = head_norm(q, q_norm), head_norm(k, k_norm) if append else k
        q_out.copy_(q.to(q_out.dtype))
        if append:
            page = kv.page_table.long()[slots, pos // kv.page_size]
            if int(page.min()) < 0:
                raise IndexError("token lands on a page the slot does not hold")
            off = pos % kv.page_size
            kv.k_pool[page, :, off] = (k * k_scale).reshape(T, n_kv, maps * d).to(kv.k_pool.dtype)
            kv.v_pool[page, :, off] = v.to(kv.v_pool.dtype)

    def retention(self, src, offsets, state, out, batch, n_head, head_dim, v_head_dim, decay, table=None, rot_dims=0,
                  pairing="half", k_scale=1.0):
        H, d, dv = n_head, head_dim, v_head_dim
        T = batch.n_tokens
        x = src.double()
        qo, ko, vo = offsets
        q = x[:, qo:qo + H * d].reshape(T, H, d)
        k = x[:, ko:ko + H * d].reshape(T, H, d)
        v = x[:, vo:vo + H * dv].reshape(T, H, dv)
        pos, slots = token_positions(batch)
        if table is not None:
            cs = table[pos].double()
            q, k = self._rotate_front(q, cs, rot_dims, pairing), self._rotate_front(k, cs, rot_dims, pairing)
        k = k * k_scale
        dec = decay.double()[:, None, None]
        for t in range(T):                                    # packed tokens of one sequence are in order
            slot = int(slots[t])
            S = dec * state[slot].double() + k[t][:, :, None] * v[t][:, None, :]
            state[slot] = S.float()
            out[t] = torch.einsum("hdv,hd->hv", S, q[t]).float()

    def retention_gate(self, o, src, gate_offset, out, n_head, v_head_dim, eps):
        T = o.shape[0]
        g = src[:, gate_offset:gate_offset + n_head * v_head_dim].double().reshape(T, n_head, v_head_dim)
        od = o.double()
        n = od * torch.rsqrt((od * od).mean(-1, keepdim=True) + eps)
        out.copy_((n * (g / (1 + torch.exp(-g)))).reshape(T, -1).to(out.dtype))

    @staticmethod
    def _unary(z, kind):
        if kind == "gelu":
            return 0.5 * z * (1 + torch.erf(z / math.sqrt(2.0)))
        if kind == "gelu_tanh":
            return 0.5 * z * (1 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))
        if kind == "silu":
            return z / (1 + torch.exp(-z))
        if kind == "relu2":
            return torch.clamp(z, min=0) ** 2
        raise ValueError(kind)

    def activation(self, x, kind, out=None):
        (x if out is None else out).copy_(self._unary(x.double(), kind).to(x.dtype))

    def rope_table(self, inv_freq, table, amplitude=1.0):
        ang = torch.arange(table.shape[0], dtype=torch.float32, device=table.device)[:, None] * inv_freq[None, :]
        table[..., 0] = (torch.cos(ang.double()) * amplitude).float()
        table[..., 1] = (torch.sin(ang.double()) * amplitude).float()

    def add_partials(self, x, pending):
        x.copy_((x.double() + pending.double().sum(0)).float())

    def rope_append(self, qkv, q_out, kv, batch, table, n_head, n_kv, head_dim, pairing="interleaved", append=True,
                    partials=None):
        H, G, d = n_head, n_kv, head_dim
        T = batch.n_tokens
        if partials is not None:
            qkv = partials.double().sum(0)
        pos, slots = token_positions(batch)
        if int(pos.max()) >= table.shape[0]:
            raise IndexError("position beyond the rotary table")
        cs = table[pos].double()                        # [T, d/2, 2]
        x = qkv.double().view(T, H + 2 * G, d)

        def rotate(v):                                  # v [T, heads, d]
            if pairing == "interleaved":
                a, b = v[..., 0::2], v[..., 1::2]
            else:
                a, b = v[..., : d // 2], v[..., d // 2:]
            c, s = cs[:, None, :, 0], cs[:, None, :, 1]
            oa, ob = a * c - b * s, b * c + a * s
            if pairing == "interleaved":
                return torch.stack([oa, ob], -1).flatten(-2)
            return torch.cat([oa, ob], -1)

        q_out.copy_(rotate(x[:, :H]).to(q_out.dtype))
        if append:
            k = rotate(x[:, H:H + G]).to(kv.k_pool.dtype)
            v = x[:, H + G:].to(kv.v_pool.dtype)
            page = kv.page_table.long()[slots, pos // kv.page_size]
            if int(page.min()) < 0:
                raise IndexError("token lands on a page the slot does not hold")
            off = pos % kv.page_size
            kv.k_pool[page, :, off] = k
            kv.v_pool[page, :, off] = v

    def advance_lengths(self, batch):
        q = (batch.cu_seqlens[1:] - batch.cu_seqlens[:-1]).to(batch.lengths.dtype)
        batch.lengths[batch.slots.long()] += q

    def add_into(self, out, y):
        out += y.float()

    # -- matrix products ---------------------------------------------------------------
    def linear(self, a, w, out, mode="store", defer=False):
        acc = a.double() @ w.double().T
        if mode == "store":
            out.copy_(acc.to(out.dtype))
        elif mode == "add":
            out.copy_((out.double() + acc).to(out.dtype))
        elif mode == "swiglu":
            g, u = acc[:, 0::2], acc[:, 1::2]
            out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))
        elif mode in ("gelu", "gelu_tanh", "silu", "relu2"):
            out.copy_(self._unary(acc, mode).to(out.dtype))
        else:
            raise ValueError(mode)

    # -- attention -----------------------------------------------------------------------
    def attention(self, q, kv, batch, out, n_head, n_kv, head_dim, scale, window=None, chunk=None, sink=None, v_head_dim=None,
                  values_in_keys=False, bias=None, slopes=None, softcap=None, keep_first=0, maps=1, diff=None):
        H, G, d = n_head, n_kv, head_dim
        dv = v_head_dim or head_dim
        pos, slots = token_positions(batch)
        rep = H // G
        res = torch.empty(batch.n_tokens, H, dv, dtype=torch.float64, device=q.device)
        for t in range(batch.n_tokens):
            p, slot = int(pos[t]), int(slots[t])
            lo = max(0, p - window + 1) if window else 0
            if chunk:
                lo = max(lo, p // chunk * chunk)
            j = torch.arange(lo, p + 1, device=q.device)
            if keep_first and window and lo > 0:
                j = torch.cat([torch.arange(0, min(keep_first, lo), device=q.device), j])
            pages = kv.page_table.long()[slot, j // kv.page_size]
            if int(pages.min()) < 0:
                raise IndexError("attention reads a page the slot does not hold")
            k = kv.k_pool[pages, :, j % kv.page_size].double()      # [n, G, d]
            v = k[..., :dv] if values_in_keys else kv.v_pool[pages, :, j % kv.page_size].double()
            k = k.repeat_interleave(rep, dim=1)
            v = v.repeat_interleave(rep, dim=1)
            if maps == 2:
                # two softmax maps per head over the same values; their difference, normed per head and scaled
                lam, eps, out_scale = diff
                qm, km = q[t].double().view(H, 2, d), k.view(-1, H, 2, d)
                o = [torch.einsum("hn,nhd->hd", torch.softmax(torch.einsum("hd,nhd->hn", qm[:, m], km[:, :, m]) * scale, -1), v)
                     for m in range(2)]
                o = o[0] - lam * o[1]
                res[t] = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * out_scale
                continue
            s = torch.einsum("hd,nhd->hn", q[t].double(), k) * scale
            if bias is not None:
                s = s + bias.double()[(p - j).clamp(max=bias.shape[0] - 1)].T
            if slopes is not None:
                s = s - slopes.double()[:, None] * (p - j).double()[None, :]
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            if sink is not None:
                w = torch.softmax(torch.cat([s, sink.double()[:, None]], dim=-1), -1)[:, :-1]
            else:
                w = torch.softmax(s, -1)
            res[t] = torch.einsum("hn,nhd->hd", w, v)
        out.copy_(res.view(batch.n_tokens, H * dv).to(out.dtype))

    # -- sampling ----------------------------------------------------------------------------
    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(out.dtype))

    def sample(self, logits, out, temperature, top_k, seed, request_ids=None, token_index=None, index_map=None,
               noise_out=None, seed_dev=None):
        if seed_dev is not None:
            seed = int(seed_dev[0])
        B, V = logits.shape
        x = logits.float().cpu() / np.float32(max(temperature, 1e-5))
        for b in range(B):
            row = x[b]
            if top_k and top_k < V:
                pivot = torch.topk(row, top_k).values[-1]
                row = torch.where(row < pivot, torch.tensor(-math.inf), row)
            req = int(request_ids[b]) if request_ids is not None else b
            tix = 0
            if token_index is not None:
                tix = int(token_index[int(index_map[b]) if index_map is not None else b])
            qn = torch.from_numpy(race_noise(seed, req, tix, V))
            if noise_out is not None:
                noise_out[b] = qn.to(noise_out.device)
            score = torch.exp(row - row.max()) / qn
            out[b] = int(torch.argmax(score))
