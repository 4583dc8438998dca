"""Plain PyTorch statements of what each CUDA kernel computes, with the call signatures of
``cima_b200.kernels.Kernels``.

Two uses: the ``-m gpu`` tests compare every kernel alone with the function of the same name here;
the ``-m "not gpu"`` tests put an instance in a model's Runtime to drive the package's host logic
(cache, block tables, step function, generation loop) on the CPU.  This is test code only: the
package itself has no CPU path.  Arithmetic is float32 (float64 where noted), results are rounded
once to the output dtype.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "plain"))
from qwen2_plain import PlainXorshift, plain_sample  # noqa: E402

SK_STORE, SK_ACCUM, SK_SWIGLU, SK_STORE_F32 = 0, 1, 2, 3


def _page_offset(kv, slot, pos):
    e = pos // kv.page_size
    if kv.ring_pages:
        e %= kv.ring_pages
    return int(kv.block_table[slot, e]), pos % kv.page_size


class ReferenceKernels:
    def __init__(self, compute=torch.float32):
        self.compute = compute
        self.launches = 0

    # ------------------------------------------------------------------ elementwise
    def embed(self, ids, table, x, scale=1.0, ssq=None, w_next=None, xw=None):
        x.copy_(table[ids.long()].float() * scale)
        if ssq is not None:
            ssq.copy_((x.double() ** 2).sum(dim=1, keepdim=True).float())
        if xw is not None:
            xw.copy_((x * w_next).to(xw.dtype))

    def rmsnorm(self, x, w, eps, out):
        xc = x.to(self.compute)
        inv = 1.0 / torch.sqrt((xc * xc).mean(dim=-1, keepdim=True) + eps)
        out.copy_((xc * inv * w.to(self.compute)).to(out.dtype))

    @staticmethod
    def gate_act(g, act):
        """The gate's activation by its code: 0 SiLU, 1 GELU with tanh, 2 GELU with erf, 3 ReLU."""
        if act == 1:
            return 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
        if act == 2:
            return 0.5 * g * (1.0 + torch.erf(g * 0.7071067811865476))
        if act == 3:
            return torch.clamp(g, min=0.0)
        return g / (1.0 + torch.exp(-g))

    @classmethod
    def gated(cls, g, u, act, limit=0.0):
        """The gated middle by its code: act(g) * u, or (4) the clamped form with its limit."""
        if act == 4:
            g = torch.clamp(g, max=limit)
            u = torch.clamp(u, min=-limit, max=limit)
            return g * torch.sigmoid(1.702 * g) * (u + 1.0)
        return cls.gate_act(g, act) * u

    def swiglu(self, gate_up, out, act=0, limit=0.0):
        I = gate_up.shape[1] // 2
        g, u = gate_up[:, :I].to(self.compute), gate_up[:, I:].to(self.compute)
        out.copy_(self.gated(g, u, act, limit).to(out.dtype))

    def add_residual(self, x, delta):
        x.add_(delta.float())

    def add_rmsnorm(self, x, delta, w, eps, out):
        self.add_residual(x, delta)
        self.rmsnorm(x, w, eps, out)

    def gather_rows(self, x, rows, out):
        out.copy_(x[rows.long()])

    def decode_advance(self, chosen, tokens, row_pos, seq_len):
        tokens.copy_(chosen)
        row_pos.add_(1)
        seq_len.add_(1)

    # ------------------------------------------------------------------ matrix products
    def linear_plain(self, a, w, bias, out, accumulate=False):
        y = a.to(self.compute) @ w.to(self.compute).t()
        if bias is not None:
            y = y + bias.to(self.compute)
        if accumulate:
            out.add_(y.to(out.dtype))
        else:
            out.copy_(y.to(out.dtype))

    def library_mm(self, a, w, out, bias=None):
        self.linear_plain(a, w, bias, out)

    def linear_skinny_norm(self, xw, ssq, eps, w, bias, out, mode, act=0):
        inv = 1.0 / torch.sqrt(ssq.to(self.compute).sum(dim=1, keepdim=True) / xw.shape[1] + eps)
        h = (xw.to(self.compute) * inv).to(torch.bfloat16)
        self.linear_skinny(h, w, bias, out, mode, act=act)

    def linear_skinny(self, a, w, bias, out, mode, ssq_out=None, w_next=None, xw_out=None, act=0, limit=0.0):
        y = a.to(self.compute) @ w.to(self.compute).t()
        if mode == SK_SWIGLU:
            I = w.shape[0] // 2
            g, u = y[:, :I], y[:, I:]
            out.copy_(self.gated(g, u, act, limit).to(out.dtype))
            return
        if bias is not None:
            y = y + bias.to(self.compute)
        if mode == SK_ACCUM:
            out.add_(y.to(out.dtype))
            if ssq_out is not None:
                N = out.shape[1]
                sq = torch.zeros(out.shape[0], ssq_out.shape[1] * 16, dtype=torch.float64)
                sq[:, :N] = out.double() ** 2
                ssq_out.copy_(sq.view(out.shape[0], -1, 16).sum(dim=2).float())
            if xw_out is not None:
                xw_out.copy_((out * w_next).to(xw_out.dtype))
        else:
            out.copy_(y.to(out.dtype))

    # ------------------------------------------------------------------ attention
    def qkv_rope(self, a, w, bias, qkv, inv_freq, row_pos, row_seq, seq_slot, kv, n_heads, n_kv_heads, head_dim, norm=None):
        if norm is not None:
            ssq, eps = norm
            inv = 1.0 / torch.sqrt(ssq.to(self.compute).sum(dim=1, keepdim=True) / a.shape[1] + eps)
            a = (a.to(self.compute) * inv).to(torch.bfloat16)
        y = a.to(self.compute) @ w.to(self.compute).t()
        if bias is not None:
            y = y + bias.to(self.compute)
        seq_len = torch.zeros(int(row_seq.max()) + 1, dtype=torch.int32)
        self.rope_append(y, inv_freq, head_dim, row_pos, row_seq, seq_slot, seq_len, kv, n_heads, n_kv_heads, head_dim)
        qkv.copy_(y.to(qkv.dtype))

    def rope_append(self, qkv, inv_freq, rotary_dim, row_pos, row_seq, seq_slot, seq_len, kv, n_heads, n_kv_heads, head_dim,
                    v_heads=None, qk_norm=None, amplitude=1.0):
        T = qkv.shape[0]
        half = rotary_dim // 2
        nv = n_kv_heads if v_heads is None else v_heads
        heads = qkv[:, :(n_heads + n_kv_heads + nv) * head_dim].view(T, n_heads + n_kv_heads + nv, head_dim)
        rot = heads[:, :n_heads + n_kv_heads, :].to(self.compute)
        if qk_norm is not None:
            wq, wk, nd, eps = qk_norm
            part = rot[..., :nd]
            part = part / torch.sqrt((part * part).mean(dim=-1, keepdim=True) + eps)
            part[:, :n_heads] = part[:, :n_heads] * wq.to(self.compute)
            part[:, n_heads:] = part[:, n_heads:] * wk.to(self.compute)
            rot[..., :nd] = part
        if half:
            ang = (row_pos[:T].to(torch.float32)[:, None] * inv_freq[None, :]).to(self.compute)
            c, s = torch.cos(ang)[:, None, :] * amplitude, torch.sin(ang)[:, None, :] * amplitude
            a, b = rot[..., :half].clone(), rot[..., half:rotary_dim].clone()
            rot[..., :half] = a * c - b * s
            rot[..., half:rotary_dim] = a * s + b * c
        heads[:, :n_heads + n_kv_heads, :] = rot.to(qkv.dtype)
        if kv is None:
            return
        for r in range(T):
            slot = int(seq_slot[int(row_seq[r])])
            if kv.ring_pages and int(row_pos[r]) + kv.ring_pages * kv.page_size < int(seq_len[int(row_seq[r])]):
                continue          # a later position of this step takes the place
            page, off = _page_offset(kv, slot, int(row_pos[r]))
            kv.storage[page, 0, :, off, :] = heads[r, n_heads:n_heads + n_kv_heads, :]
            kv.storage[page, 1, :nv, off, :] = heads[r, n_heads + n_kv_heads:, :]

    def attention(self, qkv, kv, batch, out, n_heads, n_kv_heads, head_dim, scale, window, from_cache, after_append=False,
                  sink=0.0, keep_first=0, v_group=1, head_sink=None):
        self.attention_plain(qkv, kv, batch.row_pos, batch.row_seq, batch.seq_slot, batch.seq_first_row, out,
                             n_heads, n_kv_heads, head_dim, scale, window, from_cache, sink, keep_first, v_group, head_sink)

    def attention_plain(self, qkv, kv, row_pos, row_seq, seq_slot, seq_first_row, out, n_heads, n_kv_heads,
                        head_dim, scale, window, from_cache, sink=0.0, keep_first=0, v_group=1, head_sink=None):
        T = qkv.shape[0]
        rep = n_heads // n_kv_heads
        vplane = int(getattr(kv, "planes", 2)) - 1 if from_cache else 1      # one plane: the values are the keys
        cols = (n_heads + (0 if from_cache else n_kv_heads + n_kv_heads // v_group)) * head_dim
        heads = qkv[:, :cols].view(T, cols // head_dim, head_dim)
        for r in range(T):
            pos, seq = int(row_pos[r]), int(row_seq[r])
            lo = max(0, pos + 1 - window) if window > 0 else 0
            seen = list(range(0, min(keep_first, lo))) + list(range(lo, pos + 1))      # kept first positions, then the window
            if from_cache:
                slot = int(seq_slot[seq])
                ks, vs = [], []
                for j in seen:
                    page, off = _page_offset(kv, slot, j)
                    ks.append(kv.storage[page, 0, :, off, :])
                    vs.append(kv.storage[page, vplane, :, off, :])
                k = torch.stack(ks).to(self.compute)       # [keys, nkv, hd]
                v = torch.stack(vs).to(self.compute)
            else:
                first = int(seq_first_row[seq])
                rows = torch.as_tensor(seen, dtype=torch.long) + first
                k = heads[rows, n_heads:n_heads + n_kv_heads, :].to(self.compute)
                v = heads[rows, n_heads + n_kv_heads:, :].to(self.compute)
            q = heads[r, :n_heads, :].to(self.compute)
            for h in range(n_heads):
                g = h // rep
                s = (k[:, g, :] @ q[h]) * scale
                if head_sink is not None:                   # one entry of the head's own score without a value
                    z = head_sink[h].to(self.compute)
                    m = torch.maximum(s.max(), z)
                    e = torch.exp(s - m)
                    w = e / (e.sum() + torch.exp(z - m))
                elif sink:                                  # entries of score 0 without a value in the denominator
                    m = torch.clamp(s.max(), min=0.0)
                    e = torch.exp(s - m)
                    w = e / (e.sum() + sink * torch.exp(-m))
                else:
                    w = torch.softmax(s, dim=0)
                out[r, h * head_dim:(h + 1) * head_dim] = (w @ v[:, g // v_group, :]).to(out.dtype)

    # ------------------------------------------------------------------ sampling
    def argmax(self, logits, tokens):
        for i in range(logits.shape[0]):
            row = logits[i]
            best = torch.nonzero(row == row.max()).max()
            tokens[i] = int(best)

    def sample(self, logits, row_slot, params, rng, ring, count, work, tokens, all_greedy=False, general=False):
        if all_greedy:
            return self.argmax(logits, tokens)
        for i in range(logits.shape[0]):
            slot = int(row_slot[i])
            t, k, p, rp = (float(v) for v in params[i])
            pushed = int(count[slot])
            n = min(pushed, 64)
            hist = [int(ring[slot, (pushed - n + j) % 64]) for j in range(n)]
            gen = PlainXorshift(1)
            gen.state = int(np.array(int(rng[slot]), dtype=np.int64).astype(np.uint64))
            before = gen.state
            tok = plain_sample(logits[i].tolist(), hist, dict(temperature=t, top_k=int(k), top_p=p, repeat_penalty=rp), gen)
            if t > 0 and gen.state == before:
                raise AssertionError("the sampler drew without advancing its generator")
            rng[slot] = int(np.array(gen.state, dtype=np.uint64).astype(np.int64))
            tokens[i] = tok
            ring[slot, pushed % 64] = tok
            count[slot] = pushed + 1


# ---------------------------------------------------------------------- short convolution, depth average, latents
def _short_conv(self, h, w, state, batch, out, rows_per_thread=0, add_input=True, act=-1):
    taps = w.shape[0]
    first = batch.seq_first_row
    hc = h.to(self.compute)
    for s in range(batch.n_seqs):
        lo, hi = int(first[s]), int(first[s + 1])
        slot = int(batch.seq_slot[s])
        past = state[slot].to(self.compute) if taps > 1 else hc[:0]
        line = torch.cat([past, hc[lo:hi]])                      # the inputs from taps - 1 positions before the step on
        n = hi - lo
        acc = hc[lo:hi].clone() if add_input else torch.zeros_like(hc[lo:hi])
        for j in range(taps):
            acc = acc + w[j].to(self.compute) * line[j:j + n]
        if act >= 0:
            acc = self.gate_act(acc, act)
        out[lo:hi] = acc.to(out.dtype)
        if taps > 1:
            state[slot] = line[n:].to(state.dtype)


def _depth_average(self, stack, n, a, x, w=None, eps=0.0, y=None, conv=None):
    acc = torch.zeros_like(x)
    for j in range(n):
        acc = acc + a[j] * stack[j]
    x.copy_(acc)
    if w is not None:
        self.rmsnorm(x, w, eps, y)
    if conv is not None:
        cw, state, seq_slot, u = conv
        taps = cw.shape[0]
        for r in range(x.shape[0]):
            slot = int(seq_slot[r])
            past = state[slot].to(self.compute) if taps > 1 else y[:0].to(self.compute)
            line = torch.cat([past, y[r:r + 1].to(self.compute)])
            u[r] = (y[r].to(self.compute) + (cw.to(self.compute) * line).sum(dim=0)).to(u.dtype)
            if taps > 1:
                state[slot] = line[1:].to(state.dtype)


def _latent_append(self, raw, g, eps, kv, batch):
    r = raw.to(self.compute)
    c = r / torch.sqrt((r * r).mean(dim=-1, keepdim=True) + eps) * g.to(self.compute)
    for t in range(raw.shape[0]):
        page, off = _page_offset(kv, int(batch.seq_slot[int(batch.row_seq[t])]), int(batch.row_pos[t]))
        kv.storage[page, 0, 0, off, :] = c[t].to(kv.storage.dtype)


def _head_linear(self, a, w, out, append=None, a_head=None, out_head=None):
    if append is not None:
        self.latent_append(*append)
    heads, N, K = w.shape
    ha, ho = a_head or K, out_head or N
    T = a.shape[0]
    av = torch.stack([a[:, h * ha:h * ha + K] for h in range(heads)], dim=1)
    y = torch.einsum("thk,hnk->thn", av.to(self.compute), w.to(self.compute)).to(out.dtype)
    for h in range(heads):
        out[:, h * ho:h * ho + N] = y[:, h]


def _turn_pairs(x, pos, inv_freq, amplitude, interleaved, compute):
    """x [..., rot] rotated at positions pos (broadcast over the leading dims of x): pairs of neighbours or of halves."""
    rot = x.shape[-1]
    half = rot // 2
    ang = (pos.to(torch.float32)[..., None] * inv_freq).to(compute)
    c, s = torch.cos(ang) * amplitude, torch.sin(ang) * amplitude
    x = x.to(compute)
    out = torch.empty_like(x)
    if interleaved:
        a, b = x[..., 0::2], x[..., 1::2]
        out[..., 0::2], out[..., 1::2] = a * c - b * s, b * c + a * s
    else:
        a, b = x[..., :half], x[..., half:]
        out[..., :half], out[..., half:] = a * c - b * s, b * c + a * s
    return out


def _latent_prepare(self, ql, first, q_norm, cq, c_norm, eps, rank, rot, inv_freq, amplitude, interleaved, kv, batch, step_rows=None):
    T = ql.shape[0]
    r = ql.to(self.compute)
    if cq is not None:
        p = r[:, :first]
        cq.copy_((p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps) * q_norm.to(self.compute)).to(cq.dtype))
    p = r[:, first:first + rank]
    both = torch.empty((T, rank + rot), dtype=ql.dtype)
    both[:, :rank] = (p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps) * c_norm.to(self.compute)).to(ql.dtype)
    if rot:
        both[:, rank:] = _turn_pairs(ql[:, first + rank:first + rank + rot], batch.row_pos[:T], inv_freq, amplitude, interleaved,
                                     self.compute).to(ql.dtype)
    for t in range(T):
        seq = int(batch.row_seq[t])
        if kv.ring_pages and int(batch.row_pos[t]) + kv.ring_pages * kv.page_size < int(batch.seq_len[seq]):
            continue
        page, off = _page_offset(kv, int(batch.seq_slot[seq]), int(batch.row_pos[t]))
        kv.storage[page, 0, 0, off, :] = both[t]
    if step_rows is not None:
        buf, col = step_rows
        buf[:, col:col + rank + rot] = both
        buf[:, col + rank + rot:col + 2 * (rank + rot)] = both


def _rope_rows(self, q, q_off, q_head, out, o_off, o_head, heads, rot, inv_freq, amplitude, interleaved, row_pos):
    T = q.shape[0]
    for h in range(heads):
        part = q[:, h * q_head + q_off:h * q_head + q_off + rot]
        out[:, h * o_head + o_off:h * o_head + o_off + rot] = _turn_pairs(part, row_pos[:T], inv_freq, amplitude, interleaved,
                                                                         self.compute).to(out.dtype)


def _hyper_connect(self, xs, y, C, b, mult, a_next, w_next, eps, h, spread=False):
    T, S, W = xs.shape
    if y is not None:
        if spread:
            xs.copy_(y[:, None, :].expand(T, S, W))
        else:
            new = torch.einsum("st,xsw->xtw", C.view(S, S), xs) + mult * b.view(1, S, 1) * y[:, None, :]
            xs.copy_(new)
    if a_next is not None:
        u = torch.einsum("s,xsw->xw", a_next, xs)
        h.copy_((u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps) * w_next).to(h.dtype))


def _activate(self, z, act):
    f = z.float()
    z.copy_((torch.clamp(f, min=0.0) ** 2 if act == 5 else self.gate_act(f, act)).to(z.dtype))


ReferenceKernels.short_conv = _short_conv
ReferenceKernels.depth_average = _depth_average
ReferenceKernels.latent_append = _latent_append
ReferenceKernels.head_linear = _head_linear
ReferenceKernels.latent_prepare = _latent_prepare
ReferenceKernels.rope_rows = _rope_rows
ReferenceKernels.hyper_connect = _hyper_connect
ReferenceKernels.activate = _activate


# ---------------------------------------------------------------------- Dynamic Tanh, bigram embedding
def _dyt(self, x, alpha, w, b, out):
    out.copy_((torch.tanh(alpha.to(self.compute) * x.to(self.compute)) * w + b).to(out.dtype))


def _dyt_add(self, x, y, norm, mult, next_norm=None, h=None):
    a1, w1, b1 = norm
    x.add_(mult * (torch.tanh(a1 * y) * w1 + b1))
    if next_norm is not None:
        a2, w2, b2 = next_norm
        h.copy_((torch.tanh(a2 * x) * w2 + b2).to(h.dtype))


def _embed_bigram(self, batch, table, bigram, x, scale, buckets, mul_prev, mul_cur, prev_state):
    ids = batch.tokens
    for r in range(batch.n_rows):
        seq = int(batch.row_seq[r])
        slot = int(batch.seq_slot[seq])
        k = r - int(batch.seq_first_row[seq])
        prev = int(ids[r - 1]) if k > 0 else int(prev_state[slot])
        row = buckets if int(batch.row_pos[r]) == 0 else (prev * mul_prev + int(ids[r]) * mul_cur) % buckets
        x[r] = table[int(ids[r])].float() * scale + bigram[row].float()
    for s in range(batch.n_seqs):
        prev_state[int(batch.seq_slot[s])] = int(ids[int(batch.seq_first_row[s + 1]) - 1])


# ---------------------------------------------------------------------- recurrent mixers
def _silu(z):
    return z / (1.0 + torch.exp(-z))


def _recurrence(self, q, k, v, state, batch, out, heads, kv_heads, dim, vdim, g=None, beta=None, decay=None, gate=None):
    delta = g is not None
    T = batch.n_rows
    qf, kf, vf = q.float().view(T, kv_heads, dim), k.float().view(T, kv_heads, dim), v.float().view(T, heads, vdim)
    if gate is not None:
        bias, lower = (t.view(1, heads, dim) for t in gate)
        f = lower + (1.0 - lower) * torch.sigmoid(kf + bias)
        qf = _silu(qf)
        for s in range(batch.n_seqs):
            lo, hi = int(batch.seq_first_row[s]), int(batch.seq_first_row[s + 1])
            slot = int(batch.seq_slot[s])
            S = state[slot].clone()
            for t in range(lo, hi):
                S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * vf[t][:, None, :]
                out[t] = torch.einsum("hdv,hd->hv", S, qf[t]).reshape(-1)
            state[slot] = S
        return
    if not delta:
        qf, kf, vf = _silu(qf), _silu(kf), _silu(vf)
    share = heads // kv_heads
    for s in range(batch.n_seqs):
        lo, hi = int(batch.seq_first_row[s]), int(batch.seq_first_row[s + 1])
        slot = int(batch.seq_slot[s])
        for h in range(heads):
            c = h // share
            S = state[slot, h].clone()
            for t in range(lo, hi):
                if delta:
                    S = g[t].view(heads, dim)[h][:, None] * S
                    u = beta[t, h] * (vf[t, h] - S.T @ kf[t, c])
                else:
                    S = decay[h] * S
                    u = vf[t, h]
                S = S + torch.outer(kf[t, c], u)
                out[t, h * vdim:(h + 1) * vdim] = S.T @ qf[t, c]
            state[slot, h] = S


def _delta_prepare(self, qk, a, b, A_log, dt_bias, qn, kn, g, beta, heads, kv_heads, dim):
    T = qk.shape[0]
    kd = kv_heads * dim
    qf, kf = qk[:, :kd].float().view(T, kv_heads, dim), qk[:, kd:2 * kd].float().view(T, kv_heads, dim)
    qn.copy_((qf / torch.sqrt((qf * qf).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5).view(T, kd))
    kn.copy_((kf / torch.sqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)).view(T, kd))
    step = torch.nn.functional.softplus(a.float() + dt_bias).view(T, heads, dim)
    g.copy_(torch.exp(-torch.exp(A_log)[None, :, None] * step).view(T, heads * dim))
    beta.copy_(torch.sigmoid(b.float()))


def _group_rmsnorm_gate(self, o, w, gate, out, groups, eps):
    T, W = o.shape
    n = W // groups
    z = o.view(T, groups, n)
    z = z / torch.sqrt((z * z).mean(-1, keepdim=True) + eps)
    z = z * (w.view(1, 1, n) if w.numel() == n and groups > 1 else w.view(1, groups, n))
    if gate is not None:
        z = z * torch.sigmoid(gate.float().view(T, groups, n))
    out.copy_(z.view(T, W).to(out.dtype))


def _rms_mean(self, ys, ws, x, eps, assign=False):
    acc = torch.zeros_like(x)
    for y, w in zip(ys, ws):
        acc = acc + y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w
    if assign:
        x.copy_(acc / len(ys))
    else:
        x.add_(acc / len(ys))


# ---------------------------------------------------------------------- routed feed-forward
def _moe_route(self, scores, top, groups, keep, scale, idx, wgt, experts=None, softmax=False, correction=None):
    T = scores.shape[0]
    E = scores.shape[1] if experts is None else experts
    per = E // groups
    s = torch.softmax(scores[:, :E], dim=-1) if softmax else torch.sigmoid(scores[:, :E])
    cmp = s if correction is None else s + correction
    for t in range(T):
        gs = [float(cmp[t, gi * per:(gi + 1) * per].topk(min(2, per)).values.sum()) for gi in range(groups)]
        best = sorted(range(groups), key=lambda gi: (-gs[gi], gi))[:keep]
        allowed = [e for gi in best for e in range(gi * per, (gi + 1) * per)]
        chosen = sorted(allowed, key=lambda e: (-float(cmp[t, e]), e))[:top]
        w = torch.stack([s[t, e] for e in chosen])
        idx[t] = torch.tensor(chosen, dtype=idx.dtype)
        wgt[t] = w / (w.sum() + 1e-20) * scale
    scores[:, :E] = s


def _moe_experts(self, h, gate_up, down, idx, wgt, x, act=0, assign=False, limit=0.0, shared=None):
    ff = gate_up.shape[1] // 2
    hf = h.float()
    for t in range(h.shape[0]):
        acc = torch.zeros_like(x[t])
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            gu = (gate_up[e].float() @ hf[t]).to(h.dtype).float()
            z = self.gated(gu[:ff], gu[ff:], act, limit).to(h.dtype).float()
            acc = acc + wgt[t, j] * (down[e].float() @ z)
        if shared is not None:
            rows, gate, col = shared
            acc = acc + (torch.sigmoid(gate[t, col]) if gate is not None else 1.0) * rows[t]
        x[t] = acc if assign else x[t] + acc


# ---------------------------------------------------------------------- differential attention, the norm behind a sum
def _diff_combine(self, att, gate, out, heads, rep, head_dim, v_dim, lam, post, eps):
    T = att.shape[0]
    a = att.float().view(T, heads // rep, 2, rep, head_dim)[..., :v_dim]
    o = (a[:, :, 0] - lam * a[:, :, 1]).reshape(T, heads, v_dim)
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * post
    if gate is not None:
        o = o * torch.sigmoid(gate.float())[:, :, None]
    out.copy_(o.reshape(T, heads * v_dim).to(out.dtype))


def _scale_add_group_rmsnorm(self, x, y, alpha, w, groups, eps, h=None):
    T, W = x.shape
    z = alpha * x if y is None else alpha * x + y
    z = z.view(T, groups, W // groups)
    z = (z / torch.sqrt((z * z).mean(-1, keepdim=True) + eps)).view(T, W) * w
    x.copy_(z)
    if h is not None:
        h.copy_(z.to(h.dtype))


def _cast_rows(self, x, h):
    h.copy_(x.to(h.dtype))


def _softcap(self, logits, cap):
    logits.copy_(cap * torch.tanh(logits / cap))


for _name, _fn in (("diff_combine", _diff_combine), ("scale_add_group_rmsnorm", _scale_add_group_rmsnorm), ("cast_rows", _cast_rows),
                   ("softcap", _softcap)):
    setattr(ReferenceKernels, _name, _fn)

for _name, _fn in (("dyt", _dyt), ("dyt_add", _dyt_add), ("embed_bigram", _embed_bigram), ("recurrence", _recurrence),
                   ("delta_prepare", _delta_prepare), ("group_rmsnorm_gate", _group_rmsnorm_gate), ("rms_mean", _rms_mean),
                   ("moe_route", _moe_route), ("moe_experts", _moe_experts)):
    setattr(ReferenceKernels, _name, _fn)
