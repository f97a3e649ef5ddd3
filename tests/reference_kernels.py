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

    def swiglu(self, gate_up, out, act=0):
        I = gate_up.shape[1] // 2
        g, u = gate_up[:, :I].to(self.compute), gate_up[:, I:].to(self.compute)
        out.copy_((self.gate_act(g, act) * u).to(out.dtype))

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

    def linear_skinny(self, a, w, bias, out, mode, ssq_out=None, w_next=None, xw_out=None, act=0):
        y = a.to(self.compute) @ w.to(self.compute).t()
        if mode == SK_SWIGLU:
            I = w.shape[0] // 2
            g, u = y[:, :I], y[:, I:]
            out.copy_((self.gate_act(g, act) * u).to(out.dtype))
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

    def rope_append(self, qkv, inv_freq, rotary_dim, row_pos, row_seq, seq_slot, seq_len, kv, n_heads, n_kv_heads, head_dim):
        T = qkv.shape[0]
        half = rotary_dim // 2
        heads = qkv[:, :(n_heads + 2 * n_kv_heads) * head_dim].view(T, n_heads + 2 * n_kv_heads, head_dim)
        rot = heads[:, :n_heads + n_kv_heads, :].to(self.compute)
        if half:
            ang = (row_pos[:T].to(torch.float32)[:, None] * inv_freq[None, :]).to(self.compute)
            c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
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
            kv.storage[page, 1, :, off, :] = heads[r, n_heads + n_kv_heads:, :]

    def attention(self, qkv, kv, batch, out, n_heads, n_kv_heads, head_dim, scale, window, from_cache, after_append=False):
        self.attention_plain(qkv, kv, batch.row_pos, batch.row_seq, batch.seq_slot, batch.seq_first_row, out,
                             n_heads, n_kv_heads, head_dim, scale, window, from_cache)

    def attention_plain(self, qkv, kv, row_pos, row_seq, seq_slot, seq_first_row, out, n_heads, n_kv_heads,
                        head_dim, scale, window, from_cache):
        T = qkv.shape[0]
        rep = n_heads // n_kv_heads
        heads = qkv[:, :(n_heads + 2 * n_kv_heads) * head_dim].view(T, n_heads + 2 * n_kv_heads, head_dim)
        for r in range(T):
            pos, seq = int(row_pos[r]), int(row_seq[r])
            lo = max(0, pos + 1 - window) if window > 0 else 0
            if from_cache:
                slot = int(seq_slot[seq])
                ks, vs = [], []
                for j in range(lo, pos + 1):
                    page, off = _page_offset(kv, slot, j)
                    ks.append(kv.storage[page, 0, :, off, :])
                    vs.append(kv.storage[page, 1, :, off, :])
                k = torch.stack(ks).to(self.compute)       # [keys, nkv, hd]
                v = torch.stack(vs).to(self.compute)
            else:
                first = int(seq_first_row[seq])
                k = heads[first + lo:first + pos + 1, n_heads:n_heads + n_kv_heads, :].to(self.compute)
                v = heads[first + lo:first + pos + 1, n_heads + n_kv_heads:, :].to(self.compute)
            q = heads[r, :n_heads, :].to(self.compute)
            for h in range(n_heads):
                g = h // rep
                s = (k[:, g, :] @ q[h]) * scale
                w = torch.softmax(s, dim=0)
                out[r, h * head_dim:(h + 1) * head_dim] = (w @ v[:, g, :]).to(out.dtype)

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
