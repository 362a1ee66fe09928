"""A stand-in for the kernel layer, written with torch on the CPU, for tests only.

It has the same methods as ``rbitnet_b200.kernels.ops.CudaOps`` so that the
package's host logic (parts, cache, paging, step function, generation loop,
trace replay) can be exercised where there is no GPU.  It is not part of the
product: the package never imports it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass
class _W:
    w: torch.Tensor
    n_out: int
    n_in: int


@dataclass
class _GU:
    w: torch.Tensor
    inner: int
    n_in: int


class TorchOps:
    def __init__(self, dtype=torch.float32):
        self.dtype = dtype
        self.device = torch.device("cpu")
        self.calls = 0

    def to_compute(self, t):
        return t.to(self.dtype).contiguous()

    def prepare_embedding(self, table):
        return self.to_compute(table)

    def prepare_linear(self, weights):
        w = torch.cat([self.to_compute(x) for x in weights], dim=0)
        return _W(w, w.shape[0], w.shape[1])

    def rows_of(self, weight, first, count):
        return _W(weight.w[first:first + count], count, weight.n_in)

    def prepare_gate_up(self, gate, up):
        return _GU(torch.cat([self.to_compute(gate), self.to_compute(up)], dim=0), gate.shape[0], gate.shape[1])

    def embed(self, ids, table, scale=1.0):
        return table[ids.long()].to(torch.float32) * scale

    def rmsnorm(self, x, w, eps, out_dtype=None):
        s = (x * x).sum(-1, keepdim=True) / x.shape[-1]
        return (x * w * (1.0 / torch.sqrt(s + eps))).to(out_dtype or self.dtype)

    def linear(self, x, weight, out_dtype=None, accumulate_into=None, scale=1.0):
        y = x.to(torch.float32) @ weight.w.to(torch.float32).T * scale
        if accumulate_into is not None:
            accumulate_into += y
            return accumulate_into
        return y.to(out_dtype or self.dtype)

    def gated_linear(self, x, weight):
        gu = x.to(torch.float32) @ weight.w.to(torch.float32).T
        g, u = gu[:, :weight.inner], gu[:, weight.inner:]
        return (g / (1.0 + torch.exp(-g)) * u).to(self.dtype)

    def project_rotate_append(self, h, weight, rotary, meta, view, n_heads):
        return self.rotate_append(self.linear(h, weight), rotary, meta, view, n_heads)

    def rotate_append(self, qkv, rotary, meta, view, n_heads):
        T = qkv.shape[0]
        D, Kh = view.head_dim, view.n_kv_heads
        x = qkv.to(torch.float32)
        q = x[:, :n_heads * D].reshape(T, n_heads, D)
        pos = meta.tok_pos.long()

        def rot(t):
            if rotary is None:
                return t
            inv, interleaved, _ = rotary
            ang = pos.to(torch.float32)[:, None] * inv[None, :]
            c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            out = torch.empty_like(t)
            if interleaved:
                a, b = t[..., 0::2], t[..., 1::2]
                out[..., 0::2], out[..., 1::2] = a * c - b * s, a * s + b * c
            else:
                h = D // 2
                a, b = t[..., :h], t[..., h:]
                out[..., :h], out[..., h:] = a * c - b * s, a * s + b * c
            return out

        q = rot(q)
        if view.writes:
            k = rot(x[:, n_heads * D:(n_heads + Kh) * D].reshape(T, Kh, D))
            v = x[:, (n_heads + Kh) * D:].reshape(T, Kh, D)
            for t in range(T):
                p, slot = int(meta.tok_pos[t]), int(meta.tok_slot[t])
                page = int(view.page_table[slot, p // view.page_size])
                view.k[page, :, p % view.page_size, :] = k[t].to(view.k.dtype)
                view.v[page, :, p % view.page_size, :] = v[t].to(view.v.dtype)
        return q.to(self.dtype)

    def attention(self, q, meta, view, n_heads, scale, window):
        T, H, D = q.shape
        G = H // view.n_kv_heads
        out = torch.zeros(T, H * D, dtype=torch.float32)
        for t in range(T):
            p, slot = int(meta.tok_pos[t]), int(meta.tok_slot[t])
            lo = max(0, p - window + 1) if window else 0
            idx = torch.arange(lo, p + 1)
            pages = view.page_table[slot, idx // view.page_size].long()
            ks = view.k[pages, :, idx % view.page_size, :].to(torch.float32)   # [n, Kh, D]
            vs = view.v[pages, :, idx % view.page_size, :].to(torch.float32)
            for h in range(H):
                s = (ks[:, h // G, :] @ q[t, h].to(torch.float32)) * scale
                pr = torch.softmax(s, dim=0)
                out[t, h * D:(h + 1) * D] = pr @ vs[:, h // G, :]
        return out.to(self.dtype)

    def gather_rows(self, x, rows):
        return x[rows.long()].clone()

    def sample(self, logits, temperature, uniform):
        out = []
        for r in range(logits.shape[0]):
            z = logits[r]
            z = torch.where(torch.isnan(z), torch.full_like(z, -math.inf), z)
            if float(temperature[r]) <= 0:
                out.append(int(torch.argmax(z)))
            else:
                e = torch.exp((z - z.max()) / float(temperature[r]))
                c = torch.cumsum(e, 0)
                hit = torch.nonzero(c >= float(uniform[r]) * c[-1])
                out.append(int(hit[0]) if hit.numel() else z.numel() - 1)
        return torch.tensor(out, dtype=torch.int32)
