"""A stand-in for the CUDA kernel set, written with torch operations on the CPU.

Only tests use it (through ``iian_b200.ops.use_kernels``), to exercise the host side of the engine --
batch building, block tables, page reuse, scheduling -- on a machine without a GPU.  It implements the
same calls with the same cache layout as ``iian_b200.ops.cuda_backend.CudaKernels``; it is not a
fallback of the product.
"""
from __future__ import annotations

import math

import torch


class FakeKernels:
    name = "fake-cpu"

    def prepare(self, dtype):
        pass

    def embedding(self, table, tokens, out):
        out.copy_(table[tokens.long()].float())

    def add_rms_norm(self, residual, delta, weight, eps, out):
        if delta is not None:
            residual.add_(delta.float())
        x = residual
        out.copy_((x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight).to(out.dtype))

    def rms_norm(self, x, weight, eps, out):
        xf = x.float()
        out.copy_((xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * weight).to(out.dtype))

    def swiglu(self, gate_up, out, interleave=0):
        f = out.shape[1]
        if interleave:
            v = gate_up.float().view(gate_up.shape[0], f // 8, 2, 8)
            g, u = v[:, :, 0].reshape(-1, f), v[:, :, 1].reshape(-1, f)
        else:
            g, u = gate_up[:, :f].float(), gate_up[:, f:].float()
        out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))

    def gather_rows(self, src, rows, out):
        out.copy_(src[rows.long()])

    def add_bias(self, x, bias):
        x.copy_((x.float() + bias).to(x.dtype))

    def linear(self, x, w, out):
        out.copy_((x.float() @ w.float().T).to(out.dtype))

    def qk_norm_rope_store(self, qkv, q_out, k_cache, v_cache, *, num_heads, num_kv_heads, head_dim, q_weight,
                           k_weight, eps, inv_freq, rot_dim, rope_style, positions, slots, write_kv, bias=None, table=None):
        n = qkv.shape[0]
        x = qkv.float()
        if bias is not None:
            x = x + bias
        x = x.view(n, num_heads + 2 * num_kv_heads, head_dim)
        q, k, v = x[:, :num_heads], x[:, num_heads:num_heads + num_kv_heads], x[:, num_heads + num_kv_heads:]

        def norm(t, w):
            return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * w if w is not None else t

        def rope(t):
            if inv_freq is None or rot_dim == 0:
                return t
            th = positions.float()[:, None] * inv_freq[None, : rot_dim // 2]
            cos, sin = torch.cos(th)[:, None, :], torch.sin(th)[:, None, :]
            o = t.clone()
            half = rot_dim // 2
            if rope_style == 0:
                x0, x1 = t[..., :half], t[..., half:rot_dim]
                o[..., :half] = x0 * cos - x1 * sin
                o[..., half:rot_dim] = x0 * sin + x1 * cos
            else:
                x0, x1 = t[..., 0:rot_dim:2], t[..., 1:rot_dim:2]
                o[..., 0:rot_dim:2] = x0 * cos - x1 * sin
                o[..., 1:rot_dim:2] = x0 * sin + x1 * cos
            return o

        q_out.view(n, num_heads, head_dim).copy_(rope(norm(q, q_weight)).to(q_out.dtype))
        if write_kv:
            k = rope(norm(k, k_weight))
            ps = k_cache.shape[2]
            for t in range(n):
                s = int(slots[t])
                if s < 0:
                    continue
                k_cache[s // ps, :, s % ps, :] = k[t].to(k_cache.dtype)
                v_cache[s // ps, :, s % ps, :] = v[t].to(v_cache.dtype)

    def paged_attention(self, q, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, head_dim, scale, window, n_split=None):
        n = q.shape[0]
        ps = k_cache.shape[2]
        g = num_heads // num_kv_heads
        qf = q.float().view(n, num_heads, head_dim)
        o = torch.zeros(n, num_heads, head_dim)
        for t in range(n):
            s = int(meta.seq_of_token[t])
            if s < 0:
                continue
            p = int(meta.positions[t])
            lo = max(0, p - window + 1) if window else 0
            js = torch.arange(lo, p + 1)
            pages = meta.block_table[s, (js // ps).long()].long()
            assert (pages >= 0).all(), "attention reads a page that was given back"
            kk = k_cache[pages, :, (js % ps).long(), :].float()      # [J, nkv, hd]
            vv = v_cache[pages, :, (js % ps).long(), :].float()
            for h in range(num_heads):
                sc = (kk[:, h // g, :] @ qf[t, h]) * scale
                pr = torch.softmax(sc, dim=0)
                o[t, h] = pr @ vv[:, h // g, :]
        out.copy_(o.view(n, num_heads * head_dim).to(out.dtype))

    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).int())
