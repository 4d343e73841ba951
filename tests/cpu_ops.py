"""A CPU stand-in for the kernel library, for tests only.

The engine has no CPU path.  To check its host logic (batch building, block tables, page
reuse, the run order of layers, the scheduler) on a machine without a GPU, the tests hand
the model this object in place of ``KernelOps``.  It offers the same operations on CPU
tensors with torch arithmetic in float32; it is not bit-exact with the CUDA kernels and is
never imported by the package.
"""
from __future__ import annotations

import math

import torch


class CpuOps:
    def __init__(self, dtype="float32"):
        self.dtype = dtype
        self.act_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
        self.kind = "f32" if dtype == "float32" else "bf16"
        self.launches = 0

    def embed_rows(self, table, tokens, out):
        out.copy_(table[tokens.long()].float())

    def rmsnorm(self, x, weight, eps, out, rows=None):
        src = x if rows is None else x[rows.long()]
        inv = torch.rsqrt(src.pow(2).mean(-1, keepdim=True) + eps)
        out.copy_(((src * inv) * weight).to(out.dtype))

    def linear(self, x, w, out, residual=None):
        y = x.float() @ w.float().t()
        if residual is not None:
            y = residual + y
        out.copy_(y.to(out.dtype))

    def fuses_swiglu(self, width, intermediate):
        return False

    def rope_cache(self, qkv, pos, row_seq, cos, sin, block_table, kcache, vcache, heads, kv_heads, head_dim,
                   write_kv=True):
        n = qkv.shape[0]
        page = kcache.shape[2]
        half = head_dim // 2
        q = qkv[:, :heads * head_dim].view(n, heads, head_dim).float()
        k = qkv[:, heads * head_dim:(heads + kv_heads) * head_dim].view(n, kv_heads, head_dim).float()
        v = qkv[:, (heads + kv_heads) * head_dim:].view(n, kv_heads, head_dim)
        if cos is not None:
            c = cos[pos.long()][:, None, :]
            s = sin[pos.long()][:, None, :]

            def rot(t):
                x1, x2 = t[..., :half], t[..., half:]
                return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)

            q, k = rot(q), rot(k)
        qkv[:, :heads * head_dim] = q.reshape(n, -1).to(qkv.dtype)
        if not write_kv:
            return
        for r in range(n):
            p = int(pos[r])
            blk = int(block_table[int(row_seq[r]), p // page])
            kcache[blk, :, p % page, :] = k[r].to(kcache.dtype)
            vcache[blk, :, p % page, :] = v[r]

    def attention(self, qkv, kcache, vcache, block_table, row_seq, pos, out, heads, kv_heads, head_dim, window,
                  max_keys, scale, batch=None):
        n = qkv.shape[0]
        page = kcache.shape[2]
        grp = heads // kv_heads
        for r in range(n):
            p = int(pos[r])
            lo = max(0, p - window + 1) if window and window > 0 else 0
            table = block_table[int(row_seq[r])]
            idx = torch.arange(lo, p + 1)
            blocks = table[(idx // page).long()].long()
            slots = (idx % page).long()
            k = kcache[blocks, :, slots, :].float()  # [keys, kv_heads, hd]
            v = vcache[blocks, :, slots, :].float()
            q = qkv[r, :heads * head_dim].view(heads, head_dim).float()
            kk = k.repeat_interleave(grp, dim=1)
            vv = v.repeat_interleave(grp, dim=1)
            s = torch.einsum("hd,khd->hk", q, kk) * scale
            w = torch.softmax(s, dim=-1)
            out[r] = torch.einsum("hk,khd->hd", w, vv).reshape(-1).to(out.dtype)

    def swiglu(self, gate_up, out):
        inter = out.shape[1]
        g = gate_up[:, :inter].float()
        u = gate_up[:, inter:].float()
        out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))

    def sample_rows(self, logits, temperature, uniform, out_tokens):
        for r in range(logits.shape[0]):
            t = float(temperature[r])
            row = logits[r]
            if t <= 0:
                out_tokens[r] = int(torch.argmax(row))  # torch returns the first maximum on CPU
                mx = row.max()
                out_tokens[r] = int((row == mx).nonzero()[0])
            else:
                w = torch.exp((row - row.max()) / t).double()
                cum = torch.cumsum(w, 0)
                target = float(uniform[r]) * float(cum[-1])
                hit = (cum > target).nonzero()
                out_tokens[r] = int(hit[0]) if len(hit) else int((w > 0).nonzero()[-1])

    def fingerprint_rows(self, logits, slot, state):
        import struct
        mask = (1 << 64) - 1

        def mix64(z):
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
            return z ^ (z >> 31)

        for r in range(logits.shape[0]):
            s = int(slot[r])
            h = int(state[s]) & mask
            data = logits[r].contiguous().numpy().tobytes()
            i = 0
            while i + 8 <= len(data):
                (wd,) = struct.unpack_from("<Q", data, i)
                h = ((h ^ wd) * 1099511628211) & mask
                i += 8
            while i < len(data):
                h = ((h ^ data[i]) * 1099511628211) & mask
                i += 1
            h = mix64(h)
            state[s] = h - (1 << 64) if h >= (1 << 63) else h
