"""A test double of the kernel interface (llmengine.ops.CudaOps) in plain PyTorch on the CPU.

It exists so that the host-side logic of the engine (batch building, block tables, page reuse,
scheduling, the wiring of parts) can be exercised where there is no GPU. It is never imported by
the package; the product path runs only on the CUDA kernels. Semantics follow the docstrings of
llmengine/ops.py, not the kernels' code.
"""
from __future__ import annotations


import numpy as np
import torch


class CpuOps:
    def embed(self, table, ids, out):
        n = out.shape[0]
        out.copy_(table[ids[:n].long()].float())
        return out

    def rmsnorm(self, h, weight, eps, out, delta=None, rows=None, n_rows=None, write_back=True):
        if rows is not None:
            n = rows.numel() if n_rows is None else n_rows
            idx = rows[:n].long()
            x = h[idx].clone()
            if delta is not None:
                d = delta if delta.dim() == 2 else delta.sum(0)
                x = x + d[idx]
        else:
            n = h.shape[0] if n_rows is None else n_rows
            x = h[:n]
            if delta is not None:
                d = delta if delta.dim() == 2 else delta.sum(0)
                x = x + d[:n]
                if write_back:
                    h[:n] = x
        ss = (x * x).sum(-1, keepdim=True)
        inv = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
        out[:n] = ((weight * x) * inv).to(out.dtype)
        return out

    def residual_add(self, h, delta, n_rows=None):
        n = h.shape[0] if n_rows is None else n_rows
        d = delta if delta.dim() == 2 else delta.sum(0)
        h[:n] += d[:n]
        return h

    def silu_mul(self, gate_up, out, block=0):
        ff = out.shape[1]
        if block:
            gu = gate_up.float().view(gate_up.shape[0], ff // block, 2, block)
            g, u = gu[:, :, 0].reshape(-1, ff), gu[:, :, 1].reshape(-1, ff)
        else:
            g = gate_up[:, :ff].float()
            u = gate_up[:, ff:].float()
        out.copy_(((g / (1.0 + torch.exp(-g))) * u).to(out.dtype))
        return out

    def gemm(self, a, w, out, ws=None):
        out.copy_((a.float() @ w.float().t()).to(out.dtype))
        return out

    def gemm_partials(self, a, w, ws, tag):
        parts = ws.get(tag, (2, a.shape[0], w.shape[0]), torch.float32)  # two parts, to exercise the consumers
        half = a.shape[1] // 2
        parts[0] = a[:, :half].float() @ w[:, :half].float().t()
        parts[1] = a[:, half:].float() @ w[:, half:].float().t()
        return parts

    def reduce_partials(self, parts, out):
        out.copy_(parts.sum(0).to(out.dtype))
        return out

    def silu_mul_partials(self, parts, out, block=0):
        return self.silu_mul(parts.sum(0), out, block)

    def gemm_swiglu(self, a, w_blocked, out, ws=None):
        gate_up = (a.float() @ w_blocked.float().t())
        return self.silu_mul(gate_up, out, 128)

    def rope_kv_write(self, qkv, positions, token_seq, block_table, cos, sin, kcache, vcache, n_tokens, nq, nkv, hd, parts=None):
        half = hd // 2
        src = qkv if parts is None else parts.sum(0)
        for t in range(n_tokens):
            pos = int(positions[t])
            row = src[t].float()
            q = row[: nq * hd].view(nq, hd).clone()
            k = row[nq * hd:(nq + nkv) * hd].view(nkv, hd).clone()
            v = row[(nq + nkv) * hd:].view(nkv, hd)
            if cos is not None:
                c, s = cos[pos], sin[pos]
                for x in (q, k):
                    a, b = x[:, :half].clone(), x[:, half:].clone()
                    x[:, :half] = a * c - b * s
                    x[:, half:] = b * c + a * s
            qkv[t, : nq * hd] = q.reshape(-1).to(qkv.dtype)
            if kcache is not None:
                ps = kcache.shape[2]
                page = int(block_table[int(token_seq[t]), pos // ps])
                assert page >= 0, "write into a page that was given back"
                kcache[page, :, pos % ps, :] = k.to(kcache.dtype)
                vcache[page, :, pos % ps, :] = v.to(vcache.dtype)
            else:
                qkv[t, nq * hd:(nq + nkv) * hd] = k.reshape(-1).to(qkv.dtype)

    def decode_attention_fusable(self, batch, kcache, nq, nkv, hd, out):
        return False

    def paged_attention(self, q, kcache, vcache, batch, block_table, out, nq, nkv, hd, scale, window=0):
        positions, token_seq, n_tokens = batch.positions, batch.token_seq, batch.n_tokens
        ps = kcache.shape[2]
        g = nq // nkv
        for t in range(n_tokens):
            pos = int(positions[t])
            lo = max(0, pos - window + 1) if window > 0 else 0
            tab = block_table[int(token_seq[t])]
            idx = torch.arange(lo, pos + 1)
            pages = tab[(idx // ps).long()].long()
            assert (pages >= 0).all(), "read from a page that was given back"
            K = kcache[pages, :, (idx % ps).long(), :].float()  # [S, nkv, hd]
            V = vcache[pages, :, (idx % ps).long(), :].float()
            qt = q[t].float().view(nq, hd)
            for h in range(nq):
                s = (K[:, h // g, :] @ qt[h]) * scale
                p = torch.softmax(s, dim=0)
                out[t, h * hd:(h + 1) * hd] = (p @ V[:, h // g, :]).to(out.dtype)
        return out

    @staticmethod
    def _mix32(x):
        x = x.astype(np.uint32)
        x ^= x >> np.uint32(16)
        x = (x * np.uint32(0x7FEB352D)).astype(np.uint32)
        x ^= x >> np.uint32(15)
        x = (x * np.uint32(0x846CA68B)).astype(np.uint32)
        x ^= x >> np.uint32(16)
        return x

    def sample(self, logits, out, temperature=None, seeds=None, draws=None, n_rows=None, scratch=None):
        n = logits.shape[0] if n_rows is None else n_rows
        V = logits.shape[1]
        for r in range(n):
            row = logits[r].float().numpy()
            T = float(temperature[r]) if temperature is not None else 0.0
            if T > 0:
                with np.errstate(over="ignore"):
                    k = self._mix32(np.array([int(seeds[r]) & 0xFFFFFFFF], dtype=np.uint32) ^ np.uint32(0x9E3779B9))
                    k = self._mix32(k + np.uint32(int(draws[r]) & 0xFFFFFFFF))
                    rr = self._mix32(k ^ (np.arange(V, dtype=np.uint32) * np.uint32(0x85EBCA6B)).astype(np.uint32))
                u = ((rr >> np.uint32(9)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)
                gum = -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)
                row = row * (np.float32(1.0) / np.float32(T)) + gum
            out[r] = int(np.argmax(row))
        return out
