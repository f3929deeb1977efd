"""Plain PyTorch twins of the kernel operations, one function per kernel, with the
signatures of ``hetero_serve_b200.kernels.CudaOps``.

They serve two purposes: each CUDA kernel is compared with its twin (in float64
where the twin is the reference), and, since they run on CPU tensors, the engine's
step function, cache and scheduler can be exercised without a GPU in the tests.
They are written for clarity (loops over tokens and heads), not for speed, and are
never imported by the package.
"""

from __future__ import annotations

import math

import torch

try:
    from .plain_gpt2 import gelu_erf, gelu_new, philox4x32, sample_token, uniform_for
except ImportError:  # run as a top-level module
    from plain_gpt2 import gelu_erf, gelu_new, philox4x32, sample_token, uniform_for

_ACT = {"none": lambda u: u, "gelu_tanh": gelu_new, "gelu_erf": gelu_erf}


class PlainOps:
    name = "plain"

    def __init__(self, compute_dtype=torch.float64):
        self.cd = compute_dtype

    def embed(self, x, ids, pos, req, wte, wpe, status, feedback=None):
        n = x.shape[0]
        for t in range(n):
            if int(req[t]) < 0:
                x[t] = 0
                continue
            tok = int(ids[t])
            if tok < 0 and feedback is not None:
                tok = int(feedback[-(tok + 1)])
            row = wte[tok].to(self.cd)
            if wpe is not None:
                row = row + wpe[int(pos[t])].to(self.cd)
            x[t] = row.to(x.dtype)

    def layernorm(self, out, x, gamma, beta, eps, rows=None):
        n = out.shape[0]
        src = x[rows[:n].long()] if rows is not None else x[:n]
        v = src.to(self.cd)
        mu = v.mean(-1, keepdim=True)
        c = v - mu
        var = (c * c).mean(-1, keepdim=True)
        out.copy_((c / torch.sqrt(var + eps) * gamma.to(self.cd) + beta.to(self.cd)).to(out.dtype))

    def linear(self, out, a, w, bias=None, act="none", residual=None):
        v = a.to(self.cd) @ w.to(self.cd).T
        if bias is not None:
            v = v + bias.to(self.cd)
        v = _ACT[act](v)
        if residual is not None:
            v = v + residual.to(self.cd)
        out.copy_(v.to(out.dtype))

    def norm_linear(self, out, h, x, gamma, beta, eps, w, bias=None, act="none"):
        self.layernorm(h, x, gamma, beta, eps)
        self.linear(out, h, w, bias, act=act)

    @staticmethod
    def _pool_view(pool, g):
        return pool.view(g.num_pages, 2, g.n_kv_heads, g.page_size, g.head_dim)

    def kv_append(self, pool, qkv, table, tok_pos, tok_req, g, status, n_tokens=None):
        n = qkv.shape[0] if n_tokens is None else n_tokens
        pv = self._pool_view(pool, g)
        kw = g.n_kv_heads * g.head_dim
        for t in range(n):
            r = int(tok_req[t])
            if r < 0:
                continue
            p = int(tok_pos[t])
            page = int(table[r, p // g.page_size])
            slot = p % g.page_size
            pv[page, 0, :, slot, :] = qkv[t, g.k_off:g.k_off + kw].view(g.n_kv_heads, g.head_dim)
            pv[page, 1, :, slot, :] = qkv[t, g.v_off:g.v_off + kw].view(g.n_kv_heads, g.head_dim)

    def attention(self, out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan=None):
        n = out.shape[0]
        pv = self._pool_view(pool, g)
        D, H, HK = g.head_dim, g.n_heads, g.n_kv_heads
        scale32 = float(torch.tensor(scale, dtype=torch.float32))
        for t in range(n):
            r = int(tok_req[t])
            if r < 0:
                out[t] = 0
                continue
            p = int(tok_pos[t])
            lo = max(0, p - g.window + 1) if g.window > 0 else 0
            js = torch.arange(lo, p + 1)
            pages = table[r, (js // g.page_size).to(table.device)].long()
            slots = (js % g.page_size).to(table.device)
            k = pv[pages, 0, :, slots, :].to(self.cd)       # [n_keys, HK, D]
            v = pv[pages, 1, :, slots, :].to(self.cd)
            q = qkv[t, g.q_off:g.q_off + H * D].view(H, D).to(self.cd)
            for h in range(H):
                hk = h // (H // HK)
                s = (k[:, hk, :] @ q[h]) * scale32
                pr = torch.softmax(s, 0)
                out[t, h * D:(h + 1) * D] = (pr @ v[:, hk, :]).to(out.dtype)

    def attention_append(self, out, qkv, pool, table, tok_pos, tok_req, g, scale, status,
                         plan=None, writes=True):
        if writes:
            self.kv_append(pool, qkv, table, tok_pos, tok_req, g, status)
        self.attention(out, qkv, pool, table, tok_pos, tok_req, g, scale, status, plan)

    def argmax(self, out, logits):
        rows = logits.shape[0]
        out[:rows] = torch.argmax(logits, dim=-1).to(torch.int32)

    def sample(self, out, logits, temperature, top_k, seed_lo, seed_hi, position,
               feedback=None, feedback_slot=None):
        for r in range(logits.shape[0]):
            seed = (int(seed_lo[r]) & 0xFFFFFFFF) | ((int(seed_hi[r]) & 0xFFFFFFFF) << 32)
            u = uniform_for(seed, int(position[r]))
            out[r] = sample_token(logits[r].cpu(), float(temperature[r]), int(top_k[r]), u)
            if feedback is not None and int(feedback_slot[r]) >= 0:
                feedback[int(feedback_slot[r])] = out[r]
