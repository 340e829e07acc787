"""Plain twins of the kernels, one method per kernel of ``CudaKernels``, written with
torch on the CPU in float64 and rounded once to the output type.  They are test
equipment, not a product path: the engine never picks them by itself.  They serve
(1) as the plain reference of each kernel in the ``-m gpu`` tests and (2) to run the
step function, the cache manager and the scheduler on a machine without a GPU, when
a test passes ``ops=CpuOps()`` to the runner.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


class CpuOps:
    def __init__(self):
        self.launches = 0

    def projection_buffer(self, rows, width, device, act_dtype):
        return torch.empty((rows, width), dtype=torch.float32, device=device)

    def reset_state_slots(self, state, slots, pos_start):
        for slot, p in zip(slots.tolist(), pos_start.tolist()):
            if p == 0:
                state[slot].zero_()

    def gather_tokens(self, token_ids, drawn, src):
        m = src >= 0
        token_ids[m] = drawn[src[m].long()]

    def embed(self, token_ids, table, out, scale=1.0):
        out.copy_((table[token_ids.long()].to(F64) * scale).to(torch.float32))

    def logit_transform(self, logits, scale=1.0, softcap=0.0):
        v = logits.to(F64) * scale
        if softcap > 0:
            v = softcap * torch.tanh(v / softcap)
        logits.copy_(v.to(torch.float32))

    def rmsnorm(self, x, weight, eps, out, row_index=None):
        xs = x if row_index is None else x[row_index.long()]
        xs = xs.to(F64)
        r = torch.rsqrt((xs * xs).mean(-1, keepdim=True) + eps)
        out.copy_(((xs * r) * weight.to(F64)).to(out.dtype))

    def gemm(self, a, w, out, residual=None):
        acc = a.to(F64) @ w.to(F64).t()
        if residual is not None:
            acc = residual.to(F64) + acc
        out.copy_(acc.to(out.dtype))

    def merge_gate_up(self, gate_w, up_w):
        return torch.cat([gate_w, up_w], dim=0).contiguous()

    def swiglu(self, gate_up, out, block=0):
        I = out.shape[1]
        if block:
            v = gate_up.view(gate_up.shape[0], I // block, 2, block)
            g, u = v[:, :, 0].reshape(-1, I).to(F64), v[:, :, 1].reshape(-1, I).to(F64)
        else:
            g, u = gate_up[:, :I].to(F64), gate_up[:, I:].to(F64)
        out.copy_(((g / (1.0 + torch.exp(-g))) * u).to(out.dtype))

    def rope_table(self, table, theta, rot_dim):
        half = rot_dim // 2
        i = torch.arange(half, dtype=F64)
        inv = torch.exp(-(2.0 * i / rot_dim) * math.log(theta)).to(torch.float32)
        p = torch.arange(table.shape[0], dtype=torch.float32)
        ang = (p[:, None] * inv[None, :]).to(F64)       # the angle is a float32 product
        table[..., 0] = torch.cos(ang).to(torch.float32)
        table[..., 1] = torch.sin(ang).to(torch.float32)

    def attend(self, h, w_qkv, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache, kv_layer, page_size, out,
               nq, nkv, d, scale, window, write_cache):
        q = torch.empty((h.shape[0], nq * d), dtype=out.dtype, device=out.device)
        self.qkv_project(h, w_qkv, q, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache, kv_layer, page_size,
                         nq, nkv, d, write_cache)
        self.attention(q, batch, block_table, kv_cache, kv_layer, page_size, out, nq, nkv, d, scale, window)

    def qkv_project(self, h, w_qkv, q_out, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache,
                    kv_layer, page_size, nq, nkv, d, write_cache):
        qkv = self.projection_buffer(h.shape[0], (nq + 2 * nkv) * d, h.device, h.dtype)
        self.gemm(h, w_qkv, qkv)
        self.qk_norm_rope_kv_write(qkv, q_out, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache,
                                   kv_layer, page_size, nq, nkv, d, write_cache)

    def qk_norm_rope_kv_write(self, qkv, q_out, q_w, k_w, eps, table, rot_dim, batch, block_table, kv_cache,
                              kv_layer, page_size, nq, nkv, d, write_cache):
        T = qkv.shape[0]
        x = qkv.to(F64).view(T, nq + 2 * nkv, d)
        q, k, v = x[:, :nq], x[:, nq:nq + nkv], x[:, nq + nkv:]

        def norm(t, w):
            if w is None:
                return t
            r = torch.rsqrt((t * t).mean(-1, keepdim=True) + eps)
            return (t * r) * w.to(F64)

        def rope(t):
            if table is None or rot_dim == 0:
                return t
            half = rot_dim // 2
            cs = table[batch.positions.long()].to(F64)          # [T, half, 2]
            c, s = cs[..., 0][:, None, :], cs[..., 1][:, None, :]
            a, b = t[..., :half], t[..., half:rot_dim]
            return torch.cat([a * c - b * s, a * s + b * c, t[..., rot_dim:]], dim=-1)

        q_out.copy_(rope(norm(q, q_w)).reshape(T, nq * d).to(q_out.dtype))
        if not write_cache:
            return
        kn = rope(norm(k, k_w)).to(kv_cache.dtype)
        vv = v.to(kv_cache.dtype)
        pos = batch.positions.tolist()
        req = batch.tok_req.tolist()
        for t in range(T):
            page = int(block_table[req[t], pos[t] // page_size])
            assert page >= 0, "token written to a page that was not reserved"
            kv_cache[page, kv_layer, 0, :, pos[t] % page_size, :] = kn[t]
            kv_cache[page, kv_layer, 1, :, pos[t] % page_size, :] = vv[t]

    def attention(self, q_in, batch, block_table, kv_cache, kv_layer, page_size, out,
                  nq, nkv, d, scale, window):
        T = q_in.shape[0]
        q = q_in.to(F64).view(T, nq, d)
        pos = batch.positions.tolist()
        req = batch.tok_req.tolist()
        G = nq // nkv
        for t in range(T):
            p = pos[t]
            lo = max(0, p - window + 1) if window > 0 else 0
            idx = torch.arange(lo, p + 1)
            pages = block_table[req[t]].long()[idx // page_size]
            assert (pages >= 0).all(), "attention reads a page that was given back"
            K = kv_cache[pages, kv_layer, 0, :, idx % page_size, :].to(F64)     # [n, nkv, d]
            V = kv_cache[pages, kv_layer, 1, :, idx % page_size, :].to(F64)
            for h in range(nq):
                s = (K[:, h // G, :] @ q[t, h]) * scale
                pr = torch.softmax(s, 0)
                out[t, h * d:(h + 1) * d] = (pr @ V[:, h // G, :]).to(out.dtype)

    def gated_mlp(self, h, w_gate_up, w_down, residual, inter):
        act = torch.empty((h.shape[0], inter), dtype=h.dtype, device=h.device)
        self.gemm_swiglu(h, w_gate_up, act)
        self.gemm(act, w_down, residual, residual=residual)

    def gemm_swiglu(self, a, w_gate_up, out):
        gu = a.to(F64) @ w_gate_up.to(F64).t()
        I = out.shape[1]
        g, u = gu[:, :I], gu[:, I:]
        out.copy_(((g / (1.0 + torch.exp(-g))) * u).to(out.dtype))

    def argmax(self, logits, out):
        for r in range(logits.shape[0]):
            out[r] = int((logits[r] == logits[r].max()).nonzero()[0].item())

    def sample(self, logits, temperature, uniform, out, top_k=None, top_p=None, min_p=None):
        from plain_qwen3 import sample_temperature
        for r in range(logits.shape[0]):
            out[r] = sample_temperature(
                logits[r], float(temperature[r]), float(uniform[r]),
                int(top_k[r]) if top_k is not None else 0,
                float(top_p[r]) if top_p is not None else 1.0,
                float(min_p[r]) if min_p is not None else 0.0)

    def repetition_penalty(self, logits, rows, tokens, penalty):
        for r, t, p in zip(rows.tolist(), tokens.tolist(), penalty.tolist()):
            v = float(logits[r, t])
            logits[r, t] = v / p if v > 0 else v * p
