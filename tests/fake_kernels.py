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

    # ---- post-norm layers ------------------------------------------------------------------------------
    def gated_add_layer_norm(self, x, sub, gate, gate_bias, weight, bias, alpha, eps, out, out_act):
        v = alpha * x.float()
        if sub is not None:
            s = sub.float()
            if gate is not None:
                s = s * torch.sigmoid(gate.float() + (gate_bias if gate_bias is not None else 0.0))
            v = v + s
        mu = v.mean(-1, keepdim=True)
        var = ((v - mu) ** 2).mean(-1, keepdim=True)
        y = (v - mu) / torch.sqrt(var + eps) * weight + (bias if bias is not None else 0.0)
        if out is not None:
            out.copy_(y)
        if out_act is not None:
            out_act.copy_(y.to(out_act.dtype))

    def depth_mix(self, terms, coef, rows, last_is_selected, out, out_act):
        acc = None
        for j, t in enumerate(terms):
            own = rows is None or (last_is_selected and j == len(terms) - 1)
            v = t if own else t[rows.long()]
            acc = coef[j] * v if acc is None else acc + coef[j] * v
        if out is not None:
            out.copy_(acc)
        if out_act is not None:
            out_act.copy_(acc.to(out_act.dtype))

    @staticmethod
    def _act(z, activation):
        if activation == "silu":
            return z / (1 + torch.exp(-z))
        return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))

    def gated_act(self, gate_up, out, interleave, activation):
        f = out.shape[1]
        if interleave:
            v = gate_up.float().reshape(gate_up.shape[0], f // 8, 2, 8)
            g, u = v[:, :, 0].reshape(-1, f), v[:, :, 1].reshape(-1, f)
        else:
            g, u = gate_up[:, :f].float(), gate_up[:, f:].float()
        out.copy_((self._act(g, activation) * u).to(out.dtype))

    # ---- attention over a cached latent ------------------------------------------------------------------
    def latent_prep(self, qd, q_off, dkv_off, cache_rows, q_cat, norm_weight, inv_freq, positions, slots, *, num_heads, dim,
                    rot, rank, rot_dims, eps):
        n = qd.shape[0]
        x = qd.float()
        q = x[:, q_off:q_off + num_heads * (dim + rot)].view(n, num_heads, dim + rot)
        dkv = x[:, dkv_off:dkv_off + rank + rot]

        def rope(t):
            if inv_freq is None or rot_dims == 0:
                return t
            half = rot_dims // 2
            th = positions.double()[:, None] * inv_freq.double()[None, :half]
            cos, sin = torch.cos(th).float(), torch.sin(th).float()
            while cos.dim() < t.dim():
                cos, sin = cos[:, None], sin[:, None]
            o = t.clone()
            a, b = t[..., :half], t[..., half:rot_dims]
            o[..., :half] = a * cos - b * sin
            o[..., half:rot_dims] = a * sin + b * cos
            return o

        q_cat[:, :, rank:] = rope(q[..., dim:]).to(q_cat.dtype)
        if cache_rows is not None:
            c = dkv[:, :rank]
            c = c * torch.rsqrt((c * c).mean(-1, keepdim=True) + eps) * norm_weight
            row = torch.cat([c, rope(dkv[:, rank:])], dim=-1).to(cache_rows.dtype)
            flat = cache_rows.view(-1, rank + rot)
            for t in range(n):
                s = int(slots[t])
                if s >= 0:
                    flat[s] = row[t]

    def head_linear(self, inp, in_off, in_head_stride, w, w_head_stride, w_in_stride, w_out_stride, out, out_off,
                    out_head_stride, *, num_heads, n_in, n_out):
        wf = w.float().reshape(-1)
        i = torch.arange(n_in)[:, None] * w_in_stride + torch.arange(n_out)[None, :] * w_out_stride
        for h in range(num_heads):
            x = inp[:, in_off + h * in_head_stride: in_off + h * in_head_stride + n_in].float()
            out[:, out_off + h * out_head_stride: out_off + h * out_head_stride + n_out] = (x @ wf[h * w_head_stride + i]).to(out.dtype)

    def latent_attention(self, q_cat, cache_rows, out, sink, meta, *, num_heads, rank, scale, window):
        n, _, width = q_cat.shape
        ps = cache_rows.shape[1]
        qf = q_cat.float()
        for t in range(n):
            s = int(meta.seq_of_token[t])
            if s < 0:
                out[t] = 0
                continue
            p = int(meta.positions[t])
            lo = max(0, p - window + 1) if window else 0
            js = torch.arange(lo, p + 1)
            pages = meta.block_table[s, (js // ps).long()].long()
            assert (pages >= 0).all(), "attention reads a page that was given back"
            rows = cache_rows[pages, (js % ps).long(), :].float()       # [J, width]
            sc = (qf[t] @ rows.T) * scale                                 # [H, J]
            if sink is not None:
                sc = torch.cat([sc, sink[:, None]], dim=1)
            pr = torch.softmax(sc, dim=1)[:, : rows.shape[0]]
            out[t] = (pr @ rows[:, :rank]).to(out.dtype)

    # ---- routed experts ----------------------------------------------------------------------------------
    def moe_tile_rows(self):
        return 64

    def moe_max_tiles(self, n_rows, num_experts, tile_rows=None):
        return -(-n_rows // (tile_rows or 64)) + num_experts

    def moe_route(self, logits, top, ids, weights):
        s = torch.sigmoid(logits)
        order = torch.sort(logits, dim=1, descending=True, stable=True).indices[:, :top]
        ids.copy_(order.int())
        weights.copy_(torch.gather(s, 1, order))

    def moe_plan(self, ids, num_experts, offsets, pos, tiles, tile_rows=None):
        flat = ids.reshape(-1).long()
        order = torch.sort(flat, stable=True).indices
        pos[order] = torch.arange(flat.numel(), dtype=pos.dtype)
        counts = torch.bincount(flat, minlength=num_experts)
        offsets[0] = 0
        offsets[1:] = torch.cumsum(counts, 0).int()

    def moe_scatter(self, h, pos, weights, xs, top):
        w = weights.reshape(-1)
        for i in range(pos.numel()):
            xs[int(pos[i])] = (w[i] * h[i // top].float()).to(xs.dtype)

    def moe_grouped_gemm(self, x, w, w2, out, offsets, tiles, activation="silu"):
        if w2 is w:         # gate and up interleaved in groups of 8 rows
            v = w.view(w.shape[0], w.shape[1] // 16, 2, 8, w.shape[2])
            w, w2 = v[:, :, 0].reshape(w.shape[0], -1, w.shape[2]), v[:, :, 1].reshape(w.shape[0], -1, w.shape[2])
        for e in range(w.shape[0]):
            a, b = int(offsets[e]), int(offsets[e + 1])
            if b <= a:
                continue
            y = x[a:b].float() @ w[e].float().T
            if w2 is not None:
                y = self._act(y.to(out.dtype).float(), activation) * (x[a:b].float() @ w2[e].float().T).to(out.dtype).float()
            out[a:b] = y.to(out.dtype)

    def moe_combine(self, ys, pos, out, top):
        out.copy_(ys[pos.long()].float().view(out.shape[0], top, -1).sum(1).to(out.dtype))

    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).int())
