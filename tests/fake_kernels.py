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

    def embedding_scaled(self, table, tokens, scale, out):
        out.copy_(table[tokens.long()].float() * scale)

    def add2_rms_norm(self, residual, delta, delta2, weight, eps, out):
        residual.add_(delta.float() + delta2.float())
        self.add_rms_norm(residual, None, weight, eps, out)

    def stream_concat(self, x, d1, d2, e, out):
        v = x.clone()
        if d1 is not None and d2 is not None:
            v += d1.float() + d2.float()
        elif d1 is not None or d2 is not None:
            v += (d1 if d1 is not None else d2).float()
        out.copy_(torch.cat([v, e], dim=-1).to(out.dtype))

    def sigmoid_mul(self, x, gate, out):
        out.copy_((x.float() * torch.sigmoid(gate.float())).to(out.dtype))

    def head_norm_gate(self, x, weight, gate, out, *, num_heads, eps):
        n, m = x.shape
        v = x.view(n, num_heads, m // num_heads)
        v = (v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)).reshape(n, m) * weight
        if gate is not None:
            v = v * torch.sigmoid(gate.float())
        out.copy_(v.to(out.dtype))

    def projection_norm_rope_store(self, proj, q_off, k_off, q_out, k_cache, v_cache, *, num_heads, num_kv_heads, head_dim,
                                   q_weight, k_weight, eps, inv_freq, rot_dim, rope_style, positions, slots):
        n = proj.shape[0]
        q = proj[:, q_off:q_off + num_heads * head_dim].float()
        kraw = proj[:, k_off:k_off + num_kv_heads * head_dim]
        k = kraw.float()
        if q_weight is not None:
            q = q * torch.rsqrt((q * q).mean(-1, keepdim=True) + eps) * q_weight
            k = k * torch.rsqrt((k * k).mean(-1, keepdim=True) + eps) * k_weight

        def rope(t):
            if not rot_dim:
                return t
            th = positions.double()[:, None] * inv_freq.double()[None, : rot_dim // 2]
            cos, sin = torch.cos(th).float()[:, None, :], torch.sin(th).float()[:, None, :]
            o = t.clone()
            half = rot_dim // 2
            if rope_style == 0:
                a, b = t[..., :half], t[..., half:rot_dim]
                o[..., :half] = a * cos - b * sin
                o[..., half:rot_dim] = a * sin + b * cos
            else:
                a, b = t[..., 0:rot_dim:2], t[..., 1:rot_dim:2]
                o[..., 0:rot_dim:2] = a * cos - b * sin
                o[..., 1:rot_dim:2] = a * sin + b * cos
            return o

        q_out.view(n, num_heads, head_dim).copy_(rope(q.view(n, num_heads, head_dim)).to(q_out.dtype))
        if k_cache is not None:
            k = rope(k.view(n, num_kv_heads, head_dim))
            v = kraw.reshape(n, num_kv_heads, head_dim)
            ps = k_cache.shape[2]
            for t in range(n):
                s = int(slots[t])
                if s < 0:
                    continue
                k_cache[s // ps, :, s % ps, :] = k[t].to(k_cache.dtype)
                v_cache[s // ps, :, s % ps, :] = v[t].to(v_cache.dtype)

    def sink_attention(self, q, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, head_dim, scale, window, sink=None,
                       gate=None, plan=None):
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
            kk = k_cache[pages, :, (js % ps).long(), :].float()
            vv = v_cache[pages, :, (js % ps).long(), :].float()
            for h in range(num_heads):
                sc = (kk[:, h // g, :] @ qf[t, h]) * scale
                if sink is not None:
                    sc = torch.cat([sc, sink[h:h + 1]])
                pr = torch.softmax(sc, dim=0)[: js.numel()]
                o[t, h] = pr @ vv[:, h // g, :]
        o = o.view(n, num_heads * head_dim)
        if gate is not None:
            o = o * torch.sigmoid(gate.float())
        out.copy_(o.to(out.dtype))

    def matrix_memory_scan(self, proj, q_off, k_off, v_off, gates, gate_bias, state, cu_q, state_slots, out, *, num_heads, dim,
                           v_dim, columns, cap, q_scale, max_q_len=0):
        H, d, dv, cb = num_heads, dim, v_dim, columns
        nblk = dv // cb
        for s in range(state_slots.numel()):
            t0, t1, slot = int(cu_q[s]), int(cu_q[s + 1]), int(state_slots[s])
            if slot < 0:
                out[t0:t1] = 0
                continue
            if t1 <= t0:
                continue
            st = state[slot]                                            # [H, nblk, block floats]
            C = st[:, :, : cb * d].reshape(H, nblk, cb, d).permute(0, 3, 1, 2).reshape(H, d, dv).clone()
            nn = st[:, 0, cb * d:(cb + 1) * d].clone()
            m = st[:, 0, (cb + 1) * d].clone()
            for t in range(t0, t1):
                row = proj[t].float()
                q = row[q_off:q_off + H * d].view(H, d) * q_scale
                k = row[k_off:k_off + H * d].view(H, d)
                v = row[v_off:v_off + H * dv].view(H, dv)
                z = gates[t] + gate_bias
                a = cap * torch.tanh(z[:H] / cap)
                b = torch.nn.functional.logsigmoid(cap * torch.tanh(z[H:] / cap))
                m_new = torch.maximum(b + m, a)
                keep, take = torch.exp(b + m - m_new), torch.exp(a - m_new)
                C = keep[:, None, None] * C + take[:, None, None] * k[:, :, None] * v[:, None, :]
                nn = keep[:, None] * nn + take[:, None] * k
                m = m_new
                den = torch.maximum((nn * q).sum(-1).abs(), torch.exp(-m)) + 1e-6
                out[t] = (torch.einsum("hdv,hd->hv", C, q) / den[:, None]).reshape(-1)
            st[:, :, : cb * d] = C.view(H, d, nblk, cb).permute(0, 2, 3, 1).reshape(H, nblk, cb * d)
            st[:, :, cb * d:(cb + 1) * d] = nn[:, None, :]
            st[:, :, (cb + 1) * d] = m[:, None]

    def moe_table_route(self, tokens, rows, table, num_experts, ids, weights, weight):
        t = tokens.long() if rows is None else tokens.long()[rows.long()]
        ids.copy_(table[t])
        weights.fill_(weight)

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
                    rot, rank, rot_dims, eps, queries=None, style=0):
        n = qd.shape[0]
        x = qd.float()
        q = (x[:, q_off:q_off + num_heads * (dim + rot)] if queries is None else queries.float()).view(n, num_heads, dim + rot)
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
            if style == 1:                      # neighbours are a pair
                a, b = t[..., 0:rot_dims:2], t[..., 1:rot_dims:2]
                o[..., 0:rot_dims:2] = a * cos - b * sin
                o[..., 1:rot_dims:2] = a * sin + b * cos
                return o
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

    # ---- a stream whose addends carry a factor, a second per-token input, xIELU, the logit cap -------------
    def scaled_add_rms_norm(self, residual, delta, mult, weight, eps, out, copy=None):
        if delta is not None:
            residual.add_(mult * delta.float())
        if copy is not None:
            copy.copy_(residual.to(copy.dtype))
        if out is not None:
            x = residual
            out.copy_((x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight).to(out.dtype))

    def scaled_add_unit_rms(self, residual, y, mult, weight, eps):
        v = y.float()
        residual.add_(mult * v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * weight)

    def rms_norm_rows(self, x, weight, eps, out):
        v = x.float()
        out.copy_((v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * weight).to(out.dtype))

    def gelu_mul_table(self, g, table, col_off, tokens, rows, out):
        tok = tokens.long() if rows is None else tokens.long()[rows.long()]
        e = table[tok[: g.shape[0]], col_off: col_off + g.shape[1]].float()
        out.copy_((torch.nn.functional.gelu(g.float(), approximate="tanh") * e).to(out.dtype))

    def xielu(self, x, pq, out):
        z = x.float()
        sp = torch.nn.functional.softplus
        pos = sp(pq[0]) * z * z + 0.5 * z
        zn = torch.clamp(z, max=0.0)
        neg = (0.5 + sp(pq[1])) * (torch.expm1(zn) - zn) + 0.5 * z
        out.copy_(torch.where(z > 0, pos, neg).to(out.dtype))

    def tanh_cap(self, x, cap):
        x.copy_(cap * torch.tanh(x / cap))

    # ---- attention inside chunks of positions, with a penalty on distance ----------------------------------
    def kv_store_normed(self, proj, k_off, v_off, k_cache, v_cache, slots, *, num_kv_heads, k_dim, v_dim, eps, norm_values):
        n = proj.shape[0]
        ps = k_cache.shape[2]
        kk = proj[:, k_off:k_off + num_kv_heads * k_dim].view(n, num_kv_heads, k_dim)
        vv = proj[:, v_off:v_off + num_kv_heads * v_dim].float().view(n, num_kv_heads, v_dim)
        if norm_values:
            vv = vv * torch.rsqrt((vv * vv).mean(-1, keepdim=True) + eps)
        for t in range(n):
            c = int(slots[t])
            if c >= 0:
                k_cache[c // ps, :, c % ps, :] = kk[t]
                v_cache[c // ps, :, c % ps, :] = vv[t].to(v_cache.dtype)

    def chunked_attention(self, q, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, k_dim, v_dim, scale, chunk, window,
                          r1, r2, gate, n_split=None):
        n = q.shape[0]
        ps = k_cache.shape[2]
        rep = num_heads // num_kv_heads
        qf = q.float().reshape(n, num_heads, k_dim)
        o = torch.zeros(n, num_heads, v_dim)
        for t in range(n):
            s = int(meta.seq_of_token[t])
            if s < 0:
                continue
            p = int(meta.positions[t])
            lo = (p // chunk) * chunk if chunk else max(0, p - window + 1) if window else 0
            js = torch.arange(lo, p + 1)
            pages = meta.block_table[s, (js // ps).long()].long()
            assert (pages >= 0).all(), "attention reads a page that was given back"
            kk = k_cache[pages, :, (js % ps).long(), :].float()
            vv = v_cache[pages, :, (js % ps).long(), :].float()
            for h in range(num_heads):
                sc = (kk[:, h // rep, :] @ qf[t, h]) * scale
                if r1 is not None:
                    sc = sc - r1[h] * torch.log1p(r2[h] * (p - js).float())
                o[t, h] = torch.softmax(sc, dim=0) @ vv[:, h // rep, :]
        o = o.view(n, num_heads * v_dim)
        if gate is not None:
            o = o * torch.sigmoid(gate.float())
        out.copy_(o.to(out.dtype))

    # ---- a normalised addend; two mixers side by side; heads' norm with a choice of gate ------------------------
    def normed_add_rms_norm(self, residual, y, post_weight, post_eps, extra, weight, eps, out):
        if y is not None:
            v = y.float()
            if post_weight is not None:
                v = v * torch.rsqrt((v * v).mean(-1, keepdim=True) + post_eps) * post_weight
            residual.add_(v)
        if extra is not None:
            residual.add_(extra)
        if out is not None:
            x = residual
            out.copy_((x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight).to(out.dtype))

    def weighted_sum2(self, x, a, y, b, out):
        out.copy_((a * x.float() + b * y.float()).to(out.dtype))

    def head_norm_gate_act(self, x, weight, gate, out, *, num_heads, eps, gate_act="sigmoid"):
        n, m = x.shape
        v = x.view(n, num_heads, m // num_heads)
        v = (v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)).reshape(n, m) * weight
        if gate is not None:
            g = gate.float()
            v = v * (torch.sigmoid(g) if gate_act == "sigmoid" else g * torch.sigmoid(g))
        out.copy_(v.to(out.dtype))

    # ---- rotated attention with kept first keys, a sink and a gate per head -------------------------------------
    def rotary_table_scaled(self, inv_freq64, positions, half, magnitude, out):
        th = positions.double()[:, None] * inv_freq64.double()[None, :half]
        out[..., 0] = (torch.cos(th) * magnitude).float()
        out[..., 1] = (torch.sin(th) * magnitude).float()

    def rotate_unit_store(self, proj, q_off, k_off, v_off, q_out, k_cache, v_cache, table, slots, *, num_heads, num_kv_heads,
                          k_dim, v_dim, rot_dim, eps, unit_norm):
        n = proj.shape[0]
        half = rot_dim // 2

        def turn(t):
            t = t.float().clone()
            if rot_dim:
                cos, sin = table[:, None, :, 0], table[:, None, :, 1]
                a, b = t[..., :half].clone(), t[..., half:rot_dim].clone()
                t[..., :half] = a * cos - b * sin
                t[..., half:rot_dim] = a * sin + b * cos
            if unit_norm:
                t = t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps)
            return t

        q_out.copy_(turn(proj[:, q_off:q_off + num_heads * k_dim].reshape(n, num_heads, k_dim)).to(q_out.dtype))
        if k_cache is None:
            return
        k = turn(proj[:, k_off:k_off + num_kv_heads * k_dim].reshape(n, num_kv_heads, k_dim))
        v = proj[:, v_off:v_off + num_kv_heads * v_dim].reshape(n, num_kv_heads, v_dim)
        ps = k_cache.shape[2]
        for t in range(n):
            s = int(slots[t])
            if s < 0:
                continue
            k_cache[s // ps, :, s % ps, :] = k[t].to(k_cache.dtype)
            v_cache[s // ps, :, s % ps, :] = v[t].to(v_cache.dtype)

    def window_attention(self, q, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, k_dim, v_dim, scale, window, keep_first,
                         sink, gate, gate_per_head, n_split=None):
        n = q.shape[0]
        ps = k_cache.shape[2]
        rep = num_heads // num_kv_heads
        qf = q.float().reshape(n, num_heads, k_dim)
        o = torch.zeros(n, num_heads, v_dim)
        for t in range(n):
            s = int(meta.seq_of_token[t])
            if s < 0:
                continue
            p = int(meta.positions[t])
            lo = max(0, p - window + 1) if window else 0
            js = torch.cat([torch.arange(0, min(keep_first, lo)), torch.arange(lo, p + 1)])
            pages = meta.block_table[s, (js // ps).long()].long()
            assert (pages >= 0).all(), "attention reads a page that was given back"
            kk = k_cache[pages, :, (js % ps).long(), :].float()
            vv = v_cache[pages, :, (js % ps).long(), :].float()
            for h in range(num_heads):
                sc = (kk[:, h // rep, :] @ qf[t, h]) * scale
                if sink is not None:
                    sc = torch.cat([sc, sink[h:h + 1]])
                o[t, h] = torch.softmax(sc, dim=0)[: js.numel()] @ vv[:, h // rep, :]
        if gate is not None and gate_per_head:
            o = o * torch.sigmoid(gate.float())[:, :, None]
        o = o.view(n, num_heads * v_dim)
        if gate is not None and not gate_per_head:
            o = o * torch.sigmoid(gate.float())
        out.copy_(o.to(out.dtype))

    # ---- linear attention with a decay ----------------------------------------------------------------------------
    def decay_scan(self, proj, q_off, k_off, v_off, state, cu_q, state_slots, out, *, num_heads, dim, v_dim, activation, q_scale,
                   head_decay=None, z=None, z_bias=None, tau=1.0, max_q_len=0):
        H, D, V = num_heads, dim, v_dim
        act = (lambda t: t * torch.sigmoid(t)) if activation == "silu" else (lambda t: t)
        for s in range(state_slots.numel()):
            t0, t1, slot = int(cu_q[s]), int(cu_q[s + 1]), int(state_slots[s])
            if slot < 0:
                out[t0:t1] = 0
                continue
            S = state[slot].reshape(H, -1, state.shape[-1])[:, :V, :D].transpose(1, 2).clone()     # columns in blocks of 16 -> [H, D, V]
            for t in range(t0, t1):
                q = act(proj[t, q_off:q_off + H * D].float()).view(H, D) * q_scale
                k = act(proj[t, k_off:k_off + H * D].float()).view(H, D)
                v = act(proj[t, v_off:v_off + H * V].float()).view(H, V)
                if head_decay is not None:
                    a = head_decay.float()[:, None].expand(H, D)
                else:
                    zz = z[t].float() + (z_bias if z_bias is not None else 0.0)
                    a = torch.exp(torch.nn.functional.logsigmoid(zz) / tau).view(H, D)
                S = a[:, :, None] * S + k[:, :, None] * v[:, None, :]
                out[t] = torch.einsum("hdv,hd->hv", S, q).reshape(H * V)
            full = torch.zeros(H, state.shape[2] * 16, state.shape[-1])
            full[:, :V, :D] = S.transpose(1, 2)
            state[slot] = full.view(state.shape[1:])

    def moe_route_softmax(self, logits, bias, top, ids, weights):
        z = logits.float() + (bias if bias is not None else 0.0)
        vals, idx = torch.sort(z, dim=-1, descending=True, stable=True)
        ids.copy_(idx[:, :top].to(torch.int32))
        weights.copy_(torch.softmax(vals[:, :top], dim=-1))

    def moe_combine_add(self, ys, pos, out, top, weights, add):
        n = out.shape[0]
        rows = ys[pos.long()].float().view(n, top, -1)
        if weights is not None:
            rows = rows * weights.view(n, top, 1)
        out.copy_((rows.sum(1) + add.float()).to(out.dtype))

    # ---- the delta rule with a decay per key channel --------------------------------------------------------
    def delta_rule(self, proj, col_off, b_off, z, taps, a_log, dt_bias, state, ctx, out, *, num_heads, num_kv_heads, dim, v_dim):
        H, G, D, V = num_heads, num_kv_heads, dim, v_dim
        C = 2 * G * D + H * V
        n_taps = taps.shape[1]
        back = n_taps - 1
        cu_q, slots = ctx.cu_q, ctx.state_slots
        sp = torch.nn.functional.softplus
        for s in range(slots.numel()):
            t0, t1, slot = int(cu_q[s]), int(cu_q[s + 1]), int(slots[s])
            if slot < 0:
                out[t0:t1] = 0
                continue
            if t1 <= t0:
                continue
            st = state[slot]
            S = st[: H * V * D].view(H, V, D).clone()                   # a column of S is contiguous
            tail = st[H * V * D:].view(back, C).clone()
            ext = torch.cat([tail, proj[t0:t1, col_off:col_off + C].float()], dim=0)
            for i, t in enumerate(range(t0, t1)):
                x = (ext[i: i + n_taps] * taps.T).sum(0)                # the last tap multiplies the token's own row
                a = x * torch.sigmoid(x)
                q = a[: G * D].view(G, D)
                k = a[G * D: 2 * G * D].view(G, D)
                q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
                k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
                q, k = q.repeat_interleave(H // G, dim=0), k.repeat_interleave(H // G, dim=0)
                v = a[2 * G * D:].view(H, V)
                beta = torch.sigmoid(proj[t, b_off:b_off + H].float())
                g = torch.exp(-torch.exp(a_log)[:, None] * sp(z[t].view(H, D) + dt_bias.view(H, D)))
                S = S * g[:, None, :]
                u = beta[:, None] * (v - torch.einsum("hvd,hd->hv", S, k))
                S = S + u[:, :, None] * k[:, None, :]
                out[t] = torch.einsum("hvd,hd->hv", S, q).reshape(-1)
            st[: H * V * D] = S.reshape(-1)
            st[H * V * D:] = ext[ext.shape[0] - back:].reshape(-1)

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
        w = weights.reshape(-1) if weights is not None else torch.ones(pos.numel())
        for i in range(pos.numel()):
            xs[int(pos[i])] = (w[i] * h[i // top].float()).to(xs.dtype)

    def moe_grouped_gemm(self, x, w, w2, out, offsets, tiles, activation="silu", limit=0.0):
        if w2 is w:         # gate and up interleaved in groups of 8 rows
            v = w.view(w.shape[0], w.shape[1] // 16, 2, 8, w.shape[2])
            w, w2 = v[:, :, 0].reshape(w.shape[0], -1, w.shape[2]), v[:, :, 1].reshape(w.shape[0], -1, w.shape[2])
        for e in range(w.shape[0]):
            a, b = int(offsets[e]), int(offsets[e + 1])
            if b <= a:
                continue
            y = x[a:b].float() @ w[e].float().T
            if w2 is not None:
                g, u = y.to(out.dtype).float(), (x[a:b].float() @ w2[e].float().T).to(out.dtype).float()
                if activation == "clamped_swish":
                    g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
                    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
                else:
                    y = self._act(g, activation) * u
            out[a:b] = y.to(out.dtype)

    def moe_combine(self, ys, pos, out, top, weights=None):
        y = ys[pos.long()].float().view(out.shape[0], top, -1)
        if weights is not None:
            y = y * weights.view(out.shape[0], top, 1)
        out.copy_(y.sum(1).to(out.dtype))

    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).int())
