"""Plain PyTorch statements of the engine's operators, one loop-level function each.

Two uses, both in tests only: (1) the reference each CUDA kernel is compared with, and (2) an
operator set that lets the engine's host logic (step function, cache, scheduler) be exercised on
a machine without a GPU.  The package never imports this file.  Everything is computed in
float32 (float64 where noted) whatever the element type of the inputs, and rounded once.
"""
from __future__ import annotations

import math

import torch


class TorchOps:
    name = "torch-reference"

    def __init__(self, device="cpu"):
        self.device = torch.device(device)

    def empty(self, shape, dtype):
        return torch.empty(shape, dtype=dtype, device=self.device)

    def embed(self, ids, table):
        return table[ids.long()].clone()

    def add_rmsnorm(self, x, residual, weight, eps, rows=None, dtype=None, bias=None):
        dtype = dtype or x.dtype
        s = None
        if residual is not None:
            s = residual.float()
        if x is not None:
            s = x.float() if s is None else s + x.float()
        if bias is not None:
            s = s + bias.float()
        if rows is not None:
            s = s[rows.long()]
        y = s * torch.rsqrt((s * s).mean(-1, keepdim=True) + eps) * weight.float()
        if rows is not None:
            return y.to(dtype), None
        if residual is not None:
            residual.copy_(s)
            return y.to(dtype), residual
        return y.to(dtype), s

    def linear(self, x, w, out_dtype=None):
        return (x.float() @ w.float().T).to(out_dtype or x.dtype)

    linear_simt = linear

    def linear_add(self, x, w, residual):
        return self.linear(x, w)          # never fused: the caller's norm adds it

    def fused_ffn_layout(self, dtype, hidden, inter):
        return False

    def silu_mul(self, gu):
        inter = gu.shape[1] // 2
        g, u = gu[:, :inter].float(), gu[:, inter:].float()
        return (g * torch.sigmoid(g) * u).to(gu.dtype)

    def rope_kv_write(self, qkv, positions, inv_freq, rot, slots, cache, nq, nkv, d, page_size):
        T = qkv.shape[0]
        heads = qkv.view(T, nq + 2 * nkv, d)
        if inv_freq is not None and rot > 0:
            half = rot // 2
            ang = positions.float()[:, None] * inv_freq.float()[None, :half]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
            qk = heads[:, : nq + nkv].float()
            x1, x2 = qk[..., :half].clone(), qk[..., half:rot].clone()
            qk[..., :half] = x1 * cos - x2 * sin
            qk[..., half:rot] = x2 * cos + x1 * sin
            heads[:, : nq + nkv] = qk.to(qkv.dtype)
        if cache is not None:
            for t in range(T):
                s = int(slots[t])
                if s < 0:
                    continue
                page, off = divmod(s, page_size)
                cache[page, 0, :, off, :] = heads[t, nq:nq + nkv]
                cache[page, 1, :, off, :] = heads[t, nq + nkv:]

    def paged_attention(self, q, cache, block_table, tok_req, positions, nq, nkv, d, page_size, scale,
                        window=0, splits=1, hints=None):
        T = q.shape[0]
        out = torch.zeros((T, nq * d), dtype=torch.float32, device=q.device)
        group = nq // nkv
        for t in range(T):
            r, p = int(tok_req[t]), int(positions[t])
            lo = max(0, p - window + 1) if window > 0 else 0
            keys = torch.arange(lo, p + 1)
            pages = block_table[r][(keys // page_size).long()].long()
            assert (pages >= 0).all(), "attention reads a page that was given back"
            offs = (keys % page_size).long()
            k = cache[pages, 0, :, offs, :].float()   # [n, nkv, d]
            v = cache[pages, 1, :, offs, :].float()
            qt = q[t, : nq * d].view(nq, d).float()
            for h in range(nq):
                s = (k[:, h // group] @ qt[h]) * scale
                out[t, h * d:(h + 1) * d] = torch.softmax(s, dim=0) @ v[:, h // group]
        return out.to(q.dtype)

    def sample(self, logits, temperature, top_p, u, out=None):
        rows = logits.shape[0]
        given, out = out, torch.empty(rows, dtype=torch.int32)
        for i in range(rows):
            t = 0.0 if temperature is None else float(temperature[i])
            x = logits[i].double()
            if t <= 0:
                out[i] = int(torch.argmax(x))
                continue
            p = torch.softmax(x / t, dim=-1)
            sp, idx = torch.sort(p, descending=True)
            keep_sorted = ~((torch.cumsum(sp, 0) - sp) > float(top_p[i]))
            keep = torch.zeros_like(keep_sorted)
            keep[idx] = keep_sorted
            kept = torch.where(keep, p, torch.zeros_like(p))
            cdf = torch.cumsum(kept, 0)
            tok = int(torch.searchsorted(cdf, torch.tensor(float(u[i]) * float(cdf[-1]), dtype=cdf.dtype), right=True))
            out[i] = min(tok, int(torch.nonzero(keep)[-1]))
        if given is not None:
            given.copy_(out)
            return given
        return out.to(logits.device)

    def take_tokens(self, tokens, src, sampled):
        pick = src >= 0
        tokens[pick] = sampled[src[pick].long()]

    def token_logprobs(self, logits, tokens):
        lp = torch.log_softmax(logits.double(), dim=-1)
        return lp.gather(1, tokens.long().view(-1, 1)).view(-1).float()

    def bad_token_seen(self):
        return False

    # ------------------------------------------------------------------ operators of the recurrent and chunked mixers
    # (float64 inside, rounded once to the result's type; requests are walked one by one, tokens in order)
    def embed_scaled(self, ids, table, scale, positions, base):
        x = table[ids.long()].double() * scale
        if base:
            width = table.shape[1]
            i = torch.arange(width // 2, dtype=torch.float64)
            ang = positions.double()[:, None] * base ** (-2.0 * i / width)[None, :]
            x[:, 0::2] += torch.sin(ang)
            x[:, 1::2] += torch.cos(ang)
        return x.float()

    def softcap(self, logits, cap):
        logits.copy_((cap * torch.tanh(logits.double() / cap)).float())

    @staticmethod
    def _requests(ctx):
        qs = ctx.q_start.tolist()
        for r in range(ctx.num_requests):
            if qs[r + 1] > qs[r]:
                yield qs[r], qs[r + 1], int(ctx.state_slot[r]), int(ctx.positions[qs[r]])

    def causal_conv(self, x, column, channels, w, b, state, ctx, silu=True):
        taps = w.shape[1]
        out = torch.zeros((x.shape[0], channels), dtype=torch.float64)
        for lo, hi, slot, pos0 in self._requests(ctx):
            past = state[slot, :taps - 1].double().clone() if taps > 1 else torch.zeros((0, channels), dtype=torch.float64)
            for j in range(taps - 1):            # entry j is the input at position pos0 - (taps - 1) + j: nothing before position 0
                if pos0 - (taps - 1) + j < 0:
                    past[j] = 0
            seq = torch.cat([past, x[lo:hi, column:column + channels].double()], 0)
            for k in range(taps):
                out[lo:hi] += seq[k:k + hi - lo] * w[:, k].double()
            if taps > 1:
                state[slot, :taps - 1] = seq[-(taps - 1):].float()
        if b is not None:
            out += b.double()
        if silu:
            out = out * torch.sigmoid(out)
        return out.to(x.dtype)

    def selective_scan(self, xc, dt, dt_b, A, bc, D, xz, z_column, state, ctx):
        inner, n = A.shape
        y = torch.zeros((xc.shape[0], inner), dtype=torch.float64)
        step = torch.nn.functional.softplus(dt.double() + dt_b.double(), threshold=30.0)
        for lo, hi, slot, pos0 in self._requests(ctx):
            S = state[slot].double() if pos0 > 0 else torch.zeros((inner, n), dtype=torch.float64)
            for t in range(lo, hi):
                x = xc[t].double()
                S = torch.exp(step[t][:, None] * A.double()) * S + (step[t] * x)[:, None] * bc[t, :n].double()[None, :]
                y[t] = S @ bc[t, n:2 * n].double() + D.double() * x
            state[slot] = S.float()
        z = xz[:, z_column:z_column + inner].double()
        return (y * z * torch.sigmoid(z)).to(xc.dtype)

    @staticmethod
    def _page_views(cache, page, G, ps, d, dv):
        flat = cache[page].reshape(-1)
        return flat[:G * ps * d].view(G, ps, d), flat[G * ps * d:].view(G, ps, dv)

    def kv_write_normed(self, qkv, bias, slots, cache, H, G, d, dv, page_size, eps):
        for t in range(qkv.shape[0]):
            s = int(slots[t])
            if s < 0:
                continue
            row = qkv[t].double() + (bias.double() if bias is not None else 0.0)
            k = row[H * d:(H + G) * d].view(G, d)
            v = row[(H + G) * d:(H + G) * d + G * dv].view(G, dv)
            if eps > 0:
                v = v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)
            page, off = divmod(s, page_size)
            kp, vp = self._page_views(cache, page, G, page_size, d, dv)
            kp[:, off] = k.to(cache.dtype)
            vp[:, off] = v.to(cache.dtype)

    def chunk_attention(self, qkv, bias, cache, block_table, tok_req, positions, H, G, d, dv, page_size, scale, chunk,
                        r1, r2, talk, out, column, out_scale):
        group = H // G
        for t in range(qkv.shape[0]):
            r, p = int(tok_req[t]), int(positions[t])
            if r < 0:
                continue
            lo = p // chunk * chunk if chunk else 0
            keys = torch.arange(lo, p + 1)
            q = qkv[t, :H * d].double()
            if bias is not None:
                q = q + bias[:H * d].double()
            q = q.view(H, d)
            ks, vs = [], []
            for j in keys.tolist():
                page = int(block_table[r, j // page_size])
                assert page >= 0, "attention reads a page that was given back"
                kp, vp = self._page_views(cache, page, G, page_size, d, dv)
                ks.append(kp[:, j % page_size].double())
                vs.append(vp[:, j % page_size].double())
            k, v = torch.stack(ks), torch.stack(vs)                  # [n, G, d], [n, G, dv]
            w = torch.zeros((H, len(keys)), dtype=torch.float64)
            for h in range(H):
                sc = (k[:, h // group] @ q[h]) * scale
                if r1 is not None:
                    sc = sc - float(r1[h]) * torch.log1p(float(r2[h]) * (p - keys).double())
                w[h] = torch.softmax(sc, 0)
            if talk is not None:
                w = talk.double() @ w
            o = torch.stack([w[h] @ v[:, h // group] for h in range(H)]).reshape(-1) * out_scale
            out[t, column:column + H * dv] = o.to(out.dtype)

    def gated_delta_rule(self, qkv, ba, rate, dt_bias, S_all, ctx, H, G, d, dv, unit_eps, q_scale):
        T = qkv.shape[0]
        o = torch.zeros((T, H, dv), dtype=torch.float64)
        x = qkv.double()
        q = x[:, :G * d].view(T, G, d)
        k = x[:, G * d:2 * G * d].view(T, G, d)
        v = x[:, 2 * G * d:].view(T, H, dv)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) * q_scale
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
        beta = torch.sigmoid(ba[:, :H].double())
        decay = torch.exp(-rate.double() * torch.nn.functional.softplus(ba[:, H:].double() + dt_bias.double(), threshold=30.0))
        for lo, hi, slot, pos0 in self._requests(ctx):
            S = S_all[slot].double() if pos0 > 0 else torch.zeros((H, d, dv), dtype=torch.float64)
            for t in range(lo, hi):
                for h in range(H):
                    c = h // (H // G)
                    Sh = decay[t, h] * S[h]
                    u = beta[t, h] * (v[t, h] - Sh.T @ k[t, c])
                    S[h] = Sh + torch.outer(k[t, c], u)
                    o[t, h] = S[h].T @ q[t, c]
            S_all[slot] = S.float()
        return o.reshape(T, H * dv).float()

    def gated_head_norm(self, o, weight, eps, gate, gate_column, H, dv, out, column, scale, gate_kind="silu", weight_per_head=False):
        T = o.shape[0]
        x = o.double().view(T, H, dv)
        x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (weight.double().view(H, dv) if weight_per_head else weight.double())
        g = gate[:, gate_column:gate_column + H * dv].double()
        g = torch.sigmoid(g) if gate_kind == "sigmoid" else g * torch.sigmoid(g)
        out[:, column:column + H * dv] = (x.reshape(T, H * dv) * g * scale).to(out.dtype)

    def clamped_glu(self, gu, bias, limit, alpha, up_shift):
        inter = gu.shape[1] // 2
        x = gu.double() + (bias.double() if bias is not None else 0.0)
        g = torch.clamp(x[:, :inter], max=limit)
        u = torch.clamp(x[:, inter:], -limit, limit)
        return (g * torch.sigmoid(alpha * g) * (u + up_shift)).to(gu.dtype)

    def token_side(self, residual, x, bias, tokens, table, column, dim, w_gate, w_proj, norm_w, eps):
        s = residual.double()
        if x is not None:
            s = s + x.double()
        if bias is not None:
            s = s + bias.double()
        e = table[tokens.long(), column:column + dim].double()
        z = s @ w_gate.double().T
        g = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))) * e
        y = g @ w_proj.double().T
        s = s + y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * norm_w.double()
        residual.copy_(s.float())

    # ------------------------------------------------------------------ operators of the Lilenex parts
    def stream_mix_norm(self, streams, init, y, mix, out, read, weight, eps, n_streams, rows, dtype):
        if streams is None:
            streams = init.float()[:, None, :].repeat(1, n_streams, 1).contiguous()
        new = streams.double()
        if y is not None:
            new = torch.einsum("st,nsw->ntw", mix.double(), new) + out.double()[None, :, None] * y.double()[:, None, :]
        if rows is None:
            streams.copy_(new.float())
        else:
            new = new[rows.long()]
        u = torch.einsum("s,nsw->nw", read.double(), new)
        normed = u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps) * weight.double()
        return normed.to(dtype), streams

    def qk_norm_rotate_store(self, proj, H, G, d, dv, q_norm, k_norm, eps, positions, freq, dims, amplitude, slots, cache, page_size):
        T = proj.shape[0]
        x = proj.double()
        q, k = x[:, :H * d], x[:, H * d:(H + G) * d]
        if eps > 0:
            q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * q_norm.double()
            if G:
                k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps) * k_norm.double()
        qk = torch.cat([q, k], dim=1).view(T, H + G, d).clone()
        if freq is not None and dims > 0:
            ang = positions.double()[:, None] * freq.double()[None, :dims // 2]
            c, s = (ang.cos() * amplitude)[:, None, :], (ang.sin() * amplitude)[:, None, :]
            a, b = qk[..., 0:dims:2].clone(), qk[..., 1:dims:2].clone()
            qk[..., 0:dims:2] = a * c - b * s
            qk[..., 1:dims:2] = b * c + a * s
        proj[:, :(H + G) * d] = qk.reshape(T, -1).to(proj.dtype)
        if G and cache is not None:
            for t in range(T):
                sl = int(slots[t])
                if sl < 0:
                    continue
                page, off = divmod(sl, page_size)
                kp, vp = self._page_views(cache, page, G, page_size, d, dv)
                kp[:, off] = proj[t, H * d:(H + G) * d].view(G, d)
                vp[:, off] = proj[t, (H + G) * d:(H + G) * d + G * dv].view(G, dv)

    def window_attention(self, q, cache, block_table, tok_req, positions, H, G, d, dv, page_size, scale, window=0, keep_first=0,
                         splits=1, hints=None, sink=False, temp_coef=0.0, temp_every=1, shared_values=False, distance_bias=0.0,
                         gate_column=-1, pool=0, summary=None, summary_table=None):
        T = q.shape[0]
        out = torch.zeros((T, H * dv), dtype=torch.float64)
        group = H // G
        for t in range(T):
            r, p = int(tok_req[t]), int(positions[t])
            if r < 0:
                continue
            keys = [j for j in range(p + 1) if not window or p - j < window or j < keep_first]
            ks, vs = [], []
            n_blocks = max(0, (p - window + 1) // pool) if pool and window else 0     # blocks that lie wholly behind the window
            for b in range(n_blocks):
                page = int(summary_table[r, b // page_size])
                assert page >= 0, "attention reads a page of block means that is not held"
                kp, vp = self._page_views(summary, page, G, page_size, d, dv)
                ks.append(kp[:, b % page_size].double())
                vs.append(vp[:, b % page_size].double())
            for j in keys:
                page = int(block_table[r, j // page_size])
                assert page >= 0, "attention reads a page that was given back"
                if shared_values:           # a page holds keys only; a key's first dv entries are its value
                    kp = cache[page].view(G, page_size, d)
                    vp = kp[..., :dv]
                else:
                    kp, vp = self._page_views(cache, page, G, page_size, d, dv)
                ks.append(kp[:, j % page_size].double())
                vs.append(vp[:, j % page_size].double())
            k, v = torch.stack(ks), torch.stack(vs)
            qt = q[t, :H * d].double().view(H, d)
            temp = 1.0 + temp_coef * math.log((p + 1) // temp_every + 1.0) if temp_coef else 1.0
            dist = torch.tensor([0.0] * n_blocks + [float(p - j) for j in keys], dtype=torch.float64)
            for h in range(H):
                sc = (k[:, h // group] @ qt[h]) * scale * temp
                if distance_bias:
                    sc = sc - 2.0 ** (-distance_bias * (h + 1) / H) * dist
                if sink:
                    m = max(float(sc.max()), 0.0)
                    ex = torch.exp(sc - m)
                    w = ex / (ex.sum() + math.exp(-m))
                else:
                    w = torch.softmax(sc, 0)
                out[t, h * dv:(h + 1) * dv] = w @ v[:, h // group]
        if gate_column >= 0:
            out = out * torch.sigmoid(q[:, gate_column:gate_column + H * dv].double())
        return out.to(q.dtype)

    def head_norm_rotate_store(self, proj, H, G, d, dv, q_norm, k_norm, eps, positions, inv_freq, rot, slots, cache, page_size):
        """proj [T, q | k | v | ...] in place: every q and k head divided by its own root mean square and multiplied by
        the weight [d] of its kind (eps > 0), entries i and i + rot/2 turned by position * inv_freq[i]; k, v to the cache."""
        T = proj.shape[0]
        qk = proj[:, :(H + G) * d].double().view(T, H + G, d).clone()
        if eps > 0:
            qk = qk / torch.sqrt((qk * qk).mean(-1, keepdim=True) + eps)
            qk[:, :H] = qk[:, :H] * q_norm.double()
            if G:
                qk[:, H:] = qk[:, H:] * k_norm.double()
        if inv_freq is not None and rot > 0:
            half = rot // 2
            ang = positions.double()[:, None] * inv_freq.double()[None, :half]
            c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
            a, b = qk[..., :half].clone(), qk[..., half:rot].clone()
            qk[..., :half] = a * c - b * s
            qk[..., half:rot] = b * c + a * s
        proj[:, :(H + G) * d] = qk.reshape(T, -1).to(proj.dtype)
        if G and cache is not None:
            for t in range(T):
                sl = int(slots[t])
                if sl < 0:
                    continue
                page, off = divmod(sl, page_size)
                kp, vp = self._page_views(cache, page, G, page_size, d, dv)
                kp[:, off] = proj[t, H * d:(H + G) * d].view(G, d)
                vp[:, off] = proj[t, (H + G) * d:(H + G) * d + G * dv].view(G, dv)

    def pool_blocks(self, cache, block_table, tok_req, positions, summary_slots, summary, G, d, dv, page_size, block):
        """For every token with a slot in the pages of block means: the mean key and mean value of the ``block``
        positions that end with the token's own, read from the cache."""
        for t in range(positions.shape[0]):
            sl, r, p = int(summary_slots[t]), int(tok_req[t]), int(positions[t])
            if sl < 0 or r < 0:
                continue
            ks, vs = [], []
            for j in range(p - block + 1, p + 1):
                page = int(block_table[r, j // page_size])
                assert page >= 0, "a block's mean reads a page that was given back"
                kp, vp = self._page_views(cache, page, G, page_size, d, dv)
                ks.append(kp[:, j % page_size].double())
                vs.append(vp[:, j % page_size].double())
            kp, vp = self._page_views(summary, sl // page_size, G, page_size, d, dv)
            kp[:, sl % page_size] = torch.stack(ks).mean(0).to(summary.dtype)
            vp[:, sl % page_size] = torch.stack(vs).mean(0).to(summary.dtype)

    def mean_of_normed(self, members, eps, dtype):
        total = 0.0
        for x, w in members:
            x = x.double()
            total = total + x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()
        return (total / len(members)).to(dtype)

    def post_norm_add(self, outs, weights, post_weight, eps, residual, dtype=None, results=None, index=0, coeffs=None,
                      next_weight=None):
        """u = outs[0], or with ``weights`` the mean over m of rmsnorm(outs[m]) * weights[m];  X = residual + rmsnorm(u) *
        post_weight.  With ``results`` [n, T, W]: results[index] = X and the stream becomes sum_{j <= index} coeffs[j] *
        results[j], else the stream is X.  The stream is written over ``residual``.  Returns (rmsnorm(stream) * next_weight
        in ``dtype`` or None, residual)."""
        unit = lambda x: x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
        if weights is None:
            u = outs[0].double()
        else:
            u = sum(unit(o.double()) * w.double() for o, w in zip(outs, weights)) / len(outs)
        X = residual.double() + unit(u) * post_weight.double()
        if results is not None:
            results[index] = X.float()
            X = sum(coeffs[j].double() * results[j].double() for j in range(index)) + coeffs[index].double() * X
        residual.copy_(X.float())
        y = (unit(X) * next_weight.double()).to(dtype) if next_weight is not None else None
        return y, residual

    def gla_scan(self, proj, z, bias, inv_tau, S_all, ctx, H, d, dv, q_scale, head_decay=None, k_scale=1.0):
        T = proj.shape[0]
        x = proj.double()
        q = x[:, :H * d].view(T, H, d) * q_scale
        k = x[:, H * d:2 * H * d].view(T, H, d) * k_scale
        v = x[:, 2 * H * d:2 * H * d + H * dv].view(T, H, dv)
        if head_decay is not None:          # one fixed decay per head
            decay = head_decay.double()[None, :, None].expand(T, H, d)
        else:
            decay = torch.exp(torch.nn.functional.logsigmoid(z.double() + bias.double()) * inv_tau).view(T, H, d)
        o = torch.zeros((T, H, dv), dtype=torch.float64)
        for lo, hi, slot, pos0 in self._requests(ctx):
            S = S_all[slot].double() if pos0 > 0 else torch.zeros((H, d, dv), dtype=torch.float64)
            for t in range(lo, hi):
                S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
                o[t] = torch.einsum("hde,hd->he", S, q[t])
            S_all[slot] = S.float()
        return o.reshape(T, H * dv).float()

    def gelu_tanh(self, x):
        z = x.double()
        return (0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))).to(x.dtype)

    def routed_experts(self, x, logits, w_gate_up, w_down, top, scale_input, shared, score="sigmoid", groups=1, keep_groups=1,
                       renormalise=False):
        T = x.shape[0]
        E = logits.shape[1]
        inter = w_gate_up.shape[1] // 2
        score = torch.softmax(logits.double(), dim=-1) if score == "softmax" else torch.sigmoid(logits.double())
        out = torch.zeros((T, w_down.shape[1]), dtype=torch.float64)
        for t in range(T):
            allowed = score[t].clone()
            if groups > 1 and keep_groups < groups:
                best = score[t].view(groups, E // groups).max(dim=1).values
                kept = set(best.topk(keep_groups).indices.tolist())
                for e in range(E):
                    if e // (E // groups) not in kept:
                        allowed[e] = -1.0
            chosen = allowed.topk(top).indices.tolist()
            total = sum(score[t, e] for e in chosen) + 1e-20 if renormalise else 1.0
            for e in chosen:
                w = score[t, e] / total
                u = (x[t].double() * w).to(x.dtype).double() if scale_input else x[t].double()
                gu = w_gate_up[e].double() @ u
                g, up = gu[:inter], gu[inter:]
                y = w_down[e].double() @ (g * torch.sigmoid(g) * up)
                out[t] += y if scale_input else w * y
        if shared is not None:
            out += shared.double()
        return out.float()

    # ------------------------------------------------------------------ operators of the Sogalix parts
    def add_layernorm(self, x, residual, weight, bias, eps, rows=None, dtype=None, add_bias=None, keep_sum=True):
        dtype = dtype or x.dtype
        s = None
        if residual is not None:
            s = residual.double()
        if x is not None:
            s = x.double() if s is None else s + x.double()
        if add_bias is not None:
            s = s + add_bias.double()
        if rows is not None:
            s = s[rows.long()]
        mu = s.mean(-1, keepdim=True)
        var = ((s - mu) ** 2).mean(-1, keepdim=True)
        y = ((s - mu) / torch.sqrt(var + eps) * weight.double() + bias.double()).to(dtype)
        if rows is not None or not keep_sum:
            return y, None
        if residual is not None:
            residual.copy_(s.float())
            return y, residual
        return y, s.float()

    def lowrank_tanh_linear(self, aw, column, w2):
        return (torch.tanh(aw[:, column:].double()) @ w2.double().T).float()

    def general_delta_scan(self, proj, aw, a_bias, z, w_bias, decay_limit, S_all, ctx, H, d, unit_eps):
        T, n = proj.shape[0], H * d
        x = proj.double()
        r, k, v = (x[:, i * n:(i + 1) * n].view(T, H, d) for i in range(3))
        a = torch.sigmoid(aw[:, :n].double() + a_bias.double()).view(T, H, d)
        w = torch.exp(-decay_limit * torch.sigmoid(z.double() + w_bias.double())).view(T, H, d)
        u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
        o = torch.zeros((T, H, d), dtype=torch.float64)
        for lo, hi, slot, pos0 in self._requests(ctx):
            S = S_all[slot].double() if pos0 > 0 else torch.zeros((H, d, d), dtype=torch.float64)
            for t in range(lo, hi):
                uS = torch.einsum("hc,hce->he", u[t], S)
                S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
                o[t] = torch.einsum("hce,hc->he", S, r[t])
            S_all[slot] = S.float()
        return o.reshape(T, n).float()

    def xielu(self, x, pos_factor, neg_factor):
        z = x.double()
        neg = z.clamp(max=0)
        return torch.where(z > 0, pos_factor * z * z + 0.5 * z, neg_factor * (torch.expm1(neg) - neg) + 0.5 * z).to(x.dtype)

    def latent_attention(self, q, cache, block_table, ctx, H, R, n, page_size, scale):
        """Every head's causal softmax over the kept rows [latent | rotated key part]; the latent is the value."""
        return self.window_attention(q, cache, block_table, ctx.tok_req, ctx.positions, H, 1, R + n, R, page_size, scale,
                                     shared_values=True)

    def latent_norm_store(self, proj, Q, q_norm, R, kv_norm, n, eps, positions, freq, dims, slots, cache, page_size):
        x = proj.double()
        unit = lambda t: t / torch.sqrt((t * t).mean(-1, keepdim=True) + eps)
        cq = (unit(x[:, :Q]) * q_norm.double()).to(proj.dtype)
        if R:
            c = unit(x[:, Q:Q + R]) * kv_norm.double()
            kr = x[:, Q + R:Q + R + n].clone()
            ang = (positions.float()[:, None] * freq.float()[None, :dims // 2]).double()   # the angle is a float32 product
            a, b = kr[:, 0:dims:2].clone(), kr[:, 1:dims:2].clone()
            kr[:, 0:dims:2] = a * ang.cos() - b * ang.sin()
            kr[:, 1:dims:2] = b * ang.cos() + a * ang.sin()
            row = torch.cat([c, kr], dim=1).to(cache.dtype)
            for t in range(proj.shape[0]):
                sl = int(slots[t])
                if sl >= 0:
                    page, off = divmod(sl, page_size)
                    cache[page].view(page_size, R + n)[off] = row[t]
        return cq

    def head_linear(self, x, x_ld, x_col, w, out, out_ld, out_col, H, gate=None, gate_column=0):
        T = x.shape[0]
        n_out, n_in = w.shape[1], w.shape[2]
        xs = x.double().view(T, H, x_ld)[:, :, x_col:x_col + n_in]
        y = torch.einsum("thi,hoi->tho", xs, w.double())
        if gate is not None:
            y = y * torch.sigmoid(gate[:, gate_column:gate_column + H].double())[:, :, None]
        out.view(T, H, out_ld)[:, :, out_col:out_col + n_out] = y.to(out.dtype)

    def rotate_head_part(self, x, x_ld, x_col, out, out_ld, out_col, H, n, positions, freq, dims):
        T = x.shape[0]
        part = x.double().view(T, H, x_ld)[:, :, x_col:x_col + n].clone()
        ang = (positions.float()[:, None] * freq.float()[None, :dims // 2]).double()   # the angle is a float32 product
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        a, b = part[..., 0:dims:2].clone(), part[..., 1:dims:2].clone()
        part[..., 0:dims:2] = a * c - b * s
        part[..., 1:dims:2] = b * c + a * s
        out.view(T, H, out_ld)[:, :, out_col:out_col + n] = part.to(out.dtype)
