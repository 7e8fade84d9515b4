"""Plain PyTorch versions of the engine's kernels, one function per kernel, float32 arithmetic.

Two uses, both in tests only: each CUDA kernel is compared with its function here, and the
engine's host-side logic (runner, cache, scheduler) is exercised on the CPU with this object in
place of the CUDA kernel set. The product path never imports this file.
"""

from __future__ import annotations

import numpy as np
import torch


def philox4x32_10(c, k0, k1):
    """Philox4x32-10 on numpy uint32 arrays c[4]; returns 4 arrays."""
    c = [np.asarray(x, dtype=np.uint64) for x in c]
    k0 = np.uint64(k0)
    k1 = np.uint64(k1)
    m0, m1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = m0 * c[0]
        p1 = m1 * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c = [(hi1 ^ c[1] ^ k0) & mask, lo1, (hi0 ^ c[3] ^ k1) & mask, lo0]
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return c


class PlainOps:
    name = "plain-torch"

    def __init__(self, q_tile: int = 32) -> None:
        self.q_tile = q_tile
        self.launches = 0
        self.accumulate = True  # add into the residual stream where a part offers it

    # ------------------------------------------------------------------ capabilities
    def branch_dtype(self, dtype):
        return torch.float32

    def check_attention_shape(self, head_dim, dtype, num_heads=None, num_kv_heads=None):
        if head_dim % 16:
            raise ValueError("head size must be a multiple of 16")

    # ------------------------------------------------------------------ pointwise
    def embedding(self, token_ids, table):
        return table[token_ids.long()].float()

    def add_rmsnorm(self, x, residual, weight, eps, out_dtype, rows=None):
        if rows is not None:
            v = x[rows.long()]
            if residual is not None:
                v = v + residual[rows.long()].float()
        else:
            if residual is not None:
                x += residual.float()
            v = x
        y = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight
        return y.to(out_dtype)

    def silu_mul(self, gu, out_dtype=None):
        g, u = gu.float().chunk(2, dim=-1)
        return (g / (1 + torch.exp(-g)) * u).to(out_dtype or gu.dtype)

    def linear(self, a, w, bias=None, out_dtype=None, accumulate_into=None):
        y = a.float() @ w.float().T
        if bias is not None:
            y = y + bias.float()
        if accumulate_into is not None and self.accumulate:
            accumulate_into += y
            return None
        return y.to(out_dtype or a.dtype)

    def gated_silu(self, h, w, bias=None, out_dtype=None):
        return self.silu_mul(self.linear(h, w, bias, out_dtype=torch.float32), out_dtype=out_dtype or h.dtype)

    # ------------------------------------------------------------------ attention
    def project_rope_kv_write(self, h, w, bias, *, out_dtype=None, **kw):
        qkv = self.linear(h, w, bias, out_dtype=torch.float32)
        return self.rope_kv_write(qkv, out_dtype=out_dtype or h.dtype, **kw)

    def project_attend(self, h, w, bias, *, num_heads, num_kv_heads, head_dim, scale, window, positions,
                       token_seq, cos, sin, k_pages, v_pages, writes, block_tables, page_tokens, step,
                       plan, out_dtype=None):
        q = self.project_rope_kv_write(
            h, w, bias, out_dtype=out_dtype, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
            positions=positions, token_seq=token_seq, cos=cos, sin=sin, k_pages=k_pages if writes else None,
            v_pages=v_pages if writes else None, block_tables=block_tables, page_tokens=page_tokens)
        return self.paged_attention(
            q, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, scale=scale, window=window,
            k_pages=k_pages, v_pages=v_pages, block_tables=block_tables, page_tokens=page_tokens, step=step,
            plan=plan)

    def rope_kv_write(self, qkv, *, num_heads, num_kv_heads, head_dim, positions, token_seq,
                      cos, sin, k_pages, v_pages, block_tables, page_tokens, out_dtype=None):
        T, D = qkv.shape[0], head_dim
        out_dtype = out_dtype or qkv.dtype
        heads = qkv.view(T, num_heads + 2 * num_kv_heads, D)
        pos = positions.long()
        rot = heads[:, : num_heads + num_kv_heads].float()
        if cos is not None:
            c, s = cos[pos][:, None, :], sin[pos][:, None, :]
            x1, x2 = rot[..., : D // 2], rot[..., D // 2 :]
            rot = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
        if k_pages is not None:
            page = block_tables[token_seq.long(), pos // page_tokens].long()
            off = pos % page_tokens
            k_pages[page, :, off] = rot[:, num_heads:].to(out_dtype)
            v_pages[page, :, off] = heads[:, num_heads + num_kv_heads :].to(out_dtype)
        if out_dtype == qkv.dtype:
            heads[:, :num_heads] = rot[:, :num_heads].to(qkv.dtype)
            return qkv[:, : num_heads * D]
        return rot[:, :num_heads].to(out_dtype).reshape(T, num_heads * D)

    def attention_q_tile(self, dtype, head_dim):
        return self.q_tile

    def attention_plan(self, host_step, dtype, head_dim):
        tiles, decode = [], []
        for s, n in enumerate(host_step.q_lens.tolist()):
            if n == 1:
                decode.append(s)
            else:
                tiles.extend((s, q0) for q0 in range(0, n, self.q_tile))
        return {
            "tiles": np.asarray(tiles, dtype=np.int32).reshape(-1, 2),
            "decode_seqs": np.asarray(decode, dtype=np.int32),
        }

    def paged_attention(self, q, *, num_heads, num_kv_heads, head_dim, scale, window, k_pages,
                        v_pages, block_tables, page_tokens, step, plan=None):
        T, D = q.shape[0], head_dim
        qkv = q
        q = q[:, : num_heads * D].float().reshape(T, num_heads, D)
        out = torch.zeros(T, num_heads, D)
        cu = step.cu_q.tolist()
        ctx = step.ctx_lens.tolist()
        group = num_heads // num_kv_heads
        for s in range(len(ctx)):
            a, b = cu[s], cu[s + 1]
            n = b - a
            j = torch.arange(ctx[s])
            pages = block_tables[s, j // page_tokens].long()
            k = k_pages[pages, :, j % page_tokens].float().repeat_interleave(group, dim=1)
            v = v_pages[pages, :, j % page_tokens].float().repeat_interleave(group, dim=1)
            qpos = torch.arange(ctx[s] - n, ctx[s])[:, None]
            visible = j[None, :] <= qpos
            if window > 0:
                visible &= (qpos - j[None, :]) < window
            sc = torch.einsum("thd,shd->hts", q[a:b], k) * scale
            sc = sc.masked_fill(~visible, float("-inf"))
            out[a:b] = torch.einsum("hts,shd->thd", sc.softmax(-1), v)
        return out.view(T, num_heads * D).to(qkv.dtype)

    # ------------------------------------------------------------------ sampling
    def sample(self, logits, temperature, top_k, top_p, min_p, seed, draw, kinds=3):
        R, V = logits.shape
        out = torch.empty(R, dtype=torch.int32)
        for r in range(R):
            t = float(temperature[r])
            row = logits[r].float()
            if t < 1e-5:
                out[r] = int(row.argmax())
                continue
            z = row * np.float32(1.0 / np.float32(t))
            zmax = z.max()
            p = torch.exp(z - zmax)
            keep = torch.ones(V, dtype=torch.bool)
            k, tp, mp = int(top_k[r]), float(top_p[r]), float(min_p[r])
            if (0 < k < V) or tp < 1.0:
                gt = z[None, :] > z[:, None]  # gt[i, j]: z_j above z_i
                count = gt.sum(1)
                mass = (gt * p[None, :]).sum(1)
                if 0 < k < V:
                    keep &= count < k
                keep &= mass < np.float32(tp) * p.sum()
            if mp > 0:
                keep &= z >= zmax + np.log(np.float32(mp))
            sd = int(seed[r]) & 0xFFFFFFFFFFFFFFFF
            quads = np.arange((V + 3) // 4, dtype=np.uint32)
            c = philox4x32_10(
                [quads, np.full_like(quads, int(draw[r])), np.zeros_like(quads), np.zeros_like(quads)],
                sd & 0xFFFFFFFF, sd >> 32,
            )
            bits = np.stack(c, axis=1).reshape(-1)[:V].astype(np.uint32)
            u = ((bits >> 8).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
            score = z - torch.from_numpy(np.log(-np.log(u))).float()
            score[~keep] = float("-inf")
            out[r] = int(score.argmax())
        return out

    def sample_sorted(self, logits, temperature, top_k, top_p, min_p, seed, draw):
        """The same rule as :meth:`sample` with a sort instead of the all-pairs comparison, for
        vocabularies too large for a V x V matrix. An element's strictly-above count and mass are
        those of the first element of its group of equal values in descending order; masses are
        summed in float64."""
        R, V = logits.shape
        out = torch.empty(R, dtype=torch.int32)
        for r in range(R):
            t = float(temperature[r])
            row = logits[r].float()
            if t < 1e-5:
                out[r] = int(row.argmax())
                continue
            z = row * np.float32(1.0 / np.float32(t))
            zmax = z.max()
            p = torch.exp(z - zmax).double()
            keep = torch.ones(V, dtype=torch.bool)
            k, tp, mp = int(top_k[r]), float(top_p[r]), float(min_p[r])
            if (0 < k < V) or tp < 1.0:
                zs, order = torch.sort(z, descending=True, stable=True)
                ps = p[order]
                excl = torch.cumsum(ps, 0) - ps  # mass before each sorted position
                first = torch.ones(V, dtype=torch.bool)
                first[1:] = zs[1:] != zs[:-1]
                start = torch.cummax(torch.where(first, torch.arange(V), torch.zeros(V, dtype=torch.long)), 0).values
                count, mass = start, excl[start]
                ks = torch.ones(V, dtype=torch.bool)
                if 0 < k < V:
                    ks &= count < k
                ks &= mass < float(np.float32(tp)) * float(p.sum())
                keep[order] = ks
            if mp > 0:
                keep &= z >= zmax + np.log(np.float32(mp))
            sd = int(seed[r]) & 0xFFFFFFFFFFFFFFFF
            quads = np.arange((V + 3) // 4, dtype=np.uint32)
            c = philox4x32_10(
                [quads, np.full_like(quads, int(draw[r])), np.zeros_like(quads), np.zeros_like(quads)],
                sd & 0xFFFFFFFF, sd >> 32,
            )
            bits = np.stack(c, axis=1).reshape(-1)[:V].astype(np.uint32)
            u = ((bits >> 8).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
            score = z - torch.from_numpy(np.log(-np.log(u))).float()
            score[~keep] = float("-inf")
            out[r] = int(score.argmax())
        return out

    def logsumexp(self, logits):
        return torch.logsumexp(logits.float(), dim=-1)

    def apply_penalties(self, logits, row, token, count, presence, frequency, repetition):
        for i in range(row.shape[0]):
            r, t = int(row[i]), int(token[i])
            v = float(logits[r, t])
            if int(count[i]) > 0:
                v -= float(frequency[i]) * int(count[i]) + float(presence[i])
            rp = float(repetition[i])
            if rp != 1.0:
                v = v / rp if v > 0 else v * rp
            logits[r, t] = v

    PROMPT_BIT = 1 << 30

    def token_state_add(self, state, slot, token, in_prompt):
        for s_, t, f in zip(slot.tolist(), token.tolist(), in_prompt.tolist()):
            if f:
                state[s_, t] |= self.PROMPT_BIT
            else:
                state[s_, t] += 1

    def apply_penalties_dense(self, logits, row, slot, presence, frequency, repetition, state):
        for j in range(row.shape[0]):
            r, st = int(row[j]), state[int(slot[j])]
            for t in torch.nonzero(st).flatten().tolist():
                v = float(logits[r, t])
                c = int(st[t]) & (self.PROMPT_BIT - 1)
                if c > 0:
                    v -= float(frequency[j]) * c + float(presence[j])
                rp = float(repetition[j])
                if rp != 1.0:
                    v = v / rp if v > 0 else v * rp
                logits[r, t] = v

    def ban_tokens(self, logits, row, token):
        logits[row.long(), token.long()] = float("-inf")
