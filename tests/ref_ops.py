"""Plain PyTorch versions of every kernel, with the kernels' own signatures.

Two uses: each CUDA kernel is compared with the function of the same name here, and tests
that exercise the engine's logic without a GPU (cache, step function, scheduler) run the
engine on these instead of the CUDA kernels.  Nothing in the package imports this file.
All arithmetic is 32-bit; results are rounded once to the output's dtype.
"""

from __future__ import annotations

import torch


class RefOps:
    name = "torch-reference"

    def embedding(self, table, ids, out):
        out.copy_(table[ids.long()].float())

    def rmsnorm(self, h, delta, weight, eps, out, rows=None):
        if rows is None:
            if delta is not None:
                h.add_(delta)
            x = h
        else:
            x = h[rows.long()]
            if delta is not None:
                x = x + delta[rows.long()]
        normed = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        out.copy_((weight * normed).to(out.dtype))

    def linear(self, x, w, out):
        out.copy_((x.float() @ w.float().t()).to(out.dtype))

    def rope_kv_write(self, qkv, positions, table, rotary_dim, q_out, k_cache, v_cache,
                      slot_mapping, nh, nkv, hd, page_size):
        n = qkv.shape[0]
        q = qkv[:, : nh * hd].reshape(n, nh, hd).float()
        k = qkv[:, nh * hd: (nh + nkv) * hd].reshape(n, nkv, hd).float()
        v = qkv[:, (nh + nkv) * hd:].reshape(n, nkv, hd).float()
        if table is not None and rotary_dim > 0:
            half = rotary_dim // 2
            cos = table[positions.long(), 0][:, None, :]  # [n, 1, half]
            sin = table[positions.long(), 1][:, None, :]

            def rot(x):
                x1, x2, rest = x[..., :half], x[..., half:rotary_dim], x[..., rotary_dim:]
                return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin, rest), dim=-1)

            q, k = rot(q), rot(k)
        q_out.copy_(q.reshape(n, nh * hd).to(q_out.dtype))
        if slot_mapping is not None:
            slots = slot_mapping.long()
            page, offset = slots // page_size, slots % page_size
            k_cache[page, :, offset] = k.to(k_cache.dtype)
            v_cache[page, :, offset] = v.to(v_cache.dtype)

    def paged_attention(self, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, page_size,
                        scale, window, out):
        groups = nh // nkv
        tables = block_tables.long().cpu()
        positions = ctx.positions.cpu().tolist()
        seqs = ctx.seq_of_token.cpu().tolist()
        for t in range(ctx.num_tokens):
            p, s = positions[t], seqs[t]
            lo = max(0, p - window + 1) if window else 0
            keys = torch.arange(lo, p + 1)
            pages = tables[s][keys // page_size].to(k_cache.device)
            offs = (keys % page_size).to(k_cache.device)
            k = k_cache[pages, :, offs].float()  # [keys, nkv, hd]
            v = v_cache[pages, :, offs].float()
            k = k.repeat_interleave(groups, dim=1)
            v = v.repeat_interleave(groups, dim=1)
            qt = q[t].reshape(nh, hd).float()
            scores = torch.einsum("hd,khd->hk", qt, k) * scale
            probs = scores.softmax(-1)
            out[t] = torch.einsum("hk,khd->hd", probs, v).reshape(nh * hd).to(out.dtype)

    def silu_mul(self, gate_up, out):
        i = out.shape[1]
        g, u = gate_up[:, :i].float(), gate_up[:, i:].float()
        out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))

    def argmax(self, logits, out):
        out.copy_(logits.argmax(-1).to(out.dtype))

    def check_errors(self):
        return None
