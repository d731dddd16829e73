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
        if delta is not None and delta.dim() == 3:  # the parts of a split matrix product
            delta = delta.sum(0)
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

    def linear(self, x, w, out=None, *, ws=None, tag="linear", out_dtype=None, allow_split=False):
        if out is None:
            out = ws.buffer(tag, x.shape[0], w.shape[0], out_dtype)
        out.copy_((x.float() @ w.float().t()).to(out.dtype))
        return out

    def rope_kv_write(self, qkv, positions, table, rotary_dim, q_out, k_cache, v_cache,
                      slot_mapping, nh, nkv, hd, page_size):
        if qkv.dim() == 3:
            qkv = qkv.sum(0)
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
                        scale, window, out, ragged=None):
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

    def silu_mul(self, gate_up, out, interleave=0):
        if gate_up.dim() == 3:
            gate_up = gate_up.float().sum(0)
        i = out.shape[1]
        if interleave:  # gates and ups alternate in blocks of `interleave` values
            blocks = gate_up.float().view(gate_up.shape[0], i // interleave, 2, interleave)
            g, u = blocks[:, :, 0].reshape(-1, i), blocks[:, :, 1].reshape(-1, i)
        else:
            g, u = gate_up[:, :i].float(), gate_up[:, i:].float()
        out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))

    def gated_linear(self, x, w_gate_up, interleave, *, ws, tag="ffn", out_dtype=None):
        gate_up = self.linear(x, w_gate_up, ws=ws, tag=tag + ".gate_up", out_dtype=out_dtype or x.dtype)
        act = ws.buffer(tag + ".act", x.shape[0], w_gate_up.shape[0] // 2, out_dtype or x.dtype)
        self.silu_mul(gate_up, act, interleave)
        return act

    def argmax(self, logits, out):
        out.copy_(logits.argmax(-1).to(out.dtype))

    def check_errors(self):
        return None


# --- sampling -----------------------------------------------------------------------------------


def philox_uniforms(seed: int, draw: int, n: int):
    """The uniforms the sampling kernel uses for entries 0..n-1 of a row: Philox4x32-10 with
    counter (i // 4, draw low, draw high, 0) and key (seed low, seed high); entry i takes word
    i % 4; u = ((word >> 9) + 0.5) / 2^23."""
    import numpy as np

    mask = np.uint64(0xFFFFFFFF)
    i = np.arange(n, dtype=np.uint64)
    c0 = i >> np.uint64(2)
    c1 = np.full(n, draw & 0xFFFFFFFF, dtype=np.uint64)
    c2 = np.full(n, (draw >> 32) & 0xFFFFFFFF, dtype=np.uint64)
    c3 = np.zeros(n, dtype=np.uint64)
    k0, k1 = np.uint64(seed & 0xFFFFFFFF), np.uint64((seed >> 32) & 0xFFFFFFFF)
    m0, m1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    for _ in range(10):
        p0, p1 = m0 * c0, m1 * c2
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & mask, lo1, (hi0 ^ c3 ^ k1) & mask, lo0
        k0, k1 = (k0 + np.uint64(0x9E3779B9)) & mask, (k1 + np.uint64(0xBB67AE85)) & mask
    words = np.stack([c0, c1, c2, c3], axis=1)[np.arange(n), (i & np.uint64(3)).astype(np.int64)]
    return ((words >> np.uint64(9)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)


def _sample_row(row, temperature, top_k, top_p, min_p, penalty, seen, seed, draw):
    z = row.float().clone()
    if penalty != 1.0 and seen is not None:
        idx = seen.nonzero().flatten()
        z[idx] = torch.where(z[idx] > 0, z[idx] / penalty, z[idx] * penalty)
    if not temperature > 0:
        return int(z.argmax()), None
    z = z * (torch.tensor(1.0) / torch.tensor(temperature, dtype=torch.float32))
    zmax = z.max()
    keep_min = torch.tensor(float("-inf"))
    if 0 < top_k < z.numel():
        keep_min = torch.maximum(keep_min, z.topk(top_k).values[-1])
    if top_p < 1.0:
        kept = z[z >= keep_min].sort(descending=True).values
        mass = torch.exp(kept - zmax)
        target = max(top_p - 1e-6, 0.0) * float(mass.sum())
        first = int((mass.cumsum(0) >= target).nonzero()[0]) if target > 0 else 0
        keep_min = torch.maximum(keep_min, kept[first])
    if min_p > 0.0:
        keep_min = torch.maximum(keep_min, zmax + torch.log(torch.tensor(min_p, dtype=torch.float32)))
    u = torch.from_numpy(philox_uniforms(seed, draw, z.numel()))
    score = z - torch.log(-torch.log(u))
    score[z < keep_min] = float("-inf")
    return int(score.argmax()), score


def _ref_sample(self, logits, out, temperature=None, top_k=None, top_p=None, min_p=None,
                penalty=None, seen_bits=None, seeds=None, draws=None, logprob=None):
    logits_c = logits.float().cpu()
    rows, vocab = logits_c.shape

    def get(t, r, default):
        return default if t is None else t[r].item()

    for r in range(rows):
        seen = None
        if seen_bits is not None:
            words = seen_bits[r].cpu().to(torch.int64) & 0xFFFFFFFF
            seen = ((words[:, None] >> torch.arange(32)[None, :]) & 1).reshape(-1)[:vocab].bool()
        token, _ = _sample_row(logits_c[r], get(temperature, r, 0.0), int(get(top_k, r, 0)),
                               get(top_p, r, 1.0), get(min_p, r, 0.0), get(penalty, r, 1.0), seen,
                               int(get(seeds, r, 0)), int(get(draws, r, 0)))
        out[r] = token
        if logprob is not None:
            logprob[r] = logits_c[r].log_softmax(-1)[token]


RefOps.sample = _ref_sample
