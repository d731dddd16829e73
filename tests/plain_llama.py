"""A plain, slow Llama: whole sequences, no cache, 32-bit, one function per part.

Written from the formulas of the reference (AashutoshR/inference-engine); every function
cites the file and lines it restates.  It shares no code with the package: it reads the
``config.json`` dictionary and a name -> tensor dictionary directly.  It is the oracle the
engine is compared with; ``tests/golden/make_golden.py`` compares this file once with the
reference's own model code on the CPU and stores the outputs next to it.
"""

from __future__ import annotations

import math

import torch

# The precision everything is computed in.  32-bit is what the engine is compared with;
# `in_float64()` switches to 64-bit for the duration of a block, to measure how far 32-bit
# arithmetic itself is from the exact result at a given size.
PRECISION = torch.float32


class in_float64:
    def __enter__(self):
        global PRECISION
        self.saved, PRECISION = PRECISION, torch.float64

    def __exit__(self, *exc):
        global PRECISION
        PRECISION = self.saved


def _f(t: torch.Tensor) -> torch.Tensor:
    return t.to(PRECISION)


def embed(weights: dict, token_ids: torch.Tensor) -> torch.Tensor:
    """engine/model/llama.py:25,61 -- rows of the table, no scaling."""
    return _f(weights["model.embed_tokens.weight"])[token_ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """engine/model/layers.py:41-43 -- x * rsqrt(mean(x^2) + eps), then times weight."""
    x = _f(x)
    normed = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return _f(weight) * normed


def rope_inv_freq(cfg: dict) -> torch.Tensor:
    """engine/model/layers.py:55-73 -- theta^(-2j/d), then the llama3 band scaling."""
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    theta = float(cfg.get("rope_theta", 10000.0))
    inv_freq = 1.0 / (theta ** (_f(torch.arange(0, hd, 2, dtype=torch.int64)) / hd))
    s = cfg.get("rope_scaling")
    if not s:
        return inv_freq
    factor = float(s["factor"])
    low_f = float(s.get("low_freq_factor", 1.0))
    high_f = float(s.get("high_freq_factor", 4.0))
    orig = float(s.get("original_max_position_embeddings", 8192))
    low_wavelen = orig / low_f
    high_wavelen = orig / high_f
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (orig / wavelen - low_f) / (high_f - low_f)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    is_medium = ~(wavelen < high_wavelen) & ~(wavelen > low_wavelen)
    return torch.where(is_medium, smoothed, scaled)


def rope_angles(inv_freq: torch.Tensor, positions: torch.Tensor):
    """engine/model/layers.py:75-79 -- cos and sin of position * inv_freq, halves repeated."""
    freqs = _f(positions[:, None]) * _f(inv_freq)[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """engine/model/layers.py:91-93."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """engine/model/layers.py:82-88 -- x: [heads, T, hd]; cos, sin: [T, hd]."""
    return x * cos[None] + rotate_half(x) * sin[None]


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None):
    """engine/model/layers.py:159-169 with the causal mask of layers.py:110-112 -- q: [nh, T,
    hd]; k, v: [nkv, T, hd]; query head h uses key/value head h // (nh // nkv); scores are
    scaled by hd^-0.5 (engine/kernels/paged_attention.py:161); a query sees the keys at its
    own and earlier positions (the latest ``window`` of them when one is given)."""
    nh, t, hd = q.shape
    groups = nh // k.shape[0]
    k = k.repeat_interleave(groups, dim=0)
    v = v.repeat_interleave(groups, dim=0)
    scores = q @ k.transpose(1, 2) * hd ** -0.5
    qi = torch.arange(t)[:, None]
    ki = torch.arange(t)[None, :]
    mask = ki <= qi
    if window:
        mask = mask & (ki > qi - window)
    scores = scores.masked_fill(~mask[None], float("-inf"))
    return scores.softmax(-1) @ v  # [nh, T, hd]


def attention_block(cfg: dict, weights: dict, prefix: str, x: torch.Tensor, cos, sin):
    """engine/model/layers.py:171-189 (projections, rotation) and :169 (output projection)."""
    t = x.shape[0]
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    q = (x @ _f(weights[f"{prefix}.q_proj.weight"]).t()).view(t, nh, hd).transpose(0, 1)
    k = (x @ _f(weights[f"{prefix}.k_proj.weight"]).t()).view(t, nkv, hd).transpose(0, 1)
    v = (x @ _f(weights[f"{prefix}.v_proj.weight"]).t()).view(t, nkv, hd).transpose(0, 1)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    out = attention(q, k, v).transpose(0, 1).reshape(t, nh * hd)
    return out @ _f(weights[f"{prefix}.o_proj.weight"]).t()


def swiglu(weights: dict, prefix: str, x: torch.Tensor) -> torch.Tensor:
    """engine/model/layers.py:277-281 -- down(silu(gate(x)) * up(x)), silu(g) = g / (1 + e^-g)."""
    gate = x @ _f(weights[f"{prefix}.gate_proj.weight"]).t()
    up = x @ _f(weights[f"{prefix}.up_proj.weight"]).t()
    act = gate / (1 + torch.exp(-gate)) * up
    return act @ _f(weights[f"{prefix}.down_proj.weight"]).t()


def decoder_layer(cfg: dict, weights: dict, i: int, x: torch.Tensor, cos, sin) -> torch.Tensor:
    """engine/model/layers.py:301-303 -- pre-norm, two residual adds."""
    p = f"model.layers.{i}"
    eps = float(cfg.get("rms_norm_eps", 1e-5))
    h = x + attention_block(cfg, weights, f"{p}.self_attn",
                            rms_norm(x, weights[f"{p}.input_layernorm.weight"], eps), cos, sin)
    return h + swiglu(weights, f"{p}.mlp",
                      rms_norm(h, weights[f"{p}.post_attention_layernorm.weight"], eps))


def logits_for(cfg: dict, weights: dict, token_ids, rows=None) -> torch.Tensor:
    """engine/model/llama.py:60-68 -- embed, the layers in order, final norm, head; the head
    is the embedding table when ``tie_word_embeddings`` is set (engine/model/loader.py:91-92).
    token_ids: one whole sequence -> [T, vocab] 32-bit logits for every position (or for the
    positions listed in ``rows`` only: the head of a large vocabulary is the slow part)."""
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.shape[0])
    cos, sin = rope_angles(rope_inv_freq(cfg), positions)
    x = embed(weights, ids)
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(cfg, weights, i, x, cos, sin)
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long)]
    x = rms_norm(x, weights["model.norm.weight"], float(cfg.get("rms_norm_eps", 1e-5)))
    head = "model.embed_tokens.weight" if cfg.get("tie_word_embeddings", False) else "lm_head.weight"
    return x @ _f(weights[head]).t()


def greedy_generate(cfg: dict, weights: dict, prompt: list[int], max_tokens: int,
                    stop_ids=()) -> list[int]:
    """Recompute the whole sequence for every new token and take the argmax
    (engine/runtime/sampler.py:25-26); a stop id is returned as the last token
    (engine/runtime/stop.py:62-66)."""
    ids, out = list(prompt), []
    for _ in range(max_tokens):
        token = int(logits_for(cfg, weights, ids)[-1].argmax())
        out.append(token)
        ids.append(token)
        if token in stop_ids:
            break
    return out
