"""Toy parts and a toy architecture, defined in the tests and registered from outside the
package: a mixer with a state of its own, a feed-forward with routing, an additive position
encoding, and a model description that mixes them with the package's own parts, runs a layer
twice, and lets a run read another run's cache.  They exist to show that the framework takes
new parts without a change to its files; they are not models of anyone's.

`plain_toy_logits` is the whole-sequence oracle for the toy architecture.
"""

from __future__ import annotations

import dataclasses

import torch

from inference_engine_b200.config import register_architecture
from inference_engine_b200.config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from inference_engine_b200.parts import (
    FeedForward, Mixer, PositionEncoding, StateRequest, WeightDecl, register_part,
)
from tests import plain_llama as P


# --- a mixer with state of its own: s_t = decay * s_{t-1} + x_t W_in ; out_t = s_t W_out --------


class ToyStateMixer(Mixer):
    def __init__(self, prefix: str, hidden: int, width: int) -> None:
        self.prefix, self.hidden, self.width = prefix, hidden, width

    @classmethod
    def from_spec(cls, params, env, **_):
        return cls(params["prefix"], env.hidden_size, params["width"])

    def weights(self):
        return {f"{self.prefix}.w_in": WeightDecl((self.width, self.hidden)),
                f"{self.prefix}.w_out": WeightDecl((self.hidden, self.width)),
                f"{self.prefix}.decay": WeightDecl((self.width,), "vector", "ones")}

    def bind(self, tensors, env):
        self.w_in = tensors[f"{self.prefix}.w_in"].float()
        self.w_out = tensors[f"{self.prefix}.w_out"].float()
        self.decay = torch.sigmoid(tensors[f"{self.prefix}.decay"].float())

    def cache_request(self):
        return StateRequest((self.width,))

    def forward(self, x, ctx, binding):
        group = ctx.groups[binding.group]
        state = group.state[binding.slot]  # [slots, width]
        u = x.float() @ self.w_in.t()
        out = torch.empty(x.shape[0], self.hidden, dtype=torch.float32, device=x.device)
        for start, n, slot in zip(ctx.q_starts, ctx.q_lens, group.slots_host):
            s = state[slot].clone()
            for t in range(start, start + n):  # tokens of a request strictly in order
                s = self.decay * s + u[t]
                out[t] = s @ self.w_out.t()
            state[slot] = s
        return out


# --- a feed-forward with routing: the better of two small experts per token ---------------------


class ToyRoutedFeedForward(FeedForward):
    def __init__(self, prefix: str, hidden: int, inter: int, experts: int) -> None:
        self.prefix, self.hidden, self.inter, self.experts = prefix, hidden, inter, experts

    @classmethod
    def from_spec(cls, params, env, **_):
        return cls(params["prefix"], env.hidden_size, params["intermediate_size"], params["experts"])

    def weights(self):
        w = {f"{self.prefix}.router": WeightDecl((self.experts, self.hidden))}
        for e in range(self.experts):
            w[f"{self.prefix}.experts.{e}.up"] = WeightDecl((self.inter, self.hidden))
            w[f"{self.prefix}.experts.{e}.down"] = WeightDecl((self.hidden, self.inter))
        return w

    def bind(self, tensors, env):
        self.t = {k: v.float() for k, v in tensors.items()}

    def forward(self, x, ctx):
        x = x.float()
        choice = (x @ self.t[f"{self.prefix}.router"].t()).argmax(-1)  # router logits in 32-bit
        out = torch.zeros(x.shape[0], self.hidden, dtype=torch.float32, device=x.device)
        for e in range(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                h = torch.relu(x[rows] @ self.t[f"{self.prefix}.experts.{e}.up"].t())
                out[rows] = h @ self.t[f"{self.prefix}.experts.{e}.down"].t()
        return out


# --- an additive position encoding: a learned vector per position, added after the embedding ----


class ToyLearnedPositions(PositionEncoding):
    def __init__(self, name: str, hidden: int, positions: int) -> None:
        self.name, self.hidden, self.positions = name, hidden, positions

    @classmethod
    def from_spec(cls, params, env, **_):
        return cls(params["weight"], env.hidden_size, params["positions"])

    def weights(self):
        return {self.name: WeightDecl((self.positions, self.hidden), "table")}

    def bind(self, tensors, env):
        self.table = tensors[self.name].float()

    def apply_to_embedding(self, h, ctx):
        h.add_(self.table[ctx.positions.long()])


def register_toys() -> None:
    register_part("mixer", "toy_state", ToyStateMixer, replace=True)
    register_part("feed_forward", "toy_routed", ToyRoutedFeedForward, replace=True)
    register_part("position", "toy_learned", ToyLearnedPositions, replace=True)
    register_architecture("ToyHybridForTests", ToyConfig, toy_spec, replace=True)
    register_architecture("ToyTwoAttentionsForTests", TwoAttentionsConfig, two_attentions_spec, replace=True)


# --- the toy architecture -----------------------------------------------------------------------


@dataclasses.dataclass(frozen=True)
class ToyConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    state_width: int
    window: int
    eps: float
    max_position_embeddings: int

    @classmethod
    def from_dict(cls, raw):
        return cls(raw["architectures"][0], **{f.name: raw[f.name] for f in dataclasses.fields(cls)[1:]})


TOY_CONFIG = {
    "architectures": ["ToyHybridForTests"], "vocab_size": 97, "hidden_size": 48, "num_heads": 6,
    "num_kv_heads": 2, "head_dim": 16, "intermediate_size": 40, "state_width": 24, "window": 11,
    "eps": 1e-5, "max_position_embeddings": 128,
}


def _attention_layer(cfg: ToyConfig, p: str, window, ffn: PartSpec) -> LayerSpec:
    return LayerSpec(
        prefix=p, block=PartSpec("prenorm_residual"),
        mixer=PartSpec("paged_attention", {
            "q_proj": f"{p}.q", "k_proj": f"{p}.k", "v_proj": f"{p}.v", "o_proj": f"{p}.o",
            "num_heads": cfg.num_heads, "num_kv_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
            "position": "rotary", "window": window}),
        feed_forward=ffn,
        norms={"pre_mixer": PartSpec("rms", {"weight": f"{p}.n1", "eps": cfg.eps}),
               "pre_feed_forward": PartSpec("rms", {"weight": f"{p}.n2", "eps": cfg.eps})})


def toy_spec(cfg: ToyConfig) -> ModelSpec:
    swiglu = lambda p: PartSpec("swiglu", {  # noqa: E731
        "gate_proj": f"{p}.gate", "up_proj": f"{p}.up", "down_proj": f"{p}.down",
        "intermediate_size": cfg.intermediate_size})
    layers = (
        _attention_layer(cfg, "l0", None, swiglu("l0")),
        LayerSpec(prefix="l1", block=PartSpec("prenorm_residual"),
                  mixer=PartSpec("toy_state", {"prefix": "l1.mix", "width": cfg.state_width}),
                  feed_forward=PartSpec("toy_routed", {"prefix": "l1.moe", "experts": 2,
                                                        "intermediate_size": cfg.intermediate_size}),
                  norms={"pre_mixer": PartSpec("rms", {"weight": "l1.n1", "eps": cfg.eps}),
                         "pre_feed_forward": PartSpec("rms", {"weight": "l1.n2", "eps": cfg.eps})}),
        _attention_layer(cfg, "l2", cfg.window, swiglu("l2")),
    )
    # layer 1 runs twice (each run has a state of its own); the last run of layer 0 reads the
    # keys and values that its first run cached and writes none
    schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(1),
                ScheduleEntry(0, cache_from=0))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding=PartSpec("token", {"weight": "embed", "vocab_size": cfg.vocab_size}),
        positions={"rotary": PartSpec("rotary", {"rotary_dim": cfg.head_dim, "theta": 10000.0}),
                   "learned": PartSpec("toy_learned", {"weight": "pos", "positions": cfg.max_position_embeddings})},
        layers=layers, schedule=schedule,
        final_norm=PartSpec("rms", {"weight": "norm", "eps": cfg.eps}),
        head=PartSpec("linear", {"weight": "head", "vocab_size": cfg.vocab_size}))


def toy_weights(seed: int = 0) -> dict:
    from inference_engine_b200.config import build_model_spec, config_from_dict
    from inference_engine_b200.engine.model import declared_weights

    register_toys()
    decl = declared_weights(build_model_spec(config_from_dict(TOY_CONFIG)))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, d in decl.items():
        t = torch.randn(d.shape, generator=g) * 0.08
        if name.endswith((".n1", ".n2")) or name == "norm":
            t = t + 1.0
        if name.endswith((".q", ".k")):
            t = t * 3.0
        out[name] = t.to(torch.bfloat16)
    return out


# --- the whole-sequence oracle of the toy architecture ------------------------------------------


def plain_toy_logits(weights: dict, ids: list[int]) -> torch.Tensor:
    c = TOY_CONFIG
    w = {k: v.float() for k, v in weights.items()}
    t = len(ids)
    x = w["embed"][torch.tensor(ids)] + w["pos"][:t]
    inv = 1.0 / (10000.0 ** (torch.arange(0, c["head_dim"], 2).float() / c["head_dim"]))
    cos, sin = P.rope_angles(inv, torch.arange(t))
    nh, nkv, hd = c["num_heads"], c["num_kv_heads"], c["head_dim"]
    kept = {}

    def attn_layer(x, p, window, reuse=None):
        z = P.rms_norm(x, w[f"{p}.n1"], c["eps"])
        q = P.apply_rope((z @ w[f"{p}.q"].t()).view(t, nh, hd).transpose(0, 1), cos, sin)
        if reuse is None:
            k = P.apply_rope((z @ w[f"{p}.k"].t()).view(t, nkv, hd).transpose(0, 1), cos, sin)
            v = (z @ w[f"{p}.v"].t()).view(t, nkv, hd).transpose(0, 1)
            kept[p] = (k, v)
        else:
            k, v = kept[reuse]
        h = x + P.attention(q, k, v, window).transpose(0, 1).reshape(t, nh * hd) @ w[f"{p}.o"].t()
        z = P.rms_norm(h, w[f"{p}.n2"], c["eps"])
        act = z @ w[f"{p}.gate"].t()
        act = act / (1 + torch.exp(-act)) * (z @ w[f"{p}.up"].t())
        return h + act @ w[f"{p}.down"].t()

    def state_layer(x):
        z = P.rms_norm(x, w["l1.n1"], c["eps"])
        u = z @ w["l1.mix.w_in"].t()
        decay = torch.sigmoid(w["l1.mix.decay"])
        s = torch.zeros(c["state_width"])
        rows = []
        for i in range(t):
            s = decay * s + u[i]
            rows.append(s @ w["l1.mix.w_out"].t())
        h = x + torch.stack(rows)
        z = P.rms_norm(h, w["l1.n2"], c["eps"])
        choice = (z @ w["l1.moe.router"].t()).argmax(-1)
        out = torch.zeros_like(h)
        for e in range(2):
            rows_e = (choice == e).nonzero().flatten()
            out[rows_e] = torch.relu(z[rows_e] @ w[f"l1.moe.experts.{e}.up"].t()) @ w[f"l1.moe.experts.{e}.down"].t()
        return h + out

    x = attn_layer(x, "l0", None)
    x = state_layer(x)
    x = attn_layer(x, "l2", c["window"])
    x = state_layer(x)
    x = attn_layer(x, "l0", None, reuse="l0")
    return P.rms_norm(x, w["norm"], c["eps"]) @ w["head"].t()


# --- a second toy: two attention groups of different head size, one of them windowed ------------
# (no state of its own, so decode steps can be captured and launched ahead)


@dataclasses.dataclass(frozen=True)
class TwoAttentionsConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    wide: tuple  # (query heads, key/value heads, head size) of the layer that sees everything
    narrow: tuple  # the same for the layer that sees a window
    window: int
    eps: float
    max_position_embeddings: int

    @classmethod
    def from_dict(cls, raw):
        values = {f.name: raw[f.name] for f in dataclasses.fields(cls)[1:]}
        values["wide"], values["narrow"] = tuple(values["wide"]), tuple(values["narrow"])
        return cls(raw["architectures"][0], **values)


TWO_ATTENTIONS_CONFIG = {
    "architectures": ["ToyTwoAttentionsForTests"], "vocab_size": 113, "hidden_size": 48,
    "intermediate_size": 56, "wide": [6, 2, 16], "narrow": [2, 1, 32], "window": 11, "eps": 1e-5,
    "max_position_embeddings": 256,
}


def two_attentions_spec(cfg: TwoAttentionsConfig) -> ModelSpec:
    def layer(p, shape, position, window):
        nh, nkv, hd = shape
        return LayerSpec(
            prefix=p, block=PartSpec("prenorm_residual"),
            mixer=PartSpec("paged_attention", {
                "q_proj": f"{p}.q", "k_proj": f"{p}.k", "v_proj": f"{p}.v", "o_proj": f"{p}.o",
                "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "position": position, "window": window}),
            feed_forward=PartSpec("swiglu", {"gate_proj": f"{p}.gate", "up_proj": f"{p}.up",
                                             "down_proj": f"{p}.down",
                                             "intermediate_size": cfg.intermediate_size}),
            norms={"pre_mixer": PartSpec("rms", {"weight": f"{p}.n1", "eps": cfg.eps}),
                   "pre_feed_forward": PartSpec("rms", {"weight": f"{p}.n2", "eps": cfg.eps})})

    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        max_position_embeddings=cfg.max_position_embeddings,
        embedding=PartSpec("token", {"weight": "embed", "vocab_size": cfg.vocab_size}),
        positions={"rotary_wide": PartSpec("rotary", {"rotary_dim": cfg.wide[2], "theta": 10000.0}),
                   "rotary_narrow": PartSpec("rotary", {"rotary_dim": cfg.narrow[2], "theta": 3000.0})},
        layers=(layer("a", cfg.wide, "rotary_wide", None), layer("b", cfg.narrow, "rotary_narrow", cfg.window)),
        schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)),  # the wide layer runs twice
        final_norm=PartSpec("rms", {"weight": "norm", "eps": cfg.eps}),
        head=PartSpec("linear", {"weight": None, "vocab_size": cfg.vocab_size}))


def two_attentions_weights(seed: int = 0) -> dict:
    from inference_engine_b200.config import build_model_spec, config_from_dict
    from inference_engine_b200.engine.model import declared_weights

    register_toys()
    decl = declared_weights(build_model_spec(config_from_dict(TWO_ATTENTIONS_CONFIG)))
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, d in decl.items():
        t = torch.randn(d.shape, generator=g) * 0.08
        if name.endswith((".n1", ".n2")) or name == "norm":
            t = t + 1.0
        if name.endswith((".q", ".k")):
            t = t * 3.0
        out[name] = t.to(torch.bfloat16)
    return out


def plain_two_attentions_logits(weights: dict, ids: list[int]) -> torch.Tensor:
    c = TWO_ATTENTIONS_CONFIG
    w = {k: v.float() for k, v in weights.items()}
    t = len(ids)
    x = w["embed"][torch.tensor(ids)]

    def layer(x, p, shape, theta, window):
        nh, nkv, hd = shape
        inv = 1.0 / (theta ** (torch.arange(0, hd, 2).float() / hd))
        cos, sin = P.rope_angles(inv, torch.arange(t))
        z = P.rms_norm(x, w[f"{p}.n1"], c["eps"])
        q = P.apply_rope((z @ w[f"{p}.q"].t()).view(t, nh, hd).transpose(0, 1), cos, sin)
        k = P.apply_rope((z @ w[f"{p}.k"].t()).view(t, nkv, hd).transpose(0, 1), cos, sin)
        v = (z @ w[f"{p}.v"].t()).view(t, nkv, hd).transpose(0, 1)
        h = x + P.attention(q, k, v, window).transpose(0, 1).reshape(t, nh * hd) @ w[f"{p}.o"].t()
        z = P.rms_norm(h, w[f"{p}.n2"], c["eps"])
        act = z @ w[f"{p}.gate"].t()
        act = act / (1 + torch.exp(-act)) * (z @ w[f"{p}.up"].t())
        return h + act @ w[f"{p}.down"].t()

    x = layer(x, "a", c["wide"], 10000.0, None)
    x = layer(x, "b", c["narrow"], 3000.0, c["window"])
    x = layer(x, "a", c["wide"], 10000.0, None)
    return P.rms_norm(x, w["norm"], c["eps"]) @ w["embed"].t()
