"""A toy architecture defined in the tests, to show that the framework takes other parts
without a change to its files: a mixer with state of its own (one slot per request), a
feed-forward with routing, a learned position table, windowed attention beside full
attention, a run order that names a layer twice and lets a run read another run's cache.
It is no model of anyone's; it exists for the tests only.  Its parts use torch operations
(they work on the CPU stand-in and on a GPU alike); the framework's own parts use kernels.

``plain_forward`` computes the same model over a whole sequence with the plain
implementation's functions and numpy, without any cache.
"""
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

import plain_llama as P
from bitwise_b200.config import register_architecture
from bitwise_b200.models.decoder import DecoderModel, LayerRun
from bitwise_b200.parts import (FeedForward, GQAAttention, Mixer, OutputHead, PositionEncoding, PreNormBlock, RMSNorm,
                                RotaryEncoding, SlotStateNeed, SwiGLU, TokenEmbedding, register_feed_forward,
                                register_mixer)
from bitwise_b200.weights import KEEP32, MATRIX, ParamSpec

NAMES = {"mixer_norm": "norm_a", "mixer": "mix", "ffn_norm": "norm_b", "feed_forward": "ff"}


@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int = 97
    hidden_size: int = 48
    heads: int = 3
    kv_heads: int = 1
    head_dim: int = 16
    intermediate_size: int = 40
    window: int = 24
    max_positions: int = 160
    eps: float = 1e-5
    # per layer: (mixer kind, feed-forward kind)
    layers: Tuple[Tuple[str, str], ...] = (("window_attention", "swiglu"), ("running_state", "routed"),
                                           ("attention", "swiglu"))
    # run order: (layer, cache entry, owns the entry)
    schedule: Tuple[Tuple[int, int, bool], ...] = ((0, 0, True), (1, 1, True), (2, 2, True), (1, 3, True),
                                                   (2, 2, False))
    architectures: Tuple[str, ...] = ("ToyMixForCausalLM",)
    tie_word_embeddings: bool = True
    eos_token_id: int = -1

    @staticmethod
    def from_json(d):
        return ToyConfig(**{k: (tuple(tuple(x) for x in v) if k in ("layers", "schedule") else
                                tuple(v) if k == "architectures" else v)
                            for k, v in d.items() if k in ToyConfig.__dataclass_fields__})

    def to_json(self):
        d = {k: getattr(self, k) for k in self.__dataclass_fields__}
        d["layers"] = [list(x) for x in self.layers]
        d["schedule"] = [list(x) for x in self.schedule]
        d["architectures"] = list(self.architectures)
        return d


class RunningState(Mixer):
    """state_t = sigmoid(a) * state_{t-1} + xn_t;  x_t += state_t * g.  The state is one
    vector per request, kept in the request's slot between steps."""

    def __init__(self, width):
        self.width = width
        self.a = self.g = None

    def cache_need(self):
        return SlotStateNeed((self.width,), torch.float32)

    def param_specs(self, prefix):
        return [ParamSpec(prefix + ".a", (self.width,), KEEP32), ParamSpec(prefix + ".g", (self.width,), KEEP32)]

    def load_params(self, state, prefix):
        self.a, self.g = state[prefix + ".a"], state[prefix + ".g"]

    def param_bytes(self):
        return 8 * self.width

    def forward(self, ctx, xn, x, cache):
        decay = torch.sigmoid(self.a * 50.0)
        for (r0, cnt), p0, slot in zip(ctx.host_seq_rows, ctx.host_seq_pos0, ctx.host_seq_slot):
            st = cache.state[slot]
            if p0 == 0:
                st.zero_()
            for r in range(r0, r0 + cnt):
                st.mul_(decay).add_(xn[r].float())
                x[r] += st * (self.g * 50.0)


class RoutedFFN(FeedForward):
    """Two experts, the one with the larger router logit (computed in 32-bit) takes the row:
    x += relu(xn W1_e^T) W2_e^T."""

    def __init__(self, width, inner):
        self.width, self.inner = width, inner
        self.router = self.w1 = self.w2 = None

    def param_specs(self, prefix):
        return [ParamSpec(prefix + ".router", (2, self.width), KEEP32),
                ParamSpec(prefix + ".w1", (2 * self.inner, self.width), MATRIX),
                ParamSpec(prefix + ".w2", (2 * self.width, self.inner), MATRIX)]

    def load_params(self, state, prefix):
        self.router, self.w1, self.w2 = state[prefix + ".router"], state[prefix + ".w1"], state[prefix + ".w2"]

    def forward(self, ctx, xn, x):
        xf = xn.float()
        choice = (xf @ self.router.t()).argmax(-1)
        for e in range(2):
            rows = (choice == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            w1 = self.w1[e * self.inner:(e + 1) * self.inner].float()
            w2 = self.w2[e * self.width:(e + 1) * self.width].float()
            x[rows] += torch.relu(xf[rows] @ w1.t()) @ w2.t()


class LearnedPositions(PositionEncoding):
    """x_t += table[position_t], added to the stream after the token embedding."""

    def __init__(self, positions, width):
        self.positions, self.width = positions, width
        self.table = None

    def param_specs(self, prefix):
        return [ParamSpec(prefix + ".positions.weight", (self.positions, self.width), KEEP32)]

    def load_params(self, state, prefix):
        self.table = state[prefix + ".positions.weight"]

    def param_bytes(self):
        return self.table.numel() * self.table.element_size()

    def on_embed(self, ctx, x):
        x += self.table[ctx.pos.long()]


def build_toy(c: ToyConfig) -> DecoderModel:
    rotary = RotaryEncoding(c.head_dim, 10000.0)
    learned = LearnedPositions(c.max_positions, c.hidden_size)
    emb = TokenEmbedding(c.vocab_size, c.hidden_size)
    blocks = []
    for mixer_kind, ff_kind in c.layers:
        if mixer_kind == "running_state":
            mixer = RunningState(c.hidden_size)
        else:
            mixer = GQAAttention(c.hidden_size, c.heads, c.kv_heads, c.head_dim, position=rotary,
                                 window=c.window if mixer_kind == "window_attention" else None)
        ff = RoutedFFN(c.hidden_size, c.intermediate_size) if ff_kind == "routed" else SwiGLU(c.hidden_size,
                                                                                               c.intermediate_size)
        blocks.append(PreNormBlock(c.hidden_size, mixer, ff, RMSNorm(c.hidden_size, c.eps),
                                   RMSNorm(c.hidden_size, c.eps), NAMES))
    head = OutputHead(c.vocab_size, c.hidden_size, RMSNorm(c.hidden_size, c.eps), tied_to=emb)
    # the decoder declares and loads the parameters of its position encodings itself
    return DecoderModel(c, emb, blocks, head, schedule=[LayerRun(*s) for s in c.schedule],
                        position_encodings=[rotary, learned])


def register():
    register_mixer("running_state", RunningState)
    register_feed_forward("routed", RoutedFFN)
    register_architecture("ToyMixForCausalLM", ToyConfig.from_json, build_toy)


# ----------------------------------------------------------------------------------------
# plain, whole-sequence forward of the same model

def plain_forward(folder, tokens, exp="det"):
    import json
    import os
    c = ToyConfig.from_json(json.load(open(os.path.join(folder, "config.json"))))
    w = P.read_safetensors(os.path.join(folder, "model.safetensors"))
    T = len(tokens)
    pos = np.arange(T)
    f32 = np.float32
    inv = P.rope_inv_freq(c.head_dim, 10000.0)
    x = (w["model.embed_tokens.weight"][np.asarray(tokens)] + w["model.positions.weight"][pos]).astype(f32)
    caches = {}
    for layer, entry, owns in c.schedule:
        pre = f"model.layers.{layer}."
        kind, ff = c.layers[layer]
        xn = P.rmsnorm(x, w[pre + "norm_a.weight"], c.eps)
        if kind == "running_state":
            decay = 1.0 / (1.0 + np.exp(-(w[pre + "mix.a"].astype(np.float64) * 50.0)))
            st = np.zeros(c.hidden_size, dtype=np.float64)
            out = np.zeros_like(x)
            for t in range(T):
                st = (st * decay).astype(f32).astype(np.float64) + xn[t]
                st = st.astype(f32).astype(np.float64)
                out[t] = (st * (w[pre + "mix.g"] * f32(50.0))).astype(f32)
            x = (x + out).astype(f32)
        else:
            q = P.rope(P.linear(xn, w[pre + "mix.q_proj.weight"]).reshape(T, c.heads, c.head_dim), pos, inv)
            if owns:
                k = P.rope(P.linear(xn, w[pre + "mix.k_proj.weight"]).reshape(T, c.kv_heads, c.head_dim), pos, inv)
                v = P.linear(xn, w[pre + "mix.v_proj.weight"]).reshape(T, c.kv_heads, c.head_dim)
                caches[entry] = (k, v)
            k, v = caches[entry]
            a = P.attention(q, k, v, exp, window=c.window if kind == "window_attention" else 0)
            x = (x + P.linear(a.reshape(T, -1), w[pre + "mix.o_proj.weight"])).astype(f32)
        xn = P.rmsnorm(x, w[pre + "norm_b.weight"], c.eps)
        if ff == "routed":
            choice = (xn.astype(np.float64) @ w[pre + "ff.router"].astype(np.float64).T).argmax(-1)
            out = np.zeros_like(x)
            for t in range(T):
                e = int(choice[t])
                w1 = w[pre + "ff.w1"][e * c.intermediate_size:(e + 1) * c.intermediate_size]
                w2 = w[pre + "ff.w2"][e * c.hidden_size:(e + 1) * c.hidden_size]
                out[t] = np.maximum(xn[t] @ w1.T, 0) @ w2.T
            x = (x + out).astype(f32)
        else:
            gu = np.concatenate([P.linear(xn, w[pre + "ff.gate_proj.weight"]), P.linear(xn, w[pre + "ff.up_proj.weight"])], 1)
            x = (x + P.linear(P.swiglu(gu, c.intermediate_size, exp), w[pre + "ff.down_proj.weight"])).astype(f32)
    xn = P.rmsnorm(x, w["model.norm.weight"], c.eps)
    return P.linear(xn, w["model.embed_tokens.weight"])
