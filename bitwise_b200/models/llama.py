"""Llama / SmolLM2 assembled from parts, and its entry in the architecture registry.

Every layer is a pre-norm block of grouped-query attention with rotary positions and a
dense SwiGLU feed-forward (src/model.cpp:279-306); tensors carry the Hugging Face names
the reference reads (src/model.cpp:136-171): ``model.embed_tokens.weight``,
``model.layers.N.{input_layernorm,post_attention_layernorm}.weight``,
``model.layers.N.self_attn.{q,k,v,o}_proj.weight``,
``model.layers.N.mlp.{gate,up,down}_proj.weight``, ``model.norm.weight`` and
``lm_head.weight`` unless the embeddings are tied.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..parts.attention import GQAAttention
from ..parts.block import PreNormBlock
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.mlp import SwiGLU
from ..parts.norm import RMSNorm
from ..parts.rope import RotaryEncoding
from .decoder import DecoderModel

LLAMA_BLOCK_NAMES = {"mixer_norm": "input_layernorm", "mixer": "self_attn",
                     "ffn_norm": "post_attention_layernorm", "feed_forward": "mlp"}


def build_llama(config: LlamaConfig) -> DecoderModel:
    c = config
    rotary = RotaryEncoding(c.head_dim, c.rope_theta, c.rope_scaling)
    embedding = TokenEmbedding(c.vocab_size, c.hidden_size)
    blocks = []
    for _ in range(c.num_hidden_layers):
        blocks.append(PreNormBlock(
            c.hidden_size,
            mixer=GQAAttention(c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
                               position=rotary, window=None),
            feed_forward=SwiGLU(c.hidden_size, c.intermediate_size),
            mixer_norm=RMSNorm(c.hidden_size, c.rms_norm_eps),
            ffn_norm=RMSNorm(c.hidden_size, c.rms_norm_eps),
            names=LLAMA_BLOCK_NAMES))
    head = OutputHead(c.vocab_size, c.hidden_size, RMSNorm(c.hidden_size, c.rms_norm_eps),
                      tied_to=embedding if c.tie_word_embeddings else None)
    return DecoderModel(c, embedding, blocks, head, position_encodings=[rotary])


register_architecture("LlamaForCausalLM", LlamaConfig.from_json, build_llama)
