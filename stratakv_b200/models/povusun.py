"""The Povusun decoder as a list of parts.

Embedding ``embed`` (also the output head).  Every layer ``l<i>`` norms its sublayers on both sides:
``x += norm1b(mixer(norm1(x)))``, then, if it has a feed-forward, ``x += norm2b(mlp(norm2(x)))``, then, if the model
has a per-layer token input, ``x += rmsnorm(side.proj(gelu_tanh(side.gate x) * side.embed[token, layer's part]))``.
Three mixers, chosen per layer:

* ``attention``: grouped-query attention without a rotation; queries and keys divided by their root mean square per
  head, a query temperature that grows with the position, capped scores, a sigmoid gate (``mix.g``) on every output
  number; a layer may use the keys and values of an earlier layer (``kv_from``) and then has no ``mix.k``/``mix.v``;
* ``latent_attention``: attention over one compressed vector per position (``mix.dkv``, ``mix.dkv.norm``, ``mix.uk``,
  ``mix.uv``);
* ``rglru``: a recurrent block with a real-gated linear recurrent unit (``mix.y``, ``mix.x``, ``mix.conv``,
  ``mix.ra``, ``mix.ri``, ``mix.lam``, ``mix.o`` and their biases).

The feed-forward is a gated unit with both branches clamped (``ops.PARAMETRIC_ACTIVATIONS``).  The output is
``final.norm`` and the embedding table as the head.  Layers may differ in every size.
"""
from __future__ import annotations

from ..config.povusun import ARCHITECTURE, PovusunConfig
from ..config.registry import register_architecture
from ..parts.spec import (AttentionSpec, EmbeddingSpec, GatedMlpSpec, HeadSpec, LatentAttentionSpec, LayerSpec, ModelSpec,
                          NormSpec, QueryTemperatureSpec, RgLruSpec, ScheduleEntry, TokenSideSpec)

# what the design fixes
FEED_FORWARD_ACTIVATION = "swiglu_clamp"


def _mixer_spec(config: PovusunConfig, layer, p: str):
    if layer.type == "attention":
        temperature = QueryTemperatureSpec(layer.q_temp_coef, layer.q_temp_every) if layer.q_temp_every else None
        return AttentionSpec(
            hidden_size=config.width, num_heads=layer.heads, num_kv_heads=layer.kv_heads, head_dim=layer.dim,
            scale=layer.scale, position=None, q_weight=p + "mix.q", k_weight=p + "mix.k", v_weight=p + "mix.v",
            o_weight=p + "mix.o", v_head_dim=layer.vdim, gate_weight=p + "mix.g", gate_per_element=True,
            qk_norm_eps=config.norm_eps, q_temperature=temperature, softcap=layer.softcap,
            shares_kv=layer.kv_from is not None)
    if layer.type == "latent_attention":
        return LatentAttentionSpec(
            hidden_size=config.width, num_heads=layer.heads, head_dim=layer.dim, v_head_dim=layer.vdim,
            latent_dim=layer.kv_rank, scale=layer.scale, eps=config.norm_eps, q_weight=p + "mix.q",
            down_weight=p + "mix.dkv", latent_norm=p + "mix.dkv.norm", k_up_weight=p + "mix.uk",
            v_up_weight=p + "mix.uv", o_weight=p + "mix.o")
    return RgLruSpec(
        hidden_size=config.width, channels=layer.channels, parts=layer.blocks, taps=layer.taps,
        y_weight=p + "mix.y", y_bias=p + "mix.y.b", x_weight=p + "mix.x", x_bias=p + "mix.x.b",
        conv_weight=p + "mix.conv", conv_bias=p + "mix.conv.b", r_weight=p + "mix.ra", r_bias=p + "mix.ra.b",
        i_weight=p + "mix.ri", i_bias=p + "mix.ri.b", decay=p + "mix.lam", o_weight=p + "mix.o")


def povusun_spec(config: PovusunConfig) -> ModelSpec:
    layers, schedule, entry_of = [], [], {}
    side_width = config.side_dim * len(config.layers)
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        norm = lambda name: NormSpec(config.width, config.norm_eps, p + name)
        extras = [("mixer_post_norm", "norm", norm("norm1b"))]
        ffn = ffn_norm = None
        if layer.mlp is not None:
            ffn = GatedMlpSpec(config.width, layer.mlp.ff, FEED_FORWARD_ACTIVATION, p + "mlp.gate", p + "mlp.up",
                               p + "mlp.down", activation_param=layer.mlp.limit)
            ffn_norm = norm("norm2")
            extras.append(("ffn_post_norm", "norm", norm("norm2b")))
        if config.side_dim:
            extras.append(("token_input", "token_input", TokenSideSpec(
                hidden_size=config.width, vocab_size=config.vocab, dim=config.side_dim, offset=i * config.side_dim,
                table_width=side_width, eps=config.norm_eps, table="side.embed", gate_weight=p + "side.gate",
                proj_weight=p + "side.proj", norm_weight=p + "side.norm")))
        layers.append(LayerSpec(mixer_norm=norm("norm1"), mixer=_mixer_spec(config, layer, p), ffn_norm=ffn_norm,
                                ffn=ffn, arrangement="sandwich", extras=tuple(extras)))
        # a cache entry per layer that keeps something of its own; a layer that borrows keys names the lender's
        if layer.kv_from is not None:
            schedule.append(ScheduleEntry(layer=i, cache=entry_of[layer.kv_from], writes_cache=False))
        else:
            entry_of[i] = len(entry_of)
            schedule.append(ScheduleEntry(layer=i, cache=entry_of[i]))
    return ModelSpec(
        architecture=config.architecture, hidden_size=config.width, vocab_size=config.vocab,
        embedding=EmbeddingSpec(config.vocab, config.width, "embed"), layers=tuple(layers), schedule=tuple(schedule),
        final_norm=NormSpec(config.width, config.norm_eps, "final.norm"),
        head=HeadSpec(config.vocab, config.width, "embed"))


register_architecture(ARCHITECTURE, PovusunConfig, povusun_spec)
