"""The Zepavik decoder as a list of parts.

Embedding: the token's row of ``embed`` plus a row of ``bigram`` chosen by a hash of the token and the one
before it plus the learned vector ``pos[p]``.  Every layer ``l<i>`` is parallel: ``h = norm1(x)`` and
``x += mixer(h) + mlp(h)``.  The mixer is attention without a rotation: biased projections (``mix.q``,
``mix.q.b`` and so on), value heads divided by their root mean square before they are cached, scores
``(q.k) * scale - r1 ln(1 + r2 (i - j))`` inside a sliding window, a gate per head ``sigmoid(mix.g . h)`` on the
output, then ``mix.o``.  The feed-forward is ``mlp.down(relu(mlp.up(h))^2)``; a layer may have none.  The
output is ``final.norm`` and ``head`` times a scale.  Layers may differ in every size.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zepavik import ARCHITECTURE, ZepavikConfig
from ..parts.spec import (AttentionSpec, DistanceBiasSpec, HashedPairSpec, HeadSpec, LayerSpec, LearnedPositionSpec,
                          MlpSpec, ModelSpec, NormSpec, ScheduleEntry, SummedEmbeddingSpec)

# what the design fixes: the feed-forward's activation, and that the value norm shares the layer norm's eps
FEED_FORWARD_ACTIVATION = "relu2"


def zepavik_spec(config: ZepavikConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        mixer = AttentionSpec(
            hidden_size=config.width, num_heads=layer.heads, num_kv_heads=layer.kv_heads, head_dim=layer.dim,
            scale=layer.scale, position=None,
            q_weight=p + "mix.q", k_weight=p + "mix.k", v_weight=p + "mix.v", o_weight=p + "mix.o",
            window=layer.window, v_head_dim=layer.vdim,
            q_bias=p + "mix.q.b", k_bias=p + "mix.k.b", v_bias=p + "mix.v.b",
            value_norm_eps=config.norm_eps,
            distance_bias=DistanceBiasSpec(p + "mix.r1", p + "mix.r2", max_distance=config.max_positions),
            gate_weight=p + "mix.g")
        ffn = None
        if layer.ff:
            ffn = MlpSpec(config.width, layer.ff, FEED_FORWARD_ACTIVATION, p + "mlp.up", p + "mlp.down")
        layers.append(LayerSpec(mixer_norm=NormSpec(config.width, config.norm_eps, p + "norm1"), mixer=mixer,
                                ffn=ffn, arrangement="parallel"))
    pair = None
    if config.bigram is not None:
        pair = HashedPairSpec(config.bigram.buckets, config.bigram.mul_prev, config.bigram.mul_cur, "bigram")
    embedding = SummedEmbeddingSpec(config.vocab, config.width, "embed", pair=pair,
                                    positions=LearnedPositionSpec(config.max_positions, "pos"))
    return ModelSpec(
        architecture=config.architecture, hidden_size=config.width, vocab_size=config.vocab, embedding=embedding,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i, cache=i) for i in range(len(layers))),
        final_norm=NormSpec(config.width, config.norm_eps, "final.norm"),
        head=HeadSpec(config.vocab, config.width, "head", logit_scale=config.logit_scale),
        max_positions=config.max_positions, positions_are_tabled=True)


register_architecture(ARCHITECTURE, ZepavikConfig, zepavik_spec)
