"""Small Zepavik configurations for the tests, and folders with random weights for them.

The weights of queries and keys are drawn larger than the rest, so that attention is peaked and a key that is
lost, shifted by one or taken from another page moves the logits by far more than rounding does.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch


def layer(heads, kv_heads, dim, vdim, window, ff, scale=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
             "scale": scale if scale is not None else dim ** -0.5}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(vocab, width, layers, buckets, mul_prev, mul_cur, max_positions=512, eps=1e-5, logit_scale=1.0):
    return {"architecture": "Zepavik", "vocab": vocab, "width": width, "max_positions": max_positions,
            "logit_scale": logit_scale, "norm": {"eps": eps},
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "layers": layers}


# A: head size 16 for keys and values (the kernels of one head size serve in bfloat16), then a layer whose values
#    are narrower than its keys and which has no feed-forward; windows that end inside a page.
ZA = config(96, 64, [layer(4, 2, 16, 16, 24, 96), layer(2, 2, 32, 16, 40, 0)], buckets=13, mul_prev=31, mul_cur=7)
# B: sizes that are multiples of nothing much: three query heads a key head, a window of 7, one of 130 that
#    spans pages, a layer without a window, a head of its own width, one bucket only.
ZB = config(131, 72, [layer(6, 2, 20, 12, 7, 100), layer(3, 1, 24, 40, 130, 52), layer(1, 1, 8, 8, 0, 8, scale=0.5)],
            buckets=1, mul_prev=3, mul_cur=5, eps=1e-6, logit_scale=0.5)
# C: head size 64, where prompts run on the tcgen05 attention kernel; a window of 100 (edges inside pages) and one
#    of 192 (three pages exactly); multipliers that overflow 32 bits with the vocabulary.
ZC = config(300, 128, [layer(2, 1, 64, 64, 100, 136), layer(4, 4, 64, 64, 192, 64)], buckets=251,
            mul_prev=20000003, mul_cur=10000019, max_positions=1024, logit_scale=2.0)
# D: head size 32 for both (prompts on the mma.sync kernel), eight query heads on one key head, no window at all.
ZD = config(200, 96, [layer(8, 1, 32, 32, 0, 48), layer(2, 2, 32, 32, 33, 40)], buckets=64, mul_prev=1, mul_cur=1)
ZEPAVIK = {"ZA": ZA, "ZB": ZB, "ZC": ZC, "ZD": ZD}


def make_folder(folder, raw_config, seed, dtype=torch.float32, sharpen=None):
    """A model folder with random weights stored in ``dtype``; query and key matrices times ``sharpen``.
    By default the factor is such that scores (before the design's scale, over sqrt(dim)) have a standard deviation of
    about 6 at every width: peaked attention, with the same share of bfloat16 rounding in every configuration."""
    from stratakv_b200.config import ZepavikConfig
    from stratakv_b200.engine.model import expected_tensors
    from stratakv_b200.models.zepavik import zepavik_spec
    from stratakv_b200.weights.random_init import random_tensors
    from stratakv_b200.weights.safetensors_io import write_safetensors
    typed = ZepavikConfig.from_dict(raw_config)
    if sharpen is None:
        sharpen = (2304.0 / typed.width) ** 0.5           # 0.05^2 * sharpen^2 * width = 5.76
    tensors = random_tensors(expected_tensors(zepavik_spec(typed)), seed, std=0.05, dtype=torch.float32)
    for name in tensors:
        if name.endswith((".mix.q", ".mix.k")):
            tensors[name] = tensors[name] * sharpen
        if name.endswith((".mix.q.b", ".mix.k.b", ".mix.v.b")):
            tensors[name] = tensors[name] * 10.0
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw_config, indent=1))
    write_safetensors(folder / "model.safetensors", {n: t.to(dtype) for n, t in tensors.items()})
    return folder
