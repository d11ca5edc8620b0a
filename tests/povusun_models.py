"""Small Povusun configurations for the tests, and folders with random weights for them.

The weights are drawn so that a fault shows: scales of the attention layers are large (peaked attention: a key
that is lost, shifted by one or taken from another page moves the logits by far more than rounding does), the
recurrent layers decay slowly (a lost or doubled state shows many tokens later), biases are large, and the caps
and temperatures of the scores bite within the first tokens.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch


def mlp(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def attention(heads, kv_heads, dim, vdim, scale, ff, softcap=None, q_temp=None, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        mixer["softcap"] = softcap
    if q_temp is not None:
        mixer["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": ff}


def latent(heads, dim, vdim, rank, scale, ff):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale},
            "mlp": ff}


def rglru(width, blocks, taps, ff):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": taps}, "mlp": ff}


def config(vocab, width, layers, side=None, eps=1e-5):
    raw = {"architecture": "Povusun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if side:
        raw["token_side"] = {"dim": side}
    return raw


# PA: a recurrent layer first (three taps, three parts, narrower than the model), four query heads on one key head with
#     values wider than keys, a latent wider than a head, a layer without a feed-forward, and a last layer that borrows
#     the keys of layer 1 across two others; temperature periods of 7 and 5 tokens, a cap of 6.
PA = config(97, 64, [rglru(48, 3, 3, mlp(40, 0.5)),
                     attention(4, 1, 16, 24, 0.45, mlp(96, 2.0), softcap=6.0, q_temp=(0.5, 7)),
                     latent(3, 16, 8, 40, 0.3, None),
                     attention(4, 1, 16, 24, 0.5, mlp(56, 1.5), q_temp=(0.25, 5), kv_from=1)], side=8)
# PB: sizes that are multiples of nothing much, no per-layer token input, attention without cap and temperature, a
#     single-tap convolution and a single part, a cap of 3 with a period of 64, as many key heads as query heads.
PB = config(211, 72, [attention(6, 3, 20, 12, 0.6, mlp(100, 0.75)), latent(2, 24, 40, 24, 0.25, mlp(52, 3.0)),
                      rglru(80, 1, 1, None), attention(2, 2, 32, 32, 0.4, mlp(30, 1.0), softcap=3.0, q_temp=(1.0, 64)),
                      attention(6, 3, 20, 12, 0.3, None, softcap=8.0, kv_from=0)], eps=1e-6)
# PC: head size 64 for keys and values and a latent of 64 and of 128 (the sizes that kernels of one head size serve in
#     bfloat16; the second latent layer's heads have the size at which prompts run as multi-head attention over
#     up-projected keys and values), a recurrent layer wider than the model with five taps.
PC = config(300, 128, [attention(4, 2, 64, 64, 0.25, mlp(136, 1.0), softcap=10.0, q_temp=(0.3, 48)),
                       latent(4, 32, 32, 64, 0.15, mlp(64, 2.0)), rglru(192, 2, 5, mlp(72, 1.0)),
                       latent(2, 64, 64, 128, 0.1, None),
                       attention(4, 2, 64, 64, 0.2, mlp(80, 0.5), softcap=10.0, kv_from=0)], side=16)
POVUSUN = {"PA": PA, "PB": PB, "PC": PC}


def make_folder(folder, raw_config, seed, dtype=torch.float32):
    """A model folder with random weights stored in ``dtype``."""
    from stratakv_b200.config import PovusunConfig
    from stratakv_b200.engine.model import expected_tensors
    from stratakv_b200.models.povusun import povusun_spec
    from stratakv_b200.weights.random_init import random_tensors
    from stratakv_b200.weights.safetensors_io import write_safetensors
    typed = PovusunConfig.from_dict(raw_config)
    tensors = random_tensors(expected_tensors(povusun_spec(typed)), seed, std=0.05, dtype=torch.float32)
    sharpen = (2304.0 / typed.width) ** 0.5
    for name in tensors:
        layer = int(name[1:name.index(".")]) if name.startswith("l") and name[1].isdigit() else None
        kind = typed.layers[layer].type if layer is not None else None
        if name.endswith(".mix.lam"):
            tensors[name] = tensors[name] * 10.0 - 2.5           # decays of 0.5 to 0.95 a token
        elif name.endswith(".mix.conv"):
            tensors[name] = tensors[name] * 4.0
        elif name.endswith((".b",)):
            tensors[name] = tensors[name] * 10.0
        elif kind == "latent_attention" and name.endswith((".mix.q", ".mix.uk")):
            # (no norm on these queries and keys: scores with a standard deviation of 2 to 3)
            tensors[name] = tensors[name] * (sharpen if name.endswith(".mix.q") else sharpen ** 0.5)
        elif name.endswith(".mix.dkv.norm"):
            tensors[name] = 1.0 + (tensors[name] - 1.0) * 8.0     # a latent norm's weight that is far from all ones
        elif name.endswith((".mix.ra", ".mix.ri")):
            tensors[name] = tensors[name] * 2.0
        elif name.endswith(".mix.g"):
            tensors[name] = tensors[name] * 5.0
        # (the side input's gate stays small: where gelu_tanh of all of a token's few gate values is nearly zero, the
        # norm after the projection blows up what is left of them, rounding included, in any implementation)
        elif name == "side.embed":
            tensors[name] = tensors[name] * 20.0
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw_config, indent=1))
    write_safetensors(folder / "model.safetensors", {n: t.to(dtype) for n, t in tensors.items()})
    return folder
