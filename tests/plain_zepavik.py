"""A plain, slow implementation of the Zepavik decoder in float64 on the CPU: whole sequences, no cache,
no batching, one function per mechanism.  It shares no code with the library; tests compare the engine
with it on small random models.

Notation: T tokens, W the width, H query heads on G key/value heads, d the key size, dv the value size.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

F64 = torch.float64


# ---- reading a model folder (a reader of its own: 8 bytes of length, a JSON header, the data) -----------
def load_folder(folder):
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (size,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + size])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    weights = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        begin, end = info["data_offsets"]
        flat = torch.frombuffer(bytearray(raw[8 + size + begin:8 + size + end]), dtype=kinds[info["dtype"]])
        weights[name] = flat.reshape(info["shape"]).to(F64)
    return config, weights


# ---- mechanisms ---------------------------------------------------------------------------------------
def rms_divide(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def pair_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for each token: a hash of (previous, current); the first token reads row `buckets`."""
    rows = [buckets]
    for i in range(1, len(tokens)):
        rows.append((tokens[i - 1] * mul_prev + tokens[i] * mul_cur) % buckets)
    return rows


def embed(config, weights, tokens):
    x = weights["embed"][torch.tensor(tokens)]
    pair = (config.get("embedding") or {}).get("bigram")
    if pair is not None:
        x = x + weights["bigram"][torch.tensor(pair_rows(tokens, pair["buckets"], pair["mul_prev"], pair["mul_cur"]))]
    return x + weights["pos"][:len(tokens)]


def distance_penalty(r1, r2, length):
    """[H, T, T]: r1_h * ln(1 + r2_h * (i - j)) for j <= i (zero elsewhere: those scores are masked anyway)."""
    i = torch.arange(length)[:, None]
    j = torch.arange(length)[None, :]
    distance = (i - j).clamp(min=0).to(F64)
    return r1[:, None, None] * torch.log1p(r2[:, None, None] * distance[None])


def visible(length, window):
    """[T, T] bool: query i sees key j iff 0 <= i - j < window (window 0: every j <= i)."""
    i = torch.arange(length)[:, None]
    j = torch.arange(length)[None, :]
    seen = j <= i
    if window > 0:
        seen = seen & (i - j < window)
    return seen


def attention_mixer(weights, prefix, mixer, eps, h):
    """h [T, W] -> [T, W]."""
    T = h.shape[0]
    H, d = mixer["heads"], mixer["dim"]
    G, dv = mixer.get("kv_heads", H), mixer.get("vdim", d)
    q = (h @ weights[prefix + "q"].T + weights[prefix + "q.b"]).view(T, H, d)
    k = (h @ weights[prefix + "k"].T + weights[prefix + "k.b"]).view(T, G, d)
    v = (h @ weights[prefix + "v"].T + weights[prefix + "v.b"]).view(T, G, dv)
    v = rms_divide(v, eps)                                            # per head, no weight
    window = (mixer.get("mask") or {}).get("size", 0)
    seen = visible(T, window)
    penalty = distance_penalty(weights[prefix + "r1"], weights[prefix + "r2"], T)
    gate = torch.sigmoid(h @ weights[prefix + "g"].T)                  # [T, H]
    heads = []
    for head in range(H):
        kv = head // (H // G)
        score = (q[:, head] @ k[:, kv].T) * mixer["scale"] - penalty[head]
        score = score.masked_fill(~seen, -math.inf)
        heads.append(torch.softmax(score, dim=-1) @ v[:, kv] * gate[:, head:head + 1])
    return torch.cat(heads, dim=-1) @ weights[prefix + "o"].T


def feed_forward(weights, prefix, h):
    return (torch.relu(h @ weights[prefix + "up"].T) ** 2) @ weights[prefix + "down"].T


def layer(config, weights, index, x):
    """Parallel: both branches read one norm's output."""
    spec = config["layers"][index]
    eps = config["norm"]["eps"]
    prefix = f"l{index}."
    h = rms_divide(x, eps) * weights[prefix + "norm1"]
    update = attention_mixer(weights, prefix + "mix.", spec["mixer"], eps, h)
    if spec.get("mlp") is not None:
        update = update + feed_forward(weights, prefix + "mlp.", h)
    return x + update


def residuals_of(config, weights, tokens):
    """The residual stream after every layer, [layers, T, W], and after the embedding."""
    x = embed(config, weights, tokens)
    after = []
    for index in range(len(config["layers"])):
        x = layer(config, weights, index, x)
        after.append(x)
    return torch.stack(after)


def logits_of(config, weights, tokens):
    """[T, vocab] float64."""
    x = residuals_of(config, weights, tokens)[-1]
    y = rms_divide(x, config["norm"]["eps"]) * weights["final.norm"]
    return (y @ weights["head"].T) * config.get("logit_scale", 1.0)


def greedy(config, weights, prompt, new_tokens):
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(torch.argmax(logits_of(config, weights, tokens)[-1])))
    return tokens
