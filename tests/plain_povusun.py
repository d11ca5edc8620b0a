"""A plain, slow restatement of the Povusun decoder: whole sequences, no cache, float64, one function per
mechanism.  It shares no code with the library; the GPU tests compare the engine with it.

Notation: a sequence of T tokens at positions 0..T-1, width W.  ``P`` maps tensor names to float64 tensors,
``cfg`` is the dictionary of a ``config.json`` of this design.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1) for every position p."""
    steps = torch.div(positions + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(F64) + 1.0)


def soft_cap(scores, cap):
    return cap * torch.tanh(scores / cap)


def causal_softmax(scores):
    """scores [heads, T, T]: query i sees keys j <= i."""
    T = scores.shape[-1]
    hidden = torch.ones(T, T, dtype=torch.bool).triu(1)
    return torch.softmax(scores.masked_fill(hidden, -math.inf), dim=-1)


def attention_keys_values(h, P, p, m, eps):
    """What an attention layer caches: keys after their unit norm, and values."""
    T = h.shape[0]
    k = unit_rms((h @ P[p + "mix.k"].T).view(T, m["kv_heads"], m["dim"]), eps)
    v = (h @ P[p + "mix.v"].T).view(T, m["kv_heads"], m["vdim"])
    return k, v


def attention_mixer(h, P, p, m, eps, keys_values):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    k, v = keys_values
    q = unit_rms((h @ P[p + "mix.q"].T).view(T, H, d), eps)
    if m.get("q_temp"):
        q = q * query_temperature(torch.arange(T), m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    group = H // G
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    if m.get("softcap"):
        scores = soft_cap(scores, m["softcap"])
    weights = causal_softmax(scores)
    out = torch.einsum("hij,jhd->ihd", weights, v).reshape(T, H * dv)
    out = out * torch.sigmoid(h @ P[p + "mix.g"].T)
    return out @ P[p + "mix.o"].T


def latent_attention_mixer(h, P, p, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ P[p + "mix.q"].T).view(T, H, d)
    c = rms_norm(h @ P[p + "mix.dkv"].T, P[p + "mix.dkv.norm"], eps)
    k = (c @ P[p + "mix.uk"].T).view(T, H, d)
    v = (c @ P[p + "mix.uv"].T).view(T, H, dv)
    weights = causal_softmax(torch.einsum("ihd,jhd->hij", q, k) * m["scale"])
    out = torch.einsum("hij,jhd->ihd", weights, v).reshape(T, H * dv)
    return out @ P[p + "mix.o"].T


def causal_conv(x, taps_weight, bias):
    """x [T, C]; taps_weight [C, taps], the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = taps_weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x])
    out = torch.zeros_like(x)
    for k in range(taps):
        out = out + padded[k:k + T] * taps_weight[:, k]
    return out + bias


def block_gate(u, weight, bias):
    """sigmoid(weight[b] u_b + bias[b]) for every equal part b of the channels; weight [blocks, out, in]."""
    T = u.shape[0]
    blocks, size = weight.shape[0], weight.shape[1]
    parts = u.view(T, blocks, size)
    return torch.sigmoid(torch.einsum("tbi,boi->tbo", parts, weight) + bias).reshape(T, blocks * size)


def rglru_mixer(h, P, p, m):
    T = h.shape[0]
    y = gelu_tanh(h @ P[p + "mix.y"].T + P[p + "mix.y.b"])
    u = causal_conv(h @ P[p + "mix.x"].T + P[p + "mix.x.b"], P[p + "mix.conv"], P[p + "mix.conv.b"])
    r = block_gate(u, P[p + "mix.ra"], P[p + "mix.ra.b"])
    i = block_gate(u, P[p + "mix.ri"], P[p + "mix.ri.b"])
    log_a = -8.0 * r * torch.nn.functional.softplus(P[p + "mix.lam"])
    a = torch.exp(log_a)
    driven = torch.sqrt(1.0 - a * a) * i * u
    state = torch.zeros(m["width"], dtype=F64)
    states = []
    for t in range(T):
        state = a[t] * state + driven[t]
        states.append(state)
    return (torch.stack(states) * y) @ P[p + "mix.o"].T


def dense_feed_forward(h, P, p, mlp):
    limit = mlp["limit"]
    g = torch.clamp(h @ P[p + "mlp.gate"].T, max=limit)
    u = torch.clamp(h @ P[p + "mlp.up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ P[p + "mlp.down"].T


def token_side_input(x, tokens, P, p, index, dim, eps):
    e = P["side.embed"][tokens][:, index * dim:(index + 1) * dim]
    g = gelu_tanh(x @ P[p + "side.gate"].T) * e
    y = g @ P[p + "side.proj"].T
    return x + rms_norm(y, P[p + "side.norm"], eps)


def forward(cfg, tensors, tokens, return_layers: bool = False):
    """Logits [T, vocab] of one sequence; with ``return_layers`` also the stream after every layer."""
    P = {name: t.to(F64) for name, t in tensors.items() if t.dtype.is_floating_point}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = P["embed"][tokens]
    cached = {}
    after = []
    for index, layer in enumerate(cfg["layers"]):
        p = f"l{index}."
        m = layer["mixer"]
        h = rms_norm(x, P[p + "norm1"], eps)
        if layer["type"] == "attention":
            if m.get("kv_from") is None:
                cached[index] = attention_keys_values(h, P, p, m, eps)
            mixed = attention_mixer(h, P, p, m, eps, cached[m["kv_from"] if m.get("kv_from") is not None else index])
        elif layer["type"] == "latent_attention":
            mixed = latent_attention_mixer(h, P, p, m, eps)
        elif layer["type"] == "rglru":
            mixed = rglru_mixer(h, P, p, m)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(mixed, P[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = rms_norm(x, P[p + "norm2"], eps)
            x = x + rms_norm(dense_feed_forward(h, P, p, layer["mlp"]), P[p + "norm2b"], eps)
        if cfg.get("token_side"):
            x = token_side_input(x, tokens, P, p, index, cfg["token_side"]["dim"], eps)
        after.append(x)
    logits = rms_norm(x, P["final.norm"], eps) @ P["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits


def load_folder(folder):
    """(config dictionary, tensors as float64) of a model folder; reads the safetensors container itself."""
    import json
    import struct
    from pathlib import Path
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


def logits_of(config, weights, tokens):
    return forward(config, weights, tokens)
