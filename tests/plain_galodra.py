"""A plain, slow implementation of the Galodra design: whole sequences, no cache, one function per mechanism.

It shares no code with ``iian_b200``: it takes a configuration (the ``config.json`` mapping) and the tensors by
their file names and computes with elementary torch operations on the CPU, in float64 by default, so that it can
serve as the oracle of the 32-bit and of the bfloat16 path.

Notation.  ``x`` [T, W] is the stream of one sequence, positions ``0 .. T-1``.  A layer is post-norm:
``y = LN1(a x + g1(x) * mixer(x))``, ``z = LN2(a y + g2(y) * ff(y))`` with ``g(h) = sigmoid(Wg h + bg)``; the
stream handed on is a learned mix of the embedding output and of every layer result so far.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Mapping, Optional

import torch

from plain_qwen3 import read_safetensors


def load_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ---- elementary pieces ------------------------------------------------------------------------------
def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_half(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotate the first ``dims`` entries of the last axis: entry i pairs with entry i + dims/2, angle
    ``p * base^(-2i/dims)``.  ``v`` is [T, ..., n]; entries from ``dims`` on pass unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    freq = torch.pow(torch.tensor(base, dtype=v.dtype), -2.0 * i / dims)
    ang = positions.to(v.dtype)[:, None] * freq[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    cs, sn = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    a, b = v[..., :half], v[..., half:dims]
    out = v.clone()
    out[..., :half] = a * cs - b * sn
    out[..., half:dims] = b * cs + a * sn
    return out


def window_mask(t: int, size: Optional[int]) -> torch.Tensor:
    """visible[i, j]: query i sees key j iff 0 <= i - j (< size, if a size is given)."""
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    vis = j <= i
    if size is not None:
        vis &= (i - j) < size
    return vis


def sink_softmax(scores: torch.Tensor, visible: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """Softmax over the visible keys whose denominator also holds exp(sink) (one number per head, no key, no
    value).  ``scores`` [H, T, T], ``visible`` [T, T], ``sink`` [H]."""
    s = scores.masked_fill(~visible[None], float("-inf"))
    m = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


# ---- mixer ------------------------------------------------------------------------------------------
def latent_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], pre: str, m: Mapping, eps: float) -> torch.Tensor:
    """Keys and values of every head are read out of one low-rank latent per token plus one rotated key part that all
    heads share."""
    t = h.shape[0]
    heads, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(t)
    q = (h @ w[pre + "q"].T).view(t, heads, dim + rot)
    q_plain, q_rot = q[..., :dim], q[..., dim:]
    dkv = h @ w[pre + "dkv"].T
    c = rms_norm(dkv[:, :rank], w[pre + "dkv.norm"], eps)
    k_rot = dkv[:, rank:]
    if m.get("rot"):                      # without it the "rotated" parts stay as projected
        rdims, base = m["rot"]["dims"], m["rot"]["base"]
        q_rot = rotate_half(q_rot, pos, rdims, base)
        k_rot = rotate_half(k_rot, pos, rdims, base)
    k_plain = (c @ w[pre + "uk"].T).view(t, heads, dim)
    v = (c @ w[pre + "uv"].T).view(t, heads, vdim)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    size = (m.get("mask") or {}).get("size")
    p = sink_softmax(scores, window_mask(t, size), w[pre + "sink"])
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(t, heads * vdim)
    return o @ w[pre + "o"].T


# ---- feed-forwards ----------------------------------------------------------------------------------
def dense_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor], pre: str, act) -> torch.Tensor:
    return (act(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def routed_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor], pre: str, experts: int, top: int) -> torch.Tensor:
    """Each token goes to its ``top`` experts by sigmoid score; the score scales the expert's INPUT and is not
    renormalised."""
    s = torch.sigmoid(h @ w[pre + "router"].T)
    chosen = torch.topk(s, top, dim=-1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            out[t] += dense_ff((s[t, e] * h[t])[None], w, f"{pre}e{e}.", silu)[0]
    return out


def feed_forward(h, w, pre: str, spec: Mapping):
    if spec["kind"] == "dense":
        return dense_ff(h, w, pre, gelu_tanh)
    if spec["kind"] == "moe":
        return routed_ff(h, w, pre, spec["router"]["experts"], spec["router"]["top"])
    raise ValueError(spec["kind"])


# ---- the model --------------------------------------------------------------------------------------
def gate(h, w, name):
    return torch.sigmoid(h @ w[name].T + w[name + ".b"])


def layer(x: torch.Tensor, w, i: int, spec: Mapping, alpha: float, eps: float) -> torch.Tensor:
    pre = f"l{i}."
    if spec["type"] != "latent_attention":
        raise ValueError(spec["type"])
    mix = latent_attention(x, w, pre + "mix.", spec["mixer"], eps) * gate(x, w, pre + "rg1")
    x = layer_norm(alpha * x + mix, w[pre + "norm1"], w[pre + "norm1.b"], eps)
    if spec.get("mlp") is not None:
        ff = feed_forward(x, w, pre + "mlp.", spec["mlp"]) * gate(x, w, pre + "rg2")
        x = layer_norm(alpha * x + ff, w[pre + "norm2"], w[pre + "norm2.b"], eps)
    return x


def forward(cfg: Mapping, w: Mapping[str, torch.Tensor], tokens, dtype=torch.float64, streams: Optional[List] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``streams``, if a list, receives the stream after every layer
    (after the depth mix)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    results = [x]
    for i, spec in enumerate(cfg["layers"]):
        results.append(layer(x, w, i, spec, alpha, eps))
        mix = w[f"l{i}.dwa"]
        x = sum(mix[j] * results[j] for j in range(i + 2))
        if streams is not None:
            streams.append(x)
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return x @ w["embed"].T
