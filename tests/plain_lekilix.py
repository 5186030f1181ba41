"""A plain, slow implementation of the Lekilix design: whole sequences, no cache, one function per mechanism.

It shares no code with ``iian_b200``: it takes a configuration (the ``config.json`` mapping) and the tensors by their
file names and computes with elementary torch operations on the CPU, in float64 by default, so that it can serve as the
oracle of the 32-bit and of the bfloat16 path.

Notation.  ``x`` [T, W] is the stream of one sequence, positions ``0 .. T-1``; ``e`` = table[token] * scale is what the
embedding leaves.  A layer has ONE norm whose output ``h`` feeds the mixer and the feed-forward side by side:
``x' = x + (mixer(h) + ff(h))``.  A stretch of layers may be run several times in a row with the same weights; every run
of the stretch starts with ``x <- Win [x ; e]``.
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
# What a matrix product's result passes through before anything else reads it: nothing.  A test that wants to know how far
# 16-bit products alone move the logits sets this to a rounding function for the time of a call.
product_rounding = None


def mm(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``h W^T`` (weights are stored [out, in]); with ``product_rounding`` set, its input and its result pass through it."""
    if product_rounding is None:
        return h @ w.T
    return product_rounding(product_rounding(h) @ w.T)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norm of this design: the stored weight sits around zero and one is added to it."""
    return unit_rms(x, eps) * (1.0 + w)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_pairs(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotate the first ``dims`` entries of the last axis, entry 2i with entry 2i+1, by ``p * base^(-2i/dims)``.
    ``v`` is [T, heads, n]; entries from ``dims`` on pass unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    freq = torch.pow(torch.tensor(base, dtype=v.dtype), -2.0 * i / dims)
    ang = positions.to(v.dtype)[:, None] * freq[None, :]
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out = v.clone()
    out[..., 0:dims:2] = a * cs - b * sn
    out[..., 1:dims:2] = b * cs + a * sn
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
    """Softmax over the visible keys whose denominator also holds exp(sink) (one number per head, no key, no value,
    not multiplied by the score scale).  ``scores`` [H, T, T], ``visible`` [T, T], ``sink`` [H]."""
    s = scores.masked_fill(~visible[None], float("-inf"))
    m = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


# ---- mixers ---------------------------------------------------------------------------------------------
def shared_kv_attention(h: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str, mc: Mapping, eps: float) -> torch.Tensor:
    """Attention whose values are the keys as projected.  ``h`` [T, W]."""
    T = h.shape[0]
    H, G, d = mc["heads"], mc["kv_heads"], mc["dim"]
    q = mm(h, t[pre + "q"])                                     # [T, H d]
    k = mm(h, t[pre + "k"])                                     # [T, G d]
    v = k.view(T, G, d)                                        # the values: the keys before norm and rotation
    q = unit_rms(q, eps) * t[pre + "q.norm"]                   # one norm over the whole projection, all heads at once
    k = unit_rms(k, eps) * t[pre + "k.norm"]
    q, k = q.view(T, H, d), k.view(T, G, d)
    pos = torch.arange(T)
    rot = mc.get("rot")
    if rot is not None:
        q = rotate_pairs(q, pos, rot["dims"], rot["base"])
        k = rotate_pairs(k, pos, rot["dims"], rot["base"])
    group = torch.arange(H) // (H // G)
    scores = torch.einsum("ihd,jhd->hij", q, k[:, group]) * mc["scale"]
    mask = mc.get("mask")
    vis = window_mask(T, mask["size"] if mask is not None else None)
    if (pre + "sink") in t:
        p = sink_softmax(scores, vis, t[pre + "sink"])
    else:
        p = torch.softmax(scores.masked_fill(~vis[None], float("-inf")), -1)
    o = torch.einsum("hij,jhd->ihd", p, v[:, group]).reshape(T, H * d)
    o = o * torch.sigmoid(mm(h, t[pre + "g"]))
    return mm(o, t[pre + "o"])


def soft_cap(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def matrix_memory(h: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str, mc: Mapping, eps: float,
                  state=None, return_state: bool = False):
    """The matrix-memory recurrence, one token after the other.  Per head a memory C [d, dv], a normaliser n [d] and a
    running maximum m (a scalar) that starts at ZERO:

        a_t = cap tanh((Wi h + bi) / cap)                    log input gate
        b_t = logsigmoid(cap tanh((Wf h + bf) / cap))        log forget gate
        m_t = max(b_t + m_{t-1}, a_t)
        C_t = exp(b_t + m_{t-1} - m_t) C_{t-1} + exp(a_t - m_t) k_t v_t^T        (n_t alike, with k_t alone)
        o_t = C_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
    """
    T = h.shape[0]
    H, d, dv = mc["heads"], mc["dim"], mc["vdim"]
    cap = mc["gate_cap"]
    q = mm(h, t[pre + "q"]).view(T, H, d) * d ** -0.5
    k = mm(h, t[pre + "k"]).view(T, H, d)
    v = mm(h, t[pre + "v"]).view(T, H, dv)
    a = soft_cap(mm(h, t[pre + "i"]) + t[pre + "i.b"], cap)                                    # [T, H]
    b = torch.nn.functional.logsigmoid(soft_cap(mm(h, t[pre + "f"]) + t[pre + "f.b"], cap))
    if state is None:
        C = torch.zeros(H, d, dv, dtype=h.dtype)
        n = torch.zeros(H, d, dtype=h.dtype)
        m = torch.zeros(H, dtype=h.dtype)
    else:
        C, n, m = state
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for s in range(T):
        m_new = torch.maximum(b[s] + m, a[s])
        keep = torch.exp(b[s] + m - m_new)
        take = torch.exp(a[s] - m_new)
        C = keep[:, None, None] * C + take[:, None, None] * k[s][:, :, None] * v[s][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[s]
        m = m_new
        num = torch.einsum("hdv,hd->hv", C, q[s])
        den = torch.maximum((n * q[s]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[s] = num / den[:, None]
    out = unit_rms(out, eps).reshape(T, H * dv) * t[pre + "norm"]          # each head by its own root mean square
    out = out * torch.sigmoid(mm(h, t[pre + "g"]))
    y = mm(out, t[pre + "o"])
    return (y, (C, n, m)) if return_state else y


# ---- feed-forwards ------------------------------------------------------------------------------------------
def dense_ff(h: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str) -> torch.Tensor:
    return mm(silu(mm(h, t[pre + "gate"])) * mm(h, t[pre + "up"]), t[pre + "down"])


def clamped_expert(h: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str, limit: float) -> torch.Tensor:
    g = torch.clamp(mm(h, t[pre + "gate"]), max=limit)
    u = torch.clamp(mm(h, t[pre + "up"]), -limit, limit)
    return mm(g * torch.sigmoid(1.702 * g) * (u + 1.0), t[pre + "down"])


def table_routed_ff(h: torch.Tensor, tokens: torch.Tensor, t: Mapping[str, torch.Tensor], pre: str, fc: Mapping) -> torch.Tensor:
    """No router: a table row per token id names the experts of that token; each weighs 1 / top."""
    top = fc["router"]["top"]
    table = t[pre + "table"].long()
    out = torch.zeros(h.shape[0], t[pre + "e0.down"].shape[0], dtype=h.dtype)
    for s in range(h.shape[0]):
        for e in table[int(tokens[s])].tolist():
            out[s] += clamped_expert(h[s:s + 1], t, f"{pre}e{e}.", fc["expert"]["limit"])[0] / top
    return out


# ---- the model ---------------------------------------------------------------------------------------------------
def run_order(cfg: Mapping) -> List[tuple]:
    """(layer, first of a run of the stretch?) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if loop is None:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        order += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    order += [(i, False) for i in range(loop["stop"], n)]
    return order


def forward(cfg: Mapping, tensors: Mapping[str, torch.Tensor], tokens, dtype=torch.float64, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and, on request, the stream after every layer run [runs, T, W])."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    e = t["embed"][tokens] * cfg["embedding"]["scale"]
    x = e
    layers = []
    for i, starts_run in run_order(cfg):
        lc = cfg["layers"][i]
        if starts_run:
            x = mm(torch.cat([x, e], dim=-1), t["loop.in"])
        h = offset_rms_norm(x, t[f"l{i}.norm1"], eps)
        if lc["type"] == "attention":
            y = shared_kv_attention(h, t, f"l{i}.mix.", lc["mixer"], eps)
        elif lc["type"] == "mlstm":
            y = matrix_memory(h, t, f"l{i}.mix.", lc["mixer"], eps)
        else:
            raise ValueError(lc["type"])
        fc = lc.get("mlp")
        if fc is not None:
            y = y + (dense_ff(h, t, f"l{i}.mlp.") if fc["kind"] == "dense" else table_routed_ff(h, tokens, t, f"l{i}.mlp.", fc))
        x = x + y
        layers.append(x)
    logits = mm(offset_rms_norm(x, t["final.norm"], eps), t["head"])
    return (logits, torch.stack(layers)) if return_layers else logits
