"""An attention mixer whose values are its keys, with a sink in the softmax and a gate on its output.

``q = Wq h``, ``k = Wk h``; there is no value projection: ``v = k`` as projected.  Then, for the scores only, q and k
are RMS-normalised over the WHOLE projection (all heads at once, one weight per column) and rotated by position over
the first ``position.dim`` entries of every head.  Head ``g`` reads KV head ``g // (heads / kv_heads)``; key ``j`` is
visible to position ``p`` iff ``0 <= p - j < window``; the softmax's denominator also holds ``exp(sink_g)`` (no key, no
value, not scaled).  The concatenated heads are multiplied by ``sigmoid(Wg h)`` and projected by ``Wo``.

The cache is the K/V page cache of the plain attention mixer (same ``KVNeed``, so the two kinds share page groups when
their sizes agree): the key cells hold the normalised, rotated keys, the value cells the keys as projected.  ``Wq | Wk |
Wg`` are one product.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import KVNeed, Mixer, POSITIONS, register_mixer


@register_mixer("shared_kv_attention")
class SharedKVAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``, ``window`` (None or keys visible),
    ``qk_norm`` (bool: RMS norm of q and of k over the whole projection), ``qk_norm_eps``, ``sink`` (bool), ``output_gate``
    (bool), ``position`` (a PartSpec: ``rotary`` or ``none``)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        if self.nkv <= 0 or self.nh % self.nkv:
            raise ValueError(f"shared_kv_attention: {self.nh} heads cannot share {self.nkv} KV heads")
        self.scale = float(p["scale"])
        self.qk_norm = bool(p.get("qk_norm", False))
        self.eps = float(p.get("qk_norm_eps", 0.0))
        self.window = p.get("window")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError("shared_kv_attention: window must be positive or None")
        self.has_sink = bool(p.get("sink", False))
        self.has_gate = bool(p.get("output_gate", False))
        self.position = POSITIONS.build(p["position"], dtype, device)
        if not getattr(self.position, "fused", False):
            raise ValueError("shared_kv_attention: the position encoding must be a rotation (or none)")
        if getattr(self.position, "dim", 0) > self.hd:
            raise ValueError(f"shared_kv_attention: position encoding rotates {self.position.dim} dims of a head of {self.hd}")
        self.q_size = self.nh * self.hd
        self.kv_size = self.nkv * self.hd
        self.w_in = self.w_o = self.q_norm_w = self.k_norm_w = self.sink = None

    def tensors(self) -> Dict[str, TensorSpec]:
        t = {"q": TensorSpec((self.q_size, self.hidden)), "k": TensorSpec((self.kv_size, self.hidden)),
             "o": TensorSpec((self.hidden, self.q_size))}
        if self.qk_norm:
            t["q.norm"] = TensorSpec((self.q_size,), init="ones_jitter")
            t["k.norm"] = TensorSpec((self.kv_size,), init="ones_jitter")
        if self.has_sink:
            t["sink"] = TensorSpec((self.nh,))
        if self.has_gate:
            t["g"] = TensorSpec((self.q_size, self.hidden))
        return t

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        ws = [tensors["q"], tensors["k"]] + ([tensors["g"]] if self.has_gate else [])
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()
        self.w_o = tensors["o"].contiguous()
        if self.qk_norm:
            self.q_norm_w = tensors["q.norm"].to(torch.float32).contiguous()
            self.k_norm_w = tensors["k.norm"].to(torch.float32).contiguous()
        self.sink = tensors["sink"].to(torch.float32).contiguous() if self.has_sink else None

    def cache_need(self) -> KVNeed:
        return KVNeed(self.nkv, self.hd, int(self.window) if self.window is not None else None)

    def kernel_libraries(self):
        fast = self.dtype == torch.bfloat16 and self.hd in (64, 128)         # the tensor-core kernels take these heads
        return ("shared_kv", "attention_generic", "gemm_simt") + ((("attention_mma", "stream_ops") + (("attention_tc",) if self.hd == 128 else ())) if fast else ())

    def graph_plan(self, num_seqs: int, max_ctx: int):
        k = ops.kernels()
        if not hasattr(k, "sink_attention_plan"):
            return None
        return k.sink_attention_plan(num_seqs, self.nh, self.nkv, self.hd, max_ctx, self.window, self.dtype)

    def forward(self, x, ctx, cache, writes_cache: bool):
        k = ops.kernels()
        n = x.shape[0]
        pos = self.position
        width = self.w_in.shape[0]
        proj = ctx.buf("shared_kv_in", (n, width), self.dtype)
        k.linear(x, self.w_in, proj)
        meta = ctx.page_meta(cache.group)
        q = ctx.buf("q", (n, self.nh, self.hd), self.dtype)
        k.projection_norm_rope_store(
            proj, 0, self.q_size, q, cache.k if writes_cache else None, cache.v if writes_cache else None,
            num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.hd, q_weight=self.q_norm_w, k_weight=self.k_norm_w,
            eps=self.eps, inv_freq=pos.inv_freq64, rot_dim=pos.dim, rope_style=pos.style, positions=ctx.positions,
            slots=meta.slots if writes_cache else None)
        gate = proj[:, self.q_size + self.kv_size:] if self.has_gate else None
        attn = ctx.buf("attn", (n, self.q_size), self.dtype)
        k.sink_attention(q, cache.k, cache.v, attn, meta, num_heads=self.nh, num_kv_heads=self.nkv, head_dim=self.hd,
                         scale=self.scale, window=self.window, sink=self.sink, gate=gate, plan=ctx.graph_plan(self))
        out = ctx.buf("mixer_out", (n, self.hidden), self.dtype)
        k.linear(attn, self.w_o, out)
        return out
