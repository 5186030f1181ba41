"""The matrix-memory mixer (the mLSTM of xLSTM): a recurrent layer whose state is a matrix per head.

``q = Wq h / sqrt(dim)``, ``k = Wk h`` (heads x dim), ``v = Wv h`` (heads x v_dim).  Per head a log input gate
``a = cap tanh((Wi h + bi) / cap)`` and a log forget gate ``b = logsigmoid(cap tanh((Wf h + bf) / cap))``.  With a running
maximum ``m`` that starts at ZERO (not at minus infinity), a memory ``C`` and a normaliser ``n`` that start at zero:

    m_t = max(b_t + m_{t-1}, a_t)
    C_t = exp(b_t + m_{t-1} - m_t) C_{t-1} + exp(a_t - m_t) k_t v_t^T          n_t alike with k_t alone
    o_t = C_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)

Each head's ``o`` is divided by its root mean square, the heads are concatenated, multiplied by a weight per column and by
``sigmoid(Wg h)``, and projected by ``Wo``.

The state (C, n, m per head, float32) lives in the request's state slot and is carried from step to step; a step walks
the tokens it brings in order.  ``Wq | Wk | Wv | Wg`` are one product in the activation dtype; the two gate
pre-activations are a second, small product with float32 output; gates, decays and the recurrence are float32 in both
dtypes.  The state is stored in blocks of ``columns`` columns of C, each with its own copy of n and m, which is how the
scan kernel spreads one head over several CTAs (``csrc/matrix_memory.cu``).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Mixer, StateNeed, register_mixer

DENOMINATOR_FLOOR = 1e-6        # the design's constant in o_t's denominator (also fixed in the kernel)


def state_columns(dim: int, v_dim: int) -> int:
    """Columns of C a CTA of the scan kernel owns: the largest of 16, 8, 4, 2, 1 that divides ``v_dim`` and, with the lanes
    that share a column (8 up to dim 128, 16 up to 256, 32 beyond), fits a CTA of 256 threads."""
    lanes = 8 if dim <= 128 else 16 if dim <= 256 else 32
    for c in (16, 8, 4, 2, 1):
        if v_dim % c == 0 and c * lanes <= 256:
            return c
    return 1


def state_block_floats(dim: int, columns: int) -> int:
    """Floats of one column block: its columns of C, a copy of n, m; padded to a multiple of 4."""
    return ((columns + 1) * dim + 1 + 3) // 4 * 4


@register_mixer("matrix_memory")
class MatrixMemory(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``dim`` (query/key size per head), ``v_dim``, ``gate_cap``, ``norm_eps`` (of
    the heads' root mean square), ``output_gate`` (bool, default True)."""

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["v_dim"])
        self.cap = float(p["gate_cap"])
        if self.cap <= 0:
            raise ValueError("matrix_memory: gate_cap must be positive")
        if self.dim > 512:
            raise ValueError("matrix_memory: the scan kernel holds heads of up to 512 query/key entries")
        self.eps = float(p["norm_eps"])
        self.has_gate = bool(p.get("output_gate", True))
        self.columns = state_columns(self.dim, self.vdim)
        self.qk_size = self.nh * self.dim
        self.v_size = self.nh * self.vdim
        self.w_in = self.w_gates = self.gate_bias = self.w_o = self.norm_w = None

    def tensors(self) -> Dict[str, TensorSpec]:
        t = {"q": TensorSpec((self.qk_size, self.hidden)), "k": TensorSpec((self.qk_size, self.hidden)),
             "v": TensorSpec((self.v_size, self.hidden)), "o": TensorSpec((self.hidden, self.v_size)),
             "norm": TensorSpec((self.v_size,), init="ones_jitter"),
             "i": TensorSpec((self.nh, self.hidden)), "i.b": TensorSpec((self.nh,)),
             "f": TensorSpec((self.nh, self.hidden)), "f.b": TensorSpec((self.nh,))}
        if self.has_gate:
            t["g"] = TensorSpec((self.v_size, self.hidden))
        return t

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        ws = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["g"]] if self.has_gate else [])
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()
        gs = [tensors["i"], tensors["f"]]
        if gs[0].dtype != gs[1].dtype:
            gs = [g.to(torch.float32) for g in gs]
        self.w_gates = torch.cat(gs, dim=0).contiguous()
        self.gate_bias = torch.cat([tensors["i.b"].to(torch.float32), tensors["f.b"].to(torch.float32)]).contiguous()
        self.w_o = tensors["o"].contiguous()
        self.norm_w = tensors["norm"].to(torch.float32).contiguous()

    def cache_need(self) -> StateNeed:
        return StateNeed((self.nh, self.vdim // self.columns, state_block_floats(self.dim, self.columns)), torch.float32)

    def kernel_libraries(self):
        return ("matrix_memory", "stream_ops", "gemm_simt")

    def forward(self, x, ctx, cache, writes_cache: bool):
        if not writes_cache:
            raise ValueError("matrix_memory: a recurrent layer cannot read the state another call keeps")
        k = ops.kernels()
        n = x.shape[0]
        proj = ctx.buf("memory_in", (n, self.w_in.shape[0]), self.dtype)
        k.linear(x, self.w_in, proj)
        gates = ctx.buf("memory_gates", (n, 2 * self.nh), torch.float32)
        k.linear(x, self.w_gates, gates)
        heads = ctx.buf("memory_heads", (n, self.v_size), torch.float32)
        k.matrix_memory_scan(proj, 0, self.qk_size, 2 * self.qk_size, gates, self.gate_bias, cache.state, ctx.cu_q,
                             ctx.state_slots, heads, num_heads=self.nh, dim=self.dim, v_dim=self.vdim, columns=self.columns,
                             cap=self.cap, q_scale=self.dim ** -0.5, max_q_len=ctx.max_q_len)
        gate = proj[:, 2 * self.qk_size + self.v_size:] if self.has_gate else None
        normed = ctx.buf("memory_normed", (n, self.v_size), self.dtype)
        k.head_norm_gate(heads, self.norm_w, gate, normed, num_heads=self.nh, eps=self.eps)
        out = ctx.buf("mixer_out", (n, self.hidden), self.dtype)
        k.linear(normed, self.w_o, out)
        return out
