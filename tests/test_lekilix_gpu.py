"""Lekilix on the GPU.  Each new kernel alone against the plain functions of tests/plain_lekilix.py (scaled embedding, the
norm's sum of two sub-layer outputs, the re-injection's input, gates, the norm over a whole projection with rotation and
the cache write where the values are the unrotated keys, attention with a sink and a stand-out key just inside and just
outside the window, at page borders and far away, in prompts and in decoding; the matrix-memory scan in every lane form,
cut into steps, with slots used again; experts chosen by a table); then whole models under every way of cutting the work, in
32-bit and in bfloat16; greedy generation through the engine's entry point with and without CUDA graphs; the trace runner
as a program."""
import json
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_lekilix as plain
from helpers import max_error, random_tokens, replay_and_collect, trace_mixed, trace_portions, trace_tail, trace_whole
from lekilix_cases import BLOCK_SIZE, CONFIGS, plain_logits, write_case

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


def K():
    from iian_b200 import ops
    return ops.kernels()


def close(got, want, dtype, what, rel16=2e-2, abs32=2e-5):
    got, want = got.double().cpu(), want.double().cpu()
    tol = abs32 * max(1.0, want.abs().max().item()) if dtype == "float32" else rel16 * want.abs().max().item()
    err = (got - want).abs().max().item()
    assert err <= tol, f"{what} [{dtype}]: max error {err:.3g} > {tol:.3g}"


# ---- row-wise kernels ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_scaled_embedding_and_sum_of_two_in_the_norm(dtype):
    g = torch.Generator().manual_seed(1)
    table = torch.randn(50, 72, generator=g).to(DT[dtype])
    toks = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    out = torch.empty(4, 72, device=DEV)
    K().embedding_scaled(table.to(DEV), toks.to(DEV), 7.25, out)
    close(out, table.double()[toks.long()] * 7.25, "float32", "scaled embedding")
    for h in (72, 1000, 4100):
        x = torch.randn(5, h, generator=g) * 3
        d1, d2 = torch.randn(5, h, generator=g).to(DT[dtype]), torch.randn(5, h, generator=g).to(DT[dtype])
        w = torch.randn(h, generator=g) * 0.2
        res = x.to(DEV).clone()
        normed = torch.empty(5, h, device=DEV, dtype=DT[dtype])
        K().add2_rms_norm(res, d1.to(DEV), d2.to(DEV), (w + 1.0).to(DEV), 1e-5, normed)
        s = x.double() + (d1.double() + d2.double())
        close(res, s, "float32", f"stream after the sum, width {h}")
        close(normed, plain.offset_rms_norm(s, w.double(), 1e-5), dtype, f"norm with one added to the weight, width {h}", rel16=8e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_reinjection_input_and_gates(dtype):
    g = torch.Generator().manual_seed(2)
    n, h = 6, 88
    x, e = torch.randn(n, h, generator=g), torch.randn(n, h, generator=g)
    d1, d2 = torch.randn(n, h, generator=g).to(DT[dtype]), torch.randn(n, h, generator=g).to(DT[dtype])
    out = torch.empty(n, 2 * h, device=DEV, dtype=DT[dtype])
    for a, b in ((d1, d2), (d1, None), (None, None)):
        K().stream_concat(x.to(DEV), None if a is None else a.to(DEV), None if b is None else b.to(DEV), e.to(DEV), out)
        s = x.double() + ((a.double() if a is not None else 0) + (b.double() if b is not None else 0))
        close(out, torch.cat([s, e.double()], -1), dtype, "stream and embedding side by side", rel16=5e-3)
    wide = (torch.randn(n, h + 40, generator=g) * 3).to(DT[dtype])
    v = torch.randn(n, h, generator=g).to(DT[dtype])
    got = torch.empty(n, h, device=DEV, dtype=DT[dtype])
    K().sigmoid_mul(v.to(DEV), wide.to(DEV)[:, 40:], got)
    close(got, v.double() * torch.sigmoid(wide.double()[:, 40:]), dtype, "output gate", rel16=5e-3)
    heads, dv = 3, 40
    o = torch.randn(n, heads * dv, generator=g) * torch.tensor([0.01, 1.0, 30.0]).repeat_interleave(dv)   # heads of unequal size
    w = torch.randn(heads * dv, generator=g)
    gate = (torch.randn(n, heads * dv + 8, generator=g) * 2).to(DT[dtype])
    normed = torch.empty(n, heads * dv, device=DEV, dtype=DT[dtype])
    K().head_norm_gate(o.to(DEV), w.to(DEV), gate.to(DEV)[:, 8:], normed, num_heads=heads, eps=1e-5)
    want = plain.unit_rms(o.double().view(n, heads, dv), 1e-5).reshape(n, -1) * w.double() * torch.sigmoid(gate.double()[:, 8:])
    close(normed, want, dtype, "heads by their own root mean square", rel16=8e-3)


# ---- attention whose values are its keys -----------------------------------------------------------------
def _fill_cache(dtype, nh, nkv, hd, rot, style, positions, page, seed, eps=1e-5, base=777.0, boost=None):
    """Projections of len(positions) tokens of one sequence through the prep kernel into a paged cache; returns what the
    plain functions make of the same rows."""
    g = torch.Generator().manual_seed(seed)
    n = len(positions)
    width = nh * hd + nkv * hd + nh * hd
    proj = torch.randn(n, width, generator=g)
    if boost is not None:
        for t, f in boost.items():
            proj[t, nh * hd:(nh + nkv) * hd] *= f
    proj = proj.to(DT[dtype])
    qw, kw = torch.randn(nh * hd, generator=g), torch.randn(nkv * hd, generator=g)
    n_pages = -(-(max(positions) + 1) // page) + 3
    order = torch.randperm(n_pages, generator=g)[: -(-(max(positions) + 1) // page)].to(torch.int32)       # scattered pages
    kc = torch.zeros(n_pages, nkv, page, hd, dtype=DT[dtype], device=DEV)
    vc = torch.zeros_like(kc)
    pos = torch.tensor(positions, dtype=torch.int32)
    slots = (order[(pos // page).long()] * page + pos % page).to(torch.int32)
    q = torch.empty(n, nh, hd, dtype=DT[dtype], device=DEV)
    inv = torch.pow(torch.tensor(base, dtype=F64), -2.0 * torch.arange(rot // 2, dtype=F64) / max(rot, 1)).to(DEV) if rot else None
    K().projection_norm_rope_store(proj.to(DEV), 0, nh * hd, q, kc, vc, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                                   q_weight=qw.to(DEV), k_weight=kw.to(DEV), eps=eps, inv_freq=inv, rot_dim=rot, rope_style=style,
                                   positions=pos.to(DEV), slots=slots.to(DEV))
    p64 = proj.double()
    qn = (plain.unit_rms(p64[:, :nh * hd], eps) * qw.double()).view(n, nh, hd)
    kraw = p64[:, nh * hd:(nh + nkv) * hd]
    kn = (plain.unit_rms(kraw, eps) * kw.double()).view(n, nkv, hd)
    if rot:
        qn, kn = plain.rotate_pairs(qn, pos, rot, base), plain.rotate_pairs(kn, pos, rot, base)
    return SimpleNamespace(proj=proj, q=q, kc=kc, vc=vc, order=order, slots=slots, pos=pos, q_want=qn, k_want=kn,
                           v_want=kraw.view(n, nkv, hd), gate=p64[:, (nh + nkv) * hd:])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh, nkv, hd, rot", [(6, 2, 16, 8), (3, 3, 40, 40), (2, 1, 128, 0), (8, 2, 64, 32)])
def test_projection_norm_rotation_and_cache_write(dtype, nh, nkv, hd, rot):
    page = 8
    positions = [0, 1, 7, 8, 9, 70000][: 6 if rot else 5]                     # a far position: the angle is a float64 product
    c = _fill_cache(dtype, nh, nkv, hd, rot, 1, positions, page, seed=hd)
    close(c.q, c.q_want, dtype, "normalised, rotated queries", rel16=1e-2)
    cells = c.slots.long()
    k_got = c.kc.permute(0, 2, 1, 3).reshape(-1, nkv, hd)[cells.to(DEV)]
    v_got = c.vc.permute(0, 2, 1, 3).reshape(-1, nkv, hd)[cells.to(DEV)]
    close(k_got, c.k_want, dtype, "keys in their cells", rel16=1e-2)
    assert torch.equal(v_got.cpu().double(), c.v_want), "the values must be the keys exactly as projected"
    assert int((c.kc != 0).any(-1).any(1).sum()) == len(positions), "cells of other tokens were written"


def _plain_attention(c, nh, nkv, hd, scale, window, sink, gate):
    n = c.q_want.shape[0]
    group = torch.arange(nh) // (nh // nkv)
    pos = c.pos.long()
    scores = torch.einsum("ihd,jhd->hij", c.q_want, c.k_want[:, group]) * scale
    vis = (pos[None, :] <= pos[:, None]) & ((pos[:, None] - pos[None, :] < window) if window else torch.ones(n, n, dtype=torch.bool))
    p = plain.sink_softmax(scores, vis, sink) if sink is not None else torch.softmax(scores.masked_fill(~vis[None], -math.inf), -1)
    o = torch.einsum("hij,jhd->ihd", p, c.v_want[:, group]).reshape(n, nh * hd)
    return o * torch.sigmoid(gate) if gate is not None else o, p


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh, nkv, hd, window, page", [(6, 2, 16, 37, 16), (4, 4, 64, 33, 8), (8, 2, 64, 64, 16), (2, 1, 128, None, 32),
                                                      (3, 1, 24, 5, 16), (4, 2, 128, 150, 16)])
def test_attention_sees_window_and_sink_exactly(dtype, nh, nkv, hd, window, page):
    """Two keys are made to stand out by putting a multiple of a query into their cache cells (the norm over the projection
    would undo a scaled input): one just inside and one just outside the last token's window (without a window: at position
    1, hundreds of tokens back).  Queries: a portion of the last 7 tokens, then the same tokens one by one, then the first ones."""
    n = 300 if window else 1500                 # without a window: enough keys that decoding cuts them into several parts
    w = window or n
    inside, outside = (max(n - w, 1), n - w - 1) if window else (1, -1)
    c = _fill_cache(dtype, nh, nkv, hd, min(hd, 16) // 2 * 2, 1, list(range(n)), page, seed=nh * hd)
    first_of_group = torch.arange(nkv) * (nh // nkv)
    for j, asker in ((inside, n - 1), (outside, n - 2)):
        if j < 0:
            continue
        key = (1.5 * c.q_want[asker, first_of_group]).to(DT[dtype])                       # [nkv, hd]
        cell = int(c.slots[j])
        c.kc[cell // page, :, cell % page, :] = key.to(DEV)
        c.k_want[j] = key.double()
    sink = torch.randn(nh, generator=torch.Generator().manual_seed(5)) * 2
    scale = 2.0 / math.sqrt(hd)
    want, p = _plain_attention(c, nh, nkv, hd, scale, window, sink.double(), c.gate)
    assert p[:, n - 1, inside].max() > 0.2, "the stand-out key inside the window must matter"
    if outside >= 0:
        assert p[:, n - 1, outside].max() == 0 and p[:, n - 2, outside].max() > 0.2     # one token earlier it was still seen
    bt = torch.full((1, max(64, c.order.numel())), -1, dtype=torch.int32)
    bt[0, : c.order.numel()] = c.order
    gate = c.proj.to(DEV)[:, (nh + nkv) * hd:]
    for rows in (list(range(n - 7, n)), [n - 2], [n - 1], list(range(0, 3)), list(range(n - 200, n)), list(range(0, 130))):
        r = torch.tensor(rows)
        meta = SimpleNamespace(positions=c.pos[r].to(DEV), seq_of_token=torch.zeros(len(rows), dtype=torch.int32, device=DEV),
                               cu_q=torch.tensor([0, len(rows)], dtype=torch.int32, device=DEV),
                               ctx_len=torch.tensor([rows[-1] + 1], dtype=torch.int32, device=DEV), block_table=bt.to(DEV),
                               slots=c.slots[r].to(DEV), num_seqs=1, num_tokens=len(rows), max_q_len=len(rows), max_ctx=rows[-1] + 1,
                               decode_only=len(rows) == 1, h_q_len=[len(rows)], h_ctx_len=[rows[-1] + 1])
        out = torch.empty(len(rows), nh * hd, dtype=DT[dtype], device=DEV)
        K().sink_attention(c.q[r.to(DEV)].contiguous(), c.kc, c.vc, out, meta, num_heads=nh, num_kv_heads=nkv, head_dim=hd, scale=scale,
                           window=window, sink=sink.to(DEV), gate=gate[r.to(DEV)])
        close(out, want[r], dtype, f"attention rows {rows[0]}..{rows[-1]}", rel16=2.5e-2)
    # without the sink the first tokens come out differently: it is in the denominator
    no_sink, _ = _plain_attention(c, nh, nkv, hd, scale, window, None, c.gate)
    assert (no_sink[:3] - want[:3]).abs().max() > 1e-3


# ---- the matrix-memory scan ---------------------------------------------------------------------------------------
def _plain_scan(proj, gates, bias, H, d, dv, cap, state=None):
    """o [T, H * dv] and the state after the rows, by the plain recurrence (no norm, no gate, no projection)."""
    T = proj.shape[0]
    q = proj[:, :H * d].view(T, H, d) * d ** -0.5
    k = proj[:, H * d:2 * H * d].view(T, H, d)
    v = proj[:, 2 * H * d:2 * H * d + H * dv].view(T, H, dv)
    a = plain.soft_cap(gates[:, :H] + bias[:H], cap)
    b = torch.nn.functional.logsigmoid(plain.soft_cap(gates[:, H:] + bias[H:], cap))
    C, n, m = state if state is not None else (torch.zeros(H, d, dv, dtype=F64), torch.zeros(H, d, dtype=F64), torch.zeros(H, dtype=F64))
    out = torch.zeros(T, H, dv, dtype=F64)
    for s in range(T):
        m_new = torch.maximum(b[s] + m, a[s])
        keep, take = torch.exp(b[s] + m - m_new), torch.exp(a[s] - m_new)
        C = keep[:, None, None] * C + take[:, None, None] * k[s][:, :, None] * v[s][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[s]
        m = m_new
        out[s] = torch.einsum("hdv,hd->hv", C, q[s]) / (torch.maximum((n * q[s]).sum(-1).abs(), torch.exp(-m)) + 1e-6)[:, None]
    return out.reshape(T, H * dv), (C, n, m)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, d, dv", [(3, 24, 40), (2, 16, 24), (4, 32, 32), (1, 160, 16), (1, 8, 8), (2, 64, 128), (1, 300, 6), (5, 128, 48)])
def test_matrix_memory_scan_cut_into_steps_with_slots_used_again(dtype, H, d, dv):
    from iian_b200.parts.matrix_memory import state_block_floats, state_columns
    g = torch.Generator().manual_seed(H * d + dv)
    cap = 6.0
    lens = [37, 1, 12]
    cb = state_columns(d, dv)
    state = torch.full((3, H, dv // cb, state_block_floats(d, cb)), 7.0, device=DEV)          # slots hold leftovers ...
    extra = 5                                                                                 # the product carries more columns
    width = 2 * H * d + H * dv + extra
    seqs = []
    for L in lens:
        proj = (torch.randn(L, width, generator=g) * 1.5).to(DT[dtype])
        gates = torch.randn(L, 2 * H, generator=g) * 6                                         # the cap matters
        seqs.append((proj, gates))
    bias = torch.randn(2 * H, generator=g)
    wants = [_plain_scan(p.double(), gt.double(), bias.double(), H, d, dv, cap)[0] for p, gt in seqs]
    slots = [2, 0, 2]                                                       # the third sequence inherits the first one's slot
    got = [[] for _ in lens]
    # sequences 0 and 1 side by side in portions (a single token beside a portion), then sequence 2 alone in slot 2
    plan = [[(0, 0, 5), (1, 0, 1)], [(0, 5, 7)], [(0, 7, 8)], [(0, 8, 37)], [(2, 0, 2)], [(2, 2, 3)], [(2, 3, 12)]]
    fresh = {0: True, 1: True, 2: True}
    for step in plan:
        rows_p, rows_g, cu, sl = [], [], [0], []
        for s, lo, hi in step:
            if fresh[s]:
                state[slots[s]].zero_()                                      # ... and are zeroed when a request takes them
                fresh[s] = False
            rows_p.append(seqs[s][0][lo:hi])
            rows_g.append(seqs[s][1][lo:hi])
            cu.append(cu[-1] + hi - lo)
            sl.append(slots[s])
        # a padding sequence (slot -1) rides along: it must change nothing and yield zeros
        rows_p.append(seqs[0][0][:1]); rows_g.append(seqs[0][1][:1]); cu.append(cu[-1] + 1); sl.append(-1)
        proj, gates = torch.cat(rows_p).to(DEV), torch.cat(rows_g).to(DEV)
        out = torch.full((proj.shape[0], H * dv), 9.0, device=DEV)
        K().matrix_memory_scan(proj, 0, H * d, 2 * H * d, gates, bias.to(DEV), state, torch.tensor(cu, dtype=torch.int32, device=DEV),
                               torch.tensor(sl, dtype=torch.int32, device=DEV), out, num_heads=H, dim=d, v_dim=dv, columns=cb,
                               cap=cap, q_scale=d ** -0.5)
        for j, (s, lo, hi) in enumerate(step):
            got[s].append(out[cu[j]:cu[j + 1]].cpu())
        assert out[cu[-2]:].abs().max() == 0
    for s in range(3):
        close(torch.cat(got[s]), wants[s], "float32", f"sequence {s} of {H} heads {d} x {dv}", abs32=5e-5)


# ---- experts chosen by a table --------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n, experts, top, width, ff, limit", [(1, 3, 1, 64, 32, 1.0), (9, 5, 2, 96, 48, 1.5), (300, 8, 3, 128, 64, 0.7),
                                                               (70, 1, 1, 64, 40, 3.0)])
def test_table_routed_experts(dtype, n, experts, top, width, ff, limit):
    from iian_b200.config.spec import PartSpec
    from iian_b200.parts.base import FEED_FORWARDS
    from iian_b200.engine.runner import StepContext, Workspace
    g = torch.Generator().manual_seed(n + experts)
    vocab = 31
    spec = PartSpec("routed_experts", {"hidden_size": width, "num_experts": experts, "top": top, "intermediate_size": ff,
                                       "activation": "clamped_swish", "limit": limit, "score": "table", "vocab_size": vocab,
                                       "weight_on": "output"})
    part = FEED_FORWARDS.build(spec, DT[dtype], torch.device(DEV))
    t = {"table": torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(vocab)]).to(torch.int32)}
    for e in range(experts):
        t[f"e{e}.gate"] = (torch.randn(ff, width, generator=g) * 0.3).to(DT[dtype])
        t[f"e{e}.up"] = (torch.randn(ff, width, generator=g) * 0.3).to(DT[dtype])
        t[f"e{e}.down"] = (torch.randn(width, ff, generator=g) * 0.3).to(DT[dtype])
    part.bind({k: v.to(DEV) for k, v in t.items()})
    tokens = torch.randint(0, vocab, (n,), generator=g).to(torch.int32)
    x = torch.randn(n, width, generator=g).to(DT[dtype])
    fc = {"expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    want = plain.table_routed_ff(x.double(), tokens.long(), {k: (v.double() if v.is_floating_point() else v) for k, v in t.items()}, "", fc)
    ctx = StepContext(Workspace(torch.device(DEV)))
    ctx.tokens = tokens.to(DEV)
    close(part.forward(x.to(DEV), ctx), want, dtype, "experts by table", rel16=3e-2)
    # selected rows: row r of the input belongs to token rows[r]
    rows = torch.tensor([n - 1, 0, n // 2], dtype=torch.int32)
    got = part.forward(x[rows.long()].contiguous().to(DEV), ctx, rows=rows.to(DEV))
    close(got, want[rows.long()], dtype, "experts by table on selected rows", rel16=3e-2)


# ---- whole models ---------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("lekilix_gpu")
    return {name: write_case(root, name) for name in CONFIGS}


LENGTHS = {"U": [1, 9, 40, 75, 130], "V": [3, 35, 70, 20, 100], "W": [2, 90, 33, 150], "X": [70, 5, 120, 33], "Y": [41, 3, 77]}
_plain_cache = {}


def rounded_plain(folder, reqs, dtype):
    """The plain implementation with the input and the result of every matrix product rounded to ``dtype``: how far
    rounding alone moves the logits at each position.  Random weights make some positions touchy (a memory read out where
    little is stored, a peaky softmax); there the engine may be off by as much as this is, and nowhere else."""
    cfg, w = plain.load_folder(folder)
    plain.product_rounding = lambda z: z.to(DT[dtype]).to(F64)
    try:
        return {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    finally:
        plain.product_rounding = None


def requests_and_plain(folders, name, lengths=None, seed=40, folder=None, reqs=None):
    key = (folder or name, tuple(lengths or LENGTHS[name]), seed)
    if key not in _plain_cache:
        if reqs is None:
            reqs = {f"r{i}": random_tokens(CONFIGS[name]["vocab"], n, seed + i) for i, n in enumerate(lengths or LENGTHS[name])}
        want = plain_logits(folder or folders[name], reqs)
        rough = {dt: rounded_plain(folder or folders[name], reqs, dt) for dt in DT}
        _plain_cache[key] = (reqs, (want, rough))
    return _plain_cache[key]


def run_trace(folder, name, dtype, reqs, want_rough, steps, max_tokens, what, max_requests=4):
    from iian_b200.engine.replay import TraceReplayer
    want, rough = want_rough
    rp = TraceReplayer.from_folder(folder, dtype, max_tokens, BLOCK_SIZE[name], max_requests)
    got = replay_and_collect(rp, steps)
    rp.runner.check_device_status()
    rp.runner.manager.check_invariants()
    assert all(p.num_free == p.num_blocks for p in rp.runner.manager.pools), "pages were lost"
    assert len(got) == sum(len(t) for t in reqs.values())
    scale = max(w.abs().max().item() for w in want.values())
    floor = 3e-5 * max(1.0, scale) if dtype == "float32" else 3e-2 * scale
    over = []
    for (rid, pos) in sorted(got):
        e = (got[(rid, pos)].double() - want[rid][pos]).abs().max().item()
        tol = floor + 3.0 * (rough[dtype][rid][pos] - want[rid][pos]).abs().max().item()
        assert e <= 3.0 * tol, f"{name} {dtype} {what}: first wrong logits at {(rid, pos)}: {e:.3g} > 3 x {tol:.3g}; worst {max_error(got, want)}"
        if not e <= tol:
            over.append((rid, pos, e, tol))
    # the rounded oracle is ONE draw of the rounding noise at a touchy position: a few positions may be further off than it
    assert len(over) <= 0.02 * len(got), f"{name} {dtype} {what}: {len(over)} of {len(got)} positions beyond rounding, first {over[0]}"
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_replay_under_every_cut(folders, name, dtype):
    reqs, want = requests_and_plain(folders, name)
    rounded = max(-(-len(t) // 64) * 64 for t in reqs.values())
    whole = run_trace(folders[name], name, dtype, reqs, want, trace_whole(reqs), rounded, "whole")
    for what, steps, cap, live in (("tail", trace_tail(reqs, 40), rounded, 4), ("portions", trace_portions(reqs), rounded, 4),
                                   ("mixed", trace_mixed(reqs, 2 * rounded, seed=1), 2 * rounded, 4),
                                   ("mixed, two slots", trace_mixed(reqs, rounded + 64, seed=2, max_live=2), rounded + 64, 2)):
        got = run_trace(folders[name], name, dtype, reqs, want, steps, cap, what, live)
        if dtype == "float32":      # every sum has an order fixed by the token's own position: the cut changes no bit
            worst = max((got[k] - whole[k]).abs().max().item() for k in got)
            assert worst <= 2e-6, f"{name} {what}: differs from the whole prompt by {worst}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_a_far_key(folders, dtype):
    """200 tokens decoded one by one behind a short prompt (windows pass over decoded tokens, pages are given back on the way,
    the memories run on), and a token whose embedding is large, met once early and again at the end: the memories carry it."""
    reqs, want = requests_and_plain(folders, "U", [230], seed=90)
    run_trace(folders["U"], "U", dtype, reqs, want, trace_tail(reqs, 200), 256, "long decoding")
    reqs, want = requests_and_plain(folders, "W", [200], seed=91)
    run_trace(folders["W"], "W", dtype, reqs, want, trace_tail(reqs, 190), 256, "long decoding")
    d = folders["U"] + "_far"
    if not os.path.isdir(d):
        cfg, w = plain.load_folder(folders["U"])
        from iian_b200.weights.safetensors_io import write_safetensors
        w = {k: (v.float() if v.is_floating_point() else v) for k, v in w.items()}
        w["embed"][7] *= 6.0
        os.makedirs(d)
        write_safetensors(os.path.join(d, "model.safetensors"), {k: (v.to(torch.bfloat16) if v.is_floating_point() else v) for k, v in w.items()})
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
    toks = [t if t != 7 else 8 for t in random_tokens(211, 400, 3)]
    toks[4] = toks[-1] = toks[-30] = 7
    reqs, want = requests_and_plain(folders, "U", folder=d, reqs={"far": toks})
    run_trace(d, "U", dtype, reqs, want, trace_whole(reqs), 448, "far key, whole")
    run_trace(d, "U", dtype, reqs, want, trace_tail(reqs, 40), 448, "far key, decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(folders, dtype):
    from iian_b200 import EngineConfig, SchedulerConfig
    from iian_b200.engine.engine import Engine
    name = "V"
    cfg, w = plain.load_folder(folders[name])
    prompts = [random_tokens(300, n, 70 + i) for i, n in enumerate([1, 6, 30, 50, 77])]
    want = []
    for p in prompts:
        toks, margins = list(p), []
        for _ in range(10):
            row = plain.forward(cfg, w, toks)[-1]
            top = torch.topk(row, 2).values
            margins.append((top[0] - top[1]).item())
            toks.append(int(torch.argmax(row)))
        want.append((toks[len(p):], margins))
    for kw in (dict(budget=1024, kv_cache_tokens=1024, cuda_graphs=True), dict(budget=13, kv_cache_tokens=1024, cuda_graphs=True),
               dict(budget=64, kv_cache_tokens=128, cuda_graphs=False)):
        sched = SchedulerConfig(max_num_batched_tokens=kw.pop("budget"), max_num_seqs=8)
        eng = Engine(folders[name], EngineConfig(dtype=dtype, block_size=BLOCK_SIZE[name], sched=sched, max_model_len=128, **kw))
        got = eng.generate(prompts, max_tokens=10, temperature=0.0)
        for g, (wt, margins) in zip(got, want):
            for k, (a, b) in enumerate(zip(g, wt)):
                if a != b:
                    assert dtype == "bfloat16" and margins[k] < 0.05, f"{kw}: token {k}: {g} vs {wt} (margin {margins[k]:.4f})"
                    break
        if kw.get("cuda_graphs"):
            assert eng.runner.num_graphs >= 1
        eng.cache.check_invariants()
        assert all(p.num_free == p.num_blocks for p in eng.cache.pools)


def test_trace_runner_as_a_program(folders, tmp_path):
    reqs, (want, _) = requests_and_plain(folders, "W")
    steps = trace_mixed(reqs, 384, seed=4)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["W"], "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "384", "--block-size", "32"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    fed = {}
    for s in steps:
        rows = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, 97)
        r = 0
        for ent in s["entries"]:
            for k in ent["want"]:
                p = fed.get(ent["id"], 0) + k
                assert np.abs(rows[r] - want[ent["id"]][p].numpy()).max() < 1e-4
                r += 1
            fed[ent["id"]] = fed.get(ent["id"], 0) + len(ent["tokens"])
