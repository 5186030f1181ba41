"""Galodra on the GPU.  Each new kernel alone against the plain functions of tests/plain_galodra.py (the fused
LayerNorm of the gated sum, the depth mix, the gated activation, attention over the cached latent with a stand-out key
just inside and just outside the window, at page borders and far away, in prompts and in decoding, with and without
a sink, routed experts); then whole models under every way of cutting the work, in 32-bit and in bfloat16; greedy
generation through the engine's entry point with and without CUDA graphs; the trace runner as a program."""
import json
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_galodra as plain
from galodra_cases import BLOCK_SIZE, CONFIGS, plain_logits, write_case
from helpers import first_bad, max_error, random_tokens, replay_and_collect, trace_mixed, trace_portions, trace_tail, trace_whole

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


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
@pytest.mark.parametrize("h", [96, 256, 1000])
def test_gated_sum_layer_norm(dtype, h):
    g = torch.Generator().manual_seed(h)
    n = 7
    x = torch.randn(n, h, generator=g) * 2 + 0.5
    wide = (torch.randn(n, h + 24, generator=g)).to(DT[dtype])              # sub is a column slice of a wider matrix
    gate = (torch.randn(n, 2 * h, generator=g) * 2).to(DT[dtype])
    gb, w, b = torch.randn(h, generator=g), torch.rand(h, generator=g) + 0.5, torch.randn(h, generator=g)
    sub, gl = wide[:, 24:], gate[:, h:]
    for use_gate in (True, False):
        s = sub.double() * (torch.sigmoid(gl.double() + gb.double()) if use_gate else 1.0)
        want = plain.layer_norm(1.7 * x.double() + s, w.double(), b.double(), 1e-5)
        out = torch.empty(n, h, device=DEV)
        act = torch.empty(n, h, device=DEV, dtype=DT[dtype])
        K().gated_add_layer_norm(x.to(DEV), wide.to(DEV)[:, 24:], gate.to(DEV)[:, h:] if use_gate else None,
                                 gb.to(DEV) if use_gate else None, w.to(DEV), b.to(DEV), 1.7, 1e-5, out, act)
        close(out, want, "float32", f"gated sum norm, gate={use_gate}")
        close(act, want, dtype, "its copy in the activation dtype", rel16=5e-3)
    # the plain norm of the stream (what closes the model)
    K().gated_add_layer_norm(x.to(DEV), None, None, None, w.to(DEV), b.to(DEV), 1.0, 1e-5, out, None)
    close(out, plain.layer_norm(x.double(), w.double(), b.double(), 1e-5), "float32", "plain layer norm")


def test_depth_mix_reads_selected_rows():
    g = torch.Generator().manual_seed(1)
    terms = [torch.randn(9, 40, generator=g) for _ in range(3)]
    last = torch.randn(4, 40, generator=g)
    coef = torch.randn(4, generator=g)
    rows = torch.tensor([8, 0, 3, 3], dtype=torch.int32)
    want = sum(coef[j] * terms[j][rows.long()] for j in range(3)) + coef[3] * last
    out = torch.empty(4, 40, device=DEV)
    act = torch.empty(4, 40, device=DEV, dtype=torch.bfloat16)
    K().depth_mix([t.to(DEV) for t in terms] + [last.to(DEV)], coef.to(DEV), rows.to(DEV), True, out, act)
    close(out, want, "float32", "depth mix")
    close(act, want, "bfloat16", "depth mix copy", rel16=5e-3)
    full = sum(coef[j] * terms[j] for j in range(3))
    out9 = torch.empty(9, 40, device=DEV)
    K().depth_mix([t.to(DEV) for t in terms], coef[:3].contiguous().to(DEV), None, False, out9, None)
    close(out9, full, "float32", "depth mix of all rows")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("f, interleave", [(48, 8), (50, 0)])
def test_gated_activation(dtype, f, interleave):
    g = torch.Generator().manual_seed(f)
    gate, up = torch.randn(5, f, generator=g) * 3, torch.randn(5, f, generator=g)
    if interleave:
        gu = torch.stack([gate.view(5, f // 8, 8), up.view(5, f // 8, 8)], dim=2).reshape(5, 2 * f)
    else:
        gu = torch.cat([gate, up], dim=1)
    wide = torch.cat([gu, torch.randn(5, 10, generator=g)], dim=1).to(DT[dtype]).to(DEV)
    gq, uq = gate.to(DT[dtype]).double(), up.to(DT[dtype]).double()
    for name, fn in (("gelu_tanh", plain.gelu_tanh), ("silu", plain.silu)):
        out = torch.empty(5, f, device=DEV, dtype=DT[dtype])
        K().gated_act(wide[:, : 2 * f], out, interleave, name)
        close(out, fn(gq) * uq, dtype, name, rel16=5e-3)


# ---- attention over the cached latent -----------------------------------------------------------------
def paged_meta(ctx_lens, q_lens, page_size, n_pages, seed=0):
    """Block tables that scatter every sequence's pages over the pool in a random order."""
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    max_blocks = max(-(-c // page_size) for c in ctx_lens)
    bt = torch.full((len(ctx_lens), max_blocks), -1, dtype=torch.int32)
    positions, seq = [], []
    for s, (c, ql) in enumerate(zip(ctx_lens, q_lens)):
        for b in range(-(-c // page_size)):
            bt[s, b] = order.pop()
        positions += list(range(c - ql, c))
        seq += [s] * ql
    cu = [0]
    for ql in q_lens:
        cu.append(cu[-1] + ql)
    return SimpleNamespace(positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                           seq_of_token=torch.tensor(seq, dtype=torch.int32, device=DEV),
                           cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV), num_seqs=len(ctx_lens), max_q_len=max(q_lens),
                           max_ctx=max(ctx_lens),
                           block_table=bt.to(DEV), ctx_len=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV)), bt


def plain_latent_rows(q, rows, sink, scale, window, rank, pos):
    """One query row per head against the rows of its own sequence, written with the plain softmax."""
    t = rows.shape[0]
    sc = torch.einsum("hd,jd->hj", q, rows)[:, None, :] * scale                    # [H, 1, T]
    vis = plain.window_mask(t, window)[pos][None, :]
    p = plain.sink_softmax(sc, vis, sink)
    return torch.einsum("hj,jr->hr", p[:, 0], rows[:, :rank])


def attend(kernel, q, cache, out, sink, meta, **kw):
    """The general kernel, or the tensor-core one with its keys in one part or cut into three."""
    if kernel == "general":
        K().latent_attention(q, cache, out, sink, meta, **kw)
    else:
        assert K().latent_attention_mma_ok(q, cache, kw["rank"])
        K().latent_attention_mma(q, cache, out, sink, meta, parts=1 if kernel == "mma" else 3, **kw)


@pytest.mark.parametrize("dtype, kernel, rank, rot", [("float32", "general", 24, 8), ("bfloat16", "general", 24, 8),
                                                      ("bfloat16", "mma", 64, 32), ("bfloat16", "mma3", 64, 48),
                                                      ("bfloat16", "mma", 128, 32), ("bfloat16", "mma3", 512, 64)])
@pytest.mark.parametrize("window, far", [(37, False), (None, True), (33, False), (64, False)])
def test_latent_attention_sees_the_window_exactly(dtype, kernel, rank, rot, window, far):
    """One key is made to stand out (its row is aligned with the query, scaled up): just inside the window it must
    carry the output, one step further out it must vanish; without a window a key hundreds of positions back counts.
    Queries sit at page borders and in the middle; once as the last rows of a prompt's portion, once as single
    decoded tokens."""
    heads, page = (3 if rank < 512 else 5), 16
    width = rank + rot
    g = torch.Generator().manual_seed(5)
    ctx = [300, 97, 64, 65]
    for q_lens in ([20, 5, 64, 2], [1, 1, 1, 1], [1, 30, 1, 1]):
        meta, bt = paged_meta(ctx, q_lens, page, 40, seed=len(q_lens))
        seqs = [torch.randn(c, width, generator=g) * 0.3 for c in ctx]                   # rows of the cache, per sequence
        qs = []
        for s, (c, ql) in enumerate(zip(ctx, q_lens)):
            q = torch.randn(ql, heads, width, generator=g) * 0.3 * (32.0 / width) ** 0.5
            p_last = c - 1
            for off, head in (((window - 1) if window else (p_last - 3 if far else 7), 0), ((window if window else 11), 1)):
                j = p_last - off
                if j >= 0:
                    direction = torch.randn(width, generator=g) * (32.0 / width) ** 0.5
                    seqs[s][j] = direction * 1.5
                    q[-1, head] = direction * 4.0            # the last query's head looks straight at key j
            qs.append(q)
        q_all = torch.cat(qs).to(DT[dtype])
        cache = torch.zeros(40, page, width, dtype=DT[dtype])
        for s, rows in enumerate(seqs):
            for j in range(rows.shape[0]):
                cache[bt[s, j // page], j % page] = rows[j].to(DT[dtype])
        out = torch.empty(q_all.shape[0], heads, rank, device=DEV, dtype=DT[dtype])
        sink = torch.tensor([0.5, -1.0, 2.0, 0.0, 1.0][:heads])
        attend(kernel, q_all.to(DEV), cache.to(DEV), out, sink.to(DEV), meta, num_heads=heads, rank=rank, scale=0.2, window=window)
        t0 = 0
        for s, (c, ql) in enumerate(zip(ctx, q_lens)):
            rows = seqs[s].to(DT[dtype]).double()
            for i in range(ql):
                pos = c - ql + i
                want = plain_latent_rows(q_all[t0 + i].double(), rows[: pos + 1], sink.double(), 0.2, window, rank, pos)
                close(out[t0 + i], want, dtype, f"sequence {s} position {pos} (window {window}, q_lens {q_lens})")
            t0 += ql
        # without the sink the weights sum to one
        attend(kernel, q_all.to(DEV), cache.to(DEV), out, None, meta, num_heads=heads, rank=rank, scale=0.2, window=window)
        rows = seqs[0].to(DT[dtype]).double()
        sc = (q_all[q_lens[0] - 1].double() @ rows.T) * 0.2
        vis = plain.window_mask(ctx[0], window)[ctx[0] - 1]
        want = torch.softmax(sc.masked_fill(~vis[None], float("-inf")), dim=-1) @ rows[:, :rank]
        close(out[q_lens[0] - 1], want, dtype, "no sink")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_prep_and_head_products(dtype):
    """The latent's norm, both rotations (partial: 8 of 12 rotated entries), the cache write at scattered cells, and the
    per-head products in both orientations."""
    heads, dim, rot, rank, vdim, rd, n = 3, 16, 12, 40, 24, 8, 6
    g = torch.Generator().manual_seed(9)
    width = rank + rot
    qd = (torch.randn(n, 5 + heads * (dim + rot) + width, generator=g)).to(DT[dtype])
    q_off, dkv_off = 5, 5 + heads * (dim + rot)
    pos = torch.tensor([0, 1, 17, 300, 4095, 70000], dtype=torch.int32)
    slots = torch.tensor([3, 40, -1, 7, 0, 63], dtype=torch.int32)
    nw = torch.rand(rank, generator=g) + 0.5
    inv = torch.pow(torch.tensor(30000.0, dtype=torch.float64), -2.0 * torch.arange(rd // 2, dtype=torch.float64) / rd)
    cache = torch.zeros(4, 16, width, device=DEV, dtype=DT[dtype])
    q_cat = torch.zeros(n, heads, width, device=DEV, dtype=DT[dtype])
    K().latent_prep(qd.to(DEV), q_off, dkv_off, cache, q_cat, nw.to(DEV), inv.to(DEV), pos.to(DEV), slots.to(DEV),
                    num_heads=heads, dim=dim, rot=rot, rank=rank, rot_dims=rd, eps=1e-5)
    x = qd.double()
    dkv = x[:, dkv_off:]
    c = plain.rms_norm(dkv[:, :rank], nw.double(), 1e-5)
    kr = plain.rotate_half(dkv[:, rank:], pos, rd, 30000.0)
    q = x[:, q_off:dkv_off].view(n, heads, dim + rot)
    qr = plain.rotate_half(q[..., dim:], pos, rd, 30000.0)
    flat = cache.view(-1, width)
    for t in range(n):
        if slots[t] >= 0:
            close(flat[slots[t]], torch.cat([c[t], kr[t]]), dtype, f"cache row of token {t}", rel16=6e-3)
    untouched = [s for s in range(64) if s not in slots.tolist()]
    assert float(flat[untouched].abs().max()) == 0.0
    close(q_cat[..., rank:], qr, dtype, "rotated query parts", rel16=6e-3)
    # the per-head products: up to 8 tokens and more (in bfloat16 these are different kernels), both orientations
    uk = (torch.randn(heads * dim, rank, generator=g) * 0.3).to(DT[dtype])
    uv = (torch.randn(heads * vdim, rank, generator=g) * 0.3).to(DT[dtype])
    for nn in (n, 1, 8, 9, 70):
        qd2 = torch.randn(nn, q_off + heads * (dim + rot) + 3, generator=g).to(DT[dtype])
        q2 = qd2.double()[:, q_off:q_off + heads * (dim + rot)].view(nn, heads, dim + rot)
        q_cat2 = torch.full((nn, heads, width), 7.0, device=DEV, dtype=DT[dtype])
        K().head_linear(qd2.to(DEV), q_off, dim + rot, uk.to(DEV), dim * rank, rank, 1, q_cat2.view(nn, heads * width), 0, width,
                        num_heads=heads, n_in=dim, n_out=rank)
        want = torch.einsum("thd,hdr->thr", q2[..., :dim], uk.double().view(heads, dim, rank))
        close(q_cat2[..., :rank], want, dtype, f"query moved into latent space, {nn} tokens")
        assert float((q_cat2[..., rank:].float() - 7.0).abs().max()) == 0.0, "the rotated parts behind it were touched"
        lat = torch.randn(nn, heads * rank, generator=g).to(DT[dtype])
        o = torch.empty(nn, heads * vdim, device=DEV, dtype=DT[dtype])
        K().head_linear(lat.to(DEV), 0, rank, uv.to(DEV), vdim * rank, 1, rank, o, 0, vdim, num_heads=heads, n_in=rank, n_out=vdim)
        want = torch.einsum("thr,hvr->thv", lat.double().view(nn, heads, rank), uv.double().view(heads, vdim, rank))
        close(o.view(nn, heads, vdim), want, dtype, f"values lifted per head, {nn} tokens")


# ---- routed experts -----------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts, top, n, ff", [(5, 2, 37, 48), (8, 1, 200, 48), (3, 3, 1, 50), (70, 4, 90, 48), (6, 2, 700, 128)])
def test_routed_experts_part(dtype, experts, top, n, ff):
    """Scores, choices, the plan, both grouped products (in bfloat16 on tcgen05 when the expert's width is a multiple of
    8, else and in 32-bit the general kernel; several row tiles per expert in the last case) and the sum."""
    from iian_b200.config.spec import PartSpec
    from iian_b200.engine.runner import StepContext, Workspace
    from iian_b200.parts.experts import RoutedExperts
    width = 64
    g = torch.Generator().manual_seed(experts)
    part = RoutedExperts(PartSpec("routed_experts", {"hidden_size": width, "num_experts": experts, "top": top,
                                                     "intermediate_size": ff}), DT[dtype], torch.device(DEV))
    w = {"router": torch.randn(experts, width, generator=g) * 0.5}
    for e in range(experts):
        w[f"e{e}.gate"] = torch.randn(ff, width, generator=g) * 0.2
        w[f"e{e}.up"] = torch.randn(ff, width, generator=g) * 0.2
        w[f"e{e}.down"] = torch.randn(width, ff, generator=g) * 0.2
    w = {k: v.to(DT[dtype]) for k, v in w.items()}
    part.bind({k: v.to(DEV) for k, v in w.items()})
    h = torch.randn(n, width, generator=g).to(DT[dtype])
    ctx = StepContext(Workspace(torch.device(DEV)))
    from iian_b200.ops import cuda_backend
    before = dict(cuda_backend.LAUNCHES_BY_ENTRY)
    out = part.forward(h.to(DEV), ctx)
    served = {k for k, v in cuda_backend.LAUNCHES_BY_ENTRY.items() if v > before.get(k, 0)}
    assert ("gemm_tcgen05_grouped" if dtype == "bfloat16" and ff % 8 == 0 else "moe_grouped_gemm") in served, served
    want = plain.routed_ff(h.double(), {k: v.double() for k, v in w.items()}, "", experts, top)
    close(out, want, dtype, f"{top} of {experts} experts, {n} tokens", rel16=3e-2, abs32=1e-5)
    K().check_device_status()
    ids = ctx.buf("expert_ids", (n, top), torch.int32).cpu()
    want_ids = torch.topk(torch.sigmoid(h.double() @ w["router"].double().T), top, dim=-1).indices
    assert torch.equal(ids.long(), want_ids)


# ---- whole models --------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("galodra")
    return {n: write_case(root, n) for n in CONFIGS}


LENGTHS = {"P": [1, 9, 40, 75, 130], "Q": [3, 35, 70, 20, 100], "R": [2, 90, 33, 150]}
_plain_cache = {}


def requests_and_plain(folders, name, lengths=None, seed=40):
    key = (name, tuple(lengths or LENGTHS[name]), seed)
    if key not in _plain_cache:
        reqs = {f"r{i}": random_tokens(CONFIGS[name]["vocab"], n, seed + i) for i, n in enumerate(lengths or LENGTHS[name])}
        _plain_cache[key] = (reqs, plain_logits(folders[name], reqs))
    return _plain_cache[key]


def run_trace(folder, name, dtype, reqs, want, steps, max_tokens, what):
    from iian_b200.engine.replay import TraceReplayer
    rp = TraceReplayer.from_folder(folder, dtype, max_tokens, BLOCK_SIZE[name], 4)
    got = replay_and_collect(rp, steps)
    rp.runner.check_device_status()
    rp.runner.manager.check_invariants()
    assert all(p.num_free == p.num_blocks for p in rp.runner.manager.pools), "pages were lost"
    assert len(got) == sum(len(t) for t in reqs.values())
    scale = max(w.abs().max().item() for w in want.values())
    tol = 3e-5 * max(1.0, scale) if dtype == "float32" else 3e-2 * scale
    bad = first_bad(got, want, tol)
    assert bad is None, f"{name} {dtype} {what}: first wrong logits at {bad} (tol {tol:.3g}); worst {max_error(got, want)}"
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_replay_under_every_cut(folders, name, dtype):
    reqs, want = requests_and_plain(folders, name)
    rounded = max(-(-len(t) // 64) * 64 for t in reqs.values())
    whole = run_trace(folders[name], name, dtype, reqs, want, trace_whole(reqs), rounded, "whole")
    for what, steps, cap in (("tail", trace_tail(reqs, 40), rounded), ("portions", trace_portions(reqs), rounded),
                             ("mixed", trace_mixed(reqs, 2 * rounded, seed=1), 2 * rounded),
                             ("mixed again", trace_mixed(reqs, rounded + 64, seed=2, max_live=3), rounded + 64)):
        got = run_trace(folders[name], name, dtype, reqs, want, steps, cap, what)
        if dtype == "float32":      # every sum has an order fixed by the token's own position: the cut changes no bit
            worst = max((got[k] - whole[k]).abs().max().item() for k in got)
            assert worst <= 2e-6, f"{name} {what}: differs from the whole prompt by {worst}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_a_far_key(folders, dtype):
    """200 tokens decoded one by one behind a short prompt (windows pass over decoded tokens, pages are given back on the
    way), and a token whose embedding is large, met once early and again at the end, in a layer without window."""
    reqs, want = requests_and_plain(folders, "P", [230], seed=90)
    run_trace(folders["P"], "P", dtype, reqs, want, trace_tail(reqs, 200), 256, "long decoding")
    d = folders["P"] + "_far"
    if not os.path.isdir(d):
        cfg, w = plain.load_folder(folders["P"])
        from iian_b200.weights.safetensors_io import write_safetensors
        w = {k: v.float() for k, v in w.items()}
        w["embed"][7] *= 6.0
        os.makedirs(d)
        write_safetensors(os.path.join(d, "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in w.items()})
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
    toks = [t if t != 7 else 8 for t in random_tokens(211, 400, 3)]
    toks[4] = toks[-1] = toks[-30] = 7
    reqs = {"far": toks}
    want = plain_logits(d, reqs)
    run_trace(d, "P", dtype, reqs, want, trace_whole(reqs), 448, "far key, whole")
    run_trace(d, "P", dtype, reqs, want, trace_tail(reqs, 40), 448, "far key, decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(folders, dtype):
    from iian_b200 import EngineConfig, SchedulerConfig
    from iian_b200.engine.engine import Engine
    name = "Q"
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
               dict(budget=64, kv_cache_tokens=128, cuda_graphs=False, enable_prefix_caching=False)):
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
    reqs, want = requests_and_plain(folders, "R")
    steps = trace_mixed(reqs, 384, seed=4)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["R"], "--dtype", "float32",
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
