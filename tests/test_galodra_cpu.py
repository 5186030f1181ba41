"""Galodra without a GPU: the plain implementation's mechanisms on cases worked out by hand, the configuration reader,
the tensor names, and the engine's host side (cache of one row per token, windows, page reuse, portions, mixed batches,
the scheduler's entry point) with the torch stand-in for the kernels against the plain implementation."""
import json
import math
import os

import pytest
import torch

import plain_galodra as plain
from fake_kernels import FakeKernels
from galodra_cases import BLOCK_SIZE, CONFIGS, plain_logits, write_case
from helpers import first_bad, max_error, random_tokens, replay_and_collect, trace_mixed, trace_portions, trace_tail, trace_whole
from iian_b200 import EngineConfig, SchedulerConfig, ops
from iian_b200.config.registry import architecture_of, get_architecture
from iian_b200.engine.engine import Engine
from iian_b200.engine.model import Model, declare_tensors
from iian_b200.engine.replay import TraceReplayer
from iian_b200.models.qwen3 import ConfigError


# ---- the plain implementation's mechanisms ------------------------------------------------------------
def test_plain_window_mask_edges():
    vis = plain.window_mask(6, 3)
    assert vis[5].tolist() == [False, False, False, True, True, True]       # itself and the two before it
    assert vis[1].tolist() == [True, True, False, False, False, False]
    assert plain.window_mask(4, None)[3].tolist() == [True] * 4


def test_plain_sink_joins_the_denominator_only():
    scores = torch.zeros(1, 2, 2, dtype=torch.float64)
    p = plain.sink_softmax(scores, plain.window_mask(2, None), torch.tensor([math.log(2.0)], dtype=torch.float64))
    assert torch.allclose(p[0, 0], torch.tensor([1 / 3, 0.0], dtype=torch.float64))          # e^0 / (e^0 + 2)
    assert torch.allclose(p[0, 1], torch.tensor([0.25, 0.25], dtype=torch.float64))         # 1 / (1 + 1 + 2)


def test_plain_rotation_pairs_and_passes_the_rest():
    v = torch.tensor([[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]], dtype=torch.float64).repeat(2, 1)
    out = plain.rotate_half(v, torch.tensor([0, 1]), 4, 100.0)
    assert torch.equal(out[0], v[0])                                               # position 0: no rotation
    a0, a1 = 1.0, 100.0 ** (-0.5)
    assert out[1, 0].item() == pytest.approx(1 * math.cos(a0) - 3 * math.sin(a0))   # pairs (0, 2) and (1, 3)
    assert out[1, 3].item() == pytest.approx(4 * math.cos(a1) + 2 * math.sin(a1))
    assert out[1, 4:].tolist() == [5.0, 6.0]


def test_plain_router_weight_scales_the_input():
    torch.manual_seed(0)
    w = {"r": torch.tensor([[10.0, 0.0], [0.0, 10.0]], dtype=torch.float64)}
    for e in range(2):
        for n, shape in (("gate", (3, 2)), ("up", (3, 2)), ("down", (2, 3))):
            w[f"e{e}.{n}"] = torch.randn(shape, dtype=torch.float64)
    w["router"] = w.pop("r")
    h = torch.tensor([[0.3, -1.0]], dtype=torch.float64)             # expert 0 wins with score sigmoid(3)
    got = plain.routed_ff(h, w, "", 2, 1)
    s = torch.sigmoid(torch.tensor(3.0, dtype=torch.float64))
    assert torch.allclose(got, plain.dense_ff(s * h, w, "e0.", plain.silu))
    assert not torch.allclose(got, s * plain.dense_ff(h, w, "e0.", plain.silu))


# ---- configuration and names --------------------------------------------------------------------------
def test_config_is_read_layer_by_layer():
    arch = architecture_of(CONFIGS["P"])
    assert arch.name == "Galodra"
    c = arch.load_config(CONFIGS["P"])
    assert [l.mixer.window for l in c.layers] == [24, None, 17, 24]
    assert c.layers[2].mlp is None and c.layers[1].mlp.top == 2 and c.layers[0].mixer.rot_dims == 8
    assert arch.load_config(arch.config_to_dict(c)) == c
    spec = arch.build_spec(c)
    assert [l.slot("depth_mix")["terms"] for l in spec.layers] == [2, 3, 4, 5]
    assert spec.layers[2].feed_forward is None and spec.layers[2].slot("feed_forward_gate") is None


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="other"), "unknown type"),
    (lambda c: c["layers"][1]["mlp"].update(kind="other"), "unknown kind"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "lacks 'kv_rank'"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "takes 9 of 5"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda c: c.pop("postln_alpha"), "postln_alpha"),
])
def test_config_errors_name_the_place(edit, text):
    raw = json.loads(json.dumps(CONFIGS["P"]))
    edit(raw)
    with pytest.raises(ConfigError, match=text):
        get_architecture("Galodra").load_config(raw)


def test_tensor_names():
    arch = get_architecture("Galodra")
    names = declare_tensors(arch, arch.build_spec(arch.load_config(CONFIGS["P"])))
    for n in ("embed", "final.norm", "final.norm.b", "l0.norm1", "l0.norm2.b", "l0.mix.q", "l0.mix.dkv", "l0.mix.dkv.norm",
              "l0.mix.uk", "l0.mix.uv", "l0.mix.sink", "l0.mix.o", "l0.mlp.gate", "l0.mlp.down", "l0.rg1", "l0.rg2.b", "l0.dwa",
              "l1.mlp.router", "l1.mlp.e4.up", "l3.dwa"):
        assert n in names, n
    assert "l2.norm2" not in names and "l2.rg2" not in names and "l1.mlp.e5.up" not in names
    assert names["l3.dwa"].shape == (5,) and names["l0.mix.dkv"].shape == (52, 96) and names["l0.mix.uv"].shape == (72, 40)


# ---- the host side under every way of cutting the work -------------------------------------------------
@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    root = tmp_path_factory.mktemp("galodra")
    out = {}
    for name in CONFIGS:
        d = write_case(root, name, store_dtype=torch.float32)
        with ops.use_kernels(FakeKernels()):
            out[name] = (d, Model.from_folder(d, "float32", "cpu"))
    return out


LENGTHS = {"P": [1, 9, 40, 75], "Q": [3, 35, 70, 20], "R": [2, 90, 33]}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_replay_matches_plain_under_every_cut(cases, name):
    d, model = cases[name]
    reqs = {f"r{i}": random_tokens(CONFIGS[name]["vocab"], n, 40 + i) for i, n in enumerate(LENGTHS[name])}
    want = plain_logits(d, reqs)
    rounded = max(-(-len(t) // 64) * 64 for t in reqs.values())
    for what, steps, cap in (("whole", trace_whole(reqs), rounded), ("tail", trace_tail(reqs, 20), rounded),
                             ("portions", trace_portions(reqs), rounded), ("mixed", trace_mixed(reqs, 2 * rounded, seed=3), 2 * rounded)):
        with ops.use_kernels(FakeKernels()):
            rp = TraceReplayer(model, cap, BLOCK_SIZE[name], 4, native=False)
            got = replay_and_collect(rp, steps)
        rp.runner.manager.check_invariants()
        assert all(p.num_free == p.num_blocks for p in rp.runner.manager.pools), "pages were lost"
        assert len(got) == sum(len(t) for t in reqs.values())
        bad = first_bad(got, want, 2e-4)
        assert bad is None, f"{name} {what}: first wrong logits at {bad}; worst {max_error(got, want)}"


def test_windowed_layers_give_pages_back_while_running(cases):
    d, model = cases["P"]
    with ops.use_kernels(FakeKernels()):
        rp = TraceReplayer(model, 128, 16, 4, native=False)
        toks = random_tokens(211, 120, 5)
        for p in range(0, 120, 8):
            rp.run_step({"step": p, "entries": [{"id": "a", "tokens": toks[p:p + 8], "want": []}], "end": []})
    mgr = rp.runner.manager
    by_window = {g.window: mgr.pools[i] for i, g in enumerate(mgr.groups)}
    assert set(by_window) == {24, None, 17}
    assert by_window[None].num_blocks - by_window[None].num_free == 8          # every page of 120 tokens
    assert by_window[24].num_blocks - by_window[24].num_free <= 3               # the window's pages only
    assert by_window[17].num_blocks - by_window[17].num_free <= 3


def test_greedy_generation_through_the_scheduler(cases):
    d, model = cases["Q"]
    cfg, w = plain.load_folder(d)
    prompts = [random_tokens(300, n, 70 + i) for i, n in enumerate([1, 6, 30, 50])]

    def greedy(prompt, n):
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(torch.argmax(plain.forward(cfg, w, toks)[-1])))
        return toks[len(prompt):]
    want = [greedy(p, 5) for p in prompts]
    for kw in (dict(budget=64, kv_cache_tokens=512), dict(budget=11, kv_cache_tokens=512),        # whole prompts; portions
               dict(budget=16, kv_cache_tokens=96, enable_prefix_caching=False)):                  # few pages: preemption
        sched = SchedulerConfig(max_num_batched_tokens=kw.pop("budget"), max_num_seqs=4)
        with ops.use_kernels(FakeKernels()):
            eng = Engine(model, EngineConfig(dtype="float32", block_size=8, warmup=False, sched=sched, max_model_len=96, **kw))
            assert eng.generate(prompts, max_tokens=5, temperature=0.0) == want
        eng.cache.check_invariants()
        assert all(p.num_free == p.num_blocks for p in eng.cache.pools)


def test_command_line_writes_and_loads_a_folder(tmp_path):
    """``iian random-weights`` from a Galodra config.json, then the folder through the loader (names, shapes, the plug-in)."""
    from iian_b200.cli.main import main as cli_main
    from iian_b200.config.registry import load_model_config
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CONFIGS["R"]))
    out = tmp_path / "model"
    assert cli_main(["random-weights", str(cfg_path), str(out), "--seed", "3"]) == 0
    arch, cfg = load_model_config(str(out))
    assert arch.name == "Galodra" and cfg == arch.load_config(CONFIGS["R"])
    with ops.use_kernels(FakeKernels()):
        model = Model.from_folder(str(out), "float32", "cpu")
        rp = TraceReplayer(model, 64, 16, 2, native=False)
        logits = rp.run_step({"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}], "end": ["a"]})
    want = plain.forward(*plain.load_folder(str(out)), [1, 2, 3])[-1]
    assert (logits[0].double() - want).abs().max() < 2e-4
