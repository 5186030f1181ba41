"""Lekilix without a GPU: the plain implementation's mechanisms on cases worked out by hand, the configuration reader, the
tensor names, and the engine's host side (K/V pages beside state slots, a stretch of layers run several times with caches
of its own per run, windows, page and slot reuse, portions, mixed batches, the scheduler's entry point) with the torch
stand-in for the kernels against the plain implementation."""
import json
import math

import pytest
import torch

import plain_lekilix as plain
from fake_kernels import FakeKernels
from helpers import first_bad, max_error, random_tokens, replay_and_collect, trace_mixed, trace_portions, trace_tail, trace_whole
from iian_b200 import EngineConfig, SchedulerConfig, ops
from iian_b200.config.registry import architecture_of, get_architecture
from iian_b200.engine.engine import Engine
from iian_b200.engine.model import Model, declare_tensors
from iian_b200.engine.replay import TraceReplayer
from iian_b200.models.qwen3 import ConfigError
from iian_b200.parts.base import KVNeed, StateNeed
from lekilix_cases import BLOCK_SIZE, CONFIGS, plain_logits, write_case

F64 = torch.float64


# ---- the plain implementation's mechanisms ------------------------------------------------------------
def test_plain_norm_adds_one_to_the_weight():
    x = torch.tensor([[3.0, -4.0]], dtype=F64)
    got = plain.offset_rms_norm(x, torch.tensor([0.0, 0.5], dtype=F64), 0.0)
    rms = math.sqrt(12.5)
    assert torch.allclose(got, torch.tensor([[3 / rms, -4 / rms * 1.5]], dtype=F64))


def test_plain_rotation_pairs_neighbours_and_passes_the_rest():
    v = torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], dtype=F64).view(1, 1, 6).repeat(2, 1, 1)
    out = plain.rotate_pairs(v, torch.tensor([0, 3]), 4, 100.0)
    assert torch.equal(out[0], v[0])                                                 # position 0: no rotation
    a0, a1 = 3.0, 3.0 * 100.0 ** (-0.5)
    assert out[1, 0, 0].item() == pytest.approx(1 * math.cos(a0) - 2 * math.sin(a0))  # pairs (0, 1) and (2, 3)
    assert out[1, 0, 1].item() == pytest.approx(2 * math.cos(a0) + 1 * math.sin(a0))
    assert out[1, 0, 3].item() == pytest.approx(4 * math.cos(a1) + 3 * math.sin(a1))
    assert out[1, 0, 4:].tolist() == [5.0, 6.0]


def test_plain_window_and_sink():
    vis = plain.window_mask(6, 3)
    assert vis[5].tolist() == [False, False, False, True, True, True]
    p = plain.sink_softmax(torch.zeros(1, 2, 2, dtype=F64), plain.window_mask(2, None), torch.tensor([math.log(2.0)], dtype=F64))
    assert torch.allclose(p[0, 1], torch.tensor([0.25, 0.25], dtype=F64))            # 1 / (1 + 1 + 2)


def _attention_tensors(H, G, d, W, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)
    return {"q": r(H * d, W), "k": r(G * d, W), "g": r(H * d, W), "o": r(W, H * d), "q.norm": r(H * d), "k.norm": r(G * d),
            "sink": r(H)}


def test_plain_attention_values_are_the_unrotated_unnormed_keys():
    """One token: the softmax over its own key and the sink gives p; the output is p * (Wk h) -- not the normalised key."""
    H, G, d, W = 2, 1, 4, 6
    t = _attention_tensors(H, G, d, W)
    mc = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": 0.5, "rot": {"dims": 4, "base": 10.0}}
    h = torch.randn(1, W, generator=torch.Generator().manual_seed(1), dtype=F64)
    got = plain.shared_kv_attention(h, t, "", mc, 1e-5)
    k_raw = h @ t["k"].T
    qn = plain.unit_rms(h @ t["q"].T, 1e-5) * t["q.norm"]
    kn = plain.unit_rms(k_raw, 1e-5) * t["k.norm"]
    heads = []
    for g_ in range(H):
        s = (qn[0, g_ * d:(g_ + 1) * d] * kn[0]).sum() * 0.5                          # position 0: no rotation
        p = torch.exp(s) / (torch.exp(s) + torch.exp(t["sink"][g_]))
        heads.append(p * k_raw[0])
    want = (torch.cat(heads) * torch.sigmoid(h @ t["g"].T)[0]) @ t["o"].T
    assert torch.allclose(got[0], want)


def test_plain_memory_first_steps_by_hand():
    """Two tokens of one head of size 1 x 1: the running maximum starts at zero, so the first step keeps exp(b) of nothing
    and takes exp(a - m1)."""
    t = {"q": torch.tensor([[2.0]], dtype=F64), "k": torch.tensor([[3.0]], dtype=F64), "v": torch.tensor([[5.0]], dtype=F64),
         "g": torch.tensor([[0.0]], dtype=F64), "o": torch.tensor([[1.0]], dtype=F64), "norm": torch.tensor([1.0], dtype=F64),
         "i": torch.tensor([[-1.0]], dtype=F64), "i.b": torch.tensor([0.25], dtype=F64),
         "f": torch.tensor([[0.5]], dtype=F64), "f.b": torch.tensor([-0.5], dtype=F64)}
    mc = {"heads": 1, "dim": 1, "vdim": 1, "gate_cap": 4.0}
    h = torch.tensor([[1.0], [0.5]], dtype=F64)
    y, (C, n, m) = plain.matrix_memory(h, t, "", mc, 0.0, return_state=True)
    a = [4 * math.tanh((-x + 0.25) / 4) for x in (1.0, 0.5)]
    b = [math.log(1 / (1 + math.exp(-4 * math.tanh((0.5 * x - 0.5) / 4)))) for x in (1.0, 0.5)]
    m1 = max(b[0] + 0.0, a[0])
    c1 = math.exp(a[0] - m1) * 3.0 * 5.0
    n1 = math.exp(a[0] - m1) * 3.0
    m2 = max(b[1] + m1, a[1])
    c2 = math.exp(b[1] + m1 - m2) * c1 + math.exp(a[1] - m2) * 1.5 * 2.5
    n2 = math.exp(b[1] + m1 - m2) * n1 + math.exp(a[1] - m2) * 1.5
    assert C.item() == pytest.approx(c2) and n.item() == pytest.approx(n2) and m.item() == pytest.approx(m2)
    o2 = c2 * 1.0 / (max(abs(n2 * 1.0), math.exp(-m2)) + 1e-6)                        # q = 2 * 0.5 / sqrt(1)
    assert y[1].item() == pytest.approx(o2 / abs(o2) * 0.5)                            # unit rms of one number, gate sigmoid(0)
    # a portion continued from a state equals the whole
    y1, st = plain.matrix_memory(h[:1], t, "", mc, 0.0, return_state=True)
    y2 = plain.matrix_memory(h[1:], t, "", mc, 0.0, state=st)
    assert torch.allclose(torch.cat([y1, y2]), y)


def test_plain_experts_come_from_the_table_with_equal_weights_on_the_output():
    g = torch.Generator().manual_seed(3)
    t = {"table": torch.tensor([[1, 0], [2, 1], [0, 2]], dtype=torch.int32)}
    for e in range(3):
        for n, shape in (("gate", (3, 2)), ("up", (3, 2)), ("down", (2, 3))):
            t[f"e{e}.{n}"] = torch.randn(shape, generator=g, dtype=F64) * 3
    fc = {"expert": {"ff": 3, "limit": 1.0}, "router": {"experts": 3, "top": 2}}
    h = torch.randn(2, 2, generator=g, dtype=F64)
    got = plain.table_routed_ff(h, torch.tensor([1, 2]), t, "", fc)
    want0 = 0.5 * (plain.clamped_expert(h[:1], t, "e2.", 1.0) + plain.clamped_expert(h[:1], t, "e1.", 1.0))
    assert torch.allclose(got[:1], want0)
    # the clamps: the gate only from above, the other branch on both sides, and one is added to it
    z = torch.tensor([[-5.0, 0.3, 5.0]], dtype=F64)
    eye = {"gate": torch.eye(3, dtype=F64), "up": torch.eye(3, dtype=F64), "down": torch.eye(3, dtype=F64)}
    y = plain.clamped_expert(z, eye, "", 2.0)[0]
    assert y[0].item() == pytest.approx(-5.0 / (1 + math.exp(1.702 * 5.0)) * (-2.0 + 1))
    assert y[2].item() == pytest.approx(2.0 / (1 + math.exp(-1.702 * 2.0)) * (2.0 + 1))


def test_plain_run_order_repeats_the_stretch():
    assert plain.run_order(CONFIGS["U"]) == [(0, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert plain.run_order(CONFIGS["W"]) == [(i, False) for i in range(4)]


# ---- configuration and names --------------------------------------------------------------------------
def test_config_is_read_layer_by_layer():
    arch = architecture_of(CONFIGS["U"])
    assert arch.name == "Lekilix"
    c = arch.load_config(CONFIGS["U"])
    assert [l.type for l in c.layers] == ["attention", "mlstm", "attention", "mlstm"]
    assert c.layers[0].mixer.window == 24 and c.layers[2].mixer.rot_dims == 24 and c.layers[1].mlp.limit == 1.5
    assert c.layers[2].mlp is None and c.embedding_scale == 3.7 and c.loop.times == 2
    assert arch.load_config(arch.config_to_dict(c)) == c
    spec = arch.build_spec(c)
    assert [(o.layer, o.cache, o.before) for o in spec.order] == [(0, 0, None), (1, 1, 0), (2, 2, None), (1, 3, 0), (2, 4, None),
                                                                   (3, 5, None)]
    assert spec.layers[1].feed_forward["score"] == "table" and spec.layers[0].mixer["position"]["style"] == "interleaved"
    w = arch.build_spec(arch.load_config(CONFIGS["W"]))
    assert w.stream_parts == () and all(o.before is None for o in w.order) and w.layers[2].mixer["position"].kind == "none"


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="other"), "unknown type"),
    (lambda c: c["layers"][1]["mlp"].update(kind="other"), "unknown kind"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_heads"), "lacks 'kv_heads'"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=20), "the values are the keys"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "6 heads for 4"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "takes 9 of 5"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "lacks 'limit'"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].update(gate_cap=0), "gate_cap"),
    (lambda c: c["loop"].update(stop=7), "loop runs layers"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_errors_name_the_place(edit, text):
    raw = json.loads(json.dumps(CONFIGS["U"]))
    edit(raw)
    with pytest.raises(ConfigError, match=text):
        get_architecture("Lekilix").load_config(raw)


def test_tensor_names_and_cache_needs(tmp_path):
    arch = get_architecture("Lekilix")
    names = declare_tensors(arch, arch.build_spec(arch.load_config(CONFIGS["U"])))
    for n in ("embed", "head", "final.norm", "loop.in", "l0.norm1", "l0.mix.q", "l0.mix.k", "l0.mix.q.norm", "l0.mix.k.norm",
              "l0.mix.sink", "l0.mix.g", "l0.mix.o", "l0.mlp.gate", "l0.mlp.down", "l1.mix.v", "l1.mix.norm", "l1.mix.i",
              "l1.mix.i.b", "l1.mix.f.b", "l1.mlp.table", "l1.mlp.e4.up", "l3.mlp.up"):
        assert n in names, n
    assert "l0.mix.v" not in names and "l2.mlp.gate" not in names and "l1.mlp.router" not in names and "l1.mlp.e5.up" not in names
    assert names["loop.in"].shape == (96, 192) and names["l1.mlp.table"].shape == (211, 2) and names["l1.mlp.table"].kind == "int"
    assert names["l0.mix.k.norm"].shape == (32,) and names["l1.mix.f"].shape == (3, 96) and names["l1.mix.g"].shape == (120, 96)
    assert "loop.in" not in declare_tensors(arch, arch.build_spec(arch.load_config(CONFIGS["W"])))
    d = write_case(tmp_path, "U", store_dtype=torch.float32)
    with ops.use_kernels(FakeKernels()):
        needs = Model.from_folder(d, "float32", "cpu").cache_needs()
    assert sorted(needs) == [0, 1, 2, 3, 4, 5]                                         # every run of a layer has its own
    assert needs[0] == KVNeed(2, 16, 24) and needs[2] == needs[4] == KVNeed(4, 24, 17)
    assert isinstance(needs[1], StateNeed) and needs[1] == needs[3] and needs[1].dtype == torch.float32
    table = plain.load_folder(d)[1]["l1.mlp.table"]
    assert all(len(set(r)) == 2 and 0 <= min(r) and max(r) < 5 for r in table.tolist())   # the entries of a row differ


# ---- the host side under every way of cutting the work -------------------------------------------------
@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    root = tmp_path_factory.mktemp("lekilix")
    out = {}
    for name in CONFIGS:
        d = write_case(root, name, store_dtype=torch.float32)
        with ops.use_kernels(FakeKernels()):
            out[name] = (d, Model.from_folder(d, "float32", "cpu"))
    return out


LENGTHS = {"U": [1, 9, 40, 75], "V": [3, 35, 70, 20, 2], "W": [2, 90, 33], "X": [45, 5, 20], "Y": [41, 3, 30]}


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


def test_a_slot_that_is_used_again_starts_from_zero(cases):
    """Two state slots, five requests one after another and side by side: a request that inherits a slot must not see what
    the one before left in it."""
    d, model = cases["U"]
    reqs = {f"r{i}": random_tokens(211, n, 90 + i) for i, n in enumerate([30, 12, 25, 7, 18])}
    want = plain_logits(d, reqs)
    steps = trace_mixed(reqs, 128, seed=1, max_live=2)
    with ops.use_kernels(FakeKernels()):
        rp = TraceReplayer(model, 128, 16, 2, native=False)
        got = replay_and_collect(rp, steps)
    bad = first_bad(got, want, 2e-4)
    assert bad is None, f"first wrong logits at {bad}"


def test_windowed_layers_give_pages_back_while_running(cases):
    d, model = cases["U"]
    with ops.use_kernels(FakeKernels()):
        rp = TraceReplayer(model, 128, 16, 4, native=False)
        toks = random_tokens(211, 120, 5)
        for p in range(0, 120, 8):
            rp.run_step({"step": p, "entries": [{"id": "a", "tokens": toks[p:p + 8], "want": []}], "end": []})
    mgr = rp.runner.manager
    by_window = {g.window: mgr.pools[i] for i, g in enumerate(mgr.groups)}
    assert set(by_window) == {24, 17}
    assert all(p.num_blocks - p.num_free <= 3 for p in by_window.values())              # the window's pages only


def test_greedy_generation_through_the_scheduler(cases):
    d, model = cases["V"]
    cfg, w = plain.load_folder(d)
    prompts = [random_tokens(300, n, 70 + i) for i, n in enumerate([1, 6, 30, 50])]

    def greedy(prompt, n):
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(torch.argmax(plain.forward(cfg, w, toks)[-1])))
        return toks[len(prompt):]
    want = [greedy(p, 5) for p in prompts]
    for kw in (dict(budget=64, kv_cache_tokens=512), dict(budget=11, kv_cache_tokens=512),        # whole prompts; portions
               dict(budget=16, kv_cache_tokens=96, enable_prefix_caching=True)):                   # few pages: preemption
        sched = SchedulerConfig(max_num_batched_tokens=kw.pop("budget"), max_num_seqs=4)
        with ops.use_kernels(FakeKernels()):
            eng = Engine(model, EngineConfig(dtype="float32", block_size=8, warmup=False, sched=sched, max_model_len=96, **kw))
            assert not eng.runner.prefix_caching                   # a model with state cannot start behind a shared prefix
            assert eng.generate(prompts, max_tokens=5, temperature=0.0) == want
        eng.cache.check_invariants()
        assert all(p.num_free == p.num_blocks for p in eng.cache.pools)


def test_command_line_writes_and_loads_a_folder(tmp_path):
    """``iian random-weights`` from a Lekilix config.json, then the folder through the loader (names, shapes, the plug-in)."""
    from iian_b200.cli.main import main as cli_main
    from iian_b200.config.registry import load_model_config
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CONFIGS["W"]))
    out = tmp_path / "model"
    assert cli_main(["random-weights", str(cfg_path), str(out), "--seed", "3"]) == 0
    arch, cfg = load_model_config(str(out))
    assert arch.name == "Lekilix" and cfg == arch.load_config(CONFIGS["W"])
    with ops.use_kernels(FakeKernels()):
        model = Model.from_folder(str(out), "float32", "cpu")
        rp = TraceReplayer(model, 64, 16, 2, native=False)
        logits = rp.run_step({"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}], "end": ["a"]})
    want = plain.forward(*plain.load_folder(str(out)), [1, 2, 3])[-1]
    assert (logits[0].double() - want).abs().max() < 2e-4
