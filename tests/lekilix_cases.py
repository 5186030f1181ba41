"""Shared by the Lekilix tests: small configurations that differ in every size and option, model folders with random
weights in temporary places, and the comparison of replayed logits with the plain implementation
(tests/plain_lekilix.py)."""
from __future__ import annotations

import os
from typing import Dict, List

import torch

import plain_lekilix as plain


def attention(heads, kv_heads, dim, window, rot_dims, scale, base=10000.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    if window:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m}


def memory(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


# U: odd sizes everywhere; the looped stretch starts behind the first layer and is followed by another; windows that are no
#    multiple of the page, full and partial rotation, three query heads on one key/value head and one on one, a layer without
#    feed-forward, memories whose sizes are no power of two.
# V: sizes the bfloat16 fast products take (multiples of 32); the first layer alone runs three times; one expert per token
#    and three; a window of 33; a memory wider than it is deep.
# W: no loop at all; one head, one expert of one; no rotation in one layer; a window shorter than a page and one longer than
#    any request; a memory deep enough for the 16-lane form of the scan.
# X: heads of 128 (the tensor-core attention kernels of the large shapes, tcgen05 for portions), a memory 128 deep, the
#    first two layers run twice.   Y: a width and sizes that are multiples of 4 only (no 16-byte rows for the fast products).
CONFIGS = {
    "U": {"architecture": "Lekilix", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.7},
          "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
        layer(attention(6, 2, 16, 24, 8, 0.3, 30000.0), dense(160)),
        layer(memory(3, 24, 40, 8.0), moe(5, 2, 48, 1.5)),
        layer(attention(4, 4, 24, 17, 24, 0.2), None),
        layer(memory(2, 16, 24, 15.0), dense(64))]},
    "V": {"architecture": "Lekilix", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 11.0},
          "loop": {"start": 0, "stop": 1, "times": 3}, "layers": [
        layer(memory(4, 32, 32, 10.0), moe(8, 1, 64, 7.0)),
        layer(attention(8, 2, 64, 33, 16, 0.11), dense(256)),
        layer(memory(2, 64, 128, 12.0), moe(8, 3, 64, 1.0))]},
    "W": {"architecture": "Lekilix", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "layers": [
        layer(attention(1, 1, 8, 5, 8, 0.4), moe(1, 1, 32, 2.5)),
        layer(memory(1, 160, 16, 6.0), dense(64)),
        layer(attention(2, 1, 32, 70, 0, 0.2), None),
        layer(memory(1, 8, 8, 20.0), None)]},
}
CONFIGS["X"] = {"architecture": "Lekilix", "vocab": 331, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 16.0},
                "loop": {"start": 0, "stop": 2, "times": 2}, "layers": [
    layer(attention(4, 2, 128, 40, 64, 0.09, 500000.0), dense(384)),
    layer(memory(2, 128, 64, 9.0), moe(4, 2, 64, 3.0)),
    layer(attention(2, 2, 128, 90, 128, 0.07), moe(6, 1, 128, 1.2))]}
CONFIGS["Y"] = {"architecture": "Lekilix", "vocab": 150, "width": 100, "norm": {"eps": 1e-5}, "embedding": {"scale": 10.0},
                "loop": {"start": 1, "stop": 2, "times": 3}, "layers": [
    layer(memory(5, 20, 12, 11.0), dense(52)),
    layer(attention(5, 1, 20, 9, 10, 0.25), moe(3, 2, 36, 2.0)),
    layer(memory(3, 12, 20, 7.0), None)]}
BLOCK_SIZE = {"U": 16, "V": 8, "W": 32, "X": 16, "Y": 16}
SEED = {"U": 21, "V": 22, "W": 23, "X": 24, "Y": 25}


def write_case(tmp_path, name: str, store_dtype=torch.bfloat16, std: float = 0.08) -> str:
    """A model folder of configuration ``name`` with random weights.  ``std`` is large enough that attention weights and
    gates are far from uniform."""
    from iian_b200.config.registry import get_architecture
    from iian_b200.weights.random_init import write_model_folder
    arch = get_architecture("Lekilix")
    d = os.path.join(str(tmp_path), f"lekilix{name}_{str(store_dtype).split('.')[-1]}")
    if not os.path.isdir(d):
        write_model_folder(d, arch, arch.load_config(CONFIGS[name]), seed=SEED[name], store_dtype=store_dtype, std=std,
                           norm_jitter=0.3)
    return d


def plain_logits(model_dir: str, requests: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    cfg, w = plain.load_folder(model_dir)
    return {rid: plain.forward(cfg, w, toks) for rid, toks in requests.items()}
