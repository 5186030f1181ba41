"""Shared by the Galodra tests: small configurations that differ in every size and option, model folders with random
weights in temporary places, and the comparison of replayed logits with the plain implementation
(tests/plain_galodra.py)."""
from __future__ import annotations

import os
from typing import Dict, List

import torch

import plain_galodra as plain


def mixer(heads, dim, rot_dim, vdim, rank, window, rot_dims, base=10000.0):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
         "scale": 1.0 / (dim + rot_dim) ** 0.5}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    if window:
        m["mask"] = {"size": window}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(mix, mlp):
    return {"type": "latent_attention", "mixer": mix, "mlp": mlp}


# P: odd sizes everywhere; every layer with a window of its own (one without), partial rotation, two experts per token, a
#    layer without feed-forward.   Q: sizes the bfloat16 fast products take (multiples of 32), one expert per token and
#    three, a window that is no multiple of the page size.   R: one head, one expert of one, no rotation in one layer.
CONFIGS = {
    "P": {"architecture": "Galodra", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "postln_alpha": 1.7, "layers": [
        layer(mixer(3, 16, 12, 24, 40, 24, 8, 30000.0), dense(160)),
        layer(mixer(3, 16, 12, 24, 40, None, 12), moe(5, 2, 48)),
        layer(mixer(2, 24, 8, 16, 24, 17, 8), None),
        layer(mixer(3, 16, 12, 24, 40, 24, 8, 30000.0), moe(5, 2, 48))]},
    "Q": {"architecture": "Galodra", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "postln_alpha": 3.0, "layers": [
        layer(mixer(4, 32, 32, 32, 64, 33, 32), moe(8, 1, 64)),
        layer(mixer(4, 32, 32, 32, 64, 33, 32), dense(256)),
        layer(mixer(4, 32, 32, 32, 64, 33, 32), moe(8, 3, 64))]},
    "R": {"architecture": "Galodra", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "postln_alpha": 1.0, "layers": [
        layer(mixer(1, 8, 8, 8, 16, 5, 8), moe(1, 1, 32)),
        layer(mixer(1, 8, 8, 8, 16, 70, 0), dense(64))]},
}
BLOCK_SIZE = {"P": 16, "Q": 8, "R": 32}
SEED = {"P": 11, "Q": 12, "R": 13}


def write_case(tmp_path, name: str, store_dtype=torch.bfloat16, std: float = 0.08) -> str:
    """A model folder of configuration ``name`` with random weights.  ``std`` is large enough that attention weights,
    gates and router scores are far from uniform."""
    from iian_b200.config.registry import get_architecture
    from iian_b200.weights.random_init import write_model_folder
    arch = get_architecture("Galodra")
    d = os.path.join(str(tmp_path), f"galodra{name}_{str(store_dtype).split('.')[-1]}")
    if not os.path.isdir(d):
        write_model_folder(d, arch, arch.load_config(CONFIGS[name]), seed=SEED[name], store_dtype=store_dtype, std=std,
                           norm_jitter=0.3)
    return d


def plain_logits(model_dir: str, requests: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    cfg, w = plain.load_folder(model_dir)
    return {rid: plain.forward(cfg, w, toks) for rid, toks in requests.items()}
