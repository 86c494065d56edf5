"""Small Dafolorn models for the tests: configurations that differ in every size and option,
random weights made sharp, and the plain implementation's logits for a set of requests."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

from plain import plain_dafolorn


def _layer(heads, dim, vdim, rank, window, ff, scale=None):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": dim ** -0.5 if scale is None else scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def configs():
    """name -> (config.json as a dict, page size).  Between them: one head and several; key size above,
    below and equal to the value size; latents that are no multiple of 32; windows of 1, below a page,
    exactly a page, a page + 1, above the prompt lengths, and none; a layer without feed-forward; 1 to 6
    taps and no convolution at all; a loop at the start, in the middle, over everything, run once, and
    none; with and without a cap on the logits."""
    p = {"architecture": "Dafolorn", "vocab": 300, "width": 64, "norm": {"eps": 1e-6}, "canon": {"taps": 3},
         "logit_softcap": 20.0, "loop": {"start": 0, "stop": 2, "times": 3},
         "layers": [_layer(2, 16, 24, 40, 21, 96, 0.25), _layer(3, 8, 8, 24, 7, None), _layer(1, 32, 16, 32, None, 80)]}
    q = {"architecture": "Dafolorn", "vocab": 257, "width": 96, "norm": {"eps": 1e-5}, "canon": {"taps": 1},
         "layers": [_layer(4, 12, 20, 36, 1, 112), _layer(4, 12, 20, 36, 33, 112)]}
    r = {"architecture": "Dafolorn", "vocab": 190, "width": 48, "norm": {"eps": 3e-4}, "canon": {"taps": 2},
         "logit_softcap": 8.0, "loop": {"start": 1, "stop": 3, "times": 1},
         "layers": [_layer(2, 24, 8, 64, 16, 64), _layer(2, 8, 24, 64, 17, 72), _layer(6, 8, 8, 16, 5, 56)]}
    s = {"architecture": "Dafolorn", "vocab": 128, "width": 80, "norm": {"eps": 1e-6},
         "loop": {"start": 0, "stop": 2, "times": 2},
         "layers": [_layer(5, 16, 16, 48, 300, 100), _layer(2, 40, 24, 72, 40, 60)]}
    u = {"architecture": "Dafolorn", "vocab": 211, "width": 72, "norm": {"eps": 1e-6}, "canon": {"taps": 4},
         "logit_softcap": 50.0, "loop": {"start": 1, "stop": 2, "times": 4},
         "layers": [_layer(3, 16, 8, 56, 9, 88), _layer(2, 16, 32, 24, 30, 104)]}
    v = {"architecture": "Dafolorn", "vocab": 150, "width": 40, "norm": {"eps": 1e-6}, "canon": {"taps": 6},
         "logit_softcap": 15.0, "loop": {"start": 0, "stop": 1, "times": 2},
         "layers": [_layer(2, 16, 16, 32, 12, 48), _layer(1, 8, 24, 16, None, None)]}
    return {"P": (p, 8), "Q": (q, 16), "R": (r, 16), "S": (s, 4), "U": (u, 16), "V": (v, 16)}


def write_model(raw, out_dir, seed, sharpen=10.0):
    """Random weights for `raw`, then made sharp: queries and key up-projections are scaled so that
    attention is peaked, the embedding so that tokens differ, norm weights (stored around zero) and sinks
    are spread, the activation's two numbers are not zero, convolution taps are large."""
    from inferflux_b200.config import config_from_dict
    from inferflux_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    cfg = config_from_dict(raw)
    write_random_model(cfg, out_dir, seed=seed, dtype=torch.float32, std=0.05, norm_jitter=0.2)
    path = Path(out_dir) / "model.safetensors"
    with SafetensorsFile(path) as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    g = torch.Generator().manual_seed(seed)
    for n, t in tensors.items():
        if n.endswith(".mix.q") or n.endswith(".mix.uk"):
            tensors[n] = t * sharpen
        elif n == "embed":
            tensors[n] = t * 8.0
        elif n.endswith(".mix.sink"):
            tensors[n] = torch.randn(t.shape, generator=g) * 1.5
        elif n.endswith(".mlp.act"):
            tensors[n] = torch.tensor([0.4, -0.7]) + 0.3 * torch.randn(2, generator=g)
        elif ".canon" in n:
            tensors[n] = torch.randn(t.shape, generator=g) * 0.4
        elif n == "loop.step":
            tensors[n] = torch.randn(t.shape, generator=g) * 0.5
        elif n == "loop.in":
            tensors[n] = t * 4.0
    write_safetensors(path, tensors, metadata={"format": "pt"})
    (Path(out_dir) / "config.json").write_text(json.dumps(raw, indent=1))
    return Path(out_dir)


def load(model_dir):
    from inferflux_b200.weights import SafetensorsFile
    raw = json.loads((Path(model_dir) / "config.json").read_text())
    with SafetensorsFile(Path(model_dir) / "model.safetensors") as f:
        return raw, {n: f.tensor(n).clone() for n in f.names()}


def plain_logits(model_dir, requests, weights_as=None, dtype=torch.float64):
    raw, W = load(model_dir)
    if weights_as is not None:
        W = {k: v.to(weights_as) for k, v in W.items()}
    return {rid: plain_dafolorn.forward(raw, W, toks, dtype=dtype).double().numpy() for rid, toks in requests.items()}


def requests_for(raw, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, raw["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lens)}
