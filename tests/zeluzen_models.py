"""Small Zeluzen models for the tests: configurations that differ in every size and option, random
weights made sharp, and the plain implementation's logits for a set of requests."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from plain import plain_zeluzen


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, identity, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}


def _wkv(heads, dim, mlp, rank=None):
    mixer = {"heads": heads, "dim": dim}
    if rank is not None:
        mixer["rank"] = rank
    return {"type": "wkv", "mixer": mixer, "mlp": mlp}


def _attn(heads, kv_heads, dim, vdim, mlp, chunk=None, rot=None, scaling=None, scale=None, base=10000.0, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if chunk is not None:
        mixer["mask"] = {"size": chunk}
    if rot is not None:
        mixer["rot"] = {"base": base, "dims": rot}
        if scaling is not None:
            mixer["rot"]["scaling"] = scaling
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def configs():
    """name -> (config.json as a dict, page size).  Between them: grouped and ungrouped key heads and a single one;
    values longer and shorter than keys; chunks of 1, smaller than, equal to, larger than and no multiple of a
    page, longer than every prompt, and none; rotation of a part of a head, of all of it, and none; frequency
    scaling whose three ranges are all hit, and none; layers that read the cache of the first or of a middle layer,
    with the same chunk and with another one; recurrent heads of 8, 24, 32 and 40 channels whose product is below,
    equal to and above the width, decay ranks given and left to the file; layers without feed-forward, dense
    ones, mixtures with and without input-passing experts, with only such experts, choosing 1, some and all."""
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    a = {"architecture": "Zeluzen", "vocab": 300, "width": 64, "norm": {"eps": 1e-6}, "layers": [
        _attn(4, 2, 16, 24, _dense(96), chunk=16, rot=8, scaling=sc, scale=0.3, base=100.0),
        _wkv(2, 32, _moe(40, 5, 2, 2)),
        _attn(4, 2, 16, 24, _moe(24, 3, 0, 1), chunk=16, rot=8, scaling=sc, scale=0.3, base=100.0, kv_from=0),
        _wkv(3, 24, None, rank=5)]}
    b = {"architecture": "Zeluzen", "vocab": 257, "width": 96, "norm": {"eps": 1e-5}, "layers": [
        _wkv(3, 32, None),
        _attn(6, 1, 8, 8, _moe(32, 4, 1, 5), chunk=7, rot=8),
        _attn(3, 3, 24, 16, _dense(80)),
        _attn(6, 1, 8, 8, _dense(72), chunk=21, rot=8, kv_from=1),
        _wkv(1, 40, _moe(48, 0, 3, 2))]}
    c = {"architecture": "Zeluzen", "vocab": 190, "width": 48, "norm": {"eps": 3e-4}, "layers": [
        _attn(2, 2, 32, 8, _moe(16, 2, 2, 4), chunk=1),
        _wkv(8, 8, _dense(56), rank=3),
        _attn(5, 5, 8, 40, None, chunk=300, rot=4, scaling={"factor": 8.0, "low": 2.0, "high": 3.0, "original": 16}, base=50.0),
        _attn(2, 2, 32, 8, _dense(40), chunk=1, kv_from=0)]}
    d = {"architecture": "Zeluzen", "vocab": 128, "width": 80, "norm": {"eps": 1e-6}, "layers": [
        _wkv(2, 40, _dense(100)),
        _wkv(5, 16, _moe(20, 6, 0, 3))]}
    return {"A": (a, 8), "B": (b, 16), "C": (c, 4), "D": (d, 16)}


def medium_config():
    """A model of a few hundred columns whose prompts are long enough for the kernels of many rows: heads of 64 and
    128 on pages of 16 (the tensor-core attention), values as long as keys and longer, chunks of 128 and 256, experts
    with more than 512 (token, choice) pairs a step, recurrent heads of 32, 64 and 128 channels."""
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 256}
    return {"architecture": "Zeluzen", "vocab": 700, "width": 320, "norm": {"eps": 1e-6}, "layers": [
        _attn(8, 2, 64, 64, _dense(448), chunk=128, rot=32, scaling=sc, scale=0.125, base=20000.0),
        _wkv(5, 64, _moe(96, 8, 2, 3)),
        _wkv(3, 128, _dense(448), rank=24),
        _attn(8, 2, 64, 64, _moe(96, 8, 2, 3), chunk=128, rot=32, scaling=sc, scale=0.125, base=20000.0, kv_from=0),
        _attn(4, 4, 128, 128, None, chunk=256, rot=128, scale=0.09, base=5000.0),
        _attn(6, 3, 32, 48, _dense(384), chunk=64, rot=16, scale=0.2),
        _wkv(10, 32, _moe(64, 5, 0, 2))]}, 16


def write_model(raw, out_dir, seed):
    """Random weights for `raw`, then made sharp: head norms are large so that attention is peaked (the norms in
    front of the scores take any scale of the projections away), the embedding so that tokens differ, norm weights
    are spread, the mixing weights lie between 0 and 1, decays spread from slow to fast, the bonus is not zero, the
    router decides clearly and its selection bias changes choices."""
    from inferflux_b200.config import config_from_dict
    from inferflux_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    cfg = config_from_dict(raw)
    write_random_model(cfg, out_dir, seed=seed, dtype=torch.float32, std=0.08, norm_jitter=0.2)
    path = Path(out_dir) / "model.safetensors"
    with SafetensorsFile(path) as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    g = torch.Generator().manual_seed(seed)
    for n, t in tensors.items():
        if n.endswith(".q.norm") or n.endswith(".k.norm"):
            tensors[n] = 2.2 + 0.5 * torch.randn(t.shape, generator=g)
        elif n == "embed":
            tensors[n] = t * 8.0
        elif ".mix.mu." in n:
            tensors[n] = torch.rand(t.shape, generator=g)
        elif n.endswith(".mix.w0"):
            tensors[n] = -1.5 + 1.5 * torch.randn(t.shape, generator=g)
        elif n.endswith(".mix.u"):
            tensors[n] = 0.5 * torch.randn(t.shape, generator=g)
        elif n.endswith(".mix.w2") or n.endswith(".mix.w1"):
            tensors[n] = t * 6.0
        elif n.endswith(".mlp.router"):
            tensors[n] = t * 10.0
        elif n.endswith(".mlp.correction"):
            tensors[n] = 0.3 * torch.randn(t.shape, generator=g)
        elif ".mlp.e" in n:
            tensors[n] = t * 3.0
    write_safetensors(path, tensors, metadata={"format": "pt"})
    (Path(out_dir) / "config.json").write_text(json.dumps(raw, indent=1))
    return Path(out_dir)


def load(model_dir):
    return plain_zeluzen.load_model_dir(model_dir)


def plain_logits(model_dir, requests, weights_as=None, dtype=torch.float64):
    raw, W = load(model_dir)
    if weights_as is not None:
        W = {k: (v.to(weights_as) if v.is_floating_point() else v) for k, v in W.items()}
    return {rid: plain_zeluzen.forward(raw, W, toks, dtype=dtype).double().numpy() for rid, toks in requests.items()}


def requests_for(raw, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, raw["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lens)}
