"""The Zeluzen decoder stated plainly: one function per mechanism, whole sequences at once, no cache,
no batching, nothing shared with the package.  Slow on purpose; the tests hold the engine to it.

A model is (raw, W): config.json as a dict and name -> tensor.  Every function computes in the dtype of
its inputs (the tests use float64).

    x = rmsnorm(embed[tokens], embed.norm)
    per layer:  x = x + rmsnorm(mixer(x), norm1);   x = x + rmsnorm(ff(x), norm2)      (ff may be absent)
    logits = head . rmsnorm(x, final.norm)

Mixers: `wkv` (a matrix-valued recurrence per head with a decay made from the input) and `attention`
(grouped queries, normed and partly rotated queries and keys, chunks instead of a causal triangle, one
extra unit in the softmax's denominator, optionally the keys and values of an earlier layer).
Feed-forwards: `dense` (gated, SiLU) and `moe` (a softmax router with a selection bias, squared-ReLU
experts, and experts that hand their input on unchanged).
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# ------------------------------------------------------------------------------ norms

def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rmsnorm(x, w, eps):
    return unit_rms(x, eps) * w


# ------------------------------------------------------------------------------ the recurrence

def shifted(h):
    """Row t holds h[t - 1]; the first row is zeros."""
    return torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)


def decay(raw):
    """exp(-exp(raw)): a number in (0, 1) for every head and key channel."""
    return torch.exp(-torch.exp(raw))


def wkv_scan(r, k, v, w, u, state=None):
    """r, k, w: [n, H, D]; v: [n, H, D]; u: [H, D].  For every head a matrix S [key channel, value channel]:
    out_t = (S + u k_t v_t^T)^T r_t, then S <- w_t S + k_t v_t^T (w_t scales S's rows)."""
    n, H, D = r.shape
    S = torch.zeros(H, D, v.shape[-1], dtype=r.dtype) if state is None else state.clone()
    out = []
    for t in range(n):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hij,hi->hj", S + u[:, :, None] * kv, r[t]))
        S = w[t][:, :, None] * S + kv
    return torch.stack(out), S


def wkv_mixer(h, W, p, mixer, eps):
    H, D = mixer["heads"], mixer["dim"]
    n = h.shape[0]
    before = shifted(h)
    mix = {s: h + (before - h) * W[p + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ W[p + "r"].T).view(n, H, D)
    k = (mix["k"] @ W[p + "k"].T).view(n, H, D)
    v = (mix["v"] @ W[p + "v"].T).view(n, H, D)
    gate = torch.nn.functional.silu(mix["g"] @ W[p + "g"].T)
    raw = torch.tanh(mix["w"] @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"]
    o, _S = wkv_scan(r, k, v, decay(raw).view(n, H, D), W[p + "u"])
    o = unit_rms(o, eps).reshape(n, H * D)
    return (o * W[p + "norm"] * gate) @ W[p + "o"].T


# ------------------------------------------------------------------------------ attention

def scaled_frequencies(base, dims, scaling):
    """f_i = base^(-2i/dims); long wavelengths are slowed by `factor`, short ones kept, a ramp between."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f
    factor, low, high, orig = scaling["factor"], scaling["low"], scaling["high"], scaling["original"]
    out = []
    for fi in f:
        wavelength = 2.0 * math.pi / fi
        if wavelength < orig / high:
            out.append(fi)
        elif wavelength > orig / low:
            out.append(fi / factor)
        else:
            s = (orig / wavelength - low) / (high - low)
            out.append((1.0 - s) * fi / factor + s * fi)
    return out


def rotate_pairs(x, positions, freqs):
    """x: [n, heads, dim]; elements (2i, 2i + 1), i < len(freqs), turn by position * freqs[i]; the rest stay."""
    out = x.clone()
    pos = torch.as_tensor(positions, dtype=x.dtype)
    for i, f in enumerate(freqs):
        a = pos * f
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def visible(i, j, chunk):
    """Whether the query at position i sees the key at position j."""
    return j <= i and (chunk is None or i // chunk == j // chunk)


def sink_softmax(s):
    """exp(s_j) / (1 + sum exp(s)): a unit that has score zero and no value takes part."""
    m = torch.clamp(s.max(), min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum())


def attention_keys_values(h, W, p, mixer, eps, positions):
    G, D, Dv = mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    n = h.shape[0]
    k = rmsnorm((h @ W[p + "k"].T).view(n, G, D), W[p + "k.norm"], eps)
    rot = mixer.get("rot")
    if rot:
        k = rotate_pairs(k, positions, scaled_frequencies(rot["base"], rot["dims"], rot.get("scaling")))
    return k, (h @ W[p + "v"].T).view(n, G, Dv)


def attention_mixer(h, W, p, mixer, eps, positions, keys, values):
    H, G, D, Dv = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    n = h.shape[0]
    q = rmsnorm((h @ W[p + "q"].T).view(n, H, D), W[p + "q.norm"], eps)
    rot = mixer.get("rot")
    if rot:
        q = rotate_pairs(q, positions, scaled_frequencies(rot["base"], rot["dims"], rot.get("scaling")))
    chunk = (mixer.get("mask") or {}).get("size")
    out = torch.zeros(n, H, Dv, dtype=h.dtype)
    for t in range(n):
        seen = [j for j in range(n) if visible(positions[t], positions[j], chunk)]
        for a in range(H):
            g = a // (H // G)
            s = (keys[seen, g] @ q[t, a]) * mixer["scale"]
            out[t, a] = sink_softmax(s) @ values[seen, g]
    return out.reshape(n, H * Dv) @ W[p + "o"].T


# ------------------------------------------------------------------------------ feed-forwards

def dense_ff(h, W, p):
    return (torch.nn.functional.silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, W, p, router):
    """(chosen experts [n, top], their weights [n, top]): the weights are the softmax scores themselves,
    the choice goes by score + correction."""
    s = torch.softmax(h @ W[p + "router"].T, dim=-1)
    chosen = torch.topk(s + W[p + "correction"], router["top"], dim=-1).indices
    return chosen, torch.gather(s, 1, chosen)


def expert(h, W, p, e):
    return torch.relu(h @ W[f"{p}e{e}.up"].T) ** 2 @ W[f"{p}e{e}.down"].T


def moe_ff(h, W, p, router):
    chosen, weight = route(h, W, p, router)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            out[t] += g * (expert(h[t:t + 1], W, p, e)[0] if e < router["experts"] else h[t])
    return out


# ------------------------------------------------------------------------------ the model

def forward(raw, W, tokens, dtype=torch.float64, streams=None):
    """Logits [len(tokens), vocab].  `streams`, a list, receives the residual stream after every layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = float(raw["norm"]["eps"])
    positions = list(range(len(tokens)))
    x = rmsnorm(W["embed"][torch.as_tensor(tokens, dtype=torch.long)], W["embed.norm"], eps)
    kept = {}
    for i, layer in enumerate(raw["layers"]):
        p, mixer = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "wkv":
            y = wkv_mixer(x, W, p, mixer, eps)
        elif layer["type"] == "attention":
            src = mixer.get("kv_from")
            if src is None:
                kept[i] = attention_keys_values(x, W, p, mixer, eps, positions)
                src = i
            y = attention_mixer(x, W, p, mixer, eps, positions, *kept[src])
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        x = x + rmsnorm(y, W[f"l{i}.norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            f = dense_ff(x, W, f"l{i}.mlp.") if mlp["kind"] == "dense" else moe_ff(x, W, f"l{i}.mlp.", mlp["router"])
            x = x + rmsnorm(f, W[f"l{i}.norm2"], eps)
        if streams is not None:
            streams.append(x.clone())
    return rmsnorm(x, W["final.norm"], eps) @ W["head"].T


def load_model_dir(model_dir):
    """(config.json as a dict, name -> tensor) read with nothing but the file format: 8 bytes of length,
    that much JSON (name -> dtype, shape, offsets), then the data."""
    import numpy as np
    model_dir = Path(model_dir)
    raw = json.loads((model_dir / "config.json").read_text())
    blob = (model_dir / "model.safetensors").read_bytes()
    n = int.from_bytes(blob[:8], "little")
    header = json.loads(blob[8:8 + n])
    data = memoryview(blob)[8 + n:]
    W = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = bytes(data[lo:hi])
        if info["dtype"] == "BF16":
            bits = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy())
        elif info["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f4").copy())
        elif info["dtype"] == "F64":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f8").copy())
        elif info["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<i4").copy())
        else:
            raise ValueError(f"{name}: dtype {info['dtype']} is not read here")
        W[name] = t.view(*info["shape"])
    return raw, W
