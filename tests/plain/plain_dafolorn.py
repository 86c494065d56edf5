"""A plain, slow statement of the Dafolorn decoder, one function per mechanism.

Test code only: it shares nothing with the package (no part, no kernel table, no
cache), works on whole sequences token by token where that is the clearest way to
say what a mechanism does, and computes in float64 unless told otherwise.  A model
is a configuration dictionary (the keys of config.json) and a dictionary of tensors
by name.

Notation: W is stored [out, in] and applied as W x; rms(x) = sqrt(mean(x^2) + eps).
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def unit_norm(x, eps):
    """x / rms(x) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is the distance from one."""
    return unit_norm(x, eps) * (1.0 + w)


def plain_weight_norm(x, w, eps):
    return unit_norm(x, eps) * w


def short_conv(h, w):
    """h [n, C] over time, w [C, taps]; tap `taps - 1` multiplies the present input, tap 0
    the oldest; before the sequence there are zeros.  Returns h + conv(h)."""
    n, taps = h.shape[0], w.shape[1]
    out = h.clone()
    for t in range(n):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def xielu(z, p, q):
    """Above zero a parabola with curvature softplus(p); below, an exponential
    branch with weight 1/2 + softplus(q); both with slope 1/2 at zero."""
    sp = lambda v: math.log1p(math.exp(v))
    a_pos, a_neg = sp(float(p)), 0.5 + sp(float(q))
    pos = a_pos * z * z + 0.5 * z
    neg = a_neg * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def windowed_sink_softmax(scores, sink):
    """scores [keys] of the keys one query sees, sink a number: weights over the keys whose
    denominator also counts exp(sink) once."""
    m = max(float(scores.max()), float(sink))
    e = torch.exp(scores - m)
    return e / (e.sum() + math.exp(float(sink) - m))


def latent_attention(h, t, prefix, mixer, eps):
    """h [n, width] -> [n, width].  Keys and values of every head are made from one
    normed latent per token; a query at i sees the keys at i - size + 1 .. i."""
    H, dk, dv, r = mixer["heads"], mixer["dim"], mixer["vdim"], mixer["kv_rank"]
    scale = float(mixer["scale"])
    size = mixer.get("mask", {}).get("size") if mixer.get("mask") else None
    n = h.shape[0]
    q = (h @ t[prefix + "q"].T).view(n, H, dk)
    c = plain_weight_norm(h @ t[prefix + "dkv"].T, t[prefix + "dkv.norm"], eps)      # [n, r]
    k = (c @ t[prefix + "uk"].T).view(n, H, dk)
    v = (c @ t[prefix + "uv"].T).view(n, H, dv)
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for i in range(n):
        lo = 0 if size is None else max(0, i - size + 1)
        for a in range(H):
            s = (k[lo:i + 1, a] @ q[i, a]) * scale
            p = windowed_sink_softmax(s, t[prefix + "sink"][a])
            out[i, a] = p @ v[lo:i + 1, a]
    return out.reshape(n, H * dv) @ t[prefix + "o"].T


def dense_ff(h, t, prefix):
    z = h @ t[prefix + "up"].T
    act = t[prefix + "act"]
    return xielu(z, act[0], act[1]) @ t[prefix + "down"].T


def layer(x, t, i, spec, eps, conv=True):
    """`conv` False: the design without its input convolutions (a configuration that names none)."""
    p = f"l{i}."
    h = offset_norm(x, t[p + "norm1"], eps)
    if conv:
        h = short_conv(h, t[p + "canon1"])
    if spec["type"] != "latent_attention":
        raise ValueError(spec["type"])
    x = x + offset_norm(latent_attention(h, t, p + "mix.", spec["mixer"], eps), t[p + "norm1b"], eps)
    if spec.get("mlp") is not None:
        if spec["mlp"]["kind"] != "dense":
            raise ValueError(spec["mlp"]["kind"])
        h = offset_norm(x, t[p + "norm2"], eps)
        if conv:
            h = short_conv(h, t[p + "canon2"])
        x = x + offset_norm(dense_ff(h, t, p + "mlp."), t[p + "norm2b"], eps)
    return x


def run_order(config):
    """[(layer, pass or None, first of its pass)] in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None, False) for i in range(n)]
    order = [(i, None, False) for i in range(loop["start"])]
    for rep in range(loop["times"]):
        order += [(i, rep, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    order += [(i, None, False) for i in range(loop["stop"], n)]
    return order


def forward(config, tensors, tokens, dtype=F, want_layers=False):
    """Logits [n, vocab] of one whole sequence (and the residual stream after every layer run)."""
    t = {k: v.to(dtype) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    x0 = t["embed"][torch.tensor(tokens, dtype=torch.long)]
    x, streams = x0, []
    for i, rep, first in run_order(config):
        if first:
            x = torch.cat([x, x0], dim=-1) @ t["loop.in"].T + t["loop.step"][rep]
        x = layer(x, t, i, config["layers"][i], eps, conv=bool(config.get("canon")))
        streams.append(x)
    logits = offset_norm(x, t["final.norm"], eps) @ t["embed"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(streams)) if want_layers else logits
