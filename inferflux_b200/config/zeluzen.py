"""Typed configuration of the Zeluzen decoder, read from config.json.

Keys: `architecture` ("Zeluzen"), `vocab`, `width`, `norm.eps`, and `layers`, a list whose entries have
`type` (`wkv` or `attention`), the mixer's sizes under `mixer`, and `mlp` (null, {`kind`: `dense`, `ff`} or
{`kind`: `moe`, `expert`: {`ff`}, `router`: {`experts`, `identity`, `top`}}).

    wkv        mixer: heads, dim                      (the decay's inner size is the shape of `mix.w1`)
    attention  mixer: heads, kv_heads, dim, vdim, scale, mask.size (absent: every earlier key), rot {base, dims,
               scaling {factor, low, high, original}} (absent: no rotation), kv_from (absent: keys and values
               of its own)

The design, as the plan states it: the embedding's rows are RMS-normed; a layer adds each sublayer's output
after an RMS norm of that output, and the sublayers read the stream itself; the recurrent mixer keeps a matrix
per head; the attention mixer norms query and key heads, turns part of every head in interleaved pairs with
frequencies that are slowed for long wavelengths, sees its own chunk of positions, has one more unit in the
softmax's denominator and may read an earlier layer's cache; the feed-forward is gated (SiLU) or a mixture
of squared-ReLU experts with a selection bias and experts that hand their input on; final norm and a head
of its own.  Tensor names: `embed`, `embed.norm`, `final.norm`, `head`, and per layer i `l<i>.norm1`,
`l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List

from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry, SubPart
from .registry import ConfigError, register_architecture

_TYPES = ("wkv", "attention")
_MLPS = ("dense", "moe")


def _integer(where: str, raw, key: str, least: int = 1) -> int:
    v = raw.get(key) if isinstance(raw, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json (Zeluzen): {where}`{key}` must be an integer, got {v!r}")
    if int(v) < least:
        raise ConfigError(f"config.json (Zeluzen): {where}`{key}` must be at least {least}, got {v}")
    return int(v)


def _number(where: str, raw, key: str) -> float:
    v = raw.get(key) if isinstance(raw, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json (Zeluzen): {where}`{key}` must be a number, got {v!r}")
    return float(v)


@register_architecture("Zeluzen", "zeluzen")
@dataclass
class ZeluzenConfig:
    vocab: int
    width: int
    layers: List[Dict[str, Any]]
    norm_eps: float = 1e-6
    max_positions: int = 1 << 20            # nothing in the design bounds a sequence

    architecture = "Zeluzen"
    model_type = "zeluzen"

    @property
    def vocab_size(self) -> int:            # the name generic callers use
        return self.vocab

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "ZeluzenConfig":
        for key in ("vocab", "width", "layers"):
            if raw.get(key) is None:
                raise ConfigError(f"config.json (Zeluzen): missing key `{key}`")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json (Zeluzen): `layers` must be a non-empty list")
        norm = raw.get("norm") or {}
        cfg = cls(vocab=_integer("", raw, "vocab"), width=_integer("", raw, "width"),
                  layers=copy.deepcopy(raw["layers"]), norm_eps=float(norm.get("eps", 1e-6)),
                  max_positions=_integer("", raw, "max_positions") if raw.get("max_positions") is not None else 1 << 20)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not self.norm_eps > 0:
            raise ConfigError(f"Zeluzen config: norm.eps must be positive, got {self.norm_eps}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind not in _TYPES:
                raise ConfigError(f"Zeluzen config: {where}type must be one of {_TYPES}, got {kind!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"Zeluzen config: {where}mixer is missing")
            _integer(where + "mixer.", m, "heads")
            _integer(where + "mixer.", m, "dim")
            if kind == "wkv":
                if m["dim"] > 256:
                    raise ConfigError(f"Zeluzen config: {where}mixer.dim {m['dim']} is beyond the kernel's 256")
                if m.get("rank") is not None:
                    _integer(where + "mixer.", m, "rank")
            else:
                self._validate_attention(i, m, where + "mixer.")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in _MLPS:
                raise ConfigError(f"Zeluzen config: {where}mlp.kind must be one of {_MLPS}")
            if mlp["kind"] == "dense":
                _integer(where + "mlp.", mlp, "ff")
            else:
                _integer(where + "mlp.expert.", mlp.get("expert"), "ff")
                r = mlp.get("router")
                n = _integer(where + "mlp.router.", r, "experts", least=0) + \
                    (_integer(where + "mlp.router.", r, "identity", least=0) if r.get("identity") is not None else 0)
                top = _integer(where + "mlp.router.", r, "top")
                if not 1 <= top <= n or n > 1024:
                    raise ConfigError(f"Zeluzen config: {where}mlp.router chooses {top} of {n} experts (at most 1024)")

    def _validate_attention(self, i: int, m: dict, where: str) -> None:
        m.setdefault("kv_heads", m["heads"])            # left out: a key/value head per query head, values as long as keys
        m.setdefault("vdim", m["dim"])
        for key in ("kv_heads", "vdim"):
            _integer(where, m, key)
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"Zeluzen config: {where}heads {m['heads']} is no multiple of kv_heads {m['kv_heads']}")
        for key in ("dim", "vdim"):
            if m[key] % 2 or m[key] > 256:
                raise ConfigError(f"Zeluzen config: {where}{key} {m[key]} is not an even size up to 256")
        _number(where, m, "scale")
        if m.get("mask"):
            _integer(where + "mask.", m["mask"], "size")
        rot = m.get("rot")
        if rot:
            dims = _integer(where + "rot.", rot, "dims", least=2)
            if dims % 2 or dims > m["dim"]:
                raise ConfigError(f"Zeluzen config: {where}rot.dims {dims} must be even and at most dim {m['dim']}")
            if not _number(where + "rot.", rot, "base") > 0:
                raise ConfigError(f"Zeluzen config: {where}rot.base must be positive")
            sc = rot.get("scaling")
            if sc:
                vals = {k: _number(where + "rot.scaling.", sc, k) for k in ("factor", "low", "high", "original")}
                if not (vals["factor"] > 0 and vals["original"] > 0 and vals["high"] > vals["low"] >= 0):
                    raise ConfigError(f"Zeluzen config: {where}rot.scaling {sc!r} is not usable")
        src = m.get("kv_from")
        if src is not None:
            if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                raise ConfigError(f"Zeluzen config: {where}kv_from must name an earlier layer, got {src!r}")
            other = self.layers[src]
            om = other.get("mixer") or {}
            if other.get("type") != "attention" or om.get("kv_from") is not None:
                raise ConfigError(f"Zeluzen config: {where}kv_from {src} is not an attention layer with keys of its own")
            if any(om.get(k) != m.get(k) for k in ("kv_heads", "dim", "vdim")):
                raise ConfigError(f"Zeluzen config: {where}kv_from {src} has other key/value sizes")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(self.layers)}
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        return d

    # --------------------------------------------------------------------- plan
    def _norm(self, name: str) -> SubPart:
        return SubPart("norm", PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "tensor_name": name}))

    def _readers(self, i: int) -> List[int]:
        return [j for j, l in enumerate(self.layers) if l["type"] == "attention" and l["mixer"].get("kv_from") == i]

    def _mixer_spec(self, i: int) -> PartSpec:
        layer, w = self.layers[i], self.width
        m = layer["mixer"]
        if layer["type"] == "wkv":
            return PartSpec("wkv", {"hidden_size": w, "num_heads": m["heads"], "head_dim": m["dim"],
                                    "decay_rank": m.get("rank"), "norm_eps": self.norm_eps})
        rot = m.get("rot")
        position = None if not rot else PartSpec("rope", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]),
                                                           "pairing": "interleaved", "scaling": rot.get("scaling")})
        chunk = (m.get("mask") or {}).get("size")
        # pages leave the cache when the chunk of positions they belong to is over, unless a layer that reads this
        # cache cuts its positions differently
        others = {(self.layers[j]["mixer"].get("mask") or {}).get("size") for j in self._readers(i)}
        retain = chunk if others <= {chunk} else None
        return PartSpec("attention", {
            "hidden_size": w, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "v_head_dim": m["vdim"], "window": None, "scale": float(m["scale"]), "position": position,
            "qkv_bias": False, "qk_norm": {"eps": self.norm_eps}, "chunk": chunk, "retain_chunk": retain, "sink": True,
            "own_kv": m.get("kv_from") is None,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}})

    def _ffn_spec(self, mlp: dict) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": mlp["ff"],
                                       "names": {"gate": "gate", "up": "up", "down": "down"}})
        r = mlp["router"]
        return PartSpec("moe", {"hidden_size": self.width, "expert_size": mlp["expert"]["ff"], "num_experts": r["experts"],
                                "num_identity": r.get("identity") or 0, "top": r["top"], "activation": "relu2",
                                "correction": True})

    def _layer_spec(self, i: int) -> LayerSpec:
        mlp = self.layers[i].get("mlp")
        parts = {"mixer": SubPart("mixer", self._mixer_spec(i), "mix."), "postnorm_mixer": self._norm("norm1")}
        if mlp is not None:
            parts.update({"ffn": SubPart("ffn", self._ffn_spec(mlp), "mlp."), "postnorm_ffn": self._norm("norm2")})
        return LayerSpec(f"l{i}.", PartSpec("postnorm", {"ffn": mlp is not None}), parts)

    def to_plan(self) -> ModelPlan:
        layers = [self._layer_spec(i) for i in range(len(self.layers))]
        schedule: List[ScheduleEntry] = []
        cache_of: Dict[int, int] = {}
        for i, layer in enumerate(self.layers):
            src = layer["mixer"].get("kv_from") if layer["type"] == "attention" else None
            if src is None:
                cache_of[i] = len(cache_of)
                schedule.append(ScheduleEntry(layer=i, cache=cache_of[i]))
            else:                                           # reads what the earlier layer stored, stores nothing
                schedule.append(ScheduleEntry(layer=i, cache=cache_of[src], writes_cache=False))
        plan = ModelPlan(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            max_positions=self.max_positions,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "tensor_name": "embed",
                                             "norm": {"tensor_name": "embed.norm", "eps": self.norm_eps}}),
            layers=layers, schedule=schedule,
            final_norm=PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "tensor_name": "final.norm"}),
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False,
                                         "tensor_name": "head"}),
            final_norm_prefix="", embedding_prefix="", lm_head_prefix="")
        plan.validate()
        return plan
