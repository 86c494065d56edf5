"""Typed configuration of the Dafolorn decoder, read from config.json.

Keys: `architecture` ("Dafolorn"), `vocab`, `width`, `norm.eps`, `canon.taps` (the short
convolution in front of every sublayer; absent: none), `logit_softcap` (absent: none),
`layers` (a list; each entry has `type`, the mixer's sizes under `mixer`, and `mlp`, which is
null or {`kind`, `ff`}), and `loop` {`start`, `stop`, `times`} (absent: every layer runs once).

The design, as the plan states it: a layer norms the input and the output of each sublayer and
puts a causal depthwise convolution over time in front of it; the mixer `latent_attention`
keeps one normed latent per token from which all heads' keys and values are made, sees a
sliding window, uses no position encoding, and has a learned sink per head in the softmax's
denominator; the feed-forward `dense` is up, xIELU, down.  Layers `start .. stop - 1` run
`times` times in a row with the same weights and a cache of their own per run; in front of
every run the stream is merged with the embedding output through one matrix and a learned
vector of that run is added.  The head is the embedding table, and logits are soft-capped.
Tensor names: `embed`, `final.norm`, `loop.in`, `loop.step`, and per layer i `l<i>.norm1`,
`.norm1b`, `.norm2`, `.norm2b`, `.canon1`, `.canon2`, `.mix.*`, `.mlp.*`.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry, SubPart
from .registry import ConfigError, register_architecture

_MIXERS = ("latent_attention",)
_MLPS = ("dense",)


def _integer(where: str, raw: dict, key: str, least: int = 1) -> int:
    v = raw.get(key) if isinstance(raw, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json (Dafolorn): {where}`{key}` must be an integer, got {v!r}")
    if int(v) < least:
        raise ConfigError(f"config.json (Dafolorn): {where}`{key}` must be at least {least}, got {v}")
    return int(v)


@register_architecture("Dafolorn", "dafolorn")
@dataclass
class DafolornConfig:
    vocab: int
    width: int
    layers: List[Dict[str, Any]]
    norm_eps: float = 1e-6
    canon_taps: Optional[int] = None
    logit_softcap: Optional[float] = None
    loop: Optional[Dict[str, int]] = None
    max_positions: int = 1 << 20            # the design has no position encoding and so no limit of its own

    architecture = "Dafolorn"
    model_type = "dafolorn"

    @property
    def vocab_size(self) -> int:            # the name generic callers use
        return self.vocab

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "DafolornConfig":
        for key in ("vocab", "width", "layers"):
            if raw.get(key) is None:
                raise ConfigError(f"config.json (Dafolorn): missing key `{key}`")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json (Dafolorn): `layers` must be a non-empty list")
        norm = raw.get("norm") or {}
        canon = raw.get("canon")
        loop = raw.get("loop")
        cap = raw.get("logit_softcap")
        cfg = cls(
            vocab=_integer("", raw, "vocab"),
            width=_integer("", raw, "width"),
            layers=copy.deepcopy(raw["layers"]),
            norm_eps=float(norm.get("eps", 1e-6)),
            canon_taps=None if not canon else _integer("canon.", canon, "taps"),
            logit_softcap=None if cap is None else float(cap),
            loop=None if not loop else {k: _integer("loop.", loop, k, least=0) for k in ("start", "stop", "times")},
            max_positions=_integer("", raw, "max_positions") if raw.get("max_positions") is not None else 1 << 20,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not self.norm_eps > 0:
            raise ConfigError(f"Dafolorn config: norm.eps must be positive, got {self.norm_eps}")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError(f"Dafolorn config: logit_softcap must be positive, got {self.logit_softcap}")
        if self.canon_taps is not None and self.canon_taps > 16:
            raise ConfigError(f"Dafolorn config: canon.taps {self.canon_taps} is beyond the kernels' 16")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict) or layer.get("type") not in _MIXERS:
                raise ConfigError(f"Dafolorn config: {where}type must be one of {_MIXERS}, got "
                                  f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"Dafolorn config: {where}mixer is missing")
            for key in ("heads", "dim", "vdim", "kv_rank"):
                _integer(where + "mixer.", m, key)
            if m["kv_rank"] > 1024:
                raise ConfigError(f"Dafolorn config: {where}mixer.kv_rank {m['kv_rank']} is beyond the kernels' 1024")
            if m.get("mask"):
                _integer(where + "mixer.mask.", m["mask"], "size")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in _MLPS:
                    raise ConfigError(f"Dafolorn config: {where}mlp.kind must be one of {_MLPS}")
                _integer(where + "mlp.", mlp, "ff")
        if self.loop is not None:
            lo, hi, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not 0 <= lo <= hi <= len(self.layers):
                raise ConfigError(f"Dafolorn config: loop {lo} .. {hi} does not lie inside the {len(self.layers)} layers")
            if hi > lo and times < 1:
                raise ConfigError(f"Dafolorn config: loop.times must be at least 1, got {times}")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(self.layers)}
        if self.canon_taps is not None:
            d["canon"] = {"taps": self.canon_taps}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            d["loop"] = dict(self.loop)
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        return d

    # --------------------------------------------------------------------- plan
    def run_order(self):
        """[(layer, run of the looped stretch or None, first layer of its run)] in the order the layers run."""
        n = len(self.layers)
        if self.loop is None or self.loop["stop"] <= self.loop["start"]:
            return [(i, None, False) for i in range(n)]
        lo, hi = self.loop["start"], self.loop["stop"]
        order = [(i, None, False) for i in range(lo)]
        for rep in range(self.loop["times"]):
            order += [(i, rep, i == lo) for i in range(lo, hi)]
        return order + [(i, None, False) for i in range(hi, n)]

    def _layer_spec(self, i: int) -> LayerSpec:
        layer, w = self.layers[i], self.width

        def norm(name):
            return SubPart("norm", PartSpec("rmsnorm", {"size": w, "eps": self.norm_eps, "unit_offset": True,
                                                        "tensor_name": name}))

        def conv(name):
            return SubPart("conv", PartSpec("causal_depthwise", {"channels": w, "taps": self.canon_taps,
                                                                 "tensor_name": name}))
        m = layer["mixer"]
        mask = m.get("mask") or {}
        mixer = PartSpec("latent_attention", {
            "hidden_size": w, "num_heads": m["heads"], "qk_dim": m["dim"], "v_dim": m["vdim"], "kv_rank": m["kv_rank"],
            "window": mask.get("size"), "scale": m.get("scale"), "latent_norm_eps": self.norm_eps, "sink": True})
        parts = {"norm_mixer": norm("norm1"), "mixer": SubPart("mixer", mixer, "mix."), "postnorm_mixer": norm("norm1b")}
        mlp = layer.get("mlp")
        if mlp is not None:
            ffn = PartSpec("up_act_down", {"hidden_size": w, "intermediate_size": mlp["ff"], "activation": "xielu"})
            parts.update({"norm_ffn": norm("norm2"), "ffn": SubPart("ffn", ffn, "mlp."), "postnorm_ffn": norm("norm2b")})
        if self.canon_taps is not None:
            parts["conv_mixer"] = conv("canon1")
            if mlp is not None:
                parts["conv_ffn"] = conv("canon2")
        block = PartSpec("sandwich", {"ffn": mlp is not None, "conv": self.canon_taps is not None})
        return LayerSpec(f"l{i}.", block, parts)

    def to_plan(self) -> ModelPlan:
        layers = [self._layer_spec(i) for i in range(len(self.layers))]
        order = self.run_order()
        looped = any(first for _i, _rep, first in order)
        if looped:                                         # the merge in front of every run, as one more "layer"
            merge = PartSpec("linear_reinject", {"width": self.width, "times": self.loop["times"]})
            layers.append(LayerSpec("loop.", PartSpec("reinject"), {"merge": SubPart("merge", merge)}))
        schedule: List[ScheduleEntry] = []
        for i, rep, first in order:
            if first:
                schedule.append(ScheduleEntry(layer=len(layers) - 1, cache=len(schedule), repeat=rep))
            schedule.append(ScheduleEntry(layer=i, cache=len(schedule), repeat=rep or 0))
        plan = ModelPlan(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            max_positions=self.max_positions,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": self.width, "tensor_name": "embed"}),
            layers=layers, schedule=schedule,
            final_norm=PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "unit_offset": True,
                                            "tensor_name": "final.norm"}),
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": True,
                                         "softcap": self.logit_softcap}),
            final_norm_prefix="", embedding_prefix="", lm_head_prefix="lm_head.",
            keeps_embedding_output=looped)
        plan.validate()
        return plan
