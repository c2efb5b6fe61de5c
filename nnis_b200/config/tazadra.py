"""Typed configuration of the Tazadra decoder, read from config.json.

config.json gives ``architecture`` ("Tazadra"), ``vocab``, ``width``, ``norm`` {eps},
``residual_mult``, ``logit_softcap`` and ``layers``: a list whose entries name the layer's
mixer (``type``: "attention", "wkv" or "mamba1"), the mixer's sizes and constants
(``mixer``; a wkv mixer may name ``decay_rank``, the inner size of its decay's two
projections, which otherwise is whatever the stored tensors have) and its feed-forward (``mlp``: ``kind`` "dense" with ``ff`` and ``limit``, or
"moe" with ``router`` {experts, top} and ``expert`` {ff}; or null for none).  Every size
and every constant that may differ between models comes from there, layer by layer.

The model: token embedding; layers whose norms stand on the sub-layers' OUTPUT,
x += m * norm1(mixer(x)), x += m * norm2(ff(x)), with m = ``residual_mult`` (the
sub-layers read x itself); the model's norm, the head, and a soft cap on the logits.
Mixers: attention with a norm of q and k over their whole projections, rotation of
neighbouring pairs with frequencies slowed down at long wavelengths, capped scores, a
chunked mask, a sink in the softmax and a gate per head (``kv_from``: j makes a layer read
the keys and values that layer j cached); WKV time mixing; Mamba's selective scan.
Feed-forwards: dense with a clamped gated activation, or experts with sigmoid scores on
the experts' inputs.  Tensor names: ``embed``, ``head``, ``final.norm`` and
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*`` with no ``.weight`` ending;
weights are stored in bfloat16.  Positions have no bound of the model's own.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .llama import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# angles are float32 products position * frequency; beyond 2^24 a position is no exact float32
MAX_POSITIONS = 1 << 24
# constants that the design fixes
DENSE_ALPHA = 1.702  # the dense feed-forward's activation is g * sigmoid(DENSE_ALPHA * g) * (u + 1)


def _int(raw: Mapping[str, Any], key: str, where: str, least: int = 1) -> int:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {least}; got {value!r}")
    return value


def _float(raw: Mapping[str, Any], key: str, where: str) -> float:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) \
            or value <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be finite and positive; got {value!r}")
    return float(value)


@dataclass(frozen=True)
class TazadraLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]


def _check_attention(mixer: Mapping[str, Any], where: str, index: int, entries: list) -> None:
    heads, kv_heads = _int(mixer, "heads", where), _int(mixer, "kv_heads", where)
    dim = _int(mixer, "dim", where)
    _int(mixer, "vdim", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}.heads={heads} is no multiple of kv_heads={kv_heads}")
    if dim % 2:
        raise ConfigError(f"config.json: {where}.dim={dim} must be even")
    _float(mixer, "scale", where)
    if mixer.get("softcap") is not None:
        _float(mixer, "softcap", where)
    mask = mixer.get("mask")
    if mask is not None:
        if not isinstance(mask, Mapping):
            raise ConfigError(f"config.json: {where}.mask must be an object with size, or null")
        _int(mask, "size", where + ".mask")
    rot = mixer.get("rot")
    if not isinstance(rot, Mapping):
        raise ConfigError(f"config.json: {where}.rot must be an object with dims and base")
    dims = rot.get("dims")
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most {dim}; got {dims!r}")
    _float(rot, "base", where + ".rot")
    scaling = rot.get("scaling")
    if scaling is not None:
        if not isinstance(scaling, Mapping):
            raise ConfigError(f"config.json: {where}.rot.scaling must be an object or null")
        for key in ("factor", "low", "high", "original"):
            _float(scaling, key, where + ".rot.scaling")
        if float(scaling["low"]) == float(scaling["high"]):
            raise ConfigError(f"config.json: {where}.rot.scaling.low and .high must differ")
    source = mixer.get("kv_from")
    if source is not None:
        if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < index:
            raise ConfigError(f"config.json: {where}.kv_from must name an earlier layer; got {source!r}")
        other = entries[source]
        om = other.get("mixer") if isinstance(other, Mapping) else None
        if other.get("type") != "attention" or not isinstance(om, Mapping) or om.get("kv_from") is not None:
            raise ConfigError(f"config.json: {where}.kv_from={source} names a layer without keys and values "
                              f"of its own")
        for key in ("kv_heads", "dim", "vdim"):
            if om.get(key) != mixer.get(key):
                raise ConfigError(f"config.json: {where}.{key} differs from layer {source}'s, whose keys and "
                                  f"values it reads")


@dataclass(frozen=True)
class TazadraConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_softcap: float  # 0: none
    layers: Tuple[TazadraLayer, ...]
    raw: Mapping[str, Any]

    architecture = "Tazadra"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "TazadraConfig":
        if raw.get("architecture") != cls.architecture:
            raise ConfigError(f"config.json: architecture must be {cls.architecture!r}; "
                              f"got {raw.get('architecture')!r}")
        vocab, width = _int(raw, "vocab", "config"), _int(raw, "width", "config")
        norm = raw.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("config.json: norm must be an object with eps")
        eps = _float(norm, "eps", "norm")
        mult = _float(raw, "residual_mult", "config") if raw.get("residual_mult") is not None else 1.0
        cap = _float(raw, "logit_softcap", "config") if raw.get("logit_softcap") is not None else 0.0
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: layers must be a list of at least one layer")
        layers: List[TazadraLayer] = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping) or not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} must be an object with type, mixer and mlp")
            kind, mixer = entry.get("type"), entry["mixer"]
            if kind == "attention":
                _check_attention(mixer, where + ".mixer", i, entries)
            elif kind == "wkv":
                for key in ("heads", "dim"):
                    _int(mixer, key, where + ".mixer")
                if mixer.get("decay_rank") is not None:
                    _int(mixer, "decay_rank", where + ".mixer")
            elif kind == "mamba1":
                for key in ("inner", "state", "dt_rank", "conv"):
                    _int(mixer, key, where + ".mixer")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                                  f"(attention, wkv, mamba1)")
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"config.json: {where}.mlp must be an object or null")
                if mlp.get("kind") == "dense":
                    _int(mlp, "ff", where + ".mlp")
                    _float(mlp, "limit", where + ".mlp")
                elif mlp.get("kind") == "moe":
                    router, expert = mlp.get("router"), mlp.get("expert")
                    if not isinstance(router, Mapping) or not isinstance(expert, Mapping):
                        raise ConfigError(f"config.json: {where}.mlp needs router and expert objects")
                    experts, top = _int(router, "experts", where + ".mlp.router"), \
                        _int(router, "top", where + ".mlp.router")
                    if top > experts:
                        raise ConfigError(f"config.json: {where}.mlp.router.top={top} exceeds its "
                                          f"{experts} experts")
                    _int(expert, "ff", where + ".mlp.expert")
                else:
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp.get('kind')!r} is not known "
                                      f"(dense, moe)")
            layers.append(TazadraLayer(kind, mixer, mlp))
        return cls(vocab, width, eps, mult, cap, tuple(layers), dict(raw))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
               "layers": [{"type": l.type, "mixer": dict(l.mixer),
                           "mlp": None if l.mlp is None else dict(l.mlp)} for l in self.layers]}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        return out

    # ------------------------------------------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "name": name, "leaf": ""})

    def _mixer(self, layer: TazadraLayer) -> PartSpec:
        m, W = layer.mixer, self.width
        if layer.type == "attention":
            rot = m["rot"]
            position = PartSpec("rope_frequencies", {"dims": rot["dims"], "base": rot["base"],
                                                     "pairing": "neighbours", "scaling": rot.get("scaling")})
            shared = m.get("kv_from") is not None
            return PartSpec("sink_attention", {
                "hidden_size": W, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
                "vdim": m["vdim"], "scale": m["scale"], "softcap": m.get("softcap") or 0.0,
                "chunk": m["mask"]["size"] if m.get("mask") else 0, "window": 0, "sink": True, "gate": True,
                "qk_norm": True, "eps": self.norm_eps, "position": position,
                "kv": "shared" if shared else "own", "leaf": "",
                "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "q_norm": "mix.q.norm",
                          "k_norm": "mix.k.norm", "sink": "mix.sink", "gate": "mix.g"}})
        if layer.type == "wkv":
            return PartSpec("wkv", {
                "hidden_size": W, "heads": m["heads"], "dim": m["dim"],
                # (the decay's inner size is the stored tensors' own unless the configuration names it)
                "decay_rank": m.get("decay_rank", -1), "eps": self.norm_eps, "leaf": "",
                "names": {"mu": "mix.mu", "r": "mix.r", "k": "mix.k", "v": "mix.v", "g": "mix.g",
                          "w1": "mix.w1", "w2": "mix.w2", "w0": "mix.w0", "u": "mix.u", "norm": "mix.norm",
                          "o": "mix.o"}})
        return PartSpec("selective_scan", {
            "hidden_size": W, "inner": m["inner"], "state": m["state"], "dt_rank": m["dt_rank"],
            "taps": m["conv"], "leaf": "",
            "names": {"in": "mix.in", "conv": "mix.conv", "conv_bias": "mix.conv.b", "x": "mix.x",
                      "dt": "mix.dt", "dt_bias": "mix.dt.b", "a_log": "mix.A_log", "d": "mix.D", "o": "mix.o"}})

    def to_spec(self) -> ModelSpec:
        layers, schedule = [], []
        for i, layer in enumerate(self.layers):
            parts = {"mixer": self._mixer(layer), "mixer_norm": self._norm("norm1")}
            mlp = layer.mlp
            if mlp is not None and mlp["kind"] == "dense":
                parts["ffn"] = PartSpec("gated_mlp", {
                    "hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "glu_clamp",
                    "limit": mlp["limit"], "alpha": DENSE_ALPHA, "bias": False, "leaf": "",
                    "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
            elif mlp is not None:
                parts["ffn"] = PartSpec("moe", {
                    "hidden_size": self.width, "experts": mlp["router"]["experts"],
                    "top": mlp["router"]["top"], "ff": mlp["expert"]["ff"], "shared_ff": 0,
                    "activation": "silu_gated", "scores": "sigmoid", "weight_on": "input", "leaf": "",
                    "names": {"router": "mlp.router", "expert": "mlp.e{e}", "gate": "gate", "up": "up",
                              "down": "down"}})
            if mlp is not None:
                parts["ffn_norm"] = self._norm("norm2")
            layers.append(LayerSpec(prefix=f"l{i}", block="branch_norm", parts=parts,
                                    params={"residual_mult": self.residual_mult,
                                            "tolerated": () if mlp is not None else ("norm2",)}))
            source = layer.mixer.get("kv_from") if layer.type == "attention" else None
            schedule.append(ScheduleEntry(i, cache_of=source))
        spec = ModelSpec(
            architecture=self.architecture,
            hidden_size=self.width,
            vocab_size=self.vocab,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                   "name": "embed", "leaf": ""}),
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=self._norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": self.width,
                                          "name": "head", "tied_to": None, "softcap": self.logit_softcap,
                                          "leaf": ""}),
            stop_token_ids=(),
            stored_dtype="bfloat16",
        )
        spec.validate()
        return spec
