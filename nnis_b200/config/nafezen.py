"""Typed configuration of the Nafezen decoder, read from config.json.

config.json gives ``architecture`` ("Nafezen"), ``vocab``, ``width``, ``norm`` (``eps``,
``groups``) and ``layers``: a list whose entries name the layer's mixer (``type``:
"latent_attention" or "retention"), the mixer's sizes and constants (``mixer``) and
its feed-forward (``mlp``: ``kind`` "dense" with ``ff``, or "moe" with ``router``
{experts, top}, ``expert`` {ff} and optionally ``shared`` {ff}; or null for none).
Every size and every constant comes from there, layer by layer, so two layers of a
model may differ in all of them.

The model: token embedding followed by the model's norm; parallel layers (one norm,
mixer and feed-forward both read it and both add into the residual stream); the
model's norm again and the embedding table as the head.  Norms are RMS norms in
``norm.groups`` groups.  Tensor names: ``embed``, ``embed.norm``, ``final.norm`` and
``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*`` with no ``.weight`` ending; weights are
stored in bfloat16.  Positions have no bound of the model's own.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .llama import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# the rotation's angles are float32 products position * frequency; beyond 2^24 a
# position is no exact float32 any more
MAX_POSITIONS = 1 << 24


def _int(raw: Mapping[str, Any], key: str, where: str) -> int:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer; got {value!r}")
    return value


def _float(raw: Mapping[str, Any], key: str, where: str) -> float:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) \
            or value <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be finite and positive; got {value!r}")
    return float(value)


def _rotation(mixer: Mapping[str, Any], where: str, most: int) -> Tuple[int, float]:
    rot = mixer.get("rot")
    if not isinstance(rot, Mapping):
        raise ConfigError(f"config.json: {where}.rot must be an object with dims and base")
    dims = rot.get("dims")
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > most:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most {most}; got {dims!r}")
    return dims, _float(rot, "base", where + ".rot")


@dataclass(frozen=True)
class NafezenLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]


@dataclass(frozen=True)
class NafezenConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    layers: Tuple[NafezenLayer, ...]
    raw: Mapping[str, Any]

    architecture = "Nafezen"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "NafezenConfig":
        if raw.get("architecture") != cls.architecture:
            raise ConfigError(f"config.json: architecture must be {cls.architecture!r}; "
                              f"got {raw.get('architecture')!r}")
        vocab, width = _int(raw, "vocab", "config"), _int(raw, "width", "config")
        norm = raw.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("config.json: norm must be an object with eps and groups")
        eps, groups = _float(norm, "eps", "norm"), _int(norm, "groups", "norm")
        if width % groups:
            raise ConfigError(f"config.json: norm.groups={groups} does not divide width={width}")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: layers must be a list of at least one layer")
        layers: List[NafezenLayer] = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping) or not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} must be an object with type, mixer and mlp")
            kind, mixer = entry.get("type"), entry["mixer"]
            if kind == "latent_attention":
                for key in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
                    _int(mixer, key, where + ".mixer")
                rot_dim = mixer.get("rot_dim")
                if isinstance(rot_dim, bool) or not isinstance(rot_dim, int) or rot_dim < 0:
                    raise ConfigError(f"config.json: {where}.mixer.rot_dim must be an integer >= 0")
                _float(mixer, "scale", where + ".mixer")
                _rotation(mixer, where + ".mixer", rot_dim)
            elif kind == "retention":
                for key in ("heads", "dim", "vdim"):
                    _int(mixer, key, where + ".mixer")
                decay = mixer.get("decay")
                if not isinstance(decay, list) or len(decay) != mixer["heads"] or not all(
                        isinstance(d, (int, float)) and not isinstance(d, bool) and math.isfinite(d)
                        for d in decay):
                    raise ConfigError(f"config.json: {where}.mixer.decay must list one number per head")
                _rotation(mixer, where + ".mixer", mixer["dim"])
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                                  f"(latent_attention, retention)")
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"config.json: {where}.mlp must be an object or null")
                if mlp.get("kind") == "dense":
                    _int(mlp, "ff", where + ".mlp")
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
                    if mlp.get("shared") is not None:
                        if not isinstance(mlp["shared"], Mapping):
                            raise ConfigError(f"config.json: {where}.mlp.shared must be an object or null")
                        _int(mlp["shared"], "ff", where + ".mlp.shared")
                else:
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp.get('kind')!r} is not known "
                                      f"(dense, moe)")
            layers.append(NafezenLayer(kind, mixer, mlp))
        return cls(vocab, width, eps, groups, tuple(layers), dict(raw))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
                "layers": [{"type": l.type, "mixer": dict(l.mixer),
                            "mlp": None if l.mlp is None else dict(l.mlp)} for l in self.layers]}

    # ------------------------------------------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("group_rmsnorm", {"size": self.width, "eps": self.norm_eps,
                                          "groups": self.norm_groups, "name": name, "leaf": ""})

    def to_spec(self) -> ModelSpec:
        layers = []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            position = PartSpec("rope_frequencies", {"dims": m["rot"]["dims"], "base": m["rot"]["base"]})
            if layer.type == "latent_attention":
                mixer = PartSpec("latent_attention", {
                    "hidden_size": self.width, "heads": m["heads"], "dim": m["dim"],
                    "rot_dim": m["rot_dim"], "vdim": m["vdim"], "q_rank": m["q_rank"],
                    "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": self.norm_eps,
                    "position": position, "leaf": "",
                    "names": {"dq": "mix.dq", "dq_norm": "mix.dq.norm", "uq": "mix.uq", "dkv": "mix.dkv",
                              "dkv_norm": "mix.dkv.norm", "uk": "mix.uk", "uv": "mix.uv", "o": "mix.o"}})
            else:
                mixer = PartSpec("retention", {
                    "hidden_size": self.width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                    "decay": tuple(m["decay"]), "eps": self.norm_eps, "position": position, "leaf": "",
                    "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "g": "mix.g", "o": "mix.o"}})
            parts = {"norm": self._norm("norm1"), "mixer": mixer}
            mlp = layer.mlp
            if mlp is not None and mlp["kind"] == "dense":
                parts["ffn"] = PartSpec("gated_mlp", {
                    "hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "silu",
                    "bias": False, "leaf": "",
                    "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
            elif mlp is not None:
                shared = mlp.get("shared")
                parts["ffn"] = PartSpec("moe", {
                    "hidden_size": self.width, "experts": mlp["router"]["experts"],
                    "top": mlp["router"]["top"], "ff": mlp["expert"]["ff"],
                    "shared_ff": shared["ff"] if shared is not None else 0, "activation": "relu2",
                    "leaf": "",
                    "names": {"router": "mlp.router", "router_bias": "mlp.router.b", "expert": "mlp.e{e}",
                              "up": "up", "down": "down", "shared_up": "mlp.shared.up",
                              "shared_down": "mlp.shared.down", "shared_gate": "mlp.shared.sg"}})
            layers.append(LayerSpec(prefix=f"l{i}", block="parallel", parts=parts))
        spec = ModelSpec(
            architecture=self.architecture,
            hidden_size=self.width,
            vocab_size=self.vocab,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("normed_token_embedding", {
                "vocab_size": self.vocab, "hidden_size": self.width, "name": "embed", "leaf": "",
                "norm": self._norm("embed.norm")}),
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
            final_norm=self._norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": self.width,
                                          "name": "embed", "tied_to": "embed", "leaf": ""}),
            stop_token_ids=(),
            stored_dtype="bfloat16",
        )
        spec.validate()
        return spec
