"""Small Nafezen configurations and model folders for the tests; every size differs
between them, and none is a power-of-two family throughout."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, base=10000.0, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
            "kv_rank": kv_rank, "rot": {"base": base, "dims": rot_dim},
            "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}


def retention(heads, dim, vdim, decay, rot_dims, base=1000.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay),
            "rot": {"base": base, "dims": rot_dims}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(vocab, width, groups, eps, layers):
    return {"architecture": "Nafezen", "vocab": vocab, "width": width,
            "norm": {"eps": eps, "groups": groups}, "layers": layers}


# mixed layers; three heads; sizes that are multiples of 8 but no powers of two
MIXED = config(311, 96, 3, 1e-5, [
    layer("latent_attention", latent(3, 32, 8, 24, 40, 48), dense(136)),
    layer("retention", retention(3, 24, 40, [0.9, 0.97, 0.9990234375], 16), moe(5, 2, 56, shared=72)),
    layer("latent_attention", latent(3, 32, 8, 24, 40, 48, base=300.0), moe(4, 3, 24)),
    layer("retention", retention(2, 40, 24, [0.75, 0.998046875], 40), None),
])
# one head of retention first, a wide latent, one expert per token, one norm group,
# sizes that are no multiples of eight
ODD = config(200, 132, 1, 1e-6, [
    layer("retention", retention(1, 70, 34, [0.99609375], 70, base=50.0), dense(52)),
    layer("latent_attention", latent(5, 18, 30, 44, 26, 134, base=2000.0), moe(9, 1, 36, shared=10)),
    layer("latent_attention", latent(1, 10, 2, 6, 12, 20), None),
])
# one mechanism each
ONLY_LATENT = config(150, 64, 2, 1e-5, [layer("latent_attention", latent(4, 16, 16, 24, 32, 48), None)])
ONLY_RETENTION = config(150, 64, 4, 1e-5, [layer("retention", retention(2, 32, 48, [0.9375, 0.9990234375], 24), None)])
# key size 64 with a decay near one: long prompts are cut into runs that are worked side by side
LONG_RETENTION = config(150, 64, 1, 1e-5, [layer("retention", retention(3, 64, 40, [0.96875, 0.998046875, 0.9998779296875], 64),
                                               dense(40))])
ONLY_MOE = config(150, 72, 2, 1e-5, [layer("latent_attention", latent(2, 8, 8, 8, 16, 16), moe(7, 3, 40, shared=24))])
ONLY_DENSE = config(150, 72, 3, 1e-5, [layer("retention", retention(1, 16, 16, [0.5], 8), dense(88))])
# latents wider than one run of the tensor-core attention's output values (128), and wider than two
WIDE_LATENT = config(150, 64, 1, 1e-5, [layer("latent_attention", latent(3, 16, 16, 24, 32, 192), None),
                                        layer("latent_attention", latent(2, 24, 16, 16, 40, 320), dense(48))])
CONFIGS: Dict[str, dict] = {"mixed": MIXED, "odd": ODD, "latent": ONLY_LATENT, "retention": ONLY_RETENTION,
                            "moe": ONLY_MOE, "dense": ONLY_DENSE, "long_retention": LONG_RETENTION,
                            "wide_latent": WIDE_LATENT}


def make_model(tmp_dir: str, cfg: dict, seed: int, sharpen: float = 1.0) -> str:
    """A model folder with random weights whose activations and scores are of order one.
    ``sharpen`` multiplies the query up-projections, so that attention puts most of its
    weight on single keys: a key that an implementation loses then shows."""
    from nnis_b200.weights import write_random_model
    write_random_model(cfg, seed, tmp_dir, std=1.0, norm_std=0.1, std_by_fan_in=True)
    if sharpen != 1.0:
        from safetensors.torch import load_file, save_file
        path = os.path.join(tmp_dir, "model.safetensors")
        w = load_file(path)
        for name in list(w):
            if name.endswith(".mix.uq"):
                w[name] = (w[name].float() * sharpen).to(w[name].dtype)
        save_file(w, path)
    return tmp_dir


def load_weights(model_dir: str, as_bf16: bool):
    from safetensors.torch import load_file
    w = load_file(os.path.join(model_dir, "model.safetensors"))
    return {k: (v.to(torch.bfloat16).float() if as_bf16 else v.float()) for k, v in w.items()}


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)
