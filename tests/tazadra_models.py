"""Small Tazadra configurations and model folders for the tests.  The sizes differ between
them in everything, none is a power-of-two family throughout, and each option of the
design appears switched on and off: values with a size of their own, several key/value
heads, several experts per token, a partial rotation and none, with and without slowed
frequencies, chunked masks of different sizes on a layer and on the one that reads its
keys, no mask, no cap, a multiplier of one, convolutions of one to five taps."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch


def attention(heads, kv_heads, dim, vdim, rot_dims, scale, base=10000.0, scaling=None, softcap=None,
              chunk=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "rot": {"base": base, "dims": rot_dims}}
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if softcap:
        m["softcap"] = softcap
    if chunk:
        m["mask"] = {"size": chunk}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def wkv(heads, dim, rank):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}}


def mamba(inner, state, dt_rank, taps):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": taps}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def layer(mixer, mlp):
    return {**mixer, "mlp": mlp}


def config(vocab, width, eps, mult, cap, layers):
    out = {"architecture": "Tazadra", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "residual_mult": mult, "layers": layers}
    if cap:
        out["logit_softcap"] = cap
    return out


# every mixer and both feed-forwards, a layer that reads another's keys under a mask of its own
MIXED = config(307, 96, 1e-5, 0.7, 20.0, [
    layer(attention(4, 2, 24, 16, 16, 0.3, base=1000.0, scaling=(4.0, 1.0, 4.0, 64), softcap=15.0, chunk=40),
          moe(6, 2, 40)),
    layer(wkv(3, 16, 12), dense(72, 3.0)),
    layer(mamba(80, 12, 6, 3), moe(5, 1, 24)),
    layer(attention(4, 2, 24, 16, 16, 0.25, base=1000.0, scaling=(4.0, 1.0, 4.0, 64), chunk=24, kv_from=0),
          dense(56, 1.5)),
    layer(wkv(1, 40, 8), None),
])
# sizes that are no multiples of eight or four; multiplier one; no cap on the logits; no mask, no
# cap on the scores, values wider than keys, one head for each key/value head
ODD = config(211, 76, 1e-6, 1.0, None, [
    layer(mamba(100, 5, 3, 2), dense(52, 1.5)),
    layer(attention(3, 3, 10, 34, 4, 0.4, base=50.0), None),
    layer(wkv(2, 22, 5), moe(9, 3, 36)),
    layer(attention(6, 1, 18, 6, 18, 0.2, base=2000.0, scaling=(8.0, 0.5, 2.0, 32), softcap=5.0, chunk=7),
          moe(3, 3, 20)),
    layer(mamba(36, 40, 9, 5), None),
    layer(attention(6, 1, 18, 6, 18, 0.2, base=2000.0, scaling=(8.0, 0.5, 2.0, 32), softcap=5.0, chunk=64,
                    kv_from=3), dense(20, 2.5)),
])
# one mechanism each
ONLY_ATTENTION = config(150, 64, 1e-5, 0.5, None, [
    layer(attention(4, 2, 16, 24, 8, 0.5, base=100.0, softcap=10.0, chunk=50), None),
    layer(attention(8, 1, 12, 40, 12, 0.6, base=30.0, chunk=33), None),        # eight query heads on one key/value head
    layer(attention(5, 1, 12, 40, 12, 0.6, base=30.0, softcap=6.0, kv_from=1), None)])  # five: no kernel of the group's own
ONLY_WKV = config(150, 64, 1e-5, 0.5, None, [layer(wkv(2, 32, 16), None)])
WIDE_WKV = config(150, 64, 1e-5, 0.8, None, [layer(wkv(2, 72, 10), None), layer(wkv(1, 136, 4), None),
                                             layer(wkv(1, 256, 3), None)])
ONLY_MAMBA = config(150, 64, 1e-5, 0.5, None, [layer(mamba(96, 16, 4, 4), None)])
WIDE_MAMBA = config(150, 48, 1e-5, 0.9, None, [layer(mamba(72, 70, 5, 1), None), layer(mamba(40, 130, 2, 3), None)])
ONLY_DENSE = config(150, 72, 1e-5, 0.5, 30.0, [layer(wkv(1, 8, 4), dense(88, 0.8))])
ONLY_MOE = config(150, 72, 1e-5, 0.5, None, [layer(wkv(1, 8, 4), moe(7, 3, 40))])
# attention alone, no rotation at all, scores without a cap: made sharp in the tests
SHARP = config(150, 64, 1e-5, 0.5, None, [
    layer(attention(4, 2, 16, 16, 8, 1.5, base=100.0, chunk=192), None),
    layer(attention(4, 2, 16, 16, 8, 1.5, base=100.0, chunk=70, kv_from=0), None)])
# key and value heads of 64 and of 128: the sizes of the tensor-core prompt attention; a layer that
# reads another's keys under a smaller chunk, a chunk that is no multiple of a page, one without a cap
HEADS_64 = config(150, 64, 1e-5, 0.6, None, [
    layer(attention(4, 2, 64, 64, 32, 0.2, base=100.0, softcap=12.0, chunk=100), None),
    layer(attention(6, 2, 64, 64, 32, 0.4, base=100.0, chunk=37, kv_from=0), dense(40, 2.0)),
    layer(attention(2, 1, 128, 128, 128, 0.15, base=5000.0, scaling=(4.0, 1.0, 2.0, 128), softcap=30.0), None)])
CONFIGS: Dict[str, dict] = {"mixed": MIXED, "heads64": HEADS_64, "odd": ODD, "attention": ONLY_ATTENTION, "wkv": ONLY_WKV,
                            "wide_wkv": WIDE_WKV, "mamba": ONLY_MAMBA, "wide_mamba": WIDE_MAMBA,
                            "dense": ONLY_DENSE, "moe": ONLY_MOE, "sharp": SHARP}


def make_model(tmp_dir: str, cfg: dict, seed: int) -> str:
    """A model folder with random weights whose activations and scores are of order one.
    Tensors that random numbers around zero would make harmless are moved to where they
    matter: decays spread between fast and slow, sinks of order one, bonuses of order one."""
    from nnis_b200.weights import write_random_model
    from safetensors.torch import load_file, save_file
    write_random_model(cfg, seed, tmp_dir, std=1.0, norm_std=0.1, std_by_fan_in=True)
    path = os.path.join(tmp_dir, "model.safetensors")
    w = load_file(path)
    g = torch.Generator().manual_seed(seed + 1)
    for name in list(w):
        t = w[name].float()
        if name.endswith(".mix.w0"):      # decays exp(-exp(w0 + ...)) between 0.37 and 0.998
            t = torch.empty_like(t).uniform_(-6.0, 0.0, generator=g)
        elif name.endswith(".mix.A_log"):  # -exp(A_log) between -0.05 and -2.7
            t = torch.empty_like(t).uniform_(-3.0, 1.0, generator=g)
        elif name.endswith(".mix.dt.b"):   # step sizes softplus(.) around 0.05 .. 1
            t = torch.empty_like(t).uniform_(-3.0, 0.5, generator=g)
        elif name.endswith(".mix.mu.r") or ".mix.mu." in name:
            t = torch.empty_like(t).uniform_(0.0, 1.0, generator=g)
        w[name] = t.to(torch.bfloat16)
    save_file(w, path)
    return tmp_dir


def load_weights(model_dir: str, as_bf16: bool):
    from safetensors.torch import load_file
    w = load_file(os.path.join(model_dir, "model.safetensors"))
    return {k: (v.to(torch.bfloat16).float() if as_bf16 else v.float()) for k, v in w.items()}


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)
