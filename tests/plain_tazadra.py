"""Tazadra, plainly: whole sequences, no cache, no batches, float64, one function per
mechanism, written from the design's equations.  It reads config.json's keys and the
tensor names by itself and shares no code with the package.

``emulate_bf16`` rounds where the bfloat16 engine rounds (projections' inputs, the outputs
that feed another projection or the cache, activations); norms, scores, softmax, routers,
recurrences, what enters them, and the residual sum stay exact.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def bf(x: torch.Tensor, on: bool) -> torch.Tensor:
    return x.to(torch.bfloat16).to(F) if on else x


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


# ---- rotation --------------------------------------------------------------------------
def frequencies(rot: dict) -> torch.Tensor:
    """dims / 2 frequencies base^(-2i/dims), long wavelengths slowed down when the
    configuration has ``scaling`` {factor, low, high, original}."""
    dims = int(rot["dims"])
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = float(rot["base"]) ** (-2.0 * i / dims)
        if sc:
            wavelength = 2 * math.pi / f
            orig = float(sc["original"])
            if wavelength < orig / sc["high"]:
                pass
            elif wavelength > orig / sc["low"]:
                f = f / sc["factor"]
            else:
                s = (orig / wavelength - sc["low"]) / (sc["high"] - sc["low"])
                f = (1 - s) * f / sc["factor"] + s * f
        out.append(f)
    return torch.tensor(out, dtype=F)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """x [T, heads, d]: neighbours (2i, 2i + 1) of the first 2 * len(freq) values of every
    head are turned by position * freq[i]; the rest pass."""
    n = freq.numel()
    if n == 0:
        return x
    angle = positions.to(F)[:, None] * freq[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = a * c - b * s
    out[..., 1:2 * n:2] = b * c + a * s
    return out


# ---- attention -------------------------------------------------------------------------
def attention_keys_values(h, w, p, m, eps, positions, e16):
    """What the layer keeps of every position: keys after the norm over the whole
    projection and the rotation, and values."""
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    k = h @ w[p + ".k"].T
    v = bf(h @ w[p + ".v"].T, e16)
    k = rms_norm(k, w[p + ".k.norm"], eps).reshape(T, G, d)
    k = bf(rotate_pairs(k, positions, frequencies(m["rot"])), e16)
    return k, v.reshape(T, G, dv)


def attention(h, w, p, m, eps, positions, keys, values, e16, probes: Optional[dict] = None):
    """h [T, width] -> [T, width]; keys [T, G, d], values [T, G, dv] of the same positions
    (its own, or those of the layer that ``kv_from`` names)."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms_norm(h @ w[p + ".q"].T, w[p + ".q.norm"], eps).reshape(T, H, d)
    q = bf(rotate_pairs(q, positions, frequencies(m["rot"])), e16)
    gate = torch.sigmoid(h @ w[p + ".g"].T)  # [T, H]
    out = torch.zeros(T, H, dv, dtype=F)
    chunk = int(m["mask"]["size"]) if m.get("mask") else 0
    cap = float(m.get("softcap") or 0.0)
    i, j = positions[:, None], positions[None, :]
    seen = j <= i
    if chunk:
        seen = seen & ((i // chunk) == (j // chunk))
    for hq in range(H):
        g = hq // (H // G)
        s = (q[:, hq] @ keys[:, g].T) * float(m["scale"])
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~seen, float("-inf"))
        sink = w[p + ".sink"][hq]
        top = torch.maximum(s.max(dim=1).values, sink)
        e = torch.exp(s - top[:, None])
        denom = e.sum(dim=1) + torch.exp(sink - top)
        out[:, hq] = (e / denom[:, None]) @ values[:, g]
        if probes is not None:  # [heads, T, T] softmax weights, and the sink's share [heads, T]
            probes.setdefault("weights", []).append(e / denom[:, None])
            probes.setdefault("sink", []).append(torch.exp(sink - top) / denom)
    out = out * gate[:, :, None]
    return bf(out.reshape(T, H * dv), e16) @ w[p + ".o"].T


# ---- wkv --------------------------------------------------------------------------------
def wkv(h, w, p, m, eps, e16):
    H, d = m["heads"], m["dim"]
    T = h.shape[0]
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)

    def mix(s):
        return bf(h + (prev - h) * w[p + ".mu." + s], e16)
    r = bf(mix("r") @ w[p + ".r"].T, e16).reshape(T, H, d)
    k = bf(mix("k") @ w[p + ".k"].T, e16).reshape(T, H, d)
    v = bf(mix("v") @ w[p + ".v"].T, e16).reshape(T, H, d)
    gate = silu(bf(mix("g") @ w[p + ".g"].T, e16))
    low = bf(torch.tanh(mix("w") @ w[p + ".w1"].T), e16)
    decay = torch.exp(-torch.exp(low @ w[p + ".w2"].T + w[p + ".w0"])).reshape(T, H, d)
    u = w[p + ".u"].reshape(H, d)
    out = torch.zeros(T, H, d, dtype=F)
    S = torch.zeros(H, d, d, dtype=F)  # [head, key channel, value channel]
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = decay[t][:, :, None] * S + kv
    out = rms_norm(out, None, eps).reshape(T, H * d) * w[p + ".norm"] * gate
    return bf(out, e16) @ w[p + ".o"].T


# ---- mamba ------------------------------------------------------------------------------
def mamba1(h, w, p, m, e16):
    inner, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
    T = h.shape[0]
    xz = bf(h @ w[p + ".in"].T, e16)
    x, z = xz[:, :inner], xz[:, inner:]
    padded = torch.cat([torch.zeros(taps - 1, inner, dtype=F), x], dim=0)
    conv = w[p + ".conv"]  # [inner, taps], the last column is the current token's
    x = sum(padded[j:j + T] * conv[:, j] for j in range(taps)) + w[p + ".conv.b"]
    x = bf(silu(x), e16)
    dbc = x @ w[p + ".x"].T
    dt, B, C = bf(dbc[:, :R], e16), dbc[:, R:R + N], dbc[:, R + N:]
    dt = softplus(dt @ w[p + ".dt"].T + w[p + ".dt.b"])  # [T, inner]
    A = -torch.exp(w[p + ".A_log"])  # [inner, N]
    S = torch.zeros(inner, N, dtype=F)
    y = torch.zeros(T, inner, dtype=F)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w[p + ".D"] * x[t]
    return bf(y * silu(z), e16) @ w[p + ".o"].T


# ---- feed-forwards ----------------------------------------------------------------------
def dense_ff(h, w, p, mlp, e16):
    limit = float(mlp["limit"])
    g = torch.clamp(h @ w[p + ".gate"].T, max=limit)
    u = torch.clamp(h @ w[p + ".up"].T, min=-limit, max=limit)
    return bf(g * torch.sigmoid(1.702 * g) * (u + 1), e16) @ w[p + ".down"].T


def router(h, w, p, mlp):
    """(ids [T, top], scores [T, top], gap [T] between the last score in and the first out)."""
    top = int(mlp["router"]["top"])
    s = torch.sigmoid(h @ w[p + ".router"].T)
    order = torch.sort(s, dim=1, descending=True, stable=True)
    ids, val = order.indices[:, :top], order.values[:, :top]
    gap = (order.values[:, top - 1] - order.values[:, top]) if s.shape[1] > top \
        else torch.full((h.shape[0],), float("inf"), dtype=F)
    return ids, val, gap


def moe_ff(h, w, p, mlp, e16, margins: Optional[List] = None):
    ids, val, gap = router(h, w, p, mlp)
    if margins is not None:
        margins.append(gap)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(ids[t].tolist(), val[t]):
            x = h[t] * s  # (a scalar on the input: the engine applies it to the two products' sums)
            a = silu(x @ w[f"{p}.e{e}.gate"].T) * (x @ w[f"{p}.e{e}.up"].T)
            out[t] += bf(a, e16) @ w[f"{p}.e{e}.down"].T
    return out


# ---- the model ----------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, emulate_bf16: bool = False,
            margins: Optional[List] = None, layers_out: Optional[List] = None,
            probes: Optional[Dict[int, dict]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its first token."""
    w = {k: v.to(F) for k, v in w.items()}
    e16 = emulate_bf16
    eps, m_res = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x = w["embed"][tokens]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix", layer["mixer"]
        h = bf(x, e16)
        if layer["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = attention_keys_values(h, w, p, m, eps, positions, e16)
            keys, values = kept[i if m.get("kv_from") is None else int(m["kv_from"])]
            y = attention(h, w, p, m, eps, positions, keys, values, e16,
                          probes.setdefault(i, {}) if probes is not None else None)
        elif layer["type"] == "wkv":
            y = wkv(h, w, p, m, eps, e16)
        elif layer["type"] == "mamba1":
            y = mamba1(h, w, p, m, e16)
        else:
            raise ValueError(layer["type"])
        x = x + m_res * rms_norm(y, w[f"l{i}.norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = bf(x, e16)
            y = dense_ff(h, w, f"l{i}.mlp", mlp, e16) if mlp["kind"] == "dense" \
                else moe_ff(h, w, f"l{i}.mlp", mlp, e16, margins)
            x = x + m_res * rms_norm(y, w[f"l{i}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = bf(rms_norm(x, w["final.norm"], eps), e16) @ w["head"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy_generate(cfg: dict, w: Dict[str, torch.Tensor], prompt, new_tokens: int) -> List[int]:
    """The tokens that greedy decoding appends (ties to the lower id), the slow way: the
    whole sequence again for every token."""
    seq, out = list(prompt), []
    for _ in range(new_tokens):
        logits = forward(cfg, w, seq)[-1]
        best = int(torch.nonzero(logits == logits.max())[0])
        out.append(best)
        seq.append(best)
    return out
