"""Plain, slow Nafezen decoder used as the oracle of the Nafezen tests.

Whole sequences, no cache, one function per mechanism, float64 on the CPU.  It
shares no code with ``nnis_b200``: it reads ``config.json``'s keys and the
tensor names by itself.  Notation: ``x`` the residual stream ``[T, width]``,
``h`` a layer's normed input, ``p`` positions 0..T-1.

* grouped RMS norm: the row is cut into ``G`` equal runs, each divided by
  ``sqrt(mean(run^2) + eps)``, then the whole times ``w``;
* a layer is parallel: ``x += mixer(h) + ff(h)`` with ``h = norm1(x)``;
* latent attention: ``cq = rms(Wdq h) * wq``, ``q = Wuq cq`` (per head ``dim``
  plain then ``rot_dim`` rotated); ``Wdkv h`` = (``c`` raw, ``kr``); ``c =
  rms(c raw) * wkv``; per head ``k = Wuk c``, ``v = Wuv c``; score = ``(q_plain
  . k + q_rot . kr_rot) * scale``; causal softmax; ``Wo`` on the heads;
* retention: ``S_t = g S_{t-1} + k_t v_t^T``, ``o_t = S_t^T q_t`` with q, k
  rotated and k times ``dim^-0.5``; o divided by its root mean square per head,
  times ``silu(Wg h)``, then ``Wo``;
* feed-forward: dense ``Wdown(silu(Wgate h) * Wup h)``, or experts
  ``Wdown relu(Wup h)^2`` chosen by the ``top`` largest router logits with a
  softmax over the chosen ones, plus a shared expert times ``sigmoid(wsg . h)``.

``emulate_bf16=True`` rounds to bfloat16 where the bfloat16 engine stores
bfloat16 (normed inputs, projections' outputs, activations, attention outputs).
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence

import torch

Tensor = torch.Tensor
F = torch.float64


def _r(x: Tensor, bf: bool) -> Tensor:
    return x.to(torch.bfloat16).to(F) if bf else x


def grouped_rms_norm(x: Tensor, w: Tensor, eps: float, groups: int) -> Tensor:
    t, n = x.shape
    g = x.to(F).reshape(t, groups, n // groups)
    g = g / torch.sqrt((g * g).mean(dim=-1, keepdim=True) + eps)
    return g.reshape(t, n) * w.to(F)


def rms_norm(x: Tensor, w, eps: float) -> Tensor:
    x = x.to(F)
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w.to(F)


def rotate(x: Tensor, base: float, dims: int) -> Tensor:
    """x [T, heads, d]: the first ``dims`` of each head are turned, pair (i, i + dims/2),
    by the angle p * base^(-2i/dims); angles in float32 like the engine's tables."""
    t = x.shape[0]
    half = dims // 2
    f = torch.pow(torch.tensor(base, dtype=torch.float32),
                  -(2 * torch.arange(half, dtype=torch.float32)) / float(dims))
    a = torch.arange(t, dtype=torch.float32)[:, None] * f[None, :]
    c, s = torch.cos(a).to(F)[:, None, :], torch.sin(a).to(F)[:, None, :]
    u, v = x[..., :half].to(F), x[..., half:dims].to(F)
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:].to(F)], dim=-1)


def latent_attention(h: Tensor, w: Dict[str, Tensor], pre: str, m: dict, eps: float, bf: bool,
                     probe: dict = None) -> Tensor:
    """``probe``: a dict that receives the attention weights [heads, T, T] under "weights"."""
    t = h.shape[0]
    H, d, r, dv, kvr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = _r(rms_norm(_r(h @ w[pre + "dq"].to(F).t(), bf), w[pre + "dq.norm"], eps), bf)
    q = _r(cq @ w[pre + "uq"].to(F).t(), bf).reshape(t, H, d + r)
    kv = _r(h @ w[pre + "dkv"].to(F).t(), bf)
    c = _r(rms_norm(kv[:, :kvr], w[pre + "dkv.norm"], eps), bf)
    kr = kv[:, kvr:].reshape(t, 1, r)
    k = _r(c @ w[pre + "uk"].to(F).t(), bf).reshape(t, H, d)
    v = _r(c @ w[pre + "uv"].to(F).t(), bf).reshape(t, H, dv)
    rot = m["rot"]
    q_rot = _r(rotate(q[..., d:], rot["base"], rot["dims"]), bf)
    k_rot = _r(rotate(kr, rot["base"], rot["dims"]), bf)
    s = torch.einsum("thd,shd->hts", q[..., :d], k) + torch.einsum("thd,sd->hts", q_rot, k_rot[:, 0])
    s = s * m["scale"]
    mask = torch.ones(t, t, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, -math.inf)
    p = torch.softmax(s, dim=-1)
    if probe is not None:
        probe["weights"] = p
    o = _r(torch.einsum("hts,shd->thd", p, v), bf).reshape(t, H * dv)
    return o @ w[pre + "o"].to(F).t()


def retention(h: Tensor, w: Dict[str, Tensor], pre: str, m: dict, eps: float, bf: bool) -> Tensor:
    t = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = _r(h @ w[pre + "q"].to(F).t(), bf).reshape(t, H, d)
    k = _r(h @ w[pre + "k"].to(F).t(), bf).reshape(t, H, d)
    v = _r(h @ w[pre + "v"].to(F).t(), bf).reshape(t, H, dv)
    g = h @ w[pre + "g"].to(F).t()
    g = _r(g * torch.sigmoid(g), bf)
    rot = m["rot"]
    q = rotate(q, rot["base"], rot["dims"])
    k = rotate(k, rot["base"], rot["dims"]) * (float(d) ** -0.5)
    out = torch.zeros(t, H, dv, dtype=F)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=F)
        decay = float(m["decay"][hd])
        for i in range(t):
            S = decay * S + k[i, hd][:, None] * v[i, hd][None, :]
            out[i, hd] = S.t() @ q[i, hd]
    out = rms_norm(out, None, eps).reshape(t, H * dv)
    return _r(out * g, bf) @ w[pre + "o"].to(F).t()


def dense_ff(h: Tensor, w: Dict[str, Tensor], pre: str, bf: bool) -> Tensor:
    a = h @ w[pre + "gate"].to(F).t()
    u = h @ w[pre + "up"].to(F).t()
    return _r(a * torch.sigmoid(a) * u, bf) @ w[pre + "down"].to(F).t()


def relu2_expert(h: Tensor, up: Tensor, down: Tensor, bf: bool) -> Tensor:
    a = torch.relu(h @ up.to(F).t())
    return _r(a * a, bf) @ down.to(F).t()


def moe_ff(h: Tensor, w: Dict[str, Tensor], pre: str, mlp: dict, bf: bool, margins: list = None) -> Tensor:
    """``margins`` collects, per token, how far the last chosen logit lies above the best
    one left out (a small gap: a close call that rounding may decide either way)."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = (h.to(torch.float32) @ w[pre + "router"].to(torch.float32).t()
         + w[pre + "router.b"].to(torch.float32)).to(F)
    vals, idx = torch.topk(z, top, dim=-1)
    if margins is not None and top < E:
        ranked = torch.sort(z, dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top])
    gate = torch.softmax(vals, dim=-1)
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F)
    for e in range(E):
        y = relu2_expert(h, w[pre + f"e{e}.up"], w[pre + f"e{e}.down"], bf)
        weight = (gate * (idx == e)).sum(dim=-1, keepdim=True)
        out = out + weight * y
    if mlp.get("shared"):
        y = relu2_expert(h, w[pre + "shared.up"], w[pre + "shared.down"], bf)
        out = out + torch.sigmoid(h @ w[pre + "shared.sg"].to(F).t()) * y
    return out


def forward(cfg: dict, w: Dict[str, Tensor], tokens: Sequence[int], emulate_bf16: bool = False,
            layers_out: List[Tensor] = None, probes: Dict[int, dict] = None,
            margins: list = None) -> Tensor:
    """Logits [T, vocab] (float64) of one whole sequence; ``layers_out`` collects the
    residual stream after every layer; ``probes[i]`` receives layer i's attention weights;
    ``margins`` the routers' gaps per token (see ``moe_ff``)."""
    bf = emulate_bf16
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = w["embed"].to(F)[torch.tensor(list(tokens), dtype=torch.long)]
    x = grouped_rms_norm(x, w["embed.norm"], eps, groups)
    for i, layer in enumerate(cfg["layers"]):
        h = _r(grouped_rms_norm(x, w[f"l{i}.norm1"], eps, groups), bf)
        pre = f"l{i}.mix."
        if layer["type"] == "latent_attention":
            y = latent_attention(h, w, pre, layer["mixer"], eps, bf,
                                 probes.setdefault(i, {}) if probes is not None else None)
        elif layer["type"] == "retention":
            y = retention(h, w, pre, layer["mixer"], eps, bf)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                y = y + dense_ff(h, w, f"l{i}.mlp.", bf)
            elif mlp["kind"] == "moe":
                y = y + moe_ff(h, w, f"l{i}.mlp.", mlp, bf, margins)
            else:
                raise ValueError(mlp["kind"])
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    x = _r(grouped_rms_norm(x, w["final.norm"], eps, groups), bf)
    return x @ w["embed"].to(F).t()


def greedy_generate(cfg: dict, w: Dict[str, Tensor], prompt: Sequence[int], n_new: int,
                    emulate_bf16: bool = False) -> List[int]:
    """The plain loop: the whole sequence again for every new token; ties to the lower id."""
    tokens, out = list(prompt), []
    for _ in range(n_new):
        logits = forward(cfg, w, tokens, emulate_bf16)[-1]
        best = int(torch.nonzero(logits == logits.max())[0])
        tokens.append(best)
        out.append(best)
    return out
