"""WKV time mixing: a recurrent mixer whose decay depends on the token, with a state of
fixed size per sequence.

With h the part's input and h' the input of the token before (zeros before the first
token), five streams read their own mix of the two, mix_s = h + (h' - h) * mu_s:

    r = W_r mix_r    k = W_k mix_k    v = W_v mix_v    gate = silu(W_g mix_g)
    w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))          (heads x dim values each)

Per head, with S [dim, dim] (key channel x value channel) starting at zero:

    o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t          S_t = diag(w_t) S_{t-1} + k_t v_t^T

Each head's o is divided by its root mean square, the heads are joined, multiplied by a
weight per channel and by the gate, and W_o adds the result into the residual rows it is
given.  S and h' are float32 in the cache's state area, one of each per slot, so a later
portion of a prompt or a single token goes on from what the tokens before left; the decay,
the recurrence, the unit norm and the gate's silu are float32 in every dtype.  A long prompt is cut
into runs of tokens that start from zero side by side; the states between the runs are then put
together in order (the recurrence is linear in the state, and a run's decay of key channel k is the
product of its tokens' w_k), and a second pass over the runs, each from its true state, writes the
outputs.

params: hidden_size, heads, dim, decay_rank, eps, names {mu (a stem; ".r", ".k", ".v",
".g", ".w" follow), r, k, v, g, w1, w2, w0, u, norm, o}.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..cache import StateRequest, StateView
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import MIXERS, Part
from .linear import ADD_F32, STORE, STORE_F32, linear

STREAMS = ("r", "k", "v", "g", "w")


class WKV(Part):
    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.rank = int(params.get("decay_rank", -1))  # -1: the stored tensors' own
        self.eps = float(params["eps"])
        self.names = params["names"]
        if not 0 < self.dim <= 256:
            raise ValueError(f"wkv kernels take heads of up to 256 channels; got {self.dim}")
        self.mu = self.w = self.w0 = self.u = self.norm = None

    def _name(self, key: str, tail: str = "") -> str:
        return self.tensor_name(self.names[key] + tail)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        W, C = self.hidden, self.heads * self.dim
        specs = {self._name("mu", "." + s): WeightSpec((W,), "vector") for s in STREAMS}
        for p in ("r", "k", "v", "g"):
            specs[self._name(p)] = WeightSpec((C, W), "matrix", fan_in=W)
        specs[self._name("w1")] = WeightSpec((self.rank, W), "matrix", fan_in=W)
        specs[self._name("w2")] = WeightSpec((C, self.rank), "matrix", fan_in=self.rank)
        specs[self._name("w0")] = WeightSpec((C,), "vector")
        specs[self._name("u")] = WeightSpec((self.heads, self.dim), "vector")
        specs[self._name("norm")] = WeightSpec((C,), "vector", init="ones")
        specs[self._name("o")] = WeightSpec((W, C), "matrix", fan_in=C)
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.mu = torch.stack([tensors[self._name("mu", "." + s)] for s in STREAMS]).contiguous()
        self.w = {p: tensors[self._name(p)] for p in ("r", "k", "v", "g", "w1", "w2", "o")}
        if self.w["w1"].shape[0] != self.w["w2"].shape[1]:
            raise ValueError(f"{self._name('w1')} and {self._name('w2')} differ in the decay's inner size")
        self.rank = int(self.w["w1"].shape[0])
        self.w0 = tensors[self._name("w0")]
        self.u = tensors[self._name("u")].contiguous()
        self.norm = tensors[self._name("norm")]

    def parameter_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.w.values())

    def cache_request(self) -> StateRequest:
        return StateRequest((self.heads, self.dim, self.dim), torch.float32,
                            extra=(((self.hidden,), torch.float32),))

    def check_shared_cache(self, view) -> None:
        raise ValueError("wkv keeps a state of its own")

    def step_flops(self, counts, starts) -> float:
        W, C = self.hidden, self.heads * self.dim
        return 2.0 * sum(counts) * (5 * W * C + max(self.rank, 0) * (W + C) + 2 * C * self.dim)

    SEGMENTS, FIRST_SEGMENT = "scan/segments", "scan/first_segment"

    def step_tables(self, counts, starts, have=()):
        """Prompt steps with a sequence longer than two runs: the runs of every sequence, worked side
        by side (the same list for every recurrent layer of the model that cuts its prompts so)."""
        seg = ops.SCAN_SEGMENT
        if seg <= 0 or max(counts) <= 2 * seg or self.SEGMENTS in have:
            return {}
        segments, first = ops.scan_segments(counts, seg)
        return {self.SEGMENTS: segments, self.FIRST_SEGMENT: first}

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor, cache: StateView) -> None:
        n = residual.shape[0]
        C, ws = self.heads * self.dim, ctx.workspace
        state, prev = cache.state, cache.extra[0]
        seq = (ctx.token_pos, ctx.token_seq, ctx.seq_slots, ctx.seq_first_row, ctx.seq_count)
        mixes = ws.get("wkv_mixes", (len(STREAMS), n, self.hidden), self.dtype)
        ops.wkv_mix(x, self.mu, prev, *seq, mixes)
        rkvg = ws.get("wkv_rkvg", (4, n, C), self.dtype)
        for i, p in enumerate(("r", "k", "v", "g")):
            linear(mixes[i], self.w[p], None, rkvg[i], STORE, decode=ctx.decode)
        low_raw = ws.get("wkv_low_raw", (n, self.rank), torch.float32)
        linear(mixes[4], self.w["w1"], None, low_raw, STORE_F32, decode=ctx.decode)
        low = ws.get("wkv_low", (n, self.rank), self.dtype)
        ops.tanh_rows(low_raw, low)
        decay = ws.get("wkv_decay", (n, C), torch.float32)
        linear(low, self.w["w2"], self.w0, decay, STORE_F32, decode=ctx.decode)
        o_raw = ws.get("wkv_o", (n, C), torch.float32)
        segments = ctx.tables.get(self.SEGMENTS) if not ctx.decode else None
        runs = segments.shape[0] if segments is not None else 0
        ops.wkv_scan(rkvg[0], rkvg[1], rkvg[2], decay, self.u, state, *seq, o_raw, self.heads, self.dim,
                     segments=segments, seq_first_segment=ctx.tables.get(self.FIRST_SEGMENT),
                     seg_len=ops.SCAN_SEGMENT,
                     seg_state=ws.get("wkv_run_state", (runs, self.heads, self.dim, self.dim), torch.float32)
                     if runs else None,
                     seg_logw=ws.get("wkv_run_logw", (runs, self.heads, self.dim), torch.float32) if runs else None)
        out = ws.get("wkv_out", (n, C), self.dtype)
        ops.wkv_finish(o_raw, rkvg[3], self.norm, x, prev, *seq, out, self.heads, self.dim, self.eps)
        linear(out, self.w["o"], None, residual, ADD_F32, ws, decode=ctx.decode)


MIXERS.register("wkv", WKV)
