"""Selective scan: the recurrent mixer of Mamba, with a state of fixed size per sequence.

With h the part's input: W_in h = [x | z] (``inner`` channels each).  x passes a causal
convolution per channel over its last ``taps`` inputs (weights [inner, taps], the last
column is the current token's; zeros before the sequence's start; a bias) and silu.
W_x x = [dt (``dt_rank``) | B (``state``) | C (``state``)]; the step size per channel is
dt = softplus(W_dt dt + b), and with A = -exp(A_log) [inner, state]:

    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n        y_c = sum_n S[c, n] C_n + D_c x_c

The output y * silu(z) goes through W_o into the residual rows the part is given.  S and
the convolution's last taps - 1 inputs are float32 in the cache's state area, one of each per
slot, zero when a slot is taken, so a later portion of a prompt or a single token goes on
from what the tokens before left.  Step sizes, decays, B and C, the state and the sums are
float32 in every dtype.  A long prompt is cut into runs of tokens that start from zero side by
side; the states between the runs are then put together in order (the recurrence is linear in
the state, and a run's decay is exp(A * the sum of its step sizes)), and a second pass over the
runs, each from its true state, writes the outputs.

params: hidden_size, inner, state, dt_rank, taps, names {in, conv, conv_bias, x, dt,
dt_bias, a_log, d, o}.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..cache import StateRequest, StateView
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import MIXERS, Part
from .linear import ADD_F32, STORE, STORE_F32, linear


class SelectiveScan(Part):
    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.inner = int(params["inner"])
        self.state = int(params["state"])
        self.rank = int(params["dt_rank"])
        self.taps = int(params["taps"])
        self.names = params["names"]
        if not 0 < self.state <= 256:
            raise ValueError(f"selective scan kernels take up to 256 state values a channel; got {self.state}")
        if self.taps < 1:
            raise ValueError("selective scan: the convolution has at least one tap")
        self.w_in = self.w_dt_low = self.w_bc = self.w_dt = self.w_o = None
        self.conv = self.conv_bias = self.dt_bias = self.a_log = self.d = None

    def _name(self, key: str) -> str:
        return self.tensor_name(self.names[key])

    def weight_specs(self) -> Dict[str, WeightSpec]:
        W, I, N, R = self.hidden, self.inner, self.state, self.rank
        return {self._name("in"): WeightSpec((2 * I, W), "matrix", fan_in=W),
                self._name("conv"): WeightSpec((I, self.taps), "vector", fan_in=self.taps),
                self._name("conv_bias"): WeightSpec((I,), "vector"),
                self._name("x"): WeightSpec((R + 2 * N, I), "matrix", fan_in=I),
                self._name("dt"): WeightSpec((I, R), "matrix", fan_in=R),
                self._name("dt_bias"): WeightSpec((I,), "vector"),
                self._name("a_log"): WeightSpec((I, N), "vector"),
                self._name("d"): WeightSpec((I,), "vector", init="ones"),
                self._name("o"): WeightSpec((W, I), "matrix", fan_in=I)}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_in = tensors[self._name("in")]
        w_x = tensors[self._name("x")]
        # the step size's low-rank input and [B | C] as two products: the first feeds another
        # projection (operand dtype), the second enters the recurrence (float32)
        self.w_dt_low = w_x[:self.rank].contiguous()
        self.w_bc = w_x[self.rank:].contiguous()
        self.w_dt = tensors[self._name("dt")]
        self.w_o = tensors[self._name("o")]
        self.conv = tensors[self._name("conv")].contiguous()
        self.conv_bias = tensors[self._name("conv_bias")]
        self.dt_bias = tensors[self._name("dt_bias")]
        self.a_log = tensors[self._name("a_log")].contiguous()
        self.d = tensors[self._name("d")]

    def parameter_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_dt_low, self.w_bc, self.w_dt, self.w_o))

    def cache_request(self) -> StateRequest:
        return StateRequest((self.inner, self.state), torch.float32,
                            extra=(((max(self.taps - 1, 1), self.inner), torch.float32),))

    def check_shared_cache(self, view) -> None:
        raise ValueError("a selective scan keeps a state of its own")

    def step_flops(self, counts, starts) -> float:
        W, I, N, R = self.hidden, self.inner, self.state, self.rank
        return 2.0 * sum(counts) * (3 * W * I + I * (R + 2 * N) + I * R + I * self.taps + 3 * I * N)

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
        I, N, ws = self.inner, self.state, ctx.workspace
        state, conv_state = cache.state, cache.extra[0]
        xz = ws.get("scan_xz", (n, 2 * I), self.dtype)
        linear(x, self.w_in, None, xz, STORE, decode=ctx.decode)
        xc = ws.get("scan_xc", (n, I), self.dtype)
        ops.conv_silu(xz, self.conv, self.conv_bias, conv_state, ctx.token_pos, ctx.token_seq, ctx.seq_slots,
                      ctx.seq_first_row, xc)
        dt_low = ws.get("scan_dt_low", (n, self.rank), self.dtype)
        linear(xc, self.w_dt_low, None, dt_low, STORE, decode=ctx.decode)
        bc = ws.get("scan_bc", (n, 2 * N), torch.float32)
        linear(xc, self.w_bc, None, bc, STORE_F32, decode=ctx.decode)
        dt_raw = ws.get("scan_dt", (n, I), torch.float32)
        linear(dt_low, self.w_dt, self.dt_bias, dt_raw, STORE_F32, decode=ctx.decode)
        y = ws.get("scan_y", (n, I), self.dtype)
        segments = ctx.tables.get(self.SEGMENTS) if not ctx.decode else None
        runs = segments.shape[0] if segments is not None else 0
        ops.selective_scan(xc, xz, dt_raw, bc, self.a_log, self.d, state, conv_state, ctx.token_pos,
                           ctx.token_seq, ctx.seq_slots, ctx.seq_first_row, ctx.seq_count, y, self.taps,
                           segments=segments, seq_first_segment=ctx.tables.get(self.FIRST_SEGMENT),
                           seg_len=ops.SCAN_SEGMENT,
                           seg_state=ws.get("scan_run_state", (runs, I, N), torch.float32) if runs else None,
                           seg_dt=ws.get("scan_run_dt", (runs, I), torch.float32) if runs else None)
        linear(y, self.w_o, None, residual, ADD_F32, ws, decode=ctx.decode)


MIXERS.register("selective_scan", SelectiveScan)
