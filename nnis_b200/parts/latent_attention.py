"""Causal attention whose keys and values come from one small latent per position.

The layer's input h goes down to two latents: ``cq = rms(W_dq h) * w_q`` for the
queries and ``c = rms((W_dkv h)[:kv_rank]) * w_kv`` for keys and values; the last
``rot_dim`` rows of ``W_dkv h`` are a key part that every head shares and that is
rotated by position.  Per head, ``q = W_uq cq`` is ``dim`` plain and ``rot_dim``
rotated values, the plain key is ``W_uk c`` and the value ``W_uv c``; a score is
``(q_plain . k_plain + q_rot . k_rot) * scale`` and the weights an ordinary softmax
over the positions up to the query's.

Only ``[c | k_rot]`` is cached, one row per position for all heads, in a cache
group without storage for values.  Because ``q_plain . (W_uk c) = (W_uk^T q_plain) . c``,
the queries are carried into the latent's space (one small product per head,
``W_uk`` transposed per head at load) and attention runs there: a score is one dot
product with the cached row, the output is a weighted sum of the rows' ``c`` part,
and the heads' values are made from that sum (``W_uv`` per head) before ``W_o`` adds
into the residual stream.  Prompts, later chunks and single tokens take the same way.

params: hidden_size, heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, eps,
position (a ``rope_frequencies`` PartSpec), names {dq, dq_norm, uq, dkv, dkv_norm,
uk, uv, o}.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..cache import PAGE_SIZE, KVRequest, KVView
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import MIXERS, POSITIONS, Part
from .linear import ADD_F32, STORE, STORE_F32, linear


class LatentAttention(Part):
    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.rot = int(params["rot_dim"])
        self.vdim = int(params["vdim"])
        self.q_rank = int(params["q_rank"])
        self.kv_rank = int(params["kv_rank"])
        self.scale = float(params["scale"])
        self.eps = float(params["eps"])
        self.names = params["names"]
        pos = params["position"]
        self.position = POSITIONS.build(pos.kind, pos.params, prefix, dtype, device)
        if not hasattr(self.position, "frequencies"):
            raise ValueError("latent attention rotates by a table of frequencies (rope_frequencies)")
        if self.position.dims > self.rot:
            raise ValueError(f"rotation over {self.position.dims} dimensions, the rotated part has {self.rot}")
        for what in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
            if getattr(self, what) <= 0:
                raise ValueError(f"latent attention: {what} must be positive")
        if self.kv_rank > 512:
            raise ValueError("latent attention kernels take latents of up to 512 values")
        self.row = self.kv_rank + self.rot  # a cached row, and a query in the latent's space
        self.w_down = self.w_uq = self.w_ukt = self.w_uv = self.w_o = None
        self.norm_q = self.norm_kv = None

    # -- weights ----------------------------------------------------------
    def _name(self, key: str) -> str:
        return self.tensor_name(self.names[key])

    def weight_specs(self) -> Dict[str, WeightSpec]:
        W, H = self.hidden, self.heads
        return {
            self._name("dq"): WeightSpec((self.q_rank, W), "matrix", fan_in=W),
            self._name("dq_norm"): WeightSpec((self.q_rank,), "vector", init="ones"),
            self._name("uq"): WeightSpec((H * (self.dim + self.rot), self.q_rank), "matrix", fan_in=self.q_rank),
            self._name("dkv"): WeightSpec((self.kv_rank + self.rot, W), "matrix", fan_in=W),
            self._name("dkv_norm"): WeightSpec((self.kv_rank,), "vector", init="ones"),
            self._name("uk"): WeightSpec((H * self.dim, self.kv_rank), "matrix", fan_in=self.kv_rank),
            self._name("uv"): WeightSpec((H * self.vdim, self.kv_rank), "matrix", fan_in=self.kv_rank),
            self._name("o"): WeightSpec((W, H * self.vdim), "matrix", fan_in=H * self.vdim),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        H = self.heads
        # both down-projections read h: one product [q latent | c raw | k_rot raw]
        self.w_down = torch.cat([tensors[self._name("dq")], tensors[self._name("dkv")]], 0).contiguous()
        self.norm_q = tensors[self._name("dq_norm")]
        self.norm_kv = tensors[self._name("dkv_norm")]
        self.w_uq = tensors[self._name("uq")]
        # per head [kv_rank, dim]: the product that carries q_plain into the latent's space
        self.w_ukt = tensors[self._name("uk")].view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[self._name("uv")].view(H, self.vdim, self.kv_rank).contiguous()
        self.w_o = tensors[self._name("o")]

    def parameter_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in
                   (self.w_down, self.w_uq, self.w_ukt, self.w_uv, self.w_o, self.norm_q, self.norm_kv))

    # -- cache ------------------------------------------------------------
    def cache_request(self) -> Optional[KVRequest]:
        return KVRequest(1, self.row, 0, values=False)

    def check_shared_cache(self, view: KVView) -> None:
        raise ValueError("latent attention writes a cache of its own")

    def step_flops(self, counts, starts) -> float:
        H, W = self.heads, self.hidden
        tokens = sum(counts)
        per_token = W * (self.q_rank + self.row) + self.q_rank * H * (self.dim + self.rot) \
            + H * self.dim * self.kv_rank + H * self.vdim * self.kv_rank + H * self.vdim * W
        keys = sum(c * st + c * (c + 1) // 2 for c, st in zip(counts, starts))
        return 2.0 * tokens * per_token + 2.0 * H * (self.row + self.kv_rank) * keys

    # -- work lists ---------------------------------------------------------
    def _tiles_name(self) -> str:
        return f"latent_mma/heads{self.heads}/rows{ops.latent_tile_rows(self.kv_rank)}"

    def _tensor_cores(self) -> bool:
        return self.dtype == torch.bfloat16 and ops.attention_latent_mma_takes(self.row, self.kv_rank, PAGE_SIZE)

    def step_tables(self, counts, starts, have=()):
        """The tiles of the tensor-core kernel for a prompt step: 64 or 128 stacked (token,
        head) rows each; the same for every layer with this number of heads and tile."""
        if not self._tensor_cores() or self._tiles_name() in have:
            return {}
        return {self._tiles_name(): ops.latent_tiles(counts, starts, self.heads,
                                                     ops.latent_tile_rows(self.kv_rank))}

    def _decode_splits(self, ctx, n: int) -> int:
        """Slices of the key range in a step of single tokens: enough CTAs for two per SM,
        at least two pages a slice."""
        ctas = n * -(-self.heads // ops.latent_tile_rows(self.kv_rank)) * -(-self.kv_rank // 512)
        pages = max(1, -(-ctx.max_context // PAGE_SIZE))
        want = -(-2 * ops.sm_count(self.device) // max(1, ctas * max(1, ctx.share)))
        return int(max(1, min(want, pages // 2, 64)))

    # -- run --------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor, cache: KVView) -> None:
        n = residual.shape[0]
        H, ws = self.heads, ctx.workspace
        table = ctx.page_tables[cache.group]
        freq = self.position.frequencies()
        down = ws.get("latent_down", (n, self.q_rank + self.row), torch.float32)
        linear(x, self.w_down, None, down, STORE_F32, decode=ctx.decode)
        cq = ws.get("latent_cq", (n, self.q_rank), self.dtype)
        ops.latent_prep(down, self.norm_q, self.norm_kv, freq, ctx.token_pos, ctx.token_seq, table, cq,
                        cache.k, self.q_rank, self.kv_rank, self.rot, self.position.dims, self.eps)
        q = ws.get("latent_q", (n, H * (self.dim + self.rot)), self.dtype)
        linear(cq, self.w_uq, None, q, STORE, decode=ctx.decode)
        q_lat = ws.get("latent_q_abs", (n, H * self.row), self.dtype)
        ops.batched_linear(q, self.dim + self.rot, self.w_ukt, q_lat, self.row)
        if self.rot:
            ops.rope_part(q, self.dim + self.rot, self.dim, q_lat, self.row, self.kv_rank, ctx.token_pos,
                          freq, H, self.rot, self.position.dims)
        o_lat = ws.get("latent_o", (n, H * self.kv_rank), self.dtype)
        tiles = ctx.tables.get(self._tiles_name())
        if self._tensor_cores() and (ctx.decode or tiles is not None):
            splits = self._decode_splits(ctx, n) if ctx.decode else 1
            partial = ws.get("attn_partial", (n * H * splits * (self.kv_rank + 2),), torch.float32) \
                if splits > 1 else None
            if ctx.decode:
                ops.attention_latent_mma(q_lat, cache.k, None, None, None, None, ctx.token_pos, ctx.token_seq,
                                         table, o_lat, H, self.kv_rank, self.scale, splits, partial)
            else:
                ops.attention_latent_mma(q_lat, cache.k, tiles, ctx.seq_first_row, ctx.seq_start,
                                         ctx.seq_count, ctx.token_pos, ctx.token_seq, table, o_lat, H,
                                         self.kv_rank, self.scale)
        else:
            splits = ctx.attention_splits(n * H)
            partial = ws.get("attn_partial", (n * H * splits * (self.kv_rank + 2),), torch.float32) \
                if splits > 1 else None
            ops.attention_latent(q_lat, cache.k, ctx.token_pos, ctx.token_seq, table, o_lat, H, self.kv_rank,
                                 self.scale, splits, partial)
        attn = ws.get("attn", (n, H * self.vdim), self.dtype)
        ops.batched_linear(o_lat, self.kv_rank, self.w_uv, attn, self.vdim)
        linear(attn, self.w_o, None, residual, ADD_F32, ws, decode=ctx.decode)


MIXERS.register("latent_attention", LatentAttention)
