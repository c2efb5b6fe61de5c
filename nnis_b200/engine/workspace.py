"""Scratch tensors of a step, kept between steps and grown on demand.

Buffers are looked up by name; a request larger than the buffer on hand
replaces it.  Once a CUDA graph has been captured over the workspace it is
frozen: a request that would move a buffer is an error then, because the graph
holds the old address.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch


class Workspace:
    def __init__(self, device: torch.device):
        self.device = device
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._frozen = False
        self._children: Dict[str, "Workspace"] = {}
        self._streams: Dict[str, torch.cuda.Stream] = {}

    @property
    def frozen(self) -> bool:
        return self._frozen

    @frozen.setter
    def frozen(self, value: bool) -> None:
        self._frozen = bool(value)
        for child in self._children.values():
            child.frozen = value

    def child(self, name: str) -> "Workspace":
        """Buffers of a branch of the step that runs beside the rest on a stream of its own
        (same names, other memory); frozen together with this workspace."""
        if name not in self._children:
            if self._frozen:
                raise RuntimeError(f"workspace branch {name!r} would be made after graph capture")
            self._children[name] = Workspace(self.device)
        return self._children[name]

    def stream(self, name: str) -> torch.cuda.Stream:
        """The stream of the branch ``name`` (made once; a captured graph forks it from and
        joins it to the step's stream by events)."""
        if name not in self._streams:
            self._streams[name] = torch.cuda.Stream(device=self.device)
        return self._streams[name]

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        count = 1
        for s in shape:
            count *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < count:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would move after graph capture")
            # grow with headroom so a slowly growing batch does not reallocate each step
            buf = torch.empty(max(count, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:count].view(*shape)

    def kept_zero(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        """Like ``get``, for a buffer whose users leave every value they touched at zero again
        (an accumulator that the kernel which reads it last clears): zero when first handed out
        and when it has to grow, so that it needs no fill between uses."""
        count = 1
        for s in shape:
            count *= int(s)
        key = (name + "#kept_zero", dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < count:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would move after graph capture")
            buf = torch.zeros(max(count, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:count].view(*shape)

    def zeros(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        """A buffer that is zero when first handed out and that its users leave
        zero (tickets of kernels that reset them); never moved once made."""
        count = 1
        for s in shape:
            count *= int(s)
        key = (name + "#zeros", dtype, count)
        buf = self._buffers.get(key)
        if buf is None:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would be made after graph capture")
            buf = torch.zeros(max(count, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:count].view(*shape)

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values()) + \
            sum(child.bytes() for child in self._children.values())
