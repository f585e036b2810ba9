"""Flat parameter / gradient storage laid out by optimizer tier.

All trainable parameters of a model are re-homed as views of ONE contiguous buffer (model dtype) and get a
matching fp32 ``main_grad`` view of ONE gradient buffer. The layout is
``[ AdamW tier | Muon tier grouped by matrix shape | CentroidSteer tier ]`` so that

* the AdamW tier is updated by a single fused kernel launch over a contiguous range,
* same-shape Muon matrices are already a ``[K, m, n]`` stack (batched Newton-Schulz without copies),
* a data-parallel rank owns contiguous element ranges (AdamW) or whole matrices (Muon), which is what the
  fused reduce-scatter + update + all-gather kernel consumes.

The kernels write weight gradients straight into ``main_grad`` (fp32 accumulate in the GEMM epilogue);
gradients produced by PyTorch autograd (``p.grad``) are folded in by :meth:`fold_autograd_grads`.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch


@dataclass
class Segment:
    name: str
    param: torch.nn.Parameter
    tier: str  # "adamw" | "muon" | "steer"
    offset: int
    numel: int
    shape: Tuple[int, ...]
    mat_shape: Optional[Tuple[int, int, int]] = None  # (K, m, n) view used by the matrix tiers


@dataclass
class MuonGroup:
    shape: Tuple[int, int]
    offset: int  # start of the stack in the flat buffers
    count: int  # number of matrices
    segments: List[Segment] = field(default_factory=list)


class ParamArena:
    ALIGN = 128  # elements; keeps every segment 256-byte aligned for TMA and vector access

    def __init__(self, named_params: Sequence[Tuple[str, torch.nn.Parameter]], tiers: Dict[int, str],
                 mat_views: Optional[Dict[int, Tuple[int, int, int]]] = None, master_dtype=torch.float32,
                 storage_factory=None):
        """``storage_factory(total_elems, param_dtype, device) -> (flat_param, flat_grad)`` lets a caller place the
        two arenas in special memory (the symmetric NVLink heap for the fused data-parallel step)."""
        mat_views = mat_views or {}
        seen = set()
        uniq = []
        for n, p in named_params:
            if id(p) in seen or not p.requires_grad:
                continue
            seen.add(id(p))
            uniq.append((n, p))
        if not uniq:
            raise ValueError("no trainable parameters")
        self.device = uniq[0][1].device
        self.dtype = uniq[0][1].dtype

        def mv(p):
            if id(p) in mat_views:
                return tuple(mat_views[id(p)])
            if p.dim() == 2:
                return (1, p.shape[0], p.shape[1])
            if p.dim() == 3:
                return tuple(p.shape)
            return None

        adamw = [(n, p) for n, p in uniq if tiers.get(id(p), "adamw") == "adamw"]
        muon = [(n, p) for n, p in uniq if tiers.get(id(p)) == "muon"]
        steer = [(n, p) for n, p in uniq if tiers.get(id(p)) == "steer"]
        muon.sort(key=lambda np_: (mv(np_[1])[1], mv(np_[1])[2]))

        self.segments: List[Segment] = []
        self.muon_groups: List[MuonGroup] = []
        off = 0

        def place(n, p, tier):
            nonlocal off
            seg = Segment(n, p, tier, off, p.numel(), tuple(p.shape), mv(p) if tier != "adamw" else None)
            self.segments.append(seg)
            off += p.numel()
            return seg

        for n, p in adamw:
            place(n, p, "adamw")
            off = -(-off // 8) * 8
        off = -(-off // self.ALIGN) * self.ALIGN
        self.adamw_range = (0, off)
        cur = None
        for n, p in muon:
            K, m, nn_ = mv(p)
            if cur is None or cur.shape != (m, nn_):
                off = -(-off // self.ALIGN) * self.ALIGN
                cur = MuonGroup((m, nn_), off, 0)
                self.muon_groups.append(cur)
            seg = place(n, p, "muon")
            cur.segments.append(seg)
            cur.count += K
        off = -(-off // self.ALIGN) * self.ALIGN
        self.muon_range = (self.adamw_range[1], off)
        for n, p in steer:
            off = -(-off // self.ALIGN) * self.ALIGN
            place(n, p, "steer")
        off = -(-off // self.ALIGN) * self.ALIGN
        self.steer_range = (self.muon_range[1], off)
        self.total = off

        if storage_factory is not None:
            self.flat_param, self.flat_grad = storage_factory(self.total, self.dtype, self.device)
            assert self.flat_param.numel() == self.total and self.flat_grad.numel() == self.total
            self.flat_param.zero_()
            self.flat_grad.zero_()
        else:
            self.flat_param = torch.zeros(self.total, device=self.device, dtype=self.dtype)
            self.flat_grad = torch.zeros(self.total, device=self.device, dtype=torch.float32)
        self.flat_master = None
        if self.dtype != torch.float32:
            self.flat_master = torch.zeros(self.total, device=self.device, dtype=master_dtype)
        with torch.no_grad():
            for seg in self.segments:
                view = self.flat_param[seg.offset : seg.offset + seg.numel].view(seg.shape)
                view.copy_(seg.param.data)
                seg.param.data = view
                seg.param.main_grad = self.flat_grad[seg.offset : seg.offset + seg.numel].view(seg.shape)
            if self.flat_master is not None:
                self.flat_master.copy_(self.flat_param)

    # ------------------------------------------------------------------ views
    def param_view(self, seg: Segment) -> torch.Tensor:
        return self.flat_param[seg.offset : seg.offset + seg.numel].view(seg.shape)

    def master(self) -> torch.Tensor:
        return self.flat_master if self.flat_master is not None else self.flat_param

    def master_view(self, seg: Segment) -> torch.Tensor:
        return self.master()[seg.offset : seg.offset + seg.numel].view(seg.shape)

    def grad_view(self, seg: Segment) -> torch.Tensor:
        return self.flat_grad[seg.offset : seg.offset + seg.numel].view(seg.shape)

    def group_stack(self, buf: torch.Tensor, g: MuonGroup) -> torch.Tensor:
        """[count, m, n] view of a flat buffer over a Muon shape group (segments are contiguous)."""
        m, n = g.shape
        return buf[g.offset : g.offset + g.count * m * n].view(g.count, m, n)

    # ------------------------------------------------------------------ gradient plumbing
    @torch.no_grad()
    def fold_autograd_grads(self, only: Optional[Sequence[Segment]] = None) -> None:
        for seg in (self.segments if only is None else only):
            g = seg.param.grad
            if g is not None:
                seg.param.main_grad.add_(g.to(torch.float32))
                seg.param.grad = None

    def zero_grad(self) -> None:
        self.flat_grad.zero_()
        for seg in self.segments:
            seg.param.grad = None

    @torch.no_grad()
    def sync_master_from_params(self) -> None:
        if self.flat_master is not None:
            self.flat_master.copy_(self.flat_param)

    @torch.no_grad()
    def rebind(self) -> None:
        """Re-attach parameter storage to the flat buffers (after ``model.to(...)`` or a state-dict load that
        replaced ``.data``)."""
        for seg in self.segments:
            view = self.param_view(seg)
            if seg.param.data.data_ptr() != view.data_ptr():
                view.copy_(seg.param.data.to(view.dtype))
                seg.param.data = view
            seg.param.main_grad = self.grad_view(seg)
