"""Mixture-of-experts FFN with shared expert and auxiliary-loss-free load balancing.

Parity: ``MoE_FFN`` of the reference (``triune/model/moe.py:38-599``): router ``Linear(d,E)`` with bias,
``expert_bias`` buffer steering only the top-k SELECTION (mixing weights come from the unbiased softmax and
are renormalised over the k picks), experts ``Linear -> GELU(tanh) -> Linear`` with biases, optional shared
expert scaled by 0.5, training temperature ``max(0.1, 1 - step/5000)``, training capacity
``ceil(N/E * 1.5)`` per (k-slot, expert) with highest-weight-first admission, centroid / load EMAs and a
pending bias update applied by ``step_bias()``.

Design differences: ``top_k`` and ``expert_hidden`` are constructor arguments; expert weights are stored
stacked (``w1 [E,H,d]``, ``b1 [E,H]``, ``w2 [E,d,H]``, ``b2 [E,d]``) so one grouped tcgen05 GEMM serves all
experts, and are converted to the reference's per-expert keys (``experts.{e}.{0,2}.{weight,bias}``) only in
state dicts. Training and evaluation share one sparse path (no dense all-experts evaluation).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config import (
    CENTROID_EMA,
    EXPERT_HIDDEN_MULTIPLIER,
    MOE_BIAS_CLAMP,
    MOE_BIAS_UPDATE_RATE,
    MOE_CAPACITY_MULTIPLIER,
    MOE_TEMPERATURE_STEPS,
    NUM_EXPERTS,
    SHARED_EXPERT,
    SHARED_EXPERT_SCALE,
    TOP_K_EXPERTS,
)
from ..ops import reference as ref


@dataclass
class RoutingResult:
    indices: torch.Tensor
    weights: torch.Tensor
    accepted_mask: torch.Tensor
    requested_counts: torch.Tensor
    accepted_counts: torch.Tensor
    dropped_counts: torch.Tensor


class _ExpertView:
    """``moe.experts[e][0|2]`` access for code written against the per-expert module layout."""

    def __init__(self, owner: "MoE_FFN", e: int):
        self._o, self._e = owner, e

    def __getitem__(self, i):
        o, e = self._o, self._e
        if i == 0:
            return _LinearView(o.w1[e], o.b1[e])
        if i == 2:
            return _LinearView(o.w2[e], o.b2[e])
        raise IndexError(i)

    def __call__(self, x):
        o, e = self._o, self._e
        return F.linear(ref.gelu_tanh(F.linear(x, o.w1[e], o.b1[e])), o.w2[e], o.b2[e])


class _LinearView:
    def __init__(self, w, b):
        self.weight, self.bias = w, b


class _SharedExpert(nn.Sequential):
    def __init__(self, dim, hidden):
        super().__init__(nn.Linear(dim, hidden), nn.GELU(approximate="tanh"), nn.Linear(hidden, dim))

    def forward(self, x):
        if type(self[0]) is nn.Linear and type(self[2]) is nn.Linear:
            return ops.mlp_gelu(x, self[0].weight, self[0].bias, self[2].weight, self[2].bias)
        if getattr(self[0], "fused_gelu", False):  # quantised projections take the activation into their GEMM epilogue
            return self[2](self[0](x, gelu=True))
        return self[2](ops.gelu_tanh(self[0](x)))  # wrapped projections run their own forward


class MoE_FFN(nn.Module):
    def __init__(
        self,
        dim: int,
        num_experts: int = NUM_EXPERTS,
        top_k: int = TOP_K_EXPERTS,
        use_fp4: bool = False,
        use_fp8: bool = False,
        shared_expert: bool = SHARED_EXPERT,
        shared_scale: float = SHARED_EXPERT_SCALE,
        use_sparse_eval: bool = True,
        expert_hidden: Optional[int] = None,
        capacity_multiplier: float = MOE_CAPACITY_MULTIPLIER,
    ):
        super().__init__()
        if not (1 <= top_k <= num_experts):
            raise ValueError(f"need 1 <= top_k <= num_experts, got {top_k}, {num_experts}")
        self.dim, self.num_experts, self.top_k = dim, num_experts, top_k
        self.use_fp4, self.use_fp8 = use_fp4, use_fp8
        self.shared_expert, self.shared_scale = shared_expert, shared_scale
        self.use_sparse_eval = use_sparse_eval
        self.capacity_multiplier = capacity_multiplier
        self.centroid_ema = CENTROID_EMA
        hidden = int(expert_hidden) if expert_hidden else dim * EXPERT_HIDDEN_MULTIPLIER
        self.expert_hidden = hidden
        E = num_experts
        self.w1 = nn.Parameter(torch.empty(E, hidden, dim))
        self.b1 = nn.Parameter(torch.zeros(E, hidden))
        self.w2 = nn.Parameter(torch.empty(E, dim, hidden))
        self.b2 = nn.Parameter(torch.zeros(E, dim))
        nn.init.normal_(self.w1, std=0.02)
        nn.init.normal_(self.w2, std=0.02)
        self.shared = _SharedExpert(dim, hidden) if shared_expert else None
        self.router = nn.Linear(dim, E)
        self.register_buffer("expert_bias", torch.zeros(E))
        self.register_buffer("expert_load_ratio", torch.ones(E))
        self.register_buffer("last_centroids", torch.zeros(E, dim))
        self.register_buffer("_overflow_counter", torch.tensor(0, dtype=torch.long), persistent=False)
        self.register_buffer("_global_step", torch.tensor(0, dtype=torch.long))
        self.last_counts = self.last_requested_counts = self.last_accepted_counts = None
        self.last_dropped_counts = None
        self.last_target = None
        self._pending_bias_update = None
        self._register_state_dict_hook(self._split_on_save)
        self._register_load_state_dict_pre_hook(self._stack_on_load)

    # --- reference-compatible checkpoint keys -----------------------------------------------
    @staticmethod
    def _split_on_save(module, sd, prefix, local_metadata):
        w1, b1 = sd.pop(prefix + "w1"), sd.pop(prefix + "b1")
        w2, b2 = sd.pop(prefix + "w2"), sd.pop(prefix + "b2")
        for e in range(module.num_experts):
            sd[f"{prefix}experts.{e}.0.weight"] = w1[e]
            sd[f"{prefix}experts.{e}.0.bias"] = b1[e]
            sd[f"{prefix}experts.{e}.2.weight"] = w2[e]
            sd[f"{prefix}experts.{e}.2.bias"] = b2[e]
        return sd

    def _stack_on_load(self, sd, prefix, *args):
        if f"{prefix}experts.0.0.weight" not in sd:
            return
        E = self.num_experts
        sd[prefix + "w1"] = torch.stack([sd.pop(f"{prefix}experts.{e}.0.weight") for e in range(E)])
        sd[prefix + "b1"] = torch.stack([sd.pop(f"{prefix}experts.{e}.0.bias") for e in range(E)])
        sd[prefix + "w2"] = torch.stack([sd.pop(f"{prefix}experts.{e}.2.weight") for e in range(E)])
        sd[prefix + "b2"] = torch.stack([sd.pop(f"{prefix}experts.{e}.2.bias") for e in range(E)])

    @property
    def experts(self):
        return [_ExpertView(self, e) for e in range(self.num_experts)]

    @property
    def overflow_counter(self) -> int:
        return int(self._overflow_counter.item())

    # --- routing ----------------------------------------------------------------------------
    def _temperature(self):
        if self.training:
            return (1.0 - self._global_step.float() / MOE_TEMPERATURE_STEPS).clamp(min=0.1)
        return 1.0

    def route(self, x2: torch.Tensor):
        """Returns (idx [N,k], weights [N,k] fp32 with grad, keep [N,k] bool or None)."""
        logits = ops.linear(x2, self.router.weight, self.router.bias).float()
        idx, w, _ = ops.moe_route(logits, self.expert_bias, self.top_k, self._temperature())
        keep = None
        if self.training:
            N = x2.shape[0]
            cap = max(1, min(int(math.ceil(N / self.num_experts * self.capacity_multiplier)), N))
            if cap < N:
                with torch.no_grad():
                    keep = ref.moe_capacity_mask(idx, w.detach(), self.num_experts, cap)
        return idx, w, keep

    def _capacity(self, N: int) -> Optional[int]:
        if not self.training:
            return None
        cap = max(1, min(int(math.ceil(N / self.num_experts * self.capacity_multiplier)), N))
        return cap if cap < N else None

    def sparse_forward(self, x: torch.Tensor) -> torch.Tensor:
        """The routed (top-k, grouped by expert) evaluation without touching the routing statistics: the reference's name
        for it (``triune/model/moe.py:126``); here the forward pass always takes this form."""
        return self.forward(x, update_stats=False)

    def forward(self, x: torch.Tensor, update_stats: bool = True) -> torch.Tensor:
        B, T, D = x.shape
        x2 = x.reshape(B * T, D)
        plan = None
        logits = ops.linear(x2, self.router.weight, self.router.bias).float()
        if ops.route_plan_supported(logits, self.top_k) and x2.dtype == torch.bfloat16:
            # routing, capacity admission and the dispatch plan from one sort and three kernels
            idx, w, keep, plan = ops.moe_route_plan(logits, self.expert_bias, self.top_k, self._temperature(), self._capacity(B * T))
        else:
            idx, w, keep = self.route(x2)
        shared_out = self.shared(x2) if self.shared is not None else None
        wk = w if keep is None else w * keep.to(w.dtype)
        out = ops.moe_experts(x2, idx, wk, keep, self.w1, self.b1, self.w2, self.b2, shared_out, self.shared_scale, plan=plan)
        if self.training and update_stats:
            with torch.no_grad():
                self._update_routing_stats(x2.detach(), idx, w.detach(), keep, plan)
        return out.reshape(B, T, D)

    def dense_forward(self, x: torch.Tensor) -> torch.Tensor:
        """All-experts evaluation (test oracle for the sparse path)."""
        B, T, D = x.shape
        x2 = x.reshape(B * T, D)
        idx, w, _ = self.route(x2)
        gate = torch.zeros(x2.shape[0], self.num_experts, dtype=torch.float32, device=x.device)
        gate.scatter_(1, idx, w.float())
        out = torch.zeros(x2.shape, dtype=torch.float32, device=x.device)
        for e in range(self.num_experts):
            out += gate[:, e : e + 1] * self.experts[e](x2).float()
        if self.shared is not None:
            out += self.shared_scale * self.shared(x2).float()
        return out.to(x.dtype).reshape(B, T, D)

    # --- statistics (no gradient, no host sync) ---------------------------------------------
    @torch.no_grad()
    def _update_routing_stats(self, x2, idx, w, keep, plan=None):
        E, N = self.num_experts, x2.shape[0]
        target = max(1.0, float(N * self.top_k / E))
        flat = idx.reshape(-1)
        if plan is not None and getattr(plan, "slot_counts", None) is not None:
            # the routing and plan kernels already counted: no atomics over N * k indices into E bins
            requested = plan.slot_counts.sum(1, dtype=torch.int64)
            accepted = plan[4] if keep is not None else requested
            acc_mask = keep if keep is not None else torch.ones_like(idx, dtype=torch.bool)
        elif keep is None:
            requested = torch.zeros(E, device=flat.device, dtype=torch.int64).scatter_add_(0, flat, torch.ones_like(flat))
            accepted = requested
            acc_mask = torch.ones_like(idx, dtype=torch.bool)
        else:
            requested = torch.zeros(E, device=flat.device, dtype=torch.int64).scatter_add_(0, flat, torch.ones_like(flat))
            accepted = torch.zeros(E, device=flat.device, dtype=torch.int64).scatter_add_(0, flat, keep.reshape(-1).long())
            acc_mask = keep
        dropped = (requested - accepted).clamp_min(0)
        self._overflow_counter.add_(dropped.sum())
        err = (requested.float() - target) / target
        self._pending_bias_update = -err * MOE_BIAS_UPDATE_RATE
        self.expert_load_ratio.mul_(0.9).add_(accepted.float() / target, alpha=0.1)
        self.last_counts = self.last_requested_counts = requested
        self.last_accepted_counts, self.last_dropped_counts = accepted, dropped
        self.last_target = target
        # centroid EMA: mean of accepted tokens per expert
        mask = torch.zeros(N, E, dtype=x2.dtype, device=x2.device)
        mask.scatter_(1, idx, acc_mask.to(x2.dtype))
        counts = accepted.float().unsqueeze(1) if plan is not None else mask.float().sum(0).unsqueeze(1)
        if x2.is_cuda and x2.dtype == torch.bfloat16 and E % 8 == 0 and not ops._ext.reference_ops_enabled():
            sums = ops.gemm(mask, x2.contiguous(), a_mn=True, b_mn=True, out_dtype=torch.float32)
        else:
            sums = mask.float().t() @ x2.float()
        batch_c = sums / counts.clamp_min(1.0)
        cent = self.last_centroids.float()
        uninit = cent.norm(dim=-1, keepdim=True) < 1e-6
        blended = torch.where(uninit, batch_c, cent * self.centroid_ema + batch_c * (1.0 - self.centroid_ema))
        self.last_centroids.copy_(torch.where(counts > 0, blended, cent).to(self.last_centroids.dtype))

    @torch.no_grad()
    def step_bias(self):
        """Apply the pending selection-bias update (called once per optimizer step)."""
        if self._pending_bias_update is not None:
            self.expert_bias.add_(self._pending_bias_update.to(self.expert_bias.dtype)).clamp_(-MOE_BIAS_CLAMP, MOE_BIAS_CLAMP)
            self._pending_bias_update = None

    @torch.no_grad()
    def update_routing_stats(self, x):
        B, T, D = x.shape
        x2 = x.detach().reshape(B * T, D)
        idx, w, keep = self.route(x2)
        self._update_routing_stats(x2, idx, w, keep)
