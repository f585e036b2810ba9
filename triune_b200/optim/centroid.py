"""CentroidSteerOptimizer: three optimizer tiers behind one ``step()``.

Parity: ``triune/optim/centroid.py:96-1609`` of the reference.

Tier partition (``classify_parameters``), in precedence order:
  1. explicit ``param_roles`` (exact names, fnmatch patterns or parameter objects) override everything;
  2. embeddings / ``exit_head`` / ``final_head`` / ``lm_head`` / tied weights, routers, and tall-skinny
     matrices (max dim >= 1000 and aspect >= 4)                         -> Tier 3, AdamW;
  3. routed expert weight matrices of ``MoE_FFN``                       -> Tier 2, CentroidSteer core;
  4. remaining 2-D matrices                                             -> Tier 1, Muon;
  5. everything 1-D                                                     -> Tier 3.

Tier 2 keeps, per expert matrix W [m,n], two orthonormal bases Q_L [m,r+1], Q_R [n,r+1] refreshed every
``update_gap`` steps from the gradient (Gaussian sketch + three sCholQR2 passes). Slot r holds the steering
axis: the router centroid of the expert (for the second expert layer, its hidden activation) made orthogonal
to Q_R by two Gram-Schmidt passes, and its dual G c on the left. The gradient is projected to the
(r+1)x(r+1) core S = Q_L^T G Q_R, an AdamW step runs on the core (optionally upper-triangular), the steering
row/column is amplified by (1 + steer_scale), and dW = Q_L D Q_R^T is applied with decoupled weight decay.
Optimizer state per expert matrix is therefore O((m+n) r + r^2) instead of O(mn).

Design differences: storage is a :class:`ParamArena` (flat, tier-ordered); expert matrices are already
stacked [E,m,n] so every Tier-2 product is batched over experts with no gather; the Tier-3 update is one
fused kernel over a contiguous range; the global gradient norm and clip coefficient stay on the device.
"""

from __future__ import annotations

import fnmatch
import math
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch

from .. import _ext, config as C
from ..ops import reference as ref
from .arena import MuonGroup, ParamArena, Segment
from .subspace import (batched_qr, batched_subspace_projection, flush_qr_telemetry, new_qr_telemetry, reorthogonalise,
                       two_sided_bases)

_HEAD_KEYS = ("embed", "wte", "wpe", "exit_head", "final_head", "lm_head", "classifier", "output_head", "token_table")


def muon_update_scale(d_out: int, d_in: int, rms_target: Optional[float] = None) -> float:
    s = max(1.0, d_out / d_in) ** 0.5
    return s * rms_target if rms_target else s


def classify_parameters(model: torch.nn.Module, param_roles: Optional[Dict] = None, use_muon: bool = True,
                        aspect_safeguard: bool = True):
    """Returns (tiers {id(p): tier}, mat_views {id(p): (K,m,n)}, steer_meta {id(p): (module, role)})."""
    from ..models.attention import VectorisedGLA
    from ..models.moe import MoE_FFN

    named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
    by_name = dict(named)
    tiers: Dict[int, str] = {}
    mat_views: Dict[int, Tuple[int, int, int]] = {}
    steer_meta: Dict[int, Tuple[torch.nn.Module, str]] = {}
    explicit: Dict[int, str] = {}
    for key, role in (param_roles or {}).items():
        role = str(role).lower().strip()
        if isinstance(key, str):
            if any(ch in key for ch in "*?["):
                hits = [p for n, p in named if fnmatch.fnmatch(n, key)]
                if not hits:
                    raise KeyError(f"param_roles wildcard pattern '{key}' matched zero model parameters.")
            elif key in by_name:
                hits = [by_name[key]]
            else:
                suff = [n for n in by_name if n.endswith("." + key)]
                if len(suff) > 1:
                    raise ValueError(f"param_roles key '{key}' is ambiguous and matches multiple parameters: {suff}.")
                if not suff:
                    raise KeyError(f"param_roles key '{key}' is not an exact parameter name.")
                hits = [by_name[suff[0]]]
            for p in hits:
                explicit[id(p)] = role
        else:
            explicit[id(key)] = role

    embed_ptrs = set()
    router_ids = set()
    for mn, mod in model.named_modules():
        if isinstance(mod, (torch.nn.Embedding, torch.nn.EmbeddingBag)):
            embed_ptrs.add(mod.weight.data_ptr())
        # the expert-sharded layer (parallel.expert_parallel.EPMoE_FFN) holds a slice of the same stacked weights
        is_moe = isinstance(mod, MoE_FFN) or all(hasattr(mod, a) for a in ("w1", "b1", "w2", "b2", "router", "expert_bias"))
        if is_moe:
            router_ids.update(id(p) for p in mod.router.parameters())
            for attr, role in (("w1", "input"), ("w2", "hidden")):
                p = getattr(mod, attr)
                steer_meta[id(p)] = (mod, role)
            router_ids.update((id(mod.b1), id(mod.b2)))  # stacked expert biases are 1-D per expert: Tier 3
        elif mod.__class__.__name__ in ("GumbelSoftmaxRouter", "Router", "TopKRouter") or "router" in mn.lower():
            router_ids.update(id(p) for p in mod.parameters())
        if isinstance(mod, VectorisedGLA):
            mat_views[id(mod.qkvg_weight)] = (4, mod.hidden_dim, mod.dim)

    for n, p in named:
        if id(p) in tiers:
            continue
        if id(p) in explicit:
            r = explicit[id(p)]
            if r in ("muon", "orthogonal") and p.dim() >= 2:
                tiers[id(p)] = "muon"
            elif r in ("expert", "centroid", "subspace") and p.dim() >= 2:
                tiers[id(p)] = "steer"
                steer_meta.setdefault(id(p), (None, "input"))
            else:
                tiers[id(p)] = "adamw"
            continue
        low = n.lower()
        if p.data_ptr() in embed_ptrs or any(k in low for k in _HEAD_KEYS) or id(p) in router_ids:
            tiers[id(p)] = "adamw"
            continue
        if id(p) in steer_meta and p.dim() == 3:
            tiers[id(p)] = "steer"
            continue
        if p.dim() == 2 and use_muon:
            K, m, nn_ = mat_views.get(id(p), (1, p.shape[0], p.shape[1]))
            dmax, dmin = max(m, nn_), min(m, nn_)
            if aspect_safeguard and dmax >= 1000 and dmax / max(dmin, 1) >= 4.0:
                tiers[id(p)] = "adamw"
            else:
                tiers[id(p)] = "muon"
            continue
        tiers[id(p)] = "adamw"
    return tiers, mat_views, steer_meta


class _SyncedParamGroup(dict):
    """Param-group dict whose ``lr`` writes cascade to all tiers (so torch LR schedulers work)."""

    def __init__(self, owner, *a, **kw):
        super().__init__(*a, **kw)
        self._owner = owner

    def __setitem__(self, k, v):
        super().__setitem__(k, v)
        if k == "lr" and getattr(self, "_owner", None) is not None and not self._owner._in_set_lr:
            self._owner.set_lr(float(v))


class CentroidSteerOptimizer(torch.optim.Optimizer):
    def __init__(self, model: torch.nn.Module, lr=1e-4, betas=(0.9, 0.95), weight_decay=0.05, rank=C.GALORE_RANK,
                 update_gap=C.GALORE_UPDATE_GAP, steer_scale=C.STEER_SCALE, steer_update_gap=C.STEER_UPDATE_GAP,
                 expert_lr=None, expert_betas=C.GALORE_BETAS, expert_wd=C.GALORE_WEIGHT_DECAY, use_muon=True,
                 muon_lr: Optional[float] = None, muon_momentum=C.MUON_MOMENTUM, muon_weight_decay=C.MUON_WEIGHT_DECAY,
                 muon_ns_steps=C.NS_STEPS, muon_rms_target: Optional[float] = None, ns_coeffs=C.NS_COEFFS,
                 use_triangular_core=True, core_mask_mode: str = "full", param_roles=None, eps: float = 1e-8,
                 grad_clip: Optional[float] = None, nesterov: bool = True, aspect_safeguard: bool = True,
                 adaptive_subspace_refresh: bool = False, energy_threshold: float = 0.5, min_subspace_gap: int = 5,
                 max_subspace_gap: int = 50, storage_factory=None, shard: Tuple[int, int] = (0, 1),
                 tensor_core_subspace: bool = True, use_8bit_adam: bool = False, only=None):
        if core_mask_mode not in ("full", "triu"):
            raise ValueError(f"Unknown core_mask_mode={core_mask_mode!r}; expected 'full' or 'triu'")
        self._in_set_lr = False
        self.model = model
        tiers, mat_views, steer_meta = classify_parameters(model, param_roles, use_muon, aspect_safeguard)
        self.tiers, self.steer_meta = tiers, steer_meta
        # ``only(name, param) -> bool`` restricts the optimizer to a subset (the root modules of a streamed model,
        # whose layers are updated one at a time elsewhere); tiers are still decided with the whole model in view.
        named = [(n, p) for n, p in model.named_parameters() if only is None or only(n, p)]
        self.arena = ParamArena(named, tiers, mat_views, storage_factory=storage_factory)
        self.shard = (int(shard[0]), int(shard[1]))  # (rank, world): which matrices / experts this rank updates
        group = _SyncedParamGroup(self, {"params": [s.param for s in self.arena.segments], "lr": lr, "betas": betas,
                                         "weight_decay": weight_decay})
        super().__init__([group], dict(lr=lr, betas=betas, weight_decay=weight_decay))
        self.param_groups = [group]
        group._owner = self
        self.lr, self.betas, self.weight_decay, self.eps = lr, betas, weight_decay, eps
        self.rank, self.update_gap = rank, update_gap
        self.steer_scale, self.steer_update_gap = steer_scale, steer_update_gap
        self.expert_lr = lr if expert_lr is None else expert_lr
        self.expert_betas, self.expert_wd = expert_betas, expert_wd
        self.use_muon = use_muon
        self.muon_lr = min(0.02, max(0.001, lr * 2.0)) if muon_lr is None else muon_lr
        self.muon_momentum, self.muon_weight_decay = muon_momentum, muon_weight_decay
        self.muon_ns_steps, self.muon_rms_target, self.ns_coeffs = muon_ns_steps, muon_rms_target, tuple(ns_coeffs)
        self.nesterov = nesterov
        self.use_triangular_core, self.core_mask_mode = use_triangular_core, core_mask_mode
        self.grad_clip = grad_clip
        self.adaptive_subspace_refresh, self.energy_threshold = adaptive_subspace_refresh, energy_threshold
        self.min_subspace_gap, self.max_subspace_gap = min_subspace_gap, max_subspace_gap
        self.initial_base_lr, self.initial_muon_lr, self.initial_expert_lr = lr, self.muon_lr, self.expert_lr
        self.step_count = 0
        self.qr_telemetry = new_qr_telemetry()
        a = self.arena
        dev = a.device
        lo, hi = a.adamw_range
        # Tier-3 moments: fp32, or block-wise 8-bit (``use_8bit_adam``; the reference's optional AdamW8bit tier,
        # ``triune/optim/centroid.py:10-16``) which cuts that tier's optimizer state from 8 to ~2 bytes per parameter.
        self.use_8bit_adam = bool(use_8bit_adam)
        if self.use_8bit_adam:
            from .adam8bit import BlockwiseMoments

            self.moments8 = BlockwiseMoments(hi - lo, dev)
            self.exp_avg = self.exp_avg_sq = torch.zeros(0, device=dev, dtype=torch.float32)
        else:
            self.moments8 = None
            self.exp_avg = torch.zeros(hi - lo, device=dev, dtype=torch.float32)
            self.exp_avg_sq = torch.zeros(hi - lo, device=dev, dtype=torch.float32)
        self._partial_open = False  # a global step made of several step_parameters calls is in progress
        lo, hi = a.muon_range
        self.muon_mom = torch.zeros(hi - lo, device=dev, dtype=torch.float32)
        self.steer_state: Dict[str, Dict] = {}
        self.tensor_core_subspace = bool(tensor_core_subspace)
        self._q16: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = {}  # bf16 copies of the bases (derived, not saved)
        self.capturable = False  # device-resident hyper-parameters (CUDA-graph replay)
        self.hyper = torch.zeros(8, device=dev, dtype=torch.float32)
        self._hyper_host = torch.zeros(8, dtype=torch.float32, pin_memory=(dev.type == "cuda"))
        self._clip_coef = torch.ones(1, device=dev, dtype=torch.float32)
        self._sumsq = torch.zeros(1, device=dev, dtype=torch.float32)
        self.last_grad_norm = None
        # parity attributes
        self.non_expert_params = [s.param for s in a.segments if s.tier == "adamw"]
        self.muon_params = [s.param for s in a.segments if s.tier == "muon"]
        self.layer_groups = [s for s in a.segments if s.tier == "steer"]

    # ------------------------------------------------------------------ ownership (sharded data parallel)
    def _owned(self, count: int) -> Tuple[int, int]:
        r, w = self.shard
        return (count * r) // w, (count * (r + 1)) // w

    def owned_adamw_range(self) -> Tuple[int, int]:
        lo, hi = self.arena.adamw_range
        r, w = self.shard
        per = -(-((hi - lo) // w) // 128) * 128 if w > 1 else hi - lo
        b = min(hi, lo + r * per)
        e = hi if r == w - 1 else min(hi, lo + (r + 1) * per)
        return b, e

    def owned_matrix_ranges(self):
        """Flat element ranges of the Muon matrices and experts this rank updates."""
        out = []
        for g in self.arena.muon_groups:
            m, n = g.shape
            k0, k1 = self._owned(g.count)
            if k1 > k0:
                out.append((g.offset + k0 * m * n, g.offset + k1 * m * n))
        for seg in self.arena.segments:
            if seg.tier == "steer":
                K, m, n = seg.mat_shape
                k0, k1 = self._owned(K)
                if k1 > k0:
                    out.append((seg.offset + k0 * m * n, seg.offset + k1 * m * n))
        return out

    # ------------------------------------------------------------------ learning rates
    def sync_lr_from_param_groups(self) -> None:
        """An outer PyTorch scheduler writes ``param_groups[0]["lr"]``; carry a change over to the tiers (Muon and expert
        rates keep their ratios to the base rate)."""
        if self.param_groups:
            outer = self.param_groups[0].get("lr", self.lr)
            if outer != self.lr:
                self.set_lr(float(outer))

    def set_lr(self, lr: float, expert_lr: Optional[float] = None, muon_lr: Optional[float] = None):
        """Set the base LR; Muon and expert LRs keep their initial ratio to it unless given explicitly."""
        self._in_set_lr = True
        try:
            ratio = lr / self.initial_base_lr if self.initial_base_lr > 0 else 1.0
            self.lr = lr
            self.muon_lr = self.initial_muon_lr * ratio if muon_lr is None else muon_lr
            self.expert_lr = self.initial_expert_lr * ratio if expert_lr is None else expert_lr
            for g in self.param_groups:
                g["lr"] = lr
        finally:
            self._in_set_lr = False

    # ------------------------------------------------------------------ CUDA-graph support
    def _hyper_arg(self):
        return self.hyper if self.capturable else None

    def _subspace_step_next(self) -> int:
        for st in self.steer_state.values():
            if "subspace_step" in st:
                return int(st["subspace_step"]) + 1
        return 1

    def write_hyper(self, step_count: Optional[int] = None) -> None:
        """Publish the hyper-parameters of the NEXT step to the device (one small async copy)."""
        t = (self.step_count + 1) if step_count is None else step_count
        b1, b2 = self.betas
        e1, e2 = self.expert_betas
        ts = self._subspace_step_next()
        h = self._hyper_host
        h[0], h[1], h[2] = self.lr, 1 - b1**t, 1 - b2**t
        h[3], h[4] = self.muon_lr, self.expert_lr
        h[5], h[6] = 1 - e1**ts, 1 - e2**ts
        h[7] = 1 - self.expert_lr * self.expert_wd
        self.hyper.copy_(h, non_blocking=True)

    def step_kind(self) -> str:
        """What the NEXT step will do in the CentroidSteer tier: 'refresh' (new bases; needs host decisions),
        'steer' (steering axis refresh) or 'plain'. Used to pick a captured graph or the eager path."""
        nxt = self.step_count + 1
        kind = "plain"
        for seg in self.arena.segments:
            if seg.tier != "steer" or not self.use_triangular_core:
                continue
            st = self.steer_state.get(seg.name)
            if st is None or st["proj_step"] is None or self.adaptive_subspace_refresh:
                return "refresh"
            if nxt - st["proj_step"] >= self.update_gap:
                return "refresh"
            if st["last_steer_step"] is None or nxt - st["last_steer_step"] >= self.steer_update_gap:
                kind = "steer"
        return kind

    def advance_counters(self, kind: str) -> None:
        """Host-side bookkeeping for a step that ran as a graph replay."""
        self.step_count += 1
        for seg in self.arena.segments:
            st = self.steer_state.get(seg.name)
            if st is None or "subspace_step" not in st:
                continue
            st["step"] += 1
            st["subspace_step"] += 1
            if kind == "steer":
                st["last_steer_step"] = self.step_count

    def zero_grad(self, set_to_none: bool = True):
        self.arena.zero_grad()

    # ------------------------------------------------------------------ step
    def _use_kernels(self) -> bool:
        return self.arena.device.type == "cuda" and not _ext.reference_ops_enabled() and _ext.use_kernels(self.arena.flat_grad)

    @torch.no_grad()
    def compute_clip(self):
        """Global grad-norm and clip coefficient, device-resident (no host sync)."""
        a = self.arena
        if self._use_kernels():
            self._sumsq.zero_()
            _ext.ext().sumsq(a.flat_grad, self._sumsq)
            norm = self._sumsq.sqrt()
        else:
            norm = a.flat_grad.norm().reshape(1)
        self.last_grad_norm = norm
        if self.grad_clip is not None and self.grad_clip > 0:
            self._clip_coef.copy_((self.grad_clip / (norm + 1e-6)).clamp(max=1.0))
        else:
            self._clip_coef.fill_(1.0)
        return norm

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        a = self.arena
        a.fold_autograd_grads()
        self.step_count += 1
        self.compute_clip()
        self._step_adamw()
        self._step_muon()
        self._step_steer_tf32()
        return loss

    def _step_steer_tf32(self, only=None):
        # the subspace projections are fp32 batched products; TF32 tensor cores keep ~1e-3 relative accuracy,
        # the same order as the bf16 bases the reference uses on CUDA
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        try:
            self._step_steer(only)
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev

    def set_clip_coefficient(self, coef) -> None:
        """Gradient scale applied by the next (partial) steps. Layer-wise stepping cannot know the global gradient norm
        when the first layer is updated, so the caller computes it over all layers first and passes
        ``min(1, clip / norm)`` here."""
        if torch.is_tensor(coef):
            self._clip_coef.copy_(coef.reshape(1).to(self._clip_coef))
        else:
            self._clip_coef.fill_(float(coef))

    @torch.no_grad()
    def step_parameters(self, params: Iterable[torch.nn.Parameter], is_global_step_end: bool = False):
        """Update only ``params`` (one layer, or the root modules) with their tiers' rules; several calls make up one
        global step, the last one passing ``is_global_step_end=True`` (``triune/optim/centroid.py:531`` of the
        reference). All calls of one global step share the same step number (bias corrections, refresh schedule) and
        the clip coefficient set by :meth:`set_clip_coefficient` (1 by default); every other parameter, and its
        optimizer state, is left untouched, which is what lets layer streaming keep only one layer's state on the
        device."""
        if self.shard[1] != 1:
            raise RuntimeError("step_parameters updates whole parameters: use it without optimizer-state sharding")
        ids = {id(p) for p in params}
        a = self.arena
        segs = [s for s in a.segments if id(s.param) in ids]
        if not self._partial_open:
            self.step_count += 1
            self._partial_open = True
        a.fold_autograd_grads(segs)
        if segs:
            self._step_adamw([s for s in segs if s.tier == "adamw"])
            self._step_muon({id(s.param) for s in segs if s.tier == "muon"})
            steer = {s.name for s in segs if s.tier == "steer"}
            if steer:
                self._step_steer_tf32(steer)
        if is_global_step_end:
            self._partial_open = False

    # ---- Tier 3 --------------------------------------------------------------------------------
    def _step_adamw(self, only: Optional[List[Segment]] = None):
        """AdamW over the whole Tier-3 range, or (``only``) over the element ranges of the given segments."""
        a = self.arena
        lo, hi = a.adamw_range
        if hi == lo:
            return
        if only is None:
            runs = [(lo, hi)]
        else:
            runs = []
            for seg in sorted(only, key=lambda s_: s_.offset):
                b, e = seg.offset, seg.offset + seg.numel
                if runs and b - runs[-1][1] < 8:  # neighbours (the padding between segments is < 8 elements)
                    runs[-1] = (runs[-1][0], e)
                else:
                    runs.append((b, e))
        for b, e in runs:
            self._adamw_range(b, e)

    def _adamw_range(self, b: int, e: int):
        a = self.arena
        lo, _ = a.adamw_range
        b1, b2 = self.betas
        t = self.step_count
        master = a.master()[b:e]
        grad = a.flat_grad[b:e]
        if self.moments8 is not None:
            g = grad * self._clip_coef
            m, v = self.moments8.load(b - lo, e - lo)
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            upd = (m / (1 - b1**t)) / ((v / (1 - b2**t)).sqrt() + self.eps)
            master.mul_(1 - self.lr * self.weight_decay).add_(upd, alpha=-self.lr)
            self.moments8.store(b - lo, e - lo, m, v)
            if a.flat_master is not None:
                a.flat_param[b:e].copy_(master)
            return
        ea, es = self.exp_avg[b - lo : e - lo], self.exp_avg_sq[b - lo : e - lo]
        if self._use_kernels():
            pb = a.flat_param[b:e] if a.flat_master is not None else None
            _ext.ext().adamw_flat(master, ea, es, grad, pb, self.lr, b1, b2, self.eps,
                                  self.weight_decay, t, self._clip_coef, 1.0, self._hyper_arg())
            from .. import ops
            ops._tick()
            return
        g = grad * self._clip_coef
        ea.mul_(b1).add_(g, alpha=1 - b1)
        es.mul_(b2).addcmul_(g, g, value=1 - b2)
        mh = ea / (1 - b1**t)
        vh = es / (1 - b2**t)
        master.mul_(1 - self.lr * self.weight_decay).add_(mh / (vh.sqrt() + self.eps), alpha=-self.lr)
        if a.flat_master is not None:
            a.flat_param[b:e].copy_(master)

    # ---- Tier 1 --------------------------------------------------------------------------------
    def _muon_runs(self, grp: MuonGroup, only):
        """Index ranges [k0, k1) of the group's matrix stack to update: the owned share, or (``only``: a set of
        parameter ids) the runs of consecutive matrices that belong to the selected parameters."""
        if only is None:
            k0, k1 = self._owned(grp.count)
            return [(k0, k1)] if k1 > k0 else []
        runs, k = [], 0
        for seg in grp.segments:
            K = seg.mat_shape[0]
            if id(seg.param) in only:
                if runs and runs[-1][1] == k:
                    runs[-1] = (runs[-1][0], k + K)
                else:
                    runs.append((k, k + K))
            k += K
        return runs

    def _step_muon(self, only=None):
        a = self.arena
        lo, hi = a.muon_range
        if hi == lo:
            return
        from .. import ops

        beta = self.muon_momentum
        kern = self._use_kernels()
        for grp, (k0, k1) in ((g_, r_) for g_ in a.muon_groups for r_ in self._muon_runs(g_, only)):
            m, n = grp.shape
            s, e = grp.offset + k0 * m * n, grp.offset + k1 * m * n
            grad = a.flat_grad[s:e]
            mom = self.muon_mom[s - lo : e - lo]
            if kern:
                u = torch.empty(e - s, device=a.device, dtype=torch.bfloat16)
                _ext.ext().muon_momentum(mom, grad, u, beta, self.nesterov, self._clip_coef)
                ops._tick()
            else:
                g = grad * self._clip_coef
                mom.lerp_(g, 1 - beta)
                u = torch.lerp(g, mom, beta) if self.nesterov else mom.clone()
            O = ops.muon_ns(u.view(k1 - k0, m, n), steps=self.muon_ns_steps, coeffs=self.ns_coeffs)
            scale = muon_update_scale(m, n, self.muon_rms_target)
            master = a.master()[s:e]
            if kern:
                pb = a.flat_param[s:e] if a.flat_master is not None else None
                _ext.ext().muon_apply(master, O.reshape(-1).contiguous(), pb, self.muon_lr, self.muon_weight_decay, scale, self._hyper_arg())
                ops._tick()
            else:
                master.mul_(1 - self.muon_lr * self.muon_weight_decay).add_(O.reshape(-1).float(), alpha=-self.muon_lr * scale)
                if a.flat_master is not None:
                    a.flat_param[s:e].copy_(master)

    # ---- Tier 2 --------------------------------------------------------------------------------
    def _centroid_inputs(self, seg: Segment) -> Optional[torch.Tensor]:
        mod, role = self.steer_meta.get(id(seg.param), (None, "input"))
        if mod is None or getattr(mod, "last_centroids", None) is None or self.steer_scale <= 0:
            return None
        c = mod.last_centroids.float()  # [E, d]
        if role == "hidden":
            c = ref.gelu_tanh(torch.baddbmm(mod.b1.float().unsqueeze(1), c.unsqueeze(1), mod.w1.float().transpose(1, 2))).squeeze(1)
        return c

    def _step_galore(self, seg: Segment, G: torch.Tensor, k0: int, k1: int):
        """Single-sided low-rank path (``use_triangular_core=False``; ``triune/optim/centroid.py:984-1268``): one basis
        P [dim, r] on the shorter side of the matrix, Adam moments in the projected space ([r+1, n] or [m, r+1]), a
        refresh every ``update_gap`` steps from a randomized range finder with the moments TRANSPORTED into the new
        basis through T = P_old^T P_new (first moment by T, second moment by T*T plus the energy that left the span
        replaced by the mean variance), and the steering axis in slot r: the unit residual of the expert's router
        centroid, applied on reconstruction with weight steer_scale * utilisation * residual norm."""
        a = self.arena
        b1, b2 = self.expert_betas
        K, m, n = G.shape
        left = m <= n
        dim = m if left else n
        r = max(1, min(self.rank, m, n))
        st = self.steer_state.get(seg.name)
        if st is None:
            P0 = torch.empty(K, dim, r, device=a.device)
            for i in range(K):
                torch.nn.init.orthogonal_(P0[i])
            st = self.steer_state[seg.name] = {
                "mode": "galore", "side": "left" if left else "right", "P": torch.zeros(K, dim, r + 1, device=a.device),
                "m": None, "v": None, "step": 0, "proj_step": self.step_count, "rank": r,
                "last_c": torch.zeros(K, dim, device=a.device), "steer_w": torch.zeros(K, device=a.device),
            }
            st["P"][:, :, :r] = P0
        if self.step_count - st["proj_step"] >= self.update_gap:
            Gs = G if left else G.transpose(1, 2)
            P_new = batched_subspace_projection(Gs.contiguous(), r)            # [K, dim, r]
            if P_new.shape[-1] == r and st["m"] is not None:
                T = st["P"][:, :, :r].transpose(1, 2) @ P_new                  # [K, r, r]
                T2 = T * T
                energy = T2.sum(dim=1).clamp(0.0, 1.0)                         # column sums: energy kept per new axis
                M, V = st["m"], st["v"]
                if left:
                    Mr = T.transpose(1, 2) @ M[:, :r]
                    Vr = T2.transpose(1, 2) @ V[:, :r] + (1.0 - energy).unsqueeze(-1) * V[:, :r].mean(dim=1, keepdim=True)
                    st["m"], st["v"] = torch.cat((Mr, M[:, r:]), dim=1), torch.cat((Vr, V[:, r:]), dim=1)
                else:
                    Mr = M[:, :, :r] @ T
                    Vr = V[:, :, :r] @ T2 + (1.0 - energy).unsqueeze(1) * V[:, :, :r].mean(dim=2, keepdim=True)
                    st["m"], st["v"] = torch.cat((Mr, M[:, :, r:]), dim=2), torch.cat((Vr, V[:, :, r:]), dim=2)
            else:
                st["m"] = st["v"] = None
                st["step"] = 0
            st["P"][:, :, : P_new.shape[-1]] = P_new
            st["proj_step"] = self.step_count
        # steering axis
        P = st["P"]
        P[:, :, r].zero_()
        st["steer_w"].zero_()
        c = self._centroid_inputs(seg)
        mod, role = self.steer_meta.get(id(seg.param), (None, "input"))
        if c is not None and (left and role == "hidden" or not left and role == "input" or c.shape[-1] == dim):
            c = c[k0:k1]
            if c.shape == (K, dim):
                cn = c.norm(dim=-1, keepdim=True)
                c_hat = c / cn.clamp_min(1e-8)
                res = c_hat - (P[:, :, :r] @ (P[:, :, :r].transpose(1, 2) @ c_hat.unsqueeze(-1))).squeeze(-1)
                rn = res.norm(dim=-1)
                ok = (cn.squeeze(-1) > 1e-8) & (rn > 1e-8)
                c_orth = res / rn.clamp_min(1e-8).unsqueeze(-1)
                flip = ((c_orth * st["last_c"]).sum(-1) < 0) & (st["last_c"].abs().sum(-1) > 0)  # sign continuity
                c_orth = torch.where(flip.unsqueeze(-1), -c_orth, c_orth)
                util = torch.ones(K, device=a.device)
                if mod is not None and getattr(mod, "expert_load_ratio", None) is not None:
                    util = (1.0 + (1.0 - mod.expert_load_ratio.float()[k0:k1])).clamp(0.3, 2.0)
                P[:, :, r] = torch.where(ok.unsqueeze(-1), c_orth, torch.zeros_like(c_orth))
                st["last_c"] = torch.where(ok.unsqueeze(-1), c_orth, torch.zeros_like(c_orth))
                st["steer_w"] = torch.where(ok, self.steer_scale * util * rn.clamp(0.0, 1.0), torch.zeros_like(rn))
        g_lr = P.transpose(1, 2) @ G if left else G @ P                        # [K, r+1, n] or [K, m, r+1]
        st["step"] += 1
        if st["m"] is None:
            st["m"], st["v"] = g_lr.clone(), g_lr * g_lr
        else:
            st["m"].mul_(b1).add_(g_lr, alpha=1 - b1)
            st["v"].mul_(b2).addcmul_(g_lr, g_lr, value=1 - b2)
        t = st["step"]
        d_lr = (st["m"] / (1 - b1**t)) / ((st["v"] / max(1 - b2**t, 1e-7)).sqrt() + self.eps)
        P_rec = P.clone()
        P_rec[:, :, r] = P_rec[:, :, r] * st["steer_w"].unsqueeze(-1)
        dW = P_rec @ d_lr if left else d_lr @ P_rec.transpose(1, 2)
        self._apply_steer_delta(seg, dW, k0, k1)

    def _step_steer(self, only=None):
        a = self.arena
        b1, b2 = self.expert_betas
        for seg in a.segments:
            if seg.tier != "steer" or (only is not None and seg.name not in only):
                continue
            K_all, m, n = seg.mat_shape
            k0, k1 = self._owned(K_all)
            if k1 == k0:
                continue
            K = k1 - k0
            G = a.grad_view(seg).view(K_all, m, n)[k0:k1] * self._clip_coef
            r = max(1, min(self.rank, min(m, n) - 1))
            st = self.steer_state.get(seg.name)
            if not self.use_triangular_core:
                self._step_galore(seg, G, k0, k1)
                continue
            if st is None:
                st = self.steer_state[seg.name] = {
                    "Q_L": torch.zeros(K, m, r + 1, device=a.device), "Q_R": torch.zeros(K, n, r + 1, device=a.device),
                    "m": torch.zeros(K, r + 1, r + 1, device=a.device), "v": torch.zeros(K, r + 1, r + 1, device=a.device),
                    "step": 0, "subspace_step": 0, "proj_step": None, "last_steer_step": None, "rank": r,
                    "steer_applied": torch.zeros(K, dtype=torch.bool, device=a.device),
                    "has_grad": torch.zeros(K, dtype=torch.bool, device=a.device), "last_energy_ratio": None,
                }
            gap = self.update_gap
            if self.adaptive_subspace_refresh and st["last_energy_ratio"] is not None and st["proj_step"] is not None:
                since = self.step_count - st["proj_step"]
                low = bool((st["last_energy_ratio"] < self.energy_threshold).any())
                gap = self.min_subspace_gap if low else self.max_subspace_gap
                refresh = since >= gap
            else:
                refresh = st["proj_step"] is None or (self.step_count - st["proj_step"]) >= gap
            if refresh:
                nz = G.flatten(1).abs().amax(-1) > 0  # experts that received tokens
                st["has_grad"] = nz
                if bool(nz.any()):
                    idx = nz.nonzero(as_tuple=True)[0]
                    QL, QR = two_sided_bases(G[idx], r, telemetry=self.qr_telemetry)
                    st["Q_L"][idx, :, :r] = QL
                    st["Q_R"][idx, :, :r] = QR
                if st["proj_step"] is None and bool((~nz).any()):
                    idz = (~nz).nonzero(as_tuple=True)[0]
                    eye_l = torch.eye(m, r, device=a.device)
                    eye_r = torch.eye(n, r, device=a.device)
                    st["Q_L"][idz, :, :r] = eye_l
                    st["Q_R"][idz, :, :r] = eye_r
                st["m"].zero_()
                st["v"].zero_()
                st["subspace_step"] = 0
                st["proj_step"] = self.step_count
            need_steer = refresh or st["last_steer_step"] is None or (
                self.step_count - st["last_steer_step"]) >= self.steer_update_gap
            if need_steer:
                st["m"][:, :, r].zero_()
                st["m"][:, r, :].zero_()
                st["v"][:, :, r].zero_()
                st["v"][:, r, :].zero_()
                c = self._centroid_inputs(seg)
                c = c[k0:k1] if c is not None else None
                if c is not None and c.shape == (K, n):
                    v_orth, vn = reorthogonalise(c, st["Q_R"][:, :, :r])
                    u = (G @ v_orth.unsqueeze(-1)).squeeze(-1)
                    u_orth, un = reorthogonalise(u, st["Q_L"][:, :, :r])
                    ok = (vn > 1e-8) & (un > 1e-8)
                    st["Q_L"][:, :, r] = torch.where(ok[:, None], u_orth, torch.zeros_like(u_orth))
                    st["Q_R"][:, :, r] = torch.where(ok[:, None], v_orth, torch.zeros_like(v_orth))
                    st["steer_applied"] = ok & st["has_grad"]
                else:
                    st["Q_L"][:, :, r].zero_()
                    st["Q_R"][:, :, r].zero_()
                    st["steer_applied"].zero_()
                st["last_steer_step"] = self.step_count
            QL, QR = st["Q_L"], st["Q_R"]
            tc = self._tensor_core_products(m, n)
            if tc:
                if seg.name not in self._q16:
                    self._q16[seg.name] = (self._padded_bf16(QL), self._padded_bf16(QR))
                elif refresh or need_steer:  # in place: a captured step keeps reading the same buffers
                    self._q16[seg.name][0][:, :, : r + 1].copy_(QL)
                    self._q16[seg.name][1][:, :, : r + 1].copy_(QR)
                QL16, QR16 = self._q16[seg.name]
                S = self._project_tc(G, QL16, QR16, r + 1)
            else:
                S = QL.transpose(1, 2) @ (G @ QR)
            if self.adaptive_subspace_refresh:
                st["last_energy_ratio"] = S[:, :r, :r].pow(2).sum((-2, -1)) / G.pow(2).sum((-2, -1)).clamp_min(1e-12)
            st["step"] += 1
            st["subspace_step"] += 1
            triu = self.core_mask_mode == "triu"
            if self._use_kernels():
                delta = _ext.ext().triangular_adamw(S.contiguous(), st["m"], st["v"], b1, b2, self.eps, st["subspace_step"], triu, self._hyper_arg())
                from .. import ops
                ops._tick()
            else:
                delta = ref.triangular_adamw_core(S, st["m"], st["v"], st["subspace_step"], 1.0, b1, b2, self.eps, triu)
            if self.steer_scale > 0:
                mult = torch.where(st["steer_applied"], 1.0 + self.steer_scale, 1.0)[:, None]
                delta[:, :, r] = delta[:, :, r] * mult
                if not triu:
                    delta[:, r, :r] = delta[:, r, :r] * mult
            dW = self._reconstruct_tc(delta, QL16, QR16) if tc else QL @ delta @ QR.transpose(1, 2)
            self._apply_steer_delta(seg, dW, k0, k1)

    # ------------------------------------------------------------------ subspace products on the tensor cores
    # The two per-step products of the subspace tier, S = Q_L^T G Q_R and dW = Q_L delta Q_R^T, are skinny batched
    # GEMMs (rank + 1 = 257 columns against thousands of rows). As fp32 library products they were a fifth of the
    # step of the default preset; with bf16 operands and fp32 accumulation they run on the tcgen05 GEMM. The bases are
    # kept as bf16 copies padded to a multiple of 8 columns (zero columns add nothing); they change only when the
    # subspace is refreshed or the steering column is rewritten.
    def _tensor_core_products(self, m: int, n: int) -> bool:
        return bool(self._use_kernels() and self.tensor_core_subspace and m % 8 == 0 and n % 8 == 0 and m >= 128 and n >= 128)

    @staticmethod
    def _padded_bf16(Q: torch.Tensor) -> torch.Tensor:
        K, d, r1 = Q.shape
        r1p = (r1 + 7) // 8 * 8
        out = torch.zeros(K, d, r1p, device=Q.device, dtype=torch.bfloat16)
        out[:, :, :r1] = Q
        return out

    @staticmethod
    def _project_tc(G: torch.Tensor, QL16: torch.Tensor, QR16: torch.Tensor, r1: int) -> torch.Tensor:
        from .. import ops

        G16 = G.to(torch.bfloat16)
        GQ = ops.gemm(G16, QR16, b_mn=True)                                       # [K, m, r1p] = G Q_R
        S = ops.gemm(QL16, GQ, a_mn=True, b_mn=True, out_dtype=torch.float32)     # [K, r1p, r1p] = Q_L^T (G Q_R)
        return S[:, :r1, :r1].contiguous()

    @staticmethod
    def _reconstruct_tc(delta: torch.Tensor, QL16: torch.Tensor, QR16: torch.Tensor) -> torch.Tensor:
        from .. import ops

        K, r1, _ = delta.shape
        r1p = QL16.shape[-1]
        d16 = torch.zeros(K, r1p, r1p, device=delta.device, dtype=torch.bfloat16)
        d16[:, :r1, :r1] = delta
        T = ops.gemm(QL16, d16, b_mn=True)                                        # [K, m, r1p] = Q_L delta
        return ops.gemm(T, QR16, out_dtype=torch.float32)                          # [K, m, n] = (Q_L delta) Q_R^T

    def _apply_steer_delta(self, seg: Segment, dW: torch.Tensor, k0: int, k1: int):
        a = self.arena
        master = a.master_view(seg)[k0:k1]
        if self.capturable:
            master.mul_(self.hyper[7]).sub_(dW.to(master.dtype) * self.hyper[4])
        else:
            master.mul_(1 - self.expert_lr * self.expert_wd).add_(dW.to(master.dtype), alpha=-self.expert_lr)
        if a.flat_master is not None:
            a.param_view(seg)[k0:k1].copy_(master)

    # ------------------------------------------------------------------ state dict / telemetry
    def state_dict(self):
        flush_qr_telemetry(self.qr_telemetry)
        return {
            "step_count": self.step_count, "lr": self.lr, "muon_lr": self.muon_lr, "expert_lr": self.expert_lr,
            "steer_scale": float(self.steer_scale),
            "layout": [[s.name, s.tier, s.offset, s.numel] for s in self.arena.segments],
            "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq, "muon_momentum": self.muon_mom,
            "moments8": self.moments8.state_dict() if self.moments8 is not None else None,
            "master": self.arena.flat_master,
            "steer": {k: {kk: vv for kk, vv in v.items()} for k, v in self.steer_state.items()},
            "qr_telemetry": self.qr_telemetry,
        }

    # ---- the reference's optimizer-state layout ------------------------------------------------------------------
    def reference_state_dict(self) -> Dict:
        """Optimizer state in the layout of the reference's ``CentroidSteerOptimizer.state_dict``
        (``triune/optim/centroid.py:1286-1311``): ``base_optimizer`` / ``muon_optimizer`` as torch-optimizer state
        dicts over per-parameter tensors, and one ``layer_groups`` entry per EXPERT matrix (the stacked expert weights
        are unstacked: ``w1`` of all experts first, then ``w2``, per layer) carrying Q_L / Q_R, the core moments under
        ``state`` (``momentum``, ``variance``, ``step``, ``subspace_step``) and the refresh bookkeeping. Tools written
        against the reference's checkpoints can read it; :meth:`load_reference_state_dict` is the inverse."""
        a = self.arena
        lo_a, _ = a.adamw_range
        lo_m, _ = a.muon_range
        if self.moments8 is not None:
            ea, es = self.moments8.load(0, self.moments8.numel)
        else:
            ea, es = self.exp_avg, self.exp_avg_sq
        b1, b2 = self.betas
        base_state, base_params = {}, []
        for i, seg in enumerate(s_ for s_ in a.segments if s_.tier == "adamw"):
            sl = slice(seg.offset - lo_a, seg.offset - lo_a + seg.numel)
            base_state[i] = {"step": torch.tensor(float(self.step_count)), "exp_avg": ea[sl].view(seg.shape).clone(),
                             "exp_avg_sq": es[sl].view(seg.shape).clone()}
            base_params.append(i)
        muon_state, muon_params = {}, []
        for i, seg in enumerate(s_ for s_ in a.segments if s_.tier == "muon"):
            sl = slice(seg.offset - lo_m, seg.offset - lo_m + seg.numel)
            muon_state[i] = {"momentum_buffer": self.muon_mom[sl].view(seg.shape).clone()}
            muon_params.append(i)
        groups = []
        for seg in a.segments:
            if seg.tier != "steer":
                continue
            st = self.steer_state.get(seg.name)
            K = seg.mat_shape[0]
            for e in range(K):
                if st is None or st.get("mode") == "galore" or "Q_L" not in st:
                    P = None if st is None else st["P"][e]
                    groups.append({"projection": None if P is None else P[:, :-1].clone(),
                                   "projection_side": "left" if st is None else st["side"],
                                   "proj_step": 0 if st is None else st["proj_step"], "Q_L": None, "Q_R": None,
                                   "proj_basis": None if P is None else P.clone(), "last_c_orth": None,
                                   "last_steer_step": None, "steer_applied": False, "last_energy_ratio": None,
                                   "state": {} if st is None or st["m"] is None else
                                   {"momentum": st["m"][e].clone(), "variance": st["v"][e].clone(), "step": st["step"]},
                                   "segment": seg.name, "expert_idx": e})
                    continue
                ler = st.get("last_energy_ratio")
                groups.append({
                    "projection": st["Q_L"][e, :, :-1].clone(), "projection_side": "left", "proj_step": st["proj_step"],
                    "Q_L": st["Q_L"][e].clone(), "Q_R": st["Q_R"][e].clone(), "proj_basis": None, "last_c_orth": None,
                    "last_steer_step": st["last_steer_step"], "steer_applied": bool(st["steer_applied"][e]),
                    "last_energy_ratio": None if ler is None else float(ler[e]),
                    "state": {"momentum": st["m"][e].clone(), "variance": st["v"][e].clone(), "step": st["step"],
                              "subspace_step": st["subspace_step"]},
                    "segment": seg.name, "expert_idx": e})
        return {
            "base_optimizer": {"state": base_state, "param_groups": [{"lr": self.lr, "betas": (b1, b2), "eps": self.eps,
                                                                      "weight_decay": self.weight_decay,
                                                                      "params": base_params}]},
            "muon_optimizer": {"state": muon_state, "param_groups": [{"lr": self.muon_lr, "momentum": self.muon_momentum,
                                                                      "weight_decay": self.muon_weight_decay,
                                                                      "ns_steps": self.muon_ns_steps, "params": muon_params}]},
            "step_count": self.step_count, "expert_lr": float(self.expert_lr), "steer_scale": float(self.steer_scale),
            "param_groups": [{"lr": self.lr, "betas": (b1, b2), "weight_decay": self.weight_decay}],
            "_last_synced_lr": self.lr, "layer_groups": groups,
        }

    def load_reference_state_dict(self, sd: Dict) -> None:
        """Inverse of :meth:`reference_state_dict` (same tier partition and expert order)."""
        a = self.arena
        dev = a.device
        lo_a, _ = a.adamw_range
        lo_m, _ = a.muon_range
        ea = torch.zeros(a.adamw_range[1] - lo_a, device=dev)
        es = torch.zeros_like(ea)
        base = (sd.get("base_optimizer") or {}).get("state", {})
        for i, seg in enumerate(s_ for s_ in a.segments if s_.tier == "adamw"):
            ent = base.get(i, base.get(str(i)))
            if ent is None:
                continue
            sl = slice(seg.offset - lo_a, seg.offset - lo_a + seg.numel)
            ea[sl] = ent["exp_avg"].to(dev).float().reshape(-1)
            es[sl] = ent["exp_avg_sq"].to(dev).float().reshape(-1)
        if self.moments8 is not None:
            self.moments8.store(0, self.moments8.numel, ea, es)
        else:
            self.exp_avg.copy_(ea)
            self.exp_avg_sq.copy_(es)
        muon = (sd.get("muon_optimizer") or {}).get("state", {})
        for i, seg in enumerate(s_ for s_ in a.segments if s_.tier == "muon"):
            ent = muon.get(i, muon.get(str(i)))
            if ent is not None:
                sl = slice(seg.offset - lo_m, seg.offset - lo_m + seg.numel)
                self.muon_mom[sl] = ent["momentum_buffer"].to(dev).float().reshape(-1)
        self.step_count = int(sd.get("step_count", 0))
        if "expert_lr" in sd:
            self.expert_lr = float(sd["expert_lr"])
        if "steer_scale" in sd:
            self.steer_scale = float(sd["steer_scale"])
        groups = list(sd.get("layer_groups", []))
        n_expected = sum(s_.mat_shape[0] for s_ in a.segments if s_.tier == "steer")
        if len(groups) != n_expected:
            raise ValueError(f"layer group count mismatch: saved {len(groups)}, current {n_expected}")
        pos = 0
        self.steer_state = {}
        for seg in a.segments:
            if seg.tier != "steer":
                continue
            K, m, n = seg.mat_shape
            gs = groups[pos : pos + K]
            pos += K
            if any(g.get("Q_L") is None for g in gs):
                continue  # no two-sided bases saved for this segment: it starts fresh
            r1 = gs[0]["Q_L"].shape[-1]
            stack = lambda key: torch.stack([g[key].to(dev).float() for g in gs])
            sstack = lambda key: torch.stack([g["state"][key].to(dev).float() for g in gs])
            ler = [g.get("last_energy_ratio") for g in gs]
            self.steer_state[seg.name] = {
                "Q_L": stack("Q_L"), "Q_R": stack("Q_R"), "m": sstack("momentum"), "v": sstack("variance"),
                "step": int(gs[0]["state"].get("step", 0)), "subspace_step": int(gs[0]["state"].get("subspace_step", 0)),
                "proj_step": gs[0].get("proj_step"), "last_steer_step": gs[0].get("last_steer_step"), "rank": r1 - 1,
                "steer_applied": torch.tensor([bool(g.get("steer_applied", False)) for g in gs], device=dev),
                "has_grad": torch.ones(K, dtype=torch.bool, device=dev),
                "last_energy_ratio": None if any(x is None for x in ler) else torch.tensor(ler, device=dev),
            }
        self._q16.clear()

    def load_state_dict(self, sd):
        layout = [(s.name, s.tier, s.offset, s.numel) for s in self.arena.segments]
        if [tuple(x) for x in sd["layout"]] != [tuple(x) for x in layout]:
            raise ValueError("optimizer state layout does not match this model/tier partition")
        self.step_count = int(sd["step_count"])
        self.lr, self.muon_lr, self.expert_lr = float(sd["lr"]), float(sd["muon_lr"]), float(sd["expert_lr"])
        dev = self.arena.device
        if "steer_scale" in sd:
            self.steer_scale = float(sd["steer_scale"])
        if self.moments8 is not None and sd.get("moments8") is not None:
            self.moments8.load_state_dict(sd["moments8"])
        elif self.moments8 is not None:
            self.moments8.store(0, self.moments8.numel, sd["exp_avg"].to(dev).float(), sd["exp_avg_sq"].to(dev).float())
        elif sd.get("moments8") is not None:
            from .adam8bit import BlockwiseMoments

            tmp = BlockwiseMoments(self.exp_avg.numel(), dev)
            tmp.load_state_dict(sd["moments8"])
            m8, v8 = tmp.load(0, tmp.numel)
            self.exp_avg.copy_(m8)
            self.exp_avg_sq.copy_(v8)
        else:
            self.exp_avg.copy_(sd["exp_avg"].to(dev))
            self.exp_avg_sq.copy_(sd["exp_avg_sq"].to(dev))
        self.muon_mom.copy_(sd["muon_momentum"].to(dev))
        if self.arena.flat_master is not None and sd.get("master") is not None:
            self.arena.flat_master.copy_(sd["master"].to(dev))
        self.steer_state = {
            k: {kk: (vv.to(dev) if torch.is_tensor(vv) else vv) for kk, vv in v.items()} for k, v in sd["steer"].items()
        }
        self.qr_telemetry = sd.get("qr_telemetry", self.qr_telemetry)
        self._q16.clear()  # derived from the bases just loaded

    def get_qr_telemetry(self) -> Dict:
        """Fast-path survivals against Householder fall-backs of every QR so far, with the reasons. The counters live on
        the device between reports; this is the one place that reads them back."""
        t = flush_qr_telemetry(self.qr_telemetry)
        total, fb = t["total_qr_calls"], t["householder_fallbacks"]
        return {
            "total_qr_calls": total, "cholesky_fast_path_survivals": total - fb,
            "cholesky_survival_rate_pct": round(100.0 * (total - fb) / max(1, total), 2),
            "householder_fallbacks": fb, "householder_fallback_rate_pct": round(100.0 * fb / max(1, total), 2),
            "primary_fallback_reasons": dict(t["primary_fallback_reasons"]),
            "overlapping_triggers": dict(t["overlapping_triggers"]),
        }

    @torch.no_grad()
    def profile_rank_sensitivity(self, ranks=(4, 8, 16, 32, 64, 128), max_segments: int = 8) -> Dict:
        """How much of the current expert gradients a rank-r two-sided subspace captures: for each candidate rank the
        energy ratio ||Q_L^T G Q_R||_F^2 / ||G||_F^2 and the relative reconstruction error, averaged over the experts
        that received gradient, plus the smallest rank reaching 90 % energy (``recommended_rank``). Call it after a
        backward pass (the gradients are read, nothing is updated) to choose ``rank``
        (``triune/optim/centroid.py:1542-1609`` of the reference)."""
        a = self.arena
        a.fold_autograd_grads()
        report: Dict = {"ranks": {}, "segments": []}
        sums = {int(r): [0.0, 0.0, 0] for r in ranks}
        scratch = new_qr_telemetry()  # the profiler's QR calls do not count as training telemetry
        for seg in [s_ for s_ in a.segments if s_.tier == "steer"][:max_segments]:
            K, m, n = seg.mat_shape
            G = a.grad_view(seg).view(K, m, n).float()
            nz = G.flatten(1).abs().amax(-1) > 0
            if not bool(nz.any()):
                continue
            G = G[nz]
            gn = G.pow(2).sum((-2, -1)).clamp_min(1e-30)
            report["segments"].append(seg.name)
            for r in sums:
                rr = max(1, min(r, min(m, n) - 1))
                QL, QR = two_sided_bases(G, rr, telemetry=scratch)
                S = QL.transpose(1, 2) @ (G @ QR)
                energy = S.pow(2).sum((-2, -1)) / gn
                err = (G - QL @ S @ QR.transpose(1, 2)).pow(2).sum((-2, -1)).sqrt() / gn.sqrt()
                sums[r][0] += float(energy.sum())
                sums[r][1] += float(err.sum())
                sums[r][2] += int(G.shape[0])
        rec = None
        for r in sorted(sums):
            e, err, cnt = sums[r]
            if cnt == 0:
                continue
            report["ranks"][r] = {"energy_ratio": e / cnt, "relative_error": err / cnt, "matrices": cnt}
            if rec is None and e / cnt >= 0.9:
                rec = r
        report["recommended_rank"] = rec if rec is not None else (max(report["ranks"]) if report["ranks"] else None)
        report["current_rank"] = self.rank
        return report

    def get_telemetry(self) -> Dict:
        """Parameter and optimizer-state memory by tier (bytes)."""
        a = self.arena
        out = {"tiers": {}}
        for tier in ("adamw", "muon", "steer"):
            n = sum(s.numel for s in a.segments if s.tier == tier)
            out["tiers"][tier] = {"params": n}
        out["tiers"]["adamw"]["state_bytes"] = (self.moments8.nbytes() if self.moments8 is not None
                                                else self.exp_avg.numel() * 8)
        out["tiers"]["muon"]["state_bytes"] = self.muon_mom.numel() * 4
        sb = 0
        for st in self.steer_state.values():
            sb += sum(v.numel() * v.element_size() for v in st.values() if torch.is_tensor(v))
        out["tiers"]["steer"]["state_bytes"] = sb
        n_steer = max(1, out["tiers"]["steer"]["params"])
        out["steer_state_bytes_per_param"] = sb / n_steer
        out["adamw_equivalent_bytes"] = out["tiers"]["steer"]["params"] * 8
        return out


def profile_rank_sensitivity(model: torch.nn.Module, target_energy: float = 0.85, max_rank: int = 32, min_rank: int = 4) -> Dict[str, Any]:
    """Offline: for every weight matrix of ``model`` the smallest rank whose leading singular values hold
    ``target_energy`` of the squared Frobenius norm, clamped to [``min_rank``, ``max_rank``], with the energy that rank
    captures and the parameter ratio of a rank-k factorisation; totals over the model. Guides the choice of the subspace
    rank (``triune/optim/centroid.py:1542-1609`` of the reference; the method of the same name on the optimizer measures
    the live gradients instead)."""
    layers: Dict[str, Dict[str, Any]] = {}
    full_bytes = low_bytes = 0
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() < 2:
                continue
            w = p.detach().float().reshape(p.shape[0], -1)
            m, n = w.shape
            d = min(m, n)
            try:
                e = torch.linalg.svdvals(w).square()
                cum = torch.cumsum(e, 0) / e.sum().clamp_min(1e-12)
                hit = torch.nonzero(cum >= target_energy)
                k = int(hit[0]) + 1 if hit.numel() else min(max_rank, d)
            except RuntimeError:  # the decomposition did not converge: fall back to a quarter of the small side
                cum, k = torch.ones(d), min(max_rank, max(min_rank, d // 4))
            k = max(1, min(d, max(min_rank, min(max_rank, k))))
            layers[name] = {"shape": [m, n], "recommended_rank": k, "captured_energy": round(float(cum[k - 1]), 4),
                            "compression_ratio": round(m * n / max(1, (m + n) * k), 2)}
            full_bytes += m * n * p.element_size()
            low_bytes += (m + n) * k * p.element_size()
    return {"target_energy": target_energy, "max_rank": max_rank, "min_rank": min_rank, "num_profiled_matrices": len(layers),
            "total_uncompressed_params": sum(v["shape"][0] * v["shape"][1] for v in layers.values()),
            "total_low_rank_params": sum(sum(v["shape"]) * v["recommended_rank"] for v in layers.values()),
            "overall_compression_ratio": round(full_bytes / max(1, low_bytes), 2), "layers": layers}
