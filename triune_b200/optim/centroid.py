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
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .. import _ext, config as C
from ..ops import reference as ref
from .arena import MuonGroup, ParamArena, Segment
from .subspace import batched_qr, new_qr_telemetry, reorthogonalise, two_sided_bases

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
                 tensor_core_subspace: bool = True):
        if core_mask_mode not in ("full", "triu"):
            raise ValueError(f"Unknown core_mask_mode={core_mask_mode!r}; expected 'full' or 'triu'")
        self._in_set_lr = False
        self.model = model
        tiers, mat_views, steer_meta = classify_parameters(model, param_roles, use_muon, aspect_safeguard)
        self.tiers, self.steer_meta = tiers, steer_meta
        named = list(model.named_parameters())
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
        self.exp_avg = torch.zeros(hi - lo, device=dev, dtype=torch.float32)
        self.exp_avg_sq = torch.zeros(hi - lo, device=dev, dtype=torch.float32)
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
        # the subspace projections are fp32 batched products; TF32 tensor cores keep ~1e-3 relative accuracy,
        # the same order as the bf16 bases the reference uses on CUDA
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        try:
            self._step_steer()
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
        return loss

    def step_parameters(self, params: Iterable[torch.nn.Parameter], is_global_step_end: bool = True):
        """Layer-wise stepping hook (used by layer streaming): here all tiers step together on the last call."""
        if is_global_step_end:
            self.step()

    # ---- Tier 3 --------------------------------------------------------------------------------
    def _step_adamw(self):
        a = self.arena
        lo, hi = a.adamw_range
        if hi == lo:
            return
        b1, b2 = self.betas
        t = self.step_count
        master = a.master()[lo:hi]
        grad = a.flat_grad[lo:hi]
        if self._use_kernels():
            pb = a.flat_param[lo:hi] if a.flat_master is not None else None
            _ext.ext().adamw_flat(master, self.exp_avg, self.exp_avg_sq, grad, pb, self.lr, b1, b2, self.eps,
                                  self.weight_decay, t, self._clip_coef, 1.0, self._hyper_arg())
            from .. import ops
            ops._tick()
            return
        g = grad * self._clip_coef
        self.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
        self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
        mh = self.exp_avg / (1 - b1**t)
        vh = self.exp_avg_sq / (1 - b2**t)
        master.mul_(1 - self.lr * self.weight_decay).add_(mh / (vh.sqrt() + self.eps), alpha=-self.lr)
        if a.flat_master is not None:
            a.flat_param[lo:hi].copy_(master)

    # ---- Tier 1 --------------------------------------------------------------------------------
    def _step_muon(self):
        a = self.arena
        lo, hi = a.muon_range
        if hi == lo:
            return
        from .. import ops

        beta = self.muon_momentum
        kern = self._use_kernels()
        for grp in a.muon_groups:
            m, n = grp.shape
            k0, k1 = self._owned(grp.count)
            if k1 == k0:
                continue
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

    def _step_steer(self):
        a = self.arena
        b1, b2 = self.expert_betas
        for seg in a.segments:
            if seg.tier != "steer":
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
                # dense AdamW on the experts (ablation path)
                if st is None:
                    st = self.steer_state[seg.name] = {"m": torch.zeros_like(G), "v": torch.zeros_like(G), "step": 0}
                st["step"] += 1
                st["m"].mul_(b1).add_(G, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(G, G, value=1 - b2)
                d = (st["m"] / (1 - b1 ** st["step"])) / ((st["v"] / (1 - b2 ** st["step"])).sqrt() + self.eps)
                self._apply_steer_delta(seg, d, k0, k1)
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
        return {
            "step_count": self.step_count, "lr": self.lr, "muon_lr": self.muon_lr, "expert_lr": self.expert_lr,
            "layout": [(s.name, s.tier, s.offset, s.numel) for s in self.arena.segments],
            "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq, "muon_momentum": self.muon_mom,
            "master": self.arena.flat_master,
            "steer": {k: {kk: vv for kk, vv in v.items()} for k, v in self.steer_state.items()},
            "qr_telemetry": self.qr_telemetry,
        }

    def load_state_dict(self, sd):
        layout = [(s.name, s.tier, s.offset, s.numel) for s in self.arena.segments]
        if [tuple(x) for x in sd["layout"]] != layout:
            raise ValueError("optimizer state layout does not match this model/tier partition")
        self.step_count = int(sd["step_count"])
        self.lr, self.muon_lr, self.expert_lr = float(sd["lr"]), float(sd["muon_lr"]), float(sd["expert_lr"])
        dev = self.arena.device
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
        return self.qr_telemetry

    def get_telemetry(self) -> Dict:
        """Parameter and optimizer-state memory by tier (bytes)."""
        a = self.arena
        out = {"tiers": {}}
        for tier in ("adamw", "muon", "steer"):
            n = sum(s.numel for s in a.segments if s.tier == tier)
            out["tiers"][tier] = {"params": n}
        out["tiers"]["adamw"]["state_bytes"] = self.exp_avg.numel() * 8
        out["tiers"]["muon"]["state_bytes"] = self.muon_mom.numel() * 4
        sb = 0
        for st in self.steer_state.values():
            sb += sum(v.numel() * v.element_size() for v in st.values() if torch.is_tensor(v))
        out["tiers"]["steer"]["state_bytes"] = sb
        n_steer = max(1, out["tiers"]["steer"]["params"])
        out["steer_state_bytes_per_param"] = sb / n_steer
        out["adamw_equivalent_bytes"] = out["tiers"]["steer"]["params"] * 8
        return out
