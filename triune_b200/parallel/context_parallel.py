"""Context (sequence) parallelism for gated linear attention by state hand-off.

Every rank of the group holds one contiguous segment of the sequence, in rank order. Because the recurrence is linear
in the state, a segment's output with the true incoming state S_in is its output from a zero state plus a correction:

    o_t      = o_t^{(0)} + scale * (q_t * e^{B_t})^T S_in          B_t = sum of the log decays from the segment start to t
    S_out    = diag(e^{B_end}) S_in + S_loc                          S_loc = the segment's final state from a zero state

so each rank runs the chunked kernels ONCE on its own tokens, the ranks exchange one ``[B, H, dk, dv]`` state and one
``[B, H, dk]`` total decay each (an all-gather of a few hundred KB, independent of the sequence length), every rank
folds the states of the ranks before it, and the correction is one batched product. This is what makes long prompts
(the 4 x 16384 prefill shape and beyond) splittable over GPUs without any all-to-all of activations.

The whole function is differentiable, the collectives included. On CUDA the local pass uses the tcgen05 kernels, whose
final state carries no gradient of its own; :func:`triune_b200.ops.gla_final_state_with_grad` restores it analytically, so
gradients flow from later segments back into the keys, values and decays of earlier ones on that path too. The reference has no sequence parallelism (``triune/model/attention.py:360-572`` runs whole sequences).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import ops
from ..ops import gla_cuda
from ..ops.reference import GLA_MIN_LOG_DECAY


def _gather(t: torch.Tensor, group) -> list:
    """All-gather that keeps the autograd graph when one is being recorded."""
    world = dist.get_world_size(group)
    if torch.is_grad_enabled() and t.requires_grad:
        import torch.distributed.nn.functional as dnf

        return list(dnf.all_gather(t.contiguous(), group=group))
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t.contiguous(), group=group)
    return out


def _kernel_path(q, k, v, g) -> bool:
    """Whether the local pass runs the CUDA kernels (which clamp the decay and return the state without a gradient)."""
    return gla_cuda.supported(q, k, v, g, None)


def cp_gla(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, group=None, scale: float = 1.0,
           gate_logits: bool = False, initial_state: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gated linear attention over a sequence split across ``group``.

    q, k, g: this rank's segment ``[B, T_local, H, dk]``; v: ``[B, T_local, H, dv]``; ``g`` is the per-dimension log
    decay (<= 0) or the raw gate logits when ``gate_logits``. ``initial_state`` (``[B, H, dk, dv]``) is the state before
    the FIRST segment and must be given identically on every rank. Returns this rank's outputs and the state at the END
    OF ITS SEGMENT (the last rank's is the state of the whole sequence).
    """
    group = group if group is not None else dist.group.WORLD
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    dt = torch.float64 if q.dtype == torch.float64 else torch.float32
    out0, s_loc = ops.gla(q, k, v, g, initial_state=None, scale=1.0, gate_logits=gate_logits)
    gl = F.logsigmoid(g.to(dt)) if gate_logits else g.to(dt)
    gl = torch.clamp(gl, max=0.0)
    kernel_path = _kernel_path(q, k, v, g)
    if kernel_path:
        gl = torch.clamp(gl, min=GLA_MIN_LOG_DECAY)  # the kernels clamp the per-step log decay
        if torch.is_grad_enabled() and (k.requires_grad or v.requires_grad or g.requires_grad):
            # the kernels return the state without a gradient; its dependence on k, v and the decays is restored here
            # (two batched products and two cumulative sums), so the hand-off to later segments can be trained through
            s_loc = ops.gla_final_state_with_grad(k, v, gl, None, s_loc)
    bcum = torch.cumsum(gl, dim=1)                                   # [B, T, H, dk]
    d_tot = torch.exp(bcum[:, -1])                                   # [B, H, dk]: decay over the whole segment
    s_loc = s_loc.to(dt)
    s_in = initial_state.to(dt) if initial_state is not None else torch.zeros_like(s_loc)
    if world > 1:
        # ONE collective for state and decay (packed along the last axis): a single node in the backward graph too, so
        # the ranks cannot disagree on the order of their backward collectives
        packed = _gather(torch.cat((s_loc, d_tot.unsqueeze(-1)), dim=-1), group)
        for j in range(rank):                                        # fold the segments before this one, in order
            s_in = packed[j][..., -1:] * s_in + packed[j][..., :-1]
        # every rank must run the gather's backward (a collective), also those that use no earlier segment
        s_in = s_in + 0.0 * sum(p.sum() for p in packed)
    corr = torch.einsum("bthk,bhkv->bthv", q.to(dt) * torch.exp(bcum), s_in)
    out = (out0.to(dt) + corr) * scale
    s_end = d_tot.unsqueeze(-1) * s_in + s_loc
    return out.to(q.dtype), s_end
