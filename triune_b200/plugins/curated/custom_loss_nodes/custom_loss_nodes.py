"""Three extra graph nodes: focal cross-entropy, an expert-load balance penalty, a router temperature schedule.

Same node names, ports and defaults as ``triune/modules/curated/custom_loss_nodes/custom_loss_nodes.py`` of the
reference, so graphs that use them load here. The classes and the function are importable on their own as well."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class FocalCrossEntropyLoss(nn.Module):
    """Cross-entropy with every token's term weighted by (1 - p_target)^gamma, so tokens the model already predicts well
    contribute little; ``gamma = 0`` is plain cross-entropy. The mean runs over all positions, ignored ones included (they
    contribute zero), as in the reference."""

    def __init__(self, gamma: float = 2.0, ignore_index: int = -100):
        super().__init__()
        self.gamma, self.ignore_index = float(gamma), int(ignore_index)

    def forward(self, logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        nll = F.cross_entropy(logits.reshape(-1, logits.size(-1)).float(), targets.reshape(-1), ignore_index=self.ignore_index,
                              reduction="none")
        return (torch.pow(1.0 - torch.exp(-nll), self.gamma) * nll).mean()


class CentroidBalanceLoss(nn.Module):
    """``coeff`` times the squared distance between the mean routing distribution of a batch ``[tokens, experts]`` and
    the uniform one."""

    def __init__(self, coeff: float = 0.01):
        super().__init__()
        self.coeff = float(coeff)

    def forward(self, router_probs: torch.Tensor) -> torch.Tensor:
        load = router_probs.reshape(-1, router_probs.size(-1)).float().mean(dim=0)
        return self.coeff * (load - 1.0 / router_probs.size(-1)).square().sum()


def anneal_temperature(global_step: int = 0, temp_max: float = 1.0, temp_min: float = 0.1, decay_steps: int = 5000) -> float:
    """Straight line from ``temp_max`` at step 0 to ``temp_min`` at ``decay_steps``, constant afterwards."""
    frac = min(1.0, max(0.0, global_step / max(1, decay_steps)))
    return temp_max + frac * (temp_min - temp_max)


def register(api):
    @api.register_node("FocalCrossEntropyLoss", {"logits": "tensor", "targets": "tensor"}, {"loss": "loss"},
                       "focal cross-entropy: down-weights tokens that are already predicted well")
    def focal(inputs, params, context):
        mod = FocalCrossEntropyLoss(float(params.get("gamma", 2.0)), int(params.get("ignore_index", -100)))
        return {"loss": mod(inputs["logits"], inputs["targets"])}

    @api.register_node("CentroidBalanceLoss", {"router_probs": "tensor"}, {"balance_loss": "loss"},
                       "penalty on the distance of the mean routing distribution from uniform")
    def balance(inputs, params, context):
        return {"balance_loss": CentroidBalanceLoss(float(params.get("coeff", 0.01)))(inputs["router_probs"])}

    @api.register_node("TemperatureAnnealer", {"global_step": "any"}, {"temperature": "any"},
                       "router exploration temperature as a function of the training step", optional=("global_step",))
    def annealer(inputs, params, context):
        step = inputs.get("global_step", params.get("global_step", 0))
        return {"temperature": anneal_temperature(int(step or 0), float(params.get("temp_max", 1.0)), float(params.get("temp_min", 0.1)),
                                                  int(params.get("decay_steps", 5000)))}
