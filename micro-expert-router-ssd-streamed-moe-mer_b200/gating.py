"""Mirror of the reference's LinearGate (gating.rs:118-476); routing itself runs on the GPU."""
import enum
from dataclasses import dataclass

import numpy as np


class ScoringFunc(enum.IntEnum):
    """gating.rs:94-97"""
    Softmax = 0
    Sigmoid = 1


@dataclass
class RoutingDecision:
    """gating.rs:40-47: chosen expert ids (descending score) and their mixing weights."""
    experts: np.ndarray
    weights: np.ndarray


class LinearGate:
    """Router parameters.  `new` reproduces Mixtral/Qwen3 behaviour (softmax, renormalised top-k);
    `with_routing` adds the DeepSeek-V3 surface (sigmoid, selection-only bias, groups, scaling)."""

    def __init__(self, weights, num_experts, d_model, top_k):
        if not (0 < top_k <= num_experts):
            raise ValueError("top_k must be in 1..=num_experts")  # gating.rs:150-153
        weights = np.ascontiguousarray(weights, dtype=np.float32)
        if weights.size != num_experts * d_model:
            raise ValueError("gate weight matrix must be [num_experts, d_model]")  # gating.rs:154-158
        self.weights = weights.reshape(num_experts, d_model)
        self.num_experts, self.d_model, self.top_k = num_experts, d_model, top_k
        self.normalise_topk = True
        self.scoring_func = ScoringFunc.Softmax
        self.correction_bias = None
        self.n_group, self.topk_group = 1, 1
        self.routed_scaling_factor = 1.0
        self.logit_bias = None  # harness extension (Zipf skew added to the logits)
        self._bound = None

    new = classmethod(lambda cls, weights, num_experts, d_model, top_k: cls(weights, num_experts, d_model, top_k))

    @classmethod
    def with_routing(cls, weights, num_experts, d_model, top_k, scoring_func, normalise_topk, correction_bias, n_group,
                     topk_group, routed_scaling_factor):
        gate = cls(weights, num_experts, d_model, top_k)
        gate.scoring_func = ScoringFunc(scoring_func)
        gate.normalise_topk = bool(normalise_topk)
        if correction_bias is not None:
            correction_bias = np.ascontiguousarray(correction_bias, dtype=np.float32)
            if correction_bias.size != num_experts:
                raise ValueError("correction_bias must have length num_experts")  # gating.rs:226-232
        gate.correction_bias = correction_bias
        gate.n_group = max(int(n_group), 1)
        gate.topk_group = int(topk_group)
        gate.routed_scaling_factor = float(routed_scaling_factor)
        return gate

    def bind(self, backend, layer, shared_expert_id=0xFFFFFFFF):
        """Installs this gate as `layer`'s router on a Backend."""
        backend.install_router(layer, self, shared_expert_id)
        self._bound = (backend, layer)
        return self

    def route(self, x) -> RoutingDecision:
        """LinearGate::route (gating.rs:389-392) for one hidden state, on the GPU."""
        if self._bound is None:
            raise RuntimeError("LinearGate.route needs bind(backend, layer) first: routing runs on the GPU only")
        backend, layer = self._bound
        ids, w = backend.route(layer, np.asarray(x, dtype=np.float32).reshape(1, -1))
        keep = ids[0] != 0xFFFFFFFF
        return RoutingDecision(ids[0][keep], w[0][keep])
