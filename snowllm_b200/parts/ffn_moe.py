"""Routed top-k experts, each a gated feed-forward: sigmoid-routed SwiGLU experts without a shared expert
(snowllm/models/qwen3_5/layers.py:166-188; router formula tests/test_lfm2_reference.py:113-119;
tensor names and the fused / per-expert spellings snowllm/models/lfm2/weights.py:79-92).

Steps: router in float -> sort the (token, pick) pairs by expert -> grouped gate|up product over
the sorted rows (rows gathered from x) with SwiGLU at its store -> grouped down product (float) ->
weighted sum per token in pick order (left to the norm that follows: `kernels.ExpertSum`).  Only experts that own rows are read.

Options for other designs: ``scoring`` "softmax" (scores are a softmax over ALL experts' logits, the k
largest are picked and used as they are unless ``norm_topk_prob``); ``activation`` "swish_clamp" with
``limit``: g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(1.702 g) * (u + 1); ``shared``:
one more expert of the same form (a width and a limit of its own) that every token passes, its output
added (the sum is left as a ``kernels.DeltaSum``); with ``shared["row_gate"]`` its output is first multiplied
by sigmoid(w_sg . x), one number per token (tensor ``shared_row_gate`` [1, hidden]).  ``scoring``
"softmax_picked": the router's logits, plus the bias ``expert_bias`` which is then a part of the logit, pick
the k largest, and the weights are the softmax over the picked logits alone."""
from __future__ import annotations

import torch

from ..errors import ConfigError
from ..ops import grouped_linear, grouped_linear_glu, interleave_gate_up, kernels, linear, linear_glu
from .base import Part
from .registry import register_ffn
from .spec import INIT_BIAS, KEEP_F32, KEEP_SMALL, TensorSpec


class SigmoidMoE(Part):
    libraries = ("gemm", "gemm_skinny", "gemm_tc", "gemm_tc2", "moe", "elementwise", "sublayer")

    def __init__(self, dtype, names, *, hidden_size: int, intermediate_size: int, num_experts: int,
                 top_k: int, norm_topk_prob: bool, use_expert_bias: bool, routed_scaling_factor: float,
                 scale_input: bool = False, scoring: str = "sigmoid", activation: str = "silu",
                 limit: float | None = None, shared: dict | None = None):
        """``scale_input``: a pick's weight multiplies the expert's INPUT (the output is the plain sum of
        expert(w * x) over the picks) instead of its output.  ``shared``: {"intermediate_size", "limit"}."""
        super().__init__(dtype, names)
        if scoring not in kernels.ROUTER_SCORINGS:
            raise ConfigError(f"router scoring {scoring!r} (known: {', '.join(kernels.ROUTER_SCORINGS)})")
        if activation not in ("silu", "swish_clamp"):
            raise ConfigError(f"expert activation {activation!r} (known: silu, swish_clamp)")
        if activation == "swish_clamp" and not (limit and limit > 0):
            raise ConfigError("the clamped activation needs a positive limit")
        if shared is not None and not (activation == "swish_clamp" and shared.get("limit", 0) > 0
                                       and shared.get("intermediate_size", 0) > 0):
            raise ConfigError("a shared expert has the clamped form, with a width and a positive limit of its own")
        if scoring == "softmax" and use_expert_bias:
            raise ConfigError("an expert bias goes with sigmoid scores")
        self.scoring, self.activation, self.limit = scoring, activation, limit
        self.shared = dict(shared) if shared is not None else None
        self.shared_w13 = self.shared_w2 = self.shared_row_gate = None
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_experts, self.top_k = num_experts, top_k
        self.norm_topk_prob, self.use_expert_bias = norm_topk_prob, use_expert_bias
        self.routed_scaling_factor = routed_scaling_factor
        self.scale_input = scale_input
        self.router = self.bias = self.w13 = self.w2 = None
        self._fused = False
        self._ticket = None            # the counter of the one-launch front end (zero between launches)

    def declare(self, has):
        H, I, E = self.hidden_size, self.intermediate_size, self.num_experts
        n = self.names
        specs = [TensorSpec("router", n["router"], (E, H), keep=KEEP_SMALL)]
        if self.use_expert_bias:
            specs.append(TensorSpec("expert_bias", n["expert_bias"], (E,), INIT_BIAS, KEEP_F32))
        self._fused = has(n["fused_gate_up"])
        if self._fused:
            specs += [TensorSpec("gate_up", n["fused_gate_up"], (E, 2 * I, H)),
                      TensorSpec("down", n["fused_down"], (E, H, I))]
        else:
            for e in range(E):
                p = f"{n['experts']}{e}."
                specs += [TensorSpec(f"gate.{e}", p + n["expert_gate"], (I, H)),
                          TensorSpec(f"up.{e}", p + n["expert_up"], (I, H)),
                          TensorSpec(f"down.{e}", p + n["expert_down"], (H, I))]
        if self.shared is not None:
            S = self.shared["intermediate_size"]
            specs += [TensorSpec("shared_gate", n["shared_gate"], (S, H)), TensorSpec("shared_up", n["shared_up"], (S, H)),
                      TensorSpec("shared_down", n["shared_down"], (H, S))]
            if self.shared.get("row_gate"):
                specs.append(TensorSpec("shared_row_gate", n["shared_row_gate"], (1, H)))
        return specs

    def bind(self, tensors):
        E = self.num_experts
        self.router = tensors["router"]
        self.bias = tensors.get("expert_bias") if self.use_expert_bias else None
        if self._fused:
            gate, up = tensors["gate_up"].chunk(2, dim=1)
            self.w2 = tensors["down"].contiguous()
        else:
            gate = torch.stack([tensors[f"gate.{e}"] for e in range(E)])
            up = torch.stack([tensors[f"up.{e}"] for e in range(E)])
            self.w2 = torch.stack([tensors[f"down.{e}"] for e in range(E)]).contiguous()
        # gate and up rows interleaved by 8 where the width allows: the product then applies SwiGLU itself
        self.interleaved = self.intermediate_size % 8 == 0
        self.w13 = interleave_gate_up(gate, up) if self.interleaved else torch.cat((gate, up), 1).contiguous()
        if self.shared is not None:
            self.shared_interleaved = self.shared["intermediate_size"] % 8 == 0
            self.shared_w13 = (interleave_gate_up(tensors["shared_gate"], tensors["shared_up"]) if self.shared_interleaved
                               else torch.cat((tensors["shared_gate"], tensors["shared_up"]), 0).contiguous())
            self.shared_w2 = tensors["shared_down"]
            if self.shared.get("row_gate"):
                self.shared_row_gate = tensors["shared_row_gate"].contiguous()

    def bytes_read(self, bound, picked=None):
        """Router and bias whole; of the experts only those that were picked (``picked`` None: all)."""
        experts = sum(n for name, n in bound.items() if name.split(".")[0] in ("gate", "up", "down", "gate_up"))
        # (the shared expert's tensors, ``shared_*``, count among the rest: every step reads them whole)
        rest = sum(bound.values()) - experts
        share = 1.0 if picked is None else min(picked, self.num_experts) / self.num_experts
        return rest + int(experts * share)

    def route(self, x):
        return kernels.moe_route(x, self.router, self.bias, self.top_k, self.norm_topk_prob,
                                 self.routed_scaling_factor, self.scoring)

    def forward_from_residual(self, ctx, residual, delta, norm):
        """The norm that precedes this feed-forward, the router and the sort in one launch, for the few rows
        of a decode step (csrc/moe.cu: norm_route_sort_kernel); None when this step or this norm is not
        one it takes, and the block then runs the norm and ``forward`` one after the other."""
        weight, eps = getattr(norm, "weight", None), getattr(norm, "eps", None)
        if getattr(norm, "fusable_rms", False) is not True or weight is None or eps is None:
            return None
        if self.scale_input or not kernels.FUSE_ROUTER or not kernels.norm_route_sort_ok(residual, delta, weight, self.router, self.top_k):
            return None
        if self.scoring != "sigmoid" or self.activation != "silu" or self.shared is not None:
            return None
        if self._ticket is None or self._ticket.device != residual.device:
            self._ticket = torch.zeros(1, dtype=torch.int32, device=residual.device)
        x, *routed = kernels.norm_route_sort(residual, delta, weight, eps, self.dtype, self.router, self.bias,
                                             self.top_k, self.norm_topk_prob, self.routed_scaling_factor,
                                             self._ticket)
        if ctx is not None:
            ctx.tap("ffn_in", x)
        return self._experts(ctx, x, *routed)

    def forward(self, ctx, x):
        routed = self._experts(ctx, x, *kernels.moe_route_sort(
            x, self.router, self.bias, self.top_k, self.norm_topk_prob, self.routed_scaling_factor, self.scoring))
        if self.shared is None:
            return routed
        act = linear_glu(x, self.shared_w13, self.shared_interleaved, self.activation, self.shared["limit"])
        gate = None
        if self.shared_row_gate is not None:
            gate = kernels.row_dot(x, self.shared_row_gate)        # float [M, 1]: one logit per token
            if ctx is not None:
                ctx.tap("shared_row_gate", gate)
        return kernels.DeltaSum(linear(act, self.shared_w2, out_dtype=torch.float32), routed, a_gate=gate)

    def _gate_up(self, x, offsets, rows_out, cap, a_rows, a_div):
        """The experts' activated gate|up product over the rows in expert order."""
        return grouped_linear_glu(x, self.w13, offsets, rows_out, cap, a_rows, a_div, self.interleaved,
                                  self.activation, self.limit or 0.0)

    def _experts(self, ctx, x, ids, weights, offsets, pair_pos, sorted_pair):
        M, k = x.shape[0], self.top_k
        if ctx is not None:
            ctx.tap("moe_route", ids)
            ctx.tap("moe_route_input", x)
        cap = min(M, M * k)          # an expert gets a token at most once
        if self.scale_input:
            # the rows in expert order, each times its pick's weight; the outputs are then summed as they are
            xs, weights = kernels.moe_scaled_rows(x, sorted_pair, weights, k)
            act = self._gate_up(xs, offsets, M * k, cap, None, 1)
            y = grouped_linear(act, self.w2, offsets, M * k, cap, out_dtype=torch.float32)
            return kernels.ExpertSum(y, pair_pos, weights)
        act = self._gate_up(x, offsets, M * k, cap, sorted_pair, k)
        y = grouped_linear(act, self.w2, offsets, M * k, cap, out_dtype=torch.float32)
        return kernels.ExpertSum(y, pair_pos, weights)     # the norm that follows adds it into the residual


register_ffn("sigmoid_moe", SigmoidMoE)
register_ffn("routed_experts", SigmoidMoE)
