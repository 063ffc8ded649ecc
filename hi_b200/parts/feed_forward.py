"""Feed-forward parts: dense SwiGLU, and sigmoid-routed top-k experts with a shared expert."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .basic import Part
from .context import Pending
from .linear import linear
from .registry import register
from .spec import TensorSpec


class _SwiGLU:
    """(silu(x Wg^T) * x Wu^T) Wd^T with gate and up fused into one product
    (Mlp::forward, crates/hi-mlx/src/models.rs:2307-2312)."""

    def __init__(self, prefix: str, hidden: int, inter: int):
        self.prefix, self.hidden, self.inter = prefix, hidden, inter
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}.gate_proj.weight", (self.inter, self.hidden)),
                TensorSpec(f"{self.prefix}.up_proj.weight", (self.inter, self.hidden)),
                TensorSpec(f"{self.prefix}.down_proj.weight", (self.hidden, self.inter))]

    def load(self, fetch):
        g, u = fetch(f"{self.prefix}.gate_proj.weight"), fetch(f"{self.prefix}.up_proj.weight")
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = fetch(f"{self.prefix}.down_proj.weight").contiguous()

    def forward(self, x):
        return linear(ops.swiglu(linear(x, self.w_gate_up)), self.w_down)


@register("feed_forward", "dense_swiglu")
class DenseSwiGLU(Part):
    """params: ``hidden_size``, ``intermediate_size``; tensors ``<prefix>.{gate,up,down}_proj.weight``."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.mlp = _SwiGLU(prefix, int(params["hidden_size"]), int(params["intermediate_size"]))

    def tensor_specs(self):
        return self.mlp.tensor_specs()

    def load(self, fetch):
        self.mlp.load(fetch)

    def forward(self, normed, ctx):
        return self.mlp.forward(normed)


@register("feed_forward", "routed_experts")
@register("feed_forward", "moe_sigmoid")
class SigmoidRoutedExperts(Part):
    """Router logits in float32, the k largest (ties to the lower id); by default score =
    sigmoid(logit) without renormalisation and the score scales the expert input; an always-on
    shared expert sees the unscaled input; outputs are summed (Llama4Moe::forward,
    crates/hi-mlx/src/models.rs:6055-6103; the reference is top-1 only). The other routing rules of
    the reference's donor kernel (crates/hi-cuda/src/kernels.cu:536-546) are parameters too.

    params: ``hidden_size``, ``num_experts``, ``top_k``, ``intermediate_size``, ``shared_expert``;
      ``score``        "sigmoid" (default) | "softmax" (over all experts)
      ``renormalize``  the chosen scores are divided by their sum (default False)
      ``scale``        "input" (default: the score multiplies what the expert reads) | "output"
                       (it multiplies what the expert returns, in the sum the next norm takes)
    tensors: ``<prefix>.router.weight`` [E, H]; ``<prefix>.experts.{gate,up}_proj.weight`` [E, I, H];
    ``<prefix>.experts.down_proj.weight`` [E, H, I]; ``<prefix>.shared_expert.{gate,up,down}_proj.weight``.
    """

    graph_safe = True

    FEW_ROWS = 10    # up to this many routed rows the weight-streaming kernel is used (measured: from 12
                     # rows the tcgen05 kernel streams the expert weights faster, even with nearly empty tiles)
    wants_f32_input = True   # the router reads the norm's float32 output
    OVERLAP_SHARED = True    # run the shared expert on a second stream beside the routed path

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.hidden, self.experts = int(params["hidden_size"]), int(params["num_experts"])
        self.top_k, self.inter = int(params["top_k"]), int(params["intermediate_size"])
        if not 1 <= self.top_k <= self.experts:
            raise ValueError(f"{prefix}: top_k {self.top_k} outside 1..{self.experts}")
        self.shared = _SwiGLU(f"{prefix}.shared_expert", self.hidden, self.inter) \
            if params.get("shared_expert", True) else None
        score, scale = params.get("score", "sigmoid"), params.get("scale", "input")
        if score not in ("sigmoid", "softmax") or scale not in ("input", "output"):
            raise ValueError(f"{prefix}: score {score!r} / scale {scale!r} are not known (sigmoid | softmax; input | output)")
        self.router_mode = (ops.ROUTER_SOFTMAX if score == "softmax" else 0) | \
            (ops.ROUTER_RENORMALIZE if params.get("renormalize", False) else 0)
        self.scale_output = scale == "output"
        self._ones: Optional[torch.Tensor] = None
        self.w_router = self.w_gate = self.w_up = self.w_down = None
        self._side_stream = None

    def tensor_specs(self):
        e, i, h, p = self.experts, self.inter, self.hidden, self.prefix
        specs = [TensorSpec(f"{p}.router.weight", (e, h)),
                 TensorSpec(f"{p}.experts.gate_proj.weight", (e, i, h)),
                 TensorSpec(f"{p}.experts.up_proj.weight", (e, i, h)),
                 TensorSpec(f"{p}.experts.down_proj.weight", (e, h, i))]
        return specs + (self.shared.tensor_specs() if self.shared else [])

    def load(self, fetch):
        p = self.prefix

        def expert_tensor(name):
            t = fetch(name)
            if t.dtype != self.env.dtype:
                raise ValueError(
                    f"tensor '{name}' is stored in {t.dtype} and stays so; the expert kernels of the "
                    f"{self.env.dtype} path cannot take it (run with --dtype float32)")
            return t.contiguous()

        self.w_router = expert_tensor(f"{p}.router.weight")
        self.w_gate = expert_tensor(f"{p}.experts.gate_proj.weight")
        self.w_up = expert_tensor(f"{p}.experts.up_proj.weight")
        self.w_down = expert_tensor(f"{p}.experts.down_proj.weight")
        if self.shared:
            self.shared.load(fetch)

    def _shared_on_side_stream(self, normed):
        """The shared expert has no dependency on the routing: it runs on a second stream beside
        the router, the plan and the routed experts (in a captured step: a parallel branch), and
        joins before the sum. Both paths stream weights; together they keep HBM busier than in turn."""
        cur = torch.cuda.current_stream()
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=normed.device)
        side = self._side_stream
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            shared = self.shared.forward(normed)
        normed.record_stream(side)
        shared.record_stream(cur)
        return shared, side

    def forward(self, normed, ctx, normed_f32=None):
        n = normed.shape[0]
        side = None
        if self.shared and self.OVERLAP_SHARED:
            shared, side = self._shared_on_side_stream(normed)
        router_in = normed if normed_f32 is None else normed_f32
        forced = ctx.forced.get(f"{self.prefix}.router_ids") if ctx.forced else None
        if forced is None:
            ids, scores, plan = ops.router_plan(router_in, self.w_router, self.top_k, self.router_mode)
        else:
            # debug: another run's expert choices, scored with this run's own logits (two runs in
            # different precisions can then be compared token by token)
            _own, _s, logits = ops.router_topk(router_in, self.w_router, self.top_k, want_logits=True)
            ids = forced.to(device=logits.device, dtype=torch.int32).reshape(n, self.top_k).contiguous()
            chosen = torch.gather(logits, 1, ids.long())
            scores = torch.sigmoid(chosen) if not self.router_mode & ops.ROUTER_SOFTMAX else \
                torch.exp(chosen - torch.logsumexp(logits, dim=1, keepdim=True))
            if self.router_mode & ops.ROUTER_RENORMALIZE:
                scores = scores / scores.sum(dim=1, keepdim=True)
            scores = scores.contiguous()
            plan = ops.moe_plan(ids, self.experts)
        if ctx.tap is not None:
            ctx.tap(f"{self.prefix}.router_ids", ids)
        entry_weights = None
        if self.scale_output:
            # the experts read the unscaled rows (a factor of one); their outputs take the score in the sum
            if self._ones is None or self._ones.numel() < scores.numel():
                self._ones = torch.ones(max(scores.numel(), 65536), dtype=torch.float32, device=scores.device)
            entry_weights, scores = scores.view(-1), self._ones[: scores.numel()].view_as(scores)
        tc = ops.moe_tc_supported(normed, self.w_gate)
        few = n * self.top_k <= (self.FEW_ROWS if tc else 128)
        if not few and tc:
            # many rows per expert: the grouped products run on tcgen05
            act = ops.moe_gate_up_tc(normed, plan, self.top_k, self.w_gate, self.w_up, scores)
            y = ops.moe_down_tc(act, self.w_down, plan)
        else:
            act = ops.moe_gate_up(normed, plan, self.top_k, self.w_gate, self.w_up, scores, few)
            y = ops.moe_down(act, self.w_down, plan, few)
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        else:
            shared = self.shared.forward(normed) if self.shared else None
        # the sum shared + routed rows is taken inside the next norm's residual add
        return Pending(dense=shared, routed=y, slot_of_entry=plan.slot_of_entry, top_k=self.top_k,
                       entry_weights=entry_weights)
