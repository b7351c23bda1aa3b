"""Mixture of experts: a grouped top-k router, clamped gated experts, identity outputs and a shared expert.

Steps of ``forward`` (no step waits for the host):

1. router logits in fp32 (one product), then ``ops.moe_route``: softmax over all outputs, the correction for the
   choice only, the best groups, the top-k outputs and their scores as weights;
2. ``ops.moe_group``: the (token, choice) pairs that go to real experts, sorted by expert on the device;
3. two grouped products over that order (``csrc/grouped_gemm.cu``): gate and up with the clamped activation,
   then down into fp32 rows; in bfloat16, when the experts get many rows each (prompts), the rows are gathered
   side by side instead and the two products go to the tensor cores: the vendor library's grouped product
   over the experts' row ranges where it has one, else every expert's products through ``linear``, for which the
   host reads the experts' offsets once (the only wait of the part, and never inside a graph capture);
4. ``ops.moe_combine``: each token adds its weighted rows, in the order of its choices, and its own input for
   an identity output;
5. the shared expert, if any: gate/up product, the same activation with its own limit, down with the residual add.

Options of the spec: sigmoid scores instead of the softmax (a flag of the routing kernel); ungated experts with the
squared ReLU (one up matrix per expert, the activation in the grouped product's epilogue or, after the vendor
library's product, in ``ops.activation``); weights that multiply the experts' inputs (the rows are gathered in the
sorted order and multiplied by their pair's weight in fp32 on the way, ``ops.moe_gather``; the combine then adds
the chosen rows unweighted).
"""

from __future__ import annotations

import torch

from ..config.specs import RoutedExpertsSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, register_part
from .linear import linear


# From this many rows per expert on (on average) a bfloat16 step runs each expert's products through linear().
ROWS_PER_EXPERT_FOR_TENSOR_CORES = 32


class RoutedExperts(Part):
    graph_safe = True   # the grouped products wait for no one; the per-expert form is not chosen while capturing
    returns_output = True   # forward(..., residual=None) returns the fp32 output instead of adding it
    _library_groups = True      # until the vendor library's grouped product has refused once

    def __init__(self, spec: RoutedExpertsSpec) -> None:
        super().__init__(spec)
        n_all = spec.num_experts + spec.num_identity
        if spec.num_experts < 0 or spec.num_identity < 0 or n_all <= 0:
            raise ValueError("a router needs at least one output")
        if spec.num_groups <= 0 or n_all % spec.num_groups != 0:
            raise ValueError(f"{n_all} router outputs do not form {spec.num_groups} equal groups")
        if not 0 < spec.keep_groups <= spec.num_groups:
            raise ValueError("keep_groups must be between 1 and the number of groups")
        if not 0 < spec.top_k <= spec.keep_groups * (n_all // spec.num_groups):
            raise ValueError("top_k exceeds the outputs that the kept groups hold")
        if spec.scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"scoring {spec.scoring!r} is not implemented (softmax and sigmoid are)")
        if spec.expert_form not in ("gated_clamp", "relu2"):
            raise ValueError(f"expert form {spec.expert_form!r} is not implemented (gated_clamp and relu2 are)")
        if spec.weight_on_input and spec.num_identity > 0:
            raise ValueError("identity outputs take their weight on the output")
        self.gated = spec.expert_form == "gated_clamp"
        self.n_all = n_all

    def tensor_decls(self):
        s = self.spec
        decls = [TensorDecl(s.prefix + "router", (self.n_all, s.hidden_size))]
        if s.has_correction:
            decls.append(TensorDecl(s.prefix + "correction", (self.n_all,), "zeros"))
        halves = ("gate", "up") if self.gated else ("up",)
        for e in range(s.num_experts):
            decls += [TensorDecl(f"{s.prefix}e{e}.{half}", (s.expert_size, s.hidden_size)) for half in halves]
            decls.append(TensorDecl(f"{s.prefix}e{e}.down", (s.hidden_size, s.expert_size)))
        if s.shared_size > 0:
            decls += [TensorDecl(f"{s.prefix}shared.{half}", (s.shared_size, s.hidden_size)) for half in halves]
            decls.append(TensorDecl(s.prefix + "shared.down", (s.hidden_size, s.shared_size)))
        return decls

    def load(self, fetch, runtime) -> None:
        s = self.spec
        self.runtime = runtime
        self.w_router = fetch.matrix(s.prefix + "router")
        self.correction = fetch.vector(s.prefix + "correction") if s.has_correction else None
        halves = ("gate", "up") if self.gated else ("up",)
        if s.num_experts > 0:
            # per expert: gate rows then up rows, so that one grouped product yields both (ungated: the up rows)
            self.w_gate_up = torch.stack([torch.cat([fetch.matrix(f"{s.prefix}e{e}.{half}") for half in halves], 0)
                                          for e in range(s.num_experts)])
            self.w_down = torch.stack([fetch.matrix(f"{s.prefix}e{e}.down") for e in range(s.num_experts)])
            self.counts = torch.zeros(s.num_experts, dtype=torch.int32, device=runtime.device)
        if s.shared_size > 0:
            self.w_shared_gate_up = torch.cat([fetch.matrix(f"{s.prefix}shared.{half}") for half in halves], 0)
            self.w_shared_down = fetch.matrix(s.prefix + "shared.down")

    def forward(self, x, ctx, residual):
        """Adds to ``residual`` (fp32); with ``residual`` None returns the output as a new fp32 tensor."""
        s = self.spec
        n, dev = x.shape[0], x.device
        logits = linear(x, self.w_router, out_dtype=torch.float32)
        ids = torch.empty((n, s.top_k), dtype=torch.int32, device=dev)
        weights = torch.empty((n, s.top_k), dtype=torch.float32, device=dev)
        ops.moe_route(logits, self.correction, ids, weights, n_groups=s.num_groups, keep=s.keep_groups,
                      sigmoid=s.scoring == "sigmoid")
        # single-token steps, a few rows per expert: the grouped product that streams weights through registers
        few_ok = ops.grouped_few_rows_ok((s.hidden_size, s.expert_size), x.dtype)
        table = ops.RoutingTable(n, s.top_k, max(s.num_experts, 1), dev, few_rows_ok=few_ok)
        expert_out = torch.empty((table.n_pairs, s.hidden_size), dtype=torch.float32, device=dev)
        if s.num_experts > 0:
            ops.moe_group(ids, self.counts, table)
            act = torch.empty((table.n_pairs, s.expert_size), dtype=x.dtype, device=dev)
            first_epi = ops.GROUPED_GATED_CLAMP if self.gated else ops.GROUPED_RELU2
            if (x.dtype == torch.bfloat16 and table.n_pairs >= ROWS_PER_EXPERT_FOR_TENSOR_CORES * s.num_experts
                    and not torch.cuda.is_current_stream_capturing()):
                expert_out = self._experts_one_by_one(x, table, act, expert_out, weights)
            elif s.weight_on_input:
                rows = torch.empty((table.n_pairs, s.hidden_size), dtype=x.dtype, device=dev)
                ops.moe_gather(x, table, rows, weights)
                ops.grouped_gemm_routed(rows, self.w_gate_up, act, table, gather=False, epi=first_epi, limit=s.limit,
                                        alpha=s.gate_alpha)
                ops.grouped_gemm_routed(act, self.w_down, expert_out, table, gather=False, epi=ops.GROUPED_STORE_F32)
            else:
                ops.grouped_gemm_routed(x, self.w_gate_up, act, table, gather=True, epi=first_epi, limit=s.limit,
                                        alpha=s.gate_alpha)
                ops.grouped_gemm_routed(act, self.w_down, expert_out, table, gather=False, epi=ops.GROUPED_STORE_F32)
        out = residual
        if residual is None:       # the caller wants the output itself: the combine assigns, the shared expert adds
            out = torch.empty((n, s.hidden_size), dtype=torch.float32, device=dev)
        ops.moe_combine(out, expert_out, x, ids, None if s.weight_on_input else weights, table, assign=residual is None)
        if s.shared_size > 0:
            act = torch.empty((n, s.shared_size), dtype=x.dtype, device=dev)
            self._activate(linear(x, self.w_shared_gate_up), act, s.shared_limit)
            linear(act, self.w_shared_down, residual=out, track=ctx if residual is not None else None)
        return None if residual is not None else out

    def _activate(self, product, act, limit):
        if self.gated:
            ops.gated_clamp(product, act, limit, self.spec.gate_alpha)
        else:
            ops.activation(product, act, "relu2")


    def _experts_one_by_one(self, x, table, act, expert_out, weights):
        """The experts' outputs in the sorted order of pairs: ``expert_out``, or a tensor of the library's own."""
        s = self.spec
        rows = torch.empty((table.n_pairs, s.hidden_size), dtype=x.dtype, device=x.device)
        ops.moe_gather(x, table, rows, weights if s.weight_on_input else None)
        if self._library_groups and s.hidden_size % 8 == 0 and s.expert_size % 8 == 0:
            # the vendor library's grouped product: the experts' row ranges stay on the device, nothing waits
            try:
                ends = table.offsets[1:]
                gate_up = torch._grouped_mm(rows, self.w_gate_up.transpose(1, 2), offs=ends)
                self._activate(gate_up, act, s.limit)
                down = torch._grouped_mm(act, self.w_down.transpose(1, 2), offs=ends)
                ops.LAUNCHES["library"] += 2
                return down                                   # rounded to the compute dtype; the combine widens it
            except (RuntimeError, AttributeError, TypeError, NotImplementedError) as error:
                RoutedExperts._library_groups = False           # this build of the library has none: one by one
                import sys
                print(f"[ondeviceinfer_b200] no grouped product in the vendor library ({type(error).__name__}); "
                      "routed experts run one by one", file=sys.stderr)
        bounds = table.offsets.tolist()                     # waits for the device
        for e in range(s.num_experts):
            lo, hi = bounds[e], bounds[e + 1]
            if hi > lo:
                self._activate(linear(rows[lo:hi], self.w_gate_up[e]), act[lo:hi], s.limit)
                expert_out[lo:hi].copy_(linear(act[lo:hi], self.w_down[e], out_dtype=torch.float32))
        return expert_out


register_part(RoutedExpertsSpec, RoutedExperts)
