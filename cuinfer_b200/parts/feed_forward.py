"""Dense SiLU-gated feed-forward: ``down( silu(gate(x)) · up(x) )``, no biases.

The reference stacks gate and up into one ``[2I, H]`` projection, gate first, applies
``g·u / (1 + exp(−g))`` in 32 bits and projects down (csrc/model/layers/mlp.cpp:8-27;
csrc/ops/swiglu.cu:23-32).  Spec: ``PartSpec("swiglu", intermediate_size=I)``.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from .base import FeedForward
from .context import StepContext
from .linear import Linear
from .registry import FEED_FORWARDS
from .spec import PartSpec, TensorSpec


@FEED_FORWARDS.register("swiglu")
@FEED_FORWARDS.register("gated")
class SwiGLU(FeedForward):
    """``down( act(gate(x)) * up(x) )``.  Kind ``swiglu`` is the SiLU-gated form above; kind ``gated`` takes
    ``activation`` (``"silu"`` or ``"gelu_tanh"``, the tanh form of GELU) and the tensors' names relative to the part's
    prefix: ``PartSpec("gated", intermediate_size=I, activation="gelu_tanh", names=(gate, up, down))``."""

    accepts_lazy_norm = True       # the gate/up projection can compute the norm of its input itself

    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.intermediate_size = int(spec.intermediate_size)
        self.activation = spec.get("activation", "silu")
        if self.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"gated feed-forward: activation {self.activation!r} is not silu or gelu_tanh")
        self._pair = True if self.activation == "silu" else self.activation        # what the projection's epilogue is told
        gate, up, down = spec.get("names", ("gate_proj.weight", "up_proj.weight", "down_proj.weight"))
        p = prefix
        self.gate_up = Linear([f"{p}.{gate}", f"{p}.{up}"],
                              [self.intermediate_size, self.intermediate_size], hidden_size, dtype)
        self.down = Linear([f"{p}.{down}"], [hidden_size], self.intermediate_size, dtype)

    def tensors(self) -> List[TensorSpec]:
        return self.gate_up.tensors() + self.down.tensors()

    def load(self, store) -> None:
        self.gate_up.load(store)
        self.down.load(store)
        self.gate_up.warm_next = self.down.weight

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.gate_up.weight

    def warm_after(self, weight: Optional[torch.Tensor]) -> None:
        self.down.warm_next = weight

    def workspace_bytes(self, tokens: int) -> int:
        return self.gate_up.workspace_bytes(tokens, silu_pair=True) + self.down.workspace_bytes(tokens)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = self.gate_up.forward(x, silu_pair=self._pair)       # act(gate) * up, fused where the kernel allows
        return self.down.forward(act)


@FEED_FORWARDS.register("none")
class NoFeedForward(FeedForward):
    """A layer without a feed-forward sub-layer; a block that sees ``absent`` leaves the sub-layer and its norms out."""

    absent = True

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise RuntimeError("a layer without feed-forward has nothing to run")


@FEED_FORWARDS.register("relu2")
class SquaredReluFeedForward(FeedForward):
    """``down( relu(up(x)) ** 2 )``, no gate, no biases.  Spec: ``PartSpec("relu2", intermediate_size=I,
    names=(up, down))`` with tensor names relative to the part's prefix."""

    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.intermediate_size = int(spec.intermediate_size)
        up, down = spec.get("names", ("up_proj.weight", "down_proj.weight"))
        self.up = Linear([f"{prefix}.{up}"], [self.intermediate_size], hidden_size, dtype)
        self.down = Linear([f"{prefix}.{down}"], [hidden_size], self.intermediate_size, dtype)

    def tensors(self) -> List[TensorSpec]:
        return self.up.tensors() + self.down.tensors()

    def load(self, store) -> None:
        self.up.load(store)
        self.down.load(store)
        self.up.warm_next = self.down.weight

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.up.weight

    def warm_after(self, weight: Optional[torch.Tensor]) -> None:
        self.down.warm_next = weight

    def workspace_bytes(self, tokens: int) -> int:
        return 2 * self.up.workspace_bytes(tokens) + self.down.workspace_bytes(tokens)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        y = self.up.forward(x)
        act = torch.empty_like(y)
        kernels.relu_squared(y, act)
        return self.down.forward(act)


@FEED_FORWARDS.register("gelu_tanh")
class GeluFeedForward(SquaredReluFeedForward):
    """``down( gelu_tanh(up(x)) )`` with the tanh form of GELU, no gate, no biases.  Spec: ``PartSpec("gelu_tanh",
    intermediate_size=I, names=(up, down))``."""

    accepts_lazy_norm = True       # the up projection can compute the norm of its input itself

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        y = self.up.forward(x)
        act = torch.empty_like(y)
        kernels.gelu_tanh(y, act)
        return self.down.forward(act)


@FEED_FORWARDS.register("moe_table")
class TableRoutedExperts(FeedForward):
    """A mixture of SiLU-gated experts without a router: an integer table ``[vocab, top]`` names, for every token id,
    the ``top`` experts of a token carrying that id; each has weight ``1 / top``.  An optional shared expert of the same
    form (size ``shared_size``) runs for every token and is added.

    Spec: ``PartSpec("moe_table", experts=E, top=k, intermediate_size=I, vocab_size=V, shared_size=S or 0,
    expert_names="e{}.gate|e{}.up|e{}.down", table_name="table", shared_names=("shared.gate", "shared.up", "shared.down"))``.
    The experts' matrices are stacked at load: gate and up rows of expert e side by side in ``[E, 2I, H]``, down in
    ``[E, H, I]``."""

    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.experts = int(spec.experts)
        self.top = int(spec.top)
        self.intermediate_size = int(spec.intermediate_size)
        self.vocab_size = int(spec.vocab_size)
        self.shared_size = int(spec.get("shared_size", 0) or 0)
        if not 0 < self.top <= self.experts:
            raise ValueError(f"moe_table: top={self.top} of {self.experts} experts")
        gate, up, down = spec.get("expert_names", ("e{}.gate", "e{}.up", "e{}.down"))
        p = prefix
        self._gate_up_specs = [TensorSpec(f"{p}.{n.format(e)}", (self.intermediate_size, hidden_size))
                               for e in range(self.experts) for n in (gate, up)]
        self._down_specs = [TensorSpec(f"{p}.{down.format(e)}", (hidden_size, self.intermediate_size)) for e in range(self.experts)]
        self._table_spec = TensorSpec(f"{p}.{spec.get('table_name', 'table')}", (self.vocab_size, self.top), integer=True,
                                      modulus=self.experts)
        self.shared: Optional[SwiGLU] = None
        if self.shared_size:
            sg, su, sd = spec.get("shared_names", ("shared.gate", "shared.up", "shared.down"))
            self.shared_gate_up = Linear([f"{p}.{sg}", f"{p}.{su}"], [self.shared_size, self.shared_size], hidden_size, dtype)
            self.shared_down = Linear([f"{p}.{sd}"], [hidden_size], self.shared_size, dtype)
        self.gate_up: Optional[torch.Tensor] = None
        self.down: Optional[torch.Tensor] = None
        self.table: Optional[torch.Tensor] = None

    def tensors(self) -> List[TensorSpec]:
        out = self._gate_up_specs + self._down_specs + [self._table_spec]
        if self.shared_size:
            out += self.shared_gate_up.tensors() + self.shared_down.tensors()
        return out

    def load(self, store) -> None:
        E, I, H = self.experts, self.intermediate_size, self.hidden_size
        self.gate_up = store.get_stacked(self._gate_up_specs).to(self.dtype).view(E, 2 * I, H)
        self.down = store.get_stacked(self._down_specs).to(self.dtype).view(E, H, I)
        self.table = store.get(self._table_spec).to(torch.int32).contiguous()
        if self.shared_size:
            self.shared_gate_up.load(store)
            self.shared_down.load(store)

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.shared_gate_up.weight if self.shared_size else None

    def workspace_bytes(self, tokens: int) -> int:
        width = 2 if self.dtype == torch.bfloat16 else 4
        own = tokens * (self.top * (self.intermediate_size + self.hidden_size) + self.hidden_size) * width + tokens * self.top * 16
        if self.shared_size:
            own += self.shared_gate_up.workspace_bytes(tokens, silu_pair=True) + self.shared_down.workspace_bytes(tokens)
        return own

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        base = None
        if self.shared_size:
            base = self.shared_down.forward(self.shared_gate_up.forward(x, silu_pair=True))
        out = torch.empty((x.shape[0], self.hidden_size), dtype=x.dtype, device=x.device)
        kernels.moe_table_feed_forward(x, ctx.token_ids, self.table, self.gate_up, self.down, base, out)
        return out


@FEED_FORWARDS.register("moe_routed")
class RoutedExperts(FeedForward):
    """A mixture of experts chosen by a router from its logits ``z = R h`` (32 bits); the output is the weighted sum of
    the chosen experts, plus an optional shared expert that runs for every token.

    The choice and the weights (``score``):

    * ``"softmax_chosen"`` (default): the ``top`` largest logits win and their weights are the softmax over the chosen
      logits only;
    * ``"sigmoid"``: scores ``s = sigmoid(z)``; the choice goes by ``s + correction`` (a learned number per expert,
      tensor ``correction_name``; None: no correction) among the ``groups = (count, keep)`` best groups — the experts form
      ``count`` equal groups of neighbours, a group's mark is the sum of its two largest choice scores, and only experts
      of the ``keep`` best groups can be chosen; the weights are the chosen experts' ``s`` times ``route_scale``, not
      renormalised.

    An expert (``activation``), no biases: ``"silu"``: ``down(silu(gate h) * up h)``; ``"clamped"`` with ``limit`` L:
    ``g = min(gate h, L), u = clamp(up h, -L, L)``, ``down(g * sigmoid(1.702 g) * (u + 1))``; ``"relu2"``: no gate,
    ``down(relu(up h) ** 2)`` (``expert_names`` then has two names).

    ``shared_size`` S > 0: one more expert of the mixture's form with S inner values (``shared_names``) runs for every
    token and is added, multiplied by ``sigmoid(g . h)`` when ``shared_gate_name`` names a row ``[1, W]``.

    Spec: ``PartSpec("moe_routed", experts=E, top=k, intermediate_size=I, activation, limit, score, correction_name, groups,
    route_scale, router_name="router", expert_names=("e{}.gate", "e{}.up", "e{}.down"), shared_size, shared_names,
    shared_gate_name)``.  The experts' matrices are stacked at load as for the table-routed mixture, whose kernels run
    the experts here too (rows by token and choice for few rows, grouped by expert on the tensor cores for many)."""

    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.experts, self.top, self.intermediate_size = int(spec.experts), int(spec.top), int(spec.intermediate_size)
        if not 0 < self.top <= self.experts:
            raise ValueError(f"moe_routed: top={self.top} of {self.experts} experts")
        self.activation = spec.get("activation", "silu")
        if self.activation not in ("silu", "clamped", "relu2"):
            raise ValueError(f"moe_routed: activation {self.activation!r} is not silu, clamped or relu2")
        self.gated = self.activation != "relu2"
        self.limit = float(spec.limit) if self.activation == "clamped" else None
        self.score = spec.get("score", "softmax_chosen")
        if self.score not in ("softmax_chosen", "sigmoid"):
            raise ValueError(f"moe_routed: score {self.score!r} is not softmax_chosen or sigmoid")
        groups = spec.get("groups") or (1, 1)
        self.groups, self.keep = int(groups[0]), int(groups[1])
        self.route_scale = float(spec.get("route_scale", 1.0))
        if self.score == "sigmoid":
            if self.groups <= 0 or self.experts % self.groups or not 0 < self.keep <= self.groups:
                raise ValueError(f"moe_routed: {self.groups} groups ({self.keep} kept) of {self.experts} experts")
            if self.keep * (self.experts // self.groups) < self.top:
                raise ValueError(f"moe_routed: {self.keep} groups of {self.experts // self.groups} experts cannot give {self.top}")
        elif (self.groups, self.keep) != (1, 1) or spec.get("correction_name") or self.route_scale != 1.0:
            raise ValueError("moe_routed: groups, a correction and a scale belong to score='sigmoid'")
        p = prefix
        names = spec.get("expert_names", ("e{}.gate", "e{}.up", "e{}.down") if self.gated else ("e{}.up", "e{}.down"))
        if len(names) != (3 if self.gated else 2):
            raise ValueError(f"moe_routed: activation {self.activation!r} takes {3 if self.gated else 2} expert names")
        first, down = names[:-1], names[-1]
        self._gate_up_specs = [TensorSpec(f"{p}.{n.format(e)}", (self.intermediate_size, hidden_size))
                               for e in range(self.experts) for n in first]
        self._down_specs = [TensorSpec(f"{p}.{down.format(e)}", (hidden_size, self.intermediate_size)) for e in range(self.experts)]
        correction = spec.get("correction_name")
        self._correction_spec = TensorSpec(f"{p}.{correction}", (self.experts,), keep_stored_precision=True, init="zeros") if correction else None
        # the router's rows and the shared expert's gate row are one stacked projection with 32-bit output
        self.shared_size = int(spec.get("shared_size", 0) or 0)
        gate_name = spec.get("shared_gate_name") if self.shared_size else None
        self.has_shared_gate = bool(gate_name)
        router_names = [f"{p}.{spec.get('router_name', 'router')}"] + ([f"{p}.{gate_name}"] if gate_name else [])
        self.router = Linear(router_names, [self.experts] + ([1] if gate_name else []), hidden_size, dtype)
        self.shared_first: Optional[Linear] = None
        self.shared_down: Optional[Linear] = None
        if self.shared_size:
            shared = spec.get("shared_names", ("shared.gate", "shared.up", "shared.down") if self.gated else ("shared.up", "shared.down"))
            if len(shared) != len(names):
                raise ValueError("moe_routed: the shared expert has the experts' form, and as many names")
            self.shared_first = Linear([f"{p}.{n}" for n in shared[:-1]], [self.shared_size] * (len(shared) - 1), hidden_size, dtype)
            self.shared_down = Linear([f"{p}.{shared[-1]}"], [hidden_size], self.shared_size, dtype)
            if self.activation == "clamped":
                raise ValueError("moe_routed: a shared expert with the clamped gate is not built")
        self.gate_up: Optional[torch.Tensor] = None
        self.down: Optional[torch.Tensor] = None
        self.correction: Optional[torch.Tensor] = None

    def tensors(self) -> List[TensorSpec]:
        out = self._gate_up_specs + self._down_specs + self.router.tensors()
        if self._correction_spec is not None:
            out = out + [self._correction_spec]
        if self.shared_size:
            out = out + self.shared_first.tensors() + self.shared_down.tensors()
        return out

    def load(self, store) -> None:
        E, I, H = self.experts, self.intermediate_size, self.hidden_size
        self.gate_up = store.get_stacked(self._gate_up_specs).to(self.dtype).view(E, (2 if self.gated else 1) * I, H)
        self.down = store.get_stacked(self._down_specs).to(self.dtype).view(E, H, I)
        self.router.load(store)
        rows = self.router.weight.shape[0]
        if rows % 8:
            # rows of zeros up to a multiple of eight: the product then takes the tensor-core and library paths that the
            # other projections take (nothing reads the columns they produce)
            pad = torch.zeros((8 - rows % 8, self.hidden_size), dtype=self.router.weight.dtype, device=self.router.weight.device)
            self.router.weight = torch.cat([self.router.weight, pad]).contiguous()
        if self._correction_spec is not None:
            self.correction = store.get(self._correction_spec).float().contiguous()
        if self.shared_size:
            self.shared_first.load(store)
            self.shared_down.load(store)

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.router.weight

    def workspace_bytes(self, tokens: int) -> int:
        width = 2 if self.dtype == torch.bfloat16 else 4
        own = (tokens * (self.top * (self.intermediate_size + self.hidden_size) + self.hidden_size) * width
               + tokens * (self.top * 24 + (self.experts + 1) * 4))
        if self.shared_size:
            own += 2 * self.shared_first.workspace_bytes(tokens) + self.shared_down.workspace_bytes(tokens)
        return own

    def _shared(self, x: torch.Tensor) -> torch.Tensor:
        if self.activation == "relu2":
            y = self.shared_first.forward(x)
            act = torch.empty_like(y)
            kernels.relu_squared(y, act)
        else:
            act = self.shared_first.forward(x, silu_pair=True)
        return self.shared_down.forward(act)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T = x.shape[0]
        routed = self.router.forward(x, out_dtype=torch.float32)              # [T, E (+ 1: the shared expert's gate)]
        logits = routed[:, :self.experts]
        choice = torch.empty((T, self.top), dtype=torch.int32, device=x.device)
        weight = torch.empty((T, self.top), dtype=torch.float32, device=x.device)
        if self.score == "sigmoid":
            kernels.router_scored_topk(logits, self.top, choice, weight, correction=self.correction, groups=self.groups,
                                       keep=self.keep, scale=self.route_scale)
        else:
            kernels.router_topk(logits, self.top, choice, weight)
        base = self._shared(x) if self.shared_size else None
        base_gate = routed[:, self.experts] if self.has_shared_gate else None
        out = torch.empty((T, self.hidden_size), dtype=x.dtype, device=x.device)
        kernels.moe_table_feed_forward(x, None, choice, self.gate_up, self.down, base, out, weights=weight,
                                       clamp_limit=self.limit, activation="relu2" if self.activation == "relu2" else None,
                                       base_gate=base_gate)
        return out
