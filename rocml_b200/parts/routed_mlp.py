"""Routed feed-forward: a router and many small gated feed-forwards, of which a token uses a few.

    z = Wr h (32-bit);  s = sigmoid(z);  chosen = the ``top`` experts by s + bias;  weight_e = s_e
    expert e:  y = act(Wgate_e h, Wup_e h);  out_e = Wdown_e y
    result = sum over the chosen of weight_e * out_e

``activation`` "silu": silu(g) * u.  "clamped_swish": g = min(g, limit), u = clamp(u, -limit, limit),
g * sigmoid(alpha * g) * (u + 1).  ``choice_bias`` adds a per-expert vector to the scores for the choice
only; the weights are the scores themselves, divided by their sum over the chosen (+ ``renormalize_eps``) if
``renormalize`` says so.  ``groups`` > 1: the experts form that many equal groups of neighbours, a group's
score is the sum of its two largest scores, and only experts of the ``keep_groups`` best groups can be chosen.
``shared`` (an intermediate size): one more expert of the same form that every token uses, its result multiplied
by sigmoid(w_sg . h) (one number a token) when ``shared_gate`` says so; the gate's row rides along with the
router's rows in the 32-bit router product, and the shared result joins in the kernel that sums the choices.

How a step runs, without the host ever learning who chose what (so a decode step is one CUDA graph):
the router's product, one kernel that scores, chooses and counts, one that lays every expert's rows out
from a multiple of the row tile, one that copies each token's row to its places, two products over
tiles of those rows (every tile names its expert's weight), the activation between them, and a
weighted sum back into token order.  The row tile is 16 for few tokens and 64 beyond (mma.sync, or FMA in
32-bit); from a thousand token-choices in bfloat16 it is 128 and the two products are the persistent tcgen05
product, the first with the activation in its epilogue (the experts' gate and up rows are interleaved in
blocks of 16 at load time for that).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..config.specs import FeedForwardSpec, tensor_names
from ..errors import ConfigError
from ..profile import scope
from ..weights.decl import TensorDecl
from .base import BuildEnv, FeedForward, RoutedRows, register_feed_forward

TENSOR_NAMES = {"router": "gate", "choice_bias": "e_score_correction_bias", "expert": "experts.{e}.", "gate": "gate_proj",
                "up": "up_proj", "down": "down_proj", "shared": "shared_experts.", "shared_gate": "shared_expert_gate"}

SMALL_TILE, LARGE_TILE, TENSOR_TILE = 16, 64, 128
SMALL_TILE_MAX_ROWS = 256      # token-choices up to which the 16-row tile is used
TENSOR_TILE_MIN_ROWS = 1024    # token-choices from which tiles of 128 rows go to the tcgen05 product


@register_feed_forward("routed_mlp")
class RoutedMLP(FeedForward):
    graph_safe = True

    def __init__(self, spec: FeedForwardSpec, hidden: int, env: BuildEnv):
        p = spec.params
        self.env = env
        self.hidden = hidden
        self.experts = int(p["experts"])
        self.top = int(p["top"])
        self.inter = int(p["intermediate"])
        if not 0 < self.top <= self.experts or self.experts > 512 or self.inter <= 0:
            raise ConfigError(f"routed_mlp: {self.top} of {self.experts} experts of {self.inter} is not supported "
                              "(1 to 512 experts, at least one and at most all of them a token)")
        self.act = p.get("activation", "silu")
        if self.act not in kernels.GATED_ACTS:
            raise ConfigError(f"routed_mlp: activation {self.act!r} is not built (known: {sorted(kernels.GATED_ACTS)})")
        self.limit = float(p.get("limit", 0.0))
        self.alpha = float(p.get("alpha", 1.0))
        if self.act == "clamped_swish" and not self.limit > 0:
            raise ConfigError("routed_mlp: clamped_swish needs a positive limit")
        if p.get("score", "sigmoid") != "sigmoid":
            raise ConfigError(f"routed_mlp: score {p.get('score')!r} is not built (only 'sigmoid')")
        self.renormalize = bool(p.get("renormalize", False))
        self.renormalize_eps = float(p.get("renormalize_eps", 0.0))
        self.groups = int(p.get("groups") or 1)
        self.keep_groups = int(p.get("keep_groups") or self.groups)
        if self.groups < 1 or self.experts % self.groups or not 1 <= self.keep_groups <= self.groups or \
                self.keep_groups * (self.experts // self.groups) < self.top:
            raise ConfigError(f"routed_mlp: {self.groups} groups of which {self.keep_groups} stay do not fit "
                              f"{self.experts} experts with {self.top} chosen")
        self.has_bias = bool(p.get("choice_bias", False))
        self.shared_inter = int(p.get("shared") or 0)
        self.shared_gated = bool(p.get("shared_gate", False)) and self.shared_inter > 0
        self.shared = None
        if self.shared_inter:
            if self.act != "silu":
                raise ConfigError("routed_mlp: the shared expert is built with the 'silu' activation only")
            from ..config.specs import FeedForwardSpec
            from .mlp import GatedMLP
            names = dict(p.get("names") or ())
            self.shared = GatedMLP(FeedForwardSpec.make(
                "gated_mlp", intermediate=self.shared_inter, activation="silu", bias=False,
                names={r: names[r] for r in ("gate", "up", "down") if r in names}), hidden, env)
        try:
            self.names = tensor_names(p, TENSOR_NAMES)
        except ValueError as e:
            raise ConfigError(f"routed_mlp: {e}") from None
        self.router: Optional[torch.Tensor] = None         # float32 [experts, hidden]
        self.choice_bias: Optional[torch.Tensor] = None    # float32 [experts]
        self.gate_up: Optional[torch.Tensor] = None        # [experts, 2 * inter, hidden]: gate rows, then up rows
        self.down: Optional[torch.Tensor] = None           # [experts, hidden, inter]
        self.paired = False                                # gate and up rows alternate in blocks of 16 instead

    def _expert(self, prefix: str, e: int, role: str) -> str:
        return f"{prefix}{self.names['expert'].format(e=e)}{self.names[role]}.weight"

    def declare(self, prefix: str) -> List[TensorDecl]:
        out = [TensorDecl(f"{prefix}{self.names['router']}.weight", (self.experts, self.hidden), "matrix")]
        if self.has_bias:
            out.append(TensorDecl(f"{prefix}{self.names['choice_bias']}.weight", (self.experts,), "bias"))
        if self.shared is not None:
            out += self.shared.declare(prefix + self.names["shared"])
        if self.shared_gated:
            out.append(TensorDecl(f"{prefix}{self.names['shared']}{self.names['shared_gate']}.weight", (1, self.hidden), "matrix"))
        for e in range(self.experts):
            out += [TensorDecl(self._expert(prefix, e, "gate"), (self.inter, self.hidden), "matrix"),
                    TensorDecl(self._expert(prefix, e, "up"), (self.inter, self.hidden), "matrix"),
                    TensorDecl(self._expert(prefix, e, "down"), (self.hidden, self.inter), "matrix")]
        return out

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str) -> None:
        self.router = tensors[f"{prefix}{self.names['router']}.weight"].float().contiguous()     # the router is 32-bit
        if self.shared is not None:
            self.shared.load(tensors, prefix + self.names["shared"])
        if self.shared_gated:
            # the shared expert's gate is one more row of the router's product
            sg = tensors[f"{prefix}{self.names['shared']}{self.names['shared_gate']}.weight"].float().reshape(1, self.hidden)
            self.router = torch.cat([self.router, sg], dim=0).contiguous()
        if self.has_bias:
            self.choice_bias = tensors[f"{prefix}{self.names['choice_bias']}.weight"].float().contiguous()
        gu = [torch.cat([tensors[self._expert(prefix, e, "gate")], tensors[self._expert(prefix, e, "up")]], dim=0)
              for e in range(self.experts)]
        self.gate_up = torch.stack(gu).contiguous()
        if self.gate_up.dtype == torch.bfloat16 and self.inter % 16 == 0:
            g, u = self.gate_up[:, :self.inter], self.gate_up[:, self.inter:]
            shape = (self.experts, self.inter // 16, 16, self.hidden)
            self.gate_up = torch.stack([g.reshape(shape), u.reshape(shape)], dim=2).reshape(self.gate_up.shape).contiguous()
            self.paired = True
        self.down = torch.stack([tensors[self._expert(prefix, e, "down")] for e in range(self.experts)]).contiguous()

    def weight_bytes(self) -> int:
        """What a step reads at most: the router and the experts that can be chosen."""
        esz = 4 if self.env.mode == "float32" else 2
        shared = self.shared.weight_bytes() if self.shared is not None else 0
        return self.experts * self.hidden * 4 + self.experts * 3 * self.inter * self.hidden * esz + shared

    def _expected_experts(self, n_tokens: int) -> float:
        """The experts ``n_tokens`` tokens touch when each picks ``top`` of them at random."""
        return self.experts * (1.0 - (1.0 - self.top / self.experts) ** n_tokens)

    def _tensor_tiles(self, n_tokens: int) -> bool:
        """Whether this step's products take the tcgen05 kernel: bfloat16, enough rows, sizes it addresses."""
        return (self.paired and self.env.act_dtype == torch.bfloat16 and n_tokens * self.top >= TENSOR_TILE_MIN_ROWS
                and self.hidden % 8 == 0 and self.inter % 16 == 0 and self.inter > 32 and self.hidden > 64
                and self.gate_up is not None and self.gate_up.is_cuda)

    def _tile(self, n_tokens: int) -> int:
        if self._tensor_tiles(n_tokens):
            return TENSOR_TILE
        return SMALL_TILE if n_tokens * self.top <= SMALL_TILE_MAX_ROWS else LARGE_TILE

    def _max_tiles(self, n_tokens: int) -> int:
        """Every expert's rows start on a tile: at most one partly filled tile an expert that has rows."""
        tile = self._tile(n_tokens)
        return (n_tokens * self.top + tile - 1) // tile + min(self.experts, n_tokens * self.top)

    def workspace_bytes(self, n_tokens: int) -> int:
        esz = 4 if self.env.mode == "float32" else 2
        rows = self._max_tiles(n_tokens) * self._tile(n_tokens)
        shared = self.shared.workspace_bytes(n_tokens) if self.shared is not None else 0
        return rows * (self.hidden * (esz + 4) + self.inter * 3 * esz) + n_tokens * (self.hidden * 4 + self.experts * 4) + shared

    def cost(self, q_lens, kv_lens):
        T = sum(q_lens)
        esz = 4 if self.env.mode == "float32" else 2
        # which experts a step reads depends on its tokens; counted here: the experts T tokens touch when each
        # picks ``top`` of them at random (all of them for a prompt, a part of them for a few tokens)
        used = self._expected_experts(T)
        nbytes = self.experts * self.hidden * 4 + int(used * 3 * self.inter * self.hidden * esz)
        flops = 2 * T * self.experts * self.hidden + 2 * T * self.top * 3 * self.inter * self.hidden
        if self.shared is not None:
            sb, sf = self.shared.cost(q_lens, kv_lens)
            nbytes, flops = nbytes + sb, flops + sf
        return nbytes, flops

    sums_later = True      # forward() accepts sum_later=True and may then return RoutedRows (see parts.base)

    def forward(self, xn, batch, sum_later=False):
        T = batch.n_tokens
        dev, act = self.env.device, self.env.act_dtype
        E, top = self.experts, self.top
        tile = self._tile(T)
        max_tiles = self._max_tiles(T)
        rows = max_tiles * tile
        z = torch.empty((T, self.router.shape[0]), dtype=torch.float32, device=dev)    # E scores (+ the shared expert's gate)
        with scope(op="router"):
            kernels.router_logits(xn, self.router, z, T)
        ids = torch.empty((T, top), dtype=torch.int32, device=dev)
        place = torch.empty((T, top), dtype=torch.int32, device=dev)
        weights = torch.empty((T, top), dtype=torch.float32, device=dev)
        counts = torch.zeros((E,), dtype=torch.int32, device=dev)
        starts = torch.empty((E + 1,), dtype=torch.int32, device=dev)
        tile_group = torch.empty((max_tiles,), dtype=torch.int32, device=dev)
        row_of = torch.empty((T, top), dtype=torch.int32, device=dev)
        with scope(op="route"):
            kernels.moe_route(z, self.choice_bias, batch.slot_of_token, T, top, ids, weights, place, counts,
                              n_groups=self.groups, keep_groups=self.keep_groups, renormalize=self.renormalize,
                              norm_eps=self.renormalize_eps)
            kernels.moe_plan(counts, tile, starts, tile_group)
            xs = torch.empty((rows, self.hidden), dtype=act, device=dev)
            kernels.moe_gather(xn, ids, place, starts, T, top, xs, row_of)
        y = torch.empty((rows, self.inter), dtype=act, device=dev)
        fused = False
        told = {"used": self._expected_experts(T), "rows_used": T * top}     # for a profiler's accounts only
        if tile == TENSOR_TILE:
            with scope(op="experts_gate_up"):
                fused = kernels.tile_matmul_tc5(xs, self.gate_up, y, tile_group, self.act, self.limit, self.alpha, **told)
        if not fused and self.paired:
            # the mma.sync product has the activation in its epilogue too, when the operands take it
            with scope(op="experts_gate_up"):
                fused = kernels.tile_matmul(xs, self.gate_up, y, tile_group, tile, self.act, self.limit, self.alpha, **told)
        if not fused:
            gu = torch.empty((rows, 2 * self.inter), dtype=act, device=dev)
            with scope(op="experts_gate_up"):
                kernels.tile_matmul(xs, self.gate_up, gu, tile_group, tile, **told)
            with scope(op="experts_act"):
                kernels.gated_act(gu, y, self.act, self.limit, self.alpha, paired=self.paired)
        out_rows = torch.empty((rows, self.hidden), dtype=torch.float32, device=dev)
        with scope(op="experts_down"):
            if not (tile == TENSOR_TILE and kernels.tile_matmul_tc5(y, self.down, out_rows, tile_group, **told)):
                kernels.tile_matmul(y, self.down, out_rows, tile_group, tile, **told)
        routed = RoutedRows(out_rows, row_of, weights, top, T)
        if self.shared is not None:
            # the expert every token uses: its partial sums join where the choices are summed
            with scope(op="shared_expert"):
                extra = self.shared.forward(xn, batch)
            out = torch.empty((1, T, self.hidden), dtype=torch.float32, device=dev)
            with scope(op="experts_sum"):
                kernels.moe_combine(out_rows, row_of, weights, T, top, out[0], extra=extra,
                                    extra_gate=z[:, E] if self.shared_gated else None)
            return out
        if sum_later:
            return routed
        with scope(op="experts_sum"):
            return routed.materialize()
