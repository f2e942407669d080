"""Linear attention with a fixed decay per head: a running sum in place of a softmax over all keys.

    q = aq(Wq h), k = aq(Wk h) * c_k   [heads, head_dim]       aq, av: nothing or silu
    v = av(Wv h)                        [heads, v_head_dim]
    S_t = d_n S_(t-1) + k_t v_t^T       per head n, S [head_dim, v_head_dim], zero when the sequence starts
    o_t = S_t^T q_t
    out = Wo (norm(o) * ag(Wg h))       norm: o over its root mean square, per head or over all heads
                                        together, with or without a weight vector; ag: silu or sigmoid

What a sequence keeps is the state alone (``StateRequirement``: [heads, head_dim, v_head_dim] in 32-bit),
whatever its length.  One stacked product makes q | k | v | gate from the layer's input; one kernel
carries the step's tokens through the recurrence token after token (single tokens and short pieces), or three
kernels do the same by blocks of 64 tokens that run side by side (prompts), both from the state the step before
left; one kernel normalises and gates; the output product is the one
every mixer uses.  From the projections on everything is 32-bit: decays, state, sums, the norm, the gate.
Two designs differ only in the parameters: lightning attention (silu on q, k, v; one norm with a weight over
all heads; sigmoid gate) and retention (no activation; k / sqrt(head_dim); a norm per head without weight;
silu gate).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..cache.requirements import StateRequirement
from ..config.specs import MixerSpec, tensor_names
from ..errors import ConfigError
from ..profile import scope
from ..weights.decl import TensorDecl
from .base import BuildEnv, DeferredNorm, Mixer, register_mixer
from .linear import Linear

TENSOR_NAMES = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "gate": "g_proj", "o": "o_proj", "out_norm": "out_norm"}

# A step whose longest sequence brings more tokens than this runs the recurrence by blocks of 64 tokens side by side
# (three kernels); up to it, token after token in one kernel (also every decode step).
BLOCKS_MIN_TOKENS = 16


@register_mixer("linear_attention")
class LinearAttention(Mixer):
    graph_safe = True

    def __init__(self, spec: MixerSpec, hidden: int, env: BuildEnv):
        p = spec.params
        self.env = env
        self.hidden = hidden
        self.heads = int(p["n_heads"])
        self.hd = int(p["head_dim"])
        self.vd = int(p.get("v_head_dim") or self.hd)
        if min(self.heads, self.hd, self.vd) <= 0:
            raise ConfigError("linear attention: heads and head sizes must be positive")
        decay = [float(d) for d in p["decay"]]
        if len(decay) != self.heads or not all(0.0 <= d <= 1.0 for d in decay):
            raise ConfigError(f"linear attention: {self.heads} heads need {self.heads} decays in [0, 1], found {decay}")
        self.decay_values = decay
        self.qk_act = p.get("qk_activation", "none")
        self.v_act = p.get("v_activation", "none")
        self.gate_act = p.get("gate_activation", "sigmoid")
        if self.qk_act not in ("none", "silu") or self.v_act not in ("none", "silu") or self.gate_act not in ("silu", "sigmoid"):
            raise ConfigError("linear attention: activations are 'none' or 'silu' (q, k, v) and 'silu' or 'sigmoid' (gate)")
        self.k_scale = float(p.get("k_scale", 1.0))
        self.out_norm = p.get("out_norm", "per_head")
        if self.out_norm not in ("per_head", "all_heads"):
            raise ConfigError(f"linear attention: out_norm {self.out_norm!r} is unknown (per_head, all_heads)")
        self.norm_eps = float(p.get("out_norm_eps", 1e-6))
        self.norm_has_weight = bool(p.get("out_norm_weight", False))
        if spec.position.kind != "none":
            raise ConfigError("linear attention: a position encoding inside the mixer is not built")
        try:
            self.names = n = tensor_names(p, TENSOR_NAMES)
        except ValueError as e:
            raise ConfigError(f"linear attention: {e}") from None
        qk, vw = self.heads * self.hd, self.heads * self.vd
        self.offsets = (0, qk, 2 * qk, 2 * qk + vw)          # q | k | v | gate
        self.proj = Linear([n["q"], n["k"], n["v"], n["gate"]], [qk, qk, vw, vw], hidden, False, env)
        self.o = Linear([n["o"]], [hidden], vw, False, env)
        self.norm_w: Optional[torch.Tensor] = None
        self.decay = torch.tensor(decay, dtype=torch.float32, device=env.device)

    def cache_requirement(self):
        return StateRequirement((self.heads, self.hd, self.vd), torch.float32)

    def declare(self, prefix: str) -> List[TensorDecl]:
        out = self.proj.declare(prefix) + self.o.declare(prefix)
        if self.norm_has_weight:
            out.append(TensorDecl(f"{prefix}{self.names['out_norm']}.weight", (self.heads * self.vd,), "norm"))
        return out

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str) -> None:
        self.proj.load(tensors, prefix)
        self.proj.pad_rows(8)
        self.o.load(tensors, prefix)
        if self.norm_has_weight:
            self.norm_w = tensors[f"{prefix}{self.names['out_norm']}.weight"].contiguous()

    def weight_bytes(self) -> int:
        return self.proj.weight_bytes() + self.o.weight_bytes()

    def workspace_bytes(self, n_tokens: int) -> int:
        esz = 4 if self.env.mode == "float32" else 2
        parts = 8 if n_tokens <= 128 else 1
        vw = self.heads * self.vd
        blocks = (n_tokens // 64 + 8) * self.heads * self.hd * self.vd * 4 if n_tokens > BLOCKS_MIN_TOKENS else 0
        return n_tokens * (self.proj.n * max(esz, 4 * parts if parts > 1 else esz) + vw * (4 + esz) + self.hidden * 4 * parts) + blocks

    def cost(self, q_lens, kv_lens):
        from ..profile import cost as C
        T = sum(q_lens)
        esz = 4 if self.env.mode == "float32" else 2
        live = sum(1 for n in q_lens if n > 0)
        parts = [self.proj.cost(T), self.o.cost(T), C.decay_scan(T, live, self.heads, self.hd, self.vd, 1, esz)]
        return sum(p[0] for p in parts), sum(p[1] for p in parts)

    can_add_into = True    # forward() accepts add_into=residual (see parts.base)

    def forward(self, xn, batch, view, add_into=None):
        T = batch.n_tokens
        dev, act = self.env.device, self.env.act_dtype
        if isinstance(xn, DeferredNorm):
            xn = xn.materialize()
        proj = self.proj.forward_auto(xn, T)          # [T, N] in the activations' type, or [S, T, N] float32 partial sums
        vw = self.heads * self.vd
        q_off, k_off, v_off, g_off = self.offsets
        o = torch.empty((T, vw), dtype=torch.float32, device=dev)
        with scope(op="decay_scan"):
            done = False
            if not batch.is_decode and batch.max_q_len > BLOCKS_MIN_TOKENS and max(self.hd, self.vd) <= kernels.DECAY_BLOCKS_MAX_HEAD:
                # prompts: blocks of 64 tokens side by side instead of one token after another
                work = torch.empty((T // kernels.DECAY_BLOCK + batch.n_seqs, self.heads, self.hd, self.vd),
                                   dtype=torch.float32, device=dev)
                done = kernels.decay_scan_blocks(proj, T, q_off, k_off, v_off, self.heads, self.hd, self.vd, self.qk_act,
                                                 self.v_act, self.k_scale, self.decay, view.state, batch.seq_slot,
                                                 batch.cu_q, batch.n_seqs, o, work)
            if not done:
                kernels.decay_scan(proj, T, q_off, k_off, v_off, self.heads, self.hd, self.vd, self.qk_act, self.v_act,
                                   self.k_scale, self.decay, view.state, batch.seq_slot, batch.cu_q, batch.n_seqs, o,
                                   one_token_each=batch.is_decode)
        y = torch.empty((T, vw), dtype=act, device=dev)
        with scope(op="out_norm_gate"):
            kernels.group_norm_gate(o, proj, g_off, self.norm_w, self.norm_eps,
                                    self.heads if self.out_norm == "per_head" else 1, self.gate_act, y,
                                    batch.slot_of_token, T)
        if add_into is not None and self.o.forward_add(y, T, add_into):
            return None
        return self.o.forward_delta(y, T)
