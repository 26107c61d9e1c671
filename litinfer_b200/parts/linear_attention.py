"""Linear attention with a constant decay per head, as a recurrence over a state of fixed size.

q = silu(h Wq^T), k = silu(h Wk^T) ([heads, dim]), v = silu(h Wv^T) ([heads, value_dim]); per head
``S_t = decay_h S_(t-1) + k_t v_t^T`` (S is dim x value_dim, zeros before the first token) and
``o_t = S_t^T q_t``, with no other scale.  The heads side by side are normalised together (RMSNorm with
a weight), multiplied by ``sigmoid(h Wg^T)`` and mapped out.  State, decay and all sums of the
recurrence are float32; the state of a request lives in its state slot and is read and written once per
step, whatever the step holds of that request (a portion of a prompt or one token).

One product serves q | k | v | g.  The kernels find the step's sequences and their slots on the device
(``ctx.q_start``, ``ctx.state_slots``), so steps of single tokens can be replayed from a captured graph.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import MIXERS, FixedState, Mixer
from .linear import FusedLinear
from .scan import scan_chunks


@MIXERS.register("decay_linear_attention")
class DecayLinearAttention(Mixer):
    decodes_from_device = True

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["num_heads"])
        self.dim = int(spec["head_dim"])
        self.value_dim = int(spec.get("value_dim") or self.dim)
        self.eps = float(spec["eps"])
        decay = [float(x) for x in spec["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"{len(decay)} decays for {self.heads} heads")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=self.device)
        names = spec.get("names", {})
        suffixes = tuple(spec.get("suffixes", (".weight", ".bias")))
        qk, vv = self.heads * self.dim, self.heads * self.value_dim
        self.qkvg = FusedLinear(prefix, [names.get("q", "q_proj"), names.get("k", "k_proj"), names.get("v", "v_proj"), names.get("g", "g_proj")],
                                self.hidden, [qk, qk, vv, vv], False, dtype, suffixes=suffixes)
        self.out = FusedLinear(prefix, [names.get("o", "o_proj")], vv, [self.hidden], False, dtype, suffixes=suffixes)
        self.norm_name = prefix + names.get("norm", "norm.weight")
        self.norm_weight = None

    def params(self) -> List[ParamSpec]:
        return self.qkvg.params() + self.out.params() + [
            ParamSpec(self.norm_name, (self.heads * self.value_dim,), role="vector", init="ones_normal")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.qkvg.bind(tensors)
        self.out.bind(tensors)
        self.norm_weight = tensors.pop(self.norm_name)

    def cache_requirement(self):
        return FixedState((self.heads * self.dim * self.value_dim,), torch.float32)

    def forward(self, h, ctx, cache):
        T = h.shape[0]
        qk, vv = self.heads * self.dim, self.heads * self.value_dim
        proj = self.qkvg(h)
        o32 = torch.empty((T, vv), dtype=torch.float32, device=h.device)
        K.decay_scan(proj, 0, qk, 2 * qk, self.decay, cache.state, ctx.q_start, ctx.state_slots, o32, self.heads, self.dim, self.value_dim, chunks=scan_chunks(ctx))
        y = torch.empty((T, vv), dtype=self.dtype, device=h.device)
        K.gated_rmsnorm(o32, proj, 2 * qk + vv, self.norm_weight, self.eps, 1, False, y)
        return self.out(y)
