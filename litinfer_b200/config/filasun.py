"""Configuration of the Filasun decoder, read from config.json.

config.json names the design under ``architecture`` and lists the layers one by one: each entry gives its
``type`` (which mixer it has), the mixer's sizes (``mixer``) and its feed-forward (``mlp``, or null for none).
Model-wide keys: ``vocab``, ``width``, ``max_positions`` (rows of the learned position table), ``streams`` (residual
streams of the hyper-connections), ``norm.eps``, ``logit_softcap``.

Layer types:

* ``parallel``: two mixers side by side on the same input, summed with ``left_scale`` and ``right_scale``.
  ``left`` is softmax attention over a sliding window (``mask.size`` positions, the query's own included) with grouped
  key/value heads, biases on q, k, v and the output map, no rotation, scores scaled by ``scale``, capped by
  ``softcap * tanh(s / softcap)`` and lowered by ``slope_h * distance`` with ``slope_h = 2^(-8 (h + 1) / heads)``, and one
  sigmoid gate per head.  ``right`` is linear attention with one constant ``decay`` per head.
* ``mamba2``: a selective state-space mixer (``heads``, ``vdim``, ``state``, ``groups``, ``conv`` taps, ``norm_groups``).

The feed-forward (``kind`` dense) is a gated unit whose operands are bounded by ``limit``.  Tensor names follow the
file: ``l<i>.`` per layer, ``mix.`` / ``mlp.`` / ``norm1`` / ``norm2`` / ``hc1.`` / ``hc2.`` below it, weights under the bare stem
and biases under ``<stem>.b``.  Sizes and constants all come from config.json; what the design fixes (the slopes'
rule, the activation's 1.702) is written here.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .qwen2 import ConfigError
from .spec import BlockSpec, ModelSpec, PartSpec, default_schedule

SUFFIXES = ("", ".b")             # a weight is stored under its stem, a bias under stem + ".b"
GLU_ALPHA = 1.702


def _int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}'{key}' must be a positive integer, got {v!r}")
    return v


def _float(d: Mapping[str, Any], key: str, where: str, default: Optional[float] = None) -> float:
    v = d.get(key, default)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {v!r}")
    return float(v)


def distance_slopes(heads: int) -> Tuple[float, ...]:
    """The penalty per position of distance for head h of ``heads``: 2^(-8 (h + 1) / heads)."""
    return tuple(2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads))


@dataclass(frozen=True)
class FilasunConfig:
    vocab: int
    width: int
    max_positions: int
    streams: int
    eps: float
    logit_softcap: Optional[float]
    layers: Tuple[Mapping[str, Any], ...]

    ARCHITECTURE = "Filasun"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "FilasunConfig":
        norm = d.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("config.json: missing key 'norm' (with 'eps')")
        eps = _float(norm, "eps", "norm.")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        cap = d.get("logit_softcap")
        cfg = cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""), max_positions=_int(d, "max_positions", ""),
                  streams=_int(d, "streams", "") if d.get("streams") is not None else 1, eps=eps,
                  logit_softcap=None if cap is None else _float(d, "logit_softcap", ""), layers=tuple(layers))
        cfg.to_model_spec()                       # every layer's keys are read (and refused) here, not at the first step
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
               "streams": self.streams, "norm": {"eps": self.eps}, "layers": [dict(x) for x in self.layers]}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out

    # ------------------------------------------------------------------
    def _window_attention(self, m: Mapping[str, Any], where: str) -> PartSpec:
        heads = _int(m, "heads", where)
        kv = _int(m, "kv_heads", where) if m.get("kv_heads") is not None else heads
        if heads % kv:
            raise ConfigError(f"config.json: {where}{heads} heads are not a multiple of {kv} key/value heads")
        mask = m.get("mask")
        window = _int(mask, "size", where + "mask.") if isinstance(mask, Mapping) else None
        dim = _int(m, "dim", where)
        return PartSpec("attention", {
            "hidden_size": self.width, "num_heads": heads, "num_kv_heads": kv, "head_dim": dim,
            "value_dim": _int(m, "vdim", where) if m.get("vdim") is not None else dim,
            "scale": _float(m, "scale", where, 1.0 / math.sqrt(dim)), "window": window,
            "softcap": _float(m, "softcap", where) if m.get("softcap") is not None else None,
            "distance_slopes": distance_slopes(heads), "head_gate": "g", "qkv_bias": True, "out_bias": True, "position": None,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o"}, "suffixes": SUFFIXES})

    def _decay_attention(self, m: Mapping[str, Any], where: str) -> PartSpec:
        heads = _int(m, "heads", where)
        decay = m.get("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != heads:
            raise ConfigError(f"config.json: {where}'decay' must list one number per head ({heads})")
        dim = _int(m, "dim", where)
        return PartSpec("decay_linear_attention", {
            "hidden_size": self.width, "num_heads": heads, "head_dim": dim,
            "value_dim": _int(m, "vdim", where) if m.get("vdim") is not None else dim,
            "decay": tuple(float(x) for x in decay), "eps": self.eps,
            "names": {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}, "suffixes": SUFFIXES})

    def _mixer(self, layer: Mapping[str, Any], where: str) -> PartSpec:
        kind, m = layer.get("type"), layer.get("mixer")
        if not isinstance(m, Mapping):
            raise ConfigError(f"config.json: {where}'mixer' is missing")
        if kind == "parallel":
            for side in ("left", "right"):
                if not isinstance(m.get(side), Mapping):
                    raise ConfigError(f"config.json: {where}mixer.'{side}' is missing")
            return PartSpec("parallel", {
                "left": self._window_attention(m["left"], where + "mixer.left."),
                "right": self._decay_attention(m["right"], where + "mixer.right."),
                "left_scale": _float(m, "left_scale", where + "mixer.", 1.0), "right_scale": _float(m, "right_scale", where + "mixer.", 1.0)})
        if kind == "mamba2":
            w = where + "mixer."
            return PartSpec("selective_ssm", {
                "hidden_size": self.width, "num_heads": _int(m, "heads", w), "head_dim": _int(m, "vdim", w), "state_size": _int(m, "state", w),
                "groups": _int(m, "groups", w) if m.get("groups") is not None else 1, "conv": _int(m, "conv", w),
                "norm_groups": _int(m, "norm_groups", w) if m.get("norm_groups") is not None else 1, "eps": self.eps,
                "names": {"in": "in", "o": "o", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D",
                          "norm": "norm"}, "suffixes": SUFFIXES})
        raise ConfigError(f"config.json: {where}layer type {kind!r} is not supported (parallel, mamba2)")

    def _feed_forward(self, layer: Mapping[str, Any], where: str) -> Optional[PartSpec]:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
            raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} is not supported (dense)")
        return PartSpec("clamped_glu", {"hidden_size": self.width, "intermediate_size": _int(mlp, "ff", where + "mlp."),
                                        "limit": _float(mlp, "limit", where + "mlp."), "alpha": GLU_ALPHA,
                                        "names": {"gate": "gate", "up": "up", "down": "down"}, "suffixes": SUFFIXES})

    def to_model_spec(self) -> ModelSpec:
        def norm(tensor):
            return PartSpec("rmsnorm", {"size": self.width, "eps": self.eps, "tensor": tensor})

        blocks = []
        for i, layer in enumerate(self.layers):
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            where = f"layers[{i}]."
            ff = self._feed_forward(layer, where)
            blocks.append(BlockSpec.of(
                "hyper_prenorm", f"l{i}.",
                prefixes={"mixer": "mix.", "feed_forward": "mlp.", "mixer_norm": "", "feed_forward_norm": "", "mixer_connection": "hc1.",
                          "feed_forward_connection": "hc2."},
                mixer=self._mixer(layer, where), feed_forward=ff, mixer_norm=norm("norm1"), feed_forward_norm=norm("norm2") if ff else None,
                connections=PartSpec("hyper_connections", {"streams": self.streams})))
        return ModelSpec(
            architecture=self.ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks),
            schedule=default_schedule(len(blocks)), final_norm=norm("norm"), tie_word_embeddings=False,
            max_position_embeddings=self.max_positions, embedding_name="embed", final_norm_prefix="final.", lm_head_name="head",
            position=PartSpec("learned", {"positions": self.max_positions, "size": self.width, "tensor": "pos"}), position_prefix="",
            logit_cap=self.logit_softcap, streams=self.streams)
