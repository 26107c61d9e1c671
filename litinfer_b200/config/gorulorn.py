"""Configuration of the Gorulorn decoder, read from config.json.

config.json names the design under ``architecture`` and lists the layers one by one: each entry gives its ``type``
(which mixer it has), the mixer's sizes (``mixer``) and its feed-forward (``mlp``, or null for none).  Model-wide keys:
``vocab``, ``width``, ``norm.eps``, and ``loop`` (``start``, ``stop``, ``times``): the layers start .. stop - 1 run
``times`` times in a row with the same weights, each pass with a cache of its own, and row t of the tensor ``loop.step``
is added to the residual stream right before pass t.

Every sublayer stands between two layer norms (weight, no bias): ``x += norm_b(sublayer(norm(x)))``.

Layer types:

* ``attention``: grouped-query softmax attention with biased projections, a short causal convolution on every channel
  of q, k and v (``conv`` taps), an RMS norm per head on queries and keys, rotation of the first ``rot.dims`` elements of
  each head (base ``rot.base``), scores scaled by ``scale``, a sliding window of ``mask.size`` positions that also
  keeps the first ``mask.keep_first`` tokens visible.
* ``latent_attention``: queries through a latent of ``q_rank``, keys and values from one cached latent of ``kv_rank``
  per token, no positions, a window of ``mask.size`` positions, a learned sink per head in the softmax's denominator.

The feed-forward (``kind`` moe) is a mixture of ``router.experts`` gated units of width ``expert.ff``, ``router.top`` of
them per token, chosen by the largest sigmoid scores; the scores weigh the experts' inputs and are not renormalised.

Tensor names follow the file: ``l<i>.`` per layer, ``mix.`` / ``mlp.`` / ``norm1`` / ``norm1b`` / ``norm2`` / ``norm2b``
below it, weights under the bare stem and biases under ``<stem>.b``.  Sizes and constants all come from config.json.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .filasun import _float, _int
from .qwen2 import ConfigError
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry

SUFFIXES = ("", ".b")             # a weight is stored under its stem, a bias under stem + ".b"
LOOP_TABLE = "loop.step"
# a model of this design has no position limit of its own (rotation and windows work at any position); the engine sizes
# its default cache and block tables by this, and config.json may say otherwise with 'max_positions'
MAX_POSITIONS = 32768


def _opt_int(d: Mapping[str, Any], key: str, where: str) -> Optional[int]:
    return _int(d, key, where) if d.get(key) is not None else None


@dataclass(frozen=True)
class GorulornConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[Mapping[str, Any], ...]
    loop: Optional[Tuple[int, int, int]]            # (start, stop, times)
    max_positions: int = MAX_POSITIONS

    ARCHITECTURE = "Gorulorn"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "GorulornConfig":
        norm = d.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("config.json: missing key 'norm' (with 'eps')")
        eps = _float(norm, "eps", "norm.")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        loop = d.get("loop")
        if loop is not None:
            if not isinstance(loop, Mapping):
                raise ConfigError("config.json: 'loop' must be an object with 'start', 'stop' and 'times'")
            start, stop, times = loop.get("start"), loop.get("stop"), _int(loop, "times", "loop.")
            if not isinstance(start, int) or not isinstance(stop, int) or not 0 <= start < stop <= len(layers):
                raise ConfigError(f"config.json: loop {start!r} .. {stop!r} does not lie within the {len(layers)} layers")
            loop = (start, stop, times)
        cfg = cls(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""), eps=eps, layers=tuple(layers), loop=loop,
                  max_positions=_int(d, "max_positions", "") if d.get("max_positions") is not None else MAX_POSITIONS)
        cfg.to_model_spec()                       # every layer's keys are read (and refused) here, not at the first step
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "layers": [dict(x) for x in self.layers]}
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.max_positions != MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ------------------------------------------------------------------
    def _window(self, m: Mapping[str, Any], where: str) -> Tuple[Optional[int], int]:
        mask = m.get("mask")
        if not isinstance(mask, Mapping):
            return None, 0
        size = _opt_int(mask, "size", where + "mask.")
        keep = mask.get("keep_first") or 0
        if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
            raise ConfigError(f"config.json: {where}mask.'keep_first' must be a count of tokens, got {keep!r}")
        return size, (keep if size else 0)

    def _attention(self, m: Mapping[str, Any], where: str) -> PartSpec:
        heads = _int(m, "heads", where)
        kv = _opt_int(m, "kv_heads", where) or heads
        if heads % kv:
            raise ConfigError(f"config.json: {where}{heads} heads are not a multiple of {kv} key/value heads")
        dim = _int(m, "dim", where)
        window, keep = self._window(m, where)
        rot = m.get("rot")
        position = None
        if rot is not None:
            if not isinstance(rot, Mapping):
                raise ConfigError(f"config.json: {where}'rot' must be an object with 'dims' and 'base'")
            dims = _int(rot, "dims", where + "rot.")
            if dims % 2 or dims > dim:
                raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and at most dim {dim}")
            position = PartSpec("rope", {"theta": _float(rot, "base", where + "rot."), "rotary_dim": dims})
        taps = _opt_int(m, "conv", where)                       # none: no convolution (and no such tensors)
        return PartSpec("attention", {
            "hidden_size": self.width, "num_heads": heads, "num_kv_heads": kv, "head_dim": dim, "value_dim": _opt_int(m, "vdim", where) or dim,
            "scale": _float(m, "scale", where, 1.0 / math.sqrt(dim)), "window": window, "keep_first": keep, "qkv_bias": True, "out_bias": False,
            "position": position, "conv": taps, "conv_suffix": ".conv", "qk_norm": {"q": "q.norm", "k": "k.norm", "eps": self.eps},
            "names": {"q": "q", "k": "k", "v": "v", "o": "o"}, "suffixes": SUFFIXES})

    def _latent_attention(self, m: Mapping[str, Any], where: str) -> PartSpec:
        dim = _int(m, "dim", where)
        window, _ = self._window(m, where)
        return PartSpec("latent_attention", {
            "hidden_size": self.width, "num_heads": _int(m, "heads", where), "head_dim": dim, "value_dim": _opt_int(m, "vdim", where) or dim,
            "q_rank": _int(m, "q_rank", where), "kv_rank": _int(m, "kv_rank", where), "scale": _float(m, "scale", where, 1.0 / math.sqrt(dim)),
            "window": window, "eps": self.eps,
            "names": {"dq": "dq", "dkv": "dkv", "uq": "uq", "uk": "uk", "uv": "uv", "o": "o", "dq_norm": "dq.norm", "dkv_norm": "dkv.norm",
                      "sink": "sink"}, "suffixes": SUFFIXES})

    def _mixer(self, layer: Mapping[str, Any], where: str) -> PartSpec:
        kind, m = layer.get("type"), layer.get("mixer")
        if not isinstance(m, Mapping):
            raise ConfigError(f"config.json: {where}'mixer' is missing")
        if kind == "attention":
            return self._attention(m, where + "mixer.")
        if kind == "latent_attention":
            return self._latent_attention(m, where + "mixer.")
        raise ConfigError(f"config.json: {where}layer type {kind!r} is not supported (attention, latent_attention)")

    def _feed_forward(self, layer: Mapping[str, Any], where: str) -> Optional[PartSpec]:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
            raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} is not supported (moe)")
        router, expert = mlp.get("router"), mlp.get("expert")
        if not isinstance(router, Mapping) or not isinstance(expert, Mapping):
            raise ConfigError(f"config.json: {where}mlp needs 'router' (experts, top) and 'expert' (ff)")
        experts, top = _int(router, "experts", where + "mlp.router."), _int(router, "top", where + "mlp.router.")
        if top > experts:
            raise ConfigError(f"config.json: {where}mlp.router.top {top} is more than the {experts} experts")
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "intermediate_size": _int(expert, "ff", where + "mlp.expert."), "experts": experts, "top": top,
            "scoring": "sigmoid", "renormalize": False, "weight_on": "input",
            "names": {"router": "router", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down"}, "suffixes": SUFFIXES})

    def schedule(self) -> Tuple[ScheduleEntry, ...]:
        """The layers in the order they run; a looped span's passes one after the other, each entry with a cache of its own,
        the first layer of pass t with row t of the loop's table."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(ScheduleEntry(i) for i in range(n))
        start, stop, times = self.loop
        out = [ScheduleEntry(i) for i in range(start)]
        for t in range(times):
            out += [ScheduleEntry(i, add=(LOOP_TABLE, t) if i == start else None) for i in range(start, stop)]
        return tuple(out + [ScheduleEntry(i) for i in range(stop, n)])

    def to_model_spec(self) -> ModelSpec:
        def norm(tensor):
            return PartSpec("layernorm", {"size": self.width, "eps": self.eps, "tensor": tensor})

        blocks = []
        for i, layer in enumerate(self.layers):
            if not isinstance(layer, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            where = f"layers[{i}]."
            ff = self._feed_forward(layer, where)
            blocks.append(BlockSpec.of(
                "sandwich", f"l{i}.",
                prefixes={"mixer": "mix.", "feed_forward": "mlp.", "mixer_norm": "", "mixer_post_norm": "", "feed_forward_norm": "",
                          "feed_forward_post_norm": ""},
                mixer=self._mixer(layer, where), feed_forward=ff, mixer_norm=norm("norm1"), mixer_post_norm=norm("norm1b"),
                feed_forward_norm=norm("norm2") if ff else None, feed_forward_post_norm=norm("norm2b") if ff else None))
        return ModelSpec(
            architecture=self.ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks), schedule=self.schedule(),
            final_norm=norm("norm"), tie_word_embeddings=False, max_position_embeddings=self.max_positions, embedding_name="embed",
            final_norm_prefix="final.", lm_head_name="head",
            stream_tables={LOOP_TABLE: self.loop[2]} if self.loop is not None else {})
