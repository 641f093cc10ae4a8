"""Architecture builder for ``Mumazen``: a decoder that mixes, layer by layer, a selective scan and attention side by side
with a state-space-duality recurrence, scales every branch per channel, and may run a stretch of its layers several times
in a row; its layers are listed one by one in ``config.json``.

The configuration names its architecture as a string (``"architecture": "Mumazen"``) and gives ``vocab``, ``width``,
``norm.eps``, ``embedding.scale``, ``residual_mult``, ``loop`` and ``layers``: per layer its ``type`` (the kind of mixer),
the mixer's sizes and constants under ``mixer``, and its feed-forward under ``mlp`` (null: the layer has none).  In this
file's notation, with the float32 stream x, m = ``residual_mult`` and N(y, w) = y / sqrt(mean y^2 + eps) * w:

* x = embed[token] * ``embedding.scale``; logits = head N(x, w_final);
* a layer: x <- x + m * ls1 * mixer(N(x, norm1)); x <- x + m * ls2 * ff(N(x, norm2)), ls1 and ls2 vectors of the width;
* ``loop`` {start, stop, times}: layers start .. stop - 1 run ``times`` times in a row with the same tensors, every pass
  with a cache and state of its own; before pass t the stream takes x <- x + e (e the embedding's output; not before the
  first pass) and then x <- x + loop.step[t];
* mixer ``mamba1``: see :class:`~..parts.state_space.SelectiveScan`;
* mixer ``parallel``: ``left_scale`` * left + ``right_scale`` * right on the same input
  (:class:`~..parts.state_space.ParallelMixers`): left is :class:`~..parts.attention.GatedCappedAttention` (rotation of
  halves over ``rot.dims`` dimensions with frequencies ``rot.base``^(-2i/dims) / ``rot.scaling.factor``), right is
  :class:`~..parts.state_space.StateSpaceDuality`;
* feed-forward ``dense``: :class:`~..parts.mlp.ClampedGLU` with biases; ``moe``: :class:`~..parts.moe.RoutedExperts` with
  a correction on the choice, identity experts behind the real ones, weights divided by their sum, experts
  W_down relu(W_up h)^2 and a shared expert of the same form times sigmoid(w_sg . h).

This file is the only place that knows the configuration's keys and the checkpoint's tensor names (``embed``,
``loop.step``, ``final.norm``, ``head``, ``l<i>.norm1|norm2|ls1|ls2``, ``l<i>.mix.*``, ``l<i>.mlp.*``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.model_config import ConfigError
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..registry import register_architecture

# The design sets no limit on positions; the engine's tables need one.  EngineConfig.max_context overrides it.
DEFAULT_MAX_POSITION = 131072
GATE_SLOPE = 1.702                 # the dense feed-forward's gate: g * sigmoid(1.702 g)
WEIGHT_SUM_EPS = 1e-20             # added to the sum of the chosen experts' scores before the division


@dataclass(frozen=True)
class MumazenConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    loop: Optional[Tuple[int, int, int]]           # (start, stop, times) or None
    layers: Tuple[Mapping[str, Any], ...]
    max_position_embeddings: int = DEFAULT_MAX_POSITION
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)


def _need(obj: Any, key: str, where: str, kind=None):
    if not isinstance(obj, Mapping) or key not in obj or obj[key] is None:
        raise ConfigError(f"config.json: {where}.{key} is missing")
    v = obj[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
            raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    elif kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
        v = float(v)
    return v


def _opt_number(obj: Any, key: str, default: float, where: str = "config") -> float:
    v = obj.get(key) if isinstance(obj, Mapping) else None
    if v is None:
        return float(default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


def _opt_count(obj: Any, key: str, default: int, where: str) -> int:
    v = obj.get(key) if isinstance(obj, Mapping) else None
    if v is None:
        return int(default)
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"config.json: {where}.{key} must be a non-negative integer, got {v!r}")
    return int(v)


def _mamba1(i: int, mixer: Mapping[str, Any], width: int, eps: float):
    where = f"layers[{i}].mixer"
    params = {"hidden_size": width, "inner": _need(mixer, "inner", where, int), "state": _need(mixer, "state", where, int),
              "dt_rank": _need(mixer, "dt_rank", where, int), "taps": _need(mixer, "conv", where, int)}
    names = {"mixer.in_proj": "mix.in", "mixer.conv": "mix.conv", "mixer.conv_bias": "mix.conv.b", "mixer.x_proj": "mix.x",
             "mixer.dt_proj": "mix.dt", "mixer.dt_bias": "mix.dt.b", "mixer.A_log": "mix.A_log", "mixer.D": "mix.D", "mixer.o_proj": "mix.o"}
    return PartSpec("none", {}), PartSpec("selective_scan", params), names


def _parallel(i: int, mixer: Mapping[str, Any], width: int, eps: float):
    where = f"layers[{i}].mixer"
    left, right = _need(mixer, "left", where), _need(mixer, "right", where)
    lw, rw = where + ".left", where + ".right"
    heads = _need(left, "heads", lw, int)
    kv = _need(left, "kv_heads", lw, int) if left.get("kv_heads") is not None else heads        # no groups named: one key/value head a query head
    if heads % kv:
        raise ConfigError(f"config.json: {lw}.heads {heads} must be a multiple of {lw}.kv_heads {kv}")
    dim = _need(left, "dim", lw, int)
    rot = left.get("rot")
    if rot:
        dims = _need(rot, "dims", lw + ".rot", int)
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {lw}.rot.dims {dims} must be even and at most {lw}.dim {dim}")
        factor = _opt_number(rot.get("scaling") or {}, "factor", 1.0, lw + ".rot.scaling")
        if factor <= 0.0:
            raise ConfigError(f"config.json: {lw}.rot.scaling.factor must be positive, got {factor!r}")
        position = PartSpec("rotary", {"head_dim": dim, "theta": _need(rot, "base", lw + ".rot", float), "rotary_dim": dims,
                                       "pairing": "halves", "theta_as_float32": False, "linear_factor": factor})
    else:
        position = PartSpec("none", {})
    rheads, groups = _need(right, "heads", rw, int), _opt_count(right, "groups", 1, rw) or 1
    if rheads % groups:
        raise ConfigError(f"config.json: {rw}.heads {rheads} must be a multiple of {rw}.groups {groups}")
    vdim = _need(right, "vdim", rw, int)
    norm_groups = _opt_count(right, "norm_groups", 1, rw) or 1
    if (rheads * vdim) % norm_groups:
        raise ConfigError(f"config.json: {rw}.norm_groups {norm_groups} does not divide {rheads * vdim} channels")
    params = {
        "hidden_size": width,
        "left": {"kind": "gated_capped_attention", "num_heads": heads, "num_kv_heads": kv, "head_dim": dim,
                 "value_dim": int(left.get("vdim") or dim), "scale": _need(left, "scale", lw, float),
                 "softcap": _opt_number(left, "softcap", 0.0, lw), "gate": True},
        "right": {"kind": "state_space_duality", "num_heads": rheads, "value_dim": vdim, "state": _need(right, "state", rw, int),
                  "groups": groups, "norm_groups": norm_groups, "taps": _need(right, "conv", rw, int), "norm_eps": eps},
        "left_scale": _opt_number(mixer, "left_scale", 1.0, where), "right_scale": _opt_number(mixer, "right_scale", 1.0, where),
    }
    names = {"mixer.left.q_proj": "mix.left.q", "mixer.left.k_proj": "mix.left.k", "mixer.left.v_proj": "mix.left.v",
             "mixer.left.g_proj": "mix.left.g", "mixer.left.o_proj": "mix.left.o",
             "mixer.right.in_proj": "mix.right.in", "mixer.right.conv": "mix.right.conv", "mixer.right.conv_bias": "mix.right.conv.b",
             "mixer.right.dt_bias": "mix.right.dt_bias", "mixer.right.A_log": "mix.right.A_log", "mixer.right.D": "mix.right.D",
             "mixer.right.norm": "mix.right.norm", "mixer.right.o_proj": "mix.right.o"}
    return position, PartSpec("parallel_mixers", params), names


_MIXERS = {"mamba1": _mamba1, "parallel": _parallel}


def _feed_forward(i: int, mlp: Mapping[str, Any], width: int):
    where = f"layers[{i}].mlp"
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        ff = PartSpec("clamped_glu", {"hidden_size": width, "intermediate_size": _need(mlp, "ff", where, int),
                                      "limit": _need(mlp, "limit", where, float), "alpha": GATE_SLOPE, "bias": True})
        names = {"feed_forward.gate": "mlp.gate", "feed_forward.gate_bias": "mlp.gate.b", "feed_forward.up": "mlp.up",
                 "feed_forward.up_bias": "mlp.up.b", "feed_forward.down": "mlp.down", "feed_forward.down_bias": "mlp.down.b"}
        return ff, names
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r}: this design has the feed-forwards 'dense' and 'moe'")
    router = _need(mlp, "router", where)
    experts, top = _need(router, "experts", where + ".router", int), _need(router, "top", where + ".router", int)
    identity = _opt_count(router, "identity", 0, where + ".router")
    if top > experts + identity:
        raise ConfigError(f"config.json: {where}.router.top {top} exceeds the {experts + identity} router outputs")
    shared = mlp.get("shared")
    params = {"hidden_size": width, "expert_ff": _need(_need(mlp, "expert", where), "ff", where + ".expert", int), "num_experts": experts,
              "top": top, "act": "relu2", "renormalise": True, "renormalise_eps": WEIGHT_SUM_EPS, "correction": True,
              "identity_experts": identity, "shared_ff": _need(shared, "ff", where + ".shared", int) if shared else 0,
              "shared_gate": bool(shared), "combined": True}
    names = {"feed_forward.router": "mlp.router", "feed_forward.correction": "mlp.correction", "feed_forward.shared.up": "mlp.shared.up",
             "feed_forward.shared.down": "mlp.shared.down", "feed_forward.shared.gate": "mlp.shared.sg"}
    for e in range(experts):
        names[f"feed_forward.experts.{e}.up"] = f"mlp.e{e}.up"
        names[f"feed_forward.experts.{e}.down"] = f"mlp.e{e}.down"
    return PartSpec("routed_experts", params), names


def run_order(num_layers: int, loop: Optional[Tuple[int, int, int]]):
    """[(layer, pass number that this run opens or -1)]: layers start .. stop - 1 run ``times`` times in a row."""
    if loop is None:
        return [(i, -1) for i in range(num_layers)]
    start, stop, times = loop
    order = [(i, -1) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else -1) for i in range(start, stop)]
    return order + [(i, -1) for i in range(stop, num_layers)]


def spec_from_config(cfg: MumazenConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"eps": cfg.norm_eps})
    layers = []
    for i, layer in enumerate(cfg.layers):
        kind = layer.get("type")
        if kind not in _MIXERS:
            raise ConfigError(f"config.json: layers[{i}].type {kind!r}: this design has the mixers {sorted(_MIXERS)}")
        position, mixer, names = _MIXERS[kind](i, _need(layer, "mixer", f"layers[{i}]"), cfg.hidden_size, cfg.norm_eps)
        names = dict(names)
        names.update({"norm_in.weight": "norm1", "scale_mixer.weight": "ls1"})
        mlp = layer.get("mlp")
        ff = None
        if mlp:
            ff, ff_names = _feed_forward(i, mlp, cfg.hidden_size)
            names.update(ff_names)
            names.update({"norm_post.weight": "norm2", "scale_ff.weight": "ls2"})
        layers.append(LayerSpec(block="prenorm_scaled" if ff is not None else "prenorm_scaled_mixer", mixer=mixer, feed_forward=ff,
                                norm=norm, position=position, prefix=f"l{i}.", names=names,
                                block_params={"residual_mult": cfg.residual_mult, "layer_scale": True}))
    # every run keeps a cache and state of its own, also the later passes over a layer
    runs = tuple(RunEntry(layer=i, cache=n, writes_cache=True, enter=t) for n, (i, t) in enumerate(run_order(len(layers), cfg.loop)))
    pass_input = None
    if cfg.loop is not None:
        pass_input = PartSpec("step_vector", {"times": cfg.loop[2], "add_embedding": True, "names": {"steps": "loop.step"}})
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        layers=tuple(layers), run_list=runs,
        embedding=PartSpec("table", {"name": "embed", "scale": cfg.embedding_scale}),
        final_norm=PartSpec("rmsnorm", {"eps": cfg.norm_eps, "name": "final.norm"}),
        head=PartSpec("linear", {"tied": False, "name": "head"}),
        max_position=cfg.max_position_embeddings, stop_token_ids=tuple(cfg.eos_token_ids), pass_input=pass_input,
    )


def _loop(raw: Mapping[str, Any], num_layers: int) -> Optional[Tuple[int, int, int]]:
    loop = raw.get("loop")
    if loop is None:
        return None
    start, stop = _opt_count(loop, "start", 0, "loop"), _need(loop, "stop", "loop", int)
    times = _need(loop, "times", "loop", int) if loop.get("times") is not None else 1
    if not (0 <= start < stop <= num_layers):
        raise ConfigError(f"config.json: loop.start {start} and loop.stop {stop} must name a stretch of the {num_layers} layers")
    return start, stop, times


def config_from_dict(raw: Mapping[str, Any], generation_config: Optional[Mapping[str, Any]] = None) -> MumazenConfig:
    layers = _need(raw, "layers", "config")
    if not isinstance(layers, (list, tuple)) or not layers:
        raise ConfigError("config.json: layers must be a non-empty list")
    eos = ()
    for source in (generation_config, raw):
        v = source.get("eos_token_id") if isinstance(source, Mapping) else None
        if v is not None:
            eos = tuple(int(t) for t in (v if isinstance(v, (list, tuple)) else [v]))
            break
    return MumazenConfig(
        architecture="Mumazen", vocab_size=_need(raw, "vocab", "config", int), hidden_size=_need(raw, "width", "config", int),
        norm_eps=_need(_need(raw, "norm", "config"), "eps", "config.norm", float),
        embedding_scale=_opt_number(raw.get("embedding") or {}, "scale", 1.0, "embedding"),
        residual_mult=_opt_number(raw, "residual_mult", 1.0), loop=_loop(raw, len(layers)), layers=tuple(layers),
        max_position_embeddings=DEFAULT_MAX_POSITION, eos_token_ids=eos,
    )


@register_architecture("Mumazen")
def _build(raw, generation_config=None, strict=False):
    cfg = config_from_dict(raw, generation_config)
    return cfg, spec_from_config(cfg)
