"""Architecture builder for ``Botalorn``: a decoder that keeps several copies of the residual stream, shifts every
mixer's input toward the token before, and mixes, layer by layer, windowed attention over convolved projections with
the gated delta rule; its layers are listed one by one in ``config.json``.

The configuration names its architecture as a string (``"architecture": "Botalorn"``) and gives ``vocab``, ``width``,
``norm.eps``, ``embedding.scale``, ``streams`` and ``layers``: per layer its ``type`` (the kind of mixer), the mixer's
sizes and constants under ``mixer``, and its feed-forward under ``mlp`` (null: the layer has none).  In this file's
notation, with n = ``streams`` float32 copies x_1 .. x_n of the stream and N(y, w) = y / sqrt(mean y^2 + eps) * w:

* every copy starts as embed[token] * ``embedding.scale`` + s(p), s(p)[2i] = sin(p * 10000^(-2i/width)),
  s(p)[2i+1] = cos of the same angle, p the token's position in its sequence;
* a sublayer (first the mixer, then the feed-forward) with its tensors in [n], out [n], mix [n, n]:
  u = sum_s in[s] x_s;  y = sublayer(N(u, w));  x_t <- sum_s mix[s, t] x_s + out[t] y for all t at once.
  The mixer reads N(u, w) shifted toward the token before: h + (h' - h) * shift (``parts.hyper.TokenShift``);
* mixer ``attention``: see :class:`~..parts.conv_attention.ConvGatedAttention` (slopes 2^(-8 (h+1) / heads));
  ``kv_from``: j makes the layer read the keys and values that layer j cached instead of making its own;
* mixer ``delta``: see :class:`~..parts.recurrent.GatedDeltaRule`;
* feed-forward ``dense``: W_down relu(W_up h)^2;
* logits = head N(sum_s x_s, w_final).

Without ``streams`` in the configuration the model has the one stream and the plain residual sum.

This file is the only place that knows the configuration's keys and the checkpoint's tensor names (``embed``,
``final.norm``, ``head``, ``l<i>.norm1|norm2``, ``l<i>.shift``, ``l<i>.hc1|hc2.in|out|mix``, ``l<i>.mix.*``,
``l<i>.mlp.up|down``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.model_config import ConfigError
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..registry import register_architecture

# The design sets no limit on positions; the engine's tables need one.  EngineConfig.max_context overrides it.
DEFAULT_MAX_POSITION = 131072
SINUSOID_BASE = 10000.0            # the embedding's position vector
SLOPE_EXPONENT = 8.0               # slope of head h: 2^(-8 (h + 1) / heads)


@dataclass(frozen=True)
class BotalornConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    streams: int                    # 0: no stream tensors (one stream, plain residual sum)
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


def _window(mixer: Mapping[str, Any]) -> int:
    return int((mixer.get("mask") or {}).get("size") or 0)


def _heads_divide(mixer: Mapping[str, Any], where: str) -> None:
    heads, kv = _need(mixer, "heads", where, int), _need(mixer, "kv_heads", where, int)
    if heads <= 0 or kv <= 0 or heads % kv:
        raise ConfigError(f"config.json: {where}.heads {heads} must be a positive multiple of {where}.kv_heads {kv}")


def _attention(i: int, mixer: Mapping[str, Any], width: int, eps: float, cache_window: int):
    where = f"layers[{i}].mixer"
    _heads_divide(mixer, where)
    own = mixer.get("kv_from") is None
    params = {
        "hidden_size": width, "num_heads": _need(mixer, "heads", where, int), "num_kv_heads": _need(mixer, "kv_heads", where, int),
        "head_dim": _need(mixer, "dim", where, int), "value_dim": int(mixer.get("vdim") or mixer["dim"]),
        "scale": _need(mixer, "scale", where, float), "window": _window(mixer), "cache_window": int(cache_window),
        "taps": int(mixer.get("conv") or 1), "qk_norm_eps": eps, "value_norm": True, "slope_exponent": SLOPE_EXPONENT,
        "temperature": True, "gate": True, "own_cache": own,
    }
    names = {"mixer.q_proj": "mix.q", "mixer.q_conv": "mix.q.conv", "mixer.q_norm": "mix.q.norm", "mixer.k_proj": "mix.k",
             "mixer.k_conv": "mix.k.conv", "mixer.k_norm": "mix.k.norm", "mixer.v_proj": "mix.v", "mixer.v_conv": "mix.v.conv",
             "mixer.temp": "mix.temp", "mixer.g_proj": "mix.g", "mixer.o_proj": "mix.o"}
    return PartSpec("conv_gated_attention", params), names


def _delta(i: int, mixer: Mapping[str, Any], width: int, eps: float, _cw: int):
    where = f"layers[{i}].mixer"
    _heads_divide(mixer, where)
    params = {"hidden_size": width, "num_heads": _need(mixer, "heads", where, int), "num_qk_heads": _need(mixer, "kv_heads", where, int),
              "head_dim": _need(mixer, "dim", where, int), "value_dim": int(mixer.get("vdim") or mixer["dim"]),
              "taps": int(mixer.get("conv") or 1), "norm_eps": eps}
    names = {"mixer.q_proj": "mix.q", "mixer.q_conv": "mix.q.conv", "mixer.k_proj": "mix.k", "mixer.k_conv": "mix.k.conv",
             "mixer.v_proj": "mix.v", "mixer.v_conv": "mix.v.conv", "mixer.b_proj": "mix.b", "mixer.a_proj": "mix.a",
             "mixer.A_log": "mix.A_log", "mixer.dt_bias": "mix.dt_bias", "mixer.norm": "mix.norm", "mixer.g_proj": "mix.g",
             "mixer.o_proj": "mix.o"}
    return PartSpec("gated_delta_rule", params), names


_MIXERS = {"attention": _attention, "delta": _delta}


def _cache_sources(layers) -> Dict[int, int]:
    """attention layer -> the layer whose keys and values it reads (itself when it makes its own); checked."""
    src: Dict[int, int] = {}
    for i, layer in enumerate(layers):
        if layer.get("type") != "attention":
            continue
        mixer = _need(layer, "mixer", f"layers[{i}]")
        j = mixer.get("kv_from")
        if j is None:
            src[i] = i
            continue
        where = f"layers[{i}].mixer.kv_from"
        if isinstance(j, bool) or not isinstance(j, int) or not (0 <= j < i):
            raise ConfigError(f"config.json: {where} must name an earlier layer, got {j!r}")
        other = layers[j]
        if other.get("type") != "attention" or (other.get("mixer") or {}).get("kv_from") is not None:
            raise ConfigError(f"config.json: {where} names layer {j}, which has no keys and values of its own")
        om = other["mixer"]
        for key in ("heads", "kv_heads", "dim", "vdim"):
            if int(om.get(key) or om.get("dim") or 0) != int(mixer.get(key) or mixer.get("dim") or 0):
                raise ConfigError(f"config.json: {where}: layer {j} has another {key}")
        src[i] = j
    return src


def spec_from_config(cfg: BotalornConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"eps": cfg.norm_eps})
    src = _cache_sources(cfg.layers)
    # a shared cache keeps what the widest window among its readers needs; one reader without a window keeps all
    windows: Dict[int, list] = {}
    for i, j in src.items():
        windows.setdefault(j, []).append(_window(cfg.layers[i]["mixer"]))
    keep = {j: (0 if min(ws) == 0 else max(ws)) for j, ws in windows.items()}
    streams = max(cfg.streams, 1)
    layers, runs = [], []
    for i, layer in enumerate(cfg.layers):
        kind = layer.get("type")
        if kind not in _MIXERS:
            raise ConfigError(f"config.json: layers[{i}].type {kind!r}: this design has the mixers {sorted(_MIXERS)}")
        mixer, names = _MIXERS[kind](i, _need(layer, "mixer", f"layers[{i}]"), cfg.hidden_size, cfg.norm_eps, keep.get(src.get(i, i), 0))
        names = dict(names)
        names.update({"norm_in.weight": "norm1", "shift.weight": "shift", "hc_mixer.in": "hc1.in", "hc_mixer.out": "hc1.out",
                      "hc_mixer.mix": "hc1.mix"})
        mlp = layer.get("mlp")
        ff = None
        if mlp:
            where = f"layers[{i}].mlp"
            if mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"config.json: {where}.kind {mlp.get('kind')!r}: this design has the feed-forward 'dense'")
            ff = PartSpec("mlp_act", {"hidden_size": cfg.hidden_size, "intermediate_size": _need(mlp, "ff", where, int), "act": "relu2"})
            names.update({"norm_post.weight": "norm2", "feed_forward.up": "mlp.up", "feed_forward.down": "mlp.down",
                          "hc_ff.in": "hc2.in", "hc_ff.out": "hc2.out", "hc_ff.mix": "hc2.mix"})
        block_params = {"streams": streams, "learned": cfg.streams > 0, "token_shift": True}
        layers.append(LayerSpec(block="hyper" if ff is not None else "hyper_mixer", mixer=mixer, feed_forward=ff, norm=norm,
                                position=PartSpec("none", {}), prefix=f"l{i}.", names=names, block_params=block_params))
        cache = src.get(i, i)
        runs.append(RunEntry(layer=i, cache=cache, writes_cache=cache == i))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        layers=tuple(layers), run_list=tuple(runs),
        embedding=PartSpec("table", {"name": "embed", "scale": cfg.embedding_scale, "sinusoid_base": SINUSOID_BASE}),
        final_norm=PartSpec("rmsnorm", {"eps": cfg.norm_eps, "name": "final.norm"}),
        head=PartSpec("linear", {"tied": False, "name": "head"}),
        max_position=cfg.max_position_embeddings, stop_token_ids=tuple(cfg.eos_token_ids), streams=streams,
    )


def config_from_dict(raw: Mapping[str, Any], generation_config: Optional[Mapping[str, Any]] = None) -> BotalornConfig:
    layers = _need(raw, "layers", "config")
    if not isinstance(layers, (list, tuple)) or not layers:
        raise ConfigError("config.json: layers must be a non-empty list")
    eos = ()
    for source in (generation_config, raw):
        v = source.get("eos_token_id") if isinstance(source, Mapping) else None
        if v is not None:
            eos = tuple(int(t) for t in (v if isinstance(v, (list, tuple)) else [v]))
            break
    streams = raw.get("streams")
    if streams is None:
        streams = 0
    elif isinstance(streams, bool) or not isinstance(streams, int) or not (1 <= streams <= 8):
        raise ConfigError(f"config.json: streams must be an integer from 1 to 8, got {streams!r}")
    scale = (raw.get("embedding") or {}).get("scale")
    if scale is None:
        scale = 1.0
    elif isinstance(scale, bool) or not isinstance(scale, (int, float)):
        raise ConfigError(f"config.json: embedding.scale must be a number, got {scale!r}")
    return BotalornConfig(
        architecture="Botalorn", vocab_size=_need(raw, "vocab", "config", int), hidden_size=_need(raw, "width", "config", int),
        norm_eps=_need(_need(raw, "norm", "config"), "eps", "config.norm", float), embedding_scale=float(scale),
        streams=int(streams), layers=tuple(layers), max_position_embeddings=DEFAULT_MAX_POSITION, eos_token_ids=eos,
    )


@register_architecture("Botalorn")
def _build(raw, generation_config=None, strict=False):
    cfg = config_from_dict(raw, generation_config)
    return cfg, spec_from_config(cfg)
