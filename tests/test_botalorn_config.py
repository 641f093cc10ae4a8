"""The Botalorn configuration reader on the CPU: what it builds from config.json, and what it refuses."""
import copy

import pytest

from aien_sovereign_core_mv_b200 import ConfigError, model_spec_for
from aien_sovereign_core_mv_b200.models.decoder import Decoder


def _attention(window, kv_from=None):
    m = {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 4, "scale": 0.3, "mask": {"size": window}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


CONFIG = {"architecture": "Botalorn", "vocab": 97, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0}, "streams": 3,
          "layers": [
              {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "conv": 2}, "mlp": {"kind": "dense", "ff": 56}},
              {"type": "attention", "mixer": _attention(9), "mlp": None},
              {"type": "attention", "mixer": _attention(21, kv_from=1), "mlp": {"kind": "dense", "ff": 24}},
              {"type": "attention", "mixer": _attention(5), "mlp": {"kind": "dense", "ff": 24}}]}


def test_spec_parts_run_list_and_tensor_names():
    cfg, spec = model_spec_for(CONFIG)
    assert cfg.num_hidden_layers == 4 and cfg.streams == 3 and cfg.embedding_scale == 3.0 and spec.streams == 3
    assert [l.block for l in spec.layers] == ["hyper", "hyper_mixer", "hyper", "hyper"]
    assert [(r.cache, r.writes_cache) for r in spec.run_list] == [(0, True), (1, True), (1, False), (3, True)]
    assert [l.mixer.kind for l in spec.layers] == ["gated_delta_rule"] + ["conv_gated_attention"] * 3
    # the shared cache keeps the widest window of its readers; the layer's own mask stays its own
    a1, a2, a3 = (spec.layers[i].mixer.params for i in (1, 2, 3))
    assert (a1["window"], a1["cache_window"], a1["own_cache"]) == (9, 21, True)
    assert (a2["window"], a2["cache_window"], a2["own_cache"]) == (21, 21, False)
    assert (a3["window"], a3["cache_window"]) == (5, 5)
    assert a1["taps"] == 4 and a1["slope_exponent"] == 8.0 and a1["scale"] == 0.3 and a1["value_dim"] == 12
    d = spec.layers[0].mixer.params
    assert (d["num_heads"], d["num_qk_heads"], d["head_dim"], d["value_dim"], d["taps"]) == (4, 2, 8, 6, 2)
    model = Decoder(spec)
    cat = model.catalog()
    assert cat["embed"][0] == (97, 40) and cat["head"][0] == (97, 40) and cat["final.norm"][0] == (40,)
    assert cat["l0.hc1.in"][0] == (3,) and cat["l0.hc2.mix"][0] == (3, 3) and cat["l0.shift"][0] == (40,)
    assert cat["l0.mix.q"][0] == (16, 40) and cat["l0.mix.v"][0] == (24, 40) and cat["l0.mix.q.conv"][0] == (16, 2)
    assert cat["l0.mix.A_log"][0] == (4,) and cat["l0.mix.dt_bias"][0] == (4,) and cat["l0.mix.norm"][0] == (6,)
    assert cat["l0.mix.a"][0] == (4, 40) and cat["l0.mix.b"][0] == (4, 40) and cat["l0.mix.g"][0] == (24, 40)
    assert cat["l1.mix.q"][0] == (48, 40) and cat["l1.mix.k"][0] == (16, 40) and cat["l1.mix.v"][0] == (24, 40)
    assert cat["l1.mix.q.norm"][0] == (48,) and cat["l1.mix.k.norm"][0] == (16,) and cat["l1.mix.v.conv"][0] == (24, 4)
    assert cat["l1.mix.temp"][0] == (6,) and cat["l1.mix.g"][0] == (6, 40) and cat["l1.mix.o"][0] == (40, 72)
    assert "l1.mlp.up" not in cat and "l1.norm2" not in cat and "l1.hc2.in" not in cat          # a layer without a feed-forward
    assert "l2.mix.k" not in cat and "l2.mix.v.conv" not in cat and "l2.mix.k.norm" not in cat  # it reads layer 1's cache
    assert cat["l2.mix.q.conv"][0] == (48, 4) and cat["l3.mlp.up"][0] == (24, 40) and cat["l3.mlp.down"][0] == (40, 24)
    # pages for the two caches, slots for the shift rows, the convolutions' rows and the delta rule's state
    kinds = sorted(n.kind for n in model.group_needs)
    assert kinds.count("window") == 2 and kinds.count("state") >= 3 and set(kinds) == {"state", "window"}


def test_one_stream_is_the_plain_residual():
    c = copy.deepcopy(CONFIG)
    c.pop("streams")
    _, spec = model_spec_for(c)
    assert spec.streams == 1
    assert "l0.hc1.in" not in Decoder(spec).catalog()


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 2), "earlier layer"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 3), "earlier layer"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 0), "no keys and values"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda c: c["layers"][0].__setitem__("type", "mamba"), "mixers"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "feed-forward"),
    (lambda c: c.__setitem__("streams", 9), "streams"),
    (lambda c: c["layers"][3]["mixer"].pop("dim"), "dim is missing"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 3), "multiple"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("heads", 5), "multiple"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_refusals_name_the_field(change, word):
    c = copy.deepcopy(CONFIG)
    change(c)
    with pytest.raises(ConfigError) as e:
        model_spec_for(c)
    assert word in str(e.value)
