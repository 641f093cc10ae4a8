"""The Mumazen configuration reader on the CPU: what it builds from config.json, and what it refuses."""
import copy

import pytest

from aien_sovereign_core_mv_b200 import ConfigError, model_spec_for
from aien_sovereign_core_mv_b200.models.decoder import Decoder
from aien_sovereign_core_mv_b200.models.mumazen import run_order

PARALLEL = {"left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 12, "scale": 0.2, "softcap": 25.0,
                     "rot": {"base": 50000.0, "dims": 8, "scaling": {"factor": 4.0}}},
            "right": {"heads": 6, "vdim": 4, "state": 10, "groups": 3, "norm_groups": 2, "conv": 3},
            "left_scale": 1.5, "right_scale": 0.25}
CONFIG = {"architecture": "Mumazen", "vocab": 97, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0}, "residual_mult": 0.6,
          "loop": {"start": 1, "stop": 3, "times": 2},
          "layers": [
              {"type": "mamba1", "mixer": {"inner": 24, "state": 7, "dt_rank": 3, "conv": 2}, "mlp": {"kind": "dense", "ff": 56, "limit": 2.0}},
              {"type": "parallel", "mixer": PARALLEL, "mlp": {"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 3, "identity": 2, "top": 2},
                                                                "shared": {"ff": 28}}},
              {"type": "mamba1", "mixer": {"inner": 32, "state": 5, "dt_rank": 1, "conv": 4}, "mlp": None},
              {"type": "parallel", "mixer": PARALLEL, "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 2, "top": 1}}}]}


def test_spec_parts_run_list_and_tensor_names():
    cfg, spec = model_spec_for(CONFIG)
    assert cfg.num_hidden_layers == 4 and cfg.embedding_scale == 3.0 and cfg.residual_mult == 0.6 and cfg.loop == (1, 3, 2)
    assert [l.block for l in spec.layers] == ["prenorm_scaled", "prenorm_scaled", "prenorm_scaled_mixer", "prenorm_scaled"]
    assert [l.mixer.kind for l in spec.layers] == ["selective_scan", "parallel_mixers", "selective_scan", "parallel_mixers"]
    # layers 1 and 2 run twice; every run has a cache of its own; the first run of a pass opens it
    assert [(r.layer, r.cache, r.enter) for r in spec.run_list] == [(0, 0, -1), (1, 1, 0), (2, 2, -1), (1, 3, 1), (2, 4, -1), (3, 5, -1)]
    assert all(r.writes_cache for r in spec.run_list) and spec.pass_input.kind == "step_vector" and spec.pass_input.params["times"] == 2
    p = spec.layers[1].mixer.params
    assert p["left_scale"] == 1.5 and p["right_scale"] == 0.25 and p["left"]["softcap"] == 25.0 and p["left"]["value_dim"] == 12
    assert p["right"]["norm_groups"] == 2 and p["right"]["taps"] == 3 and p["right"]["norm_eps"] == 1e-5
    rot = spec.layers[1].position.params
    assert rot["rotary_dim"] == 8 and rot["linear_factor"] == 4.0 and rot["pairing"] == "halves" and rot["theta"] == 50000.0
    f = spec.layers[1].feed_forward.params
    assert (f["num_experts"], f["identity_experts"], f["top"], f["shared_ff"], f["shared_gate"], f["correction"]) == (3, 2, 2, 28, True, True)
    f = spec.layers[3].feed_forward.params
    assert (f["identity_experts"], f["shared_ff"], f["shared_gate"]) == (0, 0, False)
    model = Decoder(spec)
    cat = model.catalog()
    assert cat["embed"][0] == (97, 40) and cat["head"][0] == (97, 40) and cat["final.norm"][0] == (40,) and cat["loop.step"][0] == (2, 40)
    assert cat["l0.mix.in"][0] == (48, 40) and cat["l0.mix.conv"][0] == (24, 2) and cat["l0.mix.conv.b"][0] == (24,)
    assert cat["l0.mix.x"][0] == (17, 24) and cat["l0.mix.dt"][0] == (24, 3) and cat["l0.mix.dt.b"][0] == (24,)
    assert cat["l0.mix.A_log"][0] == (24, 7) and cat["l0.mix.D"][0] == (24,) and cat["l0.mix.o"][0] == (40, 24)
    assert cat["l0.mlp.gate.b"][0] == (56,) and cat["l0.mlp.down.b"][0] == (40,) and cat["l0.ls1"][0] == (40,) and cat["l0.ls2"][0] == (40,)
    assert cat["l1.mix.left.q"][0] == (64, 40) and cat["l1.mix.left.k"][0] == (32, 40) and cat["l1.mix.left.v"][0] == (24, 40)
    assert cat["l1.mix.left.g"][0] == (48, 40) and cat["l1.mix.left.o"][0] == (40, 48)
    assert cat["l1.mix.right.in"][0] == (2 * 24 + 2 * 30 + 6, 40) and cat["l1.mix.right.conv"][0] == (24 + 60, 3)
    assert cat["l1.mix.right.A_log"][0] == (6,) and cat["l1.mix.right.norm"][0] == (24,) and cat["l1.mix.right.o"][0] == (40, 24)
    assert cat["l1.mlp.router"][0] == (5, 40) and cat["l1.mlp.correction"][0] == (5,) and cat["l1.mlp.e2.up"][0] == (20, 40)
    assert cat["l1.mlp.shared.sg"][0] == (1, 40) and cat["l1.mlp.shared.down"][0] == (40, 28) and "l1.mlp.e3.up" not in cat
    assert "l2.norm2" not in cat and "l2.ls2" not in cat and "l2.mlp.gate" not in cat            # a layer without a feed-forward
    assert "l3.mlp.shared.up" not in cat and cat["l3.mlp.router"][0] == (2, 40)
    # pages for the attention of three runs; state slots for the scans (runs of layers 0, 2, 2) and for the right halves
    needs = {n.kind: s for n, s in zip(model.group_needs, model.group_slots) if n.kind == "full"}
    assert needs == {"full": 3}
    states = sorted((n.state_shape[0], s) for n, s in zip(model.group_needs, model.group_slots) if n.kind == "state")
    assert states == sorted([(1 * 24 + 24 * 7, 1), (3 * 32 + 32 * 5, 2), (2 * 84 + 6 * 10 * 4, 3)])


def test_run_order():
    assert run_order(3, None) == [(0, -1), (1, -1), (2, -1)]
    assert run_order(3, (0, 1, 3)) == [(0, 0), (0, 1), (0, 2), (1, -1), (2, -1)]
    assert run_order(4, (2, 4, 1)) == [(0, -1), (1, -1), (2, 0), (3, -1)]


def test_without_a_loop_there_is_no_pass_input():
    c = copy.deepcopy(CONFIG)
    c.pop("loop")
    _, spec = model_spec_for(c)
    assert spec.pass_input is None and [r.enter for r in spec.run_list] == [-1] * 4
    assert "loop.step" not in Decoder(spec).catalog()


@pytest.mark.parametrize("path,value,word", [
    (("layers", 1, "mixer", "left", "heads"), 3, "multiple"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 7, "even"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 18, "even"),
    (("layers", 1, "mixer", "right", "groups"), 4, "multiple"),
    (("layers", 1, "mixer", "right", "norm_groups"), 5, "norm_groups"),
    (("layers", 1, "mlp", "router", "top"), 6, "top"),
    (("layers", 0, "type"), "conv", "mixers"),
    (("layers", 0, "mlp", "kind"), "glu", "feed-forwards"),
    (("layers", 0, "mlp", "limit"), None, "limit"),
    (("loop", "stop"), 5, "loop"),
    (("loop", "times"), 0, "times"),
    (("norm", "eps"), None, "eps"),
])
def test_refusals(path, value, word):
    c = copy.deepcopy(CONFIG)
    at = c
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        model_spec_for(c)
    assert word in str(e.value)
