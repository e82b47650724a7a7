"""Fovezen on the CPU: reading config.json, the order of runs, the weight plan, random weights, and the plain
implementation's own consistency."""
import copy
import json

import pytest
import torch

import fovezen_configs as fc
import plain_fovezen as pf
from geneinfer_b200.config import ConfigError, FovezenConfig, parse_config
from geneinfer_b200.weights import load_model_folder

CASES = {"a": fc.FOV_A, "b": fc.FOV_B, "c": fc.FOV_C, "d": fc.FOV_D}


@pytest.mark.parametrize("case", sorted(CASES))
def test_configuration_round_trip_and_translation(case):
    arch, cfg = parse_config(CASES[case])
    assert arch.name == "Fovezen" and isinstance(cfg, FovezenConfig)
    assert parse_config(json.loads(json.dumps(cfg.to_json())))[1] == cfg
    spec = cfg.model_spec()
    spec.validate()
    n = len(CASES[case]["layers"])
    order = pf.layer_order(CASES[case])
    assert [e.layer for e in spec.schedule] == order
    # every run has a cache of its own: the first pass the layer's, later passes a layer that owns no weights
    caches = [e.layer if e.cache_of is None else e.cache_of for e in spec.schedule]
    assert len(set(caches)) == len(caches) and len(spec.layers) == len(order)
    for e in spec.schedule:
        if e.cache_of is not None:
            assert e.cache_of >= n and spec.shared_layers[e.cache_of] == e.layer
    assert all(l.block == "hyper_connections" and l.block_params["streams"] == (CASES[case].get("streams") or 1) for l in spec.layers)
    assert (spec.logit_transform is None) == (CASES[case].get("logit_scale") in (None, 1.0))


def test_every_constant_is_read_from_the_file():
    cfg = parse_config(fc.FOV_A)[1]
    spec = cfg.model_spec()
    par = spec.layers[1].mixer.params
    lft, rgt = par["branches"][0][1].params, par["branches"][1][1].params
    assert (lft["num_heads"], lft["num_kv_heads"], lft["head_dim"], lft["value_dim"], lft["window"], lft["conv_taps"], lft["softcap"], lft["scale"]) == \
        (6, 2, 16, 24, 20, 2, 5.0, 0.3)
    assert (rgt["num_heads"], rgt["key_dim"], rgt["value_dim"], rgt["tau"], rgt["decay_rank"]) == (3, 16, 40, 8.0, 8)
    assert par["combine"] == "mean_normed" and par["combine_eps"] == 1e-5
    att = spec.layers[2].mixer.params
    assert att["qk_norm_wide"] and att["window"] is None and att["value_dim"] == 32
    assert att["position"].params["rotary_dim"] == 8 and att["position"].params["pairing"] == "half_split"
    assert att["position"].params["wavelength_scaling"] == {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    ssm = spec.layers[0].mixer.params
    assert (ssm["num_heads"], ssm["head_dim"], ssm["state_size"], ssm["groups"], ssm["conv_taps"], ssm["norm_groups"]) == (4, 24, 16, 2, 4, 2)
    ff = spec.layers[0].feed_forward.params
    assert ff["activation"] == "capped_swish" and ff["activation_limit"] == 0.8 and ff["intermediate_size"] == 136
    assert spec.layers[2].feed_forward is None and spec.layers[3].feed_forward is None
    assert spec.logit_transform.params["factor"] == 0.7


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="lightning"), "unknown type"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(mask={}), "mask"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(tau=0), "tau"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][2]["mixer"].update(kv_heads=4), "multiple"),
    (lambda c: c.update(loop={"start": 2, "stop": 2, "times": 2}), "loop"),
    (lambda c: c.update(loop={"start": 0, "stop": 9, "times": 2}), "loop"),
    (lambda c: c.update(streams=9), "streams"),
    (lambda c: c["layers"][0]["mlp"].update(limit=-1.0), "limit"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_bad_configurations_are_refused(change, message):
    cfg = copy.deepcopy(fc.FOV_A)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        parse_config(cfg)


def test_random_weights_folder_loads_by_name(tmp_path):
    folder = fc.make_model_dir(fc.FOV_A, 5, str(tmp_path / "m"))
    arch, cfg, params = load_model_folder(folder)
    assert params["layers.1.mixer.left.w_qkv"].shape == (6 * 16 + 2 * 16 + 2 * 24, 96)
    assert params["layers.1.mixer.left.conv"].shape == (6 * 16 + 2 * 16 + 2 * 24, 2)
    assert params["layers.1.mixer.right.w_in"].shape == (2 * 3 * 16 + 2 * 3 * 40, 96)
    assert params["layers.1.mixer.right.w_a1"].shape == (8, 96) and params["layers.1.mixer.right.w_a2"].shape == (48, 8)
    assert params["layers.1.mixer.left_out"].shape == (96,) and params["layers.1.hc2.mix"].shape == (3, 3)
    assert params["layers.2.mixer.q_norm"].shape == (96,) and params["layers.2.mixer.k_norm"].shape == (48,)
    assert "layers.2.hc2.in" not in params and "layers.2.feed_forward.w_down" not in params
    assert not any(k.startswith("layers.4.") for k in params)       # later passes of a looped layer own no weights
    # the rank of the decay's projection may be left to the checkpoint's shapes
    raw = json.load(open(f"{folder}/config.json"))
    for layer in raw["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["right"].pop("rank")
    json.dump(raw, open(f"{folder}/config.json", "w"))
    _, cfg2, params2 = load_model_folder(folder)
    assert cfg2.layers[1].mixer.right.rank == 0 and params2["layers.1.mixer.right.w_a1"].shape == (8, 96)
    with pytest.raises(ValueError, match="open"):
        fc.make_model_dir(raw, 5, str(tmp_path / "n"))


def test_a_model_without_copies_runs_the_block_with_unit_weights(tmp_path):
    folder = fc.make_model_dir(fc.FOV_D, 6, str(tmp_path / "m"))
    _, cfg, params = load_model_folder(folder)
    from geneinfer_b200.weights.plan import fovezen_weight_plan
    assert cfg.streams is None and not any(".hc" in r.name for r in fovezen_weight_plan(cfg).rules)
    assert params["layers.1.hc1.mix"].tolist() == [[1.0]] and params["layers.1.hc2.out"].tolist() == [1.0]


def test_plain_model_one_copy_with_unit_weights_is_a_plain_residual_stream(tmp_path):
    """The oracle's two readings of a layer agree where they must: one copy with in = out = mix = 1 is x + f(N(x))."""
    cfg = copy.deepcopy(fc.FOV_D)
    folder = fc.make_model_dir(cfg, 7, str(tmp_path / "m"))
    w, raw = pf.load(folder)
    toks = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5, 8, 9, 7, 9]
    plain = pf.forward(w, raw, toks)
    raw1 = dict(raw, streams=1)
    w1 = dict(w)
    for i, layer in enumerate(raw["layers"]):
        for c in ("hc1", "hc2") if layer["mlp"] else ("hc1",):
            w1[f"l{i}.{c}.in"], w1[f"l{i}.{c}.out"], w1[f"l{i}.{c}.mix"] = torch.ones(1), torch.ones(1), torch.ones(1, 1)
    assert torch.allclose(pf.forward(w1, raw1, toks), plain, rtol=0, atol=1e-12)


def test_plain_model_is_causal_and_its_loop_reuses_weights(tmp_path):
    folder = fc.make_model_dir(fc.FOV_A, 8, str(tmp_path / "m"))
    w, raw = pf.load(folder)
    toks = list(range(40, 75))
    full = pf.forward(w, raw, toks)
    assert torch.allclose(pf.forward(w, raw, toks[:20]), full[:20], rtol=0, atol=1e-9)
    after = []
    pf.forward(w, raw, toks, layers_out=after)
    assert len(after) == len(pf.layer_order(raw)) == 8 and pf.layer_order(raw) == [0, 1, 0, 1, 0, 1, 2, 3]
    once = pf.forward(w, dict(raw, loop=None), toks)
    assert float((once - full).abs().max()) > 1e-3
