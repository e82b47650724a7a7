"""Pinorax's configuration, weight plan, random-weights writer and plain implementation (no GPU)."""
import copy
import json
import os

import pytest
import torch

import pinorax_configs as pc
import plain_pinorax as pp
from geneinfer_b200.config import ConfigError, parse_config
from geneinfer_b200.weights import load_model_folder


def test_config_round_trip_and_translation():
    for raw in (pc.PIN_A, pc.PIN_B, pc.PIN_C, pc.PIN_D):
        arch, cfg = parse_config(raw)
        assert arch.name == "Pinorax" and cfg.to_json() == raw
        spec = cfg.model_spec()
        spec.validate()
        n = len(raw["layers"])
        assert len(spec.layers) == n and not spec.tie_word_embeddings and not spec.open_ended
        assert spec.max_position == raw["max_positions"] and spec.embedding_scale == 1.0
        assert spec.embedding_position.kind == "learned" and spec.embedding_position.params["positions"] == raw["max_positions"]
        assert spec.logit_transform.kind == "softcap" and spec.logit_transform.params["cap"] == raw["logit_softcap"]
        assert spec.final_norm.kind == "rmsnorm_scalar"
        for i, (layer, entry) in enumerate(zip(spec.layers, raw["layers"])):
            assert layer.block == "parallel" and layer.feed_forward_norm is None and layer.mixer_norm.kind == "rmsnorm_scalar"
            assert layer.block_params == {"residual_mult": raw["residual_mult"], "depth_slot": i + 1, "depth_slots": n + 1}
            p, m = layer.mixer.params, entry["mixer"]
            assert layer.mixer.kind == "latent_attention" and p["q_rank"] is None and p["rotary_dim"] == 0 and p["window"] is None
            assert (p["num_heads"], p["head_dim"], p["value_dim"], p["kv_rank"], p["scale"]) == \
                (m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["scale"])
            assert p["sink"] == "learned" and p["output_gate"] is True
            mlp = entry["mlp"]
            assert (layer.feed_forward is None) == (mlp is None)
            if mlp and mlp["kind"] == "dense":
                f = layer.feed_forward
                assert f.kind == "gated_mlp" and f.params["bias"] and f.params["activation"] == "silu" and f.params["intermediate_size"] == mlp["ff"]
            elif mlp:
                f = layer.feed_forward.params
                assert layer.feed_forward.kind == "routed_experts" and f["router"] == "table" and f["activation"] == "capped_swish"
                assert (f["experts"], f["top"], f["intermediate_size"], f["activation_limit"]) == \
                    (mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"], mlp["expert"]["limit"])
                if "shared" in mlp:
                    assert (f["shared"]["intermediate_size"], f["shared"]["activation_limit"]) == (mlp["shared"]["ff"], mlp["shared"]["limit"])
                else:
                    assert f["shared"] is None


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][0].update(type="sliding"), "unknown type"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "exceeds the number of experts"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "unknown kind"),
    (lambda c: c["layers"][0]["mlp"]["expert"].update(limit=0.0), "limit must be positive"),
    (lambda c: c["layers"][0]["mlp"]["shared"].pop("limit"), "limit"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mlp"].pop("ff"), "ff"),
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c.update(logit_softcap=0), "logit_softcap must be positive"),
    (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c.update(layers=[]), "at least one layer"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused(change, text):
    raw = copy.deepcopy(pc.PIN_A)
    change(raw)
    with pytest.raises(ConfigError, match=text):
        parse_config(raw)


def test_random_weights_folder_loads_by_name(tmp_path):
    folder = pc.make_model_dir(pc.PIN_A, 3, str(tmp_path / "m"))
    arch, cfg, params = load_model_folder(folder)
    assert arch.name == "Pinorax"
    assert tuple(params["layers.0.feed_forward.w_gate_up"].shape) == (5, 80, 96)
    assert tuple(params["layers.0.feed_forward.w_down"].shape) == (5, 96, 40)
    assert tuple(params["layers.0.feed_forward.shared.w_gate_up"].shape) == (112, 96)
    assert tuple(params["layers.0.mixer.w_down"].shape) == (3 * 24 + 48 + 3 * 40, 96)
    assert tuple(params["layers.1.feed_forward.b_gate_up"].shape) == (272,) and tuple(params["layers.1.feed_forward.b_down"].shape) == (96,)
    assert params["layers.0.mixer_norm.weight"].numel() == 1 and params["final_norm.weight"].numel() == 1
    assert [params[f"layers.{i}.depth_weights"].numel() for i in range(6)] == [2, 3, 4, 5, 6, 7]
    assert tuple(params["embedding_position.table"].shape) == (512, 96)
    assert not any(k.startswith("layers.2.feed_forward") for k in params) and "layers.3.feed_forward.shared.w_down" not in params
    table = params["layers.5.feed_forward.table"]
    assert table.dtype == torch.int32 and tuple(table.shape) == (190, 3) and int(table.min()) >= 0 and int(table.max()) < 7
    ordered = table.sort(dim=1).values
    assert not bool((ordered[:, 1:] == ordered[:, :-1]).any()) and len(set(table[:, 0].tolist())) > 1
    assert json.load(open(os.path.join(folder, "config.json")))["architecture"] == "Pinorax"


def test_plain_model_mechanisms():
    """The plain implementation against closed forms: it is what the engine is compared with."""
    g = torch.Generator().manual_seed(2)
    x = torch.randn(4, 10, generator=g, dtype=pp.F)
    n = pp.scalar_norm(x, torch.tensor(1.5, dtype=pp.F), 0.0)
    assert torch.allclose((n * n).mean(-1), torch.full((4,), 2.25, dtype=pp.F))
    # one key and a sink of the same score share the weight
    p = pp.softmax_with_sink(torch.zeros(2, 3, 3, dtype=pp.F), torch.tensor([0.0, -1e9], dtype=pp.F))
    assert abs(float(p[0, 0, 0]) - 0.5) < 1e-12 and abs(float(p[1, 0, 0]) - 1.0) < 1e-12 and float(p[0, 0, 1]) == 0.0
    assert abs(float(p[0, 2].sum()) - 0.75) < 1e-12
    # the capped activation: gate 5 is cut to 2, up -7 to -2
    one = torch.ones(1, 1, dtype=pp.F)
    y = pp.capped_expert(one, 5 * one, -7 * one, one, 2.0)
    assert abs(float(y) - 2.0 * float(torch.sigmoid(torch.tensor(3.404, dtype=pp.F))) * -1.0) < 1e-12
    assert abs(float(pp.softcap(torch.tensor(1e9, dtype=pp.F), 7.0)) - 7.0) < 1e-9
    r = [torch.full((1, 2), float(v), dtype=pp.F) for v in (1, 10, 100)]
    assert pp.depth_average(r, torch.tensor([1.0, 2.0, 3.0], dtype=pp.F)).tolist() == [[321.0, 321.0]]


def test_plain_model_runs_and_is_causal(tmp_path):
    folder = pc.make_model_dir(pc.PIN_C, 5, str(tmp_path / "m"))
    cfg, w = pp.load(folder)
    tokens = [5, 9, 130, 0, 77, 5, 31]
    logits, after = pp.forward(cfg, w, tokens)
    assert tuple(logits.shape) == (7, 131) and tuple(after.shape) == (3, 7, 100) and float(logits.abs().max()) < 4.0
    shorter, _ = pp.forward(cfg, w, tokens[:4])
    assert torch.allclose(shorter, logits[:4], atol=1e-12)
