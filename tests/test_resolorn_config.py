"""Configuration and registry of the Resolorn family, and its plain implementation's pieces (no GPU)."""
import copy
import json
import math

import pytest
import torch

import plain_resolorn as plain
import tiny_resolorn as tr


def test_configuration_reads_every_size_and_writes_it_back():
    from rust_mlx_b200.config import ResolornConfig
    from rust_mlx_b200.registry import build_model_spec, find_architecture
    for raw, _ in tr.CONFIGS.values():
        cfg = ResolornConfig.from_dict(raw)
        assert json.loads(json.dumps(cfg.to_dict())) == raw
        assert find_architecture(raw).name == "Resolorn"
        spec = build_model_spec(cfg)
        names = {p.name: tuple(p.shape) for p in spec.all_param_specs()}
        for i, layer in enumerate(raw["layers"]):
            m = layer["mixer"]
            assert names[f"l{i}.mix.uk"] == (m["heads"] * m["dim"], m["kv_rank"])
            assert names[f"l{i}.mix.uv"] == (m["heads"] * m["vdim"], m["kv_rank"])
            assert (f"l{i}.mix.dkv" in names) == ("kv_from" not in m)
            assert (f"l{i}.mlp.gate" in names) == (layer["mlp"] is not None and layer["mlp"]["kind"] == "dense")
        assert names["pos"] == (raw["max_positions"], raw["width"]) and names["head"] == (raw["vocab"], raw["width"])


def test_a_reading_layer_keeps_the_writers_latents_for_its_own_window():
    from rust_mlx_b200.config import ResolornConfig
    from rust_mlx_b200.registry import build_model_spec
    cfg = ResolornConfig.from_dict(tr.R1)
    assert cfg.cache_windows() == {0: 33, 2: 0}
    spec = build_model_spec(cfg)
    assert [c.cache for c in spec.schedule] == [0, 0, 2]
    specs = spec.cache_specs()
    assert specs[0].window == 33 and specs[0].head_dim == 32 and not specs[0].values and specs[2].window == 0
    assert spec.blocks[0].mixer.window == 20 and spec.blocks[1].mixer.window == 33


def test_every_problem_of_a_configuration_is_reported():
    from rust_mlx_b200.config import ConfigError, ResolornConfig
    bad = copy.deepcopy(tr.R2)
    del bad["width"]
    bad["layers"][0]["mixer"]["heads"] = 0
    bad["layers"][1]["mixer"]["kv_from"] = 2
    bad["layers"][2]["mlp"]["router"]["top"] = 9
    bad["layers"].append({"type": "convolution", "mixer": {}, "mlp": None})
    with pytest.raises(ConfigError) as e:
        ResolornConfig.from_dict(bad)
    text = str(e.value)
    assert "width" in text and "heads" in text and "convolution" in text
    bad = copy.deepcopy(tr.R2)
    bad["layers"][1]["mixer"]["kv_from"] = 2
    bad["layers"][2]["mlp"]["router"]["top"] = 9
    with pytest.raises(ConfigError) as e:
        ResolornConfig.from_dict(bad)
    assert "earlier layer" in str(e.value) and "top 9" in str(e.value)
    bad = copy.deepcopy(tr.R1)
    bad["layers"][1]["mixer"]["kv_rank"] = 48
    with pytest.raises(ConfigError, match="kv_rank"):
        ResolornConfig.from_dict(bad)


def test_plain_pieces():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    want = x / math.sqrt(12.5 + 0.1) * w
    assert torch.allclose(plain.rms_norm(x, w, 0.1), want)
    assert abs(plain.gelu_tanh(torch.tensor(1.0, dtype=torch.float64)).item() - 0.8411919906082768) < 1e-12
    v = plain.visible(5, 2)
    assert v.tolist() == [[True, False, False, False, False], [True, True, False, False, False],
                          [False, True, True, False, False], [False, False, True, True, False],
                          [False, False, False, True, True]]
    assert plain.visible(3, None).tolist() == [[True, False, False], [True, True, False], [True, True, True]]


def test_plain_router_takes_the_largest_and_weighs_them_among_themselves():
    torch.manual_seed(0)
    width, e = 8, 5
    w = {"m.router": torch.eye(e, width, dtype=torch.float64)}
    for k in range(e):
        w[f"m.e{k}.gate"] = torch.ones(1, width, dtype=torch.float64)
        w[f"m.e{k}.up"] = torch.ones(1, width, dtype=torch.float64)
        w[f"m.e{k}.down"] = torch.full((width, 1), float(k + 1), dtype=torch.float64)
    x = torch.zeros(1, width, dtype=torch.float64)
    x[0, 1], x[0, 3] = 2.0, 1.0           # logits: expert 1 -> 2, expert 3 -> 1, the others 0
    y = plain.routed_experts(x, w, "m", {"router": {"experts": e, "top": 2}})
    s = 3.0
    unit = plain.silu(torch.tensor(s, dtype=torch.float64)) * s
    p1 = math.exp(2.0) / (math.exp(2.0) + math.exp(1.0))
    assert torch.allclose(y, torch.full((1, width), 1.0, dtype=torch.float64) * unit * (p1 * 2 + (1 - p1) * 4))
