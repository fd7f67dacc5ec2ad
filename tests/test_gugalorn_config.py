"""Gugalorn without a GPU: configuration, tensor names, and the plain implementation's pieces on hand-made numbers."""
import math

import pytest
import torch

import plain_gugalorn as plain
import tiny_gugalorn as tg


def test_nested_configuration_is_read_and_written_back():
    from rust_mlx_b200.config import ConfigError, GugalornConfig
    from rust_mlx_b200.registry import find_architecture
    for raw, _ in tg.CONFIGS.values():
        assert find_architecture(raw).name == "Gugalorn"
        cfg = GugalornConfig.from_dict(raw)
        assert cfg.to_dict() == GugalornConfig.from_dict(cfg.to_dict()).to_dict()
        assert len(cfg.layers) == len(raw["layers"]) and cfg.vocab_size == raw["vocab"]
    cfg = GugalornConfig.from_dict(tg.G1)
    assert cfg.canon_taps == 3 and cfg.embedding_scale == 0.5 and cfg.layers[1].mixer.left.rot_dims == 8
    assert cfg.layers[1].mixer.right_scale == 1.3 and cfg.layers[0].ff == 48 and cfg.layers[1].ff == 0
    assert GugalornConfig.from_dict(tg.G3).canon_taps == 0
    bad = {"architecture": "Gugalorn", "vocab": 10, "width": 8, "norm": {"eps": 0.0},
           "layers": [tg.ssm(3, 4, 8, 2, 2, 5), tg.par((3, 2, 8, 8, 3, 10.0, 1.0), (1, 4, 4)), {"type": "other", "mixer": {}}]}
    with pytest.raises(ConfigError) as e:
        GugalornConfig.from_dict(bad)
    assert "unknown mixer" in str(e.value)
    del bad["layers"][2]
    with pytest.raises(ConfigError) as e:
        GugalornConfig.from_dict(bad)
    msg = str(e.value)
    assert "groups" in msg and "norm groups" in msg and "kv heads" in msg and "even" in msg and "eps" in msg


def test_tensor_names_shapes_and_caches():
    from rust_mlx_b200.config import GugalornConfig
    from rust_mlx_b200.registry import build_model_spec
    spec = build_model_spec(GugalornConfig.from_dict(tg.G1))
    shapes = {s.name: tuple(s.shape) for s in spec.all_param_specs()}
    assert shapes["embed"] == (211, 64) and shapes["final.norm"] == (64,)
    assert shapes["l0.mix.in"] == (2 * 32 + 2 * 16 + 4, 64) and shapes["l0.mix.conv"] == (32 + 32, 2) and shapes["l0.canon1"] == (64, 3)
    assert shapes["l2.mix.in"] == (2 * 24 + 2 * 3 * 24 + 6, 64) and shapes["l2.mix.norm"] == (24,) and shapes["l2.mix.A_log"] == (6,)
    assert shapes["l1.mix.left.q"] == (64, 64) and shapes["l1.mix.left.k"] == (16, 64) and shapes["l1.mix.left.q.norm"] == (64,)
    assert shapes["l1.mix.left.g"] == (64, 64) and shapes["l1.mix.right.lower"] == (16,) and shapes["l1.mix.right.norm"] == (12,)
    assert shapes["l3.mix.left.v"] == (48, 64) and shapes["l3.mix.left.o"] == (64, 48) and shapes["l3.mlp.down"] == (64, 40)
    assert "l1.norm2" not in shapes and "l2.norm2" not in shapes and "l0.norm2" in shapes and "head" not in shapes
    specs = spec.cache_specs()
    kinds = [specs[i].kind for i in sorted(specs)]
    # every layer: the input convolution's ring, then what its mixer keeps
    assert kinds == ["state", "state", "state"] + ["state", "paged", "state"] + ["state", "state", "state"] + ["state", "paged", "state"]
    assert specs[4].head_dim == 16 and specs[10].head_dim == 24 and specs[2].state_shape == (4, 8, 16)


def test_plain_pieces_on_hand_made_numbers():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(plain.rms(x, 0.0), x / math.sqrt(12.5))
    h = torch.tensor([[1.0], [2.0], [4.0]], dtype=torch.float64)
    w = torch.tensor([[10.0, 1.0]], dtype=torch.float64)          # the last column is the current token's
    assert plain.causal_conv(h, w).flatten().tolist() == [1.0, 12.0, 24.0]
    # a quarter turn of the pair (0, 2) at position 1 with frequency pi / 2; numbers from dims on pass
    q = torch.tensor([[[1.0, 5.0, 0.0, 7.0, 9.0]]], dtype=torch.float64)
    r = plain.rotate(q, torch.tensor([1]), 4, 1.0)[0, 0]      # base 1: every pair turns by the position, one radian here
    c, s = math.cos(1.0), math.sin(1.0)
    assert torch.allclose(r, torch.tensor([c, 5 * c - 7 * s, s, 7 * c + 5 * s, 9.0], dtype=torch.float64))
    # one key with score 0: weight exp(0) / (1 + exp(0)) = 1/2
    o = plain.sink_attention(torch.zeros(1, 1, 2, dtype=torch.float64), torch.ones(1, 1, 2, dtype=torch.float64),
                             torch.tensor([[[4.0, 6.0]]], dtype=torch.float64), 1.0)
    assert torch.allclose(o, torch.tensor([[[2.0, 3.0]]], dtype=torch.float64))
