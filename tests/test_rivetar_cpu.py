"""CPU: the Rivetar family's configuration, registry entry, tensor packing and execution order, and the plain
restatement's own mechanisms on inputs made by hand (so that the oracle the GPU tests lean on is itself pinned)."""
import json
import math

import pytest
import torch

from oracle import rivetar_oracle as O


def test_config_round_trip_and_registry(tmp_path):
    from asd_b200.models import registry
    from asd_b200.models.rivetar import RivetarConfig, tensor_shapes, tiny_config
    cfg = tiny_config()
    d = cfg.to_dict()
    assert d["architecture"] == "Rivetar"
    back = RivetarConfig.from_dict(d, name="tiny").with_shapes(tensor_shapes(cfg))
    assert back == cfg
    fam = registry.family_of_dict(d)
    assert fam.name == "rivetar" and "rivetar" in fam.components and set(fam.dtypes) == {"bfloat16", "float32"}
    assert registry.family_of_config(cfg).name == "rivetar"
    # a checkpoint directory: the size that only a tensor's shape gives comes from the safetensors header
    (tmp_path / "config.json").write_text(json.dumps(d))
    import struct
    shapes = tensor_shapes(cfg)
    header, off = {}, 0
    for k, s in shapes.items():
        n = 2 * math.prod(s)
        header[k] = {"dtype": "BF16", "shape": list(s), "data_offsets": [off, off + n]}
        off += n
    hj = json.dumps(header).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + b"\0" * off)
    fam2, cfg2 = registry.read_config(str(tmp_path))
    assert fam2.name == "rivetar" and cfg2.layers[0].decay_rank == cfg.layers[0].decay_rank


def test_unknown_mixer_layout_and_span_are_refused():
    from asd_b200.models.rivetar import RivetarConfig, tiny_config
    d = tiny_config().to_dict()
    bad = json.loads(json.dumps(d))
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ValueError):
        RivetarConfig.from_dict(bad)
    bad = json.loads(json.dumps(d))
    bad["layers"][1]["mixer"]["rot"]["layout"] = "thirds"
    with pytest.raises(ValueError):
        RivetarConfig.from_dict(bad)
    bad = json.loads(json.dumps(d))
    bad["loop"] = {"start": 2, "stop": 5, "times": 2}
    with pytest.raises(ValueError):
        RivetarConfig.from_dict(bad)


def test_execution_order_of_a_repeated_span():
    from asd_b200.models.rivetar import RivetarConfig, tiny_config
    cfg = tiny_config(loop=(1, 3, 3))
    assert cfg.runs() == [(0, -1), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2)]
    assert tiny_config(loop=None).runs() == [(0, -1), (1, -1), (2, -1)]
    assert [(i, t) for i, t, _ in O.layer_runs(cfg.to_dict())] == [(i, None if t < 0 else t) for i, t in cfg.runs()]
    assert [first for _, _, first in O.layer_runs(cfg.to_dict())] == [False, True, False, True, False, True, False]
    # cached bytes count every execution
    one = RivetarConfig.from_dict(tiny_config(loop=None).to_dict())
    assert cfg.kv_bytes_per_token() == one.kv_bytes_per_token() + 2 * (cfg.layers[1].cache_row + cfg.layers[2].cache_row) * 2


def test_packing_stacks_the_input_projections():
    from asd_b200.models.rivetar import pack, random_weights, tensor_shapes, tiny_config
    cfg = tiny_config()
    w = random_weights(cfg, seed=1)
    p = pack(w, cfg, "cpu", torch.float32)
    g, a, l = cfg.layers
    assert p[(0, "w_in")].shape == (2 * g.heads * g.dim + 2 * g.heads * g.vdim + g.decay_rank, cfg.width)
    assert torch.equal(p[(0, "w_in")][g.heads * g.dim:2 * g.heads * g.dim], w["l0.mix.k"].float())
    assert p[(1, "w_in")].shape == (a.heads * a.dim + a.kv_heads * (a.dim + a.vdim), cfg.width)
    assert p[(2, "w_in")].shape == (l.q_rank + l.kv_rank + l.rot_dim, cfg.width)
    assert p[(2, "w_uk")].shape == (l.heads, l.kv_rank, l.dim)
    assert torch.equal(p[(2, "w_uk")][1, :, 3], w["l2.mix.uk"].float()[l.dim + 3])
    assert p[(0, "w_decay")].dtype == torch.float32 and p[(-1, "loop_step")].shape == (2, cfg.width)
    assert (0, "norm2") in p and (0, "w_up") in p and (1, "norm2") not in p and (1, "w_up") not in p     # layer 1 has no feed-forward
    bad = dict(w)
    bad["l1.mix.sink"] = torch.zeros(a.heads + 1)
    with pytest.raises(ValueError):
        pack(bad, cfg, "cpu", torch.float32)
    del bad["l1.mix.sink"]
    with pytest.raises(KeyError):
        pack(bad, cfg, "cpu", torch.float32)
    assert set(tensor_shapes(cfg)) == set(w)


# ------------------------------------------------------------------------------------------------ the oracle itself
def test_oracle_norms_and_polynomial_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(O.unit_rms(x, 0.0), x / math.sqrt(12.5))
    assert torch.allclose(O.offset_norm(x, torch.tensor([0.0, 1.0], dtype=torch.float64), 0.0),
                          torch.tensor([[3.0, 8.0]], dtype=torch.float64) / math.sqrt(12.5))
    z = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    got = O.polynorm(z, torch.tensor([2.0, 3.0, 5.0, 7.0], dtype=torch.float64), 0.0)
    want = 2 * z / math.sqrt(2.5) + 3 * z ** 2 / math.sqrt(8.5) + 5 * z ** 3 / math.sqrt(32.5) + 7
    assert torch.allclose(got, want)


def test_oracle_rotation_pairs_and_inverse():
    x = torch.arange(8, dtype=torch.float64).reshape(1, 8) + 1
    pos = torch.tensor([3])
    for layout, pairs in (("interleaved", [(0, 1), (2, 3)]), ("halves", [(0, 2), (1, 3)])):
        y = O.rotate_pairs(x, pos, 4, 100.0, layout)
        for i, (a, b) in enumerate(pairs):
            ang = 3 * 100.0 ** (-2 * i / 4)
            assert math.isclose(y[0, a], x[0, a] * math.cos(ang) - x[0, b] * math.sin(ang))
            assert math.isclose(y[0, b], x[0, b] * math.cos(ang) + x[0, a] * math.sin(ang))
        assert torch.equal(y[0, 4:], x[0, 4:])
        assert torch.allclose(O.rotate_pairs(y, pos, 4, 100.0, layout, sign=-1.0), x)


def test_oracle_mask_window_and_kept_positions():
    see = O.visibility(torch.arange(8), {"size": 3, "keep_first": 2})
    assert see[7].tolist() == [True, True, False, False, False, True, True, True]
    assert see[3].tolist() == [True, True, True, True, False, False, False, False]
    assert O.visibility(torch.arange(4), None)[3].tolist() == [True] * 4
    assert O.visibility(torch.arange(4), {"size": 1})[3].tolist() == [False, False, False, True]


def test_oracle_recurrence_by_hand():
    """one head, one key channel, one value channel: S_t = alpha S_(t-1) + k v, o = S q / sqrt(1)"""
    m = {"heads": 1, "dim": 1, "vdim": 1, "tau": 2.0}
    one = torch.ones(1, 1, dtype=torch.float64)
    w = {"q": one, "k": 2 * one, "v": 3 * one, "g": one, "o": one, "norm": torch.ones(1, dtype=torch.float64),
         "a1": one, "a2": torch.zeros(1, 1, dtype=torch.float64), "a2.b": torch.zeros(1, dtype=torch.float64)}
    h = torch.ones(3, 1, dtype=torch.float64)
    _, S = O.gated_linear_attention(h, w, m, 0.0)
    alpha = math.sqrt(0.5)
    assert math.isclose(S.item(), 6 * (1 + alpha + alpha ** 2))
    _, S2 = O.gated_linear_attention(h[:1], w, m, 0.0, state=O.gated_linear_attention(h[:2], w, m, 0.0)[1])
    assert math.isclose(S2.item(), S.item())


def test_oracle_sink_takes_weight_without_a_value():
    """one position, one head: the softmax over {score, sink} gives the value the weight 1 / (1 + exp(sink - score))"""
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "rot": {"base": 10.0, "dims": 2}, "scale": 1.0}
    eye = torch.eye(2, dtype=torch.float64)
    w = {"q": eye, "k": eye, "v": eye, "o": eye, "sink": torch.tensor([1.5], dtype=torch.float64)}
    h = torch.tensor([[1.0, 2.0]], dtype=torch.float64)
    out = O.windowed_attention(h, torch.tensor([0]), w, m)
    assert torch.allclose(out, h / (1 + math.exp(1.5 - 5.0)))
