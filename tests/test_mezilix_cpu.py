"""CPU: configuration, registry, tensor naming, page table bookkeeping and the oracle's own consistency for the
Mezilix family (the engine itself is tested on the GPU in test_mezilix_gpu.py)."""
import json
import os

import pytest
import torch

from asd_b200.models import mezilix, registry
from oracle import mezilix_oracle as O


def test_config_round_trip_and_shapes():
    cfg = mezilix.tiny_config()
    d = cfg.to_dict()
    again = mezilix.MezilixConfig.from_dict(d, name="tiny")
    assert again == cfg
    shapes = mezilix.tensor_shapes(cfg)
    w = mezilix.random_weights(cfg, seed=0)
    assert set(w) == set(shapes) and all(tuple(w[k].shape) == tuple(v) for k, v in shapes.items())
    assert sum(t.numel() for t in w.values()) == cfg.params
    assert shapes["l1.dwa"] == (3,) and shapes["bigram"] == (cfg.buckets + 1, cfg.width)
    assert "l1.mlp.router" not in shapes                      # the second tiny layer has no feed-forward
    # the oracle's random model names the same tensors
    assert set(O.random_model(d, seed=0)) == set(shapes)


def test_layer_without_feed_forward_or_mask():
    d = mezilix.tiny_config().to_dict()
    d["layers"][0]["mlp"] = None
    del d["layers"][1]["mixer"]["mask"]
    cfg = mezilix.MezilixConfig.from_dict(d)
    assert cfg.layers[0].experts == 0 and cfg.layers[1].window == mezilix.NO_WINDOW
    d["layers"][0]["type"] = "something_else"
    with pytest.raises(ValueError):
        mezilix.MezilixConfig.from_dict(d)


def test_registry_reads_checkpoint_directories(tmp_path):
    a = tmp_path / "m"
    a.mkdir()
    (a / "config.json").write_text(json.dumps(mezilix.tiny_config().to_dict()))
    fam, cfg = registry.read_config(str(a))
    assert fam.name == "mezilix" and "float32" in fam.dtypes and cfg.width == 64 and cfg.name == "m"
    b = tmp_path / "q"
    b.mkdir()
    (b / "config.json").write_text(json.dumps({
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 128, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 256, "vocab_size": 512}))
    fam, cfg = registry.read_config(str(b))
    assert fam.name == "qwen2" and cfg.head_dim == 32 and fam.dtypes == ("bfloat16",)
    assert registry.family_of_config(cfg).name == "qwen2"
    assert registry.family_of_config(mezilix.tiny_config()).name == "mezilix"
    (b / "config.json").write_text(json.dumps({"architectures": ["Other"]}))
    with pytest.raises(ValueError):
        registry.read_config(str(b))


def test_pack_layer_checks_shapes_and_stacks_experts():
    cfg = mezilix.tiny_config()
    w = mezilix.random_weights(cfg, seed=1)
    t = mezilix.pack_layer(w, cfg, 0, "cpu", torch.float32)
    l = cfg.layers[0]
    assert t["wqd"].shape == (l.q_rows + l.cache_row, cfg.width)
    assert t["w_up"].shape == (l.experts, l.ff, cfg.width) and t["w_down"].shape == (l.experts, cfg.width, l.ff)
    assert torch.equal(t["w_up"][2], w["l0.mlp.e2.up"].float())
    assert mezilix.pack_layer(w, cfg, 1, "cpu", torch.float32)["router"] is None
    bad = dict(w)
    bad["l0.mix.uk"] = bad["l0.mix.uk"][:-1]
    with pytest.raises(ValueError):
        mezilix.pack_layer(bad, cfg, 0, "cpu", torch.float32)


def test_page_table_allocates_frees_and_reuses():
    from asd_b200._lib import AsdError
    from asd_b200.engine import PageTable
    pt = PageTable(max_seqs=2, max_pages=4, page_size=4, device="cpu", num_pages=5, dynamic=True)
    a, b = pt.alloc_slot(), pt.alloc_slot()
    with pytest.raises(AsdError):
        pt.alloc_slot()
    pt.reserve(a, 9)                                   # 3 pages
    pt.reserve(a, 5)                                   # shrinking requests change nothing
    pt.reserve(b, 8)                                   # 2 pages: pool empty
    assert pt.pages_in_use() == 5
    used = set(pt.table[a, :3].tolist()) | set(pt.table[b, :2].tolist())
    assert len(used) == 5
    with pytest.raises(AsdError):
        pt.reserve(b, 9)                               # no page left
    with pytest.raises(AsdError):
        pt.reserve(a, 17)                              # beyond the per-sequence limit
    pt.free_slot(a)
    pt.reserve(b, 16)
    assert pt.pages_in_use() == 4 and pt.alloc_slot() == a
    st = PageTable(max_seqs=3, max_pages=2, page_size=16, device="cpu")
    assert sorted(st.table.flatten().tolist()) == list(range(6))
    with pytest.raises(AsdError):
        st.alloc_slot()


def test_oracle_mechanisms_on_hand_made_inputs():
    # pair table: first token takes the last row; later ones the hashed row
    emb, tab = torch.arange(12.0).reshape(6, 2), 100 + torch.arange(8.0).reshape(4, 2)
    x = O.bigram_embed([1, 4, 4], emb, tab, buckets=3, mul_prev=2, mul_cur=5)
    assert torch.equal(x[0], emb[1] + tab[3]) and torch.equal(x[1], emb[4] + tab[(1 * 2 + 4 * 5) % 3])
    assert torch.equal(x[2], emb[4] + tab[(4 * 2 + 4 * 5) % 3])
    # token shift with weight 1 is the previous row, zeros first
    h = torch.arange(6.0).reshape(3, 2)
    assert torch.equal(O.token_shift(h, torch.ones(2)), torch.tensor([[0.0, 0.0], [0.0, 1.0], [2.0, 3.0]]))
    # rotation keeps norms and leaves the tail alone; position 0 is the identity
    v = torch.randn(4, 10, dtype=torch.float64)
    r = O.rotate_half_rope(v, torch.arange(4), 6, 100.0)
    assert torch.allclose(r[0], v[0]) and torch.equal(r[:, 6:], v[:, 6:])
    assert torch.allclose(r[:, :6].norm(dim=-1), v[:, :6].norm(dim=-1))
    # scalar-gain norm
    y = O.scalar_rms_norm(torch.tensor([[3.0, 4.0]]), torch.tensor(2.0), 0.0)
    assert torch.allclose(y, torch.tensor([[3.0, 4.0]]) / (12.5 ** 0.5) * 2)
    # depth average
    assert torch.equal(O.depth_average([torch.ones(2), 2 * torch.ones(2)], torch.tensor([0.5, 0.25])), torch.ones(2))
