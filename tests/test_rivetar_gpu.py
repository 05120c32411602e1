"""GPU: the Rivetar engine against the plain restatement in oracle/rivetar_oracle.py (fp64, whole sequences, no cache).
Every test makes its own small configuration and random weights.  The fp32 engine is held to 2e-4 of the logits'
spread, which a single key missed or double-counted among hundreds, a window or a kept position off by one, a lost
state, a left-out sink or a stale page all exceed; the bf16 engine to what its roundings allow."""
import copy
import json
import os
import struct
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import rivetar_oracle as O  # noqa: E402


# ------------------------------------------------------------------------------------------------ configurations
def latent(heads=2, dim=16, rot_dim=8, vdim=24, kv_rank=32, q_rank=40, base=1000.0, scale=0.2, ff=40, rot_dims=None,
           layout=None):
    rot = {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}
    if layout:
        rot["layout"] = layout
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "rot": rot, "scale": scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def gla(heads=2, dim=24, vdim=16, tau=8.0, ff=0, decay_rank=8):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": decay_rank},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def window(heads=4, kv_heads=2, dim=16, vdim=24, size=9, keep_first=3, base=1000.0, rot_dims=8, scale=0.25, ff=48,
           layout=None, mask=True):
    rot = {"base": base, "dims": rot_dims}
    if layout:
        rot["layout"] = layout
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot, "scale": scale}
    if mask:
        m["mask"] = {"size": size, "keep_first": keep_first}
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, width=64, vocab=96, eps=1e-5, scale=4.0, cap=20.0, loop=None):
    d = {"architecture": "Rivetar", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": scale},
         "layers": layers}
    if cap:
        d["logit_softcap"] = cap
    if loop:
        d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return d


# all three mixers, a repeated span in the middle
SMALL = config([latent(), gla(), window(), latent(heads=3, dim=8, rot_dim=16, vdim=8, kv_rank=40, q_rank=24, ff=0)],
               loop=(1, 3, 2))
# sizes that are multiples of nothing; the span starts at the first layer and runs three times; one key/value head per
# query head and one for all; rotation over a part of the head and over all of it; no cap on the logits
ODD = config([window(heads=3, kv_heads=3, dim=10, vdim=6, size=5, keep_first=0, rot_dims=10, ff=50),
              gla(heads=3, dim=20, vdim=7, tau=3.0, ff=9, decay_rank=5),
              latent(heads=5, dim=6, rot_dim=10, vdim=6, kv_rank=33, q_rank=17, rot_dims=6, ff=0),
              window(heads=6, kv_heads=1, dim=12, vdim=34, size=1000, keep_first=2, rot_dims=4, ff=0),
              gla(heads=1, dim=40, vdim=66, tau=1.0, ff=21, decay_rank=3)],
             width=72, vocab=101, eps=1e-3, scale=1.0, cap=0.0, loop=(0, 2, 3))
# the other pairing of rotated coordinates, a span that is the whole model and runs once, attention without a mask
HALVES = config([latent(layout="halves"), window(layout="halves", mask=False), gla(ff=32)], loop=(0, 3, 1))
PLAIN = config([gla(ff=32), window(), latent()])       # no repeated span at all


def make_engine(cfg_dict, w, dtype=torch.float32, max_tokens=64, max_seq_len=512, page_size=16, num_pages=None,
                max_seqs=4, ring=1, tc=1):
    from asd_b200.engine import RivetarEngine
    from asd_b200.models.rivetar import RivetarConfig
    cfg = RivetarConfig.from_dict(cfg_dict).with_shapes({k: tuple(v.shape) for k, v in w.items()})
    eng = RivetarEngine(cfg, max_seqs=max_seqs, max_seq_len=max_seq_len, max_tokens=max_tokens, page_size=page_size,
                        dtype=dtype, dynamic_pages=True, num_pages=num_pages, ring=ring)
    eng.load_weights(w)
    eng.set_option("tc_linear", tc)
    return eng


def close(eng):
    """no kernel of the engine gave up a wait"""
    eng.check_device()
    eng.close()


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def rel_err(got, want):
    got, want = got.double().cpu(), want.double()
    return ((got - want).norm() / want.norm()).item(), ((got - want).abs().max() / want.std()).item()


def feed(eng, slot, ids, cuts, start=0):
    """feeds ids in portions of the given sizes (the rest in one go), all logits wanted"""
    out, a = [], 0
    sizes = list(cuts)
    while a < len(ids):
        n = sizes.pop(0) if sizes else len(ids) - a
        n = min(n, len(ids) - a)
        eng.reserve(slot, start + a + n)
        out.append(eng.forward_ragged([(slot, start + a, ids[a:a + n], list(range(n)))]))
        a += n
    return torch.cat(out, 0)


def run_whole(cfg_dict, w, ids, **kw):
    eng = make_engine(cfg_dict, w, **kw)
    slot = eng.open_sequence()
    got = feed(eng, slot, ids, [])
    close(eng)
    return got


# ------------------------------------------------------------------------------------------------ whole prompts
@pytest.mark.parametrize("cfg_dict", [SMALL, ODD, HALVES, PLAIN], ids=["small", "odd", "halves", "plain"])
def test_whole_prompt_logits_and_every_layer_execution(cfg_dict):
    w = O.random_model(cfg_dict, seed=1)
    ids = tokens(45, cfg_dict["vocab"], 2)
    ref, streams = O.forward(cfg_dict, w, ids)
    eng = make_engine(cfg_dict, w)
    slot = eng.open_sequence()
    eng.reserve(slot, len(ids))
    got, st = eng.forward_ragged([(slot, 0, ids, list(range(len(ids))))], layer_out=True)
    st = torch.cat(st, 1).cpu().double()
    assert st.shape[0] == len(O.layer_runs(cfg_dict))
    for i in range(st.shape[0]):           # the first execution that differs names the mechanism
        assert (st[i] - streams[i]).abs().max() <= 2e-4 * streams[i].abs().max(), f"stream leaving execution {i}"
    assert rel_err(got, ref)[1] < 2e-4
    close(eng)


# ------------------------------------------------------------------------------------------------ mechanisms alone
def test_embedding_scale_final_norm_and_cap_alone():
    """no layers: logits = cap * tanh(head . norm(embed * scale) / cap), with a cap small enough to bend them"""
    cfg = config([], width=40, vocab=50, scale=7.0, cap=2.5)
    w = O.random_model(cfg, seed=3)
    ids = tokens(20, 50, 4)
    ref, _ = O.forward(cfg, w, ids)
    assert ref.abs().max() > 1.5 and ref.abs().max() < 2.5
    assert rel_err(run_whole(cfg, w, ids), ref)[1] < 1e-4
    uncapped, _ = O.forward(config([], width=40, vocab=50, scale=7.0, cap=0.0), w, ids)
    assert rel_err(run_whole(config([], width=40, vocab=50, scale=7.0, cap=0.0), w, ids), uncapped)[1] < 1e-4


def test_polynomial_activation_alone():
    """a layer whose mixer is silenced (zero output projection, so the norm after it gives zero): what remains is the
    feed-forward; coefficients that make every power matter"""
    cfg = config([gla(ff=56)])
    w = O.random_model(cfg, seed=5)
    w["l0.mix.o"] = torch.zeros_like(w["l0.mix.o"])
    ids = tokens(33, 96, 6)
    for coeff in ([1.0, 0.0, 0.0, 0.0], [0.0, 1.0, 0.0, 0.0], [0.0, 0.0, 1.0, 0.0], [0.3, -0.8, 0.5, 0.25]):
        w["l0.mlp.act"] = torch.tensor(coeff)
        ref, _ = O.forward(cfg, w, ids)
        assert rel_err(run_whole(cfg, w, ids), ref)[1] < 2e-4, coeff


@pytest.mark.parametrize("entry", [gla(heads=3, dim=20, vdim=12, tau=2.0), gla(heads=1, dim=64, vdim=40, tau=30.0),
                                   gla(heads=2, dim=130, vdim=33, tau=16.0, decay_rank=1),
                                   gla(heads=1, dim=300, vdim=20, tau=50.0, decay_rank=2)], ids=["a", "b", "c", "wide"])
def test_gated_linear_attention_alone(entry):
    cfg = config([entry])
    w = O.random_model(cfg, seed=7)
    ids = tokens(70, 96, 8)
    ref, _ = O.forward(cfg, w, ids)
    assert rel_err(run_whole(cfg, w, ids, max_tokens=128), ref)[1] < 2e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_many_query_heads_per_key_value_head(dtype):
    """twenty query heads share each key/value head: more than one CTA's worth in the one-warp-per-pair kernel, a row
    tile that the group does not divide in the tensor-core kernel"""
    cfg = config([window(heads=40, kv_heads=2, dim=16, vdim=16, size=30, keep_first=2, rot_dims=16, ff=0)])
    w = O.random_model(cfg, seed=45)
    ids = tokens(80, 96, 46)
    ref, _ = O.forward(cfg, w, ids)
    for cuts in ([80], [60] + [1] * 20, [7] * 12):
        eng = make_engine(cfg, w, dtype=dtype, max_tokens=128)
        slot = eng.open_sequence()
        got = feed(eng, slot, ids, cuts)
        assert (rel_err(got, ref)[1] < 2e-4) if dtype == torch.float32 else (rel_err(got, ref)[0] < 5e-2)
        close(eng)


def test_latent_attention_alone_both_pairings():
    for layout in (None, "halves"):
        cfg = config([latent(heads=3, dim=12, rot_dim=12, vdim=10, kv_rank=24, q_rank=9, rot_dims=8, ff=0, layout=layout)])
        w = O.random_model(cfg, seed=9)
        ids = tokens(60, 96, 10)
        ref, _ = O.forward(cfg, w, ids)
        assert rel_err(run_whole(cfg, w, ids), ref)[1] < 2e-4
    # the two pairings are different functions: the oracle under one does not pass for the other
    other, _ = O.forward(config([latent(heads=3, dim=12, rot_dim=12, vdim=10, kv_rank=24, q_rank=9, rot_dims=8, ff=0)]), w, ids)
    assert rel_err(other.float(), ref)[1] > 1e-2


def test_windowed_attention_alone_sink_and_value_rotation():
    cfg = config([window(heads=4, kv_heads=2, dim=16, vdim=12, size=11, keep_first=2, ff=0)])
    w = O.random_model(cfg, seed=11)
    w["l0.mix.sink"] = torch.tensor([3.0, -2.0, 0.5, 6.0])
    ids = tokens(64, 96, 12)
    ref, _ = O.forward(cfg, w, ids)
    assert rel_err(run_whole(cfg, w, ids), ref)[1] < 2e-4
    # a left-out sink and unrotated values are far outside the tolerance
    w2 = dict(w)
    w2["l0.mix.sink"] = torch.full((4,), -1e4)
    assert rel_err(O.forward(cfg, w2, ids)[0].float(), ref)[1] > 1e-2
    flat = copy.deepcopy(cfg)
    flat["layers"][0]["mixer"]["rot"]["base"] = 1e30       # angles of all pairs but the first vanish
    assert rel_err(O.forward(flat, w, ids)[0].float(), ref)[1] > 1e-2


# ------------------------------------------------------------------------------------------------ cache and state
@pytest.mark.parametrize("cfg_dict", [SMALL, ODD], ids=["small", "odd"])
@pytest.mark.parametrize("page_size", [4, 16])
def test_prefill_then_decode_and_portions(cfg_dict, page_size):
    w = O.random_model(cfg_dict, seed=13)
    ids = tokens(61, cfg_dict["vocab"], 14)
    ref, _ = O.forward(cfg_dict, w, ids)
    for cuts in ([1] * 61, [40] + [1] * 21, [2] * 30, [3, 17, 2, 1, 1, 5, 2, 30], [16, 16, 16], [15, 17, 1, 16]):
        eng = make_engine(cfg_dict, w, page_size=page_size)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[1] < 2e-4, cuts
        close(eng)


def test_forward_larger_than_the_engine_step_is_cut_inside():
    w = O.random_model(SMALL, seed=15)
    ids = tokens(100, 96, 16)
    ref, _ = O.forward(SMALL, w, ids)
    assert rel_err(run_whole(SMALL, w, ids, max_tokens=24), ref)[1] < 2e-4


def test_batch_of_unequal_requests_equals_each_alone():
    w = O.random_model(SMALL, seed=17)
    seqs = [tokens(n, 96, 20 + n) for n in (31, 5, 1, 18)]
    refs = [O.forward(SMALL, w, s)[0] for s in seqs]
    eng = make_engine(SMALL, w, max_tokens=32)
    slots = [eng.open_sequence() for _ in seqs]
    first = [12, 5, 1, 2]
    for sl, s in zip(slots, seqs):
        eng.reserve(sl, len(s))
    a = eng.forward_ragged([(sl, 0, s[:f], list(range(f))) for sl, s, f in zip(slots, seqs, first)])
    b = eng.forward_ragged([(sl, f, s[f:], list(range(len(s) - f))) for sl, s, f in zip(slots, seqs, first) if len(s) > f])
    oa = ob = 0
    for s, f, ref in zip(seqs, first, refs):
        got = a[oa:oa + f]
        oa += f
        if len(s) > f:
            got = torch.cat([got, b[ob:ob + len(s) - f]], 0)
            ob += len(s) - f
        assert rel_err(got, ref)[1] < 2e-4
    close(eng)


def test_pages_slots_and_state_freed_and_used_again():
    """a pool with room for one request at a time: the second request gets the first one's slot, pages and recurrent
    state with the old contents still in them"""
    w = O.random_model(SMALL, seed=19)
    eng = make_engine(SMALL, w, page_size=4, num_pages=12, max_seqs=1, max_seq_len=48)
    for seed, n in ((30, 44), (31, 47), (32, 9), (33, 48), (34, 1)):
        ids = tokens(n, 96, seed)
        ref, _ = O.forward(SMALL, w, ids)
        slot = eng.open_sequence()
        assert slot == 0
        assert rel_err(feed(eng, slot, ids, [7, 1, 1, 13, 2]), ref)[1] < 2e-4
        eng.close_sequence(slot)
        assert eng.pages.pages_in_use() == 0
    from asd_b200._lib import AsdError
    slot = eng.open_sequence()
    with pytest.raises(AsdError):
        eng.reserve(slot, 49)
    close(eng)


def test_refeeding_recent_positions_finds_their_state():
    """a ring of states: after 30 tokens the last three are taken back and other tokens follow, as a verification
    step does after a rejected tail"""
    w = O.random_model(SMALL, seed=21)
    ids = tokens(30, 96, 22)
    new_tail = tokens(9, 96, 23)
    eng = make_engine(SMALL, w, ring=4)
    slot = eng.open_sequence()
    feed(eng, slot, ids, [11, 1, 6])
    got = feed(eng, slot, new_tail, [4, 1], start=27)
    ref, _ = O.forward(SMALL, w, ids[:27] + new_tail)
    assert rel_err(got, ref[27:])[1] < 2e-4
    close(eng)


def test_long_decoding_keeps_the_recurrent_state_and_passes_the_window():
    """slow decays (large tau): what the first tokens wrote is still in the state after hundreds of single-token steps"""
    cfg = config([gla(heads=2, dim=24, vdim=16, tau=200.0), window(size=20, keep_first=2, ff=0)])
    w = O.random_model(cfg, seed=25)
    ids = tokens(260, 96, 26)
    ref, _ = O.forward(cfg, w, ids)
    cut = copy.deepcopy(ids)
    cut[0] = (cut[0] + 1) % 96
    assert rel_err(O.forward(cfg, w, cut)[0][-1:].float(), ref[-1:])[1] > 1e-3      # the first token still matters
    eng = make_engine(cfg, w, page_size=8)
    slot = eng.open_sequence()
    assert rel_err(feed(eng, slot, ids, [5] + [1] * 255), ref)[1] < 2e-4
    close(eng)


# ------------------------------------------------------------------------------------------------ edges of the mask
def plant_pair(cfg, w, key_tok, query_tok, boost=400.0):
    """Makes the first layer's queries of ``query_tok`` point at the unrotated key coordinates of ``key_tok`` in every
    head, so that this one score exceeds all others by about ``boost`` wherever the key is visible."""
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    H, G, dk, rd = m["heads"], m["kv_heads"], m["dim"], m["rot"]["dims"]
    f = lambda t: t.double()
    sc = cfg["embedding"]["scale"]
    hk = O.offset_norm(f(w["embed"][key_tok]) * sc, f(w["l0.norm1"]), eps)
    hq = O.offset_norm(f(w["embed"][query_tok]) * sc, f(w["l0.norm1"]), eps)
    k = (f(w["l0.mix.k"]) @ hk).reshape(G, dk)
    q = f(w["l0.mix.q"]).reshape(H, dk, -1).clone()
    for h in range(H):
        kk = k[h // (H // G), rd:]
        q[h, rd:] += boost / (m["scale"] * (kk @ kk)) * torch.outer(kk, hq) / (hq @ hq)
    w["l0.mix.q"] = q.reshape(H * dk, -1).to(torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("size,keep,page_size", [(9, 3, 16), (16, 1, 16), (33, 5, 4), (150, 16, 16), (129, 17, 8)])
def test_window_and_kept_edges_with_standout_keys(size, keep, page_size, dtype):
    """a key that outweighs everything else sits exactly size - 1 positions back (the last one visible) for one query
    and exactly size back (the first one hidden) for another; a third is the last kept position and a fourth the
    first that is not kept, both asked for from far beyond the window; in a prompt and while decoding"""
    cfg = config([window(heads=4, kv_heads=2, dim=48, vdim=16, size=size, keep_first=keep, rot_dims=8, scale=0.25, ff=0)])
    w = O.random_model(cfg, seed=27)
    V = cfg["vocab"]
    n = keep + size + 2 * page_size + 70
    ids = [t % (V - 8) for t in tokens(n, V, 28)]
    base = keep + 2 * page_size
    at_in, at_out, kept_in, kept_out = [], [], [], []
    plan = ((base - 1, base - 1 + size - 1, at_in), (base + 8, base + 8 + size, at_out),
            (keep - 1, n - 20, kept_in), (keep, n - 10, kept_out))
    for i, (a, qpos, where) in enumerate(plan):
        key_tok, query_tok = V - 1 - 2 * i, V - 2 - 2 * i          # every pair has tokens of its own
        plant_pair(cfg, w, key_tok, query_tok)
        ids[a], ids[qpos] = key_tok, query_tok
        where.append(qpos)
    ref, _ = O.forward(cfg, w, ids)
    # the oracle itself says that these places see an off-by-one of the window or of the kept count
    for (dsize, dkeep), places in (((-1, 0), at_in), ((1, 0), at_out), ((0, -1), kept_in), ((0, 1), kept_out)):
        c2 = copy.deepcopy(cfg)
        c2["layers"][0]["mixer"]["mask"] = {"size": size + dsize, "keep_first": keep + dkeep}
        other, _ = O.forward(c2, w, ids)
        for p in places:
            assert rel_err(other[p:p + 1].float(), ref[p:p + 1])[1] > 1.0, (dsize, dkeep, p)
    marked = at_in + at_out + kept_in + kept_out
    first_q = min(marked)
    for cuts in ([n], [first_q - 1, 2, 1, 1, 37, 2, 1, 1], [first_q - 3] + [1] * (n - first_q + 3), [2] * (n // 2 + 1)):
        eng = make_engine(cfg, w, max_tokens=512, page_size=page_size, max_seq_len=1280, dtype=dtype)
        slot = eng.open_sequence()
        got = feed(eng, slot, ids, cuts)
        if dtype == torch.float32:
            assert rel_err(got, ref)[1] < 1e-3
        else:
            assert rel_err(got, ref)[0] < 6e-2
        for p in marked:
            assert rel_err(got[p:p + 1], ref[p:p + 1])[1] < (1e-3 if dtype == torch.float32 else 0.3), p
        close(eng)


def test_far_key_among_hundreds_in_causal_latent_attention():
    """latent attention sees everything before it: a standout key 600 positions back decides the answer"""
    cfg = config([latent(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=40, q_rank=32, scale=3.0, ff=0)])
    w = O.random_model(cfg, seed=29, scale=2.0)
    ids = tokens(700, 96, 30)
    ref, _ = O.forward(cfg, w, ids)
    for cuts in ([700], [650] + [1] * 50, [37] * 18):
        eng = make_engine(cfg, w, max_tokens=1024, max_seq_len=1024)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[1] < 1e-3
        close(eng)


def test_both_windowed_attention_kernels_agree():
    """bf16 cache rows: the tensor-core kernel (queries and weights as two bf16 terms) and the one-warp-per-pair kernel
    read the same cache, so they differ by fp32 roundings only; both stay within bf16's reach of the oracle.  Group sizes
    that do and do not divide the row tile, value sizes up to the kernel's limit, prompts, portions and single tokens"""
    for heads, kv_heads, dim, vdim, size, keep in ((4, 4, 32, 16, 100, 5), (6, 2, 16, 48, 37, 0), (8, 1, 64, 128, 130, 70),
                                                   (5, 1, 48, 32, 1000, 3)):
        cfg = config([window(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, size=size, keep_first=keep, rot_dims=16,
                             scale=0.3, ff=0)])
        w = O.random_model(cfg, seed=41)
        w["l0.mix.sink"] = torch.linspace(-2.0, 4.0, heads)
        ids = tokens(330, 96, 42)
        ref, _ = O.forward(cfg, w, ids)
        for cuts in ([330], [200, 64, 1, 1, 1, 2, 61], [300] + [1] * 30):
            got = []
            for fused in (1, 0):
                eng = make_engine(cfg, w, dtype=torch.bfloat16, max_tokens=512, max_seq_len=512, page_size=8)
                eng.set_option("fused_attn", fused)
                slot = eng.open_sequence()
                got.append(feed(eng, slot, ids, cuts))
                close(eng)
                assert rel_err(got[-1], ref)[0] < 5e-2, (heads, kv_heads, cuts, fused)
            assert rel_err(got[0], got[1].cpu())[0] < 2e-3, (heads, kv_heads, cuts)


def test_single_token_steps_with_key_shares_over_several_ctas():
    """a long window and one sequence: single-token steps cut the key tiles into shares for several CTAs and merge them,
    with the sink entering once, after the merge"""
    cfg = config([window(heads=4, kv_heads=2, dim=32, vdim=32, size=800, keep_first=5, rot_dims=16, scale=0.3, ff=0)])
    w = O.random_model(cfg, seed=43)
    w["l0.mix.sink"] = torch.tensor([4.0, -1.0, 0.0, 2.0])
    ids = tokens(900, 96, 44)
    ref, _ = O.forward(cfg, w, ids)
    got = []
    for fused in (1, 0):
        eng = make_engine(cfg, w, dtype=torch.bfloat16, max_tokens=1024, max_seq_len=1024)
        eng.set_option("fused_attn", fused)
        slot = eng.open_sequence()
        got.append(feed(eng, slot, ids, [870] + [1] * 30)[870:])
        close(eng)
        assert rel_err(got[-1], ref[870:])[0] < 5e-2
    assert rel_err(got[0], got[1].cpu())[0] < 2e-3


def random_config(seed):
    """layers in any order and number with sizes drawn at random (multiples of 16 and of nothing), a span anywhere"""
    g = torch.Generator().manual_seed(seed)
    pick = lambda xs: xs[int(torch.randint(0, len(xs), (1,), generator=g))]
    n = pick([2, 3, 4, 5])
    layers = []
    for _ in range(n):
        kind = pick(["latent", "gla", "window"])
        ff = pick([0, 24, 64, 100])
        if kind == "latent":
            rot_dim = pick([4, 8, 16, 32])
            layers.append(latent(heads=pick([1, 2, 4, 5]), dim=pick([8, 16, 24, 64]), rot_dim=rot_dim, vdim=pick([8, 16, 20, 48]),
                                 kv_rank=pick([16, 24, 40, 64]), q_rank=pick([8, 20, 64, 72]), base=pick([100.0, 1e4, 3e5]),
                                 scale=pick([0.1, 0.25]), ff=ff, rot_dims=pick([rot_dim, rot_dim // 2 * 2 - 2 if rot_dim > 4 else rot_dim]),
                                 layout=pick([None, None, "halves"])))
        elif kind == "gla":
            layers.append(gla(heads=pick([1, 2, 4, 6]), dim=pick([8, 16, 48, 72, 128]), vdim=pick([8, 16, 32, 40, 64]),
                              tau=pick([1.0, 4.0, 12.0, 64.0]), ff=ff, decay_rank=pick([1, 4, 12])))
        else:
            kv = pick([1, 2, 4])
            dim = pick([8, 16, 32, 48, 128])
            layers.append(window(heads=kv * pick([1, 2, 4, 8]), kv_heads=kv, dim=dim, vdim=pick([8, 16, 32, 64, 128, 20]),
                                 size=pick([1, 5, 16, 33, 64, 300]), keep_first=pick([0, 1, 5, 20]), base=pick([100.0, 3e4]),
                                 rot_dims=pick([dim, dim // 2, 4]), scale=pick([0.09, 0.2]), ff=ff,
                                 layout=pick([None, None, "halves"]), mask=pick([True, True, True, False])))
    loop = None
    if pick([True, True, False]):
        a = pick(list(range(n)))
        loop = (a, pick(list(range(a + 1, n + 1))), pick([1, 2, 3]))
    return config(layers, width=pick([48, 64, 80, 128]), vocab=pick([50, 96, 257]), eps=pick([1e-5, 1e-6]),
                  scale=pick([1.0, 8.0, 11.0]), cap=pick([0.0, 14.0, 30.0]), loop=loop)


@pytest.mark.parametrize("seed", list(range(12)))
def test_configurations_drawn_at_random(seed):
    """what a checkpoint's config.json may say, drawn at random: whole prompt, prompt then single tokens, portions"""
    cfg = random_config(100 + seed)
    w = O.random_model(cfg, seed=200 + seed)
    ids = tokens(75, cfg["vocab"], 300 + seed)
    ref, _ = O.forward(cfg, w, ids)
    for dtype in (torch.float32, torch.bfloat16):
        for cuts in ([75], [50] + [1] * 25, [37, 2, 3, 1, 1, 14, 2]):
            eng = make_engine(cfg, w, dtype=dtype, max_tokens=128, page_size=8)
            slot = eng.open_sequence()
            got = feed(eng, slot, ids, cuts)
            if dtype == torch.float32:
                assert rel_err(got, ref)[1] < 3e-4, (cfg, cuts)
            else:
                assert rel_err(got, ref)[0] < 8e-2, (cfg, cuts)
            close(eng)


# ------------------------------------------------------------------------------------------------ bf16 engine
@pytest.mark.parametrize("tc", [1, 0], ids=["tcgen05", "cuda-cores"])
@pytest.mark.parametrize("cfg_dict", [SMALL, ODD], ids=["small", "odd"])
def test_bf16_engine_both_linear_paths(cfg_dict, tc):
    w = O.random_model(cfg_dict, seed=31)
    ids = tokens(90, cfg_dict["vocab"], 32)
    ref, _ = O.forward(cfg_dict, w, ids)
    for cuts in ([90], [50] + [1] * 40, [7] * 13):
        eng = make_engine(cfg_dict, w, dtype=torch.bfloat16, max_tokens=128, tc=tc)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[0] < 5e-2
        close(eng)


def test_bf16_engine_on_sizes_that_fill_tensor_core_tiles():
    """multiples of 64: every projection and the latent products take the tcgen05 kernels; 300 tokens take the
    tensor-bound CTA-pair GEMM"""
    cfg = config([latent(heads=4, dim=64, rot_dim=32, vdim=64, kv_rank=128, q_rank=64, ff=256),
                  gla(heads=2, dim=64, vdim=64, tau=16.0, ff=128, decay_rank=16),
                  window(heads=4, kv_heads=2, dim=64, vdim=64, size=37, keep_first=4, rot_dims=64, scale=0.125, ff=128)],
                 width=256, vocab=512, loop=(1, 3, 2))
    w = O.random_model(cfg, seed=33)
    ids = tokens(300, 512, 34)
    ref, _ = O.forward(cfg, w, ids)
    for cuts in ([300], [280] + [1] * 20):
        eng = make_engine(cfg, w, dtype=torch.bfloat16, max_tokens=512)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[0] < 5e-2
        close(eng)


# ------------------------------------------------------------------------------------------------ entry points
def test_greedy_generation_through_stage_and_scheduler():
    """Stage.generate (byte tokenizer, ragged prefill, the step loop and the fused sampler at temperature 0) against
    greedy decoding with the oracle"""
    from asd_b200.models.rivetar import RivetarConfig
    from asd_b200.models.stage import Stage
    cfg_dict = copy.deepcopy(SMALL)
    cfg_dict["vocab"] = 256
    w = O.random_model(cfg_dict, seed=35)
    w["head"] = (w["head"].float() * 4).to(torch.bfloat16)          # spread logits: no near ties between arg-maxima
    cfg = RivetarConfig.from_dict(cfg_dict).with_shapes({k: tuple(v.shape) for k, v in w.items()})
    st = Stage("unused", "rivetar-test", config=cfg, weights=w, max_batch=3, max_model_len=128, k=0)
    assert st.get_model_info()["family"] == "rivetar"
    prompts = ["abc", "hello world, this is longer", "z"]
    texts, _, stats = st.generate(prompts, max_tokens=12, temperature=0.0)
    assert stats["decode_steps"] >= 11
    ids = [list(p.encode()) for p in prompts]
    toks = st._generate_ids(ids, 12, 0.0)[0]
    for p, t, new in zip(ids, texts, toks):
        assert st.tokenizer.decode(new) == t and len(new) == 12
        # teacher-forced on the engine's own tokens: each one is the oracle's arg-max, or within bf16 noise of it
        lg, _ = O.forward(cfg_dict, w, p + new)
        for j, tok in enumerate(new):
            row = lg[len(p) + j - 1]
            assert row[tok] >= row.max() - 0.02 * row.std(), (j, tok, int(row.argmax()))
        assert sum(int(lg[len(p) + j - 1].argmax()) == tok for j, tok in enumerate(new)) >= 10


def test_speculative_decoding_with_a_rivetar_draft_equals_plain_greedy():
    """draft and target both carry recurrent state; a rejected tail is re-fed from the state ring"""
    from asd_b200.engine import RivetarEngine, SpecDecoder
    from asd_b200.models.rivetar import RivetarConfig
    tcfg = copy.deepcopy(SMALL)
    dcfg = config([gla(heads=1, dim=16, vdim=8, tau=4.0), window(heads=2, kv_heads=1, dim=8, vdim=8, size=6, keep_first=1, ff=0)])
    wt, wd = O.random_model(tcfg, seed=37), O.random_model(dcfg, seed=38)
    wt["head"] = (wt["head"].float() * 4).to(torch.bfloat16)
    prompts = [tokens(9, 96, 39), tokens(15, 96, 40)]

    def run(with_draft):
        kw = dict(max_seqs=2, max_seq_len=96, max_tokens=64, dtype=torch.float32, ring=6)     # fp32: no near ties
        mk = lambda c, w: RivetarEngine(RivetarConfig.from_dict(c).with_shapes({k: tuple(v.shape) for k, v in w.items()}),
                                        **kw).load_weights(w)
        t = mk(tcfg, wt)
        d = mk(dcfg, wd) if with_draft else None
        return SpecDecoder(t, d, 2, 3, temperature=0.0).generate(prompts, 16)[0].tolist()

    plain = run(False)
    assert run(True) == plain
    lg, _ = O.forward(tcfg, wt, prompts[0] + plain[0])
    assert sum(int(lg[len(prompts[0]) + j - 1].argmax()) == t for j, t in enumerate(plain[0])) >= 14


def write_checkpoint(path, cfg_dict, w):
    """config.json + model.safetensors (8-byte little-endian header length, JSON header, raw data)"""
    path.mkdir()
    cfg_dict = copy.deepcopy(cfg_dict)
    for e in cfg_dict["layers"]:
        e["mixer"].pop("decay_rank", None)          # a checkpoint's tensor shapes give this size, not its config.json
    (path / "config.json").write_text(json.dumps(cfg_dict))
    header, blobs, off = {}, [], 0
    for name, t in w.items():
        raw = t.to(torch.bfloat16).contiguous().view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    with open(path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_command_on_a_checkpoint_directory(tmp_path, dtype):
    """the command-line runner end to end: registry by config.json, safetensors loader (sizes that only tensor shapes
    give), page table with two requests one after the other (the second reuses the first one's slot, pages and state),
    portions down to one token, wanted rows only"""
    import numpy as np
    w = {k: v.to(torch.bfloat16) for k, v in O.random_model(ODD, seed=51).items()}
    write_checkpoint(tmp_path / "model", ODD, w)
    a, b = tokens(41, ODD["vocab"], 52), tokens(23, ODD["vocab"], 53)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[32:33], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[33:], "want": [7, 3]}], "end": ["a"]},
             {"step": 4, "entries": [{"id": "b", "tokens": b, "want": [22]}], "end": ["b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path / "model"), "--dtype",
                        dtype, "--out", str(out), "--max-tokens", "48"], input="\n".join(json.dumps(x) for x in steps) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(5)]
    ra, rb = O.forward(ODD, w, a)[0], O.forward(ODD, w, b)[0]
    want = {0: ra[[0, 29]], 2: ra[[32]], 3: ra[[40, 36]], 4: rb[[22]]}
    assert not (out / "1.f32").exists()
    for step, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(ref.shape[0], -1).copy())
        # fp32: largest deviation against the logits' spread; bf16 (nine layer executions deep): relative norm
        if dtype == "float32":
            assert rel_err(got, ref)[1] < 2e-4, step
        else:
            assert rel_err(got, ref)[0] < 5e-2, step
