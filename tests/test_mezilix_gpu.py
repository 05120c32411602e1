"""GPU: the Mezilix engine against the plain restatement in oracle/mezilix_oracle.py (fp64, whole sequences, keys and
values written out per head).  Every test makes its own small configuration and random weights.  The fp32 engine is
held to 2e-4 of the logits' spread, which a single key missed or double-counted among hundreds, a window off by
one, a lost state or a stale page all exceed; the bf16 engine to what its roundings allow."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import mezilix_oracle as O  # noqa: E402


def layer(heads=2, dim=16, rot_dim=8, vdim=24, kv_rank=32, window=12, base=1000.0, scale=0.2, experts=4, top=2, ff=40,
          rot_dims=None):
    e = {"type": "latent_attention",
         "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                   "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
                   "scale": scale},
         "mlp": None}
    if experts:
        e["mlp"] = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    return e


def config(layers, width=64, vocab=96, buckets=53, mul_prev=31, mul_cur=7, eps=1e-5):
    return {"architecture": "Mezilix", "width": width, "vocab": vocab, "norm": {"eps": eps},
            "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "layers": layers}


SMALL = config([layer(), layer(heads=3, dim=8, rot_dim=16, vdim=8, kv_rank=40, window=7, base=500.0, scale=0.25,
                              experts=0)])
# sizes that are multiples of nothing, one expert chosen / all experts chosen, a window longer than any sequence
ODD = config([layer(heads=3, dim=12, rot_dim=6, vdim=20, kv_rank=36, window=5, experts=5, top=5, ff=50),
              layer(heads=1, dim=10, rot_dim=4, vdim=7, kv_rank=33, window=1000, experts=3, top=1, ff=9),
              layer(heads=5, dim=6, rot_dim=10, vdim=6, kv_rank=70, window=1, experts=0, rot_dims=6)],
             width=72, vocab=101, buckets=17, mul_prev=5, mul_cur=3, eps=1e-3)


def make_engine(cfg_dict, w, dtype=torch.float32, max_tokens=64, max_seq_len=512, page_size=16, num_pages=None,
                max_seqs=4, ring=8, tc=1):
    from asd_b200.engine import MezilixEngine
    from asd_b200.models.mezilix import MezilixConfig
    cfg = MezilixConfig.from_dict(cfg_dict)
    eng = MezilixEngine(cfg, max_seqs=max_seqs, max_seq_len=max_seq_len, max_tokens=max_tokens, page_size=page_size,
                        dtype=dtype, dynamic_pages=True, num_pages=num_pages, ring=ring)
    eng.load_weights(w)
    eng.set_option("tc_linear", tc)
    return eng


def close(eng):
    """no kernel of the engine gave up a wait"""
    from asd_b200._lib import check, lib
    check(lib().asd_mezilix_device_error(eng.h), "device error")
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


@pytest.mark.parametrize("cfg_dict", [SMALL, ODD], ids=["small", "odd"])
def test_whole_prompt_logits_and_every_layer(cfg_dict):
    w = O.random_model(cfg_dict, seed=1)
    ids = tokens(45, cfg_dict["vocab"], 2)
    ref, streams = O.forward(cfg_dict, w, ids)
    eng = make_engine(cfg_dict, w)
    slot = eng.open_sequence()
    eng.reserve(slot, len(ids))
    got, st = eng.forward_ragged([(slot, 0, ids, list(range(len(ids))))], layer_out=True)
    st = torch.cat(st, 1).cpu().double()
    for i in range(len(cfg_dict["layers"])):           # the first layer that differs names the mechanism
        assert (st[i] - streams[i]).abs().max() <= 2e-4 * streams[i].abs().max(), f"stream leaving layer {i}"
    assert rel_err(got, ref)[1] < 2e-4
    eng.close()


def test_embedding_pair_table_alone():
    """no layers: logits = head . norm(embed + pair row); the previous token crosses portion borders"""
    cfg = config([], width=40, vocab=50, buckets=7, mul_prev=3, mul_cur=11)
    w = O.random_model(cfg, seed=3)
    ids = tokens(20, 50, 4)
    ref, _ = O.forward(cfg, w, ids)
    eng = make_engine(cfg, w)
    slot = eng.open_sequence()
    assert rel_err(feed(eng, slot, ids, [1, 1, 2, 5, 1]), ref)[1] < 1e-4
    eng.close()


def test_token_shift_alone_takes_previous_unshifted_input():
    """shift weights of exactly 1 hand the mixer the previous position's normed input and nothing of its own:
    a state that is lost, or stored after the shift, changes every logit"""
    cfg = config([layer(experts=0), layer(experts=0)])
    w = O.random_model(cfg, seed=5)
    for i in range(2):
        w[f"l{i}.shift"] = torch.ones_like(w[f"l{i}.shift"])
    ids = tokens(30, 96, 6)
    ref, _ = O.forward(cfg, w, ids)
    eng = make_engine(cfg, w)
    slot = eng.open_sequence()
    assert rel_err(feed(eng, slot, ids, [3, 1, 1, 2, 9, 1]), ref)[1] < 2e-4
    eng.close()


def test_router_takes_largest_scores_unnormalised():
    """one layer whose attention is silenced (zero output projection): what remains is the expert mixture"""
    cfg = config([layer(experts=6, top=2, ff=24)])
    w = O.random_model(cfg, seed=7)
    w["l0.mix.o"] = torch.zeros_like(w["l0.mix.o"])
    ids = tokens(33, 96, 8)
    ref, _ = O.forward(cfg, w, ids)
    eng = make_engine(cfg, w)
    slot = eng.open_sequence()
    assert rel_err(feed(eng, slot, ids, []), ref)[1] < 2e-4
    eng.close()


def test_depth_average_uses_every_earlier_result():
    cfg = config([layer(experts=0, window=4), layer(experts=0, window=4), layer(experts=0, window=4)])
    w = O.random_model(cfg, seed=9)
    w["l2.dwa"] = torch.tensor([0.9, -0.4, 0.3, 0.5]).to(torch.bfloat16)     # far from a plain residual stream
    ids = tokens(17, 96, 10)
    ref, _ = O.forward(cfg, w, ids)
    eng = make_engine(cfg, w)
    slot = eng.open_sequence()
    assert rel_err(feed(eng, slot, ids, []), ref)[1] < 2e-4
    eng.close()


@pytest.mark.parametrize("cfg_dict", [SMALL, ODD], ids=["small", "odd"])
@pytest.mark.parametrize("page_size", [4, 16])
def test_prefill_then_decode_and_portions(cfg_dict, page_size):
    """whole prompt == any cut into portions (down to two tokens and single tokens) == token by token, across page
    borders, window edges and the first tokens"""
    w = O.random_model(cfg_dict, seed=11)
    ids = tokens(70, cfg_dict["vocab"], 12)
    ref, _ = O.forward(cfg_dict, w, ids)
    for cuts in ([70], [1] * 70, [2] * 35, [5, 2, 9, 2, 16, 3, 1, 1, 17, 2], [37, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1]):
        eng = make_engine(cfg_dict, w, page_size=page_size)
        slot = eng.open_sequence()
        got = feed(eng, slot, ids, cuts)
        assert rel_err(got, ref)[1] < 2e-4, cuts[:4]
        eng.close()


def test_forward_smaller_than_a_portion_is_cut_inside_the_engine():
    """a portion longer than max_tokens runs as several forwards"""
    w = O.random_model(SMALL, seed=13)
    ids = tokens(50, 96, 14)
    ref, _ = O.forward(SMALL, w, ids)
    eng = make_engine(SMALL, w, max_tokens=16)
    slot = eng.open_sequence()
    assert rel_err(feed(eng, slot, ids, []), ref)[1] < 2e-4
    eng.close()


def test_batch_of_unequal_requests_equals_each_alone():
    w = O.random_model(SMALL, seed=15)
    seqs = [tokens(n, 96, 20 + n) for n in (31, 5, 1, 18)]
    refs = [O.forward(SMALL, w, s)[0] for s in seqs]
    eng = make_engine(SMALL, w, max_tokens=32)
    slots = [eng.open_sequence() for _ in seqs]
    # step 1: unequal first portions in ONE batch; step 2: the rest, also unequal, one request already finished
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
    eng.close()


def test_pages_and_slots_freed_and_used_again():
    """a pool with room for one request at a time: the second request gets the first one's slot, pages and rings
    with the old contents still in them"""
    w = O.random_model(SMALL, seed=17)
    eng = make_engine(SMALL, w, page_size=4, num_pages=12, max_seqs=1, max_seq_len=48)
    for seed, n in ((30, 44), (31, 47), (32, 9), (33, 48)):
        ids = tokens(n, 96, seed)
        ref, _ = O.forward(SMALL, w, ids)
        slot = eng.open_sequence()
        assert slot == 0
        got = feed(eng, slot, ids, [7, 1, 1, 13, 2])
        assert rel_err(got, ref)[1] < 2e-4
        eng.close_sequence(slot)
        assert eng.pages.pages_in_use() == 0
    from asd_b200._lib import AsdError
    slot = eng.open_sequence()
    with pytest.raises(AsdError):
        eng.reserve(slot, 49)
    eng.close()


def standout_model(window, n_layers=1):
    """sharp softmax (large scale) and weights that spread the scores: single keys carry most of the weight"""
    cfg = config([layer(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=40, window=window, scale=3.0, experts=0)
                  for _ in range(n_layers)])
    return cfg, O.random_model(cfg, seed=19, scale=2.0)


def plant_pair(cfg, w, key_tok, query_tok, boost=600.0):
    """Makes the first layer's queries of ``query_tok`` point at the unrotated keys of ``key_tok`` in every head, so
    that this one score exceeds all others by about ``boost`` wherever the key is visible.  The pair table and the
    first layer's shift are silenced, so that what the first layer reads depends on the token alone."""
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    H, dn, dr, R = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    w["bigram"] = torch.zeros_like(w["bigram"])
    w["l0.shift"] = torch.zeros_like(w["l0.shift"])
    f = lambda t: t.double()
    hk = O.scalar_rms_norm(f(w["embed"][key_tok]), f(w["l0.norm1"]), eps)
    hq = O.scalar_rms_norm(f(w["embed"][query_tok]), f(w["l0.norm1"]), eps)
    c = O.unit_rms(f(w["l0.mix.dkv"])[:R] @ hk, eps) * f(w["l0.mix.dkv.norm"])
    k = (f(w["l0.mix.uk"]) @ c).reshape(H, dn)
    q = f(w["l0.mix.q"]).reshape(H, dn + dr, -1).clone()
    for h in range(H):
        q[h, :dn] += boost / (m["scale"] * (k[h] @ k[h])) * torch.outer(k[h], hq) / (hq @ hq)
    w["l0.mix.q"] = q.reshape(H * (dn + dr), -1).to(torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("window,page_size", [(9, 16), (16, 16), (33, 4), (300, 16), (257, 8), (1000, 16)])
def test_window_edges_with_standout_keys(window, page_size, dtype):
    """a key that outweighs everything else sits exactly window - 1 positions back (the last one visible) for one
    query and exactly window positions back (the first one hidden) for another, in a prompt and while decoding, far
    away among hundreds of keys and on the first and last row of a page"""
    cfg, w = standout_model(window)
    V = cfg["vocab"]
    n = window + 2 * page_size + 56
    ids = [t % (V - 8) for t in tokens(n, V, 21)]
    at_in, at_out = [], []
    # (place of the key, distance to its query): last and first row of a page, and two places inside one
    for i, (a, gap, where) in enumerate(((2 * page_size - 1, window - 1, at_in), (2 * page_size, window, at_out),
                                         (2 * page_size + 40, window - 1, at_in), (2 * page_size + 51, window, at_out))):
        key_tok, query_tok = V - 1 - 2 * i, V - 2 - 2 * i          # every pair has tokens of its own
        plant_pair(cfg, w, key_tok, query_tok)
        ids[a], ids[a + gap] = key_tok, query_tok
        where.append(a + gap)
    ref, _ = O.forward(cfg, w, ids)
    # the oracle itself says that these places see an off-by-one: a shorter window loses the key of the first kind,
    # a longer one gains the key of the second kind
    for wrong, places in ((window - 1, at_in), (window + 1, at_out)):
        c2 = copy.deepcopy(cfg)
        c2["layers"][0]["mixer"]["mask"]["size"] = wrong
        other, _ = O.forward(c2, w, ids)
        for p in places:
            assert rel_err(other[p:p + 1].float(), ref[p:p + 1])[1] > 1.0
    first_q = min(at_in + at_out)
    for cuts in ([n], [first_q - 1, 2, 1, 1, 37, 2, 1, 1], [first_q - 3] + [1] * (n - first_q + 3), [2] * (n // 2)):
        eng = make_engine(cfg, w, max_tokens=512, page_size=page_size, max_seq_len=1280, dtype=dtype)
        slot = eng.open_sequence()
        got = feed(eng, slot, ids, cuts)
        # planted scores are about 600, where one fp32 ulp is 6e-5: the weights carry that rounding, an off-by-one 1.0.
        # The bf16 engine (tensor-core attention: a latent row of 48 elements) is held to its own roundings.
        tol = 1e-3 if dtype == torch.float32 else 0.3
        if dtype == torch.float32:
            assert rel_err(got, ref)[1] < tol
        else:
            assert rel_err(got, ref)[0] < 6e-2
        for p in at_in + at_out:
            assert rel_err(got[p:p + 1], ref[p:p + 1])[1] < tol
        close(eng)


def test_both_attention_kernels_agree_with_the_oracle():
    """the register-tiled kernel (with and without shares of the key range) and the one-warp-per-pair kernel on the
    same long sequence: many heads, few heads, a latent size that fills no tile"""
    for heads, kv_rank, rot_dim in ((6, 72, 12), (1, 32, 8), (20, 264, 4)):
        cfg = config([layer(heads=heads, dim=8, rot_dim=rot_dim, vdim=8, kv_rank=kv_rank, window=700, scale=0.7, experts=0)])
        w = O.random_model(cfg, seed=43, scale=2.0)
        ids = tokens(900, 96, 44)
        ref, _ = O.forward(cfg, w, ids)
        for tiled in (1, 0):
            eng = make_engine(cfg, w, max_tokens=1024, max_seq_len=1024)
            eng.set_option("attn_tiled", tiled)
            slot = eng.open_sequence()
            got = feed(eng, slot, ids, [3, 830, 1, 1, 1, 2, 40, 1, 1])
            assert rel_err(got, ref)[1] < 3e-4, (heads, tiled)
            close(eng)


def test_tensor_core_attention_keeps_fp32_scores():
    """bf16 engine: attention on the tensor cores (the query as three bf16 terms, the weights as two) against the fp32
    CUDA-core kernels on the same cache; a sharp softmax (large scale) would expose scores kept to bf16 only"""
    cfg = config([layer(heads=5, dim=16, rot_dim=16, vdim=16, kv_rank=48, window=500, scale=2.0, experts=0)], width=64)
    w = O.random_model(cfg, seed=45, scale=2.0)
    ids = tokens(700, 96, 46)
    outs = []
    for mode in (2, 1, 0):
        eng = make_engine(cfg, w, dtype=torch.bfloat16, max_tokens=1024, max_seq_len=1024)
        eng.set_option("attn_tiled", mode)
        outs.append(feed(eng, eng.open_sequence(), ids, [3, 600, 1, 1, 1, 2, 40, 1, 1]).cpu())
        close(eng)
    # both fp32 kernels form the same sums; the tensor-core kernel may round elsewhere, and in a bf16 engine every later
    # bf16 rounding amplifies that, so it is held to the oracle: no further from it than the fp32 kernels are
    assert rel_err(outs[1], outs[2].double())[1] < 2e-4
    ref, _ = O.forward(cfg, w, ids)
    e_tc, e_fp32 = rel_err(outs[0], ref)[0], rel_err(outs[1], ref)[0]
    assert e_fp32 < 4e-2 and e_tc < 1.1 * e_fp32 + 1e-4, (e_tc, e_fp32)


def test_long_decoding_past_window_ring_and_pages():
    cfg, w = standout_model(20, n_layers=2)
    ids = tokens(260, 96, 23)
    ref, _ = O.forward(cfg, w, ids)
    eng = make_engine(cfg, w, page_size=8, ring=3)
    slot = eng.open_sequence()
    assert rel_err(feed(eng, slot, ids, [4] + [1] * 256), ref)[1] < 3e-4
    eng.close()


def test_refeeding_recent_positions_finds_their_state():
    """speculative verification re-feeds positions after a rejected tail: the rings keep the state of the last
    `ring` positions, so overwriting positions p-2 .. p with other tokens and going on equals a fresh run"""
    w = O.random_model(SMALL, seed=25)
    ids = tokens(40, 96, 26)
    wrong = [(t + 1) % 96 for t in ids]
    ref, _ = O.forward(SMALL, w, ids)
    eng = make_engine(SMALL, w, ring=8)
    slot = eng.open_sequence()
    eng.reserve(slot, 40)
    eng.forward_ragged([(slot, 0, ids[:20], [])])
    eng.forward_ragged([(slot, 20, ids[20:21] + wrong[21:25], [])])  # a rejected tail: 21 .. 24 were wrong
    got = eng.forward_ragged([(slot, 21, ids[21:], list(range(19)))])
    assert rel_err(got, ref[21:])[1] < 2e-4
    eng.close()


@pytest.mark.parametrize("tc", [1, 0], ids=["tcgen05", "cuda-cores"])
def test_bf16_engine_both_linear_paths(tc):
    """sizes the tensor-core GEMM accepts (multiples of 8, rows of 16 bytes): both paths against the oracle"""
    cfg = config([layer(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=64, window=24, experts=4, top=2, ff=64),
                  layer(heads=2, dim=64, rot_dim=32, vdim=16, kv_rank=96, window=50, experts=0)], width=128, vocab=200)
    w = O.random_model(cfg, seed=27)
    ids = tokens(90, 200, 28)
    ref, _ = O.forward(cfg, w, ids)
    eng = make_engine(cfg, w, dtype=torch.bfloat16, tc=tc, max_tokens=128)
    slot = eng.open_sequence()
    whole = feed(eng, slot, ids, [])
    assert rel_err(whole, ref)[0] < 3e-2
    eng.close_sequence(slot)
    slot = eng.open_sequence()
    cut = feed(eng, slot, ids, [50, 2, 7] + [1] * 31)
    assert rel_err(cut, ref)[0] < 3e-2
    assert rel_err(cut, whole.cpu())[0] < 2e-2        # cutting changes roundings only
    close(eng)


# multiples of 8 that fill no tile of 64 (tensor-core paths with ragged edges); a latent row of 44 elements (multiple of
# 4, not of 8: register-tiled attention without 16-byte cache loads); multipliers beyond 32 bits
EIGHTS = config([layer(heads=3, dim=24, rot_dim=8, vdim=40, kv_rank=88, window=21, experts=3, top=2, ff=56),
                 layer(heads=2, dim=16, rot_dim=8, vdim=8, kv_rank=36, window=400, experts=0)],
                width=72, vocab=104, buckets=31, mul_prev=(1 << 40) + 7, mul_cur=(1 << 33) + 5)


@pytest.mark.parametrize("cfg_dict", [ODD, EIGHTS], ids=["odd", "eights"])
def test_bf16_engine_on_sizes_that_fill_no_tile(cfg_dict):
    w = O.random_model(cfg_dict, seed=37)
    ids = tokens(120, cfg_dict["vocab"], 38)
    ref, _ = O.forward(cfg_dict, w, ids)
    eng32 = make_engine(cfg_dict, w, max_tokens=128)
    exact = feed(eng32, eng32.open_sequence(), ids, [])
    assert rel_err(exact, ref)[1] < 2e-4
    close(eng32)
    for cuts in ([], [70, 2, 9] + [1] * 39):
        eng = make_engine(cfg_dict, w, dtype=torch.bfloat16, max_tokens=128)
        got = feed(eng, eng.open_sequence(), ids, cuts)
        assert rel_err(got, ref)[0] < 4e-2, cuts[:3]
        close(eng)


def test_linear_on_cuda_cores_matches_fp32_matmul():
    from asd_b200._lib import check, lib
    g = torch.Generator().manual_seed(29)
    for M, N, K in ((1, 7, 5), (70, 130, 33), (65, 64, 257)):
        x, wt = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
        xd, wd = x.cuda(), wt.cuda()
        y = torch.empty(M, N, device="cuda")
        check(lib().asd_linear_simt(xd.data_ptr(), 1, wd.data_ptr(), 1, y.data_ptr(), 1, M, N, K, None))
        torch.cuda.synchronize()
        ref = x.double() @ wt.double().T
        assert (y.cpu().double() - ref).abs().max() < 1e-4
        xb, wb = xd.bfloat16(), wd.bfloat16()
        check(lib().asd_linear_simt(xb.data_ptr(), 0, wb.data_ptr(), 0, y.data_ptr(), 1, M, N, K, None))
        torch.cuda.synchronize()
        ref = xb.cpu().double() @ wb.cpu().double().T
        assert (y.cpu().double() - ref).abs().max() < 1e-4


def test_linear_on_tensor_cores_matches_fp32_matmul():
    """plain, batched per head, and grouped with gathered rows (the expert layers), with the squared-ReLU epilogue;
    k loops long enough to reuse every shared-memory stage several times; rows and columns that fill no tile"""
    from asd_b200._lib import check, lib
    g = torch.Generator().manual_seed(41)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    for M, N, K, Z, x32, y32, relu in ((1, 8, 64, 1, 0, 1, 0), (70, 130, 72, 1, 1, 1, 0), (150, 257, 1024, 1, 0, 0, 1),
                                       (19, 40, 136, 3, 1, 1, 0), (128, 128, 512, 2, 0, 1, 1)):
        x, wt = torch.randn(Z, M, K, generator=g), torch.randn(Z, N, K, generator=g) / K ** 0.5
        xd = x.cuda() if x32 else x.cuda().bfloat16()
        wd = wt.cuda().bfloat16()
        y = torch.full((Z, M, N), float("nan"), device="cuda", dtype=torch.float32 if y32 else torch.bfloat16)
        check(lib().asd_linear_tc(xd.data_ptr(), x32, wd.data_ptr(), y.data_ptr(), y32, M, N, K, Z, None, None, relu,
                                  err.data_ptr(), None))
        torch.cuda.synchronize()
        ref = x.bfloat16().double() @ wd.cpu().double().transpose(1, 2)
        ref = ref.clamp(min=0) ** 2 if relu else ref
        tol = 1e-4 if y32 else 2e-2
        assert (y.cpu().double() - ref).abs().max() < tol * max(1.0, ref.abs().max().item()), (M, N, K, Z)
    # grouped: 5 weights, groups of unequal size (one empty, one larger than a row tile), rows gathered from x
    E, T, N, K = 5, 300, 72, 200
    sizes = [0, 7, 140, 1, 33]
    x, wt = torch.randn(T, K, generator=g), (torch.randn(E, N, K, generator=g) / K ** 0.5).bfloat16()
    gather = torch.randint(0, T, (sum(sizes),), generator=g).to(torch.int32)
    off = torch.tensor([0] + torch.tensor(sizes).cumsum(0).tolist(), dtype=torch.int32)
    y = torch.full((sum(sizes), N), float("nan"), device="cuda")
    xd, wd, off_d, gather_d = x.cuda().bfloat16(), wt.cuda(), off.cuda(), gather.cuda()     # alive until the sync
    check(lib().asd_linear_tc(xd.data_ptr(), 0, wd.data_ptr(), y.data_ptr(), 1, T, N, K, E, off_d.data_ptr(),
                              gather_d.data_ptr(), 1, err.data_ptr(), None))
    torch.cuda.synchronize()
    for e in range(E):
        rows = gather[off[e]:off[e + 1]].long()
        if len(rows) == 0:
            continue
        ref = (x.bfloat16().double()[rows] @ wt[e].double().T).clamp(min=0) ** 2
        assert (y[off[e]:off[e + 1]].cpu().double() - ref).abs().max() < 1e-4 * max(1.0, ref.abs().max().item())
    assert not torch.isnan(y).any()
    assert int(err.item()) == 0


def test_greedy_generation_through_stage_and_scheduler():
    """Stage.generate (byte tokenizer, ragged prefill, the step loop and the fused sampler at temperature 0) against
    greedy decoding with the oracle"""
    from asd_b200.models.mezilix import MezilixConfig
    from asd_b200.models.stage import Stage
    cfg_dict = config([layer(), layer(heads=3, dim=8, rot_dim=16, vdim=8, kv_rank=40, window=7, experts=0)], vocab=256)
    w = O.random_model(cfg_dict, seed=31)
    w["head"] = (w["head"].float() * 4).to(torch.bfloat16)          # spread logits: no near ties between arg-maxima
    st = Stage("unused", "mezilix-test", config=MezilixConfig.from_dict(cfg_dict), weights=w, max_batch=3,
               max_model_len=128, k=0)
    assert st.get_model_info()["family"] == "mezilix"
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


def test_speculative_decoding_with_a_mezilix_draft_equals_plain_greedy():
    from asd_b200.engine import MezilixEngine, SpecDecoder
    from asd_b200.models.mezilix import MezilixConfig
    tcfg = config([layer(), layer(heads=3, dim=8, rot_dim=16, vdim=8, kv_rank=40, window=7, experts=0)])
    dcfg = config([layer(heads=1, dim=8, rot_dim=8, vdim=8, kv_rank=16, window=6, experts=0)])
    wt, wd = O.random_model(tcfg, seed=33), O.random_model(dcfg, seed=34)
    wt["head"] = (wt["head"].float() * 4).to(torch.bfloat16)
    prompts = [tokens(9, 96, 35), tokens(15, 96, 36)]

    def run(with_draft):
        kw = dict(max_seqs=2, max_seq_len=96, max_tokens=64, dtype=torch.float32)     # fp32: no near ties
        t = MezilixEngine(MezilixConfig.from_dict(tcfg), **kw).load_weights(wt)
        d = MezilixEngine(MezilixConfig.from_dict(dcfg), **kw).load_weights(wd) if with_draft else None
        toks = SpecDecoder(t, d, 2, 3, temperature=0.0).generate(prompts, 16)[0]
        return toks.tolist()

    assert run(True) == run(False)


def write_checkpoint(path, cfg_dict, w):
    """config.json + model.safetensors (8-byte little-endian header length, JSON header, raw data)"""
    import json
    import struct
    path.mkdir()
    (path / "config.json").write_text(json.dumps(cfg_dict))
    header, blobs, off = {}, [], 0
    for name, t in w.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    with open(path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_command_on_a_checkpoint_directory(tmp_path, dtype):
    """the command-line runner end to end: registry by config.json, safetensors loader, page table with two requests one
    after the other (the second reuses the first one's slot and pages), portions down to one token, wanted rows only"""
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    w = O.random_model(ODD, seed=51)
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
    tol = 2e-4 if dtype == "float32" else 5e-2
    for step, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(ref.shape[0], -1).copy())
        assert rel_err(got, ref)[1] < tol, step
