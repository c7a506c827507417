"""Lufatar through the engine against the plain implementation (tests/plain_lufatar.py): each mechanism alone,
prompts whole and token by token, portions down to two tokens, mixed batches, pages and state slots that are used
again, keys far back and at page borders, the first tokens of a sequence, long decoding, sizes of several kinds,
greedy generation through the engine's own entry point and scheduler."""
import numpy as np
import pytest
import torch

import plain_lufatar as plain
from conftest import assert_logits_close, rel_err
from test_misudra_gpu import Harness, Want, tokens_of

pytestmark = pytest.mark.gpu

A, moe = plain.attention_layer, plain.moe

# Configurations. None is a model anyone serves: sizes differ from one another wherever two could be mistaken for each other.
MIXED = plain.make_config([A(), A(heads=6, kv_heads=3, dim=8, vdim=12, rot_dims=8, mlp=moe(ff=40, experts=6, top=3, groups=3, keep=2)),
                           A(heads=2, kv_heads=1, dim=24, vdim=16, rot_dims=12, mlp=None), A(heads=4, kv_heads=4, dim=16, vdim=8, rot_dims=None),
                           A(heads=2, kv_heads=2, dim=32, vdim=40, rot_dims=32, base=500.0, scale=0.4)], loop=(1, 4, 2))
ODD = plain.make_config([A(heads=3, kv_heads=1, dim=10, vdim=7, rot_dims=4, mlp=moe(ff=20, experts=6, top=3, groups=3, keep=2)),
                         A(heads=6, kv_heads=3, dim=12, vdim=20, rot_dims=12, scale=0.5, mlp=None),
                         A(heads=5, kv_heads=5, dim=6, vdim=9, rot_dims=0, mlp=moe(ff=11, experts=9, top=4, groups=3, keep=3)),
                         A(heads=2, kv_heads=1, dim=66, vdim=34, rot_dims=2, mlp=moe(ff=50, experts=4, top=2, groups=1, keep=1))],
                        vocab=97, width=36, eps=1e-5, groups=3, mult=1.3, taps=2, side=5, bigram=(7, 1000003, 99991), loop=(0, 3, 3))
ONES = plain.make_config([A(heads=1, kv_heads=1, dim=8, vdim=8, rot_dims=8, mlp=moe(ff=8, experts=2, top=1, groups=1, keep=1)),
                          A(heads=1, kv_heads=1, dim=8, vdim=8, rot_dims=2, mlp=moe(ff=8, experts=2, top=2, groups=2, keep=2))],
                         vocab=33, width=16, groups=1, mult=1.0, taps=1, side=1, bigram=(1, 1, 1), loop=(1, 2, 1))
# sizes in whole 16-byte pieces and larger heads: what tensor-core kernels take where the engine has them for a mechanism
SQUARE = plain.make_config([A(heads=8, kv_heads=2, dim=64, vdim=64, rot_dims=32, mlp=moe(ff=64, experts=16, top=4, groups=4, keep=2)),
                            A(heads=16, kv_heads=16, dim=32, vdim=32, rot_dims=32, mlp=moe(ff=32, experts=12, top=3, groups=4, keep=3)),
                            A(heads=4, kv_heads=1, dim=128, vdim=64, rot_dims=64, base=500000.0, mlp=None),
                            A(heads=4, kv_heads=2, dim=64, vdim=128, rot_dims=16)], width=128, groups=4, taps=4, side=16, loop=(0, 2, 2))
# every optional mechanism left out: no pair table, no input convolution, no token side input, no loop, plain norms
BARE = plain.make_config([A(), A(mlp=None)], groups=1, taps=0, side=0, bigram=None)
GAIN = 0.1      # see `plain.random_weights`: what the experts add in whole-model tests, so that a routing flip stays small in bfloat16
CONFIGS = {"mixed": (MIXED, 16), "odd": (ODD, 8), "ones": (ONES, 4), "square": (SQUARE, 16), "bare": (BARE, 32)}


def row_errors(got, want):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    got, want = got.reshape(-1, got.shape[-1]), want.reshape(-1, want.shape[-1])
    return np.abs(got - want).max(axis=-1) / np.abs(want).max(axis=-1)


def close(got, want, dtype, what):
    """Per row, the largest difference relative to the row's largest logit. float32: 1e-4, and up to 1e-3 on 3% of the rows.
    bfloat16: four times the noise that 16-bit activations give the plain implementation on this model and prompt (at least
    5e-3), and up to ten times on 5% of the rows. The few rows with more room are the ill-conditioned ones: the token side
    input divides a few numbers by their root mean square, which magnifies rounding where they are all small, and a
    routing decision between two nearly equal scores falls either way."""
    err = row_errors(got, want.rows)
    if dtype == "float32":
        tol, some, most = 1e-4, 0.03, 10.0
    else:
        tol, some, most = 4.0 * max(want.noise, 5e-3), 0.05, 2.5
    over = int((err > tol).sum())
    assert err.max() <= most * tol and over <= max(1, int(some * len(err))), \
        f"{what}: worst row {err.max():.3e}, {over} of {len(err)} rows above {tol:.1e} ({dtype}; noise of rounding {want.noise:.1e})"


def reference(w, cfg, toks):
    exact = plain.forward(w, cfg, toks)
    with plain.bfloat16_activations():
        rounded = plain.forward(w, cfg, toks)
    return Want(exact, rel_err(rounded, exact))


@pytest.fixture(scope="module")
def truth():
    memo = {}

    def get(name, toks):
        key = (name, tuple(toks))
        if key not in memo:
            cfg = CONFIGS[name][0]
            memo[key] = reference(plain.random_weights(cfg, 5, expert_gain=GAIN), cfg, toks)
        return memo[key]
    return get


# ---------------------------------------------------------------------------------------------- each mechanism alone

SINGLE = {
    "attention": plain.make_config([A(mlp=None)], groups=1, taps=0, side=0, bigram=None),
    "attention_no_rotation": plain.make_config([A(rot_dims=None, mlp=None)], groups=1, taps=0, side=0, bigram=None),
    "experts": plain.make_config([A(mlp=moe(ff=24, experts=12, top=3, groups=4, keep=2))], groups=1, taps=0, side=0, bigram=None),
    "grouped_norm": plain.make_config([A(mlp=None)], groups=4, taps=0, side=0, bigram=None),
    "input_convolution": plain.make_config([A()], groups=1, taps=4, side=0, bigram=None),
    "token_side": plain.make_config([A(mlp=None), A(mlp=None)], groups=1, taps=0, side=7, bigram=None),
    "pair_table": plain.make_config([A(mlp=None)], groups=1, taps=0, side=0, bigram=(31, 17, 5)),
    "loop": plain.make_config([A(mlp=None), A(mlp=None)], groups=1, taps=0, side=0, bigram=None, loop=(0, 2, 3)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SINGLE))
def test_each_mechanism_alone(tmp_path, name, dtype):
    """One mechanism switched on in an otherwise bare model, at full expert gain; in float32 the residual stream after
    every layer run is compared as well."""
    cfg = SINGLE[name]
    w = plain.random_weights(cfg, 11)
    toks = tokens_of(cfg, 45, 3)
    layers = []
    exact = plain.forward(w, cfg, toks, layers_out=layers)
    hs = Harness(tmp_path, cfg, w, dtype, page=8)
    got_layers = []
    if dtype == "float32":
        hs.runner.layer_hook = lambda i, x, pending: got_layers.append(x.detach().float().cpu().numpy().copy())
    got = hs.whole("w", toks)
    if dtype == "float32":
        assert len(got_layers) == len(layers)
        for i, (g, e) in enumerate(zip(got_layers, layers)):
            assert np.abs(g - e).max() <= 2e-5 * max(1.0, np.abs(e).max()), f"{name}: stream after layer run {i}"
        assert_logits_close(got, exact, dtype, name)
    else:
        with plain.bfloat16_activations():
            rounded = plain.forward(w, cfg, toks)
        err, noise = rel_err(got, exact), rel_err(rounded, exact)
        assert err <= max(3e-2, 4 * noise), f"{name}: {err:.3e} (noise {noise:.1e})"
    hs.runner.layer_hook = None
    if dtype == "float32":
        assert_logits_close(hs.in_portions("p", toks, [1, 2, 5, 1, 13]), exact, dtype, f"{name} in portions")


@pytest.mark.parametrize("shape", [(20, 4, 5, 3), (6, 3, 3, 2), (8, 3, 4, 3), (64, 8, 8, 4), (12, 1, 12, 1), (2, 1, 1, 1), (2, 2, 2, 2), (96, 6, 1, 1)])
def test_routing_kernel_against_the_plain_rule(shape):
    """Sigmoid scores, a correction that makes many choice scores negative, groups counted by their two best members,
    weights without the correction and not renormed."""
    from tiny_inference_engine_b200 import ops
    E, top, groups, keep = shape
    rng = np.random.default_rng(E * 7 + top)
    z = rng.standard_normal((300, E)).astype(np.float32) * 2.0
    corr = (rng.standard_normal(E) * 0.5 - 0.8).astype(np.float32)
    want_ids, want_w = plain.route(z, corr, top, groups, keep)
    ids = torch.zeros((300, top), dtype=torch.int32, device="cuda")
    wts = torch.zeros((300, top), dtype=torch.float32, device="cuda")
    ops.moe_route(torch.from_numpy(z).cuda(), top, groups, keep, ids, wts, score_fn=ops.ROUTE_SIGMOID,
                  correction=torch.from_numpy(corr).cuda(), group_top=2, renorm=False)
    ids, wts = ids.cpu().numpy(), wts.cpu().numpy()
    # close calls between two experts may fall either way in float32: rows whose chosen sets differ must be such calls
    s = 1.0 / (1.0 + np.exp(-z.astype(np.float64))) + corr
    differ = 0
    for t in range(300):
        if sorted(ids[t]) != sorted(want_ids[t]):
            differ += 1
            only = set(ids[t]) ^ set(want_ids[t].tolist())
            assert np.ptp([s[t, e] for e in only]) < 1e-5, f"row {t}: chose {sorted(ids[t])}, plain {sorted(want_ids[t])}"
        else:
            order = np.argsort(ids[t])
            np.testing.assert_allclose(wts[t][order], want_w[t][np.argsort(want_ids[t])], rtol=1e-5, atol=1e-6)
    assert differ <= 3


def test_groups_with_negative_choice_scores_still_shut_their_experts_out():
    """All choice scores negative: experts of a group that is not kept stay out although 0 would beat every kept one."""
    from tiny_inference_engine_b200 import ops
    z = np.array([[3.0, 2.5, 0.1, 0.2, 2.0, -1.0]], dtype=np.float32)          # groups {0,1} {2,3} {4,5}
    corr = np.full(6, -5.0, dtype=np.float32)
    want_ids, want_w = plain.route(z, corr, 3, 3, 2)
    assert sorted(want_ids[0]) == [0, 1, 4]
    ids = torch.zeros((1, 3), dtype=torch.int32, device="cuda")
    wts = torch.zeros((1, 3), dtype=torch.float32, device="cuda")
    ops.moe_route(torch.from_numpy(z).cuda(), 3, 3, 2, ids, wts, score_fn=ops.ROUTE_SIGMOID, correction=torch.from_numpy(corr).cuda(),
                  group_top=2, renorm=False)
    assert sorted(ids.cpu().numpy()[0]) == [0, 1, 4]
    np.testing.assert_allclose(np.sort(wts.cpu().numpy()[0]), np.sort(want_w[0]), rtol=1e-5)


# ---------------------------------------------------------------------------------------------- whole models

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_decoding_and_portions(tmp_path, truth, name, dtype):
    """The same logits at every position whether the prompt comes whole, token by token from the first token on (the
    pair table's first row, the convolutions' zero padding), or in portions of several sizes down to two."""
    cfg, page = CONFIGS[name]
    w = plain.random_weights(cfg, 5, expert_gain=GAIN)
    toks = tokens_of(cfg, 150, 2)
    want = truth(name, toks)
    hs = Harness(tmp_path, cfg, w, dtype, page=page, pages=256 // page * 2)
    close(hs.whole("w", toks), want, dtype, f"{name} whole")
    close(hs.in_portions("d", toks, [1]), want, dtype, f"{name} token by token")
    close(hs.in_portions("p", toks, [2, 3, 17, 2, 1, 40, 5]), want, dtype, f"{name} portions")
    close(hs.in_portions("q", toks, [1, 1, 2, 64, 7]), want, dtype, f"{name} first tokens one by one, then portions")
    rows = hs.step([("m", toks[:101], [100])])
    for i in range(101, 150):
        rows.update(hs.step([("m", toks[i:i + 1], [0])]))
    hs.cache.release(hs.live.pop("m")[0])
    close(np.stack([rows[("m", i)] for i in range(100, 150)]), want[100:], dtype, f"{name} prompt then decoding")


@pytest.mark.parametrize("n", [1, 2, 3])
def test_the_first_tokens_of_a_sequence(tmp_path, n):
    """Prompts of one to three tokens: the pair table's first row, a convolution that reaches ahead of the sequence, a
    softmax over one key and the sink."""
    cfg, page = CONFIGS["mixed"]
    w = plain.random_weights(cfg, 5)
    hs = Harness(tmp_path, cfg, w, "float32", page=page)
    for seed in range(3):
        toks = tokens_of(cfg, n, 90 + seed)
        assert_logits_close(hs.whole("w", toks), plain.forward(w, cfg, toks), "float32", f"{n} tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "square"])
def test_mixed_batches_on_a_small_pool_with_two_state_slots(tmp_path, truth, name, dtype):
    """Requests of unequal lengths, portions of some beside single tokens of others, never more than two alive:
    pages and state slots are given back and used again, and every row equals the request run alone."""
    cfg, page = CONFIGS[name]
    w = plain.random_weights(cfg, 5, expert_gain=GAIN)
    lengths = [70, 33, 2, 90, 47, 64]
    reqs = [tokens_of(cfg, n, 10 + i) for i, n in enumerate(lengths)]
    want = [truth(name, r) for r in reqs]
    hs = Harness(tmp_path, cfg, w, dtype, page=page, pages=(2 * 128) // page, slots=2)
    rows, at = {}, [0] * len(reqs)
    pending, alive, turn = list(range(len(reqs))), [], 0
    sizes = [5, 1, 2, 31, 1, 1, 16, 3]
    while pending or alive:
        while pending and len(alive) < 2:
            alive.append(pending.pop(0))
        entries, ended = [], []
        for k, i in enumerate(alive):
            n = min(1 if (turn + k) % 3 == 0 else sizes[(turn + i) % len(sizes)], lengths[i] - at[i])
            entries.append((f"r{i}", reqs[i][at[i]:at[i] + n], range(n)))
            at[i] += n
            if at[i] == lengths[i]:
                ended.append(i)
        rows.update(hs.step(entries, end=[f"r{i}" for i in ended]))
        alive = [i for i in alive if i not in ended]
        turn += 1
    assert hs.states.num_free == 2 and all(p.num_free == p.num_blocks for p in hs.cache.pools)
    for i, r in enumerate(reqs):
        close(np.stack([rows[(f"r{i}", j)] for j in range(len(r))]), want[i], dtype, f"{name} request {i} in mixed batches")


def test_a_request_left_out_of_steps_goes_on_where_it_stopped(tmp_path, truth):
    """A request pauses while others run and slots around it change hands: its ring of convolution inputs and its last token
    are its own."""
    cfg, page = CONFIGS["mixed"]
    w = plain.random_weights(cfg, 5, expert_gain=GAIN)
    a, b, c = (tokens_of(cfg, n, 60 + i) for i, n in enumerate([40, 30, 25]))
    hs = Harness(tmp_path, cfg, w, "float32", page=page, pages=16, slots=2)
    rows = hs.step([("a", a[:7], range(7)), ("b", b[:29], range(29))])
    rows.update(hs.step([("b", b[29:], [0])], end=["b"]))
    rows.update(hs.step([("c", c, range(25))], end=["c"]))
    rows.update(hs.step([("a", a[7:9], range(2))]))
    rows.update(hs.step([("a", a[9:], range(31))], end=["a"]))
    for rid, toks in (("a", a), ("b", b), ("c", c)):
        close(np.stack([rows[(rid, j)] for j in range(len(toks))]), truth("mixed", toks), "float32", rid)


# ---------------------------------------------------------------------------------------------- edges that random weights would hide

def _peaked_rows(L, page, targets, dtype, seed=0, H=4, G=2, dim=16, vdim=8, scale=0.5):
    """A cache of L keys on shuffled pages and one query per entry of `targets` = [(position of the query, key it asks for)]:
    the query is a multiple of that key, so that among hundreds of keys this one carries the softmax if the kernel sees it."""
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((L, G, dim))
    k /= np.sqrt((k * k).mean(-1, keepdims=True))
    v = rng.standard_normal((L, G, vdim))
    talk = np.eye(H) + rng.standard_normal((H, H)) * 0.2
    q = rng.standard_normal((L, H, dim)) * 0.1
    for pos, key in targets:
        for h in range(H):
            q[pos, h] += 1.6 * k[key, h // (H // G)]
    rnd = plain.round_bf16 if dtype == torch.bfloat16 else (lambda a: np.asarray(a, dtype=np.float32))
    q, k, v = (rnd(np.asarray(a, dtype=np.float32)).astype(np.float64) for a in (q, k, v))
    want = plain.attend(q, k, v, talk, scale)
    n_pages = -(-L // page)
    order = rng.permutation(n_pages + 3)[:n_pages]
    kc = torch.zeros((n_pages + 3, G, page, dim), dtype=dtype, device="cuda")
    vc = torch.zeros((n_pages + 3, G, page, vdim), dtype=dtype, device="cuda")
    kt, vt = torch.from_numpy(k).to(dtype).cuda(), torch.from_numpy(v).to(dtype).cuda()
    for j in range(L):
        kc[order[j // page], :, j % page] = kt[j]
        vc[order[j // page], :, j % page] = vt[j]
    return q, want, kc, vc, torch.from_numpy(talk.astype(np.float32)).cuda(), order, (H, G, dim, vdim, scale)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("page", [16, 8, 64])
def test_a_key_far_back_at_a_page_border_or_one_past_the_query(dtype, page):
    """Queries of a prompt's portion and a decoded token that each ask for one key: the first ones, the keys on both sides of
    page borders, one 600 back, the query's own, and the one right after it (which it must not see)."""
    from tiny_inference_engine_b200 import ops
    L, n = 700, 48
    first = L - n
    keys = [0, 1, 2, page - 1, page, page + 1, 4 * page - 1, 4 * page, 255, 256, 257, L - 600, first - 1, first]
    targets = [(first + i, keys[i]) for i in range(len(keys))]
    targets += [(first + 20 + i, first + 20 + i + d) for i, d in enumerate([0, -1, 1, 1, 0, -1, 1, -2])]     # own, before, after
    targets += [(L - 1, L - 600)]
    q, want, kc, vc, talk, order, (H, G, dim, vdim, scale) = _peaked_rows(L, page, targets, dtype)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    # a portion: rows first .. L-1 of one sequence whose earlier keys are in the cache
    qd = torch.from_numpy(q[first:].reshape(n, H * dim)).to(dtype).cuda()
    out = torch.zeros((n, H * vdim), dtype=dtype, device="cuda")
    arrays = (i32([0] * n), i32([0, n]), i32([L]), i32([list(order)]))
    ops.attention_mixed(qd, kc, vc, out, talk, arrays, n, H, G, dim, vdim, scale, True)
    got = out.float().cpu().numpy().reshape(n, H, vdim)
    assert np.abs(got - want[first:]).max() <= tol * np.abs(want).max(), "rows of a portion"
    # one decoded token at several lengths of the sequence, its keys cut into splits
    for pos in [t[0] for t in targets[len(keys):]] + [first + 3, first + 11]:
        qd = torch.from_numpy(q[pos].reshape(1, H * dim)).to(dtype).cuda()
        out = torch.zeros((1, H * vdim), dtype=dtype, device="cuda")
        arrays = (i32([0]), i32([0, 1]), i32([pos + 1]), i32([list(order)]))
        for split_keys in (64, 256):
            splits = -(-(pos + 1) // split_keys)
            scratch = torch.zeros(ops.attention_split_scratch_floats(1, H, vdim, splits), dtype=torch.float32, device="cuda")
            ops.attention_mixed(qd, kc, vc, out, talk, arrays, 0, H, G, dim, vdim, scale, True, seq_list=i32([0]), n_list=1,
                                split_keys=split_keys, max_splits=splits, scratch=scratch)
            got = out.float().cpu().numpy().reshape(H, vdim)
            assert np.abs(got - want[pos]).max() <= tol * np.abs(want).max(), f"decoded token at {pos}, splits of {split_keys}"


@pytest.mark.parametrize("geometry", [(4, 2, 128, 64), (2, 1, 64, 64), (8, 2, 64, 128), (3, 3, 128, 128), (12, 4, 64, 64), (16, 4, 64, 64),
                                      (1, 1, 64, 128), (6, 2, 128, 128), (16, 8, 128, 128), (32, 8, 128, 128), (16, 16, 128, 128),
                                      (32, 1, 64, 64), (24, 2, 64, 128), (12, 2, 128, 64)])
@pytest.mark.parametrize("page", [16, 64])
def test_prompt_portions_on_the_tensor_cores(geometry, page):
    """The bfloat16 kernel: two sequences in one call, portions that start and end inside key tiles and pages, queries that
    ask for single keys (far back, at borders, their own, the one after them), against the plain rule and against the
    CUDA-core kernel; then single rows of two sequences with their keys in splits."""
    from tiny_inference_engine_b200 import ops
    H, G, dim, vdim = geometry
    assert ops.attention_mixed_tc_takes(H, G, dim, vdim)
    assert not ops.attention_mixed_tc_takes(32, 32, 128, 128) and not ops.attention_mixed_tc_takes(4, 2, 48, 64)     # the CUDA-core kernel's
    L = 700
    spans = [(652, 700), (263, 300)]                      # rows of the step: positions [a, b) of a sequence b long
    keys = [0, 1, page - 1, page, 63, 64, 65, 255, 256, 100, 651, 652]
    targets = [(652 + i, keys[i]) for i in range(len(keys))] + [(670 + i, 670 + i + d) for i, d in enumerate([0, -1, 1, 1, 0, -2])]
    targets += [(263 + i, k) for i, k in enumerate([0, 63, 64, 127, 128, 262, 263, 200])] + [(290 + i, 290 + i + d) for i, d in enumerate([1, 0, -1])]
    q, want, kc, vc, talk, order, (_, _, _, _, scale) = _peaked_rows(L, page, targets, torch.bfloat16, seed=H, H=H, G=G, dim=dim, vdim=vdim,
                                                                    scale=0.5 * (16 / dim) ** 0.5)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    rows = [p for a, b in spans for p in range(a, b)]
    qd = torch.from_numpy(q[rows].reshape(len(rows), H * dim)).to(torch.bfloat16).cuda()
    starts, lens = [0, 48, 85], [700, 300]
    tables = i32([list(order), list(order)])
    out = torch.zeros((len(rows), H * vdim), dtype=torch.bfloat16, device="cuda")
    ops.attention_mixed_tc(qd, kc, vc, out, talk, i32(starts), i32(lens), tables, 2, 48, H, G, dim, vdim, scale, True)
    got = out.float().cpu().numpy().reshape(len(rows), H, vdim)
    assert np.abs(got - want[rows]).max() <= 1e-2 * np.abs(want).max(), "against the plain rule"
    simt = torch.zeros_like(out)
    ops.attention_mixed(qd, kc, vc, simt, talk, (i32([0] * 48 + [1] * 37), i32(starts), i32(lens), tables), len(rows), H, G, dim, vdim, scale, True)
    assert np.abs(got - simt.float().cpu().numpy().reshape(got.shape)).max() <= 1e-2 * np.abs(want).max(), "against the CUDA-core kernel"
    for sink, mix in ((False, talk), (True, None)):
        a, b = torch.zeros_like(out), torch.zeros_like(out)
        ops.attention_mixed_tc(qd, kc, vc, a, mix, i32(starts), i32(lens), tables, 2, 48, H, G, dim, vdim, scale, sink)
        ops.attention_mixed(qd, kc, vc, b, mix, (i32([0] * 48 + [1] * 37), i32(starts), i32(lens), tables), len(rows), H, G, dim, vdim, scale, sink)
        assert (a.float() - b.float()).abs().max().item() <= 1e-2 * np.abs(want).max(), f"sink {sink}, mix {mix is not None}"
    # single rows: the last row of each sequence (one asks for key 651 ... of its own sequence), splits of 64 and of 256 keys
    singles = [(699, 700), (299, 300), (663, 664), (275, 276)]          # (position, length)
    for a_row, b_row in ((0, 1), (2, 3)):
        pair = [singles[a_row], singles[b_row]]
        qd1 = torch.from_numpy(q[[p for p, _ in pair]].reshape(2, H * dim)).to(torch.bfloat16).cuda()
        lens1, starts1 = i32([n for _, n in pair]), i32([0, 1, 2])
        for split_keys, sink in ((64, True), (256, True), (128, False)):
            splits = -(-max(n for _, n in pair) // split_keys)
            got1, simt1 = torch.zeros((2, H * vdim), dtype=torch.bfloat16, device="cuda"), torch.zeros((2, H * vdim), dtype=torch.bfloat16, device="cuda")
            scratch = torch.zeros(ops.attention_split_scratch_floats(2, H, vdim, splits), dtype=torch.float32, device="cuda")
            ops.attention_mixed_tc(qd1, kc, vc, got1, talk, starts1, lens1, tables, 2, 1, H, G, dim, vdim, scale, sink,
                                   seq_list=i32([0, 1]), split_keys=split_keys, max_splits=splits, scratch=scratch)
            scratch.zero_()
            ops.attention_mixed(qd1, kc, vc, simt1, talk, (i32([0, 1]), starts1, lens1, tables), 0, H, G, dim, vdim, scale, sink,
                                seq_list=i32([0, 1]), n_list=2, split_keys=split_keys, max_splits=splits, scratch=scratch)
            assert (got1.float() - simt1.float()).abs().max().item() <= 1e-2 * np.abs(want).max(), f"single rows, splits of {split_keys}"
            if sink:
                g1 = got1.float().cpu().numpy().reshape(2, H, vdim)
                assert np.abs(g1 - want[[p for p, _ in pair]]).max() <= 1e-2 * np.abs(want).max(), f"single rows against the plain rule, splits of {split_keys}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "square"])
def test_the_token_side_input_as_matrix_products(tmp_path, truth, name, dtype, monkeypatch):
    """Steps of many rows take the side input as two matrix products between small kernels: the same logits, whole and in
    portions (portions below the bound go the other way, in the same request)."""
    from tiny_inference_engine_b200.parts import block
    monkeypatch.setattr(block, "SIDE_PRODUCT_ROWS", 12)
    cfg, page = CONFIGS[name]
    w = plain.random_weights(cfg, 5, expert_gain=GAIN)
    toks = tokens_of(cfg, 150, 2)
    want = truth(name, toks)
    hs = Harness(tmp_path, cfg, w, dtype, page=page, pages=256 // page * 2)
    close(hs.whole("w", toks), want, dtype, f"{name} whole")
    close(hs.in_portions("p", toks, [40, 3, 12, 1, 30, 11, 2]), want, dtype, f"{name} in portions")


@pytest.mark.parametrize("shape", [(256, 16, 3), (36, 5, 1), (2048, 64, 2), (40, 8, 0), (30, 6, 2)])
def test_sublayer_sum_and_token_side_input_for_few_and_for_more_rows(shape):
    """x += mult * (a + b), the token side input and the ring update: a handful of rows (a thread-block cluster a row,
    many times over: the CTAs of a cluster read the row that one of them writes), some dozens of rows (a block a row)
    and the three kernels around two matrix products, against the plain rule."""
    from types import SimpleNamespace
    from tiny_inference_engine_b200 import ops
    D, S, R = shape
    rng = np.random.default_rng(D + S)
    vocab, mult, eps = 50, 0.7, 1e-5
    table, gate = rng.standard_normal((vocab, S)).astype(np.float32), (rng.standard_normal((S, D)) / np.sqrt(D)).astype(np.float32)
    proj, norm = rng.standard_normal((D, S)).astype(np.float32), rng.standard_normal(D).astype(np.float32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    side = tuple(dev(a) for a in (table, gate, proj, norm))
    for T in (5, 40):
        x, da, db = (rng.standard_normal((T, D)).astype(np.float32) for _ in range(3))
        tokens = rng.integers(0, vocab, T)
        unit = rng.standard_normal((T, D)).astype(np.float32)
        ring0 = rng.standard_normal((2, max(R, 1), D)).astype(np.float32)
        first = 7                                           # one sequence, rows at positions 7 .. 7 + T - 1, slot 1
        xs = x.astype(np.float64) + mult * (da.astype(np.float64) + db)
        g = plain.gelu_tanh(xs @ gate.T.astype(np.float64)) * table[tokens]
        y = g @ proj.T.astype(np.float64)
        want = xs + mult * y / np.sqrt((y * y).mean(-1, keepdims=True) + eps) * norm
        want_ring = ring0.copy()
        for i in range(max(0, T - R), T):
            want_ring[1, (first + i) % R] = unit[i]
        ctx = SimpleNamespace(tokens=i32(tokens), seq_of_row=i32([0] * T), positions=i32(range(first, first + T)),
                              context_lens=i32([first + T]), state_slots=i32([1]))
        for _ in range(25 if T == 5 else 2):
            xd, ring = dev(x), dev(ring0)
            ops.parallel_finish(xd, mult, dev(da), dev(db), torch.float32, ctx=ctx, side=side, eps=eps, unit=dev(unit) if R else None,
                                ring=ring if R else None)
            assert np.abs(xd.cpu().numpy() - want).max() <= 2e-5 * np.abs(want).max(), f"{T} rows"
            if R:
                assert np.array_equal(ring.cpu().numpy(), want_ring), f"the ring after {T} rows"
        # the same through the kernels of the many-row path
        xd, ring, copy = dev(x), dev(ring0), torch.zeros((T, D), dtype=torch.float32, device="cuda")
        ops.parallel_sum(xd, mult, dev(da), dev(db), copy)
        assert np.abs(copy.cpu().numpy() - xs).max() <= 1e-5 * np.abs(xs).max() and torch.equal(copy, xd)
        gd = torch.zeros((T, S), dtype=torch.float32, device="cuda")
        ops.side_gate_act(dev((xs @ gate.T.astype(np.float64)).astype(np.float32)), side[0], ctx.tokens, gd)
        assert np.abs(gd.cpu().numpy() - g).max() <= 1e-5 * np.abs(g).max()
        ops.side_finish(xd, dev(y.astype(np.float32)), mult, eps, side[3], ctx=ctx, unit=dev(unit) if R else None, ring=ring if R else None)
        assert np.abs(xd.cpu().numpy() - want).max() <= 2e-5 * np.abs(want).max()
        if R:
            assert np.array_equal(ring.cpu().numpy(), want_ring)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(32, 2, 4), (36, 3, 2), (64, 1, 3), (24, 4, 1)])
def test_grouped_norm_with_taps_in_tiles_of_rows(shape, dtype):
    """The norm and input convolution kernel in tiles of one, five and eight rows: the same numbers to the bit, and the plain
    rule's: two sequences in one step, one going on from its ring at a position that is no multiple of the ring's length,
    one from its first token (zeros ahead of it), a third row block that starts inside a tile."""
    from types import SimpleNamespace
    from tiny_inference_engine_b200 import ops
    D, groups, taps = shape
    R = taps - 1
    rng = np.random.default_rng(D)
    spans = [(10, 21), (0, 13), (5, 7)]             # (first position, rows) of each sequence of the step; slots 2, 0, 1
    slots = [2, 0, 1]
    T = sum(n for _, n in spans)
    x = rng.standard_normal((T, D)).astype(np.float32) * 3.0
    ring = rng.standard_normal((3, max(R, 1), D)).astype(np.float32)
    wa, wb = rng.standard_normal(D).astype(np.float32), rng.standard_normal(D).astype(np.float32)
    ta, tb = rng.standard_normal((D, taps)).astype(np.float32), rng.standard_normal((D, taps)).astype(np.float32)
    eps = 1e-5
    xg = x.reshape(T, groups, D // groups).astype(np.float64)
    unit = (xg / np.sqrt((xg * xg).mean(-1, keepdims=True) + eps)).reshape(T, D)
    want_a, want_b = np.zeros((T, D)), np.zeros((T, D))
    seq_of_row, positions, starts, t = [], [], [0], 0
    for s, (p0, n) in enumerate(spans):
        for i in range(n):
            back = []                               # unit rows at positions p - taps + 1 .. p
            for r in range(R, -1, -1):
                p = p0 + i - r
                back.append(unit[t + i - r] if i - r >= 0 else ring[slots[s], p % R].astype(np.float64) if p >= 0 else np.zeros(D))
            conv_a = sum(ta[:, j] * back[j] for j in range(taps))
            conv_b = sum(tb[:, j] * back[j] for j in range(taps))
            want_a[t + i], want_b[t + i] = wa * (unit[t + i] + conv_a), wb * (unit[t + i] + conv_b)
            seq_of_row.append(s), positions.append(p0 + i)
        t += n
        starts.append(t)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    ctx = SimpleNamespace(seq_of_row=i32(seq_of_row), positions=i32(positions), query_start=i32(starts),
                          context_lens=i32([p0 + n for p0, n in spans]), state_slots=i32(slots))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    outs = []
    for tile in (1, 5, 8):
        oa, ob = torch.zeros((T, D), dtype=dtype, device="cuda"), torch.zeros((T, D), dtype=dtype, device="cuda")
        left = torch.zeros((T, D), dtype=torch.float32, device="cuda")
        ops.group_norm_taps(dev(x), groups, eps, dev(wa), oa, dev(wb), ob, dev(ta.T), dev(tb.T), ctx=ctx, unit=left if R else None,
                            ring=dev(ring) if R else None, tile=tile)
        outs.append((oa.float().cpu().numpy(), ob.float().cpu().numpy(), left.cpu().numpy()))
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert np.abs(outs[0][0] - want_a).max() <= tol * np.abs(want_a).max() and np.abs(outs[0][1] - want_b).max() <= tol * np.abs(want_b).max()
    for o in outs[1:]:
        assert all(np.array_equal(a, b) for a, b in zip(o, outs[0])), "a row's numbers depend on its tile"
    if R:
        t = 0
        for p0, n in spans:                         # the rows that will be the ring: a sequence's last taps - 1 unit rows
            for i in range(max(0, n - R), n):
                assert np.abs(outs[0][2][t + i] - unit[t + i]).max() <= 1e-5
            t += n


def test_the_sink_takes_weight_and_the_head_mix_moves_it():
    """Without the sink the weights of a row sum to one; with it, to less: a query that matches no key gives almost nothing."""
    from tiny_inference_engine_b200 import ops
    q, want, kc, vc, talk, order, (H, G, dim, vdim, scale) = _peaked_rows(40, 8, [], torch.float32, seed=3)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    arrays = (i32([0] * 40), i32([0, 40]), i32([40]), i32([list(order)]))
    qd = torch.from_numpy(q.reshape(40, H * dim)).float().cuda()
    vc.fill_(1.0)
    outs = {}
    for sink in (False, True):
        for mix in (None, talk):
            out = torch.zeros((40, H * vdim), dtype=torch.float32, device="cuda")
            ops.attention_mixed(qd, kc, vc, out, mix, arrays, 40, H, G, dim, vdim, scale, sink)
            outs[(sink, mix is not None)] = out.cpu().numpy()
    assert np.allclose(outs[(False, False)], 1.0, atol=1e-5) and np.allclose(outs[(False, True)], 1.0, atol=1e-5)
    assert (outs[(True, True)] < 1.0 - 1e-3).all() and outs[(True, True)][0].max() < 0.8      # one key and the sink share the first row
    assert np.abs(outs[(True, True)] - outs[(True, False)]).max() > 1e-3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_peaked_attention_over_a_long_prompt_and_decoding(tmp_path, dtype):
    """A large score scale makes every head pick single keys anywhere in 600 tokens; portions end inside pages."""
    cfg = plain.make_config([A(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, scale=1.2, mlp=None),
                             A(heads=2, kv_heads=1, dim=32, vdim=16, rot_dims=32, scale=0.7, mlp=None)], width=48, loop=(0, 2, 2))
    w = plain.random_weights(cfg, 21)
    toks = tokens_of(cfg, 600, 8)
    want = reference(w, cfg, toks)
    hs = Harness(tmp_path, cfg, w, dtype, page=16, pages=80, max_tokens=640)
    close(hs.whole("w", toks), want, dtype, "whole")
    rows = {}
    for a, b in [(0, 250), (250, 263), (263, 265), (265, 560)]:
        rows.update(hs.step([("p", toks[a:b], range(b - a))]))
    for i in range(560, 600):
        rows.update(hs.step([("p", toks[i:i + 1], [0])]))
    close(np.stack([rows[("p", i)] for i in range(600)]), want, dtype, "portions, then decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps_and_slots_used_again(tmp_path, truth, dtype):
    """Three requests decode together for 200 steps (steps of one token each are captured as graphs and replayed),
    end at different times, and a fourth takes over a slot and pages that were just given back."""
    cfg, page = CONFIGS["mixed"]
    w = plain.random_weights(cfg, 5, expert_gain=GAIN)
    reqs = [tokens_of(cfg, n, 20 + i) for i, n in enumerate([230, 215, 260, 120])]
    want = [truth("mixed", r) for r in reqs]
    hs = Harness(tmp_path, cfg, w, dtype, page=page, pages=3 * 272 // page, slots=3)
    rows = hs.step([(f"r{i}", reqs[i][:12 + i], range(12 + i)) for i in range(3)])
    at = [12, 13, 14, 0]
    alive = [0, 1, 2]
    while alive:
        ended = [i for i in alive if at[i] + 1 == len(reqs[i])]
        rows.update(hs.step([(f"r{i}", reqs[i][at[i]:at[i] + 1], [0]) for i in alive], end=[f"r{i}" for i in ended]))
        for i in alive:
            at[i] += 1
        alive = [i for i in alive if i not in ended]
        if ended and at[3] == 0:                          # the newcomer's prompt rides beside the others' single tokens
            rows.update(hs.step([("r3", reqs[3][:40], range(40))] + [(f"r{i}", reqs[i][at[i]:at[i] + 1], [0]) for i in alive]))
            for i in alive:
                at[i] += 1
            at[3] = 40
            alive.append(3)
    assert hs.runner.graph_replays > 100, "decode steps of this model are meant to be captured"
    for i, r in enumerate(reqs):
        close(np.stack([rows[(f"r{i}", j)] for j in range(len(r))]), want[i], dtype, f"request {i}")


# ---------------------------------------------------------------------------------------------- the engine's own entry points

def test_greedy_generation_through_the_engine_and_its_scheduler(tmp_path):
    """`load_engine` + `generate` / `generate_batch`: the scheduler admits, cuts prompts into portions under a small
    token budget, runs on a small pool; the tokens are the plain implementation's greedy ones."""
    from tiny_inference_engine_b200 import SamplingParams, ServingConfig, load_engine
    cfg, page = CONFIGS["mixed"]
    w = plain.random_weights(cfg, 5, expert_gain=GAIN)
    plain.write_model_dir(tmp_path, cfg, w)
    prompts = [tokens_of(cfg, n, 30 + i) for i, n in enumerate([19, 3, 41, 1, 27])]
    want = [plain.generate(w, cfg, p, 24) for p in prompts]
    engine = load_engine(tmp_path, dtype="float32", num_pages=40, page_size=page,
                         serving=ServingConfig(max_seqs=3, max_tokens_per_step=16))
    assert engine.generate(prompts[0], SamplingParams(max_tokens=24)) == want[0]
    assert engine.generate_batch(prompts, SamplingParams(max_tokens=24)) == want
    tight = load_engine(tmp_path, dtype="float32", num_pages=9, page_size=page,
                        serving=ServingConfig(max_seqs=3, max_tokens_per_step=16))
    assert tight.generate_batch(prompts, SamplingParams(max_tokens=24)) == want


def test_the_command_line_generates_the_plain_greedy_tokens(tmp_path, capsys):
    from tiny_inference_engine_b200.cli.main import main
    cfg, page = CONFIGS["odd"]
    w = plain.random_weights(cfg, 5, expert_gain=GAIN)
    plain.write_model_dir(tmp_path, cfg, w)
    prompt = tokens_of(cfg, 21, 77)
    assert main(["generate", "-m", str(tmp_path), "-p", " ".join(map(str, prompt)), "--temp", "0", "--max-tokens", "12",
                 "--dtype", "float32", "--kv-mem", "64M", "--max-tokens-per-step", "8", "--max-seqs", "2"]) == 0
    assert [int(t) for t in capsys.readouterr().out.split()] == plain.generate(w, cfg, prompt, 12)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_a_lufatar_model(tmp_path, truth, dtype):
    from test_replay_gpu import Replay
    cfg, page = CONFIGS["odd"]
    w = plain.random_weights(cfg, 5, expert_gain=GAIN)
    plain.write_model_dir(tmp_path / "m", cfg, w)
    reqs = [tokens_of(cfg, n, 40 + i) for i, n in enumerate([100, 37, 64, 2, 81])]
    want = [truth("odd", r) for r in reqs]
    V = cfg["vocab"]
    rp = Replay(tmp_path / "m", dtype, tmp_path / "out", max_tokens=4 * 128, page_size=page)
    try:
        got = rp.step([("a", reqs[0][:50], range(50)), ("b", reqs[1], range(37))], end=["b"]).reshape(87, V)
        close(got[:50], want[0][:50], dtype, "a, first portion")
        close(got[50:], want[1], dtype, "b whole beside it")
        got = rp.step([("c", reqs[2][:2], [1]), ("a", reqs[0][50:51], [0]), ("d", reqs[3], [0, 1])], end=["d"]).reshape(4, V)
        noise = max(x.noise for x in want)
        close(got, Want(np.stack([want[2].rows[1], want[0].rows[50], want[3].rows[0], want[3].rows[1]]), noise), dtype,
              "three requests, one step")
        assert rp.step([("e", reqs[4][:80], [])]) is None
        got = rp.step([("e", reqs[4][80:], [0]), ("a", reqs[0][51:], range(49)), ("c", reqs[2][2:], [61])],
                      end=["a", "c", "e"]).reshape(51, V)
        close(got, Want(np.concatenate([want[4].rows[80:81], want[0].rows[51:], want[2].rows[63:64]]), noise), dtype, "the rest")
    finally:
        rp.close()


# ---------------------------------------------------------------------------------------------- sizes drawn at random

def _random_config(seed):
    """A configuration with every size, count and constant, the number of layers and the loop drawn from what the design allows."""
    r = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(r.integers(len(xs)))]
    aligned = seed % 3 == 0                                # every third draw: sizes in whole 16-byte pieces

    def mlp():
        if r.random() < 0.25:
            return None
        groups = pick(1, 2, 3, 4)
        per = pick(1, 2, 4)
        keep = int(r.integers(1, groups + 1))
        return moe(ff=pick(32, 64, 96) if aligned else pick(8, 20, 33), experts=groups * per,
                   top=int(r.integers(1, min(keep * per, 6) + 1)), groups=groups, keep=keep, limit=pick(0.5, 2.0, 7.0))
    layers = []
    for _ in range(int(r.integers(1, 6))):
        kv = pick(1, 2, 3)
        heads = kv * pick(1, 2, 4)
        dim = pick(32, 64, 128) if aligned else pick(4, 10, 12, 20, 48)
        rot = pick(None, 0, 2, dim // 2 // 2 * 2, dim)
        layers.append(A(heads=heads, kv_heads=kv, dim=dim, vdim=pick(16, 64, 128) if aligned else pick(4, 10, 24, 40), rot_dims=rot,
                        base=pick(100.0, 10000.0, 5e5), scale=pick(None, 0.3, 0.05, 1.0 / dim), mlp=mlp()))
    loop = None
    if r.random() < 0.7:
        a = int(r.integers(0, len(layers)))
        b = int(r.integers(a + 1, len(layers) + 1))
        loop = (a, b, int(r.integers(1, 4)))
    width = pick(64, 128, 192) if aligned else pick(24, 36, 60, 72)
    cfg = plain.make_config(layers, vocab=pick(33, 97, 160, 301), width=width, eps=pick(1e-6, 1e-5, 1e-3),
                            groups=pick(*[g for g in (1, 2, 3, 4, 6) if width % g == 0]), mult=pick(0.5, 0.7, 1.0, 1.4), taps=pick(0, 1, 2, 3, 4, 5),
                            side=pick(0, 1, 3, 8, 16), bigram=pick(None, (1, 3, 5), (101, 31, 7), (509, 65537, 40503)), loop=loop)
    return cfg, pick(4, 8, 16, 32)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(12))
def test_configurations_drawn_at_random(tmp_path, seed, dtype):
    cfg, page = _random_config(seed)
    if dtype == "bfloat16" and (cfg.get("token_side") or {}).get("dim", 0) in (1, 3):
        # a side input of one number is a sign function of it (y / rms(y)), of three nearly one: 16-bit noise flips it
        cfg["token_side"]["dim"] = 8
    w = plain.random_weights(cfg, 100 + seed, expert_gain=GAIN)
    a, b = tokens_of(cfg, 83, seed), tokens_of(cfg, 47, 50 + seed)
    want_a, want_b = reference(w, cfg, a), reference(w, cfg, b)
    hs = Harness(tmp_path, cfg, w, dtype, page=page, pages=-(-256 // page), slots=2)
    close(hs.whole("w", a), want_a, dtype, f"seed {seed} whole")
    rows = hs.step([("a", a[:40], range(40))])
    rows.update(hs.step([("a", a[40:42], [0, 1]), ("b", b[:17], range(17))]))            # a portion of two beside a prompt
    rows.update(hs.step([("b", b[17:], range(30)), ("a", a[42:43], [0])], end=["b"]))    # a prompt's end beside one token
    rows.update(hs.step([("a", a[43:70], range(27))]))
    for i in range(70, 83):
        rows.update(hs.step([("a", a[i:i + 1], [0])]))
    close(np.stack([rows[("a", i)] for i in range(83)]), want_a, dtype, f"seed {seed} in portions and decoded")
    close(np.stack([rows[("b", i)] for i in range(47)]), want_b, dtype, f"seed {seed} the request beside it")
