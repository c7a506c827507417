"""Subivik through the engine against the plain implementation (tests/plain_subivik.py): each mechanism alone, prompts
whole and token by token, portions down to two tokens, mixed batches, pages and state slots that are used again, keys
at a chunk's edge, at page borders and far back, a state that remembers hundreds of tokens, the first tokens of a
sequence, long decoding, sizes of several kinds, greedy generation through the engine's own entry point and scheduler."""
import numpy as np
import pytest
import torch

import plain_subivik as plain
from conftest import assert_logits_close, rel_err

pytestmark = pytest.mark.gpu

A, P, moe = plain.attention_layer, plain.parallel_layer, plain.moe

MIXED = plain.make_config([A(), P(mlp=moe()), P(), A(kv_from=0, chunk=40, mlp=moe(ff=40, experts=5, top=3, scale=0.7)), P(mlp=None)])
ODD = plain.make_config([P(heads=3, kv_heads=1, dim=12, vdim=10, softcap=5.0, rheads=3, rdim=20, mlp=moe(ff=20, experts=6, top=3, scale=2.0)),
                         A(heads=6, kv_heads=3, dim=20, vdim=6, chunk=7, diff=0.8, mlp=None),
                         A(heads=2, kv_heads=2, dim=6, vdim=66, chunk=50, scale=0.31, mlp=plain.dense(50)),
                         A(heads=6, kv_heads=3, dim=20, vdim=6, chunk=13, diff=0.05, kv_from=1),
                         P(heads=6, kv_heads=3, dim=10, vdim=14, softcap=None, rheads=1, rdim=36, left_scale=1.0, right_scale=0.3, mlp=None)],
                        vocab=97, width=36, eps=1e-5)
ONES = plain.make_config([A(heads=1, kv_heads=1, dim=8, vdim=8, chunk=1, mlp=moe(ff=8, experts=2, top=1, scale=1.0)),
                          P(heads=1, kv_heads=1, dim=8, vdim=8, rheads=1, rdim=8, left_scale=1.0, right_scale=1.0),
                          A(heads=1, kv_heads=1, dim=8, vdim=8, chunk=1000, mlp=None)], vocab=33, width=16)
# sizes in whole 16-byte pieces and larger heads
SQUARE = plain.make_config([A(heads=8, kv_heads=2, dim=64, vdim=64, chunk=48, mlp=moe(ff=64, experts=8, top=2)),
                            P(heads=8, kv_heads=4, dim=32, vdim=32, rheads=2, rdim=64, mlp=moe(ff=32, experts=12, top=3, scale=0.5)),
                            A(heads=8, kv_heads=2, dim=64, vdim=64, chunk=64, kv_from=0),
                            P(heads=16, kv_heads=2, dim=64, vdim=128, rheads=4, rdim=32)], width=128)
# What the experts of the whole-model tests add to the stream is scaled down: among hundreds of random routing decisions
# some are close calls that bfloat16 rounding decides the other way; at this gain such a flip stays within the bfloat16
# tolerance. The experts at full gain are held to float32 accuracy by `test_each_mechanism_alone`.
GAIN = 0.1
CONFIGS = {"mixed": (MIXED, 8, 16), "odd": (ODD, 3, 8), "ones": (ONES, 1, 4), "square": (SQUARE, 16, 16)}


class Want:
    def __init__(self, rows, noise):
        self.rows, self.noise = np.asarray(rows), noise

    def __getitem__(self, idx):
        return Want(self.rows[idx], self.noise)


def reference(w, cfg, toks):
    exact = plain.forward(w, cfg, toks)
    with plain.bfloat16_activations():
        rounded = plain.forward(w, cfg, toks)
    return Want(exact, rel_err(rounded, exact))


def close(got, want, dtype, what):
    """float32: 1e-4 of the row's largest logit and the same argmax. bfloat16: four times the noise of 16-bit activations
    on this very model and prompt, and at least 2e-2."""
    if dtype == "float32":
        assert_logits_close(got, want.rows, dtype, what)
    else:
        err, tol = rel_err(got, want.rows), max(2e-2, 4.0 * want.noise)
        assert err <= tol, f"{what}: relative error {err:.3e} above {tol:.1e} (bfloat16; noise of rounding {want.noise:.1e})"


class Harness:
    """A model folder, the engine's model, cache, state slots and step function; `step` takes
    [(request id, tokens, wanted places)] and returns {(id, position): logits}."""

    def __init__(self, tmp, cfg, weights, dtype, page=16, pages=64, slots=4, max_tokens=512):
        from tiny_inference_engine_b200 import StepRunner, load_model, make_cache
        plain.write_model_dir(tmp, cfg, weights)
        self.model = load_model(tmp, dtype)
        self.cache, self.states = make_cache(self.model, page_size=page, num_pages=pages, max_requests=slots)
        self.runner = StepRunner(self.model, self.cache, max_tokens=max_tokens, max_seqs=8, max_logit_rows=max_tokens, states=self.states)
        self.live = {}

    def step(self, entries, end=()):
        from tiny_inference_engine_b200 import StepEntry
        batch, keys = [], []
        for rid, tokens, want in entries:
            if rid not in self.live:
                self.live[rid] = [self.cache.new_request(), 0]
            req, have = self.live[rid]
            assert self.cache.reserve(req, have + len(tokens)), "pool too small for the test"
            batch.append(StepEntry(req, list(tokens), have, list(want)))
            keys += [(rid, have + w) for w in want]
        logits = self.runner.run(batch)
        for (rid, tokens, _), e in zip(entries, batch):
            self.live[rid][1] += len(tokens)
            self.cache.advance_window(e.cache, self.live[rid][1])
        out = {}
        if logits is not None:
            host = logits.float().cpu().numpy()
            out = {k: host[i] for i, k in enumerate(keys)}
        torch.cuda.synchronize()
        self.runner.check()
        for rid in end:
            self.cache.release(self.live.pop(rid)[0])
        return out

    def whole(self, rid, tokens):
        got = self.step([(rid, tokens, range(len(tokens)))], end=[rid])
        return np.stack([got[(rid, i)] for i in range(len(tokens))])

    def in_portions(self, rid, tokens, sizes):
        rows, at, i = {}, 0, 0
        while at < len(tokens):
            n = min(sizes[i % len(sizes)], len(tokens) - at)
            rows.update(self.step([(rid, tokens[at:at + n], range(n))]))
            at, i = at + n, i + 1
        self.cache.release(self.live.pop(rid)[0])
        return np.stack([rows[(rid, j)] for j in range(len(tokens))])


def tokens_of(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


@pytest.fixture(scope="module")
def truth():
    memo = {}

    def get(name, toks):
        cfg, rank, _ = CONFIGS[name]
        key = (name, tuple(toks))
        if key not in memo:
            memo[key] = reference(plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN), cfg, toks)
        return memo[key]
    return get


# ---------------------------------------------------------------------------------------------- each mechanism alone

SINGLE = {
    "differential": plain.make_config([A(mlp=None)], vocab=60, width=48),
    "differential_no_chunks_many_heads": plain.make_config([A(heads=12, kv_heads=3, dim=8, vdim=20, chunk=0, diff=0.9, mlp=None)], vocab=60, width=40),
    "borrowed_keys_and_values": plain.make_config([A(chunk=9, mlp=None), A(kv_from=0, chunk=30, diff=0.55, mlp=None)], vocab=60, width=48),
    "talking_heads": plain.make_config([P(right_scale=0.0, mlp=None)], vocab=60, width=48),
    "talking_heads_one_kv_head_no_cap": plain.make_config([P(heads=5, kv_heads=1, dim=24, vdim=12, softcap=None, right_scale=0.0, mlp=None)], vocab=60, width=40),
    "talking_heads_a_kv_head_each": plain.make_config([P(heads=3, kv_heads=3, dim=10, vdim=34, softcap=2.0, right_scale=0.0, mlp=None)], vocab=60, width=40),
    "talking_heads_value_rows_of_1200": plain.make_config([P(heads=6, kv_heads=3, dim=8, vdim=400, right_scale=0.0, mlp=None)], vocab=60, width=40),
    "recurrence": plain.make_config([P(left_scale=0.0, mlp=None)], vocab=60, width=48),
    "recurrence_large_heads": plain.make_config([P(left_scale=0.0, rheads=1, rdim=80, mlp=None), P(left_scale=0.0, rheads=5, rdim=6, mlp=None)], vocab=60, width=40),
    "both_halves": plain.make_config([P(mlp=None)], vocab=60, width=48),
    "dense": plain.make_config([A(mlp=plain.dense(56))], vocab=60, width=48),
    "experts": plain.make_config([A(mlp=moe(ff=20, experts=7, top=3, scale=2.5))], vocab=60, width=48),
    "experts_all_chosen": plain.make_config([P(mlp=moe(ff=12, experts=3, top=3, scale=0.4))], vocab=60, width=40),
    "odd_width": plain.make_config([A(heads=2, kv_heads=1, dim=6, vdim=5, chunk=11, mlp=plain.dense(19)), P(heads=2, kv_heads=2, dim=6, vdim=5, rheads=3, rdim=7, mlp=moe(ff=9, experts=3, top=2))],
                                   vocab=51, width=38, eps=1e-3),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SINGLE))
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = SINGLE[name]
    w = plain.random_weights(cfg, 3, decay_rank=4)
    toks = tokens_of(cfg, 61, 1)
    got = Harness(tmp_path, cfg, w, dtype).whole("a", toks)
    close(got, reference(w, cfg, toks), dtype, name)


# ---------------------------------------------------------------------------------------------- whole models

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_decoding_and_portions(tmp_path, truth, name, dtype):
    """The same logits at every position whether the prompt comes whole, token by token from the first token on (a token
    before the first that is all zeros, states that start empty), or in portions of several sizes down to two."""
    cfg, rank, page = CONFIGS[name]
    w = plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN)
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "square"])
def test_mixed_batches_on_a_small_pool_with_two_state_slots(tmp_path, truth, name, dtype):
    """Requests of unequal lengths, portions of some beside single tokens of others, never more than two alive: pages and
    state slots are given back and used again, a request sits out a step now and then, and every row equals the request run alone."""
    cfg, rank, page = CONFIGS[name]
    w = plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN)
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
            if len(alive) == 2 and k == 1 and turn % 5 == 4:
                continue                                   # left out of this step, goes on later
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


# ---------------------------------------------------------------------------------------------- edges that random weights would hide

def _one_token_stands_out(w, cfg, marked, quiet):
    """The first norm becomes tanh(x). In the last even column of the width (whose sinusoid is a tiny sine) only token
    `marked` has an entry, and in the last odd column (a cosine near one) no token has any: after the norm the first is near
    one for the marked token and near zero for the others, the second is the same number, about 0.76, for everybody.
    Returns the two columns. `quiet` scales the embedding of every other column."""
    width = cfg["width"]
    mark, const = width - 2, width - 1
    emb = w["embed"].astype(np.float64) * quiet
    emb[:, mark] = 0.0
    emb[:, const] = 0.0
    emb[marked, mark] = 3.0
    w["embed"] = plain.round_bf16(emb)
    w["l0.norm1"][:] = 1.0
    w["l0.norm1.b"][:] = 0.0
    w["l0.norm1.alpha"] = np.float32(1.0)
    return mark, const


def _peaked_differential(chunk, at, n, dim=16, vdim=24, heads=4, kv_heads=2):
    """One differential attention layer in which, in the first map of every head, the key of the token at place `at`
    outweighs all other keys of its chunk together for every later query."""
    cfg = plain.make_config([A(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, chunk=chunk, diff=0.4, scale=1.0, mlp=None)], vocab=40, width=32)
    w = plain.random_weights(cfg, 8, sharp=1.0)
    marked = 7
    mark, const = _one_token_stands_out(w, cfg, marked, 0.3)
    p = "l0.mix."
    w[p + "q"] = plain.round_bf16(w[p + "q"] * 0.05)
    w[p + "k"] = plain.round_bf16(w[p + "k"] * 0.6)
    for g in range(kv_heads):
        w[p + "k"][g * 2 * dim] = 0.0
        w[p + "k"][g * 2 * dim, mark] = 6.0          # dimension 0 of map 1: the marked token only
    for h in range(heads):
        w[p + "q"][h * 2 * dim] = 0.0
        w[p + "q"][h * 2 * dim, const] = 4.0         # the same large query entry for every token
    w[p + "q.norm"][:] = 1.0
    w[p + "k.norm"][:] = 1.0
    w[p + "v"] = plain.round_bf16(w[p + "v"] * 4.0)
    toks = [t if t != marked else marked + 1 for t in tokens_of(cfg, n, 4)]
    toks[at] = marked
    other = list(toks)
    other[at] = marked + 2
    return cfg, w, toks, other


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("geometry", [(16, 24, 4, 2, 8), (64, 64, 2, 1, 16), (40, 72, 6, 2, 4)])
def test_a_key_just_inside_and_just_outside_a_chunk(tmp_path, dtype, geometry):
    """A key that dominates the first map while it is seen sits on a chunk's first place, which is a page's first slot too:
    the rows of its chunk differ visibly from the same rows without it, the last row of the chunk before and the first row
    of the chunk after do not see it. Whole, in portions cut at both edges and inside the chunk, and token by token."""
    dim, vdim, heads, kv_heads, page = geometry
    chunk, at = 32, 64
    cfg, w, toks, other = _peaked_differential(chunk, at, 130, dim, vdim, heads, kv_heads)
    ref, moved = reference(w, cfg, toks), plain.forward(w, cfg, other)
    inside, outside = list(range(at + 1, at + chunk)), list(range(0, at)) + list(range(at + chunk, 130))
    assert rel_err(moved[inside], ref.rows[inside]) > 0.15 and rel_err(moved[outside], ref.rows[outside]) < 1e-9
    hs = Harness(tmp_path, cfg, w, dtype, page=page, pages=4 * 160 // page)
    close(hs.whole("w", toks), ref, dtype, "whole")
    close(hs.in_portions("a", toks, [at, chunk, 34]), ref, dtype, "cut at the chunk's edges")
    close(hs.in_portions("b", toks, [at - 1, 2, chunk - 2, 2, 33]), ref, dtype, "two tokens across each edge")
    close(hs.in_portions("c", toks, [at + chunk - 1, 1, 1, 29]), ref, dtype, "the chunk's last row and the next chunk's first row alone")
    rows = hs.step([("d", toks[:at - 3], range(at - 3))])
    for i in range(at - 3, 130):
        rows.update(hs.step([("d", toks[i:i + 1], [0])]))
    hs.cache.release(hs.live.pop("d")[0])
    close(np.stack([rows[("d", i)] for i in range(130)]), ref, dtype, "decoded across the chunk")
    # the same key in the chunk's last place: only that very row sees it
    cfg, w, toks, other = _peaked_differential(chunk, at + chunk - 1, 130, dim, vdim, heads, kv_heads)
    ref = reference(w, cfg, toks)
    close(hs_whole(tmp_path / "z", cfg, w, dtype, page, toks), ref, dtype, "key in a chunk's last place")


def hs_whole(tmp, cfg, w, dtype, page, toks):
    return Harness(tmp, cfg, w, dtype, page=page, pages=4 * 160 // page).whole("w", toks)


def _far_key(n, at, dim=16, vdim=8, heads=4, kv_heads=2):
    """One parallel layer whose right half is switched off and in whose left half the key of the token at place `at`
    outweighs all other keys for every later query of every head, the distance bias and the cap notwithstanding."""
    cfg = plain.make_config([P(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, softcap=30.0, scale=1.0, right_scale=0.0, mlp=None)], vocab=40, width=32)
    w = plain.random_weights(cfg, 9, sharp=1.0)
    marked = 7
    mark, const = _one_token_stands_out(w, cfg, marked, 0.3)
    p = "l0.mix.left."
    w[p + "q"] = plain.round_bf16(w[p + "q"] * 0.3)
    for g in range(kv_heads):
        w[p + "k"][g * dim] = 0.0
        w[p + "k"][g * dim, mark] = 4.0
    for h in range(heads):
        w[p + "q"][h * dim] = 0.0
        w[p + "q"][h * dim, const] = 6.0
    w[p + "r1"][:] = plain.round_bf16(np.linspace(0.3, 1.0, heads))
    w[p + "r2"][:] = plain.round_bf16(np.linspace(2.0, 0.2, heads))
    w[p + "v"] = plain.round_bf16(w[p + "v"] * 4.0)
    toks = [t if t != marked else marked + 1 for t in tokens_of(cfg, n, 6)]
    toks[at] = marked
    other = list(toks)
    other[at] = marked + 2
    return cfg, w, toks, other


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("geometry", [(16, 8, 4, 2, 16, 15), (64, 64, 8, 2, 8, 16), (24, 40, 3, 3, 4, 3)])
def test_a_key_far_back_among_hundreds(tmp_path, dtype, geometry):
    """Every head's weights are mixed into every head: one key several hundred places back, on a page's border, carries the rows
    after it. In a prompt, in portions, and decoded through the splits of the single-row kernel."""
    dim, vdim, heads, kv_heads, page, at = geometry
    n = 420
    cfg, w, toks, other = _far_key(n, at, dim, vdim, heads, kv_heads)
    ref, moved = reference(w, cfg, toks), plain.forward(w, cfg, other)
    assert rel_err(moved[-20:], ref.rows[-20:]) > 0.15 and rel_err(moved[:at], ref.rows[:at]) < 1e-9
    hs = Harness(tmp_path, cfg, w, dtype, page=page, pages=2 * 448 // page)
    close(hs.whole("w", toks), ref, dtype, "whole")
    rows = hs.step([("d", toks[:at + 1], range(at + 1))])
    rows.update(hs.step([("d", toks[at + 1:300], range(299 - at))]))
    for i in range(300, n):
        rows.update(hs.step([("d", toks[i:i + 1], [0])]))
    hs.cache.release(hs.live.pop("d")[0])
    close(np.stack([rows[("d", i)] for i in range(n)]), ref, dtype, "portions, then decoded")


def _far_memory():
    """One parallel layer whose left half is switched off and whose decays are close to one: what the first tokens wrote
    into the state still decides the last rows."""
    cfg = plain.make_config([P(left_scale=0.0, rheads=2, rdim=24, mlp=None)], vocab=40, width=32)
    w = plain.random_weights(cfg, 11)
    p = "l0.mix.right."
    w[p + "w0"][:] = -7.0
    w[p + "w2"] = plain.round_bf16(w[p + "w2"] * 0.2)
    w[p + "u"][:] = 0.0
    marked = 7
    mark, const = _one_token_stands_out(w, cfg, marked, 0.3)
    w[p + "mu.k"][:] = 0.0
    w[p + "mu.v"][:] = 0.0
    w[p + "k"] = plain.round_bf16(w[p + "k"] * 0.1)      # the other tokens write little
    for h in range(2):
        w[p + "k"][h * 24] = 0.0
        w[p + "k"][h * 24, mark] = 8.0              # key channel 0 of both heads: the marked token only
        w[p + "r"][h * 24] = 0.0
        w[p + "r"][h * 24, const] = 4.0             # every token reads that channel
    w[p + "o"] = plain.round_bf16(w[p + "o"] * 3.0)
    toks = [t if t != marked else marked + 1 for t in tokens_of(cfg, 400, 12)]
    toks[3] = marked
    other = list(toks)
    other[3] = marked + 2
    return cfg, w, toks, other


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_state_remembers_a_token_hundreds_back(tmp_path, dtype):
    """The state is carried through a prompt portion, through another, and through decoding, and a second request in
    another slot in between does not touch it."""
    cfg, w, toks, other = _far_memory()
    want, moved = reference(w, cfg, toks), plain.forward(w, cfg, other)
    assert rel_err(moved[-5:], want.rows[-5:]) > 5e-2      # a token 396 back is still felt
    hs = Harness(tmp_path, cfg, w, dtype, pages=64, max_tokens=512)
    close(hs.whole("w", toks), want, dtype, "whole")
    rows = hs.step([("a", toks[:130], range(130))])
    rows.update(hs.step([("x", other[:77], [])]))                       # another request takes another slot
    rows.update(hs.step([("a", toks[130:300], range(170)), ("x", other[77:78], [])]))
    for i in range(300, 400):
        rows.update(hs.step([("a", toks[i:i + 1], [0])] + ([("x", other[78 + i - 300:79 + i - 300], [])] if i % 2 else [])))
    close(np.stack([rows[("a", i)] for i in range(400)]), want, dtype, "portions, then decoding beside another request")


def test_the_token_before_comes_from_the_slot_at_a_portions_start(tmp_path):
    """Blends that take the token before whole (mu = 1): a portion's first row must read the last row of the portion
    before, from the request's slot, and a sequence's first row zeros, also in a slot that another request has just left."""
    cfg = plain.make_config([P(left_scale=0.0, mlp=None)], vocab=40, width=32)
    w = plain.random_weights(cfg, 13)
    for s in "rkvgw":
        w["l0.mix.right.mu." + s][:] = 1.0
    a, b = tokens_of(cfg, 40, 1), tokens_of(cfg, 25, 2)
    hs = Harness(tmp_path, cfg, w, "float32", slots=1)
    close(hs.in_portions("a", a, [7, 1, 2, 13]), reference(w, cfg, a), "float32", "first request")
    close(hs.in_portions("b", b, [1, 5]), reference(w, cfg, b), "float32", "second request in the same slot")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps_and_slots_used_again(tmp_path, truth, dtype):
    """Three requests decode together for 200 steps (steps of one token each are captured as graphs and replayed), end at
    different times, and a fourth takes over a slot and pages that were just given back."""
    cfg, rank, page = CONFIGS["mixed"]
    w = plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN)
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
    from tiny_inference_engine_b200 import SamplingParams, ServingConfig, load_engine
    cfg, rank, page = CONFIGS["mixed"]
    w = plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN)
    plain.write_model_dir(tmp_path, cfg, w)
    prompts = [tokens_of(cfg, n, 30 + i) for i, n in enumerate([19, 3, 41, 1, 27])]
    want = [plain.generate(w, cfg, p, 24) for p in prompts]
    engine = load_engine(tmp_path, dtype="float32", num_pages=40, page_size=page, serving=ServingConfig(max_seqs=3, max_tokens_per_step=16))
    assert engine.generate(prompts[0], SamplingParams(max_tokens=24)) == want[0]
    assert engine.generate_batch(prompts, SamplingParams(max_tokens=24)) == want
    tight = load_engine(tmp_path, dtype="float32", num_pages=9, page_size=page, serving=ServingConfig(max_seqs=3, max_tokens_per_step=16))
    assert tight.generate_batch(prompts, SamplingParams(max_tokens=24)) == want


def test_the_command_line_generates_the_plain_greedy_tokens(tmp_path, capsys):
    from tiny_inference_engine_b200.cli.main import main
    cfg, rank, page = CONFIGS["odd"]
    w = plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN)
    plain.write_model_dir(tmp_path, cfg, w)
    prompt = tokens_of(cfg, 21, 77)
    assert main(["generate", "-m", str(tmp_path), "-p", " ".join(map(str, prompt)), "--temp", "0", "--max-tokens", "12",
                 "--dtype", "float32", "--kv-mem", "64M", "--max-tokens-per-step", "8", "--max-seqs", "2"]) == 0
    assert [int(t) for t in capsys.readouterr().out.split()] == plain.generate(w, cfg, prompt, 12)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_a_subivik_model(tmp_path, truth, dtype):
    from test_replay_gpu import Replay
    cfg, rank, page = CONFIGS["odd"]
    w = plain.random_weights(cfg, 5, decay_rank=rank, expert_gain=GAIN)
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
        close(got, Want(np.stack([want[2].rows[1], want[0].rows[50], want[3].rows[0], want[3].rows[1]]), noise), dtype, "three requests, one step")
        assert rp.step([("e", reqs[4][:80], [])]) is None
        got = rp.step([("e", reqs[4][80:], [0]), ("a", reqs[0][51:], range(49)), ("c", reqs[2][2:], [61])], end=["a", "c", "e"]).reshape(51, V)
        close(got, Want(np.concatenate([want[4].rows[80:81], want[0].rows[51:], want[2].rows[63:64]]), noise), dtype, "the rest")
    finally:
        rp.close()


# ---------------------------------------------------------------------------------------------- sizes drawn at random

def _random_config(seed):
    """A configuration with every size, count, constant and the order of layers drawn from what the design allows."""
    r = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(r.integers(len(xs)))]

    def mlp():
        kind = pick("none", "dense", "moe", "moe")
        if kind == "none":
            return None
        if kind == "dense":
            return plain.dense(pick(24, 50, 64))
        experts = pick(1, 2, 5, 8, 12)
        return moe(ff=pick(8, 20, 32), experts=experts, top=int(r.integers(1, min(experts, 6) + 1)), scale=pick(0.5, 1.0, 2.5))
    aligned = seed % 3 == 0                                # every third draw: sizes in whole 16-byte pieces
    layers, owners = [], []
    for i in range(int(r.integers(2, 6))):
        if pick("attention", "parallel") == "attention":
            if owners and r.random() < 0.4:
                src = owners[int(r.integers(len(owners)))]
                mx = layers[src]["mixer"]
                layers.append(A(heads=mx["heads"], kv_heads=mx["kv_heads"], dim=mx["dim"], vdim=mx["vdim"], chunk=pick(1, 3, 16, 33, 64, 400),
                                diff=pick(0.1, 0.5, 0.9), scale=pick(None, 0.2), kv_from=src, mlp=mlp()))
                continue
            kv = pick(1, 2, 3)
            layers.append(A(heads=kv * pick(1, 2, 4), kv_heads=kv, dim=pick(32, 64) if aligned else pick(4, 10, 20, 48), vdim=pick(16, 64) if aligned else pick(4, 10, 40, 96),
                            chunk=pick(1, 2, 5, 16, 33, 64, 400), diff=pick(0.1, 0.5, 0.9), scale=pick(None, 0.2, 0.05), mlp=mlp()))
            owners.append(i)
        else:
            kv = pick(1, 2, 4)
            layers.append(P(heads=kv * pick(1, 2, 3), kv_heads=kv, dim=pick(32, 64) if aligned else pick(4, 12, 20, 40), vdim=pick(16, 32) if aligned else pick(4, 10, 36),
                            softcap=pick(None, 3.0, 50.0), scale=pick(None, 0.3), rheads=pick(1, 2, 3), rdim=pick(16, 64) if aligned else pick(4, 12, 40, 72),
                            left_scale=pick(0.5, 1.0), right_scale=pick(0.4, 1.3), mlp=mlp()))
    cfg = plain.make_config(layers, vocab=pick(33, 97, 160, 301), width=pick(24, 36, 64, 72, 128), eps=pick(1e-6, 1e-5, 1e-3))
    return cfg, pick(1, 3, 8, 24), pick(4, 8, 16, 32)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(12))
def test_configurations_drawn_at_random(tmp_path, seed, dtype):
    cfg, rank, page = _random_config(seed)
    w = plain.random_weights(cfg, 100 + seed, decay_rank=rank, expert_gain=GAIN)
    a, b = tokens_of(cfg, 83, seed), tokens_of(cfg, 31, 50 + seed)
    want_a, want_b = reference(w, cfg, a), reference(w, cfg, b)
    hs = Harness(tmp_path, cfg, w, dtype, page=page, pages=2 * 128 // page, slots=2)
    close(hs.whole("w", a), want_a, dtype, f"seed {seed} whole")
    rows = hs.step([("a", a[:29], range(29)), ("b", b[:2], range(2))])
    rows.update(hs.step([("a", a[29:31], range(2)), ("b", b[2:], range(29))], end=["b"]))
    rows.update(hs.step([("a", a[31:70], range(39))]))
    for i in range(70, 83):
        rows.update(hs.step([("a", a[i:i + 1], [0])]))
    close(np.stack([rows[("a", i)] for i in range(83)]), want_a, dtype, f"seed {seed} in portions beside another request, then decoded")
    close(np.stack([rows[("b", i)] for i in range(31)]), want_b, dtype, f"seed {seed} the other request")


# ---------------------------------------------------------------------------------------------- kernels alone

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_norm_adds_scaled_sums_and_partial_sums_in_float(dtype):
    from tiny_inference_engine_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(1)
    T, D = 37, 50
    x = torch.randn(T, D, device="cuda", generator=g)
    a = torch.randn(T, D, device="cuda", generator=g).to(dtype)
    part = torch.randn(3, T, D, device="cuda", generator=g)
    w, b = torch.randn(D, device="cuda", generator=g), torch.randn(D, device="cuda", generator=g)
    want_x = x.double() + 0.6 * a.double() + 0.9 * part.double().sum(0)
    want = torch.tanh(0.7 * want_x) * w.double() + b.double()
    out = torch.empty(T, D, device="cuda", dtype=dtype)
    x1 = x.clone()
    ops.add_tanh_norm(x1, ops.ScaledSum([(a, 0.6), (ops.SplitSum(part.reshape(-1), 3, T, D), 0.9)]), 0.7, w, b, out)
    assert (x1.double() - want_x).abs().max() < 1e-5
    assert (out.double() - want).abs().max() < (1e-5 if dtype == torch.float32 else 4e-2)
    rows = torch.tensor([5, 0, 36], device="cuda", dtype=torch.int32)
    x2, some = x.clone(), torch.empty(3, D, device="cuda", dtype=dtype)
    ops.add_tanh_norm(x2, a, 0.7, w, b, some, rows=rows)
    assert torch.equal(x2, x)            # with rows the stream stays as it is
    want_rows = torch.tanh(0.7 * (x.double() + a.double()))[rows.long()] * w.double() + b.double()
    assert (some.double() - want_rows).abs().max() < (1e-5 if dtype == torch.float32 else 4e-2)


def test_the_sinusoid_keeps_its_precision_at_large_positions():
    from tiny_inference_engine_b200 import ops
    pos = torch.tensor([0, 1, 777, 100000], device="cuda", dtype=torch.int32)
    x = torch.zeros(4, 10, device="cuda")
    ops.sinusoid_add(x, pos)
    assert np.abs(x.cpu().numpy() - plain.sinusoid(pos.cpu().numpy(), 10)).max() < 1e-6
