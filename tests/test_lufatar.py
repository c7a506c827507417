"""Lufatar without a GPU: configuration, model description, run order, tensor names and shapes, cache and state needs,
and the plain implementation's own properties (what the pair table, the input convolution, the sink, the head mix and
the routing must and must not do)."""
import copy

import numpy as np
import pytest
import torch

import plain_lufatar as plain
from tiny_inference_engine_b200.config import load_config, lufatar_spec, parse_lufatar_config
from tiny_inference_engine_b200.errors import LoadError, UnsupportedError
from tiny_inference_engine_b200.parts.model import Model, expected_tensors
from tiny_inference_engine_b200.weights.loader import SafetensorsSource, bind_check

A, moe = plain.attention_layer, plain.moe
CFG = plain.make_config([A(heads=3, kv_heads=1, dim=10, vdim=7, rot_dims=4, mlp=moe(ff=20, experts=6, top=3, groups=3, keep=2)),
                         A(heads=6, kv_heads=3, dim=12, vdim=20, rot_dims=12, scale=0.5, mlp=None),
                         A(heads=2, kv_heads=2, dim=8, vdim=8, rot_dims=None),
                         A(heads=6, kv_heads=3, dim=12, vdim=20, rot_dims=0, mlp=moe(ff=11, experts=9, top=4, groups=3, keep=3))],
                        vocab=97, width=72, eps=1e-5, groups=3, mult=1.3, taps=3, side=5, bigram=(7, 1000003, 99991), loop=(1, 3, 2))


def test_config_json_picks_the_architecture_and_every_size_comes_from_it(tmp_path):
    w = plain.random_weights(CFG, 1)
    plain.write_model_dir(tmp_path, CFG, w)
    arch, cfg, spec = load_config(tmp_path)
    assert arch.name == "Lufatar" and spec.architecture == "Lufatar"
    assert (spec.hidden_size, spec.vocab_size, len(spec.layers)) == (72, 97, 4)
    assert (cfg.taps, cfg.side_dim, cfg.norm_groups, cfg.residual_mult, cfg.bigram["mul_prev"]) == (3, 5, 3, 1.3, 1000003)
    model = Model(spec, torch.float32)
    needs = {n: t for n, t in model.needs().items() if not t.optional}
    assert {n: tuple(t.shape) for n, t in needs.items()} == {n: tuple(s) for n, s in plain.tensor_shapes(CFG).items()}
    bind_check(model.needs(), SafetensorsSource(tmp_path), what="Lufatar")
    assert all(l.block.kind == "parallel" and l.mixer.kind == "head_mix_attention" for l in spec.layers)
    assert [None if l.ffn is None else l.ffn.kind for l in spec.layers] == ["routed_experts", None, "routed_experts", "routed_experts"]
    assert spec.embedding.kind == "pair_hash_embedding" and spec.final_norm.kind == "grouped_rmsnorm"
    # layers 1 and 2 run twice; each pass starts with its own row of the pass vectors; every entry has a cache and a ring of its own
    assert [(e.layer, e.before["index"] if e.before is not None else None) for e in spec.run_order] == \
        [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    cache = model.cache_needs()
    assert [(c.kind, c.kv_heads, c.head_dim, c.value_dim) for c in cache] == \
        [("full", 1, 10, 7), ("full", 3, 12, 20), ("full", 2, 8, 0), ("full", 3, 12, 20), ("full", 2, 8, 0), ("full", 3, 12, 20)]
    state = model.state_needs()
    assert all(s.shape == (2, 72) and s.dtype == torch.float32 for s in state)         # taps - 1 rows of the stream's width
    extra = model.extra_state_needs()
    assert list(extra) == ["embedding"] and extra["embedding"].dtype == torch.int32 and extra["embedding"].shape == ()
    # the rotation: none for layers 2 and 3; the side input of layer i reads columns [5 i, 5 i + 5) of one table
    assert [l.mixer["position"] is not None for l in spec.layers] == [True, True, False, False]
    assert [l.block["side"]["index"] for l in spec.layers] == [0, 1, 2, 3] and tuple(needs["side.embed"].shape) == (97, 20)


def test_optional_mechanisms_can_be_left_out():
    cfg = plain.make_config([A(), A(mlp=None)], groups=1, taps=0, side=0, bigram=None)
    spec = lufatar_spec(parse_lufatar_config(cfg))
    names = expected_tensors(spec)
    assert spec.embedding.kind == "token_embedding" and [(e.layer, e.before) for e in spec.run_order] == [(0, None), (1, None)]
    assert not any(n.startswith(("bigram", "side.", "loop.")) or ".canon" in n or ".side." in n for n in names)
    model = Model(spec, torch.float32)
    assert model.state_needs() == [None, None] and model.extra_state_needs() == {}
    one_tap = Model(lufatar_spec(parse_lufatar_config(plain.make_config([A()], taps=1))), torch.float32)
    assert one_tap.state_needs() == [None] and tuple(one_tap.needs()["l0.canon1"].shape) == (64, 1)
    # a layer without a feed-forward needs no second norm or convolution, and takes a checkpoint that has them
    assert names["l1.norm2"].optional and not names["l0.norm2"].optional


def test_what_the_configuration_rejects():
    def broken(change):
        c = copy.deepcopy(CFG)
        change(c)
        return c
    with pytest.raises(UnsupportedError, match="type 'conv'"):
        parse_lufatar_config(broken(lambda c: c["layers"][0].update(type="conv")))
    with pytest.raises(UnsupportedError, match="kind 'dense'"):
        parse_lufatar_config(broken(lambda c: c["layers"][0]["mlp"].update(kind="dense")))
    with pytest.raises(LoadError, match="no 'norm'"):
        parse_lufatar_config(broken(lambda c: c.pop("norm")))
    with pytest.raises(LoadError, match="not a multiple"):
        parse_lufatar_config(broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=2)))
    with pytest.raises(LoadError, match="rot.dims"):
        parse_lufatar_config(broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=12)))
    with pytest.raises(LoadError, match="cannot choose"):
        parse_lufatar_config(broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=5)))
    with pytest.raises(LoadError, match="loop"):
        parse_lufatar_config(broken(lambda c: c["loop"].update(stop=9)))
    with pytest.raises(LoadError, match="norm groups"):
        parse_lufatar_config(broken(lambda c: c["norm"].update(groups=7)))
    with pytest.raises(UnsupportedError, match="taps"):
        parse_lufatar_config(broken(lambda c: c["canon"].update(taps=40)))
    with pytest.raises(LoadError, match="buckets"):
        parse_lufatar_config(broken(lambda c: c["embedding"]["bigram"].update(buckets=0)))


def test_plain_causality_and_what_a_changed_token_reaches():
    toks = np.random.default_rng(0).integers(0, 97, 30).tolist()
    moved = list(toks)
    moved[10] = (toks[10] + 1) % 97
    w = plain.random_weights(CFG, 2)
    base, other = plain.forward(w, CFG, toks), plain.forward(w, CFG, moved)
    assert np.allclose(other[:10], base[:10]) and all(np.abs(other[i] - base[i]).max() > 1e-9 for i in range(10, 30))
    assert np.allclose(plain.forward(w, CFG, toks[:12]), base[:12])                  # a prefix does not depend on what follows
    # without attention's reach (a first token seen alone) the pair table and the convolutions still carry the token before
    assert plain.bigram_rows([5, 9, 9], 7, 3, 2).tolist() == [7, (15 + 18) % 7, (27 + 18) % 7]
    h = np.random.default_rng(1).standard_normal((6, 4))
    taps = np.random.default_rng(2).standard_normal((4, 3))
    out = plain.causal_taps(h, taps)
    assert np.allclose(out[0], taps[:, 2] * h[0]) and np.allclose(out[1], taps[:, 2] * h[1] + taps[:, 1] * h[0])
    assert np.allclose(out[5], taps[:, 2] * h[5] + taps[:, 1] * h[4] + taps[:, 0] * h[3])


def test_plain_sink_and_head_mix():
    r = np.random.default_rng(4)
    q, k, v = r.standard_normal((9, 4, 6)), r.standard_normal((9, 2, 6)), np.ones((9, 2, 3))
    out = plain.attend(q, k, v, np.eye(4), 0.4)
    assert (out < 1.0).all() and np.allclose(out[:, :, 0], out[:, :, 1])             # the sink keeps part of every row's weight
    first = 1.0 / (1.0 + np.exp(-0.4 * np.einsum("hd,hd->h", q[0], np.repeat(k[0], 2, axis=0))))
    assert np.allclose(out[0, :, 0], first)                                         # one key and the sink: a sigmoid of the score
    swap = np.eye(4)[[1, 0, 3, 2]]                                                  # heads 0/1 and 2/3 share a key head: swapped scores, same values
    assert np.allclose(plain.attend(q, k, v, swap, 0.4)[:, [1, 0, 3, 2]], out)
    assert not np.allclose(plain.attend(q, k, v, np.eye(4) + 0.3, 0.4), out)


def test_plain_routing_keeps_to_the_best_groups_and_weighs_without_the_correction():
    r = np.random.default_rng(3)
    for _ in range(50):
        z, corr = r.standard_normal((1, 12)) * 2, r.standard_normal(12) - 1.0
        ids, weights = plain.route(z, corr, top=3, group_count=4, group_keep=2)
        s = plain.sigmoid(z[0])
        choice = s + corr
        gscore = np.sort(choice.reshape(4, 3), axis=1)[:, -2:].sum(axis=1)
        best = np.argsort(-gscore)[:2]
        assert all(i // 3 in best for i in ids[0]) and len(set(ids[0].tolist())) == 3
        allowed = sorted((choice[i] for i in range(12) if i // 3 in best), reverse=True)
        assert np.allclose(sorted(choice[ids[0]], reverse=True), allowed[:3]) and np.allclose(weights[0], s[ids[0]])
    ids, _ = plain.route(np.array([[0.4, 0.1, 0.3, 0.2]]), np.zeros(4), top=2, group_count=1, group_keep=1)
    assert ids[0].tolist() == [0, 2]                           # one group: the plain top-k


def test_a_random_model_folder_from_a_configuration(tmp_path):
    """`tie make-random` writes config.json and weights of every tensor the description names; the folder loads back."""
    import json
    from tiny_inference_engine_b200.cli.main import main
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    assert main(["make-random", "-o", str(tmp_path / "m"), "--config", str(tmp_path / "config.json"), "--seed", "3"]) == 0
    arch, cfg, spec = load_config(tmp_path / "m")
    assert arch.name == "Lufatar"
    bind_check(Model(spec, torch.float32).needs(), SafetensorsSource(tmp_path / "m"), what="Lufatar")
