"""Subivik without a GPU: configuration, model description, tensor names and shapes, cache and state needs, and the plain
implementation's own properties (what a chunk, a far key, a recurrence and the routing must and must not do)."""
import copy

import numpy as np
import pytest
import torch

import plain_subivik as plain
from tiny_inference_engine_b200.config import load_config, parse_subivik_config, subivik_spec
from tiny_inference_engine_b200.errors import LoadError, UnsupportedError
from tiny_inference_engine_b200.parts.model import Model, expected_tensors
from tiny_inference_engine_b200.weights.loader import SafetensorsSource, bind_check

A, P, moe = plain.attention_layer, plain.parallel_layer, plain.moe
CFG = plain.make_config([A(heads=6, kv_heads=3, dim=20, vdim=6, chunk=7, diff=0.8),
                         P(heads=3, kv_heads=1, dim=12, vdim=10, softcap=5.0, rheads=3, rdim=20, mlp=moe(ff=20, experts=6, top=3, scale=0.7)),
                         A(heads=6, kv_heads=3, dim=20, vdim=6, chunk=13, diff=0.1, kv_from=0, mlp=None),
                         A(heads=2, kv_heads=2, dim=6, vdim=66, chunk=50, mlp=plain.dense(50))], vocab=97, width=72, eps=1e-5)


def test_config_json_picks_the_architecture_and_every_size_comes_from_it(tmp_path):
    w = plain.random_weights(CFG, 1, decay_rank=3)
    plain.write_model_dir(tmp_path, CFG, w)
    arch, cfg, spec = load_config(tmp_path)
    assert arch.name == "Subivik" and spec.architecture == "Subivik"
    assert (spec.hidden_size, spec.vocab_size, len(spec.layers)) == (72, 97, 4)
    assert cfg.decay_ranks == {1: 3}                      # read from the checkpoint's shapes: config.json has no key for it
    model = Model(spec, torch.float32)
    needs = {n: t for n, t in model.needs().items() if not t.optional}
    assert {n: tuple(t.shape) for n, t in needs.items()} == {n: tuple(s) for n, s in plain.tensor_shapes(CFG, 3).items()}
    bind_check(model.needs(), SafetensorsSource(tmp_path), what="Subivik")
    assert [l.mixer.kind for l in spec.layers] == ["differential_attention", "mixer_sum", "differential_attention", "differential_attention"]
    assert [None if l.ffn is None else l.ffn.kind for l in spec.layers] == ["two_branch_mlp", "routed_experts", None, "two_branch_mlp"]
    assert all(l.mixer_norm.kind == "dynamic_tanh" for l in spec.layers) and spec.final_norm.kind == "dynamic_tanh"
    assert spec.head["tied"] and spec.embedding.kind == "sinusoid_token_embedding"
    # layer 2 reads the keys and values of layer 0: no cache of its own, and layer 0 keeps them as far back as layer 2 looks
    assert [(e.layer, e.cache_of) for e in spec.run_order] == [(0, None), (1, None), (2, 0), (3, None)]
    cache = model.cache_needs()
    assert cache[2] is None
    assert (cache[0].kind, cache[0].kv_heads, cache[0].head_dim, cache[0].window, cache[0].value_dim) == ("window", 3, 40, 13, 6)
    assert (cache[1].kind, cache[1].kv_heads, cache[1].head_dim, cache[1].value_dim) == ("full", 1, 12, 10)
    assert (cache[3].head_dim, cache[3].value_dim, cache[3].window) == (12, 66, 50)
    state = model.state_needs()
    assert state[0] is None and state[1].shape == (3 * 20 * 20 + 72,) and state[1].dtype == torch.float32


def test_cache_groups_by_shape():
    from tiny_inference_engine_b200.cache.manager import CacheManager
    model = Model(subivik_spec(parse_subivik_config(CFG)), torch.float32)
    cm = CacheManager(model.cache_needs(), 8, num_pages=10, dtype=torch.float32)
    assert [(g.kind, g.kv_heads, g.head_dim, g.window, g.value_dim, g.entries) for g in cm.groups] == \
        [("window", 3, 40, 13, 6, (0,)), ("full", 1, 12, 0, 10, (1,)), ("window", 2, 12, 50, 66, (3,))]


def test_a_reader_without_a_mask_keeps_the_owners_cache_whole():
    cfg = plain.make_config([A(chunk=10), A(kv_from=0, chunk=0)])
    model = Model(subivik_spec(parse_subivik_config(cfg)), torch.float32)
    assert model.cache_needs()[0].kind == "full"


def test_what_the_configuration_rejects():
    def broken(change):
        cfg = copy.deepcopy(CFG)
        change(cfg)
        return cfg
    with pytest.raises(UnsupportedError, match="type 'conv'"):
        parse_subivik_config(broken(lambda c: c["layers"][0].update(type="conv")))
    with pytest.raises(LoadError, match="kv_from"):
        parse_subivik_config(broken(lambda c: c["layers"][2]["mixer"].update(kv_from=3)))
    with pytest.raises(LoadError, match="kv_from"):
        parse_subivik_config(broken(lambda c: c["layers"][2]["mixer"].update(kv_from=1)))
    with pytest.raises(LoadError, match="differ"):
        parse_subivik_config(broken(lambda c: c["layers"][2]["mixer"].update(vdim=8)))
    with pytest.raises(LoadError, match="not a multiple"):
        parse_subivik_config(broken(lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=2)))
    with pytest.raises(LoadError, match="no 'diff'"):
        parse_subivik_config(broken(lambda c: c["layers"][0]["mixer"].pop("diff")))
    with pytest.raises(LoadError, match="cannot choose"):
        parse_subivik_config(broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=7)))
    with pytest.raises(UnsupportedError, match="kind 'glu'"):
        parse_subivik_config(broken(lambda c: c["layers"][0]["mlp"].update(kind="glu")))
    with pytest.raises(LoadError, match="no 'vocab'"):
        parse_subivik_config(broken(lambda c: c.pop("vocab")))


def test_random_weights_need_no_checkpoint():
    spec = subivik_spec(parse_subivik_config(CFG))
    assert expected_tensors(spec)["l1.mix.right.w1"].shape == (16, 72)        # the default inner size


def test_plain_chunks_far_keys_and_the_recurrence_see_what_they_should():
    r = np.random.default_rng(0)
    # attention alone, chunks of 5: a changed token moves the later rows of its own chunk and no other row
    cfg = plain.make_config([A(chunk=5, mlp=None), A(kv_from=0, chunk=5, mlp=None)], vocab=40, width=32)
    w = plain.random_weights(cfg, 2)
    toks = r.integers(0, 40, 23).tolist()
    other = list(toks)
    other[11] = (toks[11] + 1) % 40
    a, b = plain.forward(w, cfg, toks), plain.forward(w, cfg, other)
    moved = np.abs(a - b).max(axis=1) > 1e-9
    assert moved.tolist() == [i in range(11, 15) for i in range(23)]
    # the left mixer alone (the right one's factor zero): every later row moves, earlier rows do not
    cfg = plain.make_config([P(right_scale=0.0, mlp=None)], vocab=40, width=32)
    w = plain.random_weights(cfg, 3)
    a, b = plain.forward(w, cfg, toks), plain.forward(w, cfg, other)
    assert (np.abs(a - b).max(axis=1) > 1e-9).tolist() == [i >= 11 for i in range(23)]
    # the right mixer alone: the same through the state; and a prefix does not depend on what follows
    cfg = plain.make_config([P(left_scale=0.0, mlp=None)], vocab=40, width=32)
    w = plain.random_weights(cfg, 4)
    a, b = plain.forward(w, cfg, toks), plain.forward(w, cfg, other)
    assert (np.abs(a - b).max(axis=1) > 1e-9).tolist() == [i >= 11 for i in range(23)]
    assert np.abs(plain.forward(w, cfg, toks[:9]) - a[:9]).max() < 1e-9


def test_plain_mechanisms_by_hand():
    # the head mix with an identity matrix is plain attention; the bias takes r1 ln(1 + r2 d) off a score
    assert np.allclose(plain.distance_bias(3, 2.0, 0.5)[2], [2.0 * np.log(2.0), 2.0 * np.log(1.5), 0.0])
    assert plain.chunk_mask(5, 2).astype(int).tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [0, 0, 1, 0, 0], [0, 0, 1, 1, 0], [0, 0, 0, 0, 1]]
    # the recurrence: the first token reads nothing but its own write through the bonus; the second reads the first's write undecayed
    r, k, v = np.ones((2, 1, 2)), np.array([[[1.0, 2.0]], [[3.0, 4.0]]]), np.array([[[5.0, 6.0]], [[7.0, 8.0]]])
    o = plain.bonus_recurrence(r, k, v, np.full((2, 1, 2), 0.5), np.array([[10.0, 100.0]]))
    assert np.allclose(o[0, 0], (10.0 * 1.0 + 100.0 * 2.0) * v[0, 0])
    assert np.allclose(o[1, 0], (1.0 + 2.0) * v[0, 0] + (10.0 * 3.0 + 100.0 * 4.0) * v[1, 0])
    # both branches of the unit meet at zero with the slope one half
    z = np.array([-1e-6, 1e-6])
    assert np.allclose(plain.two_branch_unit(z, 0.3, -0.2) / z, 0.5, atol=1e-5)
    assert plain.route(np.array([0.1, 0.4, 0.4, 0.05]), 2) == [1, 2]
    s = plain.sinusoid([0, 3], 6)
    assert np.allclose(s[0], [0, 1, 0, 1, 0, 1]) and np.isclose(s[1, 2], np.sin(3 * 10000.0 ** (-2 / 6)))


def test_a_random_model_folder_from_a_configuration(tmp_path):
    from tiny_inference_engine_b200.cli.main import main
    cfg_path = tmp_path / "c.json"
    import json
    cfg_path.write_text(json.dumps(CFG))
    out = tmp_path / "m"
    assert main(["make-random", "--config", str(cfg_path), "--out", str(out), "--seed", "3", "--device", "cpu"]) == 0
    arch, cfg, spec = load_config(out)
    assert arch.name == "Subivik" and cfg.decay_ranks == {1: 16}
    bind_check(Model(spec, torch.float32).needs(), SafetensorsSource(out), what="Subivik")
