"""Lufatar: a decoder whose layers run their mixer and their feed-forward side by side on one stream.

  embedding   x = embed[token] + bigram[row], row = (previous token * mul_prev + token * mul_cur) mod buckets, the table's
              last row for a sequence's first token (`embedding.bigram`; without it the plain token table);
  layer       x += m * (mixer(in1(norm1 x)) + ff(in2(norm2 x))), m = `residual_mult`; the norms are RMS norms over
              `norm.groups` equal parts of a row; in(h) = h + a causal convolution of `canon.taps` taps over time per channel
              (`l<i>.canon1`, `l<i>.canon2`; without `canon`, in(h) = h); then, with `token_side`, a token input of the
              layer: g = gelu_tanh(side.gate x) * side.embed[token][i * dim : (i + 1) * dim], y = side.proj g,
              x += m * y / rms(y) * side.norm;
  attention   grouped-query heads with keys of `dim` and values of `vdim`; neighbouring pairs of the first `rot.dims`
              dimensions rotated by position * base^(-2i / dims); q and k divided by their root mean square per head; scores
              times `scale`, mixed across heads by `talk` [heads, heads]; a softmax with one more key of score 0 and no value;
  moe         sigmoid router; choice by score + `correction` inside the `groups.keep` best of `groups.count` blocks of
              neighbours (a block counts as the sum of its two best choice scores); the weights are the chosen scores as
              they are; experts g = min(gate h, limit), u = clamp(up h, +-limit), down(g * sigmoid(1.702 g) * (u + 1));
  loop        layers start .. stop-1 run `times` times in a row with the same weights, each pass with a cache and a
              state of its own; ahead of pass t the vector `loop.step`[t] joins every row of the stream.

config.json:

    {"architecture": "Lufatar", "vocab": V, "width": D, "residual_mult": m, "norm": {"eps": e, "groups": n},
     "canon": {"taps": k}, "token_side": {"dim": s}, "embedding": {"bigram": {"buckets", "mul_prev", "mul_cur"}},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "rot": {"base", "dims"}},
                 "mlp": {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top", "groups": {"count", "keep"}}} | null}]}

Tensors: `embed`, `bigram`, `side.embed` [V, layers * s], `loop.step` [times, D], `final.norm`, `head`, and per layer i
`l<i>.norm1|norm2`, `l<i>.canon1|canon2` [D, taps], `l<i>.mix.q|k|v|o|talk`, `l<i>.mlp.router|correction|e<j>.gate|up|down`,
`l<i>.side.gate|proj|norm`.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..errors import LoadError, UnsupportedError
from .registry import Architecture, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

# Constants that the design fixes.
EXPERT_SLOPE = 1.702       # an expert's unit: y = g * sigmoid(EXPERT_SLOPE * g) * (u + EXPERT_UP_SHIFT)
EXPERT_UP_SHIFT = 1.0
GROUP_SCORE_MEMBERS = 2    # a block of experts counts as the sum of this many of its best choice scores
DEFAULT_MAX_POSITIONS = 1 << 17
MIXERS = ("attention",)
MAX_TAPS = 8


@dataclass
class LufatarConfig:
    vocab: int
    width: int
    eps: float
    norm_groups: int
    residual_mult: float
    taps: int                                         # 0: sublayers read the norm's output as it is
    side_dim: int                                     # 0: no token input per layer
    bigram: dict | None                               # {"buckets", "mul_prev", "mul_cur"} or None
    layers: list = field(default_factory=list)        # the configuration's own dictionaries, validated
    loop: dict | None = None                          # {"start", "stop", "times"} or None
    max_positions: int = DEFAULT_MAX_POSITIONS

    def to_dict(self) -> dict:
        d = {"architecture": "Lufatar", "layers": self.layers, "norm": {"eps": self.eps, "groups": self.norm_groups},
             "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.taps:
            d["canon"] = {"taps": self.taps}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.bigram is not None:
            d["embedding"] = {"bigram": dict(self.bigram)}
        if self.loop is not None:
            d["loop"] = dict(self.loop)
        return d

    def run_layers(self) -> tuple[list[int], dict[int, int]]:
        """(layer index of every run entry in order, {entry at which a pass of the loop starts: number of the pass})."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n)), {}
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        order, starts = list(range(a)), {}
        for t in range(times):
            starts[len(order)] = t
            order += list(range(a, b))
        return order + list(range(b, n)), starts


def _req(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise LoadError(f"config.json: {where} has no '{key}'")
    return d[key]


def _int(v, what: str, least: int = 1) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v < least:
        raise LoadError(f"config.json: {what} must be an integer of at least {least}, got {v!r}")
    return v


def _check_attention(mx: dict, where: str) -> None:
    w = where + "'s mixer"
    heads, kv = _int(_req(mx, "heads", w), f"{where} mixer.heads"), _int(_req(mx, "kv_heads", w), f"{where} mixer.kv_heads")
    dim = _int(_req(mx, "dim", w), f"{where} mixer.dim")
    _int(_req(mx, "vdim", w), f"{where} mixer.vdim")
    if heads % kv:
        raise LoadError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv heads")
    if dim % 2:
        raise LoadError(f"config.json: {where}: heads of {dim} cannot be rotated in pairs")
    float(_req(mx, "scale", w))
    rot = mx.get("rot")
    if rot is not None:
        dims = _int(_req(rot, "dims", where + "'s rot"), f"{where} rot.dims", 0)
        if dims % 2 or dims > dim:
            raise LoadError(f"config.json: {where}: rot.dims {dims} must be even and at most dim {dim}")
        if dims and not float(_req(rot, "base", where + "'s rot")) > 0:
            raise LoadError(f"config.json: {where}: rot.base must be positive")


def _check_mlp(mlp, where: str) -> None:
    if mlp is None:
        return
    w = where + "'s mlp"
    kind = _req(mlp, "kind", w)
    if kind != "moe":
        raise UnsupportedError(f"config.json: {where} has a feed-forward of kind '{kind}' (supported: moe, or null for none)")
    ex, r = _req(mlp, "expert", w), _req(mlp, "router", w)
    _int(_req(ex, "ff", w + " expert"), f"{where} mlp.expert.ff")
    float(_req(ex, "limit", w + " expert"))
    E = _int(_req(r, "experts", w + " router"), f"{where} mlp.router.experts")
    top = _int(_req(r, "top", w + " router"), f"{where} mlp.router.top")
    g = r.get("groups") or {"count": 1, "keep": 1}
    count = _int(_req(g, "count", w + " router groups"), f"{where} mlp.router.groups.count")
    keep = _int(_req(g, "keep", w + " router groups"), f"{where} mlp.router.groups.keep")
    if E % count or keep > count or top > keep * (E // count):
        raise LoadError(f"config.json: {where}: cannot choose {top} of {E} experts in {count} groups of which {keep} are kept")


def parse_lufatar_config(j: dict) -> LufatarConfig:
    top = "the configuration"
    layers = _req(j, "layers", top)
    if not isinstance(layers, list) or not layers:
        raise LoadError("config.json: 'layers' must be a non-empty list")
    for i, layer in enumerate(layers):
        where = f"layer {i}"
        kind = _req(layer, "type", where)
        if kind not in MIXERS:
            raise UnsupportedError(f"config.json: {where} has type '{kind}' (supported: {', '.join(MIXERS)})")
        _check_attention(_req(layer, "mixer", where), where)
        _check_mlp(layer.get("mlp"), where)
    width = _int(_req(j, "width", top), "width")
    norm = _req(j, "norm", top)
    groups = _int(norm.get("groups", 1), "norm.groups")
    if width % groups:
        raise LoadError(f"config.json: a width of {width} does not split into {groups} equal norm groups")
    loop = j.get("loop")
    if loop is not None:
        a, b, times = (_req(loop, k, "'loop'") for k in ("start", "stop", "times"))
        if not all(isinstance(v, int) and not isinstance(v, bool) for v in (a, b, times)) or not 0 <= a < b <= len(layers) or times < 1:
            raise LoadError(f"config.json: loop start={a!r} stop={b!r} times={times!r} does not name layers of this model")
        loop = {"start": a, "stop": b, "times": times}
    canon = j.get("canon")
    taps = _int(_req(canon, "taps", "'canon'"), "canon.taps", 0) if canon is not None else 0
    if taps > MAX_TAPS:
        raise UnsupportedError(f"config.json: canon.taps {taps} is more than the {MAX_TAPS} taps that the input convolution takes")
    side = j.get("token_side")
    side_dim = _int(_req(side, "dim", "'token_side'"), "token_side.dim", 0) if side is not None else 0
    bigram = (j.get("embedding") or {}).get("bigram")
    if bigram is not None:
        bigram = {"buckets": _int(_req(bigram, "buckets", "'embedding.bigram'"), "embedding.bigram.buckets"),
                  "mul_prev": _int(_req(bigram, "mul_prev", "'embedding.bigram'"), "embedding.bigram.mul_prev", 0),
                  "mul_cur": _int(_req(bigram, "mul_cur", "'embedding.bigram'"), "embedding.bigram.mul_cur", 0)}
    return LufatarConfig(vocab=_int(_req(j, "vocab", top), "vocab"), width=width, eps=float(_req(norm, "eps", "'norm'")),
                         norm_groups=groups, residual_mult=float(j.get("residual_mult", 1.0)), taps=taps, side_dim=side_dim,
                         bigram=bigram, layers=layers, loop=loop, max_positions=int(j.get("max_positions", DEFAULT_MAX_POSITIONS)))


def lufatar_spec(c: LufatarConfig) -> ModelSpec:
    D, n_layers = c.width, len(c.layers)

    def norm(name: str) -> PartSpec:
        return PartSpec("grouped_rmsnorm", {"name": name, "size": D, "eps": c.eps, "groups": c.norm_groups})

    layers = []
    for i, layer in enumerate(c.layers):
        p, mx = f"l{i}.", layer["mixer"]
        rot = mx.get("rot") or {}
        dims = int(rot.get("dims", 0))
        mixer = PartSpec("head_mix_attention", {
            "prefix": p + "mix.", "hidden_size": D, "num_heads": mx["heads"], "num_kv_heads": mx["kv_heads"], "head_dim": mx["dim"],
            "value_dim": mx["vdim"], "scale": float(mx["scale"]), "eps": c.eps, "unit_qk": True, "head_mix": True, "sink": True,
            "position": PartSpec("rope", {"theta": float(rot["base"]), "head_dim": mx["dim"], "rotary_dim": dims}) if dims else None})
        mlp = layer.get("mlp")
        ffn = None
        if mlp is not None:
            r = mlp["router"]
            g = r.get("groups") or {"count": 1, "keep": 1}
            ffn = PartSpec("routed_experts", {
                "prefix": p + "mlp.", "hidden_size": D, "intermediate_size": mlp["expert"]["ff"], "num_experts": r["experts"],
                "top": r["top"], "group_count": g["count"], "group_keep": g["keep"], "group_top": GROUP_SCORE_MEMBERS,
                "score": "sigmoid", "correction": True, "renorm": False, "limit": float(mlp["expert"]["limit"]),
                "slope": EXPERT_SLOPE, "up_shift": EXPERT_UP_SHIFT})
        side = None
        if c.side_dim:
            side = {"table": "side.embed", "vocab_size": c.vocab, "table_width": n_layers * c.side_dim, "index": i, "dim": c.side_dim,
                    "gate": "side.gate", "proj": "side.proj", "norm": "side.norm", "eps": c.eps}
        block = PartSpec("parallel", {"hidden_size": D, "residual_mult": c.residual_mult, "taps": c.taps,
                                      "conv_names": ("canon1", "canon2"), "side": side})
        layers.append(LayerSpec(prefix=p, block=block, mixer=mixer, mixer_norm=norm(p + "norm1"), ffn=ffn,
                                ffn_norm=norm(p + "norm2")))
    order, starts = c.run_layers()
    passes = c.loop["times"] if c.loop is not None else 0
    run_order = tuple(RunEntry(l, before=PartSpec("pass_vector", {"name": "loop.step", "index": starts[i], "passes": passes,
                                                                  "hidden_size": D}) if i in starts else None)
                      for i, l in enumerate(order))
    table = {"name": "embed", "vocab_size": c.vocab, "hidden_size": D}
    if c.bigram is not None:
        embedding = PartSpec("pair_hash_embedding", {**table, "pairs": {"name": "bigram", **c.bigram}})
    else:
        embedding = PartSpec("token_embedding", table)
    return ModelSpec(architecture="Lufatar", hidden_size=D, vocab_size=c.vocab, max_positions=c.max_positions, embedding=embedding,
                     layers=tuple(layers), run_order=run_order, final_norm=norm("final.norm"),
                     head=PartSpec("lm_head", {"name": "head", "tied": False, "vocab_size": c.vocab, "hidden_size": D}))


register_architecture(Architecture(name="Lufatar", parse_config=parse_lufatar_config, build_spec=lufatar_spec,
                                   model_types=("lufatar",)), replace=True)
