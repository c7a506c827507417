"""Subivik: a decoder whose configuration lists its layers in any order. A layer is a mixer behind a norm and, unless its
`mlp` is null, a feed-forward behind a norm, both added to the residual stream. Every norm is a dynamic tanh
(tanh(alpha x) * w + b: no statistics). The token embedding gets a sinusoid of the position added, and the output table is
the embedding table. Mixers:

  attention   differential attention (two score maps a head over the same values, a1 - lambda a2, a norm per head, a sigmoid
              output gate) with RMS-normed queries and keys, in chunks of `mask.size` positions counted from position 0;
              `kv_from: j` makes the layer read the keys and values that layer j keeps instead of projecting its own;
  parallel    two mixers side by side on the same input, `left_scale * left + right_scale * right`: left, causal
              grouped-query attention with capped scores, a bias that grows with the logarithm of the distance and softmax
              weights mixed across heads; right, a recurrence with a matrix state per head that blends its inputs with the
              token before and reads the state before it writes it.

Feed-forwards: `dense` (one hidden layer, an activation in two branches with two learned numbers) and `moe` (softmax router,
the `top` best experts, weights = scores times `router.scale`, gated experts with silu). config.json:

    {"architecture": "Subivik", "vocab": V, "width": D, "norm": {"eps": e},
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "diff", "mask": {"size"}, "kv_from"?}, "mlp": ...},
                {"type": "parallel", "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap"},
                                               "right": {"heads", "dim"}, "left_scale", "right_scale"}, "mlp": ...}],
     with "mlp": {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale"}} | null}

Tensors: `embed`, `final.norm` (+ `.b`, `.alpha`), and per layer i `l<i>.norm1|norm2` (+ `.b`, `.alpha`), `l<i>.mix.*`,
`l<i>.mlp.*`. The inner size of a right mixer's two-step decay projection (w1/w2) is not in config.json: it is read from
the checkpoint's tensor shapes, or given to `parse_subivik_config`.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..errors import LoadError, UnsupportedError
from .registry import Architecture, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

# Constants that the design fixes.
SINUSOID_BASE = 10000.0
DEFAULT_DECAY_RANK = 16    # inner size of a right mixer's w1/w2 when no checkpoint says (random weights)
DEFAULT_MAX_POSITIONS = 1 << 17
MIXERS = ("attention", "parallel")


@dataclass
class SubivikConfig:
    vocab: int
    width: int
    eps: float
    layers: list = field(default_factory=list)        # the configuration's own dictionaries, validated
    decay_ranks: dict = field(default_factory=dict)   # layer index -> inner size of the right mixer's decay projection
    max_positions: int = DEFAULT_MAX_POSITIONS

    def to_dict(self) -> dict:
        return {"architecture": "Subivik", "layers": self.layers, "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}


def _req(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise LoadError(f"config.json: {where} has no '{key}'")
    return d[key]


def _positive_int(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise LoadError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


def _check_heads(mx: dict, where: str, keys) -> None:
    for key in keys:
        _positive_int(_req(mx, key, where), f"{where}.{key}")
    if "kv_heads" in keys and mx["heads"] % mx["kv_heads"]:
        raise LoadError(f"config.json: {where}: {mx['heads']} heads are not a multiple of {mx['kv_heads']} kv heads")


def _check_mixer(kind: str, mx: dict, i: int, layers: list) -> None:
    where = f"layer {i}'s mixer"
    if kind == "attention":
        _check_heads(mx, where, ("heads", "kv_heads", "dim", "vdim"))
        _req(mx, "scale", where)
        _req(mx, "diff", where)
        if mx.get("mask") is not None:
            _positive_int(_req(mx["mask"], "size", where + "'s mask"), f"{where} mask.size")
        src = mx.get("kv_from")
        if src is not None:
            if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < i or layers[src].get("type") != "attention" or \
                    layers[src]["mixer"].get("kv_from") is not None:
                raise LoadError(f"config.json: {where}: kv_from {src!r} must name an earlier attention layer with keys and values of its own")
            other = layers[src]["mixer"]
            if any(other.get(k) != mx.get(k) for k in ("kv_heads", "dim", "vdim")):
                raise LoadError(f"config.json: {where}: kv_from {src}: the two layers' kv_heads, dim and vdim differ")
    else:
        left, right = _req(mx, "left", where), _req(mx, "right", where)
        _check_heads(left, where + " left", ("heads", "kv_heads", "dim", "vdim"))
        _req(left, "scale", where + " left")
        _check_heads(right, where + " right", ("heads", "dim"))
        _req(mx, "left_scale", where)
        _req(mx, "right_scale", where)


def _check_mlp(mlp, where: str) -> None:
    if mlp is None:
        return
    w = where + "'s mlp"
    kind = _req(mlp, "kind", w)
    if kind == "dense":
        _positive_int(_req(mlp, "ff", w), f"{where} mlp.ff")
    elif kind == "moe":
        ex, r = _req(mlp, "expert", w), _req(mlp, "router", w)
        _positive_int(_req(ex, "ff", w + " expert"), f"{where} mlp.expert.ff")
        E = _positive_int(_req(r, "experts", w + " router"), f"{where} mlp.router.experts")
        top = _positive_int(_req(r, "top", w + " router"), f"{where} mlp.router.top")
        if top > E:
            raise LoadError(f"config.json: {where}: cannot choose {top} of {E} experts")
    else:
        raise UnsupportedError(f"config.json: {where} has a feed-forward of kind '{kind}' (supported: dense, moe)")


def parse_subivik_config(j: dict, decay_ranks: dict | None = None) -> SubivikConfig:
    layers = _req(j, "layers", "the configuration")
    if not isinstance(layers, list) or not layers:
        raise LoadError("config.json: 'layers' must be a non-empty list")
    for i, layer in enumerate(layers):
        where = f"layer {i}"
        kind = _req(layer, "type", where)
        if kind not in MIXERS:
            raise UnsupportedError(f"config.json: {where} has type '{kind}' (supported: {', '.join(MIXERS)})")
        _check_mixer(kind, _req(layer, "mixer", where), i, layers)
        _check_mlp(layer.get("mlp"), where)
    return SubivikConfig(vocab=_positive_int(_req(j, "vocab", "the configuration"), "vocab"),
                         width=_positive_int(_req(j, "width", "the configuration"), "width"),
                         eps=float(_req(_req(j, "norm", "the configuration"), "eps", "'norm'")), layers=layers,
                         decay_ranks=dict(decay_ranks or {}), max_positions=int(j.get("max_positions", DEFAULT_MAX_POSITIONS)))


def decay_ranks_from_shapes(shapes: dict) -> dict:
    """layer index -> rows of `l<i>.mix.right.w1` from a checkpoint's tensor shapes."""
    out = {}
    for name, shape in shapes.items():
        parts = name.split(".")
        if len(parts) == 4 and parts[1:] == ["mix", "right", "w1"] and parts[0][:1] == "l" and parts[0][1:].isdigit():
            out[int(parts[0][1:])] = int(shape[0])
    return out


def subivik_spec(c: SubivikConfig) -> ModelSpec:
    D = c.width

    def norm(name: str) -> PartSpec:
        return PartSpec("dynamic_tanh", {"name": name, "size": D})

    def chunk_of(mx) -> int:
        return int((mx.get("mask") or {}).get("size") or 0)

    # the cache of a layer that others read is kept as far back as the longest chunk among its readers (all of it if one has none)
    spans = {}
    for i, layer in enumerate(c.layers):
        if layer["type"] == "attention":
            owner = layer["mixer"].get("kv_from", i)
            owner = i if owner is None else owner
            spans.setdefault(owner, []).append(chunk_of(layer["mixer"]))
    layers, run_order = [], []
    for i, layer in enumerate(c.layers):
        p, mx, kind = f"l{i}.", layer["mixer"], layer["type"]
        if kind == "attention":
            mixer = PartSpec("differential_attention", {
                "prefix": p + "mix.", "hidden_size": D, "num_heads": mx["heads"], "num_kv_heads": mx["kv_heads"], "head_dim": mx["dim"],
                "value_dim": mx["vdim"], "scale": float(mx["scale"]), "diff": float(mx["diff"]), "eps": c.eps,
                "chunk": chunk_of(mx), "output_gate": True, "own_kv": mx.get("kv_from") is None,
                "cache_span": 0 if min(spans.get(i, [0])) == 0 else max(spans[i])})
            run_order.append(RunEntry(i, cache_of=mx.get("kv_from")))       # no layer runs twice: entry j is layer j
        else:
            lf, rt = mx["left"], mx["right"]
            left = PartSpec("talking_heads_attention", {
                "prefix": p + "mix.left.", "hidden_size": D, "num_heads": lf["heads"], "num_kv_heads": lf["kv_heads"], "head_dim": lf["dim"],
                "value_dim": lf["vdim"], "scale": float(lf["scale"]), "softcap": float(lf.get("softcap") or 0.0), "distance_bias": True,
                "head_mix": True})
            rank = c.decay_ranks.get(i, c.decay_ranks.get(str(i), DEFAULT_DECAY_RANK))
            right = PartSpec("token_shift_recurrence", {
                "prefix": p + "mix.right.", "hidden_size": D, "num_heads": rt["heads"], "head_dim": rt["dim"], "decay_rank": int(rank), "eps": c.eps})
            mixer = PartSpec("mixer_sum", {"parts": [(left, float(mx["left_scale"])), (right, float(mx["right_scale"]))]})
            run_order.append(RunEntry(i))
        mlp = layer.get("mlp")
        if mlp is None:
            ffn = None
        elif mlp["kind"] == "dense":
            ffn = PartSpec("two_branch_mlp", {"prefix": p + "mlp.", "hidden_size": D, "intermediate_size": mlp["ff"]})
        else:
            r = mlp["router"]
            ffn = PartSpec("routed_experts", {
                "prefix": p + "mlp.", "hidden_size": D, "intermediate_size": mlp["expert"]["ff"], "num_experts": r["experts"], "top": r["top"],
                "limit": None, "slope": 1.0, "up_shift": 0.0, "renorm": False, "weight_scale": float(r.get("scale", 1.0))})
        layers.append(LayerSpec(prefix=p, block=PartSpec("prenorm", {}), mixer=mixer, mixer_norm=norm(p + "norm1"), ffn=ffn,
                                ffn_norm=None if ffn is None else norm(p + "norm2")))
    return ModelSpec(architecture="Subivik", hidden_size=D, vocab_size=c.vocab, max_positions=c.max_positions,
                     embedding=PartSpec("sinusoid_token_embedding", {"name": "embed", "vocab_size": c.vocab, "hidden_size": D,
                                                                     "base": SINUSOID_BASE}),
                     layers=tuple(layers), run_order=tuple(run_order), final_norm=norm("final.norm"),
                     head=PartSpec("lm_head", {"name": "embed.head", "tied": True, "vocab_size": c.vocab, "hidden_size": D}))


register_architecture(Architecture(name="Subivik", parse_config=parse_subivik_config, build_spec=subivik_spec,
                                   model_types=("subivik",), shapes_to_config=decay_ranks_from_shapes), replace=True)
