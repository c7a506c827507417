"""A plain, slow Lufatar in numpy: whole sequences, no cache, no state carried between calls, one function per
mechanism. Arithmetic is float64 on the stored values. Nothing here imports the engine package: the tests compare
the two.

A Lufatar model lists its layers; a span of them may run several times in a row (`loop`), and ahead of every pass
one learned vector per pass joins the stream. The embedding of a token is the sum of its own row and of a row that
the pair (previous token, token) picks from a hashed table. A layer reads the stream once through two grouped RMS
norms, lets each reading pass a short causal convolution over time that is added to it, runs attention on one and a
feed-forward of routed experts on the other, adds both to the stream with one factor, and then adds a normed
projection of a gated per-layer token embedding. Attention: grouped-query, keys and values of different sizes,
interleaved rotation of the first dimensions, unit-RMS queries and keys, scores mixed across heads before the
softmax, and a softmax whose denominator counts one key more that has score 0 and no value.
"""
from __future__ import annotations

import numpy as np

from plain_misudra import round_bf16, write_model_dir, write_safetensors  # noqa: F401  (file writers and rounding only)

EXPERT_SLOPE = 1.702


def f64(a):
    return np.asarray(a, dtype=np.float64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


_act = None


class bfloat16_activations:
    """Within this context the outputs of `linear`, of the norms and of the convolutions are rounded to bfloat16: the
    noise that a pipeline with 16-bit activations cannot avoid, against which its tolerance is measured."""

    def __enter__(self):
        global _act
        _act = lambda y: round_bf16(y).astype(np.float64)

    def __exit__(self, *exc):
        global _act
        _act = None


def kept(y):
    return y if _act is None else _act(y)


def linear(x, w):
    return kept(f64(x) @ f64(w).T)


def unit_rms(x, eps):
    x = f64(x)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


# --------------------------------------------------------------------------- embedding

def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for every position: the last row for a sequence's first token."""
    rows = [buckets]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((int(prev) * mul_prev + int(cur) * mul_cur) % buckets)
    return np.array(rows[:len(tokens)], dtype=np.int64)


def embed(w, cfg, tokens):
    x = f64(w["embed"])[np.asarray(tokens)]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = x + f64(w["bigram"])[bigram_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"])]
    return x


# --------------------------------------------------------------------------- norm, convolution, token side input

def grouped_norm(x, weight, groups, eps):
    """Each of `groups` equal consecutive parts of a row divided by its own root mean square; the whole times `weight`."""
    x = f64(x)
    T, D = x.shape
    parts = x.reshape(T, groups, D // groups)
    return (unit_rms(parts, eps).reshape(T, D)) * f64(weight)


def causal_taps(h, taps_w):
    """out[t] = sum_j taps_w[:, j] * h[t - taps + 1 + j], zeros ahead of the sequence."""
    h, taps_w = f64(h), f64(taps_w)
    T, taps = h.shape[0], taps_w.shape[1]
    out = np.zeros_like(h)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += taps_w[:, j] * h[:T - back]
    return out


def sublayer_input(x, norm_w, taps_w, groups, eps):
    h = grouped_norm(x, norm_w, groups, eps)
    return kept(h if taps_w is None else h + causal_taps(h, taps_w))


def token_side(x, tokens, w, p, index, dim, eps):
    """The normed projection of a gated slice of the per-layer token table (before the layer's factor)."""
    e = f64(w["side.embed"])[np.asarray(tokens), index * dim:(index + 1) * dim]
    g = gelu_tanh(linear(x, w[p + "side.gate"])) * e
    y = f64(g) @ f64(w[p + "side.proj"]).T
    return unit_rms(y, eps) * f64(w[p + "side.norm"])


# --------------------------------------------------------------------------- attention

def rotate_pairs(x, positions, dims, base):
    """x [T, heads, dim]: dimension 2i is turned with 2i+1 by position * base^(-2i/dims), i < dims/2; the rest stays."""
    x = f64(x).copy()
    if dims == 0:
        return x
    i = np.arange(dims // 2)
    angle = f64(positions)[:, None] * base ** (-2.0 * i / dims)
    c, s = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    a, b = x[..., 0:dims:2].copy(), x[..., 1:dims:2].copy()
    x[..., 0:dims:2] = a * c - b * s
    x[..., 1:dims:2] = b * c + a * s
    return x


def sink_softmax(scores):
    """Causal softmax over the last axis of [H, T, T] with one more key of score 0 in the denominator."""
    H, T, _ = scores.shape
    mask = np.tril(np.ones((T, T), dtype=bool))
    s = np.where(mask, scores, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), 0.0)
    e = np.exp(s - m)
    return e / (np.exp(-m) + e.sum(axis=-1, keepdims=True))


def attention_mixer(h, w, p, mx, eps, positions):
    T = h.shape[0]
    H, G, dim, vdim = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    rot = mx.get("rot") or {"dims": 0, "base": 1.0}
    q = linear(h, w[p + "q"]).reshape(T, H, dim)
    k = linear(h, w[p + "k"]).reshape(T, G, dim)
    v = linear(h, w[p + "v"]).reshape(T, G, vdim)
    q = kept(unit_rms(rotate_pairs(q, positions, rot["dims"], rot["base"]), eps))
    k = kept(unit_rms(rotate_pairs(k, positions, rot["dims"], rot["base"]), eps))
    out = attend(q, k, v, w[p + "talk"], mx["scale"])
    return linear(kept(out.reshape(T, H * vdim)), w[p + "o"])


def attend(q, k, v, talk, scale):
    """q [T, H, dim], k [T, G, dim], v [T, G, vdim] of one sequence -> [T, H, vdim]: scaled scores of every query head against
    its key head, mixed across heads by `talk` [H, H], causal softmax with the sink, weighted values."""
    q, k, v = f64(q), f64(k), f64(v)
    H, per = q.shape[1], q.shape[1] // k.shape[1]
    raw = np.stack([q[:, hd] @ k[:, hd // per].T for hd in range(H)]) * scale                 # [H, T, T]
    mixed = np.einsum("hg,gij->hij", f64(talk), raw)
    weights = sink_softmax(mixed)
    return np.stack([weights[hd] @ v[:, hd // per] for hd in range(H)], axis=1)


# --------------------------------------------------------------------------- experts

def route(z, correction, top, group_count, group_keep):
    """z [T, E] router logits -> (chosen [T, top], weights [T, top]). Choice scores are sigmoid(z) + correction; a
    group's score is the sum of its two largest choice scores; experts outside the best groups cannot be chosen;
    weights are the chosen experts' sigmoid(z), as they are."""
    s = sigmoid(f64(z))
    choice = s + f64(correction)
    T, E = s.shape
    per = E // group_count
    grouped = np.sort(choice.reshape(T, group_count, per), axis=-1)
    gscore = grouped[..., -2:].sum(axis=-1)
    chosen = np.zeros((T, top), dtype=np.int64)
    weights = np.zeros((T, top))
    for t in range(T):
        keep = np.argsort(-gscore[t], kind="stable")[:group_keep]
        allowed = np.full(E, -np.inf)
        for g in keep:
            allowed[g * per:(g + 1) * per] = choice[t, g * per:(g + 1) * per]
        chosen[t] = np.argsort(-allowed, kind="stable")[:top]
        weights[t] = s[t, chosen[t]]
    return chosen, weights


def clamped_expert(h, gate, up, down, limit):
    g = np.minimum(linear(h, gate), limit)
    u = np.clip(linear(h, up), -limit, limit)
    return f64(kept(g * sigmoid(EXPERT_SLOPE * g) * (u + 1.0))) @ f64(down).T


def moe_mlp(h, w, p, mlp, chosen_out=None):
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    z = f64(h) @ f64(w[p + "router"]).T
    chosen, weights = route(z, w[p + "correction"], r["top"], groups["count"], groups["keep"])
    if chosen_out is not None:
        chosen_out.append(chosen)
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            out[t] += wt * clamped_expert(h[t:t + 1], w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"],
                                          mlp["expert"]["limit"])[0]
    return out


# --------------------------------------------------------------------------- the model

def run_order(cfg):
    """[(layer index, pass number or None when a pass does not start here)]."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def layer(x, w, cfg, i, tokens, positions, routes_out=None):
    spec, p = cfg["layers"][i], f"l{i}."
    eps, groups, m = cfg["norm"]["eps"], cfg["norm"].get("groups", 1), cfg.get("residual_mult", 1.0)
    canon = bool(cfg.get("canon"))
    if spec["type"] != "attention":
        raise ValueError(f"no mixer '{spec['type']}'")
    h1 = sublayer_input(x, w[p + "norm1"], w[p + "canon1"] if canon else None, groups, eps)
    delta = attention_mixer(h1, w, p + "mix.", spec["mixer"], eps, positions)
    if spec.get("mlp") is not None:
        h2 = sublayer_input(x, w[p + "norm2"], w[p + "canon2"] if canon else None, groups, eps)
        delta = delta + moe_mlp(h2, w, p + "mlp.", spec["mlp"], routes_out)
    x = x + m * delta
    if cfg.get("token_side"):
        x = x + m * token_side(x, tokens, w, p, i, cfg["token_side"]["dim"], eps)
    return x


def forward(w, cfg, tokens, layers_out=None, routes_out=None):
    """Logits [T, vocab] of one whole sequence."""
    tokens = np.asarray(tokens)
    positions = np.arange(len(tokens))
    x = embed(w, cfg, tokens)
    for i, start_of_pass in run_order(cfg):
        if start_of_pass is not None:
            x = x + f64(w["loop.step"])[start_of_pass]
        x = layer(x, w, cfg, i, tokens, positions, routes_out)
        if layers_out is not None:
            layers_out.append(x.copy())
    last = kept(grouped_norm(x, w["final.norm"], cfg["norm"].get("groups", 1), cfg["norm"]["eps"]))
    return f64(last) @ f64(w["head"]).T


def generate(w, cfg, prompt, n):
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(np.argmax(forward(w, cfg, tokens)[-1])))
    return tokens[len(prompt):]


# --------------------------------------------------------------------------- small configurations and random weights

def moe(ff=24, experts=8, top=2, groups=4, keep=2, limit=1.5):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, base=10000.0, scale=None, mlp="moe"):
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if rot_dims is not None:
        mx["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "attention", "mixer": mx, "mlp": moe() if mlp == "moe" else mlp}


def make_config(layers, vocab=160, width=64, eps=1e-6, groups=2, mult=0.8, taps=3, side=6, bigram=(53, 5, 3), loop=None):
    """`bigram` = (buckets, mul_prev, mul_cur) or None; `taps` 0 and `side` 0 leave those mechanisms out."""
    cfg = {"architecture": "Lufatar", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
           "residual_mult": mult, "layers": layers}
    if taps:
        cfg["canon"] = {"taps": taps}
    if side:
        cfg["token_side"] = {"dim": side}
    if bigram is not None:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def tensor_shapes(cfg):
    D, V, n = cfg["width"], cfg["vocab"], len(cfg["layers"])
    s = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        s["bigram"] = (bg["buckets"] + 1, D)
    if cfg.get("loop"):
        s["loop.step"] = (cfg["loop"]["times"], D)
    side = (cfg.get("token_side") or {}).get("dim", 0)
    if side:
        s["side.embed"] = (V, n * side)
    taps = (cfg.get("canon") or {}).get("taps", 0)
    for i, layer in enumerate(cfg["layers"]):
        p, mx, mlp = f"l{i}.", layer["mixer"], layer.get("mlp")
        H, G, dim, vdim = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        s.update({p + "norm1": (D,), p + "mix.q": (H * dim, D), p + "mix.k": (G * dim, D), p + "mix.v": (G * vdim, D),
                  p + "mix.talk": (H, H), p + "mix.o": (D, H * vdim)})
        if taps:
            s[p + "canon1"] = (D, taps)
        if mlp is not None:
            s[p + "norm2"] = (D,)
            if taps:
                s[p + "canon2"] = (D, taps)
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            s[p + "mlp.router"], s[p + "mlp.correction"] = (E, D), (E,)
            for e in range(E):
                s.update({f"{p}mlp.e{e}.gate": (ff, D), f"{p}mlp.e{e}.up": (ff, D), f"{p}mlp.e{e}.down": (D, ff)})
        if side:
            s.update({p + "side.gate": (side, D), p + "side.proj": (D, side), p + "side.norm": (D,)})
    return s


def random_weights(cfg, seed, sharp=3.0, expert_gain=1.0):
    """float32 weights that bfloat16 holds exactly (so that both dtypes load the same model). Matrices are N(0, 1/in); the
    query and key projections are `sharp` times larger (queries and keys are normed to unit RMS, so the config's `scale`
    decides how peaked attention is; `sharp` only keeps the products well above rounding). The head mix is the identity
    plus noise, with clearly non-zero entries off the diagonal. `expert_gain` scales what the experts add to the stream (a
    close routing call that 16-bit rounding decides the other way then stays within a 16-bit tolerance)."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name in ("embed", "bigram", "side.embed", "loop.step"):
            t = rng.standard_normal(shape) * (0.5 if name != "embed" else 1.0)
        elif leaf in ("norm1", "norm2", "norm"):
            t = 1.0 + rng.standard_normal(shape) * 0.1
        elif leaf in ("canon1", "canon2"):
            t = rng.standard_normal(shape) * 0.4
        elif leaf == "talk":
            t = np.eye(shape[0]) + rng.standard_normal(shape) * 0.3
        elif leaf == "correction":
            t = rng.standard_normal(shape) * 0.3
        else:
            t = rng.standard_normal(shape) / np.sqrt(shape[-1])
            if leaf in ("q", "k") and ".mix." in name:
                t = t * sharp
            if leaf == "router":
                t = t * 4.0
            if leaf == "down" and ".mlp.e" in name:
                t = t * expert_gain
        w[name] = round_bf16(np.asarray(t, dtype=np.float32))
    return w
