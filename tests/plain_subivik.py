"""A plain, slow Subivik in numpy: whole sequences, no cache, no state carried between calls, one function per
mechanism. Arithmetic is float64 on the stored values. Nothing here imports the engine package: the tests compare
the two.

A Subivik model lists its layers in any order. A layer is a mixer behind a norm and, optionally, a feed-forward
behind a norm, both added to the residual stream. The norm is a dynamic tanh: tanh(alpha x) * w + b, no mean, no
variance. The token embedding gets a sinusoid of the position added. Mixers:

  attention   differential attention in chunks: two score maps per head over the same values, each with a softmax of
              its own, combined as a1 - lambda a2, normed per head, gated by a sigmoid of a projection of the input.
              A position sees the earlier positions of its own chunk only. A layer may read the keys and values that
              an earlier layer made (`kv_from`).
  parallel    two mixers side by side on the same input, summed with one factor each:
              left, causal attention with capped scores, a bias that grows with the logarithm of the distance, and
              softmax weights that are mixed across heads; right, a recurrence with a matrix state per head that
              decays per key channel, reads the state before it writes, and blends every input with the token before.

Feed-forwards: `dense` (one hidden layer with a piecewise activation of two learned numbers) and `moe` (softmax
router, the best `top` experts, weights = scores times a constant, gated experts with silu).
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


# --------------------------------------------------------------------------- small functions

def f64(a):
    return np.asarray(a, dtype=np.float64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = f64(x)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def round_bf16(x):
    a = np.ascontiguousarray(x, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).reshape(np.shape(x))


_act = None       # with `bfloat16_activations()`: rounds what a 16-bit pipeline would keep in 16 bits


class bfloat16_activations:
    """Within this context the outputs of `linear` and of the layers' norms are rounded to bfloat16 (the weights of the
    tests are bfloat16 values already): the distance to the exact result is the noise that a pipeline with 16-bit
    activations cannot avoid, which is what a tolerance for such a pipeline is measured against."""

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


def dynamic_tanh(x, w, name):
    """tanh(alpha x) * weight + bias with the scalar `<name>.alpha` and the vector `<name>.b`."""
    return kept(np.tanh(float(f64(w[name + ".alpha"])) * f64(x)) * f64(w[name]) + f64(w[name + ".b"]))


def sinusoid(positions, width):
    """[n, width]: entry 2i = sin(p / 10000^(2i/width)), entry 2i+1 = cos of the same angle."""
    out = np.zeros((len(positions), width))
    for i in range((width + 1) // 2):
        angle = f64(positions) * 10000.0 ** (-2.0 * i / width)
        out[:, 2 * i] = np.sin(angle)
        if 2 * i + 1 < width:
            out[:, 2 * i + 1] = np.cos(angle)
    return out


def softmax_where(scores, visible):
    """Row-wise softmax over the entries where `visible`; zero elsewhere."""
    s = np.where(visible, scores, -np.inf)
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def causal(n):
    i = np.arange(n)
    return i[None, :] <= i[:, None]


def chunk_mask(n, size):
    """Position i sees j <= i of its own chunk; chunks of `size` positions counted from 0 (size None or 0: all of them)."""
    i = np.arange(n)
    m = causal(n)
    if size:
        m = m & ((i[:, None] // size) == (i[None, :] // size))
    return m


# --------------------------------------------------------------------------- differential attention

def diff_lambda(w, p, diff):
    return float(np.exp(np.sum(f64(w[p + "lq1"]) * f64(w[p + "lk1"]))) - np.exp(np.sum(f64(w[p + "lq2"]) * f64(w[p + "lk2"]))) + diff)


def diff_keys_values(h, w, p, mx, eps):
    """What a layer of this kind keeps per token: normed keys [n, G, 2, dim] and values [n, G, vdim]."""
    n, G, dim, vdim = h.shape[0], mx["kv_heads"], mx["dim"], mx["vdim"]
    k = linear(h, w[p + "k"]).reshape(n, G, 2, dim)
    k = kept(unit_rms(k, eps) * f64(w[p + "k.norm"]))
    v = linear(h, w[p + "v"]).reshape(n, G, vdim)
    return k, v


def diff_attention_mixer(h, w, p, mx, eps, kv):
    """h [n, width]; kv = (keys, values) of this layer or of the layer it borrows them from."""
    n, H, G, dim, vdim = h.shape[0], mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    k, v = kv
    q = linear(h, w[p + "q"]).reshape(n, H, 2, dim)
    q = unit_rms(q, eps) * f64(w[p + "q.norm"])
    see = chunk_mask(n, (mx.get("mask") or {}).get("size"))
    lam = diff_lambda(w, p, float(mx["diff"]))
    out = np.zeros((n, H, vdim))
    for head in range(H):
        g = head // (H // G)
        maps = [softmax_where(float(mx["scale"]) * (q[:, head, m] @ k[:, g, m].T), see) @ v[:, g] for m in (0, 1)]
        o = maps[0] - lam * maps[1]
        out[:, head] = unit_rms(o, eps) * (1.0 - float(mx["diff"]))
    gate = sigmoid(linear(h, w[p + "g"]))
    return linear(kept(out.reshape(n, H * vdim) * gate), w[p + "o"])


# --------------------------------------------------------------------------- the two halves of a parallel mixer

def capped(s, cap):
    return s if not cap else cap * np.tanh(s / cap)


def distance_bias(n, r1, r2):
    """[n, n]: r1 ln(1 + r2 (i - j)) for j <= i (0 elsewhere; those are masked anyway)."""
    i = np.arange(n)
    d = np.maximum(i[:, None] - i[None, :], 0)
    return r1 * np.log1p(r2 * d)


def talking_attention(h, w, p, mx):
    """Causal attention whose softmax weights are mixed across heads before they meet the values."""
    n, H, G, dim, vdim = h.shape[0], mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = linear(h, w[p + "q"]).reshape(n, H, dim)
    k = linear(h, w[p + "k"]).reshape(n, G, dim)
    v = linear(h, w[p + "v"]).reshape(n, G, vdim)
    see = causal(n)
    r1, r2, talk = f64(w[p + "r1"]), f64(w[p + "r2"]), f64(w[p + "talk"])
    weights = np.zeros((H, n, n))
    for head in range(H):
        s = capped(float(mx["scale"]) * (q[:, head] @ k[:, head // (H // G)].T), mx.get("softcap"))
        weights[head] = softmax_where(s - distance_bias(n, r1[head], r2[head]), see)
    mixed = np.einsum("hg,gij->hij", talk, weights)
    out = np.stack([mixed[head] @ v[:, head // (H // G)] for head in range(H)], axis=1)
    return linear(kept(out.reshape(n, H * vdim)), w[p + "o"])


def bonus_recurrence(r, k, v, decay, bonus):
    """Per head: o_t = (S + diag(bonus) k_t v_t^T)^T r_t, then S <- diag(decay_t) S + k_t v_t^T; S starts at zero.
    r, k, v, decay [n, H, dim]; bonus [H, dim]."""
    n, H, dim = r.shape
    out = np.zeros((n, H, dim))
    for head in range(H):
        S = np.zeros((dim, dim))
        for t in range(n):
            kv = np.outer(k[t, head], v[t, head])
            out[t, head] = (S + bonus[head][:, None] * kv).T @ r[t, head]
            S = decay[t, head][:, None] * S + kv
    return out


def time_mix(h, w, p, mx, eps):
    n, H, dim = h.shape[0], mx["heads"], mx["dim"]
    h = f64(h)
    before = np.concatenate([np.zeros((1, h.shape[1])), h[:-1]], axis=0)
    blend = lambda s: kept(h + (before - h) * f64(w[p + "mu." + s]))
    r = linear(blend("r"), w[p + "r"]).reshape(n, H, dim)
    k = linear(blend("k"), w[p + "k"]).reshape(n, H, dim)
    v = linear(blend("v"), w[p + "v"]).reshape(n, H, dim)
    gate = silu(linear(blend("g"), w[p + "g"]))
    inner = kept(np.tanh(linear(blend("w"), w[p + "w1"])))
    decay = np.exp(-np.exp(f64(inner) @ f64(w[p + "w2"]).T + f64(w[p + "w0"]))).reshape(n, H, dim)
    o = bonus_recurrence(r, k, v, decay, f64(w[p + "u"]))
    o = unit_rms(o, eps).reshape(n, H * dim) * f64(w[p + "norm"]) * gate
    return linear(kept(o), w[p + "o"])


def parallel_mixer(h, w, p, mx, eps):
    left = talking_attention(h, w, p + "left.", mx["left"])
    right = time_mix(h, w, p + "right.", mx["right"], eps)
    return float(mx["left_scale"]) * left + float(mx["right_scale"]) * right


# --------------------------------------------------------------------------- feed-forwards

def two_branch_unit(z, a_pos, a_neg):
    """z > 0: softplus(a_pos) z^2 + z/2;  z <= 0: (1/2 + softplus(a_neg)) (exp(z) - 1 - z) + z/2."""
    z = f64(z)
    zn = np.minimum(z, 0.0)
    return np.where(z > 0, softplus(a_pos) * z * z + 0.5 * z, (0.5 + softplus(a_neg)) * (np.expm1(zn) - zn) + 0.5 * z)


def dense_mlp(h, w, p):
    a = f64(w[p + "act"])
    return linear(kept(two_branch_unit(linear(h, w[p + "up"]), a[0], a[1])), w[p + "down"])


def route(scores, top):
    """The `top` largest scores of a row, ties to the lower index."""
    order = sorted(range(len(scores)), key=lambda e: (-scores[e], e))
    return order[:top]


def expert(h, gate, up, down):
    return linear(kept(silu(linear(h, gate)) * linear(h, up)), down)


def moe_mlp(h, w, p, mlp, chosen_out=None):
    r = mlp["router"]
    z = f64(h) @ f64(w[p + "router"]).T
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    s = e / e.sum(axis=-1, keepdims=True)
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        chosen = route(s[t], r["top"])
        if chosen_out is not None:
            chosen_out.append(chosen)
        for ex in chosen:
            q = f"{p}e{ex}."
            out[t] += float(r["scale"]) * s[t, ex] * expert(h[t:t + 1], w[q + "gate"], w[q + "up"], w[q + "down"])[0]
    return out


# --------------------------------------------------------------------------- the model

def forward(w, cfg, tokens, layers_out=None, routes_out=None):
    """Logits [n, vocab] of a whole sequence from position 0."""
    n, width, eps = len(tokens), cfg["width"], float(cfg["norm"]["eps"])
    x = f64(w["embed"])[list(tokens)] + sinusoid(np.arange(n), width)
    kept_kv = {}
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        h = dynamic_tanh(x, w, p + "norm1")
        if layer["type"] == "attention":
            if mx.get("kv_from") is None:
                kept_kv[i] = diff_keys_values(h, w, p + "mix.", mx, eps)
            x = x + diff_attention_mixer(h, w, p + "mix.", mx, eps, kept_kv[i if mx.get("kv_from") is None else mx["kv_from"]])
        else:
            x = x + parallel_mixer(h, w, p + "mix.", mx, eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = dynamic_tanh(x, w, p + "norm2")
            x = x + (dense_mlp(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_mlp(h, w, p + "mlp.", mlp, routes_out))
        if layers_out is not None:
            layers_out.append(x.copy())
    return f64(dynamic_tanh(x, w, "final.norm")) @ f64(w["embed"]).T


def generate(w, cfg, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(forward(w, cfg, toks)[-1])))
    return toks[len(prompt):]


# --------------------------------------------------------------------------- configurations and weights for the tests

def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(ff=24, experts=6, top=2, scale=1.5):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, chunk=24, diff=0.3, scale=None, kv_from=None, mlp="dense"):
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": float(scale if scale is not None else dim ** -0.5)}
    if chunk:
        mx["mask"] = {"size": chunk}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "attention", "mixer": mx, "mlp": dense() if mlp == "dense" else mlp}


def parallel_layer(heads=4, kv_heads=2, dim=16, vdim=8, softcap=20.0, scale=None, rheads=2, rdim=24, left_scale=0.7,
                   right_scale=1.2, mlp="dense"):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "softcap": softcap,
            "scale": float(scale if scale is not None else dim ** -0.5)}
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": rheads, "dim": rdim}, "left_scale": left_scale,
                                          "right_scale": right_scale}, "mlp": dense() if mlp == "dense" else mlp}


def make_config(layers, vocab=160, width=64, eps=1e-6):
    return {"architecture": "Subivik", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def tensor_shapes(cfg, decay_rank=8):
    D = cfg["width"]
    s = {"embed": (cfg["vocab"], D)}

    def norm(name):
        s[name], s[name + ".b"], s[name + ".alpha"] = (D,), (D,), ()

    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        norm(p + "norm1")
        m = p + "mix."
        if layer["type"] == "attention":
            H, G, dim, vdim = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            s[m + "q"], s[m + "q.norm"] = (H * 2 * dim, D), (dim,)
            if mx.get("kv_from") is None:
                s[m + "k"], s[m + "v"], s[m + "k.norm"] = (G * 2 * dim, D), (G * vdim, D), (dim,)
            for leaf in ("lq1", "lk1", "lq2", "lk2"):
                s[m + leaf] = (dim,)
            s[m + "g"], s[m + "o"] = (H * vdim, D), (D, H * vdim)
        else:
            lf, rt = mx["left"], mx["right"]
            H, G, dim, vdim = lf["heads"], lf["kv_heads"], lf["dim"], lf["vdim"]
            a = m + "left."
            s[a + "q"], s[a + "k"], s[a + "v"], s[a + "o"] = (H * dim, D), (G * dim, D), (G * vdim, D), (D, H * vdim)
            s[a + "r1"], s[a + "r2"], s[a + "talk"] = (H,), (H,), (H, H)
            b, n = m + "right.", rt["heads"] * rt["dim"]
            for leaf in ("r", "k", "v", "g", "w"):
                s[b + "mu." + leaf] = (D,)
            for leaf in ("r", "k", "v", "g"):
                s[b + leaf] = (n, D)
            s[b + "w1"], s[b + "w2"], s[b + "w0"] = (decay_rank, D), (n, decay_rank), (n,)
            s[b + "u"], s[b + "norm"], s[b + "o"] = (rt["heads"], rt["dim"]), (n,), (D, n)
        mlp = layer.get("mlp")
        if mlp is not None:
            norm(p + "norm2")
            q = p + "mlp."
            if mlp["kind"] == "dense":
                s[q + "up"], s[q + "down"], s[q + "act"] = (mlp["ff"], D), (D, mlp["ff"]), (2,)
            else:
                ff = mlp["expert"]["ff"]
                s[q + "router"] = (mlp["router"]["experts"], D)
                for e in range(mlp["router"]["experts"]):
                    s[f"{q}e{e}.gate"], s[f"{q}e{e}.up"], s[f"{q}e{e}.down"] = (ff, D), (ff, D), (D, ff)
    norm("final.norm")
    return s


def random_weights(cfg, seed, decay_rank=8, sharp=3.0, expert_gain=1.0):
    """float32 weights that bfloat16 holds exactly (so that both dtypes load the same model). Matrices are N(0, 1/in);
    queries and keys are `sharp` times larger so that attention is not flat and a key that is lost or misplaced moves
    the logits; decays are spread between fast and slow channels. `expert_gain` scales what the experts add: a router's
    close call that 16-bit rounding decides the other way then stays inside a 16-bit tolerance."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg, decay_rank).items():
        leaf = name.split(".")[-1]
        if name == "embed":
            t = rng.standard_normal(shape)
        elif leaf == "alpha":
            t = np.asarray(rng.uniform(0.4, 0.9))
        elif leaf in ("norm1", "norm2") or name == "final.norm" or leaf == "norm":
            t = 1.0 + rng.standard_normal(shape) * 0.1
        elif leaf == "b":
            t = rng.standard_normal(shape) * 0.1
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = rng.standard_normal(shape) * 0.15
        elif leaf == "r1":
            t = rng.uniform(0.2, 1.0, shape)
        elif leaf == "r2":
            t = rng.uniform(0.1, 2.0, shape)
        elif leaf == "talk":
            t = np.eye(shape[0]) + rng.standard_normal(shape) * 0.3
        elif ".mu." in name:
            t = rng.uniform(0.0, 1.0, shape)
        elif leaf == "w0":
            t = rng.uniform(-6.0, 0.5, shape)
        elif leaf == "u":
            t = rng.standard_normal(shape) * 0.5
        elif leaf == "act":
            t = rng.standard_normal(shape) * 0.5
        else:
            t = rng.standard_normal(shape) / np.sqrt(shape[-1])
            if leaf in ("q", "k") and ".right." not in name:
                t = t * sharp
            if leaf == "router":
                t = t * 4.0
            if leaf == "down" and ".mlp.e" in name:
                t = t * expert_gain
        w[name] = round_bf16(np.asarray(t, dtype=np.float32))
    return w


def write_safetensors(path, tensors, bf16=True):
    """One file: 8-byte little-endian header length, JSON header, data. bf16 stores the upper 16 bits."""
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        shape = list(np.shape(t))
        a = np.ascontiguousarray(t, dtype=np.float32).reshape(-1)
        if bf16:
            data = (a.view(np.uint32) >> 16).astype("<u2").tobytes()
            dt = "BF16"
        else:
            data = a.astype("<f4").tobytes()
            dt = "F32"
        header[name] = {"dtype": dt, "shape": shape, "data_offsets": [off, off + len(data)]}
        blobs.append(data)
        off += len(data)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def write_model_dir(path, cfg, weights, bf16=True):
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(path / "model.safetensors", weights, bf16=bf16)
