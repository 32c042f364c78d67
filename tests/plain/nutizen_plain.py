"""Plain, slow Nutizen forward pass in numpy float64: the yardstick of its tests.

Whole sequences, no cache, no paging, no batches; one function per mechanism.
Nothing here is imported by the product package and nothing of the product
package is imported here.  Weights arrive as a dict of tensor name -> numpy
array and are widened to float64; ``cfg`` is the dict of a config.json.

Notation: T tokens, d the model width, H heads, dk the per-head query/key size,
dv the per-head value size, Rq / R the sizes of the query latent and of the
key/value latent, S residual streams, W a window.
"""
from __future__ import annotations

import numpy as np


def f64(a):
    return np.asarray(a, dtype=np.float64)


def rmsnorm(x, gain, eps):
    x = f64(x)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * f64(gain)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def embed(table, ids, scale):
    return f64(table)[np.asarray(ids, dtype=np.int64)] * float(scale)


# ---- residual streams ------------------------------------------------------------

def streams_read(xs, w_in):
    """u = sum_s w_in[s] xs[s]; xs [S, T, d]."""
    return np.einsum("s,std->td", f64(w_in), f64(xs))


def streams_write(xs, y, w_mix, w_out):
    """xs'[t] = sum_s w_mix[s, t] xs[s] + w_out[t] y, every new stream from the old ones."""
    xs = f64(xs)
    return np.einsum("st,sTd->tTd", f64(w_mix), xs) + f64(w_out)[:, None, None] * f64(y)[None]


# ---- the mixer --------------------------------------------------------------------

def window_mask(T, window):
    """visible[i, j]: 0 <= i - j < window (no window: 0 <= i - j)."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    vis = j <= i
    if window:
        vis &= (i - j) < window
    return vis


def softmax_with_sink(scores, visible, sink):
    """Row-wise softmax over the visible scores with one more term exp(sink) in the
    denominator that has no value; scores [T, T], sink a number."""
    s = np.where(visible, scores, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.where(visible, np.exp(s - m), 0.0)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - m))


def latent(h, w_down, gain, eps):
    """RMS-normed low-rank projection of h."""
    return rmsnorm(f64(h) @ f64(w_down).T, gain, eps)


def latent_attention(h, w, p, m, eps, c_kv=None):
    """The mixer on its input h [T, d]; tensors ``p + name``; m the mixer's config dict.
    ``c_kv``: the key/value latents of another layer to use instead of this layer's own.
    Returns (output [T, d], the key/value latents used [T, R])."""
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    cq = latent(h, w[p + "dq"], w[p + "dq.norm"], eps)
    q = (cq @ f64(w[p + "uq"]).T).reshape(T, H, dk)
    c = latent(h, w[p + "dkv"], w[p + "dkv.norm"], eps) if c_kv is None else f64(c_kv)
    k = (c @ f64(w[p + "uk"]).T).reshape(T, H, dk)
    v = (c @ f64(w[p + "uv"]).T).reshape(T, H, dv)
    vis = window_mask(T, (m.get("mask") or {}).get("size"))
    sink = f64(w[p + "sink"])
    out = np.zeros((T, H, dv))
    for hh in range(H):
        pr = softmax_with_sink(q[:, hh] @ k[:, hh].T * m["scale"], vis, sink[hh])
        out[:, hh] = pr @ v[:, hh]
    return out.reshape(T, H * dv) @ f64(w[p + "o"]).T, c


# ---- feed-forwards ----------------------------------------------------------------

def dense_ff(h, w, p):
    g, u = f64(h) @ f64(w[p + "gate"]).T, f64(h) @ f64(w[p + "up"]).T
    return (g * sigmoid(g) * u) @ f64(w[p + "down"]).T


def clamped_expert(h, w, p, limit):
    """W_down (g sigmoid(1.702 g) (u + 1)) with g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit)."""
    g = np.minimum(f64(h) @ f64(w[p + "gate"]).T, limit)
    u = np.clip(f64(h) @ f64(w[p + "up"]).T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ f64(w[p + "down"]).T


def table_experts(h, ids, w, p, mlp):
    """Every token runs the experts that the table lists for its id, each weighted 1 / top."""
    table = np.asarray(w[p + "table"], dtype=np.int64)
    top = mlp["router"]["top"]
    y = np.zeros_like(f64(h))
    for t, tok in enumerate(ids):
        for e in table[tok]:
            y[t] += clamped_expert(f64(h)[t:t + 1], w, f"{p}e{int(e)}.", mlp["expert"]["limit"])[0] / top
    return y


def shared_expert(h, w, p, limit):
    """An expert that every token runs, times sigmoid(w_sg . h)."""
    return clamped_expert(h, w, p, limit) * sigmoid(f64(h) @ f64(w[p + "sg"]).T)


def feed_forward(h, ids, w, p, mlp):
    if mlp["kind"] == "dense":
        return dense_ff(h, w, p)
    y = table_experts(h, ids, w, p, mlp)
    if mlp.get("shared"):
        y = y + shared_expert(h, w, p + "shared.", mlp["shared"]["limit"])
    return y


# ---- the model --------------------------------------------------------------------

def forward(w, cfg, ids, taps=None):
    """Logits float64 [T, vocab] of one sequence.  ``taps``: a list that receives the residual
    stream (the sum of the streams) after every layer."""
    eps = cfg["norm"]["eps"]
    S = cfg.get("streams")
    x = embed(w["embed"], ids, cfg["embedding"]["scale"])
    xs = np.stack([x] * S) if S else None
    latents = {}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        subs = [("mix", 1)] + ([("mlp", 2)] if L.get("mlp") else [])
        for name, q in subs:
            u = streams_read(xs, w[f"{p}hc{q}.in"]) if S else x
            hn = rmsnorm(u, w[f"{p}norm{q}"], eps)
            if name == "mix":
                src = L["mixer"].get("kv_from")
                y, latents[i] = latent_attention(hn, w, p + "mix.", L["mixer"], eps,
                                                 c_kv=None if src is None else latents[src])
            else:
                y = feed_forward(hn, ids, w, p + "mlp.", L["mlp"])
            if S:
                xs = streams_write(xs, y, w[f"{p}hc{q}.mix"], w[f"{p}hc{q}.out"])
            else:
                x = x + y
        if taps is not None:
            taps.append(xs.sum(axis=0) if S else x.copy())
    if S:
        x = xs.sum(axis=0)
    return rmsnorm(x, w["final.norm"], eps) @ f64(w["head"]).T


# ---- random models for the tests ----------------------------------------------------

def tensor_shapes(cfg):
    """name -> (shape, kind) of every tensor of a configuration; kind: matrix, gain, sink,
    stream_in, stream_out, stream_mix, table."""
    d, V, S = cfg["width"], cfg["vocab"], cfg.get("streams")
    out = {"embed": ((V, d), "matrix"), "head": ((V, d), "matrix"), "final.norm": ((d,), "gain")}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, dk, dv, Rq, R = m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"]
        out[p + "norm1"] = ((d,), "gain")
        out[p + "mix.dq"] = ((Rq, d), "matrix")
        out[p + "mix.dq.norm"] = ((Rq,), "gain")
        out[p + "mix.uq"] = ((H * dk, Rq), "matrix")
        if m.get("kv_from") is None:
            out[p + "mix.dkv"] = ((R, d), "matrix")
            out[p + "mix.dkv.norm"] = ((R,), "gain")
        out[p + "mix.uk"] = ((H * dk, R), "matrix")
        out[p + "mix.uv"] = ((H * dv, R), "matrix")
        out[p + "mix.sink"] = ((H,), "sink")
        out[p + "mix.o"] = ((d, H * dv), "matrix")
        qs = [1]
        mlp = L.get("mlp")
        if mlp:
            qs.append(2)
            out[p + "norm2"] = ((d,), "gain")
            if mlp["kind"] == "dense":
                f = mlp["ff"]
                for n, s in (("gate", (f, d)), ("up", (f, d)), ("down", (d, f))):
                    out[p + "mlp." + n] = (s, "matrix")
            else:
                f = mlp["expert"]["ff"]
                for e in range(mlp["router"]["experts"]):
                    for n, s in (("gate", (f, d)), ("up", (f, d)), ("down", (d, f))):
                        out[f"{p}mlp.e{e}.{n}"] = (s, "matrix")
                out[p + "mlp.table"] = ((V, mlp["router"]["top"]), "table")
                if mlp.get("shared"):
                    f = mlp["shared"]["ff"]
                    for n, s in (("gate", (f, d)), ("up", (f, d)), ("down", (d, f)), ("sg", (1, d))):
                        out[p + "mlp.shared." + n] = (s, "matrix")
        if S:
            for q in qs:
                out[f"{p}hc{q}.in"] = ((S,), "stream_in")
                out[f"{p}hc{q}.out"] = ((S,), "stream_out")
                out[f"{p}hc{q}.mix"] = ((S, S), "stream_mix")
    return out


def round_bf16(a):
    """float32 array rounded to the nearest bfloat16 (ties to even), as float32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    bits = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return bits.view(np.float32).reshape(a.shape)


def random_weights(cfg, seed, std=0.05, qk_boost=1.0):
    """Random tensors (all exactly representable in bfloat16) of a configuration.  Stream
    weights lie near the values that make the streams a plain residual sum; the rows of an
    expert table hold distinct experts."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        if kind == "matrix":
            a = rng.normal(0.0, std, size=shape)
            if name.endswith("mix.uq") or name.endswith("mix.uk"):
                a *= qk_boost
        elif kind == "gain":
            a = 1.0 + rng.normal(0.0, 0.1, size=shape)
        elif kind == "sink":
            a = rng.normal(0.0, 1.0, size=shape)
        elif kind == "stream_in":
            a = 1.0 / shape[0] + rng.normal(0.0, 0.1, size=shape)
        elif kind == "stream_out":
            a = 1.0 + rng.normal(0.0, 0.2, size=shape)
        elif kind == "stream_mix":
            a = np.eye(shape[0]) + rng.normal(0.0, 0.1, size=shape)
        elif kind == "table":
            E = next(L["mlp"]["router"]["experts"] for i, L in enumerate(cfg["layers"]) if name.startswith(f"l{i}."))
            w[name] = np.stack([rng.permutation(E)[:shape[1]] for _ in range(shape[0])]).astype(np.int32)
            continue
        w[name] = round_bf16(a.astype(np.float32))
    return w
