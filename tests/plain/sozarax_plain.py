"""Plain, slow Sozarax forward pass in numpy float64: the yardstick of its tests.

Whole sequences, no cache, no paging, no batches; one function per mechanism.
Nothing here is imported by the product package and nothing of the product
package is imported here.  Weights arrive as a dict of tensor name -> numpy
array and are widened to float64; ``cfg`` is the dict of a config.json.

Notation: T tokens, d the model width, H query heads, G key/value heads, dk the
per-head query/key size, dv the per-head value size, N the key/value size of a
recurrent head.
"""
from __future__ import annotations

import numpy as np


def f64(a):
    return np.asarray(a, dtype=np.float64)


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = f64(x)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def rmsnorm(x, gain, eps):
    return rms_unit(x, eps) * f64(gain)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def embed(table, ids, scale):
    return f64(table)[np.asarray(ids, dtype=np.int64)] * float(scale)


# ---- the recurrent mixer ------------------------------------------------------

def token_shift(h, mu, first=None):
    """h + (h_prev - h) * mu, h_prev the row before (``first`` or zeros for row 0)."""
    h = f64(h)
    prev = np.zeros_like(h)
    prev[1:] = h[:-1]
    if first is not None:
        prev[0] = f64(first)
    return h + (prev - h) * f64(mu)


def wkv_decay(mix_w, w1, w2, w0):
    """exp(-exp(W2 tanh(W1 m) + w0)), one value per head and key channel."""
    return np.exp(-np.exp(np.tanh(f64(mix_w) @ f64(w1).T) @ f64(w2).T + f64(w0)))


def wkv_scan(r, k, v, w, u, heads, size, state=None):
    """Per head, with S [N, N] (key channel x value channel) starting at zero:
    o_t[j] = sum_i r_t[i] (S[i, j] + u[i] k_t[i] v_t[j]);  S <- diag(w_t) S + k_t v_t^T.
    Returns (o [T, heads*N], S [heads, N, N])."""
    T = r.shape[0]
    r, k, v, w = (f64(a).reshape(T, heads, size) for a in (r, k, v, w))
    u = f64(u).reshape(heads, size)
    S = np.zeros((heads, size, size)) if state is None else f64(state).copy()
    o = np.zeros((T, heads, size))
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S = w[t][:, :, None] * S + kv
    return o.reshape(T, heads * size), S


def wkv_mixer(h, w, p, heads, size, eps):
    """The whole recurrent mixer on its input h [T, d]; tensors ``p + name``."""
    mix = {s: token_shift(h, w[p + "mu." + s]) for s in "rkvgw"}
    r = mix["r"] @ f64(w[p + "r"]).T
    k = mix["k"] @ f64(w[p + "k"]).T
    v = mix["v"] @ f64(w[p + "v"]).T
    gate = silu(mix["g"] @ f64(w[p + "g"]).T)
    decay = wkv_decay(mix["w"], w[p + "w1"], w[p + "w2"], w[p + "w0"])
    o, _ = wkv_scan(r, k, v, decay, w[p + "u"], heads, size)
    T = h.shape[0]
    o = rms_unit(o.reshape(T, heads, size), eps).reshape(T, heads * size)
    return (o * f64(w[p + "norm"]) * gate) @ f64(w[p + "o"]).T


# ---- the attention mixer --------------------------------------------------------

def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1)."""
    p = np.asarray(positions, dtype=np.int64)
    return 1.0 + float(coef) * np.log(((p + 1) // int(every)) + 1.0)


def head_slopes(heads):
    """2^(-8 (h + 1) / H) for h = 0 .. H-1."""
    return 2.0 ** (-8.0 * (np.arange(heads) + 1.0) / heads)


def biased_attention(q, k, v, H, G, dk, dv, scale, slopes):
    """Causal softmax attention; score(i, j) = q_i . k_j * scale - slope_h (i - j)."""
    q, k, v = f64(q), f64(k), f64(v)
    T = q.shape[0]
    pos = np.arange(T)
    dist = (pos[:, None] - pos[None, :]).astype(np.float64)
    seen = dist >= 0
    out = np.zeros((T, H * dv))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h * dk:(h + 1) * dk] @ k[:, g * dk:(g + 1) * dk].T) * scale - slopes[h] * dist
        s = np.where(seen, s, -np.inf)
        e = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h * dv:(h + 1) * dv] = (e / e.sum(axis=1, keepdims=True)) @ v[:, g * dv:(g + 1) * dv]
    return out


def attention_mixer(h, w, p, m, eps, positions=None):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    positions = np.arange(T) if positions is None else positions
    q = rmsnorm(f64(h) @ f64(w[p + "q"]).T, w[p + "q.norm"], eps)
    k = rmsnorm(f64(h) @ f64(w[p + "k"]).T, w[p + "k.norm"], eps)
    v = f64(h) @ f64(w[p + "v"]).T
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(positions, qt["coef"], qt["every"])[:, None]
    a = biased_attention(q, k, v, H, G, dk, dv, m["scale"], head_slopes(H))
    return a @ f64(w[p + "o"]).T


# ---- feed-forwards ----------------------------------------------------------------

def dense_ff(h, w, p):
    """W_down relu(W_up h)^2."""
    z = np.maximum(f64(h) @ f64(w[p + "up"]).T, 0.0)
    return (z * z) @ f64(w[p + "down"]).T


def route(h, router, top):
    """(indices [T, top], weights [T, top]): the ``top`` largest sigmoid scores, as they are."""
    s = sigmoid(f64(h) @ f64(router).T)
    idx = np.argsort(-s, axis=1, kind="stable")[:, :top]
    return idx, np.take_along_axis(s, idx, axis=1)


def moe_ff(h, w, p, experts, top):
    """sum over the chosen experts e of expert_e(s_e * h), expert = W_down(silu(W_gate x) * W_up x)."""
    h = f64(h)
    idx, wt = route(h, w[p + "router"], top)
    out = np.zeros((h.shape[0], f64(w[p + "e0.down"]).shape[0]))
    for t in range(h.shape[0]):
        for e, s in zip(idx[t], wt[t]):
            x = h[t] * s
            q = f"{p}e{int(e)}."
            out[t] += (silu(x @ f64(w[q + "gate"]).T) * (x @ f64(w[q + "up"]).T)) @ f64(w[q + "down"]).T
    return out


# ---- the model -----------------------------------------------------------------------

def layer_order(cfg):
    """Indices of the layers in the order they run: the layers start .. stop-1 of the loop
    ``times`` times in a row, where they stand."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def layer(x, w, cfg, i):
    L = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    p = f"l{i}."
    h = rmsnorm(x, w[p + "norm1"], eps)
    if L["type"] == "wkv":
        y = wkv_mixer(h, w, p + "mix.", L["mixer"]["heads"], L["mixer"]["dim"], eps)
    elif L["type"] == "attention":
        y = attention_mixer(h, w, p + "mix.", L["mixer"], eps)
    else:
        raise ValueError(L["type"])
    x = x + rmsnorm(y, w[p + "norm1b"], eps)
    if L.get("mlp"):
        h = rmsnorm(x, w[p + "norm2"], eps)
        if L["mlp"]["kind"] == "dense":
            y = dense_ff(h, w, p + "mlp.")
        else:
            y = moe_ff(h, w, p + "mlp.", L["mlp"]["router"]["experts"], L["mlp"]["router"]["top"])
        x = x + rmsnorm(y, w[p + "norm2b"], eps)
    return x


def forward(w, cfg, ids, taps=None):
    """Logits [T, vocab] of one whole sequence; ``taps`` (a list) receives the residual
    stream after every layer run."""
    x = embed(w["embed"], ids, cfg["embedding"]["scale"])
    for i in layer_order(cfg):
        x = layer(x, w, cfg, i)
        if taps is not None:
            taps.append(x.copy())
    return rmsnorm(x, w["final.norm"], cfg["norm"]["eps"]) @ f64(w["head"]).T


# ---- random models for the tests ----------------------------------------------------------

def tensor_shapes(cfg):
    d, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, d), "final.norm": (d,), "head": (V, d)}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if L.get("mlp") else ()):
            out[p + n] = (d,)
        m = L["mixer"]
        if L["type"] == "wkv":
            A = m["heads"] * m["dim"]
            for s in "rkvgw":
                out[p + "mix.mu." + s] = (d,)
            for s in "rkvg":
                out[p + "mix." + s] = (A, d)
            lora = m.get("decay_rank", 8)
            out.update({p + "mix.w1": (lora, d), p + "mix.w2": (A, lora), p + "mix.w0": (A,),
                        p + "mix.u": (m["heads"], m["dim"]), p + "mix.norm": (A,), p + "mix.o": (d, A)})
        else:
            Q, K, Vv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
            out.update({p + "mix.q": (Q, d), p + "mix.k": (K, d), p + "mix.v": (Vv, d), p + "mix.q.norm": (Q,),
                        p + "mix.k.norm": (K,), p + "mix.o": (d, m["heads"] * m["vdim"])})
        ml = L.get("mlp")
        if ml and ml["kind"] == "dense":
            out.update({p + "mlp.up": (ml["ff"], d), p + "mlp.down": (d, ml["ff"])})
        elif ml:
            f = ml["expert"]["ff"]
            out[p + "mlp.router"] = (ml["router"]["experts"], d)
            for e in range(ml["router"]["experts"]):
                out.update({f"{p}mlp.e{e}.gate": (f, d), f"{p}mlp.e{e}.up": (f, d), f"{p}mlp.e{e}.down": (d, f)})
    return out


def random_weights(cfg, seed, bf16=True):
    """Weights whose faults show: sharp attention, decays spread between fast and slow,
    routers with clear winners.  With ``bf16`` every value is a bfloat16 number."""
    rng = np.random.default_rng(seed)
    d = cfg["width"]
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") else name
        if len(shape) == 1 and ("norm" in leaf):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf.startswith("mix.mu."):
            a = rng.uniform(0.0, 1.0, shape)
        elif leaf == "mix.w0":
            a = rng.uniform(-6.0, 0.5, shape)
        elif leaf == "mix.u":
            a = 0.5 * rng.standard_normal(shape)
        elif leaf == "mlp.router":
            a = rng.standard_normal(shape) * 2.0 / np.sqrt(d)
        elif leaf in ("mix.q", "mix.k") and len(shape) == 2 and cfg_is_attention(cfg, name):
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
        elif name == "embed":
            a = rng.standard_normal(shape)
        else:
            a = rng.standard_normal(shape) / np.sqrt(shape[-1])
        w[name] = round_bf16(a) if bf16 else a
    return w


def cfg_is_attention(cfg, name):
    return cfg["layers"][int(name[1:].split(".")[0])]["type"] == "attention"


def round_bf16(a):
    """Nearest bfloat16 (ties to even) of every element, returned as float64."""
    a32 = np.ascontiguousarray(np.asarray(a, dtype=np.float32))
    b = a32.view(np.uint32).astype(np.uint64)
    b = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) << 16
    return b.astype(np.uint32).view(np.float32).astype(np.float64).reshape(a32.shape)
