"""The Sozarax design in the engine against its plain implementation (tests/plain/sozarax_plain.py).

Small configurations of their own, random weights whose values are bfloat16 numbers (so both
dtypes load the same model): each mechanism's kernel alone, whole prompts, prompts against
token-by-token decoding, portions down to two tokens, unequal batches, slots and pages that
are used again, keys far away and at page borders that one score makes stand out, the first
tokens, long decoding through CUDA graphs, and greedy generation through the scheduler.
"""
import types

import numpy as np
import pytest

from helpers import write_model_dir
from plain import sozarax_plain as P

pytestmark = pytest.mark.gpu

# Every size differs from layer to layer; heads, kv heads, key and value sizes, ranks, expert
# counts and the loop take values that are neither equal to each other nor 1 where they could be.
CFG_A = {
    "architecture": "Sozarax", "vocab": 96, "width": 64, "embedding": {"scale": 3.5}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3,
                                        "q_temp": {"coef": 0.5, "every": 4}},
         "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 4, "top": 2}}},
        {"type": "wkv", "mixer": {"heads": 2, "dim": 32, "decay_rank": 6}, "mlp": {"kind": "dense", "ff": 80}},
        {"type": "wkv", "mixer": {"heads": 3, "dim": 16, "decay_rank": 5}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.2},
         "mlp": {"kind": "dense", "ff": 40}},
    ],
    "loop": {"start": 1, "stop": 3, "times": 3},
}
CFG_B = {
    "architecture": "Sozarax", "vocab": 70, "width": 48, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "wkv", "mixer": {"heads": 1, "dim": 48, "decay_rank": 3},
         "mlp": {"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 3, "top": 3}}},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 1, "dim": 8, "vdim": 4, "scale": 0.5,
                                        "q_temp": {"coef": 0.25, "every": 1}},
         "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 5, "top": 1}}},
    ],
}
# Sizes that fit no vector width, tile or tensor-core shape: every kernel's general form.
CFG_C = {
    "architecture": "Sozarax", "vocab": 61, "width": 50, "embedding": {"scale": 7.07}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "wkv", "mixer": {"heads": 2, "dim": 12, "decay_rank": 4},
         "mlp": {"kind": "moe", "expert": {"ff": 7}, "router": {"experts": 2, "top": 1}}},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 10, "vdim": 6, "scale": 0.4,
                                        "q_temp": {"coef": 0.1, "every": 7}},
         "mlp": {"kind": "dense", "ff": 13}},
        {"type": "wkv", "mixer": {"heads": 5, "dim": 3, "decay_rank": 2}, "mlp": None},
    ],
    "loop": {"start": 0, "stop": 2, "times": 2},
}
CFGS = {"A": (CFG_A, 11), "B": (CFG_B, 12), "C": (CFG_C, 13)}
# max |engine - plain| over a row, as a fraction of the largest |logit|.  float32: float32 sums
# against float64 ones.  bfloat16: the plain implementation rounds nothing, so this is the whole
# rounding of bfloat16 activations through the layers; a router's choice between two experts
# whose scores lie within that rounding may fall the other way, so a twentieth of the rows may
# miss the bound.
TOL = {"float32": 4e-5, "bfloat16": 8e-2}


def make_model(tmp_path, name):
    cfg, seed = CFGS[name]
    w = P.random_weights(cfg, seed)
    d = write_model_dir(str(tmp_path / f"sozarax_{name}"), cfg,
                        {k: np.asarray(v, dtype=np.float32) for k, v in w.items()})
    return cfg, w, d


def check_rows(got, want, dtype, what):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    scale = max(1e-6, float(np.abs(want).max()))
    err = np.abs(got - want).max(axis=-1) / scale
    bad = int((err > TOL[dtype]).sum())
    allowed = 0 if dtype == "float32" else max(1, len(err) // 20)
    assert bad <= allowed, f"{what}: {bad} of {len(err)} rows over {TOL[dtype]:.0e} (worst {err.max():.2e} at row {int(err.argmax())})"


def engine_for(model_dir, dtype, **kw):
    from kllm_b200.engine import Engine, Options
    opts = dict(dtype=dtype, max_seq=512, block_size=16, num_blocks=64, max_step_tokens=512, max_batch=4)
    opts.update(kw)
    return Engine(model_dir, Options(**opts))


def run_cut(eng, ids, cuts):
    """Feed ``ids`` in portions of the given sizes (the last size repeats); all logits."""
    from kllm_b200.engine.step import StepEntry
    c = eng.cache.open()
    rows, pos, i = [], 0, 0
    while pos < len(ids):
        n = min(cuts[min(i, len(cuts) - 1)], len(ids) - pos)
        rows.append(eng.runner.run([StepEntry(c, ids[pos:pos + n], list(range(n)))]).float().cpu().numpy().copy())
        pos += n
        i += 1
    eng.cache.close(c)
    return np.concatenate(rows)


# ---- whole models --------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompt_and_every_way_of_cutting(tmp_path, name, dtype):
    cfg, w, d = make_model(tmp_path, name)
    rng = np.random.default_rng(5)
    ids = rng.integers(0, cfg["vocab"], size=150).tolist()
    want = P.forward(w, cfg, ids)
    eng = engine_for(d, dtype)
    try:
        whole = run_cut(eng, ids, [len(ids)])
        check_rows(whole, want, dtype, f"{name} whole")
        # the first tokens of a sequence on their own
        check_rows(run_cut(eng, ids[:3], [3]), want[:3], dtype, f"{name} first tokens")
        check_rows(run_cut(eng, ids[:1], [1]), want[:1], dtype, f"{name} one token")
        # most of it at once, then token by token (the decode steps replay as CUDA graphs)
        check_rows(run_cut(eng, ids, [len(ids) - 40, 1]), want, dtype, f"{name} prompt then decode")
        # token by token from the first token on
        check_rows(run_cut(eng, ids[:70], [1]), want[:70], dtype, f"{name} decode from the start")
        # portions of several sizes, down to two tokens, cut inside pages
        for cuts in ([2], [3, 2, 37, 16, 5, 2, 64, 1], [17], [16, 16, 1, 31, 2]):
            got = run_cut(eng, ids, cuts)
            check_rows(got, want, dtype, f"{name} portions {cuts}")
            if dtype == "float32":
                # the same position however it was cut: sums in another order, nothing more
                assert np.abs(got - whole).max() <= 1e-5 * np.abs(want).max(), cuts
        eng.cache.audit()
    finally:
        eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_and_reuse_of_slots_and_pages(tmp_path, dtype):
    """Four requests of unequal length in one batch, portions of some beside single tokens of
    others, then new requests in the slots and pages that the finished ones gave back; a pool
    that holds little more than what is live."""
    from kllm_b200.engine.step import StepEntry
    cfg, w, d = make_model(tmp_path, "A")
    rng = np.random.default_rng(9)
    lens = [37, 90, 5, 64, 21, 50]
    seqs = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lens]
    want = [P.forward(w, cfg, s) for s in seqs]
    eng = engine_for(d, dtype, num_blocks=20, max_batch=4)      # 320 tokens of pages, four slots
    try:
        got = [np.zeros_like(x) for x in want]
        fed = [0] * len(seqs)
        caches = {}
        queue = list(range(len(seqs)))
        sizes = [3, 1, 16, 2, 29, 1, 7]
        turn = 0
        slots_seen = []
        while queue or caches:
            while queue and len(caches) < 4:
                i = queue.pop(0)
                caches[i] = eng.cache.open()
                slots_seen.append(caches[i].state_slot)
            entries, order = [], []
            for i in list(caches):
                left = len(seqs[i]) - fed[i]
                n = 1 if left <= 8 else min(left, sizes[(turn + i) % len(sizes)])
                entries.append(StepEntry(caches[i], seqs[i][fed[i]:fed[i] + n], list(range(n))))
                order.append((i, n))
            lg = eng.runner.run(entries).float().cpu().numpy()
            r = 0
            for i, n in order:
                got[i][fed[i]:fed[i] + n] = lg[r:r + n]
                r += n
                fed[i] += n
                if fed[i] == len(seqs[i]):
                    eng.cache.close(caches.pop(i))
            turn += 1
            eng.cache.audit()
        assert len(slots_seen) > len(set(slots_seen)), "no state slot was used again"
        for i in range(len(seqs)):
            check_rows(got[i], want[i], dtype, f"request {i} in mixed batches")
    finally:
        eng.close()


def test_long_decoding(tmp_path):
    """A short prompt and then hundreds of single tokens: the decode route (graphs, the
    attention's key chunks and their merge, pages added one by one) over several chunk and
    page borders."""
    cfg, w, d = make_model(tmp_path, "B")
    rng = np.random.default_rng(3)
    ids = rng.integers(0, cfg["vocab"], size=600).tolist()
    want = P.forward(w, cfg, ids)
    eng = engine_for(d, "float32", max_seq=640, num_blocks=40)
    try:
        check_rows(run_cut(eng, ids, [9, 1]), want, "float32", "long decoding")
    finally:
        eng.close()


def test_greedy_generation_through_the_scheduler(tmp_path):
    """``Engine.generate`` (scheduler, sampler, pipelined steps) on several prompts at once
    against greedy decoding with the plain implementation."""
    cfg, w, d = make_model(tmp_path, "A")
    rng = np.random.default_rng(21)
    prompts = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in (7, 30, 2, 19, 45)]
    steps = 12
    eng = engine_for(d, "float32", max_step_tokens=48, max_batch=3)
    try:
        outs = eng.generate(prompts, max_new_tokens=steps)
        alone = eng.generate(prompts[1], max_new_tokens=steps)
    finally:
        eng.close()
    assert alone == outs[1]
    for p, out in zip(prompts, outs):
        ids = list(p)
        for k in range(steps):
            z = P.forward(w, cfg, ids)[-1]
            best = int(z.argmax())
            # a near-tie in float32 against float64 is not a fault of the engine
            assert out[k] == best or z[best] - z[out[k]] < 1e-4 * np.abs(z).max(), (len(p), k)
            ids.append(out[k])


def test_replay_program(tmp_path):
    """bin/trace_run on a model of this design: whole, decode, portions and mixed batches of up
    to four live requests in a pool as small as the trace allows (ways as in test_gpu_replay)."""
    from test_gpu_replay import build_trace
    from trace_tools import run_trace
    cfg, w, d = make_model(tmp_path, "A")
    rng = np.random.default_rng(4)
    seqs = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in (5, 33, 64, 100, 18)]
    want = [P.forward(w, cfg, s) for s in seqs]
    tb = build_trace(seqs, [7, 2, 13, 3, 1, 29], seed=8)
    for dtype in ("float32", "bfloat16"):
        rows = run_trace(d, dtype, tb, str(tmp_path / ("out_" + dtype)), cfg["vocab"])
        by_way = {}
        for (rid, pos), z in rows.items():
            by_way.setdefault((rid[0], int(rid[1:])), {})[pos] = z
        for (way, i), zs in by_way.items():
            pos = sorted(zs)
            check_rows(np.stack([zs[p] for p in pos]), want[i][pos], dtype, f"replay {way}{i}")


# ---- each mechanism's kernel alone ----------------------------------------------------------------

def _t(a, dtype="float32", dev="cuda"):
    import torch
    return torch.tensor(np.asarray(a), dtype=getattr(torch, dtype), device=dev).contiguous()


def _ctx(n_new, start, slots=None):
    """What the kernels read of a step: rows of request s are q_start[s] .. q_start[s + 1]."""
    import torch
    S = len(n_new)
    q_start = np.concatenate([[0], np.cumsum(n_new)]).astype(np.int32)
    return types.SimpleNamespace(
        n_tokens=int(q_start[-1]), n_requests=S, q_start=_t(q_start, "int32"),
        token_req=_t(np.repeat(np.arange(S), n_new), "int32"), start_pos=_t(start, "int32"),
        positions=_t(np.concatenate([np.arange(s, s + c) for s, c in zip(start, n_new)]), "int32"),
        state_slots=_t(slots if slots is not None else np.arange(S), "int32"),
        host_n_new=list(n_new), host_start_pos=list(start), all_single=all(c == 1 for c in n_new),
        max_ctx=max(s + c for s, c in zip(start, n_new)), split_bound=0, max_new=max(n_new))


@pytest.mark.parametrize("size,heads", [(64, 2), (16, 3), (48, 1), (96, 1), (128, 2)])
def test_wkv_scan_carries_its_state(size, heads):
    """The recurrence over two requests of unequal length in one launch, cut in two launches at
    an odd place, in slots 2 and 0, against the plain scan over each whole sequence."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(size)
    A = heads * size
    lens = [23, 9]
    r, k, v = (rng.standard_normal((sum(lens), A)) for _ in range(3))
    z = rng.uniform(-5, 1, (sum(lens), A))
    w0, u = rng.uniform(-1, 0.5, A), rng.standard_normal(A)
    state = torch.full((3, A * size + 8), 0.0, device="cuda")
    slots = [2, 0]
    outs = []
    cuts = [(0, 14), (0, 4)], [(14, 23), (4, 9)]
    offs = [0, lens[0]]
    for part in cuts:
        rows = np.concatenate([np.arange(offs[s] + a, offs[s] + b) for s, (a, b) in enumerate(part)])
        ctx = _ctx([b - a for a, b in part], [a for a, _ in part], slots)
        o = kernels.wkv_scan(_t(r[rows]), _t(k[rows]), _t(v[rows]), _t(z[rows]), _t(w0), _t(u), state, ctx, heads, size)
        outs.append((rows, o.cpu().numpy()))
    got = np.zeros((sum(lens), A))
    for rows, o in outs:
        got[rows] = o
    for s in range(2):
        sl = slice(offs[s], offs[s] + lens[s])
        want, S = P.wkv_scan(r[sl], k[sl], v[sl], np.exp(-np.exp(z[sl] + w0)), u, heads, size)
        assert np.abs(got[sl] - want).max() <= 2e-5 * np.abs(want).max()
        S_got = state[slots[s], :A * size].cpu().numpy().reshape(heads, size, size).transpose(0, 2, 1)   # [h][j][i] in the slot
        assert np.abs(S_got - S).max() <= 2e-5 * np.abs(S).max()
    assert float(state[1].abs().max()) == 0.0 and float(state[:, A * size:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_token_shift_reads_and_leaves_the_last_row(dtype):
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(1)
    d, off = 40, 13
    h = P.round_bf16(rng.standard_normal((12, d)))
    mu = rng.uniform(0, 1, (5, d))
    prev = P.round_bf16(rng.standard_normal((3, d)))
    state = torch.zeros((3, off + d), device="cuda")
    state[:, off:] = _t(prev)
    ctx = _ctx([7, 1, 4], [5, 9, 0], [1, 2, 0])
    out = kernels.wkv_shift_mix(_t(h, dtype), _t(mu), state, off, ctx).float().cpu().numpy()
    tol = 1e-6 if dtype == "float32" else 1e-2
    for s, (a, b, slot) in enumerate([(0, 7, 1), (7, 8, 2), (8, 12, 0)]):
        for m in range(5):
            want = P.token_shift(h[a:b], mu[m], first=prev[slot])
            assert np.abs(out[m, a:b] - want).max() <= tol * 4
        assert np.array_equal(state[slot, off:].cpu().numpy(), h[b - 1].astype(np.float32))
    assert float(state[:, :off].abs().max()) == 0.0


def test_gate_norm_unary_and_post_norm():
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(2)
    heads, size, n = 3, 20, 9
    o, g = rng.standard_normal((n, heads * size)) * 3, rng.standard_normal((n, heads * size))
    gain = rng.uniform(0.5, 1.5, heads * size)
    y = kernels.wkv_gate_norm(_t(o), _t(g), _t(gain), 1e-5, heads, size, torch.float32).cpu().numpy()
    want = P.rms_unit(o.reshape(n, heads, size), 1e-5).reshape(n, -1) * gain * P.silu(g)
    assert np.abs(y - want).max() <= 1e-5
    x = rng.standard_normal((n, 50))
    assert np.abs(kernels.unary(_t(x), "relu2", torch.float32).cpu().numpy() - np.maximum(x, 0) ** 2).max() <= 1e-6
    assert np.abs(kernels.unary(_t(x), "tanh", torch.float32).cpu().numpy() - np.tanh(x)).max() <= 1e-6
    low, w2 = rng.standard_normal((n, 5)) * 2, P.round_bf16(rng.standard_normal((37, 5)))
    for dt in ("float32", "bfloat16"):
        z = kernels.wkv_decay_outer(_t(low), _t(w2, dt)).cpu().numpy()
        assert np.abs(z - np.tanh(low) @ w2.T).max() <= 1e-5
    xs, ys, g1, g2 = rng.standard_normal((n, 50)), rng.standard_normal((n, 50)) * 4, rng.uniform(.5, 2, 50), rng.uniform(.5, 2, 50)
    xt, out = _t(xs), torch.empty((n, 50), device="cuda")
    kernels.rmsnorm_add(xt, _t(ys), _t(g1), 1e-6, out=out, gain2=_t(g2), eps2=1e-3)
    want_x = xs + P.rmsnorm(ys, g1, 1e-6)
    assert np.abs(xt.cpu().numpy() - want_x).max() <= 1e-5
    assert np.abs(out.cpu().numpy() - P.rmsnorm(want_x, g2, 1e-3)).max() <= 1e-5


def _paged(k, v, page, n_pages, order_seed):
    """Keys [T, G, dk] and values [T, G, dv] laid into pages in a shuffled order."""
    import torch
    T, G, dk = k.shape
    dv = v.shape[2]
    need = -(-T // page)
    ids = np.random.default_rng(order_seed).permutation(n_pages)[:need]
    kc, vc = np.full((n_pages, G, page, dk), np.nan), np.full((n_pages, G, page, dv), np.nan)
    for t in range(T):
        kc[ids[t // page], :, t % page] = k[t]
        vc[ids[t // page], :, t % page] = v[t]
    return kc, vc, ids


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv", [(4, 1, 96, 96), (4, 2, 16, 24), (6, 1, 8, 4), (2, 2, 32, 64), (3, 1, 10, 6),
                                       (8, 2, 64, 64), (40, 2, 16, 16)])
def test_biased_attention_far_keys_and_page_borders(dtype, H, G, dk, dv):
    """One key far back is made to stand out (its score beats the distance bias); it sits just
    before or just after a page border, and the query is a prompt row or a single decoded token
    whose context is cut into chunks.  Unused pages hold NaN.  The shapes reach every kernel
    that takes the bias: tensor cores (head sizes in steps of 16, values as wide as keys, in
    bfloat16), the CUDA-core tiles (multiples of 4, values of their own size, float32), and one
    warp per row (any size)."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(H * 100 + dk)
    T, page = 700, 16
    scale = 0.4
    slopes = P.head_slopes(H)
    for far in (31, 32, 255, 256, 0, 511):
        q = P.round_bf16(rng.standard_normal((T, H * dk)))
        k = P.round_bf16(rng.standard_normal((T, G * dk)))
        v = P.round_bf16(rng.standard_normal((T, G * dv)))
        # the last query looks for key `far`; on the last head (the smallest slope) its score
        # beats the distance bias and every other key
        kf = k[far].reshape(G, dk)
        kf = P.round_bf16(kf / np.linalg.norm(kf, axis=1, keepdims=True) * np.sqrt(dk))
        q[-1] = P.round_bf16(np.repeat(kf, H // G, axis=0).reshape(-1) * 6.0)
        k[far] = (kf * 4.0).reshape(-1)
        want = P.biased_attention(q, k, v, H, G, dk, dv, scale, slopes)
        kc, vc, ids = _paged(k.reshape(T, G, dk), v.reshape(T, G, dv), page, 64, far)
        table = np.full((1, 50), -1)
        table[0, :len(ids)] = ids
        tol = 2e-5 if dtype == "float32" else 2e-2
        for n_new in (1, 60):            # the last token decoded alone; the last 60 as a portion
            ctx = _ctx([n_new], [T - n_new])
            out = torch.empty((n_new, H * dv), dtype=getattr(torch, dtype), device="cuda")
            kernels.attention(out, _t(q[T - n_new:], dtype), _t(kc, dtype), _t(vc, dtype), ctx, _t(table, "int32"), H, G, dk,
                              0, scale, score_slopes=_t(slopes), v_head_dim=dv, exact_weights=True)
            got = out.float().cpu().numpy()
            assert np.isfinite(got).all()
            assert np.abs(got - want[T - n_new:]).max() <= tol * np.abs(want).max(), (far, n_new)
        # the far key carries the last row's last head: without it the result is another
        assert np.abs(want[-1].reshape(H, dv)[H - 1] - v[far].reshape(G, dv)[G - 1]).max() < 0.05 * np.abs(v[far]).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_qk_norm_temperature_and_cache_write(dtype):
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(6)
    H, G, dk, dv, page = 3, 2, 8, 12, 4
    n_new, start = [5, 1, 2], [3, 10, 0]
    ctx = _ctx(n_new, start)
    n = sum(n_new)
    qkv = rng.standard_normal((n, H * dk + G * dk + G * dv)) * 2
    gq, gk = rng.uniform(.5, 1.5, H * dk), rng.uniform(.5, 1.5, G * dk)
    table = np.array([[5, 1, -1], [0, 2, 7], [3, -1, -1]])
    tdt = getattr(torch, dtype)
    kc = torch.full((8, G, page, dk), float("nan"), dtype=tdt, device="cuda")
    vc = torch.full((8, G, page, dv), float("nan"), dtype=tdt, device="cuda")
    q = torch.empty((n, H * dk), dtype=tdt, device="cuda")
    kernels.qknorm_append(q, _t(qkv), _t(gq), _t(gk), 1e-5, 0.7, 3, ctx.positions, ctx.token_req, _t(table, "int32"),
                          kc, vc, H, G, dk, dv)
    pos = ctx.positions.cpu().numpy()
    want_q = P.rmsnorm(qkv[:, :H * dk], gq, 1e-5) * P.query_temperature(pos, 0.7, 3)[:, None]
    want_k = P.rmsnorm(qkv[:, H * dk:H * dk + G * dk], gk, 1e-5)
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert np.abs(q.float().cpu().numpy() - want_q).max() <= tol * np.abs(want_q).max()
    req = ctx.token_req.cpu().numpy()
    written = 0
    for t in range(n):
        pg, sl = table[req[t], pos[t] // page], pos[t] % page
        assert np.abs(kc[pg, :, sl].float().cpu().numpy().reshape(-1) - want_k[t]).max() <= tol * 4
        assert np.abs(vc[pg, :, sl].float().cpu().numpy().reshape(-1) - qkv[t, H * dk + G * dk:]).max() <= tol * 8
        written += 1
    assert int(torch.isfinite(kc.float()).sum()) == written * G * dk      # nothing else was touched


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,on,d,f", [(8, 1, "input", 36, 28), (5, 3, "input", 40, 24), (4, 4, "output", 72, 100),
                                          (40, 2, "input", 64, 30), (3, 2, "input", 200, 136)])
def test_routed_experts(dtype, E, top, on, d, f):
    """Widths that are and are not multiples of 8 (the tensor-core tiles want 16-byte rows; the
    others run on the CUDA cores), feed-forward sizes that do not fill a tile."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(E)
    n = 77
    h = P.round_bf16(rng.standard_normal((n, d)))
    w = {"router": rng.standard_normal((E, d))}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"] = (P.round_bf16(rng.standard_normal((f, d)) / 6) for _ in range(2))
        w[f"e{e}.down"] = P.round_bf16(rng.standard_normal((d, f)) / 5)
    idx_w, wt_w = P.route(h, w["router"], top)
    tdt = getattr(torch, dtype)
    idx, wt = kernels.moe_route(_t(h, dtype), _t(w["router"]), top)
    assert np.array_equal(idx.cpu().numpy(), idx_w)
    assert np.abs(wt.cpu().numpy() - wt_w).max() <= 1e-5
    gu = torch.stack([torch.cat([_t(w[f"e{e}.gate"], dtype), _t(w[f"e{e}.up"], dtype)]) for e in range(E)]).contiguous()
    dn = torch.stack([_t(w[f"e{e}.down"], dtype) for e in range(E)]).contiguous()
    offsets, perm = kernels.moe_sort(idx, E)
    o, p = offsets.cpu().numpy(), perm.cpu().numpy()
    assert o[0] == 0 and o[-1] == n * top and sorted(p.tolist()) == list(range(n * top))
    flat = idx_w.reshape(-1)
    for e in range(E):
        assert (flat[p[o[e]:o[e + 1]]] == e).all()
    act = kernels.moe_gemm(_t(h, dtype), gu, offsets, perm, wt, top, gated=True, scale_in=on == "input")
    y = kernels.moe_combine(kernels.moe_gemm(act, dn, offsets, perm, wt, top, gated=False, scale_out=on == "output"), top)
    if on == "input":
        want = P.moe_ff(h, w, "", E, top)
    else:
        want = np.zeros((n, d))
        for t in range(n):
            for e, s in zip(idx_w[t], wt_w[t]):
                q = f"e{int(e)}."
                want[t] += s * ((P.silu(h[t] @ w[q + "gate"].T) * (h[t] @ w[q + "up"].T)) @ w[q + "down"].T)
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert np.abs(y.cpu().numpy() - want).max() <= tol * np.abs(want).max()
