"""The Nutizen design in the engine against its plain implementation (tests/plain/nutizen_plain.py).

Small configurations of their own, random weights whose values are bfloat16 numbers (so both
dtypes load the same model): each mechanism's kernel alone, whole prompts, prompts against
token-by-token decoding, portions down to two tokens, unequal batches, slots and pages that
are used again, keys far away, at page borders and just inside and outside a window that one
score makes stand out, sinks that take a visible share, the first tokens, long decoding through CUDA
graphs, and greedy generation through the scheduler.
"""
import numpy as np
import pytest

from helpers import write_model_dir
from plain import nutizen_plain as P
from test_gpu_sozarax import _ctx, _paged, _t, check_rows, engine_for, run_cut

pytestmark = pytest.mark.gpu


def _mix(heads, dim, vdim, q_rank, kv_rank, scale, window=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(ff, limit, experts, top, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def _layer(mixer, mlp):
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


# Every size differs from layer to layer.  A: latents whose size suits every vector width; a
# reader whose window is wider than its writer's; a window wider than a chunk of decoded keys.
CFG_A = {
    "architecture": "Nutizen", "vocab": 96, "width": 64, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5}, "streams": 2,
    "layers": [
        _layer(_mix(4, 16, 24, 40, 32, 0.3, window=40), {"kind": "dense", "ff": 80}),
        _layer(_mix(2, 32, 16, 24, 48, 0.2, window=24), _moe(24, 1.2, 4, 2, shared=(40, 0.8))),
        _layer(_mix(3, 8, 12, 16, 48, 0.4, window=56, kv_from=1), _moe(16, 2.0, 5, 1)),
        _layer(_mix(2, 16, 8, 32, 48, 0.25, window=24, kv_from=1), None),
        _layer(_mix(4, 8, 8, 16, 16, 0.35, window=300), {"kind": "dense", "ff": 40}),
    ],
}
# B: sizes that fit no vector width or tile; one stream; a reader without a window.
CFG_B = {
    "architecture": "Nutizen", "vocab": 61, "width": 50, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6}, "streams": 1,
    "layers": [
        _layer(_mix(3, 10, 6, 7, 10, 0.5, window=17), _moe(7, 0.9, 3, 3, shared=(9, 1.5))),
        _layer(_mix(5, 3, 5, 9, 22, 0.6, window=5), {"kind": "dense", "ff": 13}),
        _layer(_mix(1, 12, 7, 5, 10, 0.3, kv_from=0), _moe(11, 1.0, 2, 1, shared=(5, 0.7))),
    ],
}
# C: no ``streams`` key (one plain residual stream), a layer without a window, many heads on one latent.
CFG_C = {
    "architecture": "Nutizen", "vocab": 70, "width": 48, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_mix(12, 4, 4, 20, 24, 0.5), _moe(12, 1.1, 6, 4)),
        _layer(_mix(2, 24, 20, 12, 8, 0.2, window=9), None),
        _layer(_mix(6, 8, 16, 28, 24, 0.45, window=33, kv_from=0), {"kind": "dense", "ff": 24}),
    ],
}
# D: five streams, a window of one (a token sees itself alone) and one of two.
CFG_D = {
    "architecture": "Nutizen", "vocab": 50, "width": 32, "embedding": {"scale": 1.5}, "norm": {"eps": 1e-5}, "streams": 5,
    "layers": [
        _layer(_mix(2, 8, 8, 8, 12, 0.4, window=1), _moe(8, 1.0, 2, 2, shared=(8, 1.0))),
        _layer(_mix(3, 4, 12, 12, 20, 0.5, window=2), {"kind": "dense", "ff": 16}),
    ],
}
CFGS = {"A": (CFG_A, 31), "B": (CFG_B, 32), "C": (CFG_C, 33), "D": (CFG_D, 34)}


def make_model(tmp_path, name):
    cfg, seed = CFGS[name]
    w = P.random_weights(cfg, seed, qk_boost=3.0)
    d = write_model_dir(str(tmp_path / f"nutizen_{name}"), cfg,
                        {k: (np.asarray(v, dtype=np.float32) if v.dtype != np.int32 else v) for k, v in w.items()})
    return cfg, w, d


# ---- whole models --------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompt_and_every_way_of_cutting(tmp_path, name, dtype):
    cfg, w, d = make_model(tmp_path, name)
    rng = np.random.default_rng(5)
    ids = rng.integers(0, cfg["vocab"], size=150).tolist()
    taps = []
    want = P.forward(w, cfg, ids, taps)
    eng = engine_for(d, dtype)
    try:
        got_taps = []
        eng.model.tap = lambda i, x: got_taps.append(x.detach().float().cpu().numpy().copy())
        whole = run_cut(eng, ids, [len(ids)])
        eng.model.tap = None
        check_rows(whole, want, dtype, f"{name} whole")
        for i, (g, t) in enumerate(zip(got_taps, taps)):      # the residual stream after every layer
            assert np.abs(g - t).max() <= (1e-4 if dtype == "float32" else 1e-1) * np.abs(t).max(), (name, i)
        check_rows(run_cut(eng, ids[:3], [3]), want[:3], dtype, f"{name} first tokens")
        check_rows(run_cut(eng, ids[:1], [1]), want[:1], dtype, f"{name} one token")
        check_rows(run_cut(eng, ids, [len(ids) - 70, 1]), want, dtype, f"{name} prompt then decode")
        check_rows(run_cut(eng, ids[:70], [1]), want[:70], dtype, f"{name} decode from the start")
        for cuts in ([2], [3, 2, 37, 16, 5, 2, 64, 1], [17], [16, 16, 1, 31, 2]):
            got = run_cut(eng, ids, cuts)
            check_rows(got, want, dtype, f"{name} portions {cuts}")
            if dtype == "float32":
                assert np.abs(got - whole).max() <= 1e-5 * np.abs(want).max(), cuts
        eng.cache.audit()
    finally:
        eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_batches_and_reuse_of_slots_and_pages(tmp_path, name, dtype):
    """Four requests of unequal length in one batch, portions of some beside single tokens of
    others, then new requests in the slots and pages that the finished ones gave back; a pool
    that holds little more than what is live."""
    from kllm_b200.engine.step import StepEntry
    cfg, w, d = make_model(tmp_path, name)
    rng = np.random.default_rng(9)
    lens = [37, 90, 5, 64, 21, 50]
    seqs = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lens]
    want = [P.forward(w, cfg, s) for s in seqs]
    eng = engine_for(d, dtype, num_blocks=20, max_batch=4)
    try:
        got = [np.zeros_like(x) for x in want]
        fed = [0] * len(seqs)
        caches, queue = {}, list(range(len(seqs)))
        sizes = [3, 1, 16, 2, 29, 1, 7]
        turn, slots_seen, pages_seen = 0, [], []
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
            pages_seen += [p for c in caches.values() for t in c.tables for p in t if p >= 0]
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


@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding(tmp_path, name):
    """A short prompt and then hundreds of single tokens: every window passes over decoded tokens,
    the widest one's keys are cut into chunks that are merged with the sink, pages come and go."""
    cfg, w, d = make_model(tmp_path, name)
    rng = np.random.default_rng(3)
    ids = rng.integers(0, cfg["vocab"], size=640).tolist()
    want = P.forward(w, cfg, ids)
    eng = engine_for(d, "float32", max_seq=704, num_blocks=44)
    try:
        check_rows(run_cut(eng, ids, [9, 1]), want, "float32", "long decoding")
        check_rows(run_cut(eng, ids, [333, 2, 1]), want, "float32", "a long prompt, then decoding")
    finally:
        eng.close()


def test_greedy_generation_through_the_scheduler(tmp_path):
    """``Engine.generate`` (scheduler, sampler, pipelined steps: the experts' table is asked with
    ids that are still on the device) on several prompts at once against greedy decoding with the
    plain implementation."""
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
            assert out[k] == best or z[best] - z[out[k]] < 1e-4 * np.abs(z).max(), (len(p), k)
            ids.append(out[k])


def test_replay_program(tmp_path):
    """bin/trace_run on a model of this design: whole, decode, portions and mixed batches of up
    to four live requests in a pool as small as the trace allows."""
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

def latent_heads_attention(q, c, H, R, scale, window, sink):
    """H heads over one key/value head whose keys and values are both the rows of c [T, R];
    q [T, H * R]; plain softmax with a sink."""
    T = q.shape[0]
    vis = P.window_mask(T, window)
    out = np.zeros((T, H, R))
    for h in range(H):
        out[:, h] = P.softmax_with_sink(q[:, h * R:(h + 1) * R] @ c.T * scale, vis, sink[h]) @ c
    return out.reshape(T, H * R)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,R,window", [(4, 32, 64), (3, 48, 300), (8, 128, 0), (5, 10, 33), (2, 6, 7), (72, 16, 40),
                                        (2, 320, 50), (4, 256, 100), (20, 192, 0), (3, 144, 20)])
def test_sink_attention_far_keys_window_edges_and_page_borders(dtype, H, R, window):
    """The last query looks for one key: far back, just before or after a page border, the first
    key its window keeps (distance window - 1) or the one just outside (distance window), which
    must then count for nothing.  The sinks are large enough to take a visible share.  The query
    is a prompt row or a single decoded token (whose keys are cut into chunks where the window is
    wide).  Unused pages hold NaN.  Shapes for every kernel that takes a sink."""
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(H * 100 + R)
    T, page, scale = 700, 16, 0.4
    sink = rng.normal(0.0, 1.0, H) + 2.0
    dists = [1, 15, 16, 17, 255, 256, 699] if not window else [window - 1, window, window - 2, 1, 16]
    for dist in dists:
        far = T - 1 - dist
        q = P.round_bf16(rng.standard_normal((T, H * R)))
        c = P.round_bf16(rng.standard_normal((T, R)))
        cf = P.round_bf16(c[far] / np.linalg.norm(c[far]) * np.sqrt(R))
        q[-1] = P.round_bf16(np.tile(cf, H) * 5.0)
        c[far] = cf * 4.0
        want = latent_heads_attention(q, c, H, R, scale, window, sink)
        kc, _, ids = _paged(c.reshape(T, 1, R), c.reshape(T, 1, R), page, 64, dist)
        table = np.full((1, 50), -1)
        table[0, :len(ids)] = ids
        tol = 2e-5 if dtype == "float32" else 2e-2
        store = _t(kc, dtype)
        for n_new in (1, 60):
            ctx = _ctx([n_new], [T - n_new])
            out = torch.empty((n_new, H * R), dtype=getattr(torch, dtype), device="cuda")
            kernels.attention(out, _t(q[T - n_new:], dtype), store, store, ctx, _t(table, "int32"), H, 1, R, window, scale,
                              sinks=_t(sink), exact_weights=True)
            got = out.float().cpu().numpy()
            assert np.isfinite(got).all()
            assert np.abs(got - want[T - n_new:]).max() <= tol * np.abs(want).max(), (dist, n_new)
        seen = not window or dist < window
        hit = np.abs(want[-1].reshape(H, R) - c[far]).max() < 0.05 * np.abs(c[far]).max()
        assert hit == seen, (dist, window)          # the far key carries the last row, or is not seen at all


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("S,d", [(1, 40), (2, 64), (3, 50), (5, 300), (16, 24)])
def test_residual_streams_step(dtype, S, d):
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(S * 7 + d)
    n = 11
    x0, y1, y2 = ((rng.standard_normal((n, d)) * 3).astype(np.float32).astype(np.float64) for _ in range(3))
    w_in, w_out = rng.standard_normal((2, S)), rng.standard_normal((2, S))
    w_mix = np.eye(S) + 0.3 * rng.standard_normal((2, S, S))
    g = rng.uniform(0.5, 1.5, (2, d))
    tdt = getattr(torch, dtype)
    tol = 1e-5 if dtype == "float32" else 1e-2
    xs = torch.full((S, n, d), float("nan"), device="cuda")
    normed = torch.empty((n, d), dtype=tdt, device="cuda")
    kernels.streams_step(xs, init=_t(x0), in_w=_t(w_in[0]), gain=_t(g[0]), eps=1e-5, normed=normed)
    ref = np.stack([x0] * S)
    assert np.abs(xs.cpu().numpy() - ref).max() == 0.0
    want = P.rmsnorm(P.streams_read(ref, w_in[0]), g[0], 1e-5)
    assert np.abs(normed.float().cpu().numpy() - want).max() <= tol * np.abs(want).max()
    # a write, the next read and its norm in one pass
    kernels.streams_step(xs, y=_t(y1), mix=_t(w_mix[0]), out_w=_t(w_out[0]), in_w=_t(w_in[1]), gain=_t(g[1]), eps=1e-6,
                         normed=normed)
    ref = P.streams_write(ref, y1, w_mix[0], w_out[0])
    assert np.abs(xs.cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()
    want = P.rmsnorm(P.streams_read(ref, w_in[1]), g[1], 1e-6)
    assert np.abs(normed.float().cpu().numpy() - want).max() <= tol * np.abs(want).max()
    # the last write and the sum of the streams
    total = torch.empty((n, d), device="cuda")
    kernels.streams_step(xs, y=_t(y2), mix=_t(w_mix[1]), out_w=_t(w_out[1]), total=total)
    ref = P.streams_write(ref, y2, w_mix[1], w_out[1])
    assert np.abs(total.cpu().numpy() - ref.sum(axis=0)).max() <= 1e-5 * np.abs(ref).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_latent_norms_and_cache_write(dtype):
    import torch
    from kllm_b200 import kernels
    rng = np.random.default_rng(6)
    Rq, R, page = 13, 22, 4
    n_new, start = [5, 1, 2], [3, 10, 0]
    ctx = _ctx(n_new, start)
    n = sum(n_new)
    proj = rng.standard_normal((n, Rq + R)) * 2
    gq, gkv = rng.uniform(.5, 1.5, Rq), rng.uniform(.5, 1.5, R)
    table = np.array([[5, 1, -1], [0, 2, 7], [3, -1, -1]])
    tdt = getattr(torch, dtype)
    store = torch.full((8, 1, page, R), float("nan"), dtype=tdt, device="cuda")
    cq = torch.empty((n, Rq), dtype=tdt, device="cuda")
    kernels.latent_norm_append(cq, _t(proj), _t(gq), _t(gkv), 1e-5, ctx.positions, ctx.token_req, _t(table, "int32"), store)
    tol = 1e-5 if dtype == "float32" else 2e-2
    want_q, want_c = P.rmsnorm(proj[:, :Rq], gq, 1e-5), P.rmsnorm(proj[:, Rq:], gkv, 1e-5)
    assert np.abs(cq.float().cpu().numpy() - want_q).max() <= tol * np.abs(want_q).max()
    pos, req = ctx.positions.cpu().numpy(), ctx.token_req.cpu().numpy()
    for t in range(n):
        pg, sl = table[req[t], pos[t] // page], pos[t] % page
        assert np.abs(store[pg, 0, sl].float().cpu().numpy() - want_c[t]).max() <= tol * 4
    assert int(torch.isfinite(store.float()).sum()) == n * R          # nothing else was touched
    # a layer that reads another layer's latents norms its query latent alone
    cq2 = torch.empty((n, Rq), dtype=tdt, device="cuda")
    kernels.latent_norm_append(cq2, _t(proj[:, :Rq]), _t(gq), None, 1e-5, ctx.positions, ctx.token_req, None, None)
    assert torch.equal(cq, cq2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,a,b", [(4, 16, 32), (3, 10, 7), (1, 24, 24), (12, 4, 24)])
def test_products_per_head(dtype, H, a, b):
    from kllm_b200 import kernels
    rng = np.random.default_rng(H + a)
    n = 19
    x = P.round_bf16(rng.standard_normal((n, H * a)))
    w = P.round_bf16(rng.standard_normal((H, b, a)) / 4)
    want = np.einsum("hba,nha->nhb", w.astype(np.float64), x.reshape(n, H, a).astype(np.float64)).reshape(n, H * b)
    tol = 1e-5 if dtype == "float32" else 1e-2
    got = kernels.linear_per_head(_t(x, dtype), _t(w, dtype)).float().cpu().numpy()
    assert np.abs(got - want).max() <= tol * np.abs(want).max()
    got = kernels.linear_per_head(_t(x, dtype), _t(w.transpose(0, 2, 1), dtype), transposed=True).float().cpu().numpy()
    assert np.abs(got - want).max() <= tol * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,top,d,f,fs", [(8, 2, 64, 24, 40), (5, 1, 36, 28, 0), (3, 3, 50, 7, 9), (40, 4, 72, 100, 16)])
def test_table_experts_clamped_activation_and_shared_expert(dtype, E, top, d, f, fs):
    """The experts a table gives (ids on the host's side of the step and ids that are still on the
    device), the clamped activation with inputs beyond the limit on both sides, and the shared
    expert with its gate."""
    import torch
    import types
    from kllm_b200.parts.moe import RoutedExperts
    from kllm_b200.parts.spec import BuildEnv, PartSpec
    rng = np.random.default_rng(E * 10 + top)
    n, V, limit = 77, 30, 0.6
    h = P.round_bf16(rng.standard_normal((n, d)) * 2)
    mlp = {"kind": "moe", "expert": {"ff": f, "limit": limit}, "router": {"experts": E, "top": top}}
    w = {"table": np.stack([rng.permutation(E)[:top] for _ in range(V)]).astype(np.int32)}
    names = [f"e{e}." for e in range(E)] + (["shared."] if fs else [])
    for p in names:
        ff = fs if p == "shared." else f
        w[p + "gate"], w[p + "up"] = (P.round_bf16(rng.standard_normal((ff, d)) / 4) for _ in range(2))
        w[p + "down"] = P.round_bf16(rng.standard_normal((d, ff)) / 5)
    shared = None
    if fs:
        mlp["shared"] = {"ff": fs, "limit": 0.9}
        w["shared.sg"] = P.round_bf16(rng.standard_normal((1, d)) / 3)
        shared = {"ff": fs, "activation": "clamped", "limit": 0.9, "alpha": 1.702,
                  "tensors": {"gate": "shared.gate", "up": "shared.up", "down": "shared.down", "gate_logit": "shared.sg"}}
    ids = rng.integers(0, V, size=n)
    want = P.feed_forward(h, ids, w, "", mlp)
    part = RoutedExperts(PartSpec("routed_experts", "", {
        "hidden": d, "experts": E, "top": top, "expert_ff": f, "routing": "table", "table_tensor": "table", "vocab": V,
        "weight_on": "output", "activation": "clamped", "limit": limit, "alpha": 1.702, "shared": shared,
        "expert_tensors": "e{e}.{m}"}), BuildEnv(getattr(torch, dtype), torch.device("cuda"), d, 1 << 20))
    part.bind({s.name: _t(w[s.name], {"compute": dtype, "float32": "float32", "int32": "int32"}[s.store])
               for s in part.tensor_specs()})
    tol = 2e-5 if dtype == "float32" else 2e-2
    got = part.forward(_t(h, dtype), types.SimpleNamespace(token_ids=_t(ids, "int32"), last_token=None)).cpu().numpy()
    assert np.abs(got - want).max() <= tol * np.abs(want).max()
    # the same ids, every third one still on the device in a request slot
    slots = rng.permutation(n)
    dev_ids = np.where(np.arange(n) % 3 == 0, -(slots + 1), ids)
    last = np.zeros(n, dtype=np.int32)
    last[slots] = ids
    got2 = part.forward(_t(h, dtype), types.SimpleNamespace(token_ids=_t(dev_ids, "int32"),
                                                            last_token=_t(last, "int32"))).cpu().numpy()
    assert np.array_equal(got, got2)
    # a step whose ids the host knows and that is large enough is sorted by the host and runs the
    # library's batched products over blocks of rows: the same numbers up to the order of the sums
    part.planned_rows = 1
    known = types.SimpleNamespace(token_ids=_t(ids, "int32"), last_token=None, host_token_ids=ids.astype(np.int32))
    assert (E, top) not in ((8, 2), (3, 3)) or part._plan(known, n) is not None       # those do take that route
    got3 = part.forward(_t(h, dtype), known).cpu().numpy()
    assert np.abs(got3 - want).max() <= tol * np.abs(want).max()
    assert np.abs(got3 - got).max() <= (1e-5 if dtype == "float32" else 2e-2) * np.abs(want).max()


# ---- configurations drawn at random -----------------------------------------------------------------

def draw_config(seed):
    """Sizes that are and are not multiples of what the kernels like, every branch of the design."""
    rng = np.random.default_rng(7000 + seed)
    width = int(rng.choice([24, 40, 50, 64, 72, 96, 128, 136]))
    n_layers = int(rng.integers(2, 6))
    streams = int(rng.choice([0, 1, 2, 3, 4, 6, 9]))
    layers, owners = [], []
    for i in range(n_layers):
        src = None
        if owners and rng.random() < 0.4:
            src = int(rng.choice(owners))
        R = layers[src]["mixer"]["kv_rank"] if src is not None else int(rng.choice([8, 10, 16, 24, 32, 48, 64, 80, 96, 112, 128,
                                                                                    144, 160, 192, 256]))
        window = None if rng.random() < 0.2 else int(rng.choice([1, 3, 16, 17, 40, 64, 100, 130]))
        m = _mix(int(rng.choice([1, 2, 3, 4, 6, 8, 12, 20])), int(rng.choice([4, 6, 8, 16, 24, 32])),
                 int(rng.choice([4, 5, 8, 16, 20, 40])), int(rng.choice([6, 8, 16, 24, 40])), R,
                 float(rng.choice([0.2, 0.35, 0.5])), window=window, kv_from=src)
        if src is None:
            owners.append(i)
        kind = rng.choice(["dense", "moe", "moe_shared", "none"])
        if kind == "dense":
            mlp = {"kind": "dense", "ff": int(rng.choice([16, 24, 50, 64]))}
        elif kind == "none":
            mlp = None
        else:
            E = int(rng.choice([2, 3, 4, 8]))
            mlp = _moe(int(rng.choice([8, 12, 24, 33])), float(rng.choice([0.7, 1.0, 2.5])), E, int(rng.integers(1, E + 1)),
                       shared=(int(rng.choice([8, 20, 32])), float(rng.choice([0.5, 1.25]))) if kind == "moe_shared" else None)
        layers.append(_layer(m, mlp))
    cfg = {"architecture": "Nutizen", "vocab": int(rng.choice([61, 97, 128, 300])), "width": width,
           "embedding": {"scale": float(rng.choice([1.0, 2.0, 5.5]))}, "norm": {"eps": float(rng.choice([1e-5, 1e-6]))},
           "layers": layers}
    if streams:
        cfg["streams"] = streams
    return cfg


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(12))
def test_drawn_configuration(tmp_path, seed, dtype):
    """A whole prompt, most of it and then its last tokens one by one, and three requests decoding side
    by side, for a configuration drawn at random."""
    from kllm_b200.engine.step import StepEntry
    cfg = draw_config(seed)
    w = P.random_weights(cfg, 900 + seed, qk_boost=2.0)
    d = write_model_dir(str(tmp_path / "m"), cfg,
                        {k: (np.asarray(v, dtype=np.float32) if v.dtype != np.int32 else v) for k, v in w.items()})
    rng = np.random.default_rng(seed)
    page = int(rng.choice([16, 32, 64]))
    eng = engine_for(d, dtype, max_seq=256, block_size=page, num_blocks=1024 // page)
    what = f"drawn {seed} {dtype}"
    try:
        ids = rng.integers(0, cfg["vocab"], size=int(rng.integers(140, 200))).tolist()
        want = P.forward(w, cfg, ids)
        check_rows(run_cut(eng, ids, [len(ids)]), want, dtype, what + " whole")
        check_rows(run_cut(eng, ids, [len(ids) - 9, 1]), want, dtype, what + " prompt then decode")
        check_rows(run_cut(eng, ids, [5, 2, 50, 1, 1, 33]), want, dtype, what + " portions")
        seqs = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in (9, 33, 150)]
        wants = [P.forward(w, cfg, s) for s in seqs]
        reqs = [eng.cache.open() for _ in seqs]
        eng.runner.run([StepEntry(r, s[:-4], []) for r, s in zip(reqs, seqs)])
        for back in range(4, 0, -1):
            got = eng.runner.run([StepEntry(r, [s[-back]], [0]) for r, s in zip(reqs, seqs)]).float().cpu().numpy()
            for j, (s, wj) in enumerate(zip(seqs, wants)):
                check_rows(got[j:j + 1], wj[len(s) - back:len(s) - back + 1], dtype, what + f" batch of 3, request {j}")
        for r in reqs:
            eng.cache.close(r)
        eng.cache.audit()
    finally:
        eng.close()
