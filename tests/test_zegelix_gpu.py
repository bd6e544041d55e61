"""The Zegelix decoder on the GPU against the plain implementation (``plain_zegelix.py``): each mechanism's kernels
alone, then whole models through the step function, the cache and the scheduler, in float32 and in bfloat16."""
import types

import numpy as np
import pytest
import torch

import plain_zegelix as plain
import zegelix_cases as zc

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = ["Z1", "Z2", "Z3"]
DEV = "cuda:0"
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("zegelix")
    return {n: zc.make_folder(base, n) for n in NAMES}


@pytest.fixture(scope="module")
def models(folders):
    from coheryn_ai_studio_b200.engine import load_model
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = load_model(folders[name], dtype)[1]
        return cache[(name, dtype)]
    return get


def vocab(name):
    return zc.CASES[name][0]["vocab"]


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=dtype).to(DEV)


def bf(a):
    """A float64 array rounded to bfloat16 values."""
    return plain.round_bf16(np.asarray(a, dtype=np.float64))


def host(t):
    return t.float().cpu().numpy().astype(np.float64)


def runtime(dtype):
    from coheryn_ai_studio_b200.parts.base import Runtime
    return Runtime(TORCH[dtype], torch.device(DEV))


def bind(part, W, prefix, dtype):
    """Hand a part its tensors from a dict of float64 arrays, kept as the loader keeps them."""
    from coheryn_ai_studio_b200.weights.loader import kept_dtype
    specs = part.tensor_specs()
    part.bind({n: dev(W[prefix + n]).to(kept_dtype(s, TORCH[dtype], TORCH[dtype])).contiguous() for n, s in specs.items()})
    return part


class Pages:
    """Hand-made caches for one window attention with block means: requests whose pages (of positions, and of blocks) are
    handed out in scrambled orders, full of noise, and steps over any runs of their positions."""

    def __init__(self, lengths, G, dk, dv, page, pool, dtype, seed=0):
        from coheryn_ai_studio_b200.parts.base import LayerCache
        self.page = page
        pages = [-(-n // page) for n in lengths]
        rng = np.random.default_rng(seed)
        self.tables = []
        for _ in range(2):
            order = rng.permutation(sum(pages) + 3)
            tab = np.full((len(lengths), max(pages) + 1), -1, dtype=np.int32)
            at = 0
            for r, n in enumerate(pages):
                tab[r, :n] = order[at:at + n]
                at += n
            self.tables.append(tab)
        n_pages = sum(pages) + 3
        noise = lambda *shape: torch.randn(shape, device=DEV).mul_(7.0).to(TORCH[dtype])
        self.k, self.v = noise(n_pages, G, page, dk), noise(n_pages, G, page, dv)
        parts = [LayerCache(kind="paged", group=0, page_size=page, k=self.k, v=self.v, writes=True)]
        if pool is not None:
            rows = -(-page // pool)
            self.pk, self.pv = noise(n_pages, G, rows, dk), noise(n_pages, G, rows, dv)
            parts.append(LayerCache(kind="paged", group=1, page_size=page, k=self.pk, v=self.pv, writes=True))
            self.cache = LayerCache(kind="several", parts=parts, writes=True)
        else:
            self.pk = self.pv = None
            self.cache = parts[0]

    def step(self, runs):
        """``runs``: (request, first position, tokens) in batch order; the requests' lengths are first + tokens."""
        req = np.concatenate([np.full(n, i) for i, (_, _, n) in enumerate(runs)]).astype(np.int32)
        pos = np.concatenate([np.arange(s, s + n) for _, s, n in runs]).astype(np.int32)
        cu = np.concatenate([[0], np.cumsum([n for _, _, n in runs])]).astype(np.int32)
        tabs = [np.stack([t[r] for r, _, _ in runs]) for t in self.tables]
        slots = np.concatenate([self.tables[0][r][np.arange(s, s + n) // self.page] * self.page + np.arange(s, s + n) % self.page
                                for r, s, n in runs]).astype(np.int32)
        kv = [s + n for _, s, n in runs]
        return types.SimpleNamespace(
            num_requests=len(runs), num_tokens=int(cu[-1]), token_req=dev(req, torch.int32), positions=dev(pos, torch.int32),
            cu_q=dev(cu, torch.int32), kv_lens=dev(kv, torch.int32), block_tables=[dev(t, torch.int32) for t in tabs],
            slots=[dev(slots, torch.int32), None], q_lens=[n for _, _, n in runs], kv_lens_host=kv,
            max_q_len=max(n for _, _, n in runs), max_kv_len=max(kv), prior_positions_settled=True, tail=None, tail_rows=None)


def state_step(runs, slots):
    """A step without pages: ``runs`` as above; ``slots``: the state slot of every request."""
    req = np.concatenate([np.full(n, i) for i, (_, _, n) in enumerate(runs)]).astype(np.int32)
    pos = np.concatenate([np.arange(s, s + n) for _, s, n in runs]).astype(np.int32)
    cu = np.concatenate([[0], np.cumsum([n for _, _, n in runs])]).astype(np.int32)
    return types.SimpleNamespace(
        num_requests=len(runs), num_tokens=int(cu[-1]), token_req=dev(req, torch.int32), positions=dev(pos, torch.int32),
        cu_q=dev(cu, torch.int32), state_slots=dev([slots[r] for r, _, _ in runs], torch.int32), tail=None, tail_rows=None)


def cuts(lengths, portions):
    """Steps of a schedule: request r advances by portions[r][k] tokens in its k-th step (requests join in order)."""
    at = [0] * len(lengths)
    steps = []
    k = 0
    while any(a < n for a, n in zip(at, lengths)):
        runs = []
        for r, n in enumerate(lengths):
            ps = portions[r]
            if at[r] < n and k >= r:           # request r joins at step r
                take = min(ps[(k - r) % len(ps)], n - at[r])
                runs.append((r, at[r], take))
                at[r] += take
        steps.append(runs)
        k += 1
    return steps


# ------------------------------------------------------------------------------ the recurrence
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,channels,blocks,taps", [(64, 64, 4, 4), (100, 36, 3, 2), (48, 130, 1, 1), (32, 256, 16, 3)])
def test_gated_linear_recurrence_in_portions_and_decoded(dtype, width, channels, blocks, taps):
    """Two requests in portions of many sizes (across the scan's chunks, down to one token) over state slots full of noise:
    channels whose decay is nearly 1 carry the first tokens' inputs through hundreds of steps."""
    from coheryn_ai_studio_b200.parts.base import LayerCache
    from coheryn_ai_studio_b200.parts.recurrent import GatedLinearRecurrence
    rng = np.random.default_rng(channels)
    r8 = (lambda a: bf(a)) if dtype == "bfloat16" else (lambda a: np.asarray(a, dtype=np.float32).astype(np.float64))
    bs = channels // blocks
    W = {"m.y": r8(rng.normal(0, 0.2, (channels, width))), "m.y.b": r8(rng.normal(0, 0.3, channels)),
         "m.x": r8(rng.normal(0, 0.2, (channels, width))), "m.x.b": r8(rng.normal(0, 0.3, channels)),
         "m.conv": r8(rng.normal(0, 0.5, (channels, taps))), "m.conv.b": r8(rng.normal(0, 0.2, channels)),
         "m.ra": r8(rng.normal(0, 0.3, (blocks, bs, bs))), "m.ra.b": r8(rng.normal(0, 0.5, (blocks, bs))),
         "m.ri": r8(rng.normal(0, 0.3, (blocks, bs, bs))), "m.ri.b": r8(rng.normal(0, 0.5, (blocks, bs))),
         "m.lam": r8(np.linspace(-12.0, 2.0, channels)), "m.o": r8(rng.normal(0, 0.2, (width, channels)))}
    mixer = bind(GatedLinearRecurrence(runtime(dtype), width, channels, blocks, taps), W, "m.", dtype)
    lengths = [331, 45]
    hs = [r8(rng.normal(0, 1.0, (n, width))) for n in lengths]
    hs[0][0] *= 12.0                     # the first token's input is loud: the slow channels still carry it at the end
    want = [plain.gated_linear_recurrence(h, W, "m.", {}) for h in hs]
    silent = plain.gated_linear_recurrence(np.concatenate([hs[0][:1] / 12.0, hs[0][1:]]), W, "m.", {})
    assert np.abs(silent[-1] - want[0][-1]).max() > 0.01 * np.abs(want[0][-1]).max()       # a lost state would show
    state = torch.randn((5, channels * taps), device=DEV) * 3.0
    slots = [3, 1]
    cache = LayerCache(kind="state", state=state, writes=True)
    got = [np.zeros_like(w) for w in want]
    fresh = set()
    for runs in cuts(lengths, [[130, 2, 1, 67, 31, 33, 1, 1, 1, 64], [7, 1, 2, 30, 1]]):
        for r, s, _ in runs:
            if r not in fresh:
                state[slots[r]].zero_()          # what admission does
                fresh.add(r)
        x = dev(np.concatenate([hs[r][s:s + n] for r, s, n in runs]), TORCH[dtype])
        out = host(mixer.forward(x, state_step(runs, slots), cache))
        o = 0
        for r, s, n in runs:
            got[r][s:s + n] = out[o:o + n]
            o += n
    for g, w in zip(got, want):
        tol = 3e-5 if dtype == "float32" else 4e-2
        assert np.abs(g - w).max() <= tol * np.abs(w).max(), np.abs(g - w).max() / np.abs(w).max()


# ------------------------------------------------------------------------------ the router and the experts
@pytest.mark.parametrize("experts,top,bias", [(16, 3, 0.3), (5, 5, 2.0), (3, 1, 0.0), (40, 7, 5.0), (2, 2, 0.1)])
def test_router_takes_the_largest_logits_and_weighs_the_chosen_alone(experts, top, bias):
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(experts * 10 + top)
    T = 70
    z = rng.normal(0, 2.0, (T, experts)).astype(np.float32)
    b = rng.normal(0, bias, experts).astype(np.float32)
    wide = dev(np.concatenate([z, rng.normal(0, 9.0, (T, 2)).astype(np.float32)], axis=1))     # columns behind the logits are not read
    ids, weights = ops.route_select(wide[:, :experts], dev(b), 1, 1, top, 1.0, chosen_softmax=True)
    total = z.astype(np.float64) + b
    order = np.argsort(-total, axis=1, kind="stable")[:, :top]
    chosen = np.take_along_axis(total, order, axis=1)
    e = np.exp(chosen - chosen.max(1, keepdims=True))
    assert np.array_equal(ids.cpu().numpy(), order)
    assert np.abs(host(weights) - e / e.sum(1, keepdims=True)).max() < 2e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,ff,limit,experts,top,shared,T", [(64, 32, 0.7, 6, 2, (48, 2.5), 77), (100, 50, 2.0, 5, 5, None, 33),
                                                                 (128, 64, 1.0, 4, 2, (32, 0.25), 300), (64, 16, 4.0, 3, 1, (16, 1.0), 2)])
def test_expert_mixture_with_a_shared_expert(dtype, width, ff, limit, experts, top, shared, T):
    from coheryn_ai_studio_b200.parts.routed import RoutedExperts
    rng = np.random.default_rng(width + T)
    r8 = (lambda a: bf(a)) if dtype == "bfloat16" else (lambda a: np.asarray(a, dtype=np.float32).astype(np.float64))
    W = {"f.router": r8(rng.normal(0, 0.5, (experts, width))), "f.router.b": r8(rng.normal(0, 1.0, experts))}
    for e in range(experts):
        W[f"f.e{e}.gate"], W[f"f.e{e}.up"] = r8(rng.normal(0, 0.3, (ff, width))), r8(rng.normal(0, 0.3, (ff, width)))
        W[f"f.e{e}.down"] = r8(rng.normal(0, 0.3, (width, ff)))
    mlp = {"expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
        W["f.shared.gate"], W["f.shared.up"] = r8(rng.normal(0, 0.3, (shared[0], width))), r8(rng.normal(0, 0.3, (shared[0], width)))
        W["f.shared.down"], W["f.shared.sg"] = r8(rng.normal(0, 0.3, (width, shared[0]))), r8(rng.normal(0, 0.4, (1, width)))
    part = bind(RoutedExperts(runtime(dtype), width, ff, experts, top, activation="swish_clamped", activation_constant=limit,
                              selection="top_softmax", router_bias=True,
                              shared=dict(size=shared[0], activation_constant=shared[1], gate=True) if shared else None), W, "f.", dtype)
    h = r8(rng.normal(0, 1.0, (T, width)))
    want = plain.expert_mixture(h, W, "f.", mlp)
    got = host(part.forward(dev(h, TORCH[dtype]), None))
    # a near tie of two logits may fall the other way in float32 sums: such rows are left out (there are few)
    z = h @ W["f.router"].T + W["f.router.b"]
    srt = np.sort(z, axis=1)[:, ::-1]
    clear = (srt[:, top - 1] - srt[:, top] > 1e-3) if top < experts else np.ones(T, bool)
    assert clear.mean() > 0.9
    tol = 3e-5 if dtype == "float32" else 3e-2
    assert np.abs(got - want)[clear].max() <= tol * np.abs(want).max()
    # the same rows in another order and beside others: the same bits
    perm = np.random.default_rng(1).permutation(T)
    again = host(part.forward(dev(h[perm], TORCH[dtype]), None))
    assert np.array_equal(again, got[perm]) or T >= 200      # many rows per expert take another product kernel per row count


def test_stream_mixed_with_the_embedding_output():
    from coheryn_ai_studio_b200 import ops
    rng = np.random.default_rng(5)
    T, H, V = 37, 100, 50
    x, table = rng.normal(0, 1, (T, H)).astype(np.float32), bf(rng.normal(0, 1, (V, H)))
    ids = rng.integers(0, V, T)
    for dtype in DTYPES:
        for delta in (None, rng.normal(0, 1, (T, H)).astype(np.float32), rng.normal(0, 1, (3, T, H)).astype(np.float32)):
            got = host(ops.stream_join(dev(x), dev(delta) if delta is not None else None, dev(table, TORCH[dtype]), dev(ids, torch.int32),
                                       2.5, TORCH[dtype]))
            full = x.astype(np.float64) + (0 if delta is None else delta.sum(0) if delta.ndim == 3 else delta)
            want = np.concatenate([full, table[ids] * 2.5], axis=1)
            assert np.abs(got - want).max() <= (1e-5 if dtype == "float32" else 2e-2) * np.abs(want).max()
        got = host(ops.stream_join(dev(x), dev(bf(x), torch.bfloat16), dev(table, torch.bfloat16), dev(ids, torch.int32), None, torch.float32))
        assert np.abs(got[:, :H] - (x + bf(x))).max() < 1e-5 and np.array_equal(got[:, H:], table[ids])


# ------------------------------------------------------------------------------ the attention's kernels
def run_kernels(q, k, v, lengths, steps, size, pool, page, scale, cap, temp, sink, dtype, G):
    """Write k and v through ``pooled_prepare`` (no rotation), keep the block means, attend; rows [sum lengths][H, dv]."""
    from coheryn_ai_studio_b200 import ops
    H, dk, dv = q[0].shape[1], q[0].shape[2], v[0].shape[2]
    pages = Pages(lengths, G, dk, dv, page, pool, dtype, seed=len(steps))
    got = [np.zeros((n, H, dv)) for n in lengths]
    for runs in steps:
        st = pages.step(runs)
        proj = np.concatenate([np.concatenate([q[r][s:s + n].reshape(n, -1), k[r][s:s + n].reshape(n, -1), v[r][s:s + n].reshape(n, -1)], axis=1)
                               for r, s, n in runs])
        qd = ops.pooled_prepare(dev(proj), st.positions, None, 0, None, st.slots[0], pages.k, pages.v, H, G, dk, dv, page, TORCH[dtype])
        if pool is not None:
            ops.pooled_means(pages.k, pages.v, pages.pk, pages.pv, st, 0, 1, G, dk, dv, page, pool)
        out = torch.empty((qd.shape[0], H * dv), dtype=TORCH[dtype], device=DEV)
        ops.pooled_attention(qd, out, pages.k, pages.v, pages.pk, pages.pv, st, 0, 1 if pool is not None else None, H, G, dk, dv, page,
                             size, pool, scale, cap, dev(temp) if temp is not None else None, dev(sink) if sink is not None else None,
                             None, None)
        o = 0
        for r, s, n in runs:
            got[r][s:s + n] = host(out[o:o + n]).reshape(n, H, dv)
            o += n
    return got


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size,pool,page,H,G,dk,dv", [(24, 8, 16, 4, 2, 32, 16), (7, 3, 16, 3, 3, 20, 14), (5, 9, 8, 6, 2, 10, 6),
                                                      (1, 1, 16, 6, 1, 16, 48), (36, 12, 64, 2, 1, 80, 256), (12, None, 16, 2, 2, 8, 8)])
def test_one_key_that_stands_out_at_every_edge(dtype, size, pool, page, H, G, dk, dv):
    """A marked position j*: its key and the queries of ALL rows carry one large component, so a row puts nearly all its
    weight on j* while it sees it as a position, none when it has left the window and its block is not complete behind the
    window, and most of it on the block's mean from the row that first sees the block.  Whole, in portions and decoded."""
    rng = np.random.default_rng(size * 100 + (pool or 0))
    T = 150
    r8 = bf if dtype == "bfloat16" else (lambda a: np.asarray(a, dtype=np.float32).astype(np.float64))
    marks = [0, 70]                             # position 0; the middle of a block and of a page
    q = r8(rng.normal(0, 0.3, (T, H, dk))); k = r8(rng.normal(0, 0.3, (T, G, dk))); v = r8(rng.normal(0, 1.0, (T, G, dv)))
    big = 9.0 * max(1.0, np.sqrt(pool or 1))
    q[:, :, 0] = big
    for j in marks:
        k[j, :, 0] = big
    scale = 0.2
    temp, sink = r8(rng.uniform(0.7, 1.3, H)), r8(rng.normal(0, 1.0, H))
    want = plain.attend_window_and_blocks(q, k, v, size, pool, scale, 25.0, temp, sink, rounder=r8 if dtype == "bfloat16" else (lambda a: a))
    # the weights make the edges show: the last row that sees a mark as a position differs from the next one (unless that one
    # sees the mark's block at once), and the first row that sees the mark's block from the one before it
    shown = 0
    for j in marks:
        edge = j + size - 1
        first = (j // pool) * pool + pool - 1 + size if pool is not None else None
        if first is None or first > edge + 1:
            assert np.abs(want[edge] - want[edge + 1]).max() > 0.2, (j, "window edge")
            shown += 1
        if first is not None and edge + 1 < first < T:
            assert np.abs(want[first] - want[first - 1]).max() > 0.05, (j, "block edge")
            shown += 1
    assert shown or pool == 1
    from coheryn_ai_studio_b200 import ops
    tol = 2e-5 if dtype == "float32" else 3e-2
    for tensor_cores in ((True, False) if dtype == "bfloat16" else (True,)):      # bfloat16 portions: both kernels
        ops.set_pooled_tc(tensor_cores)
        try:
            for steps in ([[(0, 0, T)]], cuts([T], [[40, 1, 1, 1, 17, 2, 1, 3, 64, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1]]), [[(0, t, 1)] for t in range(T)]):
                got = run_kernels([q], [k], [v], [T], steps, size, pool, page, scale, 25.0, temp, sink, dtype, G)[0]
                d = np.abs(got - want).max(axis=(1, 2))
                assert d.max() <= tol * np.abs(want).max(), (tensor_cores, int(d.argmax()), d.max())
        finally:
            ops.set_pooled_tc(True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_takes_weight_per_head_and_carries_no_value(dtype):
    rng = np.random.default_rng(8)
    T, H, G, dk, dv = 30, 4, 2, 16, 16
    r8 = bf if dtype == "bfloat16" else (lambda a: np.asarray(a, dtype=np.float32).astype(np.float64))
    q, k, v = r8(rng.normal(0, 1, (T, H, dk))), r8(rng.normal(0, 1, (T, G, dk))), r8(rng.normal(0, 1, (T, G, dv)))
    sink = np.array([-30.0, 0.0, 6.0, 40.0])
    want = plain.attend_window_and_blocks(q, k, v, 6, 4, 0.25, None, None, sink, rounder=r8 if dtype == "bfloat16" else (lambda a: a))
    got = run_kernels([q], [k], [v], [T], [[(0, 0, T)]], 6, 4, 16, 0.25, None, None, sink, dtype, G)[0]
    assert np.abs(got - want).max() <= (2e-5 if dtype == "float32" else 3e-2) * np.abs(want).max()
    assert np.abs(got[:, 3]).max() < 1e-10 and np.abs(got[:, 0]).max() > 0.1          # a sink far above every score takes all


# ------------------------------------------------------------------------------ the attention mixer
def attention_weights(rng, width, m, r8):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    return {"m.q": r8(rng.normal(0, 0.25, (H * dk, width))), "m.q.b": r8(rng.normal(0, 0.3, H * dk)),
            "m.k": r8(rng.normal(0, 0.25, (G * dk, width))), "m.k.b": r8(rng.normal(0, 0.3, G * dk)),
            "m.v": r8(rng.normal(0, 0.25, (G * dv, width))), "m.v.b": r8(rng.normal(0, 0.3, G * dv)),
            "m.temp": r8(rng.uniform(0.6, 1.5, H)), "m.sink": r8(rng.normal(0, 1.0, H)),
            "m.g": r8(rng.normal(0, 0.25, (H * dv, width))), "m.o": r8(rng.normal(0, 0.25, (width, H * dv)))}


def shape(heads, kv_heads, dim, vdim, rot_dims, base, size, pool, scale=0.2, softcap=10.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"dims": rot_dims, "base": base},
            "mask": {"size": size, "pool": pool}, "scale": scale, "softcap": softcap}


MIXERS = [(shape(4, 2, 32, 16, 16, 1000.0, 24, 8), 64, 16), (shape(3, 3, 20, 14, 12, 77.0, 7, 3), 100, 16),
          (shape(6, 2, 10, 6, 2, 9.0, 5, 9), 40, 8), (shape(6, 1, 16, 48, 16, 10000.0, 1, 1), 64, 16),
          (shape(2, 1, 80, 112, 48, 20000.0, 33, 12), 128, 64), (shape(1, 1, 256, 130, 64, 500.0, 16, 16), 64, 16)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,width,page", MIXERS)
def test_attention_mixer_in_portions_and_decoded(dtype, m, width, page):
    """The whole mixer (projections with biases, rotation of queries, keys and values, block means, factors per head, cap,
    sink, the output turned back, gate, output product) for two requests cut into portions over scrambled pages."""
    from coheryn_ai_studio_b200.config.spec import PartSpec
    from coheryn_ai_studio_b200.parts.attention import PooledWindowAttention
    from coheryn_ai_studio_b200.parts.base import POSITIONS, build_part
    rng = np.random.default_rng(m["dim"] + m["vdim"])
    r8 = bf if dtype == "bfloat16" else (lambda a: np.asarray(a, dtype=np.float32).astype(np.float64))
    W = attention_weights(rng, width, m, r8)
    rt = runtime(dtype)
    pos = build_part(POSITIONS, "position", PartSpec("rope_computed", dict(rotary_dim=m["rot"]["dims"], theta=m["rot"]["base"])), rt)
    mixer = bind(PooledWindowAttention(rt, width, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], window=m["mask"]["size"],
                                       pool=m["mask"]["pool"], qkv_bias=True, rotate_values=True, value_base=m["rot"]["base"],
                                       head_temps=True, softcap=m["softcap"], sink=True, gate=True, position=pos), W, "m.", dtype)
    lengths = [139, 30]
    hs = [r8(rng.normal(0, 1.0, (n, width))) for n in lengths]
    rounder = r8 if dtype == "bfloat16" else (lambda a: a)
    want = [plain.pooled_window_attention(h, range(len(h)), W, "m.", m, rounder=rounder) for h in hs]
    pages = Pages(lengths, m["kv_heads"], m["dim"], m["vdim"], page, m["mask"]["pool"], dtype, seed=width)
    got = [np.zeros_like(w) for w in want]
    for runs in cuts(lengths, [[33, 2, 1, 17, 1, 1, 1, 40, 2, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1], [5, 1, 1, 20, 1]]):
        x = dev(np.concatenate([hs[r][s:s + n] for r, s, n in runs]), TORCH[dtype])
        out = host(mixer.forward(x, pages.step(runs), pages.cache))
        o = 0
        for r, s, n in runs:
            got[r][s:s + n] = out[o:o + n]
            o += n
    for g, w in zip(got, want):
        tol = 3e-5 if dtype == "float32" else 4e-2
        assert np.abs(g - w).max() <= tol * np.abs(w).max(), np.abs(g - w).max() / np.abs(w).max()


# ------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(name, dtype, folders, models):
    for i, n in enumerate([1, 2, 23, 97]):
        seq = zc.prompt(30 + i, n, vocab(name))
        r = zc.noisy_replay(folders[name], dtype, 128, models(name, dtype))
        r.step([("r", seq, list(range(n)))], end=["r"])
        zc.check_rows(r.rows, folders[name], {"r": seq}, dtype, f"whole {n}")


def test_layer_outputs_equal_the_plain_layers(folders, models):
    for name in NAMES:
        seq = zc.prompt(3, 29, vocab(name))
        config, w = zc.read_model(folders[name])
        want = []
        plain.forward(seq, w, config, layer_outputs=want)
        r = zc.noisy_replay(folders[name], "float32", 64, models(name, "float32"), layer_outputs=True)
        r.step([("r", seq[:20], [19])])
        r.step([("r", seq[20:], [8])])
        assert len(want) == len(models(name, "float32").spec.schedule)
        for t in range(29):
            got = r.layers[("r", t)]
            for i in range(len(want)):
                assert np.abs(got[i] - want[i][t]).max() <= 2e-4 * max(1.0, np.abs(want[i][t]).max()), (name, i, t)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_token_by_token(name, dtype, folders, models):
    n = 120
    seq = zc.prompt(41, n, vocab(name))
    r = zc.noisy_replay(folders[name], dtype, 128, models(name, dtype))
    r.step([("r", seq[:n - 50], list(range(0, n - 50, 3)))])
    for t in range(n - 50, n):
        r.step([("r", [seq[t]], [0])])
    zc.check_rows(r.rows, folders[name], {"r": seq}, dtype, "tail")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_every_token_decoded(name, dtype, folders, models):
    """From the first token on, one by one (the first tokens of a sequence, then a long decode over many pages, windows and
    blocks)."""
    n = 70 if dtype == "bfloat16" else 260
    seq = zc.prompt(42, n, vocab(name))
    r = zc.noisy_replay(folders[name], dtype, 272, models(name, dtype))
    for t in range(n):
        r.step([("r", [seq[t]], [0] if t < 4 or t % 4 == 0 or t > n - 5 else [])])
    zc.check_rows(r.rows, folders[name], {"r": seq}, dtype, "decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_down_to_two_tokens(name, dtype, folders, models):
    portions = [7, 2, 16, 3, 2, 33, 1, 15, 2, 17, 2, 5, 1, 1, 2, 40]
    n = sum(portions)
    seq = zc.prompt(43, n, vocab(name))
    r = zc.noisy_replay(folders[name], dtype, 160, models(name, dtype), page_size=8)
    o = 0
    for p in portions:
        r.step([("r", seq[o:o + p], list(range(p)))])
        o += p
    zc.check_rows(r.rows, folders[name], {"r": seq}, dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(name, dtype, folders, models):
    """Five requests over three state slots and a pool of 14 pages of 16: portions of some beside single tokens of others;
    a request that ends gives its pages and its slot (with the state it left) to the next, which must not see them."""
    V = vocab(name)
    seqs = {f"s{i}": zc.prompt(50 + i, n, V) for i, n in enumerate([61, 9, 130, 33, 47])}
    r = zc.noisy_replay(folders[name], dtype, 14 * 16, models(name, dtype), max_requests=3)
    at = {k: 0 for k in seqs}

    def take(rid, n):
        toks = seqs[rid][at[rid]:at[rid] + n]
        want = [i for i in range(len(toks)) if (at[rid] + i) % 3 == 0 or at[rid] + i == len(seqs[rid]) - 1]
        at[rid] += len(toks)
        return (rid, toks, want)

    def done(*rids):
        return [x for x in rids if at[x] == len(seqs[x])]

    r.step([take("s0", 20), take("s1", 2)])
    r.step([take("s0", 1), take("s1", 1), take("s2", 50)])
    r.step([take("s0", 40), take("s1", 6), take("s2", 1)], end=["s0", "s1"])
    r.step([take("s2", 1), take("s3", 33)], end=["s3"])
    r.step([take("s4", 2), take("s2", 30)])
    while at["s2"] < 130 or at["s4"] < 47:
        batch = [take(x, 1 if x == "s2" else 5) for x in ("s2", "s4") if at[x] < len(seqs[x])]
        r.step(batch, end=done(*[b[0] for b in batch]))
    assert all(at[k] == len(seqs[k]) for k in seqs)
    zc.check_rows(r.rows, folders[name], seqs, dtype, "mixed")
    assert len(r.cache.requests) == 0 and r.cache.available_pages() == [14] * len(r.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Z1", "Z3"])
def test_batched_rows_equal_the_rows_of_each_request_alone(name, dtype, folders, models):
    """What a request's rows are does not depend on what else is in the batch, nor on pages and slots, beyond rounding (the
    scan's chunks and the products' kernels follow the step's rows)."""
    a, b = zc.prompt(60, 45, vocab(name)), zc.prompt(61, 18, vocab(name))
    alone = zc.noisy_replay(folders[name], dtype, 128, models(name, dtype))
    alone.step([("a", a[:30], list(range(30)))]); alone.step([("a", a[30:], list(range(15)))])
    both = zc.noisy_replay(folders[name], dtype, 128, models(name, dtype))
    both.step([("b", b[:10], [9]), ("a", a[:30], list(range(30)))])
    both.step([("a", a[30:], list(range(15))), ("b", b[10:], [7])])
    for p in range(45):
        d = np.abs(alone.rows[("a", p)] - both.rows[("a", p)]).max()
        assert d <= (1e-4 if dtype == "float32" else 0.05) * np.std(alone.rows[("a", p)]), (p, d)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_few_wanted_rows_take_the_last_layers_shortcut(name, dtype, folders, models):
    """Steps that want few rows (or none) run the last layer's attention scores, output products and experts for those rows
    only (Z1, Z2: a last layer that is a recurrence or an attention without feed-forward; Z3: a window attention with blocks
    of one): the logits equal the plain implementation's, the cache and the state that later steps read are complete, and
    switching the shortcut off changes nothing beyond rounding."""
    n = 131
    seq, other = zc.prompt(33, n, vocab(name)), zc.prompt(34, 40, vocab(name))
    runs = {}
    for shortcut in (True, False):
        r = zc.noisy_replay(folders[name], dtype, 256, models(name, dtype))
        r.runner.tail_shortcut = shortcut
        r.step([("r", seq[:30], [])])
        r.step([("r", seq[30:60], [29, 3]), ("o", other[:20], [19])])
        r.step([("r", seq[60:n - 5], [0]), ("o", other[20:], [])])
        r.step([("r", seq[n - 5:], list(range(5)))])
        assert set(k for k in r.rows if k[0] == "r") == {("r", p) for p in [59, 33, 60] + list(range(n - 5, n))}
        zc.check_rows(r.rows, folders[name], {"r": seq, "o": other}, dtype, f"shortcut {shortcut}")
        runs[shortcut] = r.rows
    assert models(name, dtype).layers[-1].supports_tail
    for key, row in runs[True].items():
        d = np.abs(row - runs[False][key]).max()
        assert d <= (1e-4 if dtype == "float32" else 0.08 * np.std(row)), (key, d)


def test_tensor_core_attention_equals_the_float32_arithmetic_one_in_a_model(folders, models):
    """The same bfloat16 steps with the tensor-core attention switched off: rows agree within rounding."""
    from coheryn_ai_studio_b200 import ops
    for name in ("Z1", "Z3"):
        seq, other = zc.prompt(62, 150, vocab(name)), zc.prompt(63, 70, vocab(name))
        rows = {}
        for on in (True, False):
            ops.set_pooled_tc(on)
            try:
                r = zc.noisy_replay(folders[name], "bfloat16", 256, models(name, "bfloat16"))
                r.step([("r", seq[:91], list(range(0, 91, 2)))])
                r.step([("r", seq[91:140], list(range(0, 49, 3))), ("o", other, [69, 5])])
                for t in range(140, 150):
                    r.step([("r", [seq[t]], [0])])
                rows[on] = r.rows
            finally:
                ops.set_pooled_tc(True)
        zc.check_rows(rows[True], folders[name], {"r": seq, "o": other}, "bfloat16", "tensor cores")
        near = [np.abs(rows[True][k] - rows[False][k]).max() <= 0.05 * np.std(rows[False][k]) for k in rows[True]]
        assert np.mean(near) > 0.9          # a router's near tie may fall the other way at single rows


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["Z1", "Z3"])
def test_greedy_generation_through_the_engine(name, dtype, folders):
    """The Python entry point with its scheduler, continuous batching, portions of 16 tokens and decode steps replayed
    from CUDA graphs: every generated token is the plain implementation's first maximum given the tokens before it (in
    bfloat16: or a near tie)."""
    from coheryn_ai_studio_b200.engine import Engine
    eng = Engine.from_folder(folders[name], dtype, context=128, max_num_seqs=3, max_num_batched_tokens=16, page_size=8)
    prompts = [zc.prompt(70 + i, n, vocab(name)) for i, n in enumerate((3, 29, 50, 1))]
    res = eng.generate(prompts, max_tokens=12)
    for p, out in zip(prompts, res):
        ids = list(p)
        assert out.completion_tokens == 12 and out.finish_reason == "length"
        for tok in out.token_ids:
            ref = zc.plain_rows(folders[name], ids)[-1]
            best = int(np.argmax(ref))
            if tok != best:
                gap = float(ref[best] - ref[tok]) / float(np.std(ref))
                assert gap <= (1e-3 if dtype == "float32" else 0.4), (name, len(ids), tok, best, gap)
            ids.append(tok)
    eng.cache.check()
    assert len(eng.cache.requests) == 0


def test_trace_program_replays_a_schedule(folders, tmp_path):
    """bin/trace_run on a folder of this design: portions, a second request, an ended request, a step that wants nothing."""
    import json, os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "Z2"
    a, b = zc.prompt(80, 40, vocab(name)), zc.prompt(81, 12, vocab(name))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:25], "want": [0, 24]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[25:27], "want": []}, {"id": "b", "tokens": b, "want": [11]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[27:], "want": [12]}], "end": ["a"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders[name], "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    V = vocab(name)
    got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, V)
    got1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, V)
    got2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(1, V)
    rows = {("a", 0): got0[0], ("a", 24): got0[1], ("b", 11): got1[0], ("a", 39): got2[0]}
    zc.check_rows(rows, folders[name], {"a": a, "b": b}, "float32", "trace")


def test_command_line_runs_and_inspects_the_design(folders):
    import os, subprocess, sys
    from coheryn_ai_studio_b200 import api
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "Z1"
    p = zc.prompt(85, 27, vocab(name))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "coheryn"), "run", folders[name], "--tokens", ",".join(map(str, p)),
                        "--max-tokens", "5", "--context", "64", "--dtype", "float32", "--stream"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [int(t) for t in r.stdout.split()]
    ids = list(p)
    for tok in got:
        assert tok == int(np.argmax(zc.plain_rows(folders[name], ids)[-1]))
        ids.append(tok)
    assert api.generate(folders[name], [p], max_tokens=5, context=64, dtype="float32")[0]["token_ids"] == got
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "coheryn"), "models", "inspect", folders[name]], capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0 and "Zegelix" in r.stdout, r.stderr[-2000:]


def test_zz_report():
    print(f"\nZegelix rows against the plain implementation: float32 largest |d| = {zc.WORST['float32']:.2e}; "
          f"bfloat16 largest median distance = {zc.WORST['bfloat16']:.2f} of the bound")
