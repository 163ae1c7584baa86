"""Fapenex through the engine against the plain implementation (tests/plain_fapenex.py): each mechanism alone, whole
models of several sizes and layer orders, prompts cut in every way, batches, reused pages and state slots, keys at the
edges of windows and chunks, long decoding, and greedy generation through the scheduler."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import random_tokens
import plain_fapenex as plain
from trace_helpers import by_position, mixed, portions, staggered_plan, tail_decode, whole

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 5e-2}
F = torch.float64


def latent(heads, dim, vdim, kv_rank, q_rank, scale, window):
    return "latent_attention", {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
                                "mask": {"size": window}}


def delta(heads, kv_heads, dim, vdim, conv):
    return "delta", {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def chunked(heads, kv_heads, dim, vdim, scale, chunk, rot_dims, base=1e4, scaling=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk}}
    if rot_dims:
        out["rot"] = {"base": base, "dims": rot_dims}
        if scaling is not None:
            out["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return "attention", out


def moe(experts, top, ff, limit, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def layer(mixer, mlp=None):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


def config(width, vocab, layers, loop=None, scale=1.0, cap=None, eps=1e-5, positions=512):
    out = {"architecture": "Fapenex", "norm": {"eps": eps}, "vocab": vocab, "width": width, "max_positions": positions, "layers": layers,
           "logit_scale": scale, "logit_softcap": cap}
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


# Sizes that differ from one another in everything: every order of the three mixers, key and value sizes that are unequal
# in both directions, as many key heads as query heads and fewer, rotation of a part of a head, of the whole head and
# none, with and without stretched frequencies, windows and chunks shorter than a page, no multiple of one and longer than
# every prompt here, convolutions of two to five taps, one expert a row, several and all, with and without the shared
# unit, layers without feed-forward, a span that runs twice or three times from the first layer or later to the last or
# earlier, no span, no cap on the logits, a logit scale that is no power of two.
MODELS = {
    "one-each": config(64, 97, [layer(delta(3, 1, 8, 24, 4), moe(5, 2, 40, 1.5, (48, 1.0))),
                                layer(chunked(4, 2, 16, 24, 0.3, 21, 8), moe(3, 3, 24, 0.7)),
                                layer(latent(2, 24, 16, 20, 28, 0.25, 13), None)], scale=0.7, cap=9.0),
    "looped": config(96, 211, [layer(latent(4, 16, 24, 40, 24, 0.3, 40), moe(6, 1, 32, 2.5, (40, 2.0))),
                               layer(delta(4, 4, 24, 8, 2), moe(4, 2, 24, 1.2)),
                               layer(chunked(6, 2, 16, 16, 0.3, 33, 16, 300.0, (8.0, 32, 16.0, 1.0)), None),
                               layer(chunked(1, 1, 64, 40, 0.125, 300, 64, 2.5e5, (4.0, 128, 32.0, 1.0)), moe(7, 3, 24, 3.0, (16, 0.5)))],
                     loop=(1, 3, 3), scale=2.0, cap=15.0),
    "loop-all": config(64, 130, [layer(chunked(2, 1, 24, 32, 0.35, 9, 12, 1e3), moe(4, 2, 48, 1.0, (24, 1.5))),
                                 layer(delta(2, 1, 16, 40, 5), None)], loop=(0, 2, 2), scale=1.0, cap=None, eps=3e-6),
    "loop-tail": config(80, 77, [layer(delta(5, 5, 16, 16, 3), moe(2, 1, 11, 1.2)),
                                 layer(latent(5, 8, 8, 12, 9, 0.4, 7), moe(7, 3, 24, 3.0, (32, 0.8))),
                                 layer(latent(2, 40, 24, 64, 48, 0.2, 50), None)], loop=(1, 3, 2), scale=3.3, cap=30.0),
    # nothing a multiple of anything: odd width, odd sizes everywhere, a prime vocabulary
    "awkward": config(50, 61, [layer(chunked(3, 3, 10, 7, 0.4, 13, 6, 555.0), moe(2, 1, 11, 1.2, (9, 0.6))),
                               layer(delta(3, 1, 5, 7, 3), moe(3, 2, 13, 0.9)),
                               layer(latent(3, 6, 9, 11, 7, 0.5, 5), None)], loop=(0, 1, 3), scale=1.3, cap=11.0),
    # heads of 64 and 128, as the tensor-core kernels take them; prompts longer than the recurrence's staged rows
    "wide": config(256, 333, [layer(chunked(4, 2, 64, 64, 0.125, 48, 64, 1e4, (4.0, 64, 16.0, 1.0)), moe(4, 2, 128, 2.0, (256, 1.5))),
                              layer(delta(2, 1, 128, 128, 4), None),
                              layer(latent(4, 64, 64, 128, 96, 0.125, 100), moe(8, 2, 64, 1.5)),
                              layer(chunked(2, 1, 128, 128, 0.09, 100, 64), None)], loop=(1, 3, 2), scale=2.0, cap=20.0),
}
STD = 0.16     # matrices N(0, STD): products keep their input's spread, so scores, gates and routers are far from flat
STDS = {"wide": 0.08}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """(folder, config.json as written, float64 weights) of every model."""
    from infinicore_infer_b200.config import config_class_for
    from infinicore_infer_b200.weights import index_directory, read_tensor, write_model_folder
    out = {}
    for seed, (name, cfg) in enumerate(MODELS.items()):
        d = str(tmp_path_factory.mktemp("fapenex_" + name))
        write_model_folder(config_class_for(cfg).from_dict(cfg), d, seed=seed + 71, std=STDS.get(name, STD), norm_std=0.2)
        with open(os.path.join(d, "config.json")) as f:
            disk = json.load(f)
        out[name] = (d, disk, {n: read_tensor(i).double().numpy() for n, i in index_directory(d).items()})
    return out


@pytest.fixture(scope="module")
def engines(folders):
    from infinicore_infer_b200.engine import Engine
    cache = {}

    def get(name, dtype, cache_tokens=512, max_requests=3, **kw):
        key = (name, dtype, cache_tokens, max_requests, tuple(sorted(kw.items())))
        if key not in cache:
            cache[key] = Engine.from_folder(folders[name][0], dtype=DTYPES[dtype], max_tokens=512, cache_tokens=cache_tokens,
                                            page_size=16, max_requests=max_requests, max_step_tokens=512, **kw)
        return cache[key]
    return get


_plain = {}
# A row whose router leaves the last chosen expert this close to the first one left out may go to another expert once the
# activations are rounded to bfloat16: such a row's logits are those of another, equally valid, choice, and are not compared.
CLOSE_CALL = {"float32": 1e-4, "bfloat16": 0.08}


class Expected(np.ndarray):
    """Logits [T, vocab] with ``margin`` [T]: the smallest router margin of each row over the model's routed layers, and
    ``noise`` [T]: how far each row's logits move (as ``row_error`` measures it) when the plain implementation rounds the
    operands of its matrix products to bfloat16 and does nothing else differently: what 16-bit operands alone do to that
    row.  These models are sensitive on purpose (sharp softmaxes, routers that decide): a choice that flips early in a
    sequence travels on through a recurrence's state, and the rows it reaches differ by tenths of the logits' spread in
    ANY bfloat16 implementation; which rows those are depends on the last bit."""


def row_error(got, want):
    """Per row: the difference with its mean taken off, root mean square over the vocabulary, against the logits' spread."""
    diff = got - want
    return (diff - diff.mean(1, keepdims=True)).std(1) / (want - want.mean(1, keepdims=True)).std()


def rounded_operands(cfg, w, toks):
    """The plain model's logits with the operands of every matrix product rounded to bfloat16."""
    exact = plain.operand
    plain.operand = lambda a: torch.tensor(a).to(torch.bfloat16).double().numpy()
    try:
        return plain.forward(cfg, w, toks)
    finally:
        plain.operand = exact


def expected(folders, name, seed, n):
    key = (name, seed, n)
    if key not in _plain:
        _, cfg, w = folders[name]
        toks = random_tokens(seed, n, cfg["vocab"])
        margins = []
        want = plain.forward(cfg, w, toks, margins=margins).view(Expected)
        want.margin = np.stack(margins).min(0) if margins else np.full(n, np.inf)
        want.noise = row_error(rounded_operands(cfg, w, toks), np.asarray(want))
        _plain[key] = (toks, want)
    return _plain[key]


def run(engine, steps):
    from infinicore_infer_b200.trace import replay
    return by_position(steps, replay(engine, steps))


def check(got, rid, want, tol, what):
    """float32: every logit of every position within ``tol`` of the logits' scale, the sharp test; one row in twenty may reach
    five times that (a norm on a sublayer's OUTPUT turns a small output's rounding into a large relative error: the plain
    implementation shows the same rows when its weights are moved by float32's rounding).  bfloat16: the rows' errors
    (``row_error``) against what 16-bit operands alone do to the plain model (``Expected.noise``): the median row within
    ``tol`` or twice the median noise, the ninth decile within three times ``tol`` or twice the noise's ninth decile.  Rows
    whose router call is close are left out (``CLOSE_CALL``).  The sharp tests of the bfloat16 kernels are those of the
    mechanisms alone, further down, whose inputs are made so that one key decides."""
    loose = tol > 1e-3
    margin = getattr(want, "margin", np.full(len(want), np.inf))
    sure = margin >= CLOSE_CALL["bfloat16" if loose else "float32"]
    noise = getattr(want, "noise", np.zeros(len(want)))
    assert len(want) < 20 or sure.sum() >= 0.4 * len(want), f"{what}: the router is sure of {int(sure.sum())} of {len(want)} rows only"
    want = np.asarray(want, dtype=np.float64)
    diff = np.stack([got[(rid, p)].astype(np.float64) - want[p] for p in range(len(want))])
    if not loose:
        errs, scale = np.abs(diff).max(1) * sure, np.abs(want).max()
        worst = int(errs.argmax())
        assert errs.max() <= 5 * tol * scale, f"{what}: request {rid} position {worst}: error {errs.max():.3e} > {5 * tol * scale:.3e}"
        assert (errs > tol * scale).sum() <= max(1, len(errs) // 20), f"{what}: request {rid}: {(errs > tol * scale).sum()} of {len(errs)} rows beyond {tol * scale:.3e}"
        return
    errs, noise = row_error(diff + want, want)[sure], noise[sure]
    if not len(errs):
        return
    assert np.median(errs) <= max(tol, 2 * np.median(noise)), \
        f"{what}: request {rid}: the median row differs by {np.median(errs):.3f} of the logits' spread, the rounded plain model's by {np.median(noise):.3f}"
    assert np.quantile(errs, 0.9) <= max(3 * tol, 2 * np.quantile(noise, 0.9)), \
        f"{what}: request {rid}: the ninth decile differs by {np.quantile(errs, 0.9):.3f}, the rounded plain model's by {np.quantile(noise, 0.9):.3f}"


# ---- whole models ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", list(MODELS))
def test_whole_tail_and_portions_agree_with_the_plain_implementation(folders, engines, name, dtype):
    eng = engines(name, dtype)
    for i, n in enumerate((1, 37, 150)):
        toks, want = expected(folders, name, 300 + i, n)
        for what, steps in (("whole", whole("r", toks)), ("tail", tail_decode("r", toks, tail=20)),
                            ("portions", portions("r", toks)), ("pairs", portions("r", toks, sizes=(2,))),
                            ("uneven", portions("r", toks, sizes=(17, 3, 31, 2, 16)))):
            check(run(eng, steps), "r", want, TOL[dtype], f"{name} {dtype} {what} n={n}")
        eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_every_token_decoded_alone_through_graphs(folders, engines, dtype):
    """Long decoding: every token a step of its own (captured steps), so pages, the convolutions' tails and the states move
    one position at a time, and windows and chunk borders pass over decoded tokens."""
    for name in ("looped", "loop-tail", "one-each"):
        toks, want = expected(folders, name, 77, 300)
        eng = engines(name, dtype)
        before = eng.steps_run
        check(run(eng, tail_decode("r", toks, tail=len(toks))), "r", want, TOL[dtype], f"{name} {dtype} token by token")
        assert eng.steps_run - before >= 300


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("name", ["looped", "loop-all", "awkward"])
def test_batches_of_unequal_requests_in_a_small_pool(folders, name, dtype):
    """Up to three live requests, portions beside single tokens; the pool holds three requests, so the pages and state
    slots of finished requests are the next ones handed out.  Every row equals the request run alone."""
    from infinicore_infer_b200.engine import Engine
    lengths = [70, 9, 33, 50, 2, 41, 64]
    reqs, wants = {}, {}
    for i, n in enumerate(lengths):
        toks, want = expected(folders, name, 500 + i, n)
        reqs[f"q{i}"], wants[f"q{i}"] = toks, want
    steps = mixed(reqs, staggered_plan(reqs, live=3, portion=6, tail=5))
    eng = Engine.from_folder(folders[name][0], dtype=DTYPES[dtype], max_tokens=128, cache_tokens=3 * 80, page_size=16,
                             max_requests=3, max_step_tokens=128)
    got = run(eng, steps)
    for rid, want in wants.items():
        check(got, rid, want, TOL[dtype], f"{name} {dtype} mixed")
    eng.cache.check_invariants()
    assert eng.cache.slots.available == 3 and all(g.pool.in_use == 0 for g in eng.cache.groups)


def test_a_reused_slot_starts_from_zero_state_and_empty_tails(folders, engines):
    """The same request twice in a row lands in the slot (and pages) that its first run left: the recurrence's state and
    the convolutions' tails start from zero again."""
    toks, want = expected(folders, "looped", 9, 45)
    eng = engines("looped", "float32", max_requests=1)
    check(run(eng, whole("r", toks)), "r", want, TOL["float32"], "first run")
    check(run(eng, portions("r", toks, sizes=(5, 2))), "r", want, TOL["float32"], "second run in the same slot")


def test_passes_of_a_span_keep_caches_and_states_apart(folders):
    from infinicore_infer_b200.config import read_config
    from infinicore_infer_b200.parts import cache_needs, state_needs
    spec = read_config(folders["looped"][0], max_tokens=64).model_spec()
    assert [e.layer for e in spec.order] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [e.cache for e in spec.order] == list(range(8)) and all(e.writes_cache for e in spec.order)
    assert [e.before.index if e.before else None for e in spec.order] == [None, 0, None, 1, None, 2, None, None]
    needs, states = cache_needs(spec), state_needs(spec)
    assert (needs[0].num_kv_heads, needs[0].head_dim, needs[0].v_head_dim, needs[0].window, needs[0].values_in_keys) == (1, 40, 40, 40, True)
    assert needs[1].shape == (4, 24, 8) and needs[3].shape == (4, 24, 8) and states[1].shape == (1, 2 * 96 + 32)
    assert (needs[2].num_kv_heads, needs[2].head_dim, needs[2].v_head_dim, needs[2].window) == (2, 16, None, 33)
    assert needs[7].window == 300 and needs[7].v_head_dim == 40 and states[2] is None


# ---- mechanisms alone, with inputs made so that one key decides ------------------------------------------------------------
def paged(k, v, page, dev, dtype):
    """Keys [T, G, dk] and values [T, G, dv] of one request into pages handed out in a scrambled order."""
    T, G, dk = k.shape
    blocks = (T + page - 1) // page
    order = torch.randperm(blocks, generator=torch.Generator().manual_seed(3)) + 1
    kp = torch.zeros(blocks + 1, G, page, dk, dtype=dtype, device=dev)
    vp = torch.zeros(blocks + 1, G, page, v.shape[-1], dtype=dtype, device=dev)
    for t in range(T):
        kp[order[t // page], :, t % page] = k[t].to(dtype)
        vp[order[t // page], :, t % page] = v[t].to(dtype)
    return kp, vp, order.to(torch.int32).view(1, -1).to(dev)


def chunk_edge_case(T, H, G, dk, dv, chunk, seed, bf16):
    """Queries, keys and values in which, for chosen rows i, head 0 scores the last key of the chunk before (just outside)
    above the first key of the row's own chunk (just inside) above all others, and head 1 scores a key far back, in an
    earlier chunk, above everything: a border that is one off in either direction, or chunks counted from elsewhere than
    position 0, moves the row's output from one value to another.  And the last row of every chunk scores, with its last
    head, the chunk's SECOND key above everything: a key as far back as the mask allows, among all the others, decides that
    row (``far`` lists (row, key))."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, H, dk, generator=g, dtype=F)
    k = 0.3 * torch.randn(T, G, dk, generator=g, dtype=F)
    v = torch.randn(T, G, dv, generator=g, dtype=F)
    rows = [i for i in range(chunk + 2, T, 7) if i % chunk not in (0, 1)]
    for i in rows:                                # heads 0 and 1 read key head 0
        start = i // chunk * chunk
        unit = q[i, 0] / (q[i, 0] @ q[i, 0])
        k[start - 1, 0] = 14.0 * unit
        k[start, 0] = 9.0 * unit
        q[i, 1] = q[i, 0]
    far = []
    for start in range(0, T, chunk):              # the last head reads the last key head
        last = min(start + chunk, T) - 1
        if last - start >= 8:
            k[start + 1, G - 1] = 16.0 * q[last, H - 1] / (q[last, H - 1] @ q[last, H - 1])
            far.append((last, start + 1))
    if bf16:
        q, k, v = (t.to(torch.bfloat16).double() for t in (q, k, v))
    chunk_edge_case.far = far
    return q, k, v, rows


def far_keys_decide(want, v, far, G):
    """The rows that were given a far key do read its value, almost alone."""
    for row, key in far:
        assert np.abs(want[row, -1] - v[key, G - 1].numpy()).max() < 0.05, f"row {row} does not rest on key {key}"


def plain_chunks(q, k, v, chunk, positions, shift=0, sink=True):
    see = np.array([[j <= i and (i + shift) // chunk == (j + shift) // chunk for j in positions] for i in positions])
    return plain.masked_softmax_attention(q.numpy(), k.numpy(), v.numpy(), 1.0, see, sink)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("chunk,page", [(7, 8), (16, 16), (33, 8), (40, 16), (64, 16)])
def test_chunk_borders_and_the_sink_of_the_row_attention(dtype, chunk, page):
    """The kernel of one warp a row and head: whole prompts and single decoded rows, values of another size than keys."""
    from infinicore_infer_b200 import kernels as K
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    T, H, G, dk, dv = 150, 4, 2, 24, 40
    q, k, v, rows = chunk_edge_case(T, H, G, dk, dv, chunk, chunk, dt == torch.bfloat16)
    want = plain_chunks(q, k, v, chunk, np.arange(T))
    far_keys_decide(want, v, chunk_edge_case.far, G)
    for other in (plain_chunks(q, k, v, chunk, np.arange(T), shift=1), plain_chunks(q, k, v, chunk, np.arange(T), shift=-1),
                  plain_chunks(q, k, v, chunk, np.arange(T), sink=False)):
        assert np.abs(other - want)[rows].max() > 0.05       # the inputs do tell a border that is one off, and a lost sink
    kp, vp, table = paged(k, v, page, dev, dt)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    out = torch.empty(T, H, dv, dtype=dt, device=dev)
    K.attention_rows(q.to(dt).to(dev).contiguous(), kp, vp, out, pos, torch.zeros_like(pos), table, T, H, 1.0, -chunk, sink=True)
    tol = 2e-5 if dt == torch.float32 else 3e-2
    err = np.abs(out.double().cpu().numpy() - want).max()
    assert err <= tol, f"prompt rows differ by {err}"
    for i in rows[-4:] + [0, chunk - 1, chunk, chunk + 1] + [row for row, _ in chunk_edge_case.far]:       # the same rows one by one, as a decode step sees them
        one = torch.empty(1, H, dv, dtype=dt, device=dev)
        K.attention_rows(q[i:i + 1].to(dt).to(dev).contiguous(), kp, vp, one, pos[i:i + 1], torch.zeros(1, dtype=torch.int32, device=dev), table,
                         1, H, 1.0, -chunk, sink=True)
        assert np.abs(one.double().cpu().numpy()[0] - want[i]).max() <= tol, f"decoded row {i}"


@pytest.mark.parametrize("dh", [32, 64, 128])
@pytest.mark.parametrize("chunk", [17, 40, 64, 130, 200])
def test_chunk_borders_on_the_tensor_cores(dh, chunk):
    """The bfloat16 kernels of the generation path: tiles of a prompt's rows (a whole prompt, and a portion that starts in
    the middle of a page and of a chunk behind cached keys), and single rows whose keys are cut into ranges.  Chunks shorter
    and longer than a tile of keys, so that whole tiles of keys are invisible to the later rows of a tile."""
    from infinicore_infer_b200 import kernels as K
    dev, dt = torch.device("cuda:0"), torch.bfloat16
    T, H, G, page = 333, 4, 2, 16
    q, k, v, rows = chunk_edge_case(T, H, G, dh, dh, chunk, chunk + dh, True)
    want = plain_chunks(q, k, v, chunk, np.arange(T))
    far_keys_decide(want, v, chunk_edge_case.far, G)
    rows = rows + [row for row, _ in chunk_edge_case.far]
    kp, vp, table = paged(k, v, page, dev, dt)
    qd = q.to(dt).to(dev).contiguous()
    kernels = [("legacy tiles", K.attention_prefill)]
    if K.attention_tcgen05_supports(dh, page):
        kernels.append(("tcgen05 tiles", None))
    for start in (0, 203):                        # the rows of positions start .. T - 1 as one portion
        n = T - start
        tiles = torch.tensor([[0, r0] for r0 in range(0, n, K.TILE_ROWS)], dtype=torch.int32, device=dev)
        req_start = torch.tensor([0, n], dtype=torch.int32, device=dev)
        req_pos = torch.tensor([start], dtype=torch.int32, device=dev)
        for name, fn in kernels:
            out = torch.zeros(n, H, dh, dtype=dt, device=dev)
            if fn is None:
                K.attention_tcgen05(qd[start:].contiguous(), kp, vp, out, tiles, len(tiles), n, req_start, req_pos, table, H, 1.0, -chunk, sink=True)
                K.check_gemm_status(dev)
            else:
                fn(qd[start:].contiguous(), kp, vp, out, tiles, len(tiles), req_start, req_pos, table, H, 1.0, -chunk, sink=True)
            err = np.abs(out.double().cpu().numpy() - want[start:]).max()
            assert err <= 3e-2, f"{name} from position {start}: {err}"
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    some = torch.tensor(rows[-6:] + [0, chunk - 1, chunk, chunk + 1], dtype=torch.int32, device=dev)
    for splits in (1, 3, 8):
        out = torch.zeros(T, H, dh, dtype=dt, device=dev)
        K.attention_decode(qd, kp, vp, out, some, len(some), pos, torch.zeros_like(pos), table, H, 1.0, -chunk, splits, sink=True)
        got = out.double().cpu().numpy()
        for i in some.tolist():
            assert np.abs(got[i] - want[i]).max() <= 3e-2, f"single row {i}, {splits} ranges"


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_biases_head_norms_ahead_of_the_rotation_and_cache_rows(dtype):
    """Two requests side by side at unequal positions in scrambled pages: biases on q, k and v, every head of q and k normed
    with its projection's weight, THEN its leading elements rotated in halves by stretched frequencies; values as they come;
    keys and values land in the pages at the rows' positions."""
    from infinicore_infer_b200 import kernels as K
    from infinicore_infer_b200.config import FrequencyRampSpec, PairRotarySpec
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    H, G, dk, dv, dims, page, eps = 4, 2, 24, 16, 16, 8, 1e-3
    rot = {"dims": dims, "base": 300.0, "scaling": {"factor": 4.0, "original": 32, "fast": 4.0, "slow": 1.0}}
    f, mag = PairRotarySpec(dims=dims, base=300.0, scaling=FrequencyRampSpec(4.0, 32.0, 4.0, 1.0, magnitude_slope=0.1), layout="halves").frequencies()
    g = torch.Generator().manual_seed(2)
    starts, n = (3, 41), 30
    nq, nk, nv = H * dk, G * dk, G * dv
    ld = nq + nk + nv + 5
    u = torch.randn(2 * n, ld, generator=g, dtype=F) * 2.0
    bias = torch.randn(ld, generator=g, dtype=F).float()
    wq, wk = (1 + 0.5 * torch.randn(dk, generator=g, dtype=F)).float(), (1 + 0.5 * torch.randn(dk, generator=g, dtype=F)).float()
    pos = np.concatenate([np.arange(s, s + n) for s in starts])
    blocks = (max(starts) + n + page - 1) // page
    table = torch.tensor([[2 * b + 2 for b in range(blocks)], [2 * b + 1 for b in range(blocks)]], dtype=torch.int32, device=dev)
    kp = torch.zeros(2 * blocks + 1, G, page, dk, dtype=dt, device=dev)
    vp = torch.zeros(2 * blocks + 1, G, page, dv, dtype=dt, device=dev)
    q_out = torch.empty(2 * n, H, dk, dtype=dt, device=dev)
    K.conv_qkv(u.float().to(dev), (0, nq, nq + nk), H, G, dk, dv, True, (None, None, None), 0, (wq.to(dev), wk.to(dev)), eps,
               torch.tensor(f, dtype=torch.float32, device=dev), dims, None, torch.tensor(pos, dtype=torch.int32, device=dev),
               torch.tensor([0] * n + [1] * n, dtype=torch.int32, device=dev), torch.tensor([0, n, 2 * n], dtype=torch.int32, device=dev),
               torch.tensor([1, 2], dtype=torch.int32, device=dev), table, page, q_out, kp, vp, rot_half=True, rot_mag=mag, head_norm=2,
               bias=bias.to(dev))
    uf = u.float().double().numpy() + bias.double().numpy()
    q = plain.rotate_half(plain.norm_plain(uf[:, :nq].reshape(2 * n, H, dk), wq.double().numpy(), eps), pos, rot)
    k = plain.rotate_half(plain.norm_plain(uf[:, nq:nq + nk].reshape(2 * n, G, dk), wk.double().numpy(), eps), pos, rot)
    v = uf[:, nq + nk:nq + nk + nv].reshape(2 * n, G, dv)
    other = plain.norm_plain(plain.rotate_half(uf[:, :nq].reshape(2 * n, H, dk), pos, rot), wq.double().numpy(), eps)
    assert np.abs(other - q).max() > 0.1          # norm and rotation do not commute here: the order shows
    tol = 2e-5 if dt == torch.float32 else 2e-2
    assert np.abs(q_out.double().cpu().numpy() - q).max() < tol * np.abs(q).max()
    for r in range(2 * n):
        pg, at = table[r // n, pos[r] // page].item(), pos[r] % page
        assert np.abs(kp[pg, :, at].double().cpu().numpy() - k[r]).max() < tol * np.abs(k).max(), f"key of row {r}"
        assert np.abs(vp[pg, :, at].double().cpu().numpy() - v[r]).max() < tol * np.abs(v).max(), f"value of row {r}"


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("H,R,window,page", [(3, 20, 7, 8), (8, 64, 33, 16), (2, 96, 40, 16), (16, 128, 130, 16), (5, 24, 300, 8)])
def test_window_edges_of_the_latent_attention(dtype, H, R, window, page):
    """All heads over one cached row per position, on the row kernel and (bfloat16) the tensor-core kernel, whole prompts,
    a portion behind cached keys, and single rows with their keys cut into ranges: head 0 scores the key just outside the
    window above the key just inside above all others."""
    from infinicore_infer_b200 import kernels as K
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    T = 210
    g = torch.Generator().manual_seed(R + window)
    q = torch.randn(T, H, R, generator=g, dtype=F)
    c = 0.3 * torch.randn(T, R, generator=g, dtype=F)
    rows = list(range(window + 3, T, 5))         # none when the window is longer than the sequence
    for i in rows:
        unit = q[i, 0] / (q[i, 0] @ q[i, 0])
        c[i - window], c[i - window + 1] = 14.0 * unit, 9.0 * unit
    far = []
    if window >= T:                               # every key is seen: the last rows' last head rests on the second key, far back
        for i in (T - 1, T - 2):
            q[i, H - 1] = q[T - 1, H - 1]
            far.append(i)
        c[1] = 16.0 * q[T - 1, H - 1] / (q[T - 1, H - 1] @ q[T - 1, H - 1])
    if dt == torch.bfloat16:
        q, c = q.to(dt).double(), c.to(dt).double()
    see = plain.visibility(np.arange(T), plain.sees_window, window)
    want = plain.masked_softmax_attention(q.numpy(), c.numpy()[:, None], c.numpy()[:, None], 1.0, see, sink=False)
    for i in far:
        assert np.abs(want[i, -1] - c[1].numpy()).max() < 0.05 * np.abs(c[1].numpy()).max()
    for w2 in (window - 1, window + 1):
        other = plain.masked_softmax_attention(q.numpy(), c.numpy()[:, None], c.numpy()[:, None], 1.0,
                                               plain.visibility(np.arange(T), plain.sees_window, w2), sink=False)
        assert not rows or np.abs(other - want)[rows].max() > 0.05
    kp, _, table = paged(c[:, None], c[:, None], page, dev, dt)
    pages = kp[:, 0].contiguous()                 # [pages, page, R]
    tol = 2e-5 if dt == torch.float32 else 3e-2
    for start in (0, 77):
        n = T - start
        pos = torch.arange(start, T, dtype=torch.int32, device=dev)
        req_start = torch.tensor([0, n], dtype=torch.int32, device=dev)
        for with_tiles in (False, True):
            out = torch.empty(n, H, R, dtype=dt, device=dev)
            K.latent_attention(q[start:].to(dt).to(dev).contiguous(), pages, out, pos, torch.zeros_like(pos), table, H, R, 0, 1.0,
                               req_start=req_start if with_tiles else None, window=window)
            err = np.abs(out.double().cpu().numpy() - want[start:]).max()
            assert err <= tol, f"rows from {start} (tiles {with_tiles}): {err}"
    for i in rows[-3:] + far + [0, min(window, T) - 1, min(window, T - 1)]:
        for splits in (1, 4):
            one = torch.empty(1, H, R, dtype=dt, device=dev)
            p1 = torch.tensor([i], dtype=torch.int32, device=dev)
            K.latent_attention(q[i:i + 1].to(dt).to(dev).contiguous(), pages, one, p1, torch.zeros_like(p1), table, H, R, 0, 1.0, splits=splits,
                               req_start=torch.tensor([0, 1], dtype=torch.int32, device=dev), window=window)
            assert np.abs(one.double().cpu().numpy()[0] - want[i]).max() <= tol, f"single row {i}, {splits} ranges"


@pytest.mark.parametrize("H,G,dk,dv,taps", [(1, 1, 40, 24, 2), (4, 2, 24, 40, 4), (2, 1, 64, 64, 3), (6, 3, 7, 5, 5), (2, 2, 128, 128, 4), (3, 1, 200, 16, 3)])
def test_delta_rule_across_cuts_and_slots(H, G, dk, dv, taps):
    """Two sequences cut into portions (down to one row; one longer than the rows a block stages at a time) that go through
    state slots side by side: the convolutions from the kept tails, unit q and k, write strengths and decays from their
    logits, the state corrected toward each value.  An early key is written strongly and the decays are slow, so that a lost
    state, a decay that is applied after the write, or a read-out ahead of the write moves late outputs.  All in float32."""
    from infinicore_infer_b200 import kernels as K
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(H * dk + taps)
    T, eps = 150, 1e-4
    nk, nv = G * dk, H * dv
    C = 2 * nk + nv
    ld = C + 2 * H + nv
    W = {"q.conv": torch.randn(nk, taps, generator=g, dtype=F).numpy(), "k.conv": torch.randn(nk, taps, generator=g, dtype=F).numpy(),
         "v.conv": torch.randn(nv, taps, generator=g, dtype=F).numpy(), "A_log": (torch.randn(H, generator=g, dtype=F) - 5.0).numpy(),
         "dt_bias": torch.randn(H, generator=g, dtype=F).numpy(), "norm": (1 + 0.3 * torch.randn(dv, generator=g, dtype=F)).numpy()}
    us = [torch.randn(T, ld, generator=g, dtype=F).float().double().numpy() for _ in range(2)]
    us[0][1, C:C + H] += 6.0                      # an early row written with beta near one
    want = []
    for u in us:                                  # the plain mixer from the projections on
        q = plain.silu(plain.short_conv(u[:, :nk], W["q.conv"])).reshape(T, G, dk)
        k = plain.silu(plain.short_conv(u[:, nk:2 * nk], W["k.conv"])).reshape(T, G, dk)
        v = plain.silu(plain.short_conv(u[:, 2 * nk:C], W["v.conv"])).reshape(T, H, dv)
        q, k = np.repeat(plain.unit_vector(q) * dk ** -0.5, H // G, 1), np.repeat(plain.unit_vector(k), H // G, 1)
        beta = plain.sigmoid(u[:, C:C + H])
        gd = np.exp(-np.exp(W["A_log"]) * plain.softplus(u[:, C + H:C + 2 * H] + W["dt_bias"]))
        o, _ = plain.delta_recurrence(q, k, v, gd, beta)
        want.append((plain.rms_unit(o, eps) * W["norm"] * plain.silu(u[:, C + 2 * H:]).reshape(T, H, dv)).reshape(T, nv))
        early = plain.delta_recurrence(q, k, v, gd, beta * (np.arange(T) != 1)[:, None])[0]
        assert u is not us[0] or np.abs(early - o)[35:60].max() > 1e-3 * np.abs(o).max()     # rows beyond the first cuts do see the early write
    f32 = lambda a: torch.tensor(a, dtype=torch.float32, device=dev)
    conv = f32(np.concatenate([W["q.conv"], W["k.conv"], W["v.conv"]]))
    state = torch.zeros(4, H, dk, dv, dtype=torch.float32, device=dev)
    tails = torch.zeros(4, taps - 1, C, dtype=torch.float32, device=dev)
    state[0], tails[0] = 7.0, 7.0                 # slot 0 is nobody's; what lies there must not matter
    slots = torch.tensor([3, 1], dtype=torch.int32, device=dev)
    got = [[], []]
    cuts = [0, 1, 2, 4, 30, 31, 120, 145, T]
    for a, b in zip(cuts, cuts[1:]):
        rows = b - a
        u = f32(np.concatenate([us[0][a:b], us[1][a:b]]))
        req_start = torch.tensor([0, rows, 2 * rows], dtype=torch.int32, device=dev)
        row_req = torch.tensor([0] * rows + [1] * rows, dtype=torch.int32, device=dev)
        c = torch.empty(2 * rows, C, dtype=torch.float32, device=dev)
        K.causal_conv(u, 0, C, conv, None, K.ACT_SILU, tails, row_req, req_start, slots, c, None)
        o = torch.empty(2 * rows, nv, dtype=torch.float32, device=dev)
        K.delta_rule(c, (0, nk, 2 * nk), u, C, C + H, f32(W["A_log"]), f32(W["dt_bias"]), H, G, dk, dv, dk ** -0.5, 1e-6, state, req_start, slots, o)
        out = torch.empty(2 * rows, nv, dtype=torch.float32, device=dev)
        K.norm_gate(o, u, C + 2 * H, f32(W["norm"]), eps, H, dv, 1, K.ACT_SILU, out)
        got[0].append(out[:rows].cpu()); got[1].append(out[rows:].cpu())
    for i in range(2):
        o = torch.cat(got[i]).double().numpy()
        err = np.abs(o - want[i]).max() / np.abs(want[i]).max()
        assert err < 3e-5, f"sequence {i}: relative error {err}"
    assert torch.all(state[0] == 7.0) and torch.all(state[2] == 0.0) and torch.all(tails[0] == 7.0) and torch.all(tails[2] == 0.0)


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("experts,top,ff,limit,shared", [(5, 2, 40, 1.5, (24, 0.8)), (3, 3, 24, 0.5, None), (9, 1, 88, 2.0, (96, 2.0)), (70, 4, 9, 1.0, (8, 1.0))])
def test_biased_router_clamped_experts_and_the_gated_shared_unit(dtype, experts, top, ff, limit, shared):
    """The largest logits (product plus bias) choose, the softmax over the chosen ones weighs the units' outputs; the shared
    unit of the same clamped form, with its own limit, times a sigmoid gate per row.  The biases are large enough to change
    the choice, the inputs large enough for the limits to bite."""
    from infinicore_infer_b200.config import GLUSpec, RoutedExpertsSpec
    from infinicore_infer_b200.parts import RoutedExperts, Runtime
    from infinicore_infer_b200.weights import DictWeights
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    g = torch.Generator().manual_seed(experts)
    d = 48
    bf = lambda t: t.to(torch.bfloat16).double()
    W = {"router": bf(torch.randn(experts, d, generator=g)).numpy(), "router.b": bf(2.0 * torch.randn(experts, generator=g)).numpy()}
    names = [f"e{e}." for e in range(experts)] + (["shared."] if shared else [])
    for p in names:
        f = shared[0] if p == "shared." else ff
        W[p + "gate"] = bf(torch.randn(f, d, generator=g) * d ** -0.5).numpy()
        W[p + "up"] = bf(torch.randn(f, d, generator=g) * d ** -0.5).numpy()
        W[p + "down"] = bf(torch.randn(d, f, generator=g) * f ** -0.5).numpy()
    if shared:
        W["shared.sg"] = bf(torch.randn(1, d, generator=g) * d ** -0.5).numpy()
    mlp = {"router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    spec = RoutedExpertsSpec(hidden_size=d, num_experts=experts, top=top, expert_size=ff, act="swish_clamp", scale_input=False,
                             score_form="softmax_renorm", limit=limit, router_bias=True,
                             shared=GLUSpec(hidden_size=d, intermediate_size=shared[0], act="swish_clamp", limit=shared[1]) if shared else None,
                             shared_gate_name="sg" if shared else None)
    part = RoutedExperts(spec, DictWeights({n: torch.tensor(a) for n, a in W.items()}, dt, dev), "", Runtime(dt, dev))
    for T in (1, 5, 200):
        h = torch.randn(T, d, generator=g, dtype=F) * 2.0
        if dt == torch.bfloat16:
            h = bf(h)
        margins = []
        want = plain.experts_ff(h.numpy(), mlp, W, "", margins)
        unbiased = np.argsort(-(h.numpy() @ W["router"].T), axis=-1)[:, :top]
        assert T < 5 or (np.sort(unbiased, -1) != np.sort(plain.route(h.numpy(), W, "", top)[0], -1)).any() or top == experts
        got = part.forward(h.to(dt).to(dev).contiguous(), None).double().cpu().numpy()
        sure = margins[0] >= CLOSE_CALL[dtype]
        err = (np.abs(got - want).max(1) * sure).max()
        assert err <= (3e-5 if dt == torch.float32 else 3e-2) * max(np.abs(want).max(), 1.0), f"{T} rows: {err}"


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_position_vectors_and_a_row_for_every_pass(dtype):
    from infinicore_infer_b200 import kernels as K
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    g = torch.Generator().manual_seed(5)
    x = torch.randn(9, 20, generator=g).to(dev)
    table = torch.randn(30, 20, generator=g).to(dt).to(dev)
    pos = torch.tensor([3, 4, 5, 0, 29, 7, 7, 1, 2], dtype=torch.int32, device=dev)
    want = x.double() + table.double()[pos.long()]
    got = K.add_rows(x.clone(), table, pos)
    assert (got.double() - want).abs().max() < 1e-6
    got = K.add_rows(x.clone(), table, None, row=11)
    assert (got.double() - (x.double() + table.double()[11])).abs().max() < 1e-6


# ---- generation through the scheduler ---------------------------------------------------------------------------------
def test_greedy_generation_through_the_scheduler_matches_the_plain_model(folders):
    """Requests of unequal length through ``Generator`` (admission, portions of 16 tokens, decoding beside prompts, three
    slots for five requests): every generated token is the plain model's argmax given the tokens before it."""
    from infinicore_infer_b200.engine import Engine, Generator
    d, cfg, w = folders["looped"]
    eng = Engine.from_folder(d, dtype=torch.float32, max_tokens=160, cache_tokens=3 * 96, page_size=16, max_requests=3, max_step_tokens=64)
    gen = Generator(eng, chunk_size=16)
    prompts = [random_tokens(900 + i, n, cfg["vocab"]) for i, n in enumerate((40, 3, 25, 61, 12))]
    outs = gen.generate(prompts, max_new_tokens=12)
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        logits = plain.forward(cfg, w, p + o)
        for j, tok in enumerate(o):
            row = logits[len(p) + j - 1]
            best = int(row.argmax())
            assert tok == best or row[best] - row[tok] < 1e-4 * np.abs(row).max(), f"token {j} of a prompt of {len(p)}"
    eng.cache.check_invariants()


def test_command_line_runs_a_small_model_with_random_weights(tmp_path):
    """``--random fapenex-tiny`` with three prompts through the scheduler, greedy: the printed tokens are the plain model's."""
    import re
    import subprocess
    import sys
    from infinicore_infer_b200.config import PRESETS, FapenexConfig
    from infinicore_infer_b200.weights import index_directory, read_tensor, write_model_folder
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    preset = PRESETS["fapenex-tiny"]
    proc = subprocess.run([sys.executable, "-m", "infinicore_infer_b200.jiuge", "--nvidia", "--random", "fapenex-tiny", "--seed", "3",
                           "--prompt-lens", "2,19,40", "--chunk-size", "11", "--num-pages", "24", "--max-batch", "3",
                           "--max-tokens-per-step", "24", "--temperature", "0", "--max-steps", "8", "--dtype", "float32"],
                          capture_output=True, text=True, cwd=root, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = {int(m.group(1)): [int(t) for t in m.group(2).split()] for m in re.finditer(r"request (\d+): ([\d ]*)", proc.stdout)}
    assert sorted(got) == [0, 1, 2]
    cfg = FapenexConfig.from_dict(preset.config)
    write_model_folder(cfg, str(tmp_path), seed=3, std=preset.std, norm_std=preset.norm_std)
    w = {n: read_tensor(i).double().numpy() for n, i in index_directory(str(tmp_path)).items()}
    for k, n in enumerate((2, 19, 40)):
        prompt = torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(3 + k)).tolist()
        assert len(got[k]) == 8
        logits = plain.forward(cfg.to_dict(), w, prompt + got[k])
        for j, tok in enumerate(got[k]):
            row = logits[n + j - 1]
            assert tok == int(row.argmax()) or row.max() - row[tok] < 1e-4 * np.abs(row).max(), f"request {k}, token {j}"
