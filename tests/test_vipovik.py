"""Vipovik through the engine against the plain implementation (tests/plain_vipovik.py): each mechanism alone, whole
models of several sizes and layer orders, prompts cut in every way, batches, reused pages and state slots, keys at the
window's edges and among the kept first ones, long decoding, and greedy generation through the scheduler."""
import json
import math
import os

import numpy as np
import pytest
import torch

from conftest import random_tokens
import plain_vipovik as plain
from trace_helpers import by_position, mixed, portions, staggered_plan, tail_decode, whole

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 5e-2}
F = torch.float64


def left(heads, kv_heads, dim, vdim, scale, cap, window, keep, rot_dims, base=1e4, scaling=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": cap}
    if window is not None:
        out["mask"] = {"size": window, "keep_first": keep}
    if rot_dims:
        out["rot"] = {"base": base, "dims": rot_dims}
        if scaling is not None:
            out["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def layer(left_, right_heads, right_dim, rank, scales=(1.0, 1.0), mlp=None):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left_, "right": {"heads": right_heads, "dim": right_dim, "rank": rank},
                      "left_scale": scales[0], "right_scale": scales[1]}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}


def config(width, vocab, layers, loop=None, scale=3.0, eps=1e-5):
    out = {"architecture": "Vipovik", "embedding": {"scale": scale}, "norm": {"eps": eps}, "vocab": vocab, "width": width, "layers": layers}
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


# Sizes that differ from one another in everything: key and value sizes that are unequal, as many key heads as query
# heads and fewer, rotation of a part of a head, of the whole head and none, with and without stretched frequencies,
# windows shorter than a page, no multiple of one and longer than every prompt here, no window, no kept keys, one and
# several (more than a page of them), one expert a row, several and all, layers without feed-forward, a span that runs
# twice or three times from the first layer or later to the last or earlier, no span, recurrences whose heads are no
# multiple of anything, factors of the two sides that are 1, unequal and 0.
MODELS = {
    "one": config(64, 97, [layer(left(4, 2, 16, 24, 0.3, 12.0, 21, 3, 8), 3, 8, 5, (0.7, 0.4), dense(72))]),
    "routed": config(64, 101, [layer(left(2, 2, 32, 16, 0.2, 30.0, 16, 1, 32, 5e4, (4.0, 64, 8.0, 2.0)), 2, 24, 4, (0.5, 0.6), moe(5, 2, 40, 1.5)),
                               layer(left(3, 1, 8, 8, 0.4, 8.0, 7, 0, 0), 4, 16, 7, (1.0, 1.0), moe(3, 3, 24, 0.7))], eps=1e-6),
    "looped": config(96, 211, [layer(left(4, 4, 24, 8, 0.25, 15.0, 40, 17, 12, 300.0), 1, 40, 6, (0.9, 0.3), dense(80)),
                               layer(left(6, 2, 16, 16, 0.3, 20.0, 33, 2, 16, 1e4, (8.0, 32, 16.0, 1.0)), 5, 8, 3, (0.6, 0.5), moe(6, 1, 32, 2.5)),
                               layer(left(2, 1, 48, 40, 0.15, 25.0, 300, 4, 24), 3, 24, 9, (0.4, 0.8), None),
                               layer(left(1, 1, 64, 64, 0.125, 18.0, None, 0, 64, 2.5e5, (4.0, 128, 32.0, 1.0)), 2, 32, 8, (1.0, 0.0), dense(56))],
                     loop=(1, 3, 3)),
    "loop-all": config(64, 130, [layer(left(2, 1, 24, 32, 0.35, 10.0, 9, 5, 12, 1e3), 2, 16, 4, (0.5, 0.5), moe(4, 2, 48, 1.0)),
                                 layer(left(4, 2, 8, 16, 0.5, 6.0, 18, 1, 8), 4, 8, 2, (0.8, 0.7), dense(40))], loop=(0, 2, 2), scale=8.0, eps=3e-6),
    "loop-tail": config(80, 77, [layer(left(5, 5, 16, 16, 0.3, 14.0, 25, 2, 16), 1, 16, 3, (0.3, 1.1), dense(64)),
                                 layer(left(2, 2, 40, 24, 0.2, 22.0, 12, 12, 20, 777.0, (2.0, 16, 4.0, 0.5)), 3, 24, 5, (0.7, 0.7), moe(7, 3, 24, 3.0)),
                                 layer(left(4, 1, 16, 32, 0.3, 9.0, 50, 3, 4), 2, 40, 4, (1.0, 0.5), None)], loop=(1, 3, 2)),
    # nothing a multiple of anything: odd width, odd sizes everywhere, a prime vocabulary
    "awkward": config(50, 61, [layer(left(3, 3, 10, 7, 0.4, 11.0, 13, 2, 6, 555.0), 3, 5, 3, (0.6, 0.9), moe(2, 1, 11, 1.2)),
                               layer(left(2, 1, 6, 9, 0.5, 5.0, 5, 1, 2), 1, 7, 2, (1.2, 0.4), dense(21))], loop=(0, 1, 3)),
    # heads of 64 and 128 for keys, values and the recurrence, as the tensor-core attention kernels and the scan's instances for
    # whole heads take them; prompts longer than a piece of the scan
    "wide": config(256, 333, [layer(left(4, 2, 64, 64, 0.125, 20.0, 48, 2, 64, 1e4, (4.0, 64, 16.0, 1.0)), 3, 64, 32, (0.6, 0.5), dense(512)),
                              layer(left(2, 1, 128, 128, 0.09, 25.0, 100, 3, 64), 2, 128, 64, (0.5, 0.7), moe(4, 2, 128, 2.0))],
                   loop=(1, 2, 2), scale=4.0),
}
STD = 0.16     # matrices N(0, STD): products keep their input's spread, so scores, gates and routers are far from flat
STDS = {"wide": 0.08}       # the same for rows four times as wide


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """(folder, config.json as written, float64 weights) of every model.  The written configuration does not say how wide a
    recurrence's decay projection is: the engine reads that from the checkpoint's shapes."""
    from infinicore_infer_b200.config import config_class_for
    from infinicore_infer_b200.weights import index_directory, read_tensor, write_model_folder
    out = {}
    for seed, (name, cfg) in enumerate(MODELS.items()):
        d = str(tmp_path_factory.mktemp("vipovik_" + name))
        write_model_folder(config_class_for(cfg).from_dict(cfg), d, seed=seed + 51, std=STDS.get(name, STD), norm_std=0.2)
        path = os.path.join(d, "config.json")
        with open(path) as f:
            disk = json.load(f)
        for entry in disk["layers"]:
            entry["mixer"]["right"].pop("rank")
        with open(path, "w") as f:
            json.dump(disk, f)
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
# A row whose router leaves the last chosen expert this close (in the router's output) to the first one left out may go to
# another expert once the activations are rounded to bfloat16: such a row's logits are those of another, equally valid,
# choice, and are not compared.  (float32 reproduces every choice.)
CLOSE_CALL = {"float32": 1e-4, "bfloat16": 0.08}


class Expected(np.ndarray):
    """Logits [T, vocab] with ``margin`` [T]: the smallest router margin of each row over the model's routed layers."""


def expected(folders, name, seed, n):
    key = (name, seed, n)
    if key not in _plain:
        _, cfg, w = folders[name]
        toks = random_tokens(seed, n, cfg["vocab"])
        margins = []
        want = plain.forward(cfg, w, toks, margins=margins).view(Expected)
        want.margin = np.stack(margins).min(0) if margins else np.full(n, np.inf)
        _plain[key] = (toks, want)
    return _plain[key]


def run(engine, steps):
    from infinicore_infer_b200.trace import replay
    return by_position(steps, replay(engine, steps))


def check(got, rid, want, tol, what):
    """float32: every logit of every position within ``tol`` of the logits' scale: the sharp test.  bfloat16: the difference
    of a position's logits (its mean taken off, root mean square over the vocabulary) against the spread of the logits: half
    the rows within ``tol``, nine in ten within three times it, all within half the logits' spread.  Rows whose router call
    is close are left out (``CLOSE_CALL``)."""
    loose = tol > 1e-3
    margin = getattr(want, "margin", np.full(len(want), np.inf))
    sure = margin >= CLOSE_CALL["bfloat16" if loose else "float32"]
    assert len(want) < 20 or sure.sum() >= 0.5 * len(want), f"{what}: the router is sure of {int(sure.sum())} of {len(want)} rows only"
    want = np.asarray(want, dtype=np.float64)
    diff = np.stack([got[(rid, p)].astype(np.float64) - want[p] for p in range(len(want))])
    if not loose:
        errs, scale = np.abs(diff).max(1) * sure, np.abs(want).max()
        worst = int(errs.argmax())
        assert errs.max() <= tol * scale, f"{what}: request {rid} position {worst}: error {errs.max():.3e} > {tol * scale:.3e}"
        return
    scale = (want - want.mean(1, keepdims=True)).std()
    errs = ((diff - diff.mean(1, keepdims=True)).std(1) / scale)[sure]
    if not len(errs):
        return
    assert np.median(errs) <= tol, f"{what}: request {rid}: the median row differs by {np.median(errs):.3f} of the logits' spread"
    assert (errs > 3 * tol).sum() <= max(1, len(errs) // 10), f"{what}: request {rid}: {(errs > 3 * tol).sum()} of {len(errs)} rows beyond {3 * tol}"
    assert errs.max() <= 0.5, f"{what}: request {rid}: a row differs by {errs.max():.3f} of the logits' spread"


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
    """Long decoding: every token a step of its own (captured steps), so pages, the shifted row and the states move one
    position at a time, the window passes over decoded tokens and leaves the kept ones behind."""
    for name in ("looped", "loop-tail", "routed"):
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


def test_a_reused_slot_starts_from_zero_state_and_no_shifted_row(folders, engines):
    """The same request twice in a row lands in the slot (and pages) that its first run left: the state, and the last row
    that the shift keeps, start from zero again."""
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
    assert [e.before.step_index if e.before else None for e in spec.order] == [None, 0, None, 1, None, 2, None, None]
    needs, states = cache_needs(spec), state_needs(spec)
    assert (needs[0].num_kv_heads, needs[0].head_dim, needs[0].v_head_dim, needs[0].window, needs[0].keep_first) == (4, 24, 8, 40, 17)
    assert needs[7].window is None and needs[7].keep_first == 0
    # beside the pages: the recurrence's state and the last row that the shift reads
    assert [s.shape for s in states[1].slots] == [(5, 8, 8), (96,)] and [s.shape for s in states[7].slots] == [(2, 32, 32), (96,)]
    assert spec.layers[1].mixer.right.decay_rank == 3           # read from the checkpoint's shapes


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


def edge_case(T, H, G, dk, dv, window, keep, seed, bf16):
    """Queries, keys and values in which, for chosen rows i, head 0 scores the key just outside the window (i - W) above
    the key just inside (i - W + 1) above all others, and head 1 scores the first key that is not kept (position `keep`)
    above the last kept one (keep - 1) above all others: a window or a count that is one off in either direction moves
    the row's output from one value to another.  The scores are large enough for the cap to bend them."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, H, dk, generator=g, dtype=F)
    k = 0.3 * torch.randn(T, G, dk, generator=g, dtype=F)
    v = torch.randn(T, G, dv, generator=g, dtype=F)
    rows = list(range(window + keep + 3, T, 5))
    marks = torch.randn(2, dk, generator=g, dtype=F)
    marks[1] -= marks[0] * (marks[0] @ marks[1]) / (marks[0] @ marks[0])       # two directions at right angles
    if keep > 0:
        k[keep - 1, 0], k[keep, 0] = marks[0], marks[1]
    for i in rows:                                # heads 0 and 1 read key head 0
        unit = q[i, 0] / (q[i, 0] @ q[i, 0])
        k[i - window, 0] = 14.0 * unit
        k[i - window + 1, 0] = 9.0 * unit
        if keep > 0:
            q[i, 1] = 10.0 * marks[0] / (marks[0] @ marks[0]) + 15.0 * marks[1] / (marks[1] @ marks[1])
    if bf16:
        q, k, v = (t.to(torch.bfloat16).double() for t in (q, k, v))
    return q, k, v, rows


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("window,keep,page,cap", [(7, 3, 8, 12.0), (16, 1, 16, 0.0), (33, 20, 8, 9.0), (40, 0, 16, 20.0), (64, 16, 16, 15.0)])
def test_window_edges_kept_first_keys_and_cap_of_the_row_attention(dtype, window, keep, page, cap):
    """The kernel of one warp a row and head: whole prompts and single decoded rows, values of another size than keys."""
    from infinicore_infer_b200 import kernels as K
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    T, H, G, dk, dv = 150, 4, 2, 24, 40
    q, k, v, rows = edge_case(T, H, G, dk, dv, window, keep, window, dt == torch.bfloat16)
    mask = {"size": window, "keep_first": keep}
    want = plain.capped_attention(q.numpy(), k.numpy(), v.numpy(), 1.0, cap, mask, np.arange(T))
    off_by_one = [plain.capped_attention(q.numpy(), k.numpy(), v.numpy(), 1.0, cap, {"size": window + a, "keep_first": keep + b}, np.arange(T))
                  for a, b in ((1, 0), (-1, 0)) + (((0, 1), (0, -1)) if keep else ())]
    for other in off_by_one:                      # the inputs do tell a window or a count that is one off
        assert np.abs(other - want)[rows].max() > 0.3
    kp, vp, table = paged(k, v, page, dev, dt)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    out = torch.empty(T, H, dv, dtype=dt, device=dev)
    K.attention_rows(q.to(dt).to(dev).contiguous(), kp, vp, out, pos, torch.zeros_like(pos), table, T, H, 1.0, window, cap=cap, keep_first=keep)
    tol = 2e-5 if dt == torch.float32 else 3e-2
    err = np.abs(out.double().cpu().numpy() - want).max()
    assert err <= tol, f"prompt rows differ by {err}"
    for i in rows[-4:] + [0, keep, window]:       # the same rows one by one, as a decode step sees them
        one = torch.empty(1, H, dv, dtype=dt, device=dev)
        K.attention_rows(q[i:i + 1].to(dt).to(dev).contiguous(), kp, vp, one, pos[i:i + 1], torch.zeros(1, dtype=torch.int32, device=dev), table,
                         1, H, 1.0, window, cap=cap, keep_first=keep)
        assert np.abs(one.double().cpu().numpy()[0] - want[i]).max() <= tol, f"decoded row {i}"


@pytest.mark.parametrize("dh", [32, 64, 128])
@pytest.mark.parametrize("window,keep,cap", [(40, 3, 12.0), (64, 16, 0.0), (130, 70, 9.0), (200, 0, 20.0), (17, 1, 15.0), (128, 5, 10.0)])
def test_window_edges_kept_first_keys_and_cap_on_the_tensor_cores(dh, window, keep, cap):
    """The bfloat16 kernels of the generation path: tiles of a prompt's rows (a whole prompt, and a portion that starts in
    the middle of a page behind cached keys), and single rows whose keys are cut into ranges.  Kept keys that fill less than
    a tile of keys, more than one, and none; windows shorter and longer than a tile."""
    from infinicore_infer_b200 import kernels as K
    dev, dt = torch.device("cuda:0"), torch.bfloat16
    T, H, G, page = 333, 4, 2, 16
    q, k, v, rows = edge_case(T, H, G, dh, dh, window, keep, window + dh, True)
    mask = {"size": window, "keep_first": keep}
    want = plain.capped_attention(q.numpy(), k.numpy(), v.numpy(), 1.0, cap, mask, np.arange(T))
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
                K.attention_tcgen05(qd[start:].contiguous(), kp, vp, out, tiles, len(tiles), n, req_start, req_pos, table, H, 1.0, window,
                                    cap=cap, keep_first=keep)
                K.check_gemm_status(dev)
            else:
                fn(qd[start:].contiguous(), kp, vp, out, tiles, len(tiles), req_start, req_pos, table, H, 1.0, window, cap=cap, keep_first=keep)
            err = np.abs(out.double().cpu().numpy() - want[start:]).max()
            assert err <= 3e-2, f"{name} from position {start}: {err}"
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    some = torch.tensor(rows[-6:] + [0, keep, window, window + 1], dtype=torch.int32, device=dev)
    for splits in (1, 3, 8):
        out = torch.zeros(T, H, dh, dtype=dt, device=dev)
        K.attention_decode(qd, kp, vp, out, some, len(some), pos, torch.zeros_like(pos), table, H, 1.0, window, splits, cap=cap, keep_first=keep)
        got = out.double().cpu().numpy()
        for i in some.tolist():
            assert np.abs(got[i] - want[i]).max() <= 3e-2, f"single row {i}, {splits} ranges"


@pytest.mark.parametrize("dtype", list(DTYPES))
def test_rotation_in_halves_unit_norm_and_cache_rows(dtype):
    """Two requests side by side at unequal positions in scrambled pages: each head's leading elements rotated in halves by
    stretched frequencies, the rest passed on, then every head of q and k divided by its root mean square; values as they
    come; keys and values land in the pages at the rows' positions."""
    from infinicore_infer_b200 import kernels as K
    from infinicore_infer_b200.config import FrequencyRampSpec, PairRotarySpec
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    H, G, dk, dv, dims, page, eps = 4, 2, 24, 16, 16, 8, 1e-3
    rot = {"dims": dims, "base": 300.0, "scaling": {"factor": 4.0, "original": 32, "fast": 4.0, "slow": 1.0}}
    spec = PairRotarySpec(dims=dims, base=300.0, scaling=FrequencyRampSpec(4.0, 32.0, 4.0, 1.0, magnitude_slope=0.1), layout="halves")
    f, mag = spec.frequencies()
    pf, pm = plain.rotary_frequencies(rot)
    assert np.allclose(f, pf, rtol=1e-12) and abs(mag - pm) < 1e-12 and abs(mag - (0.1 * math.log(4.0) + 1)) < 1e-12
    assert f[0] == 1.0 and abs(f[-1] - 300.0 ** (-14 / 16) / 4.0) < 1e-12      # the fastest pair keeps its frequency, the slowest is stretched
    g = torch.Generator().manual_seed(2)
    starts, n = (3, 41), 30
    nq, nk, nv = H * dk, G * dk, G * dv
    ld = nq + nk + nv + 5
    u = torch.randn(2 * n, ld, generator=g, dtype=F) * 2.0
    pos = np.concatenate([np.arange(s, s + n) for s in starts])
    blocks = (max(starts) + n + page - 1) // page
    table = torch.tensor([[2 * b + 2 for b in range(blocks)], [2 * b + 1 for b in range(blocks)]], dtype=torch.int32, device=dev)
    kp = torch.zeros(2 * blocks + 1, G, page, dk, dtype=dt, device=dev)
    vp = torch.zeros(2 * blocks + 1, G, page, dv, dtype=dt, device=dev)
    q_out = torch.empty(2 * n, H, dk, dtype=dt, device=dev)
    K.conv_qkv(u.float().to(dev), (0, nq, nq + nk), H, G, dk, dv, True, (None, None, None), 0, (None, None), eps,
               torch.tensor(f, dtype=torch.float32, device=dev), dims, None, torch.tensor(pos, dtype=torch.int32, device=dev),
               torch.tensor([0] * n + [1] * n, dtype=torch.int32, device=dev), torch.tensor([0, n, 2 * n], dtype=torch.int32, device=dev),
               torch.tensor([1, 2], dtype=torch.int32, device=dev), table, page, q_out, kp, vp, rot_half=True, rot_mag=mag, head_norm=True)
    uf = u.float().double().numpy()
    q = plain.rms_unit(plain.rotate_half(uf[:, :nq].reshape(2 * n, H, dk), pos, rot), eps)
    k = plain.rms_unit(plain.rotate_half(uf[:, nq:nq + nk].reshape(2 * n, G, dk), pos, rot), eps)
    v = uf[:, nq + nk:nq + nk + nv].reshape(2 * n, G, dv)
    tol = 2e-5 if dt == torch.float32 else 2e-2
    assert np.abs(q_out.double().cpu().numpy() - q).max() < tol * np.abs(q).max()
    for r in range(2 * n):
        pg, at = table[r // n, pos[r] // page].item(), pos[r] % page
        assert np.abs(kp[pg, :, at].double().cpu().numpy() - k[r]).max() < tol * np.abs(k).max(), f"key of row {r}"
        assert np.abs(vp[pg, :, at].double().cpu().numpy() - v[r]).max() < tol * np.abs(v).max(), f"value of row {r}"


@pytest.mark.parametrize("H,dk,rank", [(1, 40, 6), (3, 24, 5), (2, 64, 16), (5, 7, 3), (2, 128, 4)])
def test_shift_decay_and_bonus_recurrence_across_cuts_and_slots(H, dk, rank):
    """Two sequences cut into portions (down to one row; one longer than a piece of the scan) that go through state slots
    side by side: the shifted mixtures from the kept last row, decays exp(-exp(.)) behind a tanh, the bonus on a row's own
    key, a unit norm per head times a weight and a silu gate.  An early key is made large and its channels' decay slow, so
    that a lost state, a wrong decay, or a row that reads its own decay moves late outputs.  All of it in float32."""
    from infinicore_infer_b200 import kernels as K
    from infinicore_infer_b200.parts import LinearAttention
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(H * dk)
    T, d, eps = 230, 48, 1e-4
    n = H * dk
    W = {"mu." + s: torch.rand(d, generator=g, dtype=F).numpy() for s in "rkvgw"}
    for s in "rkvg":
        W[s] = (torch.randn(n, d, generator=g, dtype=F) * d ** -0.5).numpy()
    W["w1"] = (torch.randn(rank, d, generator=g, dtype=F) * d ** -0.5).numpy()
    W["w2"] = (torch.randn(n, rank, generator=g, dtype=F) * 0.5).numpy()
    W["w0"] = (torch.randn(n, generator=g, dtype=F) - 3.0).numpy()             # slow decays: exp(-exp(-3)) = 0.95
    W["u"] = torch.randn(H, dk, generator=g, dtype=F).numpy()
    W["norm"] = (1 + 0.3 * torch.randn(n, generator=g, dtype=F)).numpy()
    W["o"] = np.eye(n)
    hs = [torch.randn(T, d, generator=g, dtype=F).float().double().numpy() for _ in range(2)]
    hs[0][1] *= 6.0                               # an early row that late rows still see
    m = {"heads": H, "dim": dk}
    want = [plain.time_mix(h, m, W, "", eps)[0] for h in hs]
    mu = torch.tensor(np.stack([W["mu." + s] for s in "rkvgw"]), dtype=torch.float32, device=dev)
    w_in = [torch.tensor(W[s], dtype=torch.float64) for s in ("r", "k", "v", "g", "w1")]
    state = torch.zeros(4, H, dk, dk, dtype=torch.float32, device=dev)
    last = torch.zeros(4, d, dtype=torch.float32, device=dev)
    state[0], last[0] = 7.0, 7.0                  # slot 0 is nobody's; what lies there must not matter
    slots = torch.tensor([3, 1], dtype=torch.int32, device=dev)
    got = [[], []]
    cuts = [0, 1, 2, 4, 30, 31, 180, 225, T]      # 149 rows in one portion: more than a piece of the scan
    for a, b in zip(cuts, cuts[1:]):
        rows = b - a
        h = torch.tensor(np.concatenate([hs[0][a:b], hs[1][a:b]]), dtype=torch.float32, device=dev)
        req_start = torch.tensor([0, rows, 2 * rows], dtype=torch.int32, device=dev)
        row_req = torch.tensor([0] * rows + [1] * rows, dtype=torch.int32, device=dev)
        mixes = torch.empty(5, 2 * rows, d, dtype=torch.float32, device=dev)
        K.token_shift(h, mu, last, row_req, req_start, slots, mixes)
        u = torch.cat([mixes[i].double().cpu() @ w_in[i].T for i in range(5)], dim=1).float().to(dev)      # the products, here on the host
        caps = LinearAttention.step_list_capacity(2 * rows, 2)
        arrays = {name: np.zeros(max(1, c), dtype=np.int32) for name, c in caps.items()}
        counts = LinearAttention.fill_step_lists(2, 2, [rows, rows], [a, a], arrays)
        lists = {name: torch.from_numpy(arrays[name][:max(1, counts[name][0] * w)]).to(dev) if counts[name][0] else None
                 for name, w in (("direct", 1), ("pieces", 2), ("piece_reqs", 3))}
        o = torch.empty(2 * rows, n, dtype=torch.float32, device=dev)
        K.linear_scan(u, (0, n, 2 * n), H, dk, dk, K.ACT_NONE, 1.0, None, torch.tensor(W["w2"], dtype=torch.float32, device=dev),
                      torch.tensor(W["w0"], dtype=torch.float32, device=dev), 4 * n, 0.0, state, req_start, slots, o, direct=lists["direct"],
                      pieces=lists["pieces"], piece_reqs=lists["piece_reqs"], bonus=torch.tensor(W["u"], dtype=torch.float32, device=dev),
                      decay_form=1, rank_act=K.ACT_TANH)
        out = torch.empty(2 * rows, n, dtype=torch.float32, device=dev)
        K.norm_gate(o, u, 3 * n, torch.tensor(W["norm"], dtype=torch.float32, device=dev), eps, H, dk, 2, K.ACT_SILU, out)
        got[0].append(out[:rows].cpu()); got[1].append(out[rows:].cpu())
    for i in range(2):
        o = torch.cat(got[i]).double().numpy()
        err = np.abs(o - want[i]).max() / np.abs(want[i]).max()
        assert err < 3e-5, f"sequence {i}: relative error {err}"
    assert torch.all(state[0] == 7.0) and torch.all(state[2] == 0.0) and torch.all(last[0] == 7.0) and torch.all(last[2] == 0.0)
    assert np.abs(last[3].double().cpu().numpy() - hs[0][-1]).max() < 1e-6 and np.abs(last[1].double().cpu().numpy() - hs[1][-1]).max() < 1e-6


@pytest.mark.parametrize("dtype", list(DTYPES))
@pytest.mark.parametrize("experts,top,ff,limit", [(5, 2, 40, 1.5), (3, 3, 24, 0.5), (9, 1, 88, 2.0), (70, 4, 9, 1.0)])
def test_softmax_routed_clamped_experts_choose_weigh_and_add_up(dtype, experts, top, ff, limit):
    """Scores by a softmax over all experts, the chosen ones' scores divided by their sum, on the units' outputs; the unit
    with its gate cut off above and its other half on both sides.  The inputs are large enough for the limits to bite."""
    from infinicore_infer_b200 import kernels as K
    dev, dt = torch.device("cuda:0"), DTYPES[dtype]
    g = torch.Generator().manual_seed(experts)
    d = 48
    for T in (1, 5, 200):
        h = torch.randn(T, d, generator=g, dtype=F) * 2.0
        if dt == torch.bfloat16:
            h = h.to(dt).double()
        W = {"router": torch.randn(experts, d, generator=g, dtype=F).numpy()}
        for e in range(experts):            # matrices as a 16-bit checkpoint holds them
            W[f"e{e}.gate"] = (torch.randn(ff, d, generator=g) * d ** -0.5).to(torch.bfloat16).double().numpy()
            W[f"e{e}.up"] = (torch.randn(ff, d, generator=g) * d ** -0.5).to(torch.bfloat16).double().numpy()
            W[f"e{e}.down"] = (torch.randn(d, ff, generator=g) * ff ** -0.5).to(torch.bfloat16).double().numpy()
        mlp = {"router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
        want = plain.experts_ff(h.numpy(), mlp, W, "")
        clipped = np.abs(h.numpy() @ W["e0.up"].T) > limit
        assert T < 5 or 0.02 < clipped.mean() < 0.98
        delta = torch.full((T, d), 9.0, dtype=torch.float32, device=dev)
        w_gu = torch.tensor(np.concatenate([W[f"e{e}.{n}"] for e in range(experts) for n in ("gate", "up")])).to(dt).to(dev).contiguous()
        w_dn = torch.tensor(np.concatenate([W[f"e{e}.down"] for e in range(experts)])).to(dt).to(dev).contiguous()
        K.routed_experts(h.to(dt).to(dev).contiguous(), torch.tensor(W["router"], dtype=torch.float32, device=dev), w_gu, w_dn, delta, False,
                         experts, top, K.ACT_SWISH_CLAMP, score_form=1, limit=limit)
        err = np.abs(delta.double().cpu().numpy() - want).max()
        assert err <= (3e-5 if dt == torch.float32 else 2e-2) * max(np.abs(want).max(), 1.0), f"{T} rows: {err}"


def test_exact_gelu_between_the_products_of_a_feed_forward_without_a_gate():
    from infinicore_infer_b200 import kernels as K
    dev = torch.device("cuda:0")
    u = torch.randn(9, 70, generator=torch.Generator().manual_seed(1), dtype=F) * 3
    out = torch.empty(9, 64, dtype=torch.float32, device=dev)
    K.act_rows(u.float().to(dev)[:, 3:67], out, K.ACT_GELU_ERF)
    assert np.abs(out.double().cpu().numpy() - plain.gelu_erf(u.float().double().numpy()[:, 3:67])).max() < 1e-5


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
    """``--random vipovik-tiny`` with three prompts through the scheduler, greedy: the printed tokens are the plain model's."""
    import re
    import subprocess
    import sys
    from infinicore_infer_b200.config import PRESETS, VipovikConfig
    from infinicore_infer_b200.weights import index_directory, read_tensor, write_model_folder
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    preset = PRESETS["vipovik-tiny"]
    proc = subprocess.run([sys.executable, "-m", "infinicore_infer_b200.jiuge", "--nvidia", "--random", "vipovik-tiny", "--seed", "3",
                           "--prompt-lens", "2,19,40", "--chunk-size", "11", "--num-pages", "24", "--max-batch", "3",
                           "--max-tokens-per-step", "24", "--temperature", "0", "--max-steps", "8", "--dtype", "float32"],
                          capture_output=True, text=True, cwd=root, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = {int(m.group(1)): [int(t) for t in m.group(2).split()] for m in re.finditer(r"request (\d+): ([\d ]*)", proc.stdout)}
    assert sorted(got) == [0, 1, 2]
    cfg = VipovikConfig.from_dict(preset.config)
    write_model_folder(cfg, str(tmp_path), seed=3, std=preset.std, norm_std=preset.norm_std)
    w = {n: read_tensor(i).double().numpy() for n, i in index_directory(str(tmp_path)).items()}
    for k, n in enumerate((2, 19, 40)):
        prompt = torch.randint(0, cfg.vocab, (n,), generator=torch.Generator().manual_seed(3 + k)).tolist()
        assert len(got[k]) == 8
        logits = plain.forward(cfg.to_dict(), w, prompt + got[k])
        for j, tok in enumerate(got[k]):
            row = logits[n + j - 1]
            assert tok == int(row.argmax()) or row.max() - row[tok] < 1e-4 * np.abs(row).max(), f"request {k}, token {j}"
