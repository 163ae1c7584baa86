"""Fapenex without a GPU: the configuration, the run order of a looped span, the manifest, what the cache keeps for a window
and for chunks, and the plain implementation's own small cases."""
import numpy as np
import pytest

import plain_fapenex as plain
from infinicore_infer_b200.config import ConfigError, FapenexConfig, config_class_for
from infinicore_infer_b200.parts import cache_needs, model_manifest, state_needs


def cfg(loop=None, cap=7.0):
    layers = [
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "conv": 3},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 8, "limit": 1.5}, "shared": {"ff": 12, "limit": 0.5}}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.3, "mask": {"size": 5},
                                        "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}}},
         "mlp": {"kind": "moe", "router": {"experts": 5, "top": 1}, "expert": {"ff": 4, "limit": 2.5}}},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 4, "vdim": 6, "kv_rank": 8, "q_rank": 12, "scale": 0.4, "mask": {"size": 3}},
         "mlp": None},
    ]
    out = {"architecture": "Fapenex", "norm": {"eps": 1e-5}, "vocab": 40, "width": 16, "max_positions": 64, "logit_scale": 1.7,
           "logit_softcap": cap, "layers": layers}
    if loop:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


def test_the_registry_finds_the_configuration_and_it_reads_back():
    c = config_class_for(cfg())
    assert c is FapenexConfig
    typed = c.from_dict(cfg(loop=(1, 3, 2)), max_tokens=48)
    assert typed.max_positions == 48 and typed.position_rows == 64 and typed.loop == (1, 3, 2) and typed.tie_word_embeddings
    assert typed.logit_scale == 1.7 and typed.logit_softcap == 7.0
    assert FapenexConfig.from_dict(typed.to_dict(), max_tokens=48) == typed
    assert FapenexConfig.from_dict(cfg(), max_tokens=1000).max_positions == 64          # no sequence outgrows the position table
    bare = FapenexConfig.from_dict(cfg(cap=None))
    assert bare.logit_softcap == 0.0 and bare.model_spec().logit_softcap == 0.0


def test_run_order_of_a_span_that_runs_several_times():
    spec = FapenexConfig.from_dict(cfg(loop=(0, 2, 3))).model_spec()
    assert [e.layer for e in spec.order] == [0, 1, 0, 1, 0, 1, 2]
    assert [e.cache for e in spec.order] == list(range(7))
    assert [(e.before.index, e.before.steps) if e.before else None for e in spec.order] == [(0, 3), None, (1, 3), None, (2, 3), None, None]
    assert [(i, t) for i, t, _ in FapenexConfig.from_dict(cfg(loop=(0, 2, 3))).run_order()] == \
        [(i, None if t is None else t) for i, t in [(0, 0), (1, 0), (0, 1), (1, 1), (0, 2), (1, 2), (2, None)]]
    assert plain.run_order(cfg(loop=(0, 2, 3))) == [(0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None), (2, None)]
    once = FapenexConfig.from_dict(cfg()).model_spec().order
    assert [e.layer for e in once] == [0, 1, 2] and all(e.before is None for e in once)
    needs, states = cache_needs(spec), state_needs(spec)
    assert needs[0].shape == (4, 6, 10) and states[0].shape == (2, 2 * 12 + 40)
    assert (needs[1].num_kv_heads, needs[1].head_dim, needs[1].v_head_dim, needs[1].window) == (2, 6, 10, 5) and states[1] is None
    assert (needs[6].num_kv_heads, needs[6].head_dim, needs[6].v_head_dim, needs[6].window, needs[6].values_in_keys) == (1, 8, 8, 3, True)
    assert needs[1] == needs[3] and needs[0] == needs[2]


def test_manifest_names_every_tensor_once():
    names = model_manifest(FapenexConfig.from_dict(cfg(loop=(0, 2, 3))).model_spec())
    assert names["pos"].shape == (64, 16) and names["loop.step"].shape == (3, 16) and names["embed"].shape == (40, 16)
    assert names["l0.mix.q"].shape == (12, 16) and names["l0.mix.k.conv"].shape == (12, 3) and names["l0.mix.v.conv"].shape == (40, 3)
    assert names["l0.mix.b"].shape == (4, 16) and names["l0.mix.a"].shape == (4, 16) and names["l0.mix.A_log"].shape == (4,)
    assert names["l0.mix.dt_bias"].shape == (4,) and names["l0.mix.norm"].shape == (10,) and names["l0.mix.g"].shape == (40, 16)
    assert names["l0.mix.o"].shape == (16, 40) and names["l0.mlp.shared.sg"].shape == (1, 16) and names["l0.mlp.shared.gate"].shape == (12, 16)
    assert names["l0.mlp.router.b"].shape == (3,) and names["l0.mlp.e2.down"].shape == (16, 8)
    assert names["l1.mix.q"].shape == (24, 16) and names["l1.mix.q.b"].shape == (24,) and names["l1.mix.v.b"].shape == (20,)
    assert names["l1.mix.q.norm"].shape == (6,) and names["l1.mix.k.norm"].shape == (6,) and names["l1.mix.o"].shape == (16, 40)
    assert "l1.mlp.shared.gate" not in names and "l1.mlp.shared.sg" not in names
    assert names["l2.mix.dq"].shape == (12, 16) and names["l2.mix.dq.norm"].shape == (12,) and names["l2.mix.uq"].shape == (8, 12)
    assert names["l2.mix.dkv"].shape == (8, 16) and names["l2.mix.uk"].shape == (8, 8) and names["l2.mix.uv"].shape == (12, 8)
    assert "l2.mix.q" not in names and "l2.mix.g" not in names and "l2.norm2" not in names and "l2.norm1b" in names
    assert "loop.step" not in model_manifest(FapenexConfig.from_dict(cfg()).model_spec())


def test_what_a_window_and_a_chunk_see():
    see = plain.visibility(np.arange(8), plain.sees_window, 3)
    assert see[7].tolist() == [False] * 5 + [True] * 3 and see[1].tolist() == [True, True] + [False] * 6
    see = plain.visibility(np.arange(8), plain.sees_chunk, 3)
    assert see[7].tolist() == [False] * 6 + [True, True] and see[6].tolist() == [False] * 6 + [True, False]
    assert see[5].tolist() == [False] * 3 + [True] * 3 + [False] * 2 and see[0].tolist() == [True] + [False] * 7
    # chunks are counted from position 0 whatever rows are at hand
    assert plain.visibility([4, 5, 6], plain.sees_chunk, 3).tolist() == [[True, False, False], [True, True, False], [False, False, True]]


@pytest.mark.parametrize("size,page,chunked", [(5, 4, False), (16, 16, True), (40, 16, False), (7, 8, True), (33, 16, True)])
def test_the_cache_gives_back_the_pages_that_the_mask_has_passed(size, page, chunked):
    """A request grows token by token in a pool that holds the mask's pages and two more: it never runs out, and every key
    that a row can see still has its page."""
    from infinicore_infer_b200.cache import CacheManager, PagedKV
    live = (size + page - 1) // page + 3
    mgr = CacheManager([PagedKV(1, 8, size, None)], num_pages=live, page_size=page, max_requests=1, max_positions=20 * page, device=None)
    mgr.admit("r")
    rule = plain.sees_chunk if chunked else plain.sees_window
    for n in range(1, 20 * page + 1):
        mgr.reserve("r", n)
        table = mgr.groups[0].row("r")
        for j in range(n):
            if rule(n - 1, j, size):
                assert table[j // page] > 0, f"{n} tokens: the page of position {j} is gone"
        mgr.commit("r", n)
    mgr.release("r")
    mgr.check_invariants()
    assert mgr.groups[0].pool.in_use == 0


@pytest.mark.parametrize("change,what", [
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=8), "rot.dims"),
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "experts"),
    (lambda c: c.update(loop={"start": 2, "stop": 5, "times": 2}), "loop"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "heads"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "heads"),
    (lambda c: c["layers"][1]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][2]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][0]["mlp"]["shared"].pop("limit"), "limit"),
    (lambda c: c.pop("max_positions"), "max_positions"),
])
def test_what_the_configuration_refuses(change, what):
    c = cfg()
    change(c)
    with pytest.raises(ConfigError, match=what):
        FapenexConfig.from_dict(c)


def test_the_delta_rule_by_hand_and_in_portions():
    """One head, one key channel, numbers one can follow: the decay comes first, the write corrects toward the value, the
    read-out sees the row's own write.  And a sequence cut in two with the state handed over equals the whole."""
    q = np.ones((3, 1, 1)); k = np.ones((3, 1, 1)); v = np.array([4.0, 8.0, 2.0]).reshape(3, 1, 1)
    g = np.full((3, 1), 0.5); beta = np.full((3, 1), 0.5)
    o, S = plain.delta_recurrence(q, k, v, g, beta)
    # S1 = 0.5 * 4 = 2;  S2: 1 + 0.5 (8 - 1) = 4.5;  S3: 2.25 + 0.5 (2 - 2.25) = 2.125
    assert o[:, 0, 0].tolist() == [2.0, 4.5, 2.125] and S[0, 0, 0] == 2.125
    r = np.random.default_rng(1)
    q, k, v = r.standard_normal((9, 2, 3)), r.standard_normal((9, 2, 3)), r.standard_normal((9, 2, 4))
    g, beta = r.uniform(0.5, 1.0, (9, 2)), r.uniform(0.0, 1.0, (9, 2))
    whole, S = plain.delta_recurrence(q, k, v, g, beta)
    a, Sa = plain.delta_recurrence(q[:4], k[:4], v[:4], g[:4], beta[:4])
    b, Sb = plain.delta_recurrence(q[4:], k[4:], v[4:], g[4:], beta[4:], state=Sa)
    assert np.allclose(np.concatenate([a, b]), whole) and np.allclose(Sb, S)


def test_a_short_convolution_reads_the_rows_before_a_cut():
    r = np.random.default_rng(2)
    u, taps = r.standard_normal((10, 5)), r.standard_normal((5, 4))
    whole = plain.short_conv(u, taps)
    assert np.allclose(whole[0], u[0] * taps[:, 3]) and np.allclose(whole[1], u[1] * taps[:, 3] + u[0] * taps[:, 2])
    tail = plain.short_conv(u[6:], taps, before=u[3:6])
    assert np.allclose(tail, whole[6:])


def test_weights_of_the_chosen_experts_are_the_softmax_over_the_chosen_logits():
    g = np.random.default_rng(0)
    h, W = g.standard_normal((40, 16)), {"router": g.standard_normal((6, 16)), "router.b": 3.0 * g.standard_normal(6)}
    chosen, weights = plain.route(h, W, "", 3)
    z = h @ W["router"].T + W["router.b"]
    assert np.allclose(weights.sum(-1), 1.0) and np.all(chosen[:, 0] == z.argmax(-1)) and np.all(weights[:, 0] >= weights[:, 1])
    zc = np.take_along_axis(z, chosen, -1)
    assert np.allclose(weights, np.exp(zc) / np.exp(zc).sum(-1, keepdims=True))
    assert (chosen[:, 0] != (h @ W["router"].T).argmax(-1)).any()          # the bias does change choices


def test_the_sink_takes_its_share():
    q = np.zeros((1, 1, 2)); k = np.zeros((1, 1, 2)); v = np.ones((1, 1, 3))
    see = np.ones((1, 1), dtype=bool)
    assert np.allclose(plain.masked_softmax_attention(q, k, v, 1.0, see, sink=True), 0.5)
    assert np.allclose(plain.masked_softmax_attention(q, k, v, 1.0, see, sink=False), 1.0)
