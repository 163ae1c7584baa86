"""Vipovik without a GPU: the configuration, the run order of a looped span, the manifest, the rotation's frequencies, what
the cache keeps for a window with kept first keys, and the plain implementation's own small cases."""
import math

import numpy as np
import pytest

import plain_vipovik as plain
from infinicore_infer_b200.config import ConfigError, FrequencyRampSpec, PairRotarySpec, VipovikConfig, config_class_for
from infinicore_infer_b200.parts import cache_needs, model_manifest, state_needs


def cfg(loop=None, rank=True):
    def right(heads, dim, r):
        return {"heads": heads, "dim": dim, **({"rank": r} if rank else {})}
    layers = [
        {"type": "parallel", "mlp": {"kind": "dense", "ff": 20},
         "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.3, "softcap": 9.0, "mask": {"size": 5, "keep_first": 2},
                            "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}}},
                   "right": right(3, 4, 2), "left_scale": 0.7, "right_scale": 0.4}},
        {"type": "parallel", "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 8, "limit": 1.5}},
         "mixer": {"left": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.5, "softcap": 4.0, "rot": {"base": 50.0, "dims": 8}},
                   "right": right(1, 12, 5), "left_scale": 1.0, "right_scale": 1.0}},
        {"type": "parallel", "mlp": None,
         "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 6, "scale": 0.4, "softcap": 0.0, "mask": {"size": 3, "keep_first": 0}},
                   "right": right(2, 6, 3), "left_scale": 0.5, "right_scale": 2.0}},
    ]
    out = {"architecture": "Vipovik", "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5}, "vocab": 40, "width": 16, "layers": layers}
    if loop:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


def test_the_registry_finds_the_configuration_and_it_reads_back():
    c = config_class_for(cfg())
    assert c is VipovikConfig
    typed = c.from_dict(cfg(loop=(1, 3, 2)), max_tokens=99)
    assert typed.max_positions == 99 and typed.loop == (1, 3, 2) and typed.embedding_scale == 2.5 and typed.tie_word_embeddings
    assert VipovikConfig.from_dict(typed.to_dict(), max_tokens=99) == typed


def test_the_decay_projections_width_comes_from_the_checkpoints_shapes():
    shapes = {f"l{i}.mix.right.w1": (r, 16) for i, r in enumerate((2, 5, 3))}
    spec = VipovikConfig.from_dict(cfg(rank=False), shapes=shapes).model_spec()
    assert [l.mixer.right.decay_rank for l in spec.layers] == [2, 5, 3]
    with pytest.raises(ConfigError, match="rank"):
        VipovikConfig.from_dict(cfg(rank=False)).model_spec()


def test_run_order_of_a_span_that_runs_several_times():
    spec = VipovikConfig.from_dict(cfg(loop=(0, 2, 3))).model_spec()
    assert [e.layer for e in spec.order] == [0, 1, 0, 1, 0, 1, 2]
    assert [e.cache for e in spec.order] == list(range(7))
    assert [(e.before.step_index, e.before.steps) if e.before else None for e in spec.order] == [(0, 3), None, (1, 3), None, (2, 3), None, None]
    assert plain.run_order(cfg(loop=(0, 2, 3))) == VipovikConfig.from_dict(cfg(loop=(0, 2, 3))).run_order()
    assert plain.run_order(cfg(loop=(1, 2, 1))) == VipovikConfig.from_dict(cfg(loop=(1, 2, 1))).run_order() == [(0, None, False), (1, 0, True), (2, None, False)]
    once = VipovikConfig.from_dict(cfg()).model_spec().order
    assert [e.layer for e in once] == [0, 1, 2] and all(e.before is None for e in once)
    needs, states = cache_needs(spec), state_needs(spec)
    assert (needs[0].num_kv_heads, needs[0].head_dim, needs[0].v_head_dim, needs[0].window, needs[0].keep_first) == (2, 6, 10, 5, 2)
    assert needs[0] == needs[2] and needs[1].window is None and needs[1].keep_first == 0 and needs[6].keep_first == 0
    assert [s.shape for s in states[0].slots] == [(3, 4, 4), (16,)] and [s.shape for s in states[1].slots] == [(1, 12, 12), (16,)]


def test_manifest_names_every_tensor_once():
    names = model_manifest(VipovikConfig.from_dict(cfg(loop=(0, 2, 3))).model_spec())
    assert names["loop.in"].shape == (16, 32) and names["loop.step"].shape == (3, 16) and names["embed"].shape == (40, 16)
    assert names["l0.mix.left.q"].shape == (24, 16) and names["l0.mix.left.k"].shape == (12, 16) and names["l0.mix.left.v"].shape == (20, 16)
    assert names["l0.mix.left.o"].shape == (16, 40) and names["l0.mix.right.w1"].shape == (2, 16) and names["l0.mix.right.w2"].shape == (12, 2)
    assert names["l0.mix.right.u"].shape == (3, 4) and names["l0.mix.right.norm"].shape == (12,) and names["l0.mix.right.mu.w"].shape == (16,)
    assert names["l0.mix.right.r"].shape == (12, 16) and names["l0.mix.right.o"].shape == (16, 12) and names["l0.mix.right.w0"].shape == (12,)
    assert names["l0.mlp.up"].shape == (20, 16) and "l0.mlp.gate" not in names
    assert names["l1.mlp.e2.down"].shape == (16, 8) and names["l1.mlp.router"].shape == (3, 16) and names["final.norm"].shape == (16,)
    assert "l2.norm2" not in names and "l2.norm1" in names
    assert "loop.in" not in model_manifest(VipovikConfig.from_dict(cfg()).model_spec())


@pytest.mark.parametrize("dims,base,scaling", [(8, 1e4, None), (32, 5e5, (4.0, 256, 16.0, 2.0)), (6, 300.0, (16.0, 8, 2.0, 0.25))])
def test_stretched_frequencies(dims, base, scaling):
    spec = PairRotarySpec(dims=dims, base=base, scaling=None if scaling is None else FrequencyRampSpec(*scaling), layout="halves")
    f, m = spec.frequencies()
    rot = {"dims": dims, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    pf, pm = plain.rotary_frequencies(rot)
    assert all(abs(a - b) <= 1e-12 * b for a, b in zip(f, pf.tolist())) and abs(m - pm) < 1e-12
    if scaling:
        assert abs(m - (0.1 * math.log(scaling[0]) + 1.0)) < 1e-12


def test_rotation_pairs_the_halves_of_the_leading_elements():
    x = np.arange(1.0, 7.0).reshape(1, 1, 6)
    out = plain.rotate_half(x, [1], {"dims": 4, "base": 1.0})      # every pair turns by one radian
    c, s = math.cos(1.0), math.sin(1.0)
    assert np.allclose(out[0, 0], [1 * c - 3 * s, 2 * c - 4 * s, 3 * c + 1 * s, 4 * c + 2 * s, 5.0, 6.0])


def test_what_a_window_with_kept_first_keys_sees():
    mask = {"size": 3, "keep_first": 2}
    see = plain.visibility(np.arange(8), mask)
    assert see[7].tolist() == [True, True, False, False, False, True, True, True]
    assert see[3].tolist() == [True, True, True, True, False, False, False, False] and see[0].tolist() == [True] + [False] * 7
    assert all(plain.visible(i, j, mask) == see[i, j] for i in range(8) for j in range(8))
    assert plain.visibility(np.arange(4), None).tolist() == np.tril(np.ones((4, 4), dtype=bool)).tolist()


@pytest.mark.parametrize("window,keep,page", [(5, 2, 4), (16, 17, 16), (40, 1, 16), (7, 0, 8)])
def test_the_cache_gives_back_the_pages_that_the_window_has_passed_but_never_the_kept_ones(window, keep, page):
    """A request grows token by token in a pool that holds the kept pages, the window's and one more: it never runs out."""
    from infinicore_infer_b200.cache import CacheManager, PagedKV
    kept_pages = (keep + page - 1) // page
    live = kept_pages + (window + page - 1) // page + 2
    mgr = CacheManager([PagedKV(1, 8, window, None, keep_first=keep)], num_pages=live, page_size=page, max_requests=1,
                       max_positions=20 * page, device=None)
    mgr.admit("r")
    most = 0
    for n in range(1, 20 * page + 1):
        mgr.reserve("r", n)
        table = mgr.groups[0].row("r")
        for j in range(n):
            if plain.visible(n - 1, j, {"size": window, "keep_first": keep}):
                assert table[j // page] > 0, f"{n} tokens: the page of position {j} is gone"
        mgr.commit("r", n)
        most = max(most, mgr.groups[0].pool.in_use)
    assert most <= live - 1
    mgr.release("r")
    mgr.check_invariants()
    assert mgr.groups[0].pool.in_use == 0


@pytest.mark.parametrize("change,what", [
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=8), "rot.dims"),
    (lambda c: c["layers"][0].update(type="serial"), "type"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=4), "experts"),
    (lambda c: c.update(loop={"start": 2, "stop": 5, "times": 2}), "loop"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "heads"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "kind"),
    (lambda c: c["layers"][2]["mixer"].pop("right_scale"), "right_scale"),
])
def test_what_the_configuration_refuses(change, what):
    c = cfg()
    change(c)
    with pytest.raises(ConfigError, match=what):
        VipovikConfig.from_dict(c)


def test_the_bonus_and_the_order_of_decay_and_read_show():
    """The plain recurrence itself: with one head, one key channel and numbers one can follow by hand."""
    r = np.ones((3, 1, 1)); k = np.array([1.0, 2.0, 3.0]).reshape(3, 1, 1); v = np.array([1.0, 10.0, 100.0]).reshape(3, 1, 1)
    decay = np.full((3, 1, 1), 0.5); u = np.array([[2.0]])
    o, S = plain.bonus_recurrence(r, k, v, decay, u)
    assert o[:, 0, 0].tolist() == [2.0, 1.0 + 40.0, 0.5 + 20.0 + 600.0] and S[0, 0, 0] == 0.25 + 10.0 + 300.0


def test_weights_of_the_chosen_experts_add_up_to_one():
    g = np.random.default_rng(0)
    h, W = g.standard_normal((40, 16)), {"router": g.standard_normal((6, 16))}
    chosen, weights = plain.route(h, W, "", 3)
    z = h @ W["router"].T
    assert np.allclose(weights.sum(-1), 1.0) and np.all(chosen[:, 0] == z.argmax(-1)) and np.all(weights[:, 0] >= weights[:, 1])
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    assert np.allclose(weights[:, 1] / weights[:, 0], np.take_along_axis(s, chosen, -1)[:, 1] / np.take_along_axis(s, chosen, -1)[:, 0])


