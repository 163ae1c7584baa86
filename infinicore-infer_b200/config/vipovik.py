"""The Vipovik configuration: a decoder whose layers each run two mixers side by side, and may run a span of layers several
times.

Keys read: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``loop`` (``start``, ``stop``, ``times``; absent or null:
every layer runs once) and ``layers``, a list whose entries give ``type`` ("parallel"), ``mixer`` and ``mlp`` (or null).
Every layer is x += mixer(norm1(x)); x += ff(norm2(x)) with RMS norms; the model ends with an RMS norm and the embedding
table as the output matrix.

    mixer.left         softmax attention with grouped heads: rotation of a head's leading ``rot.dims`` elements in halves
                       (element i with i + dims / 2) with stretched frequencies, then every head of q and k divided by its
                       root mean square; scores capped by c tanh(s / c); a sliding window that keeps the first tokens
                            heads, kv_heads, dim, vdim, scale, softcap, mask.{size, keep_first},
                            rot.{base, dims, scaling.{factor, original, fast, slow}}
    mixer.right        a recurrence per head with a decay per key channel, exp(-exp(.)), behind a token shift with one mixing
                       vector per projection, a bonus for the current token, a norm per head and a silu gate      heads, dim
                       (the width of the decay's projection is the shape of ``w1``)
    mixer.left_scale, mixer.right_scale    the factors of the two in their sum
    mlp.kind dense     down(gelu(up h)), the exact gelu                                                            ff
    mlp.kind moe       router.experts clamped gated units of expert.ff (expert.limit), router.top a row by softmax scores,
                       renormalised over the chosen ones, which multiply the units' outputs

Layers ``loop.start`` .. ``loop.stop`` - 1 run ``loop.times`` times in a row with the same weights, each pass with a cache
and state of its own; before the first layer of every pass x <- loop.in [x | embedding output] + loop.step[pass].

Tensor names: ``embed``, ``final.norm``, ``loop.in``, ``loop.step`` and below ``l<i>.``: ``norm1``, ``norm2``,
``mix.left.q / k / v / o``, ``mix.right.r / k / v / g / o / w1 / w2 / w0 / u / norm / mu.r / mu.k / mu.v / mu.g / mu.w``,
``mlp.up / down``, ``mlp.router``, ``mlp.e<j>.gate / up / down``.  The configuration names no longest sequence: the
engine's is given when the configuration is read.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .specs import (BlockSpec, ConfigError, ConvAttentionSpec, FrequencyRampSpec, LinearAttentionSpec, MLPSpec, ModelSpec,
                    PairRotarySpec, ParallelMixerSpec, ReinjectSpec, RMSNormSpec, RoutedExpertsSpec, RunEntry)
from .vunelix import DEFAULT_MAX_POSITIONS, _need, _pos_float, _pos_int

DECAY_RANK_OF = "right.w1"       # the tensor (below a layer's ``mix.``) whose rows are the decay projection's width


def _count(d, key: str, where: str) -> int:
    v = d.get(key, 0) if isinstance(d, dict) else 0
    if v is None:
        return 0
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or v < 0:
        raise ConfigError(f"config.json: {where}.{key} must be a count, found {v!r}")
    return int(v)


@dataclass(frozen=True)
class VipovikConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[dict, ...]           # the entries of config.json's ``layers``, checked
    loop: Optional[Tuple[int, int, int]] = None        # (start, stop, times)
    max_positions: int = DEFAULT_MAX_POSITIONS
    model_type: str = "vipovik"

    reads_shapes = True

    # ---- reading -------------------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: dict, max_tokens: Optional[int] = None, shapes: Optional[dict] = None) -> "VipovikConfig":
        layers = _need(cfg, "layers", "the configuration")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one entry")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind != "parallel":
                raise ConfigError(f"config.json: {where}.type {kind!r} is not parallel")
            m = dict(_need(layer, "mixer", where))
            left = dict(_need(m, "left", where + ".mixer"))
            right = dict(_need(m, "right", where + ".mixer"))
            lw = where + ".mixer.left"
            heads, kv = _pos_int(left, "heads", lw), _pos_int(left, "kv_heads", lw)
            if heads % kv:
                raise ConfigError(f"config.json: {lw}: {heads} heads are no multiple of {kv} key/value heads")
            dim = _pos_int(left, "dim", lw)
            _pos_int(left, "vdim", lw)
            _pos_float(left, "scale", lw)
            if left.get("softcap") is not None and not float(left["softcap"]) >= 0:
                raise ConfigError(f"config.json: {lw}.softcap must not be negative")
            mask = left.get("mask")
            if mask is not None:
                if mask.get("size") is not None:
                    _pos_int(mask, "size", lw + ".mask")
                _count(mask, "keep_first", lw + ".mask")
            rot = left.get("rot")
            if rot is not None:
                dims = _count(rot, "dims", lw + ".rot")
                if dims % 2 or dims > dim:
                    raise ConfigError(f"config.json: {lw}.rot.dims {dims} must be even and at most dim {dim}")
                if dims:
                    _pos_float(rot, "base", lw + ".rot")
                if rot.get("scaling") is not None:
                    for key in ("factor", "original", "fast", "slow"):
                        _pos_float(rot["scaling"], key, lw + ".rot.scaling")
            _pos_int(right, "heads", where + ".mixer.right")
            _pos_int(right, "dim", where + ".mixer.right")
            if "rank" not in right and shapes is not None and f"l{i}.mix.{DECAY_RANK_OF}" in shapes:
                right["rank"] = int(shapes[f"l{i}.mix.{DECAY_RANK_OF}"][0])
            m["left"], m["right"] = left, right
            m["left_scale"], m["right_scale"] = float(_need(m, "left_scale", where + ".mixer")), float(_need(m, "right_scale", where + ".mixer"))
            mlp = layer.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                form = _need(mlp, "kind", where + ".mlp")
                if form == "dense":
                    _pos_int(mlp, "ff", where + ".mlp")
                elif form == "moe":
                    router = _need(mlp, "router", where + ".mlp")
                    n, top = _pos_int(router, "experts", where + ".mlp.router"), _pos_int(router, "top", where + ".mlp.router")
                    if top > n:
                        raise ConfigError(f"config.json: {where}.mlp.router takes {top} of {n} experts")
                    expert = _need(mlp, "expert", where + ".mlp")
                    _pos_int(expert, "ff", where + ".mlp.expert")
                    _pos_float(expert, "limit", where + ".mlp.expert")
                else:
                    raise ConfigError(f"config.json: {where}.mlp.kind {form!r} is none of dense, moe")
            checked.append({"type": kind, "mixer": m, "mlp": mlp})
        loop = cfg.get("loop")
        if loop is not None:
            start, stop = int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop"))
            times = _pos_int(loop, "times", "loop")
            if not 0 <= start < stop <= len(checked):
                raise ConfigError(f"config.json: loop {start} .. {stop} does not lie within the {len(checked)} layers")
            loop = (start, stop, times)
        return cls(vocab=_pos_int(cfg, "vocab", "the configuration"), width=_pos_int(cfg, "width", "the configuration"),
                   norm_eps=float(_need(_need(cfg, "norm", "the configuration"), "eps", "norm")),
                   embedding_scale=float(_need(_need(cfg, "embedding", "the configuration"), "scale", "embedding")),
                   layers=tuple(checked), loop=loop,
                   max_positions=int(max_tokens) if max_tokens else int(cfg.get("max_positions", DEFAULT_MAX_POSITIONS)))

    # what the entry points ask of any configuration
    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions

    @property
    def tie_word_embeddings(self) -> bool:
        return True

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def to_dict(self) -> dict:
        """config.json contents that read back to this configuration."""
        def mixer(m):
            out = dict(m)
            out["left"], out["right"] = dict(m["left"]), dict(m["right"])
            return out
        out = {"architecture": "Vipovik", "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "vocab": self.vocab, "width": self.width,
               "layers": [{"type": l["type"], "mixer": mixer(l["mixer"]), "mlp": None if l["mlp"] is None else dict(l["mlp"])}
                          for l in self.layers]}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    # ---- the model as parts ------------------------------------------------------------------------------------------
    def _left_spec(self, m: dict) -> ConvAttentionSpec:
        rot, position = m.get("rot"), None
        if rot is not None and int(rot.get("dims") or 0):
            scaling = None
            if rot.get("scaling") is not None:
                s = rot["scaling"]
                scaling = FrequencyRampSpec(factor=float(s["factor"]), original=float(s["original"]), fast=float(s["fast"]),
                                            slow=float(s["slow"]), magnitude_slope=0.1)
            position = PairRotarySpec(dims=int(rot["dims"]), base=float(rot["base"]), scaling=scaling, layout="halves")
        mask = m.get("mask") or {}
        window = int(mask["size"]) if mask.get("size") is not None else None
        return ConvAttentionSpec(hidden_size=self.width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), head_dim=int(m["dim"]),
                                 v_head_dim=int(m["vdim"]), softmax_scale=float(m["scale"]), window=window, conv_taps=0, qk_norm=False,
                                 qk_norm_eps=self.norm_eps, position=position, head_norm=True, score_cap=float(m.get("softcap") or 0.0),
                                 keep_first=int(mask.get("keep_first") or 0) if window else 0)

    def _right_spec(self, m: dict) -> LinearAttentionSpec:
        if "rank" not in m:
            raise ConfigError("the decay projection of a layer's recurrence has no width: config.json gives no mixer.right.rank and "
                              f"no checkpoint was at hand to read the shape of mix.{DECAY_RANK_OF} from")
        return LinearAttentionSpec(hidden_size=self.width, num_heads=int(m["heads"]), head_dim=int(m["dim"]), v_head_dim=int(m["dim"]),
                                   norm_eps=self.norm_eps, qkv_act="none", q_scale=1.0, decay=None, decay_rank=int(m["rank"]),
                                   norm_per_head="unit", gate_act="silu", q_name="r", decay_down_name="w1", decay_up_name="w2",
                                   decay_bias_name="w0", token_shift=True, bonus_name="u", decay_form="exp_neg_exp", decay_act="tanh")

    def _ffn_spec(self, mlp: Optional[dict]):
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return MLPSpec(hidden_size=self.width, intermediate_size=int(mlp["ff"]), act="gelu_erf")
        return RoutedExpertsSpec(hidden_size=self.width, num_experts=int(mlp["router"]["experts"]), top=int(mlp["router"]["top"]),
                                 expert_size=int(mlp["expert"]["ff"]), act="swish_clamp", scale_input=False, score_form="softmax_renorm",
                                 limit=float(mlp["expert"]["limit"]))

    def run_order(self):
        """(layer, pass number or None, whether the pass starts here) for every layer run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None, False) for i in range(n)]
        start, stop, times = self.loop
        runs = [(i, None, False) for i in range(start)]
        for t in range(times):
            runs += [(i, t, i == start) for i in range(start, stop)]
        return runs + [(i, None, False) for i in range(stop, n)]

    def model_spec(self) -> ModelSpec:
        norm = RMSNormSpec(size=self.width, eps=self.norm_eps, weight_name="")
        blocks = []
        for layer in self.layers:
            m = layer["mixer"]
            ffn = self._ffn_spec(layer["mlp"])
            mixer = ParallelMixerSpec(left=self._left_spec(m["left"]), right=self._right_spec(m["right"]),
                                      left_scale=float(m["left_scale"]), right_scale=float(m["right_scale"]))
            blocks.append(BlockSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm, ffn_norm=None if ffn is None else norm,
                                    residual_scale=1.0, mixer_prefix="mix.", ffn_prefix="mlp.", mixer_norm_prefix="norm1",
                                    ffn_norm_prefix="norm2"))
        order = []
        for run, (i, t, opens) in enumerate(self.run_order()):       # every run of a layer has a cache and state of its own
            before = ReinjectSpec(hidden_size=self.width, steps=self.loop[2], step_index=t) if opens else None
            order.append(RunEntry(layer=i, cache=run, writes_cache=True, before=before))
        return ModelSpec(architecture="vipovik", hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
                         layers=tuple(blocks), order=tuple(order), final_norm=norm, embed_scale=self.embedding_scale, logit_scale=1.0,
                         tie_embeddings=True, embed_name="embed", lm_head_name="head", final_norm_prefix="final.norm",
                         layer_prefix="l{}.", eos_token_ids=())
