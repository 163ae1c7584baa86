"""The Fapenex configuration: a decoder with learned positions whose config.json lists its layers one by one and may run a
span of them several times.

Keys read: ``vocab``, ``width``, ``max_positions`` (the rows of the position table), ``norm.eps``, ``logit_scale``,
``logit_softcap``, ``loop`` (``start``, ``stop``, ``times``; absent or null: every layer runs once) and ``layers``, a list
whose entries give ``type`` (the mixer), ``mixer`` (its sizes and constants) and ``mlp`` (the feed-forward, or null for
none).  The embedding's output gets a learned vector per position.  Every layer is x += norm1b(mixer(norm1(x)));
x += norm2b(ff(norm2(x))) with RMS norms whose weights are stored around zero (the factor is 1 + w); the model ends with
such a norm, the embedding table as the output matrix, a scale, and c tanh(logits / c).

    latent_attention   attention whose keys and values are maps of one normed latent vector per position and whose queries
                       pass a normed latent of their own; no rotation; a sliding window
                                heads, dim, vdim, kv_rank, q_rank, scale, mask.size
    delta              the gated delta rule behind short convolutions with silu on q, k and v; unit q and k; a decay and a
                       write strength per head; a norm per head and a silu gate      heads, kv_heads, dim, vdim, conv
    attention          grouped heads with biases, an RMS norm per head of q and k ahead of a rotate-half rotation of the
                       leading rot.dims elements with stretched frequencies, keys of the query's own chunk of mask.size
                       positions only, a softmax with one more in its denominator
                                heads, kv_heads, dim, vdim, scale, mask.size, rot.{base, dims, scaling.{factor, original, fast, slow}}
    mlp.kind moe       router.experts clamped gated units of expert.ff (expert.limit), router.top a row by the largest
                       logits (router product plus bias), weighed by the softmax over the chosen logits; shared.{ff, limit}:
                       one more such unit that every row passes, times a sigmoid gate per row

Layers ``loop.start`` .. ``loop.stop`` - 1 run ``loop.times`` times in a row with the same weights, each pass with a cache
and state of its own; before the first layer of every pass x <- x + loop.step[pass].

Tensor names: ``embed``, ``pos``, ``final.norm``, ``loop.step`` and below ``l<i>.``: ``norm1``, ``norm1b``, ``norm2``,
``norm2b``, ``mix.<name>``, ``mlp.router``, ``mlp.router.b``, ``mlp.e<j>.gate / up / down``, ``mlp.shared.gate / up / down /
sg``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .specs import (ConfigError, ConvAttentionSpec, DeltaRuleSpec, FrequencyRampSpec, GLUSpec, LatentAttentionSpec, ModelSpec,
                    PairRotarySpec, RMSNormSpec, RoutedExpertsSpec, RunEntry, SandwichBlockSpec, StepVectorSpec)
from .vunelix import _need, _pos_float, _pos_int

UNIT_EPS = 1e-6             # q and k of the delta rule become x / sqrt(sum(x^2) + UNIT_EPS)
MAGNITUDE_SLOPE = 0.1       # cos and sin of a stretched rotation are multiplied by MAGNITUDE_SLOPE ln(factor) + 1
MIXERS = ("latent_attention", "delta", "attention")


@dataclass(frozen=True)
class FapenexConfig:
    vocab: int
    width: int
    norm_eps: float
    position_rows: int                 # rows of the learned position table
    logit_scale: float
    logit_softcap: float               # 0: none
    layers: Tuple[dict, ...]           # the entries of config.json's ``layers``, checked
    loop: Optional[Tuple[int, int, int]] = None        # (start, stop, times)
    max_positions: int = 0             # the longest sequence the engine plans for: at most position_rows
    model_type: str = "fapenex"

    # ---- reading -------------------------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: dict, max_tokens: Optional[int] = None) -> "FapenexConfig":
        layers = _need(cfg, "layers", "the configuration")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one entry")
        checked = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            m = dict(_need(layer, "mixer", where))
            mw = where + ".mixer"
            if kind == "latent_attention":
                for key in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
                    _pos_int(m, key, mw)
                _pos_float(m, "scale", mw)
                if m.get("mask") is not None:
                    _pos_int(m["mask"], "size", mw + ".mask")
            elif kind == "delta":
                for key in ("heads", "kv_heads", "dim", "vdim", "conv"):
                    _pos_int(m, key, mw)
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: {mw}: {m['heads']} heads are no multiple of {m['kv_heads']} key heads")
            elif kind == "attention":
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _pos_int(m, key, mw)
                if m["heads"] % m["kv_heads"]:
                    raise ConfigError(f"config.json: {mw}: {m['heads']} heads are no multiple of {m['kv_heads']} key/value heads")
                _pos_float(m, "scale", mw)
                if m.get("mask") is not None:
                    _pos_int(m["mask"], "size", mw + ".mask")
                rot = m.get("rot")
                if rot is not None and int(rot.get("dims") or 0):
                    dims = _pos_int(rot, "dims", mw + ".rot")
                    if dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"config.json: {mw}.rot.dims {dims} must be even and at most dim {m['dim']}")
                    _pos_float(rot, "base", mw + ".rot")
                    if rot.get("scaling") is not None:
                        for key in ("factor", "original", "fast", "slow"):
                            _pos_float(rot["scaling"], key, mw + ".rot.scaling")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is none of {', '.join(MIXERS)}")
            mlp = layer.get("mlp")
            if mlp is not None:
                mlp = dict(mlp)
                form = _need(mlp, "kind", where + ".mlp")
                if form != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind {form!r} is not moe")
                router = _need(mlp, "router", where + ".mlp")
                n, top = _pos_int(router, "experts", where + ".mlp.router"), _pos_int(router, "top", where + ".mlp.router")
                if top > n:
                    raise ConfigError(f"config.json: {where}.mlp.router takes {top} of {n} experts")
                expert = _need(mlp, "expert", where + ".mlp")
                _pos_int(expert, "ff", where + ".mlp.expert")
                _pos_float(expert, "limit", where + ".mlp.expert")
                if mlp.get("shared") is not None:
                    _pos_int(mlp["shared"], "ff", where + ".mlp.shared")
                    _pos_float(mlp["shared"], "limit", where + ".mlp.shared")
            checked.append({"type": kind, "mixer": m, "mlp": mlp})
        loop = cfg.get("loop")
        if loop is not None:
            start, stop = int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop"))
            times = _pos_int(loop, "times", "loop")
            if not 0 <= start < stop <= len(checked):
                raise ConfigError(f"config.json: loop {start} .. {stop} does not lie within the {len(checked)} layers")
            loop = (start, stop, times)
        rows = _pos_int(cfg, "max_positions", "the configuration")
        cap, scale = cfg.get("logit_softcap"), cfg.get("logit_scale")
        return cls(vocab=_pos_int(cfg, "vocab", "the configuration"), width=_pos_int(cfg, "width", "the configuration"),
                   norm_eps=float(_need(_need(cfg, "norm", "the configuration"), "eps", "norm")), position_rows=rows,
                   logit_scale=float(scale) if scale else 1.0, logit_softcap=float(cap) if cap else 0.0, layers=tuple(checked),
                   loop=loop, max_positions=min(int(max_tokens), rows) if max_tokens else rows)

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
        out = {"architecture": "Fapenex", "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width,
               "max_positions": self.position_rows, "logit_scale": self.logit_scale, "logit_softcap": self.logit_softcap or None,
               "layers": [{"type": l["type"], "mixer": dict(l["mixer"]), "mlp": None if l["mlp"] is None else dict(l["mlp"])}
                          for l in self.layers]}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    # ---- the model as parts ------------------------------------------------------------------------------------------
    def _mixer_spec(self, kind: str, m: dict):
        mask = m.get("mask") or {}
        size = int(mask["size"]) if mask.get("size") is not None else None
        if kind == "latent_attention":
            return LatentAttentionSpec(hidden_size=self.width, num_heads=int(m["heads"]), head_dim=int(m["dim"]), rot_dim=0,
                                       v_head_dim=int(m["vdim"]), latent_size=int(m["kv_rank"]), softmax_scale=float(m["scale"]),
                                       norm_eps=self.norm_eps, position=None, output_gate=False, window=size, q_rank=int(m["q_rank"]))
        if kind == "delta":
            return DeltaRuleSpec(hidden_size=self.width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), head_dim=int(m["dim"]),
                                 v_head_dim=int(m["vdim"]), conv_taps=int(m["conv"]), norm_eps=self.norm_eps, unit_eps=UNIT_EPS)
        rot, position = m.get("rot"), None
        if rot is not None and int(rot.get("dims") or 0):
            scaling = None
            if rot.get("scaling") is not None:
                s = rot["scaling"]
                scaling = FrequencyRampSpec(factor=float(s["factor"]), original=float(s["original"]), fast=float(s["fast"]),
                                            slow=float(s["slow"]), magnitude_slope=MAGNITUDE_SLOPE)
            position = PairRotarySpec(dims=int(rot["dims"]), base=float(rot["base"]), scaling=scaling, layout="halves")
        return ConvAttentionSpec(hidden_size=self.width, num_heads=int(m["heads"]), num_kv_heads=int(m["kv_heads"]), head_dim=int(m["dim"]),
                                 v_head_dim=int(m["vdim"]), softmax_scale=float(m["scale"]), window=None, conv_taps=0, qk_norm=False,
                                 qk_norm_eps=self.norm_eps, position=position, sink=True, head_norm="before_rotation", bias=True,
                                 chunk=size)

    def _ffn_spec(self, mlp: Optional[dict]):
        if mlp is None:
            return None
        shared = mlp.get("shared")
        return RoutedExpertsSpec(hidden_size=self.width, num_experts=int(mlp["router"]["experts"]), top=int(mlp["router"]["top"]),
                                 expert_size=int(mlp["expert"]["ff"]), act="swish_clamp", scale_input=False, score_form="softmax_renorm",
                                 limit=float(mlp["expert"]["limit"]), router_bias=True,
                                 shared=None if shared is None else GLUSpec(hidden_size=self.width, intermediate_size=int(shared["ff"]),
                                                                            act="swish_clamp", limit=float(shared["limit"])),
                                 shared_gate_name=None if shared is None else "sg")

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
        norm = RMSNormSpec(size=self.width, eps=self.norm_eps, weight_name="", one_plus=True)
        blocks = []
        for layer in self.layers:
            ffn = self._ffn_spec(layer["mlp"])
            blocks.append(SandwichBlockSpec(mixer=self._mixer_spec(layer["type"], layer["mixer"]), feed_forward=ffn,
                                            mixer_norm=norm, mixer_post_norm=norm, ffn_norm=None if ffn is None else norm,
                                            ffn_post_norm=None if ffn is None else norm))
        order = []
        for run, (i, t, opens) in enumerate(self.run_order()):       # every run of a layer has a cache and state of its own
            before = StepVectorSpec(hidden_size=self.width, steps=self.loop[2], index=t) if opens else None
            order.append(RunEntry(layer=i, cache=run, writes_cache=True, before=before))
        return ModelSpec(architecture="fapenex", hidden_size=self.width, vocab_size=self.vocab, max_positions=self.max_positions,
                         layers=tuple(blocks), order=tuple(order), final_norm=norm, embed_scale=1.0, logit_scale=self.logit_scale,
                         logit_softcap=self.logit_softcap, position_table_name="pos", position_rows=self.position_rows,
                         tie_embeddings=True, embed_name="embed", lm_head_name="head", final_norm_prefix="final.norm",
                         layer_prefix="l{}.", eos_token_ids=())
