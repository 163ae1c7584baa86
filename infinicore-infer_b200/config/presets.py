"""Named configurations for the random-weights mode: config.json contents as data, not sizes in code.

``tiny-A`` and ``tiny-B`` are two small configurations of the architecture that differ in every size and option
(multi-head against grouped heads 3:1, tied against untied embeddings, every scale, eps and theta); ``1b``, ``2b``
and ``8b`` have the layer sizes of MiniCPM-1B, MiniCPM-2B and an FM9G/MiniCPM4-8B-class model.  Each entry gives
the keys of a config.json of this architecture (the ones ``MiniCPMConfig.from_dict`` reads) and the spread of its
random weights: matrices N(0, std), norm weights 1 + N(0, norm_std).  The reference has no random mode.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict


@dataclass(frozen=True)
class Preset:
    config: dict
    std: float
    norm_std: float
    page_size: int          # the cache page this configuration is meant to run with


PRESETS: Dict[str, Preset] = {
    "tiny-A": Preset(dict(model_type="minicpm", num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                          num_key_value_heads=4, intermediate_size=160, vocab_size=256, max_position_embeddings=64,
                          rms_norm_eps=1e-5, rope_theta=1e4, scale_emb=12, scale_depth=1.4, dim_model_base=16,
                          tie_word_embeddings=True, eos_token_id=2), 0.02, 0.01, 16),
    "tiny-B": Preset(dict(model_type="fm9g", num_hidden_layers=3, hidden_size=96, num_attention_heads=3,
                          num_key_value_heads=1, intermediate_size=224, vocab_size=384, max_position_embeddings=96,
                          rms_norm_eps=1e-6, rope_theta=1e6, scale_emb=2.5, scale_depth=1.0, dim_model_base=48,
                          tie_word_embeddings=False, eos_token_id=2), 0.03, 0.02, 8),
    "1b": Preset(dict(model_type="minicpm", num_hidden_layers=52, hidden_size=1536, num_attention_heads=24,
                      num_key_value_heads=8, intermediate_size=3840, vocab_size=73440, max_position_embeddings=4096,
                      rms_norm_eps=1e-5, rope_theta=10000.0, scale_emb=12, scale_depth=1.4, dim_model_base=256,
                      tie_word_embeddings=True, eos_token_id=2), 0.02, 0.01, 16),
    "2b": Preset(dict(model_type="minicpm", num_hidden_layers=40, hidden_size=2304, num_attention_heads=36,
                      num_key_value_heads=36, intermediate_size=5760, vocab_size=122753, max_position_embeddings=4096,
                      rms_norm_eps=1e-5, rope_theta=10000.0, scale_emb=12, scale_depth=1.4, dim_model_base=256,
                      tie_word_embeddings=True, eos_token_id=2), 0.02, 0.01, 16),
    "8b": Preset(dict(model_type="fm9g", num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                      num_key_value_heads=2, intermediate_size=16384, vocab_size=73448, max_position_embeddings=4096,
                      rms_norm_eps=1e-5, rope_theta=10000.0, scale_emb=12, scale_depth=1.4, dim_model_base=256,
                      tie_word_embeddings=False, eos_token_id=2), 0.02, 0.01, 16),
    # a small Sitelorn: every kind of layer, a layer that borrows its keys, one without feed-forward
    "sitelorn-tiny": Preset(dict(
        architecture="Sitelorn", vocab=320, width=96, embedding={"scale": 4.0}, norm={"eps": 1e-5}, layers=[
            {"type": "lightning", "mixer": {"heads": 3, "dim": 16, "vdim": 32, "decay": [0.7, 0.97, 0.999]}, "mlp": {"kind": "dense", "ff": 160}},
            {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 24, "conv": 3, "rot": {"dims": 12, "base": 1e5},
                                            "scale": 0.2, "mask": {"size": 48}}, "mlp": {"kind": "dense", "ff": 160}},
            {"type": "gla", "mixer": {"heads": 2, "dim": 24, "vdim": 48, "tau": 8.0, "rank": 8}, "mlp": None},
            {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 24, "conv": 3, "rot": {"dims": 12, "base": 1e5},
                                            "scale": 0.2, "mask": {"size": 24}, "kv_from": 1}, "mlp": {"kind": "dense", "ff": 160}},
        ]), 0.1, 0.05, 16),
    # a small Vunelix: a span of two layers that runs twice, latent attention, a selective scan, dense and routed feed-forwards
    "vunelix-tiny": Preset(dict(
        architecture="Vunelix", vocab=320, width=96, norm={"eps": 1e-5}, logit_softcap=25.0, loop={"start": 1, "stop": 3, "times": 2}, layers=[
            {"type": "latent_attention", "mixer": {"heads": 4, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 48, "scale": 0.2,
                                                   "rot": {"base": 1e4, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}}},
             "mlp": {"kind": "dense", "ff": 160}},
            {"type": "mamba1", "mixer": {"inner": 128, "state": 12, "dt_rank": 6, "conv": 4},
             "mlp": {"kind": "moe", "router": {"experts": 6, "top": 2}, "expert": {"ff": 48}, "shared": {"ff": 64}}},
            {"type": "latent_attention", "mixer": {"heads": 2, "dim": 24, "rot_dim": 16, "vdim": 16, "kv_rank": 32, "scale": 0.15,
                                                   "rot": {"base": 5e4, "dims": 12}}, "mlp": None},
            {"type": "mamba1", "mixer": {"inner": 64, "state": 20, "dt_rank": 4, "conv": 3},
             "mlp": {"kind": "moe", "router": {"experts": 4, "top": 1}, "expert": {"ff": 80}}},
        ]), 0.1, 0.05, 16),
    # a small Vipovik: a span of two layers that runs twice, attention beside a recurrence in every layer, a dense and a
    # routed feed-forward and a layer without one, a window with kept first tokens, partial rotation with and without stretching
    "vipovik-tiny": Preset(dict(
        architecture="Vipovik", vocab=320, width=96, embedding={"scale": 3.0}, norm={"eps": 1e-5}, loop={"start": 1, "stop": 3, "times": 2}, layers=[
            {"type": "parallel", "mixer": {
                "left": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 16, "scale": 0.3, "softcap": 15.0, "mask": {"size": 40, "keep_first": 3},
                         "rot": {"base": 1e4, "dims": 16, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}}},
                "right": {"heads": 3, "dim": 16, "rank": 8}, "left_scale": 0.7, "right_scale": 0.4},
             "mlp": {"kind": "dense", "ff": 160}},
            {"type": "parallel", "mixer": {
                "left": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.25, "softcap": 30.0, "mask": {"size": 24, "keep_first": 1},
                         "rot": {"base": 5e4, "dims": 32}},
                "right": {"heads": 2, "dim": 24, "rank": 4}, "left_scale": 0.5, "right_scale": 0.6},
             "mlp": {"kind": "moe", "router": {"experts": 6, "top": 2}, "expert": {"ff": 48, "limit": 1.5}}},
            {"type": "parallel", "mixer": {
                "left": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 24, "scale": 0.35, "softcap": 10.0, "mask": {"size": 17, "keep_first": 5},
                         "rot": {"base": 1e4, "dims": 8}},
                "right": {"heads": 4, "dim": 8, "rank": 6}, "left_scale": 1.0, "right_scale": 1.0},
             "mlp": None},
        ]), 0.1, 0.05, 16),
    # a small Fapenex: learned positions, a span of two layers that runs twice, one layer of each mixer (a delta rule, chunked
    # attention with partial stretched rotation, windowed latent attention), routed experts with and without the shared unit
    "fapenex-tiny": Preset(dict(
        architecture="Fapenex", vocab=320, width=96, max_positions=256, norm={"eps": 1e-5}, logit_scale=1.5, logit_softcap=20.0,
        loop={"start": 1, "stop": 3, "times": 2}, layers=[
            {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 4},
             "mlp": {"kind": "moe", "router": {"experts": 6, "top": 2}, "expert": {"ff": 48, "limit": 1.5}, "shared": {"ff": 64, "limit": 2.0}}},
            {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 16, "scale": 0.3, "mask": {"size": 24},
                                            "rot": {"base": 1e4, "dims": 16, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}}},
             "mlp": {"kind": "moe", "router": {"experts": 4, "top": 1}, "expert": {"ff": 80, "limit": 1.0}}},
            {"type": "latent_attention", "mixer": {"heads": 3, "dim": 16, "vdim": 24, "kv_rank": 32, "q_rank": 40, "scale": 0.25,
                                                   "mask": {"size": 17}}, "mlp": None},
        ]), 0.1, 0.05, 16),
}
