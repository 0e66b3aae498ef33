"""Mukenex as a registry entry: configuration, parts and checkpoint names.

Checkpoint names: ``embed``, ``head``, ``final.norm``; per layer i ``l<i>.norm1`` and, with a feed-forward,
``l<i>.norm2``; with several residual streams ``l<i>.hc1.{in,out,mix}`` and ``l<i>.hc2.{in,out,mix}``; the mixer's
tensors ``l<i>.mix.*`` and the feed-forward's ``l<i>.mlp.*``:

    latent_attention  q, dkv, dkv.norm, uk, uv, sink, g, o      (q, dkv and g rows are packed into one matrix)
    attention         q, k, v with q.b, k.b, v.b, q.norm, k.norm, o      (q, k, v rows and biases are packed)
    lightning         q, k, v, g, o, norm                        (q, k, v, g rows are packed)
    dense             up, down
    moe               e<j>.gate, e<j>.up, e<j>.down for every expert j, table (int32 [vocab, top])

Linear weights are [out, in].
"""
from __future__ import annotations

from typing import List

from ..config.mukenex import MukenexConfig
from ..config.registry import Architecture, register_architecture
from ..weights.plan import SourceTensor, WeightBinding


def mukenex_weight_plan(c: MukenexConfig) -> List[WeightBinding]:
    w = c.width
    plan = [WeightBinding("embedding.weight", (SourceTensor("embed", (c.vocab, w)),))]

    def stream_mix(dst: str, src: str):
        if c.streams is None:
            return []
        s = c.streams
        return [WeightBinding(dst + ".in", (SourceTensor(src + ".in", (s,), "fill", fill=1.0 / s),)),
                WeightBinding(dst + ".out", (SourceTensor(src + ".out", (s,), "fill", fill=1.0),)),
                WeightBinding(dst + ".mix", (SourceTensor(src + ".mix", (s, s), "identity"),))]

    for i, l in enumerate(c.layers):
        src, dst = f"l{i}.", f"layers.{i}."
        plan.append(WeightBinding(dst + "input_norm.weight", (SourceTensor(src + "norm1", (w,), "offset_norm"),)))
        plan += stream_mix(dst + "mixer_mix", src + "hc1")
        m = src + "mix."
        if l.kind == "latent_attention":
            q_rows, down_rows, out_rows = l.heads * (l.dim + l.rot_dim), l.kv_rank + l.rot_dim, l.heads * l.vdim
            plan += [WeightBinding(dst + "mixer.qdkv_proj", (
                         SourceTensor(m + "q", (q_rows, w)), SourceTensor(m + "dkv", (down_rows, w)),
                         SourceTensor(m + "g", (out_rows, w)))),
                     WeightBinding(dst + "mixer.latent_norm", (SourceTensor(m + "dkv.norm", (l.kv_rank,), "norm"),)),
                     WeightBinding(dst + "mixer.uk_proj", (SourceTensor(m + "uk", (l.heads * l.dim, l.kv_rank)),)),
                     WeightBinding(dst + "mixer.uv_proj", (SourceTensor(m + "uv", (out_rows, l.kv_rank)),)),
                     WeightBinding(dst + "mixer.sink", (SourceTensor(m + "sink", (l.heads,)),)),
                     WeightBinding(dst + "mixer.o_proj", (SourceTensor(m + "o", (w, out_rows)),))]
        elif l.kind == "attention":
            q_rows, k_rows, v_rows = l.heads * l.dim, l.kv_heads * l.dim, l.kv_heads * l.vdim
            plan += [WeightBinding(dst + "mixer.qkv_proj", (
                         SourceTensor(m + "q", (q_rows, w)), SourceTensor(m + "k", (k_rows, w)),
                         SourceTensor(m + "v", (v_rows, w)))),
                     WeightBinding(dst + "mixer.qkv_bias", (
                         SourceTensor(m + "q.b", (q_rows,)), SourceTensor(m + "k.b", (k_rows,)),
                         SourceTensor(m + "v.b", (v_rows,)))),
                     WeightBinding(dst + "mixer.q_norm", (SourceTensor(m + "q.norm", (l.dim,), "norm"),)),
                     WeightBinding(dst + "mixer.k_norm", (SourceTensor(m + "k.norm", (l.dim,), "norm"),)),
                     WeightBinding(dst + "mixer.o_proj", (SourceTensor(m + "o", (w, l.heads * l.vdim)),))]
        else:
            qk_rows, v_rows = l.heads * l.dim, l.heads * l.vdim
            plan += [WeightBinding(dst + "mixer.qkvg_proj", (
                         SourceTensor(m + "q", (qk_rows, w)), SourceTensor(m + "k", (qk_rows, w)),
                         SourceTensor(m + "v", (v_rows, w)), SourceTensor(m + "g", (v_rows, w)))),
                     WeightBinding(dst + "mixer.norm", (SourceTensor(m + "norm", (v_rows,), "norm"),)),
                     WeightBinding(dst + "mixer.o_proj", (SourceTensor(m + "o", (w, v_rows)),))]
        if l.ff is not None:
            plan.append(WeightBinding(dst + "post_mixer_norm.weight", (SourceTensor(src + "norm2", (w,), "offset_norm"),)))
            plan += stream_mix(dst + "ff_mix", src + "hc2")
            f = src + "mlp."
            if l.ff.kind == "dense":
                plan += [WeightBinding(dst + "feed_forward.up_proj", (SourceTensor(f + "up", (l.ff.ff, w)),)),
                         WeightBinding(dst + "feed_forward.down_proj", (SourceTensor(f + "down", (w, l.ff.ff)),))]
            else:
                gate_up, down = [], []
                for e in range(l.ff.experts):
                    gate_up += [SourceTensor(f"{f}e{e}.gate", (l.ff.ff, w)), SourceTensor(f"{f}e{e}.up", (l.ff.ff, w))]
                    down.append(SourceTensor(f"{f}e{e}.down", (w, l.ff.ff)))
                plan += [WeightBinding(dst + "feed_forward.gate_up_proj", tuple(gate_up)),
                         WeightBinding(dst + "feed_forward.down_proj", tuple(down)),
                         WeightBinding(dst + "feed_forward.table", (
                             SourceTensor(f + "table", (c.vocab, l.ff.top), "choices", integer=True,
                                          modulus=l.ff.experts),))]
    plan.append(WeightBinding("final_norm.weight", (SourceTensor("final.norm", (w,), "offset_norm"),)))
    plan.append(WeightBinding("lm_head.weight", (SourceTensor("head", (c.vocab, w)),)))
    return plan


MUKENEX = Architecture(name=MukenexConfig.architecture, model_type=MukenexConfig.model_type,
                       parse_config=MukenexConfig.parse, model_spec=MukenexConfig.model_spec,
                       weight_plan=mukenex_weight_plan, checkpoint_dtype=lambda c: "bfloat16")

register_architecture(MUKENEX, replace=True)
