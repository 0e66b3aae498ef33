"""Kefetar as a registry entry: configuration, parts and checkpoint names.

Checkpoint names: ``embed``, ``head``, ``final.norm``; per layer i ``l<i>.norm1`` / ``l<i>.canon1`` (mixer
sublayer) and, with a feed-forward, ``l<i>.norm2`` / ``l<i>.canon2`` and ``l<i>.mlp.{up,down,act}``; the mixer's
``l<i>.mix.{q,k,v,g,o}``, for attention also ``l<i>.mix.{q,k,v}.conv`` and ``l<i>.mix.vmix``.  Linear weights are
[out, in].  q, k, v and gate rows are packed in that order into one matrix, the three convolutions' taps likewise.
"""
from __future__ import annotations

from typing import List

from ..config.kefetar import KefetarConfig
from ..config.registry import Architecture, register_architecture
from ..weights.plan import SourceTensor, WeightBinding


def kefetar_weight_plan(c: KefetarConfig) -> List[WeightBinding]:
    w = c.width
    plan = [WeightBinding("embedding.weight", (SourceTensor("embed", (c.vocab, w)),))]
    for i, l in enumerate(c.layers):
        src, dst = f"l{i}.", f"layers.{i}."
        plan.append(WeightBinding(dst + "input_norm.weight", (SourceTensor(src + "norm1", (), "norm"),)))
        if c.canon_taps >= 1:
            plan.append(WeightBinding(dst + "mixer_conv.weight", (SourceTensor(src + "canon1", (w, c.canon_taps)),)))
        kv = l.kv_heads if l.kind == "attention" else l.heads
        q_rows, k_rows, v_rows, g_rows = l.heads * l.dim, kv * l.dim, kv * l.vdim, l.heads * l.vdim
        plan.append(WeightBinding(dst + "mixer.qkvg_proj", (
            SourceTensor(src + "mix.q", (q_rows, w)), SourceTensor(src + "mix.k", (k_rows, w)),
            SourceTensor(src + "mix.v", (v_rows, w)), SourceTensor(src + "mix.g", (g_rows, w)))))
        plan.append(WeightBinding(dst + "mixer.o_proj", (SourceTensor(src + "mix.o", (w, g_rows)),)))
        if l.kind == "attention":
            if l.conv >= 1:
                plan.append(WeightBinding(dst + "mixer.conv", (
                    SourceTensor(src + "mix.q.conv", (q_rows, l.conv)), SourceTensor(src + "mix.k.conv", (k_rows, l.conv)),
                    SourceTensor(src + "mix.v.conv", (v_rows, l.conv)))))
            if l.v_mix:
                plan.append(WeightBinding(dst + "mixer.vmix", (SourceTensor(src + "mix.vmix", ()),)))
        if l.ff is not None:
            plan.append(WeightBinding(dst + "post_mixer_norm.weight", (SourceTensor(src + "norm2", (), "norm"),)))
            if c.canon_taps >= 1:
                plan.append(WeightBinding(dst + "ff_conv.weight", (SourceTensor(src + "canon2", (w, c.canon_taps)),)))
            plan += [WeightBinding(dst + "feed_forward.up_proj", (SourceTensor(src + "mlp.up", (l.ff, w)),)),
                     WeightBinding(dst + "feed_forward.down_proj", (SourceTensor(src + "mlp.down", (w, l.ff)),)),
                     WeightBinding(dst + "feed_forward.act", (SourceTensor(src + "mlp.act", (4,), "norm"),))]
    plan.append(WeightBinding("final_norm.weight", (SourceTensor("final.norm", (), "norm"),)))
    plan.append(WeightBinding("lm_head.weight", (SourceTensor("head", (c.vocab, w)),)))
    return plan


KEFETAR = Architecture(name=KefetarConfig.architecture, model_type=KefetarConfig.model_type,
                       parse_config=KefetarConfig.parse, model_spec=KefetarConfig.model_spec,
                       weight_plan=kefetar_weight_plan, checkpoint_dtype=lambda c: "bfloat16")

register_architecture(KEFETAR, replace=True)
