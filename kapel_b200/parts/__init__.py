"""Layer parts: mixers, feed-forwards, norms, position encodings, blocks, and the two ends."""
from .attention import Attention
from .base import (BuildContext, LayerCache, Part, linear, matrix_for, matrix_named, pad_columns, product_width,
                   require_product_widths, stack_rows)
from .block import ParallelBlock, PostNormBlock, PreNormBlock, SandwichBlock
from .delta import Delta
from .embedding import Embedding, VocabHead
from .feed_forward import MLP, GatedMLP
from .forget_gate import ForgetGate
from .general_delta import GeneralDelta
from .input_mix import InputAdd, InputMix
from .latent_attention import LatentAttention
from .mlstm import MLSTM
from .moe import MoE
from .norm import LayerNorm, RMSNorm, add_branch
from .parallel import ParallelMixer
from .position import NoPosition, Rope
from .registry import (
    build_part,
    part_class,
    register_block,
    register_feed_forward,
    register_mixer,
    register_norm,
    register_part,
    register_position,
    unregister_part,
)

register_part("mixer", "attention", Attention)
register_part("mixer", "mlstm", MLSTM)
register_part("mixer", "latent_attention", LatentAttention)
register_part("mixer", "delta", Delta)
register_part("mixer", "general_delta", GeneralDelta)
register_part("mixer", "forget_gate", ForgetGate)
register_part("mixer", "parallel", ParallelMixer)
register_part("merge", "input_mix", InputMix)
register_part("merge", "input_add", InputAdd)
register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "mlp", MLP)
register_part("feed_forward", "moe", MoE)
register_part("norm", "rms", RMSNorm)
register_part("norm", "layer", LayerNorm)
register_part("position", "rope", Rope)
register_part("position", "none", NoPosition)
register_part("block", "sandwich", SandwichBlock)
register_part("block", "prenorm", PreNormBlock)
register_part("block", "postnorm", PostNormBlock)
register_part("block", "parallel", ParallelBlock)
register_part("embedding", "embedding", Embedding)
register_part("head", "vocab_head", VocabHead)


def expected_tensors(spec) -> dict:
    """{tensor name: shape} of everything a model built from `spec` reads."""
    out = {spec.embed.weight: (spec.vocab_size, spec.hidden_size)}
    if getattr(spec.embed, "positions", None):
        out[spec.embed.positions] = (spec.embed.max_positions, spec.hidden_size)
    out[spec.head.weight] = (spec.vocab_size, spec.hidden_size)
    n = spec.final_norm
    out.update(part_class("norm", n.kind).expected_tensors(n))
    for layer in spec.layers:
        out.update(part_class("block", layer.kind).expected_tensors(layer))
    for e in spec.schedule:
        if getattr(e, "before", None) is not None:
            out.update(part_class("merge", e.before.kind).expected_tensors(e.before))
    return out
