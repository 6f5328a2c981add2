"""Which tensors get packed: a class from the tensor's name, shape and dtype.

  linear  decoder projections that enter a matmul (attention, linear attention, MLP, experts,
          per-layer-embedding projections)
  embed   token embedding and lm_head
  ple     per-layer embedding tables (gather only)
  mm      vision / audio towers and their projectors
  other   norms, routers, scalars, anything unrecognised
Same decisions as the reference's binade/classify.py:43-75.
"""

from __future__ import annotations

import re
from dataclasses import dataclass

MIN_DIM = 256
MM_MARKERS = ("vision_tower", "audio_tower", "vision_embedder", "embed_vision", "embed_audio", "vision_model", "multi_modal_projector", "mm_projector", ".visual.")
# first match wins, in this order
LINEAR_KINDS = (
    ("experts", {"experts"}),
    ("linattn", {"linear_attn"}),
    ("attn", {"q_proj", "k_proj", "v_proj", "o_proj", "qkv_proj", "out_proj"}),
    ("mlp", {"gate_proj", "up_proj", "down_proj", "gate_up_proj", "w1", "w2", "w3"}),
    ("ple_proj", {"per_layer_input_gate", "per_layer_projection", "per_layer_model_projection"}),
)
_LAYER = re.compile(r"^(.*?\blayers\.(\d+))\.")


@dataclass(frozen=True)
class Klass:
    cls: str
    sub: str
    layer: int | None  # decoder layer index; None outside the main stack
    block: str | None = None  # module prefix through the layer index


def classify(name: str, shape: tuple, dtype: str) -> Klass:
    m = _LAYER.search(name)
    block = m.group(1) if m else None
    layer = int(m.group(2)) if m and not name.startswith("mtp.") else None
    parts = name.split(".")
    if any(marker in f".{name}." for marker in MM_MARKERS):
        return Klass("mm", "mm", layer, block)
    if "embed_tokens_per_layer" in parts:
        return Klass("ple", "ple", None)
    for suffix, sub in (("embed_tokens.weight", "embed_tokens"), ("lm_head.weight", "lm_head")):
        if name.endswith(suffix):
            return Klass("embed", sub, None)
    big_matrix = dtype == "BF16" and len(shape) in (2, 3) and min(shape[-2:]) >= MIN_DIM
    # a weight is `<module>.weight`, or a fused expert stack stored without the suffix
    weight_like = parts[-1] == "weight" or (len(shape) == 3 and "experts" in parts)
    if big_matrix and weight_like:
        words = set(parts)
        for sub, names in LINEAR_KINDS:
            if words & names:
                return Klass("linear", sub, layer, block)
    return Klass("other", "norm" if any("norm" in p for p in parts) else "other", layer, block)
