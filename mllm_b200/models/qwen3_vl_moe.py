"""Qwen3-VL with a mixture-of-experts text model (``Qwen3VLMoeForConditionalGeneration``): the Qwen3-VL
vision tower, deepstack injection and 3-D rope positions on top of the Qwen3-MoE decoder (router,
grouped expert GEMMs, tensor / expert parallelism).  Both parents derive from the dense Qwen3 model, so the
class only has to put them in the right order: the vision-language wrapper's ``forward`` / ``load_weights``
first, the MoE model's decoder class, expert loader and post-load step behind it."""

from __future__ import annotations

from .qwen3_moe import Qwen3MoeForCausalLM
from .qwen3_vl import Qwen3VLForConditionalGeneration


class Qwen3VLMoeForConditionalGeneration(Qwen3VLForConditionalGeneration, Qwen3MoeForCausalLM):
    pass


EntryClass = Qwen3VLMoeForConditionalGeneration
