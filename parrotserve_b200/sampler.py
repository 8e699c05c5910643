"""Drop-in for the builtin engine's token sampler with the reference's interface
(parrot/engine/builtin/models/sampler.py:13-66): ``Sampler(config, embd_weight)`` and
``forward(hidden_states, sampling_config) -> int64 ids``.

The logits are one library GEMM against the (tied) embedding matrix, as in the reference; everything
after it (temperature, nucleus filtering, softmax, the draw) is one CUDA kernel, ``pb_sample_top_p``,
which replaces the reference's sort / softmax / cumsum / gather / softmax / multinomial chain."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import ops


class Sampler(torch.nn.Module):
    def __init__(self, config, embd_weight: torch.Tensor):
        super().__init__()
        self.embd_weight = embd_weight  # a reference to the model's embedding, not a copy
        self.vocab_size = config.vocab_size
        self.generator: Optional[torch.Generator] = None  # source of the uniform numbers; None = torch's default

    def forward(self, hidden_states: torch.Tensor, sampling_config: Sequence) -> torch.Tensor:
        if hidden_states.shape[0] == 0:
            return torch.zeros(0, dtype=torch.int64, device=hidden_states.device)
        if hidden_states.shape[0] != len(sampling_config):
            raise AssertionError("one sampling config per row of hidden states")
        logits = torch.matmul(hidden_states, self.embd_weight.t())
        return ops.sample_top_p(logits, [sc.temperature for sc in sampling_config],
                                [sc.top_p for sc in sampling_config], generator=getattr(self, "generator", None))


def install() -> None:
    """Gives the reference's own ``Sampler`` class (parrot/engine/builtin/models/sampler.py:13-17,
    built by the models with ``Sampler(config, embed_tokens.weight)``) this module's ``forward``,
    without editing Parrot: existing models pick it up at their next call."""
    from parrot.engine.builtin.models import sampler as ref_sampler

    ref_sampler.Sampler.forward = Sampler.forward
