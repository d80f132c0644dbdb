"""Fixed-slot store for recurrent mixers, the counterpart of the KV pool for layers whose memory does not grow
with the sequence: per recurrent layer one fp32 state tensor ``[slots, *spec.state_shape]`` (a state-space or
linear-attention memory ``heads x state x head_dim``, or one value per channel of an element-wise recurrence) and,
for mixers with a short convolution, its tail ``[slots, taps - 1, channels]`` (the last inputs, in the activation dtype;
a mixer with several convolutions names one tail per convolution in ``spec.conv_tails``).

A request holds one slot from admission to release; the same slot number indexes the request -> rows table of the
KV pool (``ModelRunner.b_req_tokens_table``), as the reference's slot scheme does for attention
(lite_llama/executor/slot_batch.py:28-60).  Slots are not cleared when they change hands: a sequence with no cached
tokens never reads its slot (the kernels start it from zero), so reuse costs nothing.
"""

from __future__ import annotations

import torch

from .model_config import LayeredConfig


class RecurrentStateManager:
    def __init__(self, config: LayeredConfig, num_slots: int, dtype: torch.dtype, device: str = "cuda") -> None:
        self.num_slots = num_slots
        self.device = device
        self.ssm_state: dict[int, torch.Tensor] = {}
        self.conv_tail: dict[int, torch.Tensor] = {}
        self.named_tail: dict[int, dict[str, torch.Tensor]] = {}     # mixers with several convolutions: one tail each
        for i in config.recurrent_layers():
            m = config.layers[i].mixer
            self.ssm_state[i] = torch.zeros((num_slots, *m.state_shape), dtype=torch.float32, device=device)
            if m.conv_tail_shape is not None:
                self.conv_tail[i] = torch.zeros((num_slots, *m.conv_tail_shape), dtype=dtype, device=device)
            if getattr(m, "conv_tails", None):
                self.named_tail[i] = {name: torch.zeros((num_slots, *shape), dtype=dtype, device=device)
                                      for name, shape in m.conv_tails.items()}
        self._free = list(range(num_slots - 1, -1, -1))
        self._held: set[int] = set()

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def acquire(self) -> int:
        if not self._free:
            raise RuntimeError(f"all {self.num_slots} request slots are held")
        slot = self._free.pop()
        self._held.add(slot)
        return slot

    def release(self, slot: int) -> None:
        if slot not in self._held:
            raise ValueError(f"slot {slot} is not held")
        self._held.remove(slot)
        self._free.append(slot)

    def nbytes(self) -> int:
        named = [t for d in self.named_tail.values() for t in d.values()]
        return sum(t.numel() * t.element_size() for t in [*self.ssm_state.values(), *self.conv_tail.values(), *named])
