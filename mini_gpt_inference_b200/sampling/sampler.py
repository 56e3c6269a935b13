"""Choose the next token of each request from its logits, on the device.

Rows whose temperature is 0 (or below) take the argmax; the others are drawn as the
reference draws (src/minigpt_infer/sampling.py:97-137: temperature, top-k, top-p, softmax,
one draw), each row with its own parameters.  A vocabulary limit plays the part of the
reference's mask over padding ids (src/minigpt_infer/tokenizer.py:37-46: ids at or above
the tokenizer's size are never produced).  Every request draws from its own counter-based
stream: word ``n`` of request ``r`` depends on ``(seed_r, n)`` only.
"""

from __future__ import annotations

import numpy as np
import torch

_MASK32 = 0xFFFFFFFF


def _as_i32(values) -> np.ndarray:
    return np.asarray(values, dtype=np.uint32).view(np.int32)


class Sampler:
    def __init__(self, ops, device, vocab_limit: int | None = None, base_seed: int = 0) -> None:
        self.ops = ops
        self.device = torch.device(device)
        self.vocab_limit = vocab_limit
        self._seed_source = np.random.SeedSequence(base_seed)
        self._rng = np.random.default_rng(self._seed_source)
        # Two pinned staging buffers for the per-row parameters, used in turn: the copy to the
        # device is asynchronous, so the host does not wait for the step that is still running.
        self._staging = [None, None]
        self._copied = [None, None]
        self._turn = 0

    def _to_device(self, packed: np.ndarray) -> torch.Tensor:
        if self.device.type != "cuda":
            return torch.from_numpy(packed).to(self.device)
        slot, self._turn = self._turn, self._turn ^ 1
        if self._copied[slot] is not None:
            self._copied[slot].synchronize()              # the copy before last has left this buffer
        need = packed.size
        if self._staging[slot] is None or self._staging[slot].numel() < need:
            self._staging[slot] = torch.empty(max(need, 6 * 64), dtype=torch.int32, pin_memory=True)
        flat = self._staging[slot][:need]
        flat.numpy()[:] = packed.reshape(-1)
        dev = flat.to(self.device, non_blocking=True).view(packed.shape)
        if self._copied[slot] is None:
            self._copied[slot] = torch.cuda.Event()
        self._copied[slot].record()
        return dev

    def fresh_seed(self) -> int:
        """A seed for a request that gave none."""
        return int(self._rng.integers(0, 2**63 - 1))

    def sample(self, logits: torch.Tensor, params, seeds, draw_numbers, greedy_ids=None,
               out=None) -> torch.Tensor:
        """``params[i]`` has temperature/top_k/top_p; returns int32 ids ``[rows]`` on the device.

        ``greedy_ids``: the argmax of every row if the step that made the logits took it already
        (a replayed decode step does); it is returned as it is when every row is greedy.
        ``out``: where to write the ids instead of a new tensor."""
        rows = logits.shape[0]
        if rows == 0:
            return torch.empty((0,), dtype=torch.int32, device=logits.device)
        if all(p.temperature <= 0 for p in params):
            if greedy_ids is not None:
                return greedy_ids
            if out is not None:
                return self.ops.argmax(logits, self.vocab_limit, out=out)
            return self.ops.argmax(logits, self.vocab_limit)
        vocab = logits.shape[1]
        packed = np.zeros((6, rows), dtype=np.int32)
        packed[0] = np.asarray([p.temperature for p in params], dtype=np.float32).view(np.int32)
        packed[1] = [p.top_k if p.top_k is not None else 0 for p in params]
        packed[2] = np.asarray([p.top_p if p.top_p is not None else 1.0 for p in params],
                               dtype=np.float32).view(np.int32)
        packed[3] = _as_i32([s & _MASK32 for s in seeds])
        packed[4] = _as_i32([(s >> 32) & _MASK32 for s in seeds])
        packed[5] = _as_i32([n & _MASK32 for n in draw_numbers])
        dev = self._to_device(packed)
        use_k = any(p.top_k is not None and p.top_k < vocab for p in params)
        use_p = any(p.top_p is not None and p.top_p < 1.0 for p in params)
        extra = {} if out is None else {"out": out}
        return self.ops.sample(logits, dev[0].view(torch.float32), dev[1] if use_k else None,
                               dev[2].view(torch.float32) if use_p else None,
                               dev[3], dev[4], dev[5], self.vocab_limit, **extra)
