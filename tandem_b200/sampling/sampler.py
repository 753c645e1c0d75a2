"""From logits to tokens: greedy, or temperature sampling with top-k, top-p and min-p.

The rules are 12vivi/tandem's (python/tandem/layers/sampler.py:19-64): a request is greedy when
its temperature is below 1e-5; otherwise logits / temperature, keep the top_k largest, softmax,
keep the smallest head of the sorted distribution whose preceding mass exceeds top_p nowhere,
drop what is below min_p times the largest probability, renormalise, draw.  All of it runs in
one CUDA kernel per step, a cluster of blocks per row (``tandem_b200/csrc/sampling.cu``); the draw is the inverse CDF at a
uniform number that depends only on the request's seed and the index of the token, so it does
not depend on the batch (``tandem_b200.sampling.rng``).
"""

from __future__ import annotations

from typing import Sequence

import torch

from tandem_b200.kernels import ops
from tandem_b200.sampling.params import SamplingParams
from tandem_b200.sampling.rng import uniform


def sample(logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
           counters: Sequence[int]) -> list:
    """logits [R, V] float32 on the device -> R token ids on the host.  Row r is drawn with
    ``uniform(seeds[r], counters[r])``."""
    if logits.shape[0] == 0:
        return []
    return sample_on_device(logits, params, seeds, counters).tolist()


def sample_on_device(logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
                     counters: Sequence[int]) -> torch.Tensor:
    """As ``sample``, but the R token ids stay on the device (int32): the caller decides when
    the host reads them."""
    if all(p.greedy for p in params):
        return ops.argmax(logits)
    dev = logits.device
    host = torch.tensor(
        [[p.temperature for p in params], [p.top_p for p in params], [p.min_p for p in params],
         [uniform(s, c) for s, c in zip(seeds, counters)]], dtype=torch.float32).pin_memory()
    ks = torch.tensor([p.top_k for p in params], dtype=torch.int32).pin_memory()
    f = host.to(dev, non_blocking=True)
    k = ks.to(dev, non_blocking=True)
    return ops.sample(logits, f[0], k, f[1], f[2], f[3], any_top_k=any(p.top_k > 0 for p in params),
                      any_top_p=any(p.top_p < 1.0 for p in params))
