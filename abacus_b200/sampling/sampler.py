"""Choosing the next token: greedy, or top-k at a temperature, as src/main.c:31-56.

abacus samples one sequence with one xorshift64 state seeded by --seed. Here
every request has a state of its own, `stream_seed(seed, request index)`, so
what a request draws does not depend on which batch it runs in; request 0 uses
`seed` itself and so draws what abacus would. One deviation: xorshift64 never
leaves state 0 (every draw would take the top token), and abacus never starts
there because its default seed is the time (src/main.c:112); here a stream whose
state would be 0 starts from a fixed non-zero constant instead.
"""
import torch

from ..kernels import ops

MASK64 = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15


def stream_seed(seed, request_index):
    """Initial xorshift64 state of a request; never 0 (the state xorshift64 cannot leave)."""
    return ((seed ^ (request_index * GOLDEN)) & MASK64) or GOLDEN


def as_signed(u):
    return u - (1 << 64) if u >= (1 << 63) else u


class Sampler:
    """temperature <= 0: first maximum (src/main.c:31-36). Else: draw among the top_k logits with
    p_j = exp((l_j - l_max) / temperature) (src/main.c:39-56; abacus fixes top_k at 20). top_k = 0: the whole
    vocabulary, walked in index order instead of by falling logit (the same distribution, no list to sort)."""

    def __init__(self, device, temperature=0.7, top_k=20, seed=0):
        self.device, self.temperature, self.top_k, self.seed = device, float(temperature), int(top_k), int(seed)
        if self.temperature > 0 and not 0 <= self.top_k <= 64:
            raise ValueError(f"top_k {top_k} is neither 0 (the whole vocabulary) nor in 1..64")

    @property
    def greedy(self):
        return self.temperature <= 0.0

    def states(self, request_indices):
        """xorshift64 states (as int64 bit patterns) for the given requests, on the device."""
        vals = [as_signed(stream_seed(self.seed, i)) for i in request_indices]
        return torch.tensor(vals, dtype=torch.int64, device=self.device)

    def sample(self, logits, states, index=None, out=None):
        """logits float32 [rows, vocab]. Row r draws with states[index[r]] (states[r] without index),
        which advances. Returns int32 [rows] on the device."""
        n = logits.shape[0]
        if out is None:
            out = torch.empty(n, dtype=torch.int32, device=logits.device)
        if self.greedy:
            ops.argmax(logits, out, n)
        elif self.top_k == 0:
            ops.sample_all(logits, self.temperature, states, out, n, rng_index=index)
        else:
            ops.sample_topk(logits, self.temperature, self.top_k, states, out, n, rng_index=index)
        return out
