"""The sampler's device side: one xorshift64 state per cache slot (a fixed-size record that
lives as long as the sequence), and the two kernels: first-maximum argmax for greedy,
radix top-k sampling otherwise."""
import torch

from ..csrc import ops
from .params import SamplingParams


def to_signed(u):
    return u - (1 << 64) if u >= (1 << 63) else u


class DeviceSampler:
    def __init__(self, n_slots, device):
        self.state = torch.zeros(n_slots, dtype=torch.int64, device=device)
        self.scratch = torch.zeros(n_slots, dtype=torch.int32, device=device)  # a word per row for the sampling kernels
        self.device = device

    def seed(self, slots, params: SamplingParams, first_request_index=0):
        """Start the streams of the sequences in `slots` (request i of the call uses seed + i)."""
        if params.greedy or not slots:
            return
        vals = torch.tensor([to_signed(params.initial_state(first_request_index + i)) for i in range(len(slots))], dtype=torch.int64)
        idx = torch.tensor(list(slots), dtype=torch.int64)
        self.state.index_copy_(0, idx.to(self.device), vals.to(self.device))

    def sample(self, logits, params: SamplingParams, seq_slots, out):
        """out[r] <- the token chosen from logits[r]; row r draws from the stream of slot seq_slots[r]."""
        if params.greedy:
            ops.argmax_rows(logits, out)
        else:
            scratch = self.scratch if logits.shape[0] <= self.scratch.numel() else None
            ops.sample_topk(logits, float(params.temperature), int(params.top_k), self.state, out, state_index=seq_slots, scratch=scratch)
        return out
