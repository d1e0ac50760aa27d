"""Mixture-of-experts feed-forward with a sigmoid top-k router.

Router logits are computed in float; the ``top`` experts with the largest sigmoid scores are chosen, and their
weights are the scores divided by their sum (+ 1e-20) times ``scale``.  Experts are two-matrix feed-forwards with a
squared-ReLU activation, stored stacked ([experts, ff, width] / [experts, width, ff]) so that ONE grouped launch runs
all of them over the (token, choice) pairs sorted by expert - for a prompt portion of thousands of tokens and for a
decode step of a few rows per expert alike, with no group size ever read back to the host.  ``forward`` returns the
per-pair outputs and weights;
the weighted sum over a token's choices is taken, in a fixed order, by the residual kernel that consumes them."""
import torch
from torch import nn

from .. import _native as nat


class SigmoidTopKMoE(nn.Module):
    def __init__(self, width: int, ff: int, experts: int, top: int, scale: float):
        super().__init__()
        self.width, self.ff, self.experts, self.top, self.scale = width, ff, experts, top, scale
        self.router = nn.Parameter(torch.zeros(experts, width, dtype=torch.float32), requires_grad=False)
        self.up = nn.Parameter(torch.empty(experts, ff, width), requires_grad=False)
        self.down = nn.Parameter(torch.empty(experts, width, ff), requires_grad=False)

    def route(self, h: torch.Tensor):
        n, dev = h.shape[0], h.device
        top_idx = torch.empty(n, self.top, dtype=torch.int32, device=dev)
        top_w = torch.empty(n, self.top, dtype=torch.float32, device=dev)
        offsets = torch.empty(self.experts + 1, dtype=torch.int32, device=dev)
        sorted_pair = torch.empty(n * self.top, dtype=torch.int32, device=dev)
        nat.moe_route(h, self.router, top_idx, top_w, offsets, sorted_pair, self.top, self.scale)
        return top_idx, top_w, offsets, sorted_pair

    def forward(self, h: torch.Tensor):
        """h [n, width] -> (z [n * top, width], weights [n, top]): z[t * top + k] is the output of token t's k-th expert."""
        n = h.shape[0]
        pairs = n * self.top
        _, top_w, offsets, sorted_pair = self.route(h)
        y = torch.empty(pairs, self.ff, dtype=h.dtype, device=h.device)
        nat.grouped_gemm(h, self.up, y, offsets, sorted_pair, pairs, self.top, in_by_token=True, out_by_pair=False, act=1)
        z = torch.empty(pairs, self.width, dtype=h.dtype, device=h.device)
        nat.grouped_gemm(y, self.down, z, offsets, sorted_pair, pairs, self.top, in_by_token=False, out_by_pair=True, act=0)
        return z, top_w
