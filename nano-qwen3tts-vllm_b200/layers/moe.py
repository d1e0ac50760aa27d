"""Mixture-of-experts feed-forward with a sigmoid top-k router.

Router logits are computed in float; the ``top`` experts with the largest sigmoid scores are chosen, and their
weights are the scores divided by their sum (+ 1e-20) times ``scale``.  Experts are two-matrix feed-forwards with a
squared-ReLU activation, stored stacked ([experts, ff, width] / [experts, width, ff]) so that ONE grouped launch runs
all of them over the (token, choice) pairs sorted by expert.  ``forward`` returns the per-pair outputs and weights;
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

    # (token, choice) pairs from which the experts run as one library GEMM each over their gathered rows (compute-bound
    # prompt portions); below it - decoding - the one grouped launch serves all experts and nothing waits on the host
    SORTED_GEMM_MIN_PAIRS = 2048

    def forward(self, h: torch.Tensor):
        """h [n, width] -> (z [n * top, width], weights [n, top]): z[t * top + k] is the output of token t's k-th expert."""
        n = h.shape[0]
        pairs = n * self.top
        _, top_w, offsets, sorted_pair = self.route(h)
        if pairs >= self.SORTED_GEMM_MIN_PAIRS and not torch.cuda.is_current_stream_capturing():
            return self._sorted_gemms(h, offsets, sorted_pair, pairs), top_w
        y = torch.empty(pairs, self.ff, dtype=h.dtype, device=h.device)
        nat.grouped_gemm(h, self.up, y, offsets, sorted_pair, pairs, self.top, in_by_token=True, out_by_pair=False, act=1)
        z = torch.empty(pairs, self.width, dtype=h.dtype, device=h.device)
        nat.grouped_gemm(y, self.down, z, offsets, sorted_pair, pairs, self.top, in_by_token=False, out_by_pair=True, act=0)
        return z, top_w

    def _sorted_gemms(self, h, offsets, sorted_pair, pairs):
        """Rows gathered in expert order, one GEMM pair per expert over its contiguous slice (the group sizes are read
        back: one host synchronisation per layer), results scattered back to (token, choice) order."""
        from .linear import linear
        xs = nat.permute_rows(h, torch.empty(pairs, self.width, dtype=h.dtype, device=h.device), sorted_pair, div=self.top)
        bounds = offsets.tolist()
        y = torch.empty(pairs, self.ff, dtype=h.dtype, device=h.device)
        for e in range(self.experts):
            lo, hi = bounds[e], bounds[e + 1]
            if hi > lo:
                linear(xs[lo:hi], self.up[e], out=y[lo:hi])
        nat.relu_sq_(y)
        zs = xs                                             # the gathered inputs are dead: reuse their rows
        for e in range(self.experts):
            lo, hi = bounds[e], bounds[e + 1]
            if hi > lo:
                linear(y[lo:hi], self.down[e], out=zs[lo:hi])
        return nat.permute_rows(zs, torch.empty(pairs, self.width, dtype=h.dtype, device=h.device), sorted_pair, scatter=True)
