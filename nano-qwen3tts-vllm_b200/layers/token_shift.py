"""Token shift: a sublayer's input row is blended, channel by channel, with the previous position's row,

    h_t <- h_t + (h_(t-1) - h_t) * mu,        h_(-1) = 0,

where h_(t-1) is the previous row as it was BEFORE its own blend.  A sequence that runs in portions carries its last
input row in a state slot (float, one row per live sequence and layer); the kernel reads it for the first token of a
portion and replaces it with the portion's last row."""
import torch
from torch import nn

from .. import _native as nat
from ..utils.context import get_context


class TokenShift(nn.Module):
    def __init__(self, width: int):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(width, dtype=torch.float32), requires_grad=False)

    def forward(self, x: torch.Tensor, state: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        """x [n, width] float (the residual stream), state [slots, width] float -> blended rows in ``dtype``."""
        out = torch.empty(x.shape, dtype=dtype, device=x.device)
        nat.token_shift(x, self.weight, state, get_context().step_layout, out)
        return out
