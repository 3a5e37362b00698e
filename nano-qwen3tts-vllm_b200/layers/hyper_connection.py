"""Several residual streams mixed by small learned matrices around every sublayer ("hyper-connections").

A token carries ``streams`` copies x_1 .. x_s of the residual vector.  Around a sublayer f with its pre-norm:

    u   = sum_s in[s] x_s                      (the sublayer's input, read out of the streams)
    y   = f(norm(u))
    x_t <- sum_s mix[s, t] x_s + out[t] y      (all streams at once from the old ones; mix is indexed [from, to])

With one stream, in = out = mix = 1 is the ordinary pre-norm residual, which is what ``StreamConnection(1)`` holds until
tensors are loaded.  The update after one sublayer and the read-out + norm in front of the next ride in one launch
(``step``); the streams tensor [n, streams, width] is float and updated in place."""
import torch
from torch import nn

from .. import _native as nat


class StreamConnection(nn.Module):
    def __init__(self, streams: int):
        super().__init__()
        f32 = dict(dtype=torch.float32)
        self.streams = streams
        self.in_w = nn.Parameter(torch.ones(streams, **f32), requires_grad=False)
        self.out_w = nn.Parameter(torch.ones(streams, **f32), requires_grad=False)
        self.mix = nn.Parameter(torch.eye(streams, **f32), requires_grad=False)


def step(xs: torch.Tensor, outputs, post: StreamConnection | None, pre: StreamConnection | None, norm, dtype: torch.dtype):
    """``outputs`` = (y1, y2, c1, c2) of the sublayer just run (its result is c1*y1 + c2*y2; y2 may be None), written
    into the streams through ``post``; then the next sublayer's normed input is read through ``pre`` and ``norm``
    (an RMS norm module with ``weight`` and ``eps``).  Either half may be absent.  Returns the normed input or None."""
    n, _, width = xs.shape
    h = torch.empty(n, width, dtype=dtype, device=xs.device) if pre is not None else None
    y1, y2, c1, c2 = outputs if outputs is not None else (None, None, 1.0, 0.0)
    nat.stream_mix_norm(xs, y1, y2, c1, c2, post.mix if post is not None else None, post.out_w if post is not None else None,
                        pre.in_w if pre is not None else None, norm.weight if pre is not None else None, h,
                        norm.eps if pre is not None else 0.0, dtype)
    return h
