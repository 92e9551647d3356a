"""How a layer's parts are arranged around the residual stream.

Pre-norm (somi_inference/models/qwen2.py:325-339):
    x = x + mixer(norm1(x));  x = x + feed_forward(norm2(x)).
The residual stream `x` is float32 and the sums are made in float32, inside the
norm kernel: a block receives the previous block's output as `pending`, adds it
while normalising, and returns its own feed-forward output as the next `pending`.
"""

from __future__ import annotations

from .registry import ARRANGEMENTS


@ARRANGEMENTS.register("pre_norm")
class PreNormBlock:
    def __init__(self, mixer, feed_forward, norms) -> None:
        if mixer is None or feed_forward is None:
            raise ValueError("the pre-norm arrangement needs a mixer and a feed-forward")
        if set(norms) != {"mixer", "feed_forward"}:
            raise ValueError("the pre-norm arrangement takes the norms 'mixer' and "
                             f"'feed_forward', got {sorted(norms)}")
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = norms["mixer"]
        self.feed_forward_norm = norms["feed_forward"]

    def forward(self, residual, pending, batch, cache, owns_cache):
        h = self.mixer_norm.forward(residual, pending)
        a = self.mixer.forward(h, batch, cache, owns_cache)
        h = self.feed_forward_norm.forward(residual, a)
        return self.feed_forward.forward(h, batch)
