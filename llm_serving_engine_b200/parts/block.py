"""The arrangement of the parts in a layer."""
from __future__ import annotations

from .base import Block, ResidualStream, register_block


@register_block("prenorm_residual")
class PreNormResidualBlock(Block):
    """h = h + mixer(norm1(h)); h = h + feed_forward(norm2(h))
    (reference ``src/llmserve/model.py:199-201,233-234``).  Each branch output
    stays pending in the stream; the next norm adds it to the float32 residual."""

    graph_safe = True

    def forward(self, stream: ResidualStream, step, cache) -> None:
        x = self.mixer_norm.forward(stream)
        stream.delta = self.mixer.forward(x, step, cache)
        x = self.feed_forward_norm.forward(stream)
        stream.delta = self.feed_forward.forward(x)
