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
        if self.mixer.fuses_with_stream:
            stream.pend(self.mixer.forward(self.mixer_norm.forward(stream, lazy=True), step, cache, stream=stream))
        else:
            stream.pend(self.mixer.forward(self.mixer_norm.forward(stream), step, cache))
        if self.feed_forward.fuses_with_stream:
            stream.pend(self.feed_forward.forward(self.feed_forward_norm.forward(stream, lazy=True), stream=stream))
        else:
            stream.pend(self.feed_forward.forward(self.feed_forward_norm.forward(stream)))
