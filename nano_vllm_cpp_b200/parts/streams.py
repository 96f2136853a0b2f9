"""Several copies of the residual stream, and the sublayers wired around them (hyper-connections).

A model with ``streams`` = n keeps n copies ``x_1 .. x_n`` of its residual stream, all equal to the embedding at the
start, in one float32 matrix ``[T, n * hidden]`` (copy after copy inside a row).  A sublayer F with its norm and its
link (three small learned tensors: ``read`` [n], ``carry`` [n, n] indexed [from, to], ``write`` [n]) computes

    u = sum_c read[c] x_c;   y = F(norm(u));   x_d <- sum_c carry[c, d] x_c + write[d] y    (all d from the old copies)

and at the end of the model the copies are summed.  With n = 1, read = write = carry = 1 this is the pre-norm layer.

The update is not done where y is computed: as everywhere in this package the sublayer's output stays *pending*
(here a ``StreamUpdate``: y together with the link it goes through) and whoever reads the stream next, the next
sublayer's norm or the model's final norm, brings the copies up to date in its own kernel (``ops.stream_mix_norm``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..csrc import ops
from .base import Part, RowMix, TensorSpec
from .block import Arrangement
from .registry import register_part


class StreamLink(Part):
    """The three tensors that tie one sublayer to the copies of the stream; held in float32."""

    def __init__(self, streams: int, read_name: str = "in", write_name: str = "out", carry_name: str = "mix"):
        if not 1 <= streams <= ops.STREAM_MAX_STREAMS:
            raise ValueError(f"a model keeps 1 to {ops.STREAM_MAX_STREAMS} copies of its stream, found {streams}")
        self.streams = streams
        self.read_name, self.write_name, self.carry_name = read_name, write_name, carry_name

    def tensor_specs(self, available=None):
        n = self.streams
        return {self.read_name: TensorSpec((n,), init="mean", kind="vector"),
                self.write_name: TensorSpec((n,), init="ones", kind="vector"),
                self.carry_name: TensorSpec((n, n), init="identity", kind="vector")}

    def load(self, fetch, ctx):
        self.ctx = ctx
        self.read = fetch(self.read_name).float().contiguous()
        self.write = fetch(self.write_name).float().contiguous()
        self.carry = fetch(self.carry_name).float().contiguous()


register_part("connection", "stream_link", StreamLink)


@dataclass
class StreamUpdate:
    """A sublayer's output (a float32 matrix or a ``RowMix``) that the copies of the stream have not taken in yet,
    with the link it goes through."""
    branch: object
    link: StreamLink


def read_streams(norm, x, streams: int, pending, read, want_f32: bool = False):
    """Brings the copies ``x`` up to date with ``pending`` (a ``StreamUpdate`` or None), reads them with ``read``
    ([streams] float32, None: the plain sum) and norms the result.  A norm that has ``read_streams`` does all of it
    in one kernel; any other norm gets what was read as a stream of its own."""
    branch = carry = write = None
    if pending is not None:
        if not isinstance(pending, StreamUpdate):
            raise TypeError("the copies of a stream take a StreamUpdate")
        branch, carry, write = pending.branch, pending.link.carry, pending.link.write
    if hasattr(norm, "read_streams"):
        return norm.read_streams(x, streams, branch, carry, write, read, want_f32)
    mix = None
    if isinstance(branch, RowMix):
        if branch.gate_logit is None and branch.index.shape[1] <= ops.STREAM_MAX_MIX:
            mix, branch = branch.as_tuple(), None
        else:
            branch = branch.sum()
    u = torch.empty((x.shape[0], x.shape[1] // streams), dtype=torch.float32, device=x.device)
    ops.stream_mix_norm(x, streams, branch=branch, mix=mix, carry=carry, write=write, read=read, out32=u)
    return norm.forward(u, None, want_f32)


class HyperConnectedBlock(Arrangement):
    """A pre-norm layer around ``streams`` copies of the residual stream (``LayerSpec.params["streams"]``): the mixer
    behind ``norm1`` through ``link1``, then, if the layer has one, the feed-forward behind ``norm2`` through
    ``link2``.  ``x`` is ``[T, streams * hidden]``; the layer's last output is handed on as a ``StreamUpdate``."""
    slots = {"norm1": "norm", "mixer": "mixer", "link1": "connection", "norm2": "norm", "feed_forward": "feed_forward",
             "link2": "connection"}
    optional = ("norm2", "feed_forward", "link2")

    def __init__(self, spec):
        super().__init__(spec)
        self.streams = int(spec.params.get("streams", 1))
        present = [getattr(self, s) is not None for s in self.optional]
        if any(present) != all(present):
            raise ValueError("a hyper-connected layer's feed-forward comes with its norm and its link")
        for link in (self.link1, self.link2):
            if link is not None and link.streams != self.streams:
                raise ValueError("a layer's links must have as many copies as the layer")

    def forward(self, x, pending, batch, cache):
        h, _ = read_streams(self.norm1, x, self.streams, pending, self.link1.read)
        pending = StreamUpdate(self.mixer.forward(h, batch, cache), self.link1)
        if self.feed_forward is not None:
            h, h32 = read_streams(self.norm2, x, self.streams, pending, self.link2.read,
                                  want_f32=self.feed_forward.wants_f32_input)
            pending = StreamUpdate(self.feed_forward.forward(h, h32, batch), self.link2)
        return pending


register_part("arrangement", "hyper_connected", HyperConnectedBlock)
