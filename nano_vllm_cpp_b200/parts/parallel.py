"""Several mixers side by side on the same input."""
from __future__ import annotations

from .base import Mixer, CompositeCacheSpec, TensorSpec, PartSpec
from .registry import register_part, build_part


class MixedBranches:
    """What ``SideBySide`` returns instead of one branch: the members' outputs, still to be RMS-normed over the
    model width each with its own weight, summed and scaled.  The norm that follows the mixer does that in its own
    kernel (``Norm.add_normed``)."""

    def __init__(self, branches: list, weights: list, scale: float):
        self.branches, self.weights, self.scale = branches, weights, scale


class SideBySide(Mixer):
    """``members`` (PartSpecs of mixers) all read the same rows; the result is ``scale`` times the sum of their
    outputs, each first RMS-normed over the model width with a weight of its own (``<name>.out`` by default, see
    ``out_names``).  ``names`` are the prefixes of the members' tensors.  Each member keeps its own cache."""

    def __init__(self, hidden_size: int, members: list, names: list, eps: float, scale: float | None = None,
                 out_names: list | None = None):
        if len(members) != len(names) or not 1 <= len(members) <= 4:
            raise ValueError("one name per member, one to four members")
        self.hidden, self.eps = hidden_size, float(eps)
        self.members = [build_part("mixer", m) if isinstance(m, PartSpec) else m for m in members]
        self.names = list(names)
        self.out_names = list(out_names) if out_names else [n + "out" for n in self.names]
        self.scale = 1.0 / len(members) if scale is None else float(scale)

    @property
    def graph_safe(self):
        return all(m.graph_safe for m in self.members)

    def tensor_specs(self, available=None):
        s = {}
        for name, m in zip(self.names, self.members):
            sub = (lambda n, p=name: available(p + n)) if available is not None else None
            for k, ts in m.tensor_specs(sub).items():
                s[name + k] = ts
        for n in self.out_names:
            s[n] = TensorSpec((self.hidden,), init="ones", kind="vector")
        return s

    def load(self, fetch, ctx):
        self.ctx = ctx
        for name, m in zip(self.names, self.members):
            m.load(_Sub(fetch, name), ctx)
        self.out_weights = [fetch(n) for n in self.out_names]

    def cache_spec(self):
        return CompositeCacheSpec(tuple(m.cache_spec() for m in self.members))

    def forward(self, h, batch, cache):
        outs = [m.forward(h, batch, c) for m, c in zip(self.members, cache.parts)]
        return MixedBranches(outs, self.out_weights, self.scale)


class _Sub:
    def __init__(self, fetch, prefix):
        self.fetch, self.prefix = fetch, prefix

    def __call__(self, name):
        return self.fetch(self.prefix + name)

    def has(self, name):
        return self.fetch.has(self.prefix + name)


register_part("mixer", "side_by_side", SideBySide)
