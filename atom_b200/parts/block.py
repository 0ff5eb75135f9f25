"""Arrangements of a layer's parts around the residual stream.

An arrangement declares the parts it is put together from: ``slots`` maps each part's name in
the layer to its category in the registries (the model builds exactly these from the layer's
spec and hands them to the constructor by name); names listed in ``optional`` may be left out
of a layer.  The part named ``mixer``, if there is one, is the one whose cache the run entry's
cache slot holds.

"prenorm" is the one of atom/models/qwen3.py:248-258: the residual is a running 32-bit
sum; each sub-block's output is added to it inside the next norm's kernel:
   r += delta;  a = norm1(r);  m = mixer(a);  r += m;  b = norm2(r);  delta' = ffn(b).

Between parts that say they can, an output travels as a product still to run and normalised rows
as ``ScaledRows`` (parts/linear.py), so that in a step of few rows the norms need no kernel of their
own; a part that says nothing gets and gives plain tensors.
"""
from __future__ import annotations

from .linear import resolve
from .registry import register


def _add_norm(norm, residual, delta, tag, receiver):
    if getattr(norm, "fuses_products", False):
        return norm.add_norm(residual, delta, tag, scaled_ok=getattr(receiver, "takes_scaled_rows", False))
    return norm.add_norm(residual, resolve(delta), tag)


def _forward(part, *args):
    if getattr(part, "defers_output", False):
        return part.forward(*args, defer=True)
    return part.forward(*args)


@register("arrangement", "prenorm")
class PreNormBlock:
    slots = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "ffn"}
    optional = ()
    takes_pending = True      # delta may be a PendingProduct, and so may what run() returns

    def __init__(self, mixer_norm, mixer, ffn_norm, ffn):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def run(self, residual, delta, step, cache, writes_cache):
        """residual: [T, hidden] float32, updated in place.  delta: the previous block's output
        (None for the first).  Returns this block's output, to be added by the next norm."""
        a = _add_norm(self.mixer_norm, residual, delta, "norm.mixer", self.mixer)
        m = _forward(self.mixer, a, step, cache, writes_cache)
        b = _add_norm(self.ffn_norm, residual, m, "norm.ffn", self.ffn)
        return _forward(self.ffn, b, step)
