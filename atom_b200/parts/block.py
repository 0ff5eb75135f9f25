"""Arrangements of a layer's parts around the residual stream.

An arrangement declares the parts it is put together from: ``slots`` maps each part's name in
the layer to its category in the registries (the model builds exactly these from the layer's
spec and hands them to the constructor by name); names listed in ``optional`` may be left out
of a layer.  The part named ``mixer``, if there is one, is the one whose cache the run entry's
cache slot holds.

"prenorm" is the one of atom/models/qwen3.py:248-258: the residual is a running 32-bit
sum; each sub-block's output is added to it inside the next norm's kernel:
   r += delta;  a = norm1(r);  m = mixer(a);  r += m;  b = norm2(r);  delta' = ffn(b).
"""
from __future__ import annotations

from .registry import register


@register("arrangement", "prenorm")
class PreNormBlock:
    slots = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "ffn"}
    optional = ()

    def __init__(self, mixer_norm, mixer, ffn_norm, ffn):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def run(self, residual, delta, step, cache, writes_cache):
        """residual: [T, hidden] float32, updated in place.  delta: the previous block's output
        (None for the first).  Returns this block's output, to be added by the next norm."""
        a = self.mixer_norm.add_norm(residual, delta, "norm.mixer")
        m = self.mixer.forward(a, step, cache, writes_cache)
        b = self.ffn_norm.add_norm(residual, m, "norm.ffn")
        return self.ffn.forward(b, step)
