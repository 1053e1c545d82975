"""Registry of layer parts.  A part is chosen by the `kind` of its PartSpec and built from the
spec's parameters alone; it never learns which model it is in.

Interfaces (duck-typed; `ctx` is the step's StepContext):

  norm      weight_specs(prefix) -> [WeightSpec];  load(prefix, weights);
            forward(ctx, x_f32[T, H], rows=None) -> h[T', H] in the engine's dtype
            (rows: int32 device tensor of the rows to normalise, None = all)
  position  tables(device) -> prepared on first use;  rotary parts expose `cos`, `sin`, `rot_dim`
            for the fused rotate-and-cache kernel; any part may instead offer
            apply(ctx, q[T, heads, hd], k[T, kv_heads, hd]) that rewrites q and k in place
  mixer     weight_specs(prefix); load(prefix, weights); cache_need() -> KVNeed | StateNeed | None;
            forward(ctx, h[T, H], resid_f32[T, H], cache) adds the mixer's output into `resid`;
            `cache` is a KVView, a StateView or None as the need says
            (a mixer built with shares_cache=True writes nothing and reads the view it is given)
  ffn       weight_specs(prefix); load(prefix, weights); forward(ctx, h[T, H], resid_f32[T, H])
            adds its output into `resid`
  hook      weight_specs(prefix); load(prefix, weights); forward(ctx, x_f32) rewrites x in place
            (the model runs one after the embedding and one on the logits when its spec names them)

A block arranges a layer's parts.  `register_block(kind, factory)`; factory(layer_spec, shares_cache)
returns an object with
            parts() -> every part it built (the model asks each whether its steps may be captured);
            mixer (the part whose cache_need() the cache manager reads, or None);
            weight_specs() -> [WeightSpec]; load(weights); forward(ctx, resid_f32[T, H], cache).
`resid` passed to a mixer or ffn need not be the residual stream itself: a block that norms a branch
before it joins the stream hands the part a zeroed float32 buffer and joins it itself.
"""
from __future__ import annotations

from typing import Callable, Dict

from ..config.spec import PartSpec

_FAMILIES = ("norm", "position", "mixer", "ffn", "hook")
_PARTS: Dict[str, Dict[str, Callable]] = {f: {} for f in _FAMILIES}


def register_part(family: str, kind: str, factory: Callable) -> None:
    if family not in _PARTS:
        raise ValueError(f"unknown part family {family!r}; families: {', '.join(_FAMILIES)}")
    _PARTS[family][kind] = factory


def build_part(family: str, spec: PartSpec, **extra):
    kinds = _PARTS[family]
    if spec.kind not in kinds:
        raise KeyError(f"no {family} part named {spec.kind!r}; registered: {', '.join(sorted(kinds)) or '(none)'}")
    return kinds[spec.kind](**spec.params, **extra)


def registered_parts(family: str):
    return sorted(_PARTS[family])


_BLOCKS: Dict[str, Callable] = {}


def register_block(kind: str, factory: Callable) -> None:
    _BLOCKS[kind] = factory


def build_block(layer_spec, shares_cache: bool = False):
    if layer_spec.block not in _BLOCKS:
        raise KeyError(f"no block arrangement named {layer_spec.block!r}; registered: {', '.join(sorted(_BLOCKS)) or '(none)'}")
    return _BLOCKS[layer_spec.block](layer_spec, shares_cache)


def registered_blocks():
    return sorted(_BLOCKS)
