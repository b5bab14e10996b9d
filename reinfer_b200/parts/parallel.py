"""Several mixers side by side on the same input: result = sum_i scale_i * branch_i(h).

Each branch is a mixer of any registered kind that takes an `out_scale` parameter; it gets the
tensors under `<name>.`, its own part of the layer's state (`cache.state[name]`) and - the one
branch that has a paged cache - the layer's pages.  Every branch adds into the residual stream
through its own output projection; only the last may leave its sum to the norm that reads the
stream next.
"""
from __future__ import annotations

from typing import Mapping, Sequence

from .base import Mixer, build_part, register_part
from .context import LayerCache
from .spec import PartSpec


class ParallelMixer(Mixer):
    def __init__(self, branches: Sequence[Mapping]):
        """branches: [{"name": tensor-name prefix, "kind": mixer kind, "params": {...}, "scale": s}, ...]"""
        self.names, self.subs = [], []
        for b in branches:
            params = dict(b["params"])
            params["out_scale"] = float(b.get("scale", 1.0)) * float(params.get("out_scale", 1.0))
            self.names.append(str(b["name"]))
            self.subs.append(build_part("mixer", PartSpec(b["kind"], params)))
        if len(set(self.names)) != len(self.names) or not self.subs:
            raise ValueError("parallel mixer: branches need names of their own")
        if sum(1 for s in self.subs if s.cache_spec() is not None) > 1:
            raise ValueError("parallel mixer: at most one branch may keep keys and values in pages")

    @property
    def steps_from_device_tables(self):
        return all(getattr(s, "steps_from_device_tables", False) or s.state_spec() is None for s in self.subs)

    def param_specs(self):
        return {f"{n}.{local}": ps for n, s in zip(self.names, self.subs) for local, ps in s.param_specs().items()}

    def bind(self, tensors):
        for n, s in zip(self.names, self.subs):
            pre = n + "."
            s.bind({k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)})

    def prepare(self, device, dtype):
        for s in self.subs:
            s.prepare(device, dtype)

    def cache_spec(self):
        return next((s.cache_spec() for s in self.subs if s.cache_spec() is not None), None)

    def state_spec(self):
        out = {n: s.state_spec() for n, s in zip(self.names, self.subs) if s.state_spec() is not None}
        return out or None

    def forward(self, ctx, xn, residual, cache):
        last = len(self.subs) - 1
        ahead, defer = ctx.norm_ahead, ctx.defer_residual
        left = None
        for i, (n, s) in enumerate(zip(self.names, self.subs)):
            paged = s.cache_spec() is not None
            sub = LayerCache(kv=cache.kv if paged else None, group=cache.group if paged else None, write=cache.write,
                             state=cache.state.get(n) if isinstance(cache.state, dict) else None)
            if i < last:
                ctx.norm_ahead, ctx.defer_residual = None, False
            else:
                ctx.norm_ahead, ctx.defer_residual = ahead, defer
            left = s.forward(ctx, xn, residual, sub)
        return left


register_part("mixer", "parallel", ParallelMixer)
