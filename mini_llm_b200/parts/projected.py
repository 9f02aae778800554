"""Mixers of the form out = W_out core(W_in h), and several of them side by side.

A ``ProjectedMixer`` names the matrices whose rows make up its input projection
(``in_matrices``), a ``core`` that turns the projected columns into the input of
its output projection, and that output matrix.  Alone it runs as any mixer:
one product in, the core, one product out that adds into the residual.

``ParallelMixer`` runs several of them on the same input and adds their
results with fixed factors: out = sum_b scale_b * W_out_b core_b(W_in_b h).
Because every branch has this form, the branches' input matrices are stacked
into ONE matrix when the weights are bound and their output matrices are
joined along the contraction dimension: the whole mixer is one product in, the
cores (each reads its columns of the projection and writes its columns,
already multiplied by its factor, of one buffer) and one product out whose
epilogue adds into the 32-bit residual.
"""
from __future__ import annotations

from typing import Any, Dict, List, Sequence

import torch

from .base import Mixer, get_part_factory, register_part


class ProjectedMixer(Mixer):
    accepts_lazy_norm = True            # the first thing done with the input is a product
    can_overwrite = True                # forward(..., accumulate=False) writes the result instead of adding it
    in_names: Sequence[str] = ()        # parameters stacked (by rows) into the input projection, in this order
    out_name: str = "out_weight"        # the output projection [hidden, core_width]
    in_bias = None                      # a bias on the input projection (float32 [in_width]), set at bind by a mixer that has one

    @property
    def in_width(self) -> int:
        specs = self.param_specs()
        return sum(specs[n].shape[0] for n in self.in_names)

    @property
    def core_width(self) -> int:
        return self.param_specs()[self.out_name].shape[1]

    def core(self, proj, ctx, cache, out, out_scale: float = 1.0) -> None:  # pragma: no cover
        """proj [T, in_width] (columns in the order of in_names) -> out [T, core_width], times out_scale."""
        raise NotImplementedError

    def bind(self, params: Dict[str, Any], rt) -> None:
        super().bind(params, rt)
        if all(n in params for n in self.in_names) and self.in_names:
            self.in_weight = torch.cat([params[n] for n in self.in_names], 0).contiguous()

    def forward(self, h, ctx, cache, out_accum, accumulate: bool = True):
        ops = self.rt.ops
        T = h.shape[0]
        n_in = self.in_weight.shape[0]
        proj = ctx.ws.buf("mix_proj", T, -(-n_in // 8) * 8, self.rt.act_dtype)[:, :n_in]    # rows stay 16-byte aligned
        ops.linear(h, self.in_weight, self.in_bias, out=proj)
        mid = ctx.ws.buf("mix_core", T, self.core_width, self.rt.act_dtype)
        self.core(proj, ctx, cache, mid)
        ops.linear(mid, getattr(self, self.out_name), None, out=out_accum, accumulate=accumulate)


class ParallelMixer(Mixer):
    """``branches``: a list of {"name", "kind", "params"} (kind: a registered ProjectedMixer);
    ``scales``: the factor on each branch's result.  Parameters are named "<branch name>.<local name>"."""

    accepts_lazy_norm = True

    def __init__(self, branches: List[Dict[str, Any]], scales: Sequence[float]):
        if len(branches) != len(scales) or not branches:
            raise ValueError("ParallelMixer: one scale per branch, at least one branch")
        self.names = [b["name"] for b in branches]
        self.branches: List[ProjectedMixer] = []
        for b in branches:
            part = get_part_factory("mixer", b["kind"])(**b["params"])
            if not isinstance(part, ProjectedMixer):
                raise ValueError(f"ParallelMixer: branch {b['name']!r} ({b['kind']}) is not a ProjectedMixer")
            self.branches.append(part)
        self.scales = [float(s) for s in scales]

    def param_specs(self):
        return {f"{n}.{k}": v for n, b in zip(self.names, self.branches) for k, v in b.param_specs().items()}

    def kernel_limits(self, dtype: str):
        return [m for b in self.branches for m in b.kernel_limits(dtype)]

    def set_positions(self, positions) -> None:
        self.positions = positions
        for b in self.branches:
            b.set_positions(positions)

    def cache_need(self):
        needs = [b.cache_need() for b in self.branches]
        needs = [n for n in needs if n is not None]
        return needs if needs else None

    def bind(self, params: Dict[str, Any], rt) -> None:
        self.rt = rt
        for n, b in zip(self.names, self.branches):
            b.bind({k[len(n) + 1:]: v for k, v in params.items() if k.startswith(n + ".")}, rt)
        if params:
            self.in_weight = torch.cat([b.in_weight for b in self.branches], 0).contiguous()
            self.out_weight = torch.cat([getattr(b, b.out_name) for b in self.branches], 1).contiguous()
            # the branches keep views of the joined matrices, not copies of their own
            r = c = 0
            for b in self.branches:
                b.in_weight = self.in_weight[r:r + b.in_width]
                for n in b.in_names:
                    rows = getattr(b, n).shape[0]
                    setattr(b, n, self.in_weight[r:r + rows])
                    r += rows
                setattr(b, b.out_name, self.out_weight[:, c:c + b.core_width])
                c += b.core_width

    def forward(self, h, ctx, cache, out_accum):
        ops = self.rt.ops
        T = h.shape[0]
        n_in = self.in_weight.shape[0]
        proj = ctx.ws.buf("mix_proj", T, -(-n_in // 8) * 8, self.rt.act_dtype)[:, :n_in]    # rows stay 16-byte aligned
        ops.linear(h, self.in_weight, None, out=proj)
        mid = ctx.ws.buf("mix_core", T, self.out_weight.shape[1], self.rt.act_dtype)
        r = c = 0
        for b, s in zip(self.branches, self.scales):
            b.core(proj[:, r:r + b.in_width], ctx, cache, mid[:, c:c + b.core_width], out_scale=s)
            r += b.in_width
            c += b.core_width
        ops.linear(mid, self.out_weight, None, out=out_accum, accumulate=True)


register_part("mixer", "parallel", ParallelMixer)
