"""Arrangements of parts around the residual stream."""
from __future__ import annotations

from typing import Dict

import torch

from .base import BLOCKS, Block, FeedForward, Mixer, Norm, Part


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x))
    (maeddesg/ROCmForge src/gpu/forward.rs:930-1161; src/cpu/forward.rs:18-337).

    ``names`` maps the four parts to their prefixes inside the layer, as the
    architecture's tensor names have them.  ``ffn`` (with ``norm2``) may be None: the block is then its first half.  A
    mixer made of mixers (``leaf_parts``) brings its leaves' tensors under the joined prefixes.
    """

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm = None, ffn: FeedForward = None, names: Dict[str, str] = None):
        if (ffn is None) != (norm2 is None):
            raise ValueError("prenorm block: ffn and norm2 come together or not at all")
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.names = dict(names)

    def sub_parts(self) -> Dict[str, Part]:
        out = {self.names["norm1"]: self.norm1}
        out.update(_leaves(self.names["mixer"], self.mixer))
        if self.ffn is not None:
            out[self.names["norm2"]] = self.norm2
            out.update(_leaves(self.names["ffn"], self.ffn))
        elif self.names.get("norm2") is not None:
            # a layer without feed-forward: a folder that stores the second norm all the same is not at fault
            import dataclasses
            out[""] = UnusedTensors({self.names["norm2"] + local: dataclasses.replace(spec, optional=True)
                                     for local, spec in self.norm1.param_specs().items()})
        return out

    def entry_norm(self):
        return self.norm1 if self.mixer.accepts_scaled_rows else None

    def forward(self, ctx, stream, cache_view):
        after = stream.after_block                   # the norm that follows this block (the model knows the order)
        y = self.norm1.forward(ctx, stream, deferred_ok=self.mixer.accepts_scaled_rows)
        if self.ffn is None:
            stream.next_norm = after
            self.mixer.forward(ctx, y, cache_view, stream)
            stream.next_norm = None
            return
        # a mixer that adds its result to the stream with a kernel of its own may run the next norm in the same pass
        stream.next_norm = (self.norm2 if self.ffn.accepts_scaled_rows or getattr(self.mixer, "prepares_next_norm", False)
                            else None)
        self.mixer.forward(ctx, y, cache_view, stream)
        y = self.norm2.forward(ctx, stream, deferred_ok=self.ffn.accepts_scaled_rows)
        stream.next_norm = after
        self.ffn.forward(ctx, y, stream)
        stream.next_norm = None


class UnusedTensors(Part):
    """Tensors that a folder may hold although the model does not use them (the norms of a sub-layer that a layer does not
    have): they are accepted and left alone."""

    def __init__(self, specs: Dict[str, "ParamSpec"]):
        self.specs = dict(specs)

    def param_specs(self):
        return self.specs


class ReadsStream(Norm):
    """Stands where a sub-layer has no norm on its way in: the sub-layer reads the stream itself, rounded to the compute
    dtype (on the 32-bit path the stream as it is).  It has no tensors.  Whoever updated the stream last may have left
    the rounded copy in ``stream.prepared``; else one small kernel makes it."""

    def forward(self, ctx, stream, rows=None, deferred_ok=False):
        from .. import kernels
        prepared, stream.prepared = stream.prepared, None
        if rows is not None:
            raise NotImplementedError("a sub-layer that reads the stream itself reads all of its rows")
        if prepared is not None and prepared[0] is self and stream.pending is None:
            return prepared[1]
        stream.flush()
        return stream.h if ctx.compute_dtype == torch.float32 else kernels.round_rows(stream.h, ctx.compute_dtype)

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]


READS_STREAM = ReadsStream()     # one for all: a block that prepares the next block's input finds it by identity


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """x += post1(mixer(norm1(x))); x += post2(ffn(norm2(x))): every sub-layer is normed on its way in and on its way
    out.  ``ffn`` (with norm2 and post2) may be None: the block is then its first half.  ``norm1`` / ``norm2`` None: that
    sub-layer has a norm on its way out only and reads the stream itself, x += post(sub-layer(x)).

    The outputs of the sub-layers, their norms and the sums are 32-bit.  One kernel per sub-layer forms the mixer's
    merge (if it hands out a ``NormedMean``), the out-norm, the sum into the stream, a row vector that the schedule
    adds after the block (``stream.after_extra``) and the norm that reads the stream next, which therefore never
    launches on its own.
    """

    def __init__(self, norm1: Norm, mixer: Mixer, post1: Norm, norm2: Norm = None, ffn: FeedForward = None,
                 post2: Norm = None, names: Dict[str, str] = None):
        if (ffn is None) != (post2 is None) or (ffn is None and norm2 is not None):
            raise ValueError("sandwich block: ffn and post2 come together or not at all, norm2 only with them")
        self.norm1, self.mixer, self.post1 = norm1 if norm1 is not None else READS_STREAM, mixer, post1
        self.norm2 = (norm2 if norm2 is not None else READS_STREAM) if ffn is not None else None
        self.ffn, self.post2 = ffn, post2
        self.names = dict(names)

    def sub_parts(self) -> Dict[str, Part]:
        out = {self.names["post1"]: self.post1}
        if self.norm1 is not READS_STREAM:
            out[self.names["norm1"]] = self.norm1
        if hasattr(self.mixer, "leaf_parts"):                # a mixer made of mixers: its halves have prefixes of their own
            for sub, part in self.mixer.leaf_parts().items():
                out[self.names["mixer"] + sub] = part
        else:
            out[self.names["mixer"]] = self.mixer
        if self.ffn is not None:
            out.update({self.names["ffn"]: self.ffn, self.names["post2"]: self.post2})
            if self.norm2 is not READS_STREAM:
                out[self.names["norm2"]] = self.norm2
        else:
            # a layer without feed-forward: a folder that stores the second sub-layer's norms all the same is not at fault
            from ..weights.spec import ParamSpec
            unused = [n for n in ("norm2", "post2") if self.names.get(n) is not None]
            if unused:
                out[""] = UnusedTensors({self.names[n] + self.post1.param_name:
                                         ParamSpec((self.post1.size,), kind="vector", init="ones", optional=True) for n in unused})
        return out

    def entry_norm(self):
        return self.norm1

    @staticmethod
    def _add(ctx, stream, result, post, next_norm, extra):
        """stream += post(result) (+ extra); leaves ``next_norm`` of the new stream prepared if it is a plain RMS norm
        of the same eps."""
        from .. import kernels
        from .base import NormedMean
        weight, eps = post.deferred_params()
        if isinstance(result, NormedMean):
            if result.eps != eps:
                raise NotImplementedError("sandwich block: the merge and the out-norm must share eps")
            branches = result.branches
        else:
            branches = [(result, None)]
        nxt = next_norm.deferred_params() if next_norm is not None else None
        if nxt is not None and nxt[1] != eps:
            nxt = None
        stream.flush()
        stream.prepared = None
        y = kernels.branch_norm_add(stream.h, branches, weight, eps, ctx.compute_dtype, extra=extra,
                                    next_weight=nxt[0] if nxt is not None else None,
                                    next_rounded=next_norm is READS_STREAM and ctx.compute_dtype != torch.float32)
        if y is not None:
            stream.prepared = (next_norm, y)

    def forward(self, ctx, stream, cache_view):
        after, extra = stream.after_block, stream.after_extra
        stream.after_extra = None                    # added here, with the block's last update
        stream.next_norm = None
        y = self.norm1.forward(ctx, stream)
        r = self.mixer.output(ctx, y, cache_view)
        if self.ffn is None:
            self._add(ctx, stream, r, self.post1, after, extra)
            return
        self._add(ctx, stream, r, self.post1, self.norm2, None)
        y = self.norm2.forward(ctx, stream)
        self._add(ctx, stream, self.ffn.output(ctx, y), self.post2, after, extra)


def _leaves(prefix: str, part) -> Dict[str, Part]:
    """{prefix: part}, or for a part made of parts (``leaf_parts``) its leaves under the joined prefixes."""
    if hasattr(part, "leaf_parts"):
        out: Dict[str, Part] = {}
        for sub, leaf in part.leaf_parts().items():
            out.update(_leaves(prefix + sub, leaf))
        return out
    return {prefix: part}


@BLOCKS.register("scaled_prenorm")
class ScaledPreNormBlock(Block):
    """x += mult * mixer(norm1(x)); x += mult * ffn(norm2(x)), with one number ``mult`` for all sub-layers.  ``ffn`` (with
    ``norm2``) may be None.

    The sub-layers hand out their results in 32-bit (``output``: a tensor, a stack of partial sums, a ``NormedMean`` of
    two mixers side by side, a ``SumOf``), and one kernel per sub-layer (``kernels.scaled_add``) forms the merge or the
    sum, scales, adds into the 32-bit stream and, where the norm that reads the stream next is a Dynamic Tanh, computes
    it in the same pass, so that norm never launches on its own (the first layer's and the final one apart).
    """

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm = None, ffn: FeedForward = None, *, mult: float = 1.0,
                 names: Dict[str, str] = None):
        if (ffn is None) != (norm2 is None):
            raise ValueError("scaled_prenorm block: ffn and norm2 come together or not at all")
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self.mult = float(mult)
        self.names = dict(names)

    def sub_parts(self) -> Dict[str, Part]:
        out = {self.names["norm1"]: self.norm1}
        out.update(_leaves(self.names["mixer"], self.mixer))
        if self.ffn is not None:
            out[self.names["norm2"]] = self.norm2
            out.update(_leaves(self.names["ffn"], self.ffn))
        elif self.names.get("norm2") is not None:
            # a layer without feed-forward: a folder that stores the second norm all the same is not at fault
            from ..weights.spec import ParamSpec
            import dataclasses
            out[""] = UnusedTensors({self.names["norm2"] + local: dataclasses.replace(spec, optional=True)
                                     for local, spec in self.norm1.param_specs().items()})
        return out

    def entry_norm(self):
        return self.norm1

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]

    def _add(self, ctx, stream, result, next_norm):
        from .. import kernels
        from .base import NormedMean, SumOf
        eps = 0.0
        if isinstance(result, NormedMean):
            addends, eps = result.branches, result.eps
        elif isinstance(result, SumOf):
            addends = [(a, None) for a in result.addends]
        else:
            addends = [(result, None)]
        nxt = next_norm.dyt_params() if next_norm is not None and hasattr(next_norm, "dyt_params") else None
        stream.flush()
        stream.prepared = None
        y = kernels.scaled_add(stream.h, addends, self.mult, ctx.compute_dtype, eps=eps, next_dyt=nxt)
        if y is not None:
            stream.prepared = (next_norm, y)

    def forward(self, ctx, stream, cache_view):
        after = stream.after_block
        stream.next_norm = None
        y = self.norm1.forward(ctx, stream)
        r = self.mixer.output(ctx, y, cache_view)
        if self.ffn is None:
            self._add(ctx, stream, r, after)
            return
        self._add(ctx, stream, r, self.norm2)
        y = self.norm2.forward(ctx, stream)
        self._add(ctx, stream, self.ffn.output(ctx, y), after)
