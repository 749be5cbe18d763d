"""Arrangement of a mixer and a feed-forward in one block: pre-norm with residual sums,
``x = x + mixer(norm1(x)); x = x + ffn(norm2(x))`` (tokasaurus/model/llama.py:342-359 with the
norms at :230 and :325 and the sums at :284 and :336).  The sums are carried in the float32
residual stream and are folded into the norm kernel that follows them.

Optionally an input stage (``parts.base.InputStage``, a short convolution for instance) stands between each norm
and the sublayer that reads it, and the feed-forward may be left out (``ffn=None``: the block is its mixer alone).
A stage's per-request state is a cache entry of the layer call, beside the mixer's."""

from __future__ import annotations

import torch

from tokasaurus_b200.kernels import ops
from tokasaurus_b200.parts.base import FeedForward, InputStage, Mixer, Norm, Part, ResidualStream


class PreNormBlock(Part):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm | None, ffn: FeedForward | None,
                 mixer_stage: InputStage | None = None, ffn_stage: InputStage | None = None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a block has a feed-forward and its norm, or neither")
        if ffn is None and ffn_stage is not None:
            raise ValueError("an input stage of the feed-forward needs a feed-forward")
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.ffn_norm = ffn_norm
        self.ffn = ffn
        self.mixer_stage = mixer_stage
        self.ffn_stage = ffn_stage

    def parts(self):
        return tuple(p for p in (self.mixer_norm, self.mixer_stage, self.mixer, self.ffn_norm, self.ffn_stage, self.ffn)
                     if p is not None)

    def weight_specs(self):
        return tuple(s for p in self.parts() for s in p.weight_specs())

    def kernel_modules(self, dtype):
        return tuple(m for p in self.parts() for m in p.kernel_modules(dtype))

    def bind(self, weights, rt) -> None:
        for p in self.parts():
            p.bind(weights, rt)

    def state_needs(self) -> dict:
        """{name: StateNeed} of the input stages: state a layer call holds beside its mixer's cache entry."""
        out = {}
        for name, stage in (("mixer_stage", self.mixer_stage), ("ffn_stage", self.ffn_stage)):
            need = stage.state_need() if stage is not None else None
            if need is not None:
                out[name] = need
        return out

    @staticmethod
    def _staged(ctx, norm, stage, stream, state):
        if stage is None:
            return norm.forward(ctx, stream)
        if hasattr(stage, "forward_with_norm"):
            return stage.forward_with_norm(ctx, norm, stream, state)
        return stage.forward(ctx, norm.forward(ctx, stream), state)

    def forward(self, ctx, stream: ResidualStream, cache, out_rows=None, stage_state=None) -> ResidualStream:
        """``out_rows`` (int32 device tensor or None): only these rows are needed after the block
        (the last block of a step: tokasaurus/model/llama.py:273-278); the stream that comes back
        then has len(out_rows) rows.  ``stage_state``: {name: StateLayerCache} for ``state_needs``."""
        stage_state = stage_state or {}
        h = self._staged(ctx, self.mixer_norm, self.mixer_stage, stream, stage_state.get("mixer_stage"))
        # an input stage of the feed-forward sees every token (its state moves with each), so the rows are cut
        # only after it
        cut_late = self.ffn_stage is not None and out_rows is not None
        if out_rows is not None and not cut_late:
            stream = self._cut(stream, out_rows)
        stream.delta = self.mixer.forward(ctx, h, cache, None if cut_late else out_rows)
        if self.ffn is None:
            return stream
        h = self._staged(ctx, self.ffn_norm, self.ffn_stage, stream, stage_state.get("ffn_stage"))
        if cut_late:
            stream = self._cut(stream, out_rows)
            hc = torch.empty((out_rows.numel(), h.shape[1]), dtype=h.dtype, device=h.device)
            ops.gather_rows(h, out_rows, hc)
            h = hc
        stream.delta = self.ffn.forward(ctx, h)
        return stream

    @staticmethod
    def _cut(stream: ResidualStream, rows) -> ResidualStream:
        x = torch.empty((rows.numel(), stream.x.shape[1]), dtype=stream.x.dtype, device=stream.x.device)
        ops.gather_rows(stream.x, rows, x)
        return ResidualStream(x)


class OutputNormBlock(Part):
    """A block whose sublayers read the residual stream itself and whose norms sit on the sublayers' OUTPUTS:

        x <- x + mult * scale1 * norm1(mixer(x)),      x <- x + mult * scale2 * norm2(ffn(x))

    ``mult`` is a number, ``scale1`` / ``scale2`` optional per-channel vectors (a layer scale; tensor names).  The
    norms are RMS norms (``parts.norm.RMSNorm``: weight and eps).  The stream stays float32; the kernel that adds a
    sublayer's normed output also writes the new stream in the activation type for the sublayer that reads it next; a
    sublayer's output may be the float32 slices of a K-split product (few rows), which that kernel adds.
    A mixer may carry an ``out_bias`` (the bias of its output projection), which is added before the norm."""

    def __init__(self, mixer: Mixer, mixer_norm, ffn: FeedForward | None, ffn_norm, mult: float = 1.0,
                 mixer_scale_name: str | None = None, ffn_scale_name: str | None = None):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a block has a feed-forward and its norm, or neither")
        self.mixer, self.mixer_norm, self.ffn, self.ffn_norm = mixer, mixer_norm, ffn, ffn_norm
        self.mult = float(mult)
        self.scale_names = (mixer_scale_name, ffn_scale_name if ffn is not None else None)
        self.scales: list[torch.Tensor | None] = [None, None]
        self.width = mixer_norm.width
        self.dtype: torch.dtype | None = None

    def parts(self):
        return tuple(p for p in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm) if p is not None)

    def weight_specs(self):
        from tokasaurus_b200.parts.base import WeightSpec
        own = tuple(WeightSpec(n, (self.width,), role="vector") for n in self.scale_names if n is not None)
        return tuple(s for p in self.parts() for s in p.weight_specs()) + own

    def kernel_modules(self, dtype):
        return (("post_norm.cu", None),) + tuple(m for p in self.parts() for m in p.kernel_modules(dtype))

    def bind(self, weights, rt) -> None:
        for p in self.parts():
            p.bind(weights, rt)
        self.scales = [weights[n].contiguous() if n is not None else None for n in self.scale_names]
        self.dtype = rt.dtype

    def state_needs(self) -> dict:
        return {}

    def _input(self, stream: ResidualStream) -> torch.Tensor:
        if self.dtype == torch.float32:
            return stream.x
        if stream.h is None:
            stream.h = torch.empty(stream.x.shape, dtype=self.dtype, device=stream.x.device)
            ops.cast_rows(stream.x, stream.h)
        return stream.h

    def _add(self, stream: ResidualStream, y: torch.Tensor, norm, scale, bias=None) -> None:
        h = None if self.dtype == torch.float32 else torch.empty(stream.x.shape, dtype=self.dtype, device=y.device)
        ops.scaled_norm_add(stream.x, y, norm.weight, scale, self.mult, norm.eps, h, bias)
        stream.h = h

    def forward(self, ctx, stream: ResidualStream, cache, out_rows=None, stage_state=None) -> ResidualStream:
        y = self.mixer.forward(ctx, self._input(stream), cache, out_rows)
        if out_rows is not None:
            stream = PreNormBlock._cut(stream, out_rows)
        self._add(stream, y, self.mixer_norm, self.scales[0], getattr(self.mixer, "out_bias", None))
        if self.ffn is not None:
            self._add(stream, self.ffn.forward(ctx, self._input(stream)), self.ffn_norm, self.scales[1])
        return stream


class PostNormBlock(Part):
    """A block that norms AFTER each residual sum, with the stream scaled on its way into the sum:

        x <- norm1(alpha * x + mixer(x)),      x <- norm2(alpha * x + ffn(x)),      x <- side(x)  (optional)

    The sublayers read x itself.  The norms are ``parts.norm.GroupRMSNorm`` (RMS norm in equal parts of a row, one
    weight vector); ``side`` is a part that adds a per-token input to the stream after the feed-forward
    (``parts.side_input.TokenSideInput``).  The stream stays float32: the kernel that norms a sum writes the new stream
    in both types, a sublayer's output arrives as float32 rows, as the float32 slices of a K-split product (few rows),
    or in the activation type.  A block without a feed-forward has no second sum and no second norm; if it is given a
    second norm all the same (an optional one, whose weight a checkpoint may or may not hold) and the weight is there,
    the second step runs with nothing added: ``x <- norm2(alpha * x)``."""

    def __init__(self, mixer: Mixer, mixer_norm, ffn: FeedForward | None, ffn_norm, alpha: float = 1.0, side=None):
        if ffn is not None and ffn_norm is None:
            raise ValueError("a feed-forward needs its norm")
        self.mixer, self.mixer_norm, self.ffn, self.ffn_norm, self.side = mixer, mixer_norm, ffn, ffn_norm, side
        self.alpha = float(alpha)
        self.dtype: torch.dtype | None = None

    def parts(self):
        return tuple(p for p in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm, self.side) if p is not None)

    def weight_specs(self):
        return tuple(s for p in self.parts() for s in p.weight_specs())

    def kernel_modules(self, dtype):
        return (("post_norm.cu", None),) + tuple(m for p in self.parts() for m in p.kernel_modules(dtype))

    def bind(self, weights, rt) -> None:
        for p in self.parts():
            p.bind(weights, rt)
        self.dtype = rt.dtype

    def state_needs(self) -> dict:
        return {}

    def _input(self, stream: ResidualStream) -> torch.Tensor:
        if self.dtype == torch.float32:
            return stream.x
        if stream.h is None:
            stream.h = torch.empty(stream.x.shape, dtype=self.dtype, device=stream.x.device)
            ops.cast_rows(stream.x, stream.h)
        return stream.h

    def forward(self, ctx, stream: ResidualStream, cache, out_rows=None, stage_state=None) -> ResidualStream:
        y = self.mixer.forward(ctx, self._input(stream), cache, out_rows)
        if out_rows is not None:
            stream = PreNormBlock._cut(stream, out_rows)
        stream.h = self.mixer_norm.apply_sum(stream.x, y, self.alpha)
        if self.ffn is not None:
            stream.h = self.ffn_norm.apply_sum(stream.x, self.ffn.forward(ctx, self._input(stream)), self.alpha)
        elif self.ffn_norm is not None and self.ffn_norm.weight is not None:
            stream.h = self.ffn_norm.apply_sum(stream.x, None, self.alpha)
        if self.side is not None:
            self.side.forward(ctx, stream, self._input(stream), out_rows)
        return stream
