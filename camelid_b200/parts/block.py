"""Arrangements of a layer's parts. ``prenorm`` is the reference's decoder layer
(src/inference.rs:6228-6804): r = x + mixer(norm1(x)); out = r + ffn(norm2(r)). The
residual stream stays float32; mixer and feed-forward add into it in place."""
from __future__ import annotations

from .base import Part, build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Part):
    def __init__(self, layer_spec):
        super().__init__({}, "")
        self.norm1 = build_part("norm", layer_spec.norm1)
        self.shift = build_part("shift", layer_spec.shift) if layer_spec.shift is not None else None
        self.mixer = build_part("mixer", layer_spec.mixer)
        # a layer without a feed-forward has only the first sublayer
        self.ffn = build_part("ffn", layer_spec.ffn) if layer_spec.ffn is not None else None
        self.norm2 = build_part("norm", layer_spec.norm2) if self.ffn is not None else None

    def parts(self):
        return tuple(p for p in (self.norm1, self.shift, self.mixer, self.norm2, self.ffn) if p is not None)

    def tensor_specs(self):
        out = {}
        for p in self.parts():
            out.update(p.tensor_specs())
        return out

    def load(self, tensors, device, dtype):
        for p in self.parts():
            p.load(tensors, device, dtype)

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts())

    @property
    def graph_safe_any_step(self):
        return all(p.graph_safe_any_step for p in self.parts())

    def cache_spec(self):
        if self.shift is None:
            return self.mixer.cache_spec()
        return [self.mixer.cache_spec(), self.shift.cache_spec()]

    def query_tile_sizes(self):
        return self.mixer.query_tile_sizes()

    def forward(self, ctx, h):
        # A built-in mixer or feed-forward may leave split sums pending on the context (or a
        # product deferred); the norm that reads the stream next adds them. Before any part that
        # does not declare ``handles_pending`` the block settles the stream itself, so a part
        # from outside the library, graph safe or not, reads and writes complete rows.
        # A part that declares ``accepts_row_scale`` takes ``ctx.take_row_scale()`` and applies
        # it, which lets the norm before it run inside the product before that.
        # A shift part between the first norm and the mixer reads complete rows (no scale left undone).
        ctx.rows_copy = None                # this arrangement adds into the stream without keeping its rows in the compute type
        for norm, part in ((self.norm1, self.mixer), (self.norm2, self.ffn)):
            if part is None:
                continue
            shift = self.shift if part is self.mixer else None
            if not norm.handles_pending:
                ctx.settle(h)
            x = shift.norm_and_shift(ctx, h, norm) if shift is not None and hasattr(shift, "norm_and_shift") else None
            if x is None:
                x = norm.forward(ctx, h, allow_row_scale=part.accepts_row_scale and shift is None)
                if shift is not None:
                    x = shift.forward(ctx, x)
            if not part.handles_pending:
                ctx.settle(h)
            part.forward(ctx, x, h)


@register_part("block", "sandwich")
class SandwichBlock(Part):
    """Norms before and after every sublayer: x += s * post_norm1(mixer(norm1(x))), then
    x += s * post_norm2(ffn(norm2(x))), s one number of the layer. The sublayers hand their output over as
    float32 rows (or split sums) instead of adding it into the stream: the mixer by ``branch_output(ctx, x,
    name)``, the feed-forward by ``output(ctx, x, name) -> (y, bias or None)``; the norm after them adds
    (``add_normed``). A layer without a feed-forward has only the first sublayer."""

    def __init__(self, layer_spec):
        super().__init__({}, "")
        from ..errors import ConfigError
        if layer_spec.post_norm1 is None or (layer_spec.ffn is not None and layer_spec.post_norm2 is None):
            raise ConfigError("block.arrangement", "the sandwich arrangement needs post_norm1 (and post_norm2 with a feed-forward)")
        self.scale = float(layer_spec.residual_scale)
        self.norm1 = build_part("norm", layer_spec.norm1)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.post1 = build_part("norm", layer_spec.post_norm1)
        self.ffn = build_part("ffn", layer_spec.ffn) if layer_spec.ffn is not None else None
        self.norm2 = build_part("norm", layer_spec.norm2) if self.ffn is not None else None
        self.post2 = build_part("norm", layer_spec.post_norm2) if self.ffn is not None else None
        if not hasattr(self.mixer, "branch_output"):
            raise ConfigError("mixer.kind", f"the mixer {self.mixer.kind!r} does not hand its output over (branch_output)")
        if self.ffn is not None and not hasattr(self.ffn, "output"):
            raise ConfigError("ffn.kind", f"the feed-forward {self.ffn.kind!r} does not hand its output over (output)")
        for n in (self.post1, self.post2):
            if n is not None and not hasattr(n, "add_normed"):
                raise ConfigError("norm.kind", f"the norm {n.kind!r} cannot stand behind a sublayer (add_normed)")

    def parts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.post1, self.norm2, self.ffn, self.post2) if p is not None)

    def tensor_specs(self):
        out = {}
        for p in self.parts():
            out.update(p.tensor_specs())
        return out

    def load(self, tensors, device, dtype):
        for p in self.parts():
            p.load(tensors, device, dtype)

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts())

    @property
    def graph_safe_any_step(self):
        return all(p.graph_safe_any_step for p in self.parts())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def query_tile_sizes(self):
        return self.mixer.query_tile_sizes()

    def forward(self, ctx, h):
        ctx.settle(h)                       # whatever a layer of another arrangement left undone
        ctx.rows_copy = None
        x = self.norm1.forward(ctx, h)
        # the norm behind the mixer and the one before the feed-forward share a pass over the rows where they can
        x = self.post1.add_normed(ctx, self.mixer.branch_output(ctx, x, "mixer_out"), h, self.scale, None, then=self.norm2)
        if self.ffn is not None:
            if x is None:
                x = self.norm2.forward(ctx, h)
            y, bias = self.ffn.output(ctx, x, "ffn_out")
            self.post2.add_normed(ctx, y, h, self.scale, bias)


@register_part("block", "postnorm")
class PostNormBlock(Part):
    """The norm after the sum, on the stream itself: x <- norm1(a x + mixer(x)), then x <- norm2(a x + ffn(x)), a one
    number of the layer (``residual_scale``). The sublayers read x as it is (in the compute type: ``ctx.stream_rows``)
    and hand their output over as float32 rows or split sums (``branch_output`` of a mixer, ``output`` of a feed-forward);
    the norm adds and norms in one pass over the row (``sum_normed``) and leaves the new rows in the compute type for the
    next reader. A layer without a feed-forward has only the first sublayer. ``after``: a part that runs at the end of
    the layer (a per-layer token input)."""

    def __init__(self, layer_spec):
        super().__init__({}, "")
        from ..errors import ConfigError
        self.alpha = float(layer_spec.residual_scale)
        self.norm1 = build_part("norm", layer_spec.norm1)
        self.mixer = build_part("mixer", layer_spec.mixer)
        self.ffn = build_part("ffn", layer_spec.ffn) if layer_spec.ffn is not None else None
        self.norm2 = build_part("norm", layer_spec.norm2) if self.ffn is not None else None
        self.after = build_part("layer_input", layer_spec.after) if layer_spec.after is not None else None
        if self.ffn is not None and layer_spec.norm2 is None:
            raise ConfigError("block.arrangement", "the postnorm arrangement needs norm2 with a feed-forward")
        if not hasattr(self.mixer, "branch_output"):
            raise ConfigError("mixer.kind", f"the mixer {self.mixer.kind!r} does not hand its output over (branch_output)")
        if self.ffn is not None and not hasattr(self.ffn, "output"):
            raise ConfigError("ffn.kind", f"the feed-forward {self.ffn.kind!r} does not hand its output over (output)")
        for n in (self.norm1, self.norm2):
            if n is not None and not hasattr(n, "sum_normed"):
                raise ConfigError("norm.kind", f"the norm {n.kind!r} cannot norm a residual sum in place (sum_normed)")

    def parts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm2, self.ffn, self.after) if p is not None)

    def tensor_specs(self):
        out = {}
        for p in self.parts():
            out.update(p.tensor_specs())
        return out

    def load(self, tensors, device, dtype):
        for p in self.parts():
            p.load(tensors, device, dtype)

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts())

    @property
    def graph_safe_any_step(self):
        return all(p.graph_safe_any_step for p in self.parts())

    def cache_spec(self):
        return self.mixer.cache_spec()

    def query_tile_sizes(self):
        return self.mixer.query_tile_sizes()

    def forward(self, ctx, h):
        ctx.settle(h)                       # whatever a layer of another arrangement left undone
        x = ctx.stream_rows(h)
        x = self.norm1.sum_normed(ctx, self.mixer.branch_output(ctx, x, "mixer_out"), h, self.alpha)
        if self.ffn is not None:
            # a feed-forward whose experts may be the identity wants the stream's own float rows for those
            y, bias = self.ffn.output(ctx, x, "ffn_out", stream=h) if getattr(self.ffn, "takes_stream", False) \
                else self.ffn.output(ctx, x, "ffn_out")
            x = self.norm2.sum_normed(ctx, y, h, self.alpha, bias)
        if self.after is not None:
            self.after.forward(ctx, x, h)
