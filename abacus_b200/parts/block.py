"""A layer: two norms, a mixer and a feed-forward, wired as src/model.c:292-310.

pre_norm:  x += y;  xn = norm1(x);  y = mixer(xn);  x += y;  xn = norm2(x);  y = ffn(xn)
The last y is handed on and added by whoever norms next (the next block or the
final norm), as abacus's add_norm does (src/model.c:297, 311).
"""
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS


@BLOCKS.register("pre_norm")
class PreNormBlock:
    def __init__(self, spec):
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.mixer_norm)
        self.mixer = MIXERS.build(spec.mixer)
        self.ffn_norm = NORMS.build(spec.ffn_norm)
        self.ffn = FEED_FORWARDS.build(spec.ffn)

    def parts(self):
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    def bind(self, params, ctx):
        """params: {part name: {slot: tensor}}."""
        self.ctx = ctx
        for name, part in self.parts().items():
            part.bind(params[name], ctx)

    def forward(self, x, y, batch, cache, ws):
        n, d = batch.n_rows, x.shape[1]
        xn = ws.get("xn", (n, d), self.ctx.dtype)
        out = ws.get("branch", (n, d), x.dtype)
        self.mixer_norm.forward(x, y, xn, n_rows=n)
        self.mixer.forward(xn, out, batch, cache, ws)
        self.ffn_norm.forward(x, out, xn, n_rows=n)
        self.ffn.forward(xn, out, batch, ws)
        return out
