"""Plain, slow restatement of the Kedasun decoder, one function per mechanism, for the tests.

Kedasun is a decoder-only model given as a list of layers.  A layer wraps each of its two sublayers
in a norm before and a norm after:

    h <- h + n1b(mixer(n1(h)));   h <- h + n2b(ff(n2(h)))

n(x): the vector is cut into `groups` equal consecutive pieces, every piece is divided by its own
sqrt(mean(piece^2) + eps), and the whole is multiplied by a gain.  The embedding is multiplied by a
constant; the logits are head . n_final(h).

Two mixers:

* "attention": grouped-query softmax attention, no biases, rotary positions on interleaved pairs
  of the first `rot.dims` entries of every query and key head, a configured score scale.
* "attention_2": biased projections; a short causal convolution over time on every channel of q, k
  and v right after the projection; q and k heads divided by their root mean square (no gain); a
  per-head linear penalty on the distance slope_a * (i - j), slope_a = 2^(-8 (a + 1) / heads);
  a sliding window that also keeps the first tokens of the sequence; after the softmax the heads'
  weights are mixed by a heads x heads matrix; every head's output is multiplied by a sigmoid gate
  computed from the mixer's input; biased output projection.

Both may take part in *value mixing*: every layer that says so, except the first one that does,
blends its values with the values the first one computed for the same token,
v <- (1 - lam) v + lam v_first, and stores the blend.

Feed-forward: g = min(W_g x, limit), u = clamp(W_u x, -limit, limit), y = g sigmoid(1.702 g) (u + 1),
out = W_d y.

Nothing here shares code with the engine.  Tensors go in as a dict of torch tensors under the
checkpoint's names; every function is written for clarity, not speed.  `forward` runs a whole
sequence at once; `Stepper` runs it token by token from explicit state (cached keys and values, the
last projected values the convolutions need), so that the two can be compared.
"""
from __future__ import annotations

import torch

GATE_SHARPNESS = 1.702      # y = g * sigmoid(GATE_SHARPNESS * g) * (u + 1)
SLOPE_EXPONENT = 8.0        # slope of head a: 2^(-SLOPE_EXPONENT * (a + 1) / heads)


def grouped_rms_norm(x: torch.Tensor, gain: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """x [..., W]; W = groups * piece."""
    shape = x.shape
    p = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    return p.reshape(shape) * gain


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, no gain."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate_pairs(v: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """v [T, heads, D], pos [T]: (v[2i], v[2i+1]) turns by pos * base^(-2i/dims), i < dims/2; the rest passes."""
    out = v.clone()
    i = torch.arange(dims // 2, dtype=v.dtype)
    freq = torch.as_tensor(base, dtype=v.dtype) ** (-2.0 * i / dims)
    ang = pos.to(v.dtype)[:, None, None] * freq[None, None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def causal_short_conv(u: torch.Tensor, taps_w: torch.Tensor, before: torch.Tensor | None = None) -> torch.Tensor:
    """u [T, C]; taps_w [C, taps]: y_t = sum_j taps_w[:, j] * u_(t - taps + 1 + j).  `before` [taps - 1, C] holds the
    values that precede u (zeros when the sequence starts here)."""
    T, C = u.shape
    taps = taps_w.shape[1]
    if before is None:
        before = torch.zeros(taps - 1, C, dtype=u.dtype)
    ext = torch.cat([before, u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + taps_w[:, j][None, :] * ext[j:j + T]
    return y


def head_slopes(heads: int, dtype) -> torch.Tensor:
    return torch.tensor([2.0 ** (-SLOPE_EXPONENT * (a + 1) / heads) for a in range(heads)], dtype=dtype)


def visible(qpos: torch.Tensor, kpos: torch.Tensor, window: int | None, keep_first: int) -> torch.Tensor:
    """[Tq, Tk] bool: key j is seen from query i when j <= i and (no window, or i - j < window, or j < keep_first)."""
    i, j = qpos[:, None], kpos[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def softmax_weights(scores: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """scores [heads, Tq, Tk]; masked keys get weight exactly zero."""
    s = scores.masked_fill(~mask[None], float("-inf"))
    return torch.softmax(s, -1)


def attend(q, k, v, qpos, kpos, scale, *, slopes=None, window=None, keep_first=0, talk=None):
    """q [Tq, H, D], k [Tk, G, D], v [Tk, G, Dv] -> [Tq, H, Dv].  Query head a reads key/value head a // (H / G).
    slopes [H]: slope_a * (i - j) is subtracted from the scores.  talk [H, H]: the softmax weights of the heads are mixed,
    w'_a = sum_b talk[a, b] w_b, and head a applies w'_a to the values of its own key/value head."""
    H, G = q.shape[1], k.shape[1]
    rep = H // G
    kk = k.repeat_interleave(rep, 1)
    vv = v.repeat_interleave(rep, 1)
    s = torch.einsum("iad,jad->aij", q, kk) * scale
    if slopes is not None:
        s = s - slopes[:, None, None] * (qpos[:, None] - kpos[None, :]).to(q.dtype)[None]
    w = softmax_weights(s, visible(qpos, kpos, window, keep_first))
    if talk is not None:
        w = torch.einsum("ab,bij->aij", talk, w)
    return torch.einsum("aij,jad->iad", w, vv)


def blend_values(v: torch.Tensor, v_first: torch.Tensor, lam: torch.Tensor) -> torch.Tensor:
    return (1.0 - lam) * v + lam * v_first


def clamped_gated_ff(x: torch.Tensor, w: dict, pre: str, limit: float) -> torch.Tensor:
    g = torch.clamp(x @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(x @ w[pre + "up"].T, min=-limit, max=limit)
    y = g * torch.sigmoid(GATE_SHARPNESS * g) * (u + 1.0)
    return y @ w[pre + "down"].T


def first_value_layer(cfg: dict) -> int:
    for i, L in enumerate(cfg["layers"]):
        if L["mixer"].get("v_mix"):
            return i
    return -1


class Stepper:
    """Token-by-token evaluation from explicit state.  `feed(tokens)` appends tokens and returns (logits [n, vocab],
    residual streams [layers + 1][n, W]: entry 0 after the embedding, entry i + 1 after layer i)."""

    def __init__(self, cfg: dict, w: dict, dtype=torch.float64):
        self.cfg, self.dtype = cfg, dtype
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
        self.n = 0
        nl = len(cfg["layers"])
        self.keys = [None] * nl        # [n, G, D] as stored (rotated, or convolved and normalised)
        self.vals = [None] * nl        # [n, G, Dv] as stored (blended)
        self.tail = [dict() for _ in range(nl)]  # attention_2: the last taps - 1 projected q / k / v rows
        self.first = first_value_layer(cfg)

    def _norm(self, x, name):
        return grouped_rms_norm(x, self.w[name], self.cfg["norm"].get("groups", 1), self.cfg["norm"]["eps"])

    def _mixer(self, li, L, x, pos, v_first):
        m, w, pre = L["mixer"], self.w, "l%d.mix." % li
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        T = x.shape[0]
        two = L["type"] == "attention_2"
        q, k, v = x @ w[pre + "q"].T, x @ w[pre + "k"].T, x @ w[pre + "v"].T
        if two:
            q, k, v = q + w[pre + "q.b"], k + w[pre + "k.b"], v + w[pre + "v.b"]
            taps = m["conv"]
            conv = {}
            for name, u in (("q", q), ("k", k), ("v", v)):
                before = self.tail[li].get(name)
                conv[name] = causal_short_conv(u, w[pre + name + ".conv"], before)
                ext = u if before is None else torch.cat([before, u], 0)
                if ext.shape[0] < taps - 1:
                    ext = torch.cat([torch.zeros(taps - 1 - ext.shape[0], u.shape[1], dtype=u.dtype), ext], 0)
                self.tail[li][name] = ext[ext.shape[0] - (taps - 1):] if taps > 1 else ext[:0]
            q, k, v = conv["q"], conv["k"], conv["v"]
        q, k, v = q.reshape(T, H, D), k.reshape(T, G, D), v.reshape(T, G, Dv)
        if two:
            q, k = unit_rms(q, self.cfg["norm"]["eps"]), unit_rms(k, self.cfg["norm"]["eps"])
        elif m.get("rot"):
            q = rotate_pairs(q, pos, m["rot"]["base"], m["rot"]["dims"])
            k = rotate_pairs(k, pos, m["rot"]["base"], m["rot"]["dims"])
        if m.get("v_mix"):
            if li == self.first:
                v_first = v
            else:
                v = blend_values(v, v_first, w[pre + "vmix"])
        self.keys[li] = k if self.keys[li] is None else torch.cat([self.keys[li], k], 0)
        self.vals[li] = v if self.vals[li] is None else torch.cat([self.vals[li], v], 0)
        kpos = torch.arange(self.keys[li].shape[0])
        if two:
            mask = m.get("mask")
            o = attend(q, self.keys[li], self.vals[li], pos, kpos, m["scale"], slopes=head_slopes(H, self.dtype),
                       window=mask["size"] if mask else None, keep_first=mask.get("keep_first", 0) if mask else 0, talk=w[pre + "talk"])
            o = o * torch.sigmoid(x @ w[pre + "g"].T)[:, :, None]
            return o.reshape(T, H * Dv) @ w[pre + "o"].T + w[pre + "o.b"], v_first
        o = attend(q, self.keys[li], self.vals[li], pos, kpos, m["scale"])
        return o.reshape(T, H * Dv) @ w[pre + "o"].T, v_first

    def feed(self, tokens):
        cfg, w = self.cfg, self.w
        tok = torch.as_tensor(tokens, dtype=torch.long)
        pos = torch.arange(self.n, self.n + len(tok))
        h = w["embed"][tok] * cfg.get("embedding", {}).get("scale", 1.0)
        streams = [h.clone()]
        v_first = None
        for li, L in enumerate(cfg["layers"]):
            pre = "l%d." % li
            y, v_first = self._mixer(li, L, self._norm(h, pre + "norm1"), pos, v_first)
            h = h + self._norm(y, pre + "norm1b")
            if L.get("mlp"):
                y = clamped_gated_ff(self._norm(h, pre + "norm2"), w, pre + "mlp.", L["mlp"]["limit"])
                h = h + self._norm(y, pre + "norm2b")
            streams.append(h.clone())
        self.n += len(tok)
        return self._norm(h, "final.norm") @ w["head"].T, streams


    def greedy(self, prompt, steps: int):
        out = []
        logits, _ = self.feed(prompt)
        for _ in range(steps):
            t = int(logits[-1].argmax())
            out.append(t)
            logits, _ = self.feed([t])
        return out


def forward(cfg: dict, w: dict, tokens, dtype=torch.float64):
    """The whole sequence in one call."""
    return Stepper(cfg, w, dtype).feed(tokens)


def random_weights(cfg: dict, seed: int, spread: float = 1.0) -> dict:
    """Random tensors under the checkpoint's names, every value exactly representable in bfloat16."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def r(*shape, s=1.0):
        return (torch.randn(*shape, generator=g) * s * spread).to(torch.bfloat16).to(torch.float32)

    def gain():
        return (1.0 + r(W, s=0.1)).to(torch.bfloat16).to(torch.float32)

    w = {"embed": r(cfg["vocab"], W, s=0.5), "head": r(cfg["vocab"], W, s=W ** -0.5), "final.norm": gain()}
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], "l%d." % i
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if L.get("mlp") else ()):
            w[p + n] = gain()
        w[p + "mix.q"], w[p + "mix.k"] = r(H * D, W, s=W ** -0.5), r(G * D, W, s=W ** -0.5)
        w[p + "mix.v"], w[p + "mix.o"] = r(G * Dv, W, s=W ** -0.5), r(W, H * Dv, s=(H * Dv) ** -0.5)
        w[p + "mix.vmix"] = torch.rand((), generator=g).to(torch.bfloat16).to(torch.float32)
        if L["type"] == "attention_2":
            for n, c in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                w[p + "mix.%s.b" % n] = r(c, s=0.1)
                w[p + "mix.%s.conv" % n] = r(c, m["conv"], s=m["conv"] ** -0.5)
            w[p + "mix.talk"] = (torch.eye(H) + r(H, H, s=0.3)).to(torch.bfloat16).to(torch.float32)
            w[p + "mix.g"], w[p + "mix.o.b"] = r(H, W, s=W ** -0.5), r(W, s=0.1)
        if L.get("mlp"):
            F = L["mlp"]["ff"]
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = r(F, W, s=W ** -0.5), r(F, W, s=W ** -0.5), r(W, F, s=F ** -0.5)
    return w
