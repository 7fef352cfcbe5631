"""Plain, slow restatement of the Lerasun decoder, one function per mechanism, for the tests.

Lerasun is a decoder-only model whose layers add a mixer branch and a feed-forward branch, both
computed from the same residual stream, back onto it:

    h <- h + mixer(n1(h)) + ff(n2(h)),       n(x) = x / sqrt(mean(x^2) + eps) * (1 + g)

Mixer: attention over a shared low-rank latent.  Every token stores one latent vector c (kv_rank
numbers, unit-RMS-normalised with a plain gain) and one rotated key piece r (rot_dim numbers) that all
heads share; head a rebuilds its keys U_k[a] c and values U_v[a] c from the latent.  The softmax of
every head has one extra term exp(sink[a]) in its denominator that belongs to no key.  A layer may
read the latent and rotated piece that an earlier layer stored instead of producing its own.

Feed-forward: a routed mixture of small two-matrix experts with a squared-ReLU between them.  The
router scores are sigmoids; a per-expert offset is added for the *choice* only; experts are grouped
and only the best groups (by the sum of their two best choice scores) may supply experts; the
chosen experts' plain scores, normalised to sum one, weight their outputs.

Nothing here shares code with the engine: tensors go in as a dict of fp32/fp64 torch tensors under
the checkpoint's names and every function is written for clarity, not speed.
"""
from __future__ import annotations

import math

import torch

NORM_SUM_GUARD = 1e-20   # added to the sum of the chosen scores before the division


def unit_offset_rms_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """x / rms(x) * (1 + g); the gain is stored around zero."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (1.0 + g)


def plain_rms_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * g


def rotate_pairs(v: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Rotary positions, interleaved layout: (v[2i], v[2i+1]) turns by pos * base^(-2i/dims) for the first `dims`
    entries of the last axis; the rest passes.  v [..., T, D], pos [T]."""
    out = v.clone()
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    freq = torch.as_tensor(base, dtype=v.dtype) ** (-2.0 * i / dims)
    ang = pos.to(v.dtype)[:, None] * freq[None, :]          # [T, half]
    c, s = torch.cos(ang), torch.sin(ang)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def latent_and_rotated_key(x: torch.Tensor, pos: torch.Tensor, w: dict, pre: str, m: dict, eps: float):
    """What one layer stores per token: the normalised latent [T, kv_rank] and the rotated shared key piece [T, rot_dim]."""
    d = x @ w[pre + "dkv"].T
    r = m["kv_rank"]
    c = plain_rms_norm(d[:, :r], w[pre + "dkv.norm"], eps)
    kr = rotate_pairs(d[:, r:r + m["rot_dim"]], pos, m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(x: torch.Tensor, pos: torch.Tensor, c_all: torch.Tensor, kr_all: torch.Tensor, w: dict, pre: str,
                     m: dict) -> torch.Tensor:
    """x [T, W] are the new tokens at positions pos; c_all / kr_all hold the stored latent and rotated piece of positions
    0 .. pos[-1] of the same sequence (the new tokens' own included).  Written head by head, key by key."""
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    T = x.shape[0]
    q = (x @ w[pre + "q"].T).reshape(T, H, dn + dr)
    outs = torch.zeros(T, H * dv, dtype=x.dtype)
    for a in range(H):
        qn = q[:, a, :dn]
        qr = rotate_pairs(q[:, a, dn:], pos, m["rot"]["base"], m["rot"]["dims"])
        kn = c_all @ w[pre + "uk"][a * dn:(a + 1) * dn].T      # [S, dn]
        vv = c_all @ w[pre + "uv"][a * dv:(a + 1) * dv].T      # [S, dv]
        s = (qn @ kn.T + qr @ kr_all.T) * m["scale"]           # [T, S]
        keys = torch.arange(c_all.shape[0])
        s = s.masked_fill(keys[None, :] > pos[:, None], -math.inf)
        sink = w[pre + "sink"][a]
        mx = torch.maximum(s.max(-1, keepdim=True).values, sink)
        e = torch.exp(s - mx)
        den = e.sum(-1, keepdim=True) + torch.exp(sink - mx)
        outs[:, a * dv:(a + 1) * dv] = (e / den) @ vv
    return outs @ w[pre + "o"].T


def route(x: torch.Tensor, w: dict, pre: str, r: dict):
    """Returns (expert indices [T, top], weights [T, top])."""
    E, top = r["experts"], r["top"]
    G, keep = r["groups"]["count"], r["groups"]["keep"]
    s = torch.sigmoid(x @ w[pre + "router"].T)
    choice = s + w[pre + "correction"]
    per = E // G
    grp = choice.reshape(-1, G, per)
    gscore = grp.topk(min(2, per), dim=-1).values.sum(-1)        # [T, G]
    kept = gscore.topk(keep, dim=-1).indices
    allowed = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, kept, True)
    masked = torch.where(allowed[:, :, None].expand(-1, -1, per).reshape(-1, E), choice, torch.full_like(choice, -math.inf))
    idx = masked.topk(top, dim=-1).indices
    sc = s.gather(1, idx)
    return idx, sc / (sc.sum(-1, keepdim=True) + NORM_SUM_GUARD)


def expert_mixture(x: torch.Tensor, w: dict, pre: str, mlp: dict) -> torch.Tensor:
    idx, wt = route(x, w, pre, mlp["router"])
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for k in range(idx.shape[1]):
            e = int(idx[t, k])
            u = torch.relu(w[f"{pre}e{e}.up"] @ x[t]) ** 2
            out[t] += wt[t, k] * (w[f"{pre}e{e}.down"] @ u)
    return out


class Oracle:
    """Holds the stored latents of one sequence and runs new tokens through the model."""

    def __init__(self, cfg: dict, weights: dict, dtype=torch.float64):
        self.cfg = cfg
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
        self.dtype = dtype
        self.store: dict[int, list] = {}   # layer -> [c, kr] of all positions so far
        self.n = 0

    def forward(self, tokens, capture_layers: bool = False):
        cfg, w, eps = self.cfg, self.w, self.cfg["norm"]["eps"]
        T = len(tokens)
        pos = torch.arange(self.n, self.n + T)
        h = unit_offset_rms_norm(w["embed"][torch.as_tensor(tokens)], w["embed.norm"], eps)
        trace = []
        for i, layer in enumerate(cfg["layers"]):
            m = layer["mixer"]
            pre = f"l{i}.mix."
            x1 = unit_offset_rms_norm(h, w[f"l{i}.norm1"], eps)
            if layer["type"] != "latent_attention":
                raise ValueError("unknown mixer " + layer["type"])
            src = m.get("kv_from")
            if src is None:
                c, kr = latent_and_rotated_key(x1, pos, w, pre, m, eps)
                if i in self.store:
                    self.store[i] = [torch.cat([self.store[i][0], c]), torch.cat([self.store[i][1], kr])]
                else:
                    self.store[i] = [c, kr]
                src = i
            c_all, kr_all = self.store[src]
            y = latent_attention(x1, pos, c_all, kr_all, w, pre, m)
            if layer.get("mlp") is not None:
                if layer["mlp"]["kind"] != "moe":
                    raise ValueError("unknown feed-forward " + layer["mlp"]["kind"])
                x2 = unit_offset_rms_norm(h, w[f"l{i}.norm2"], eps)
                y = y + expert_mixture(x2, w, f"l{i}.mlp.", {"router": layer["mlp"]["router"]})
            h = h + y
            if capture_layers:
                trace.append(h.clone())
        self.n += T
        logits = (unit_offset_rms_norm(h, w["final.norm"], eps) @ w["head"].T) * cfg["logit_scale"]
        return (logits, torch.stack(trace)) if capture_layers else logits

    def greedy(self, prompt, steps: int):
        out = []
        logits = self.forward(prompt)
        for _ in range(steps):
            t = int(logits[-1].argmax())
            out.append(t)
            logits = self.forward([t])
        return out


def tensor_shapes(cfg: dict) -> dict:
    W, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, W), "embed.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        p = f"l{i}."
        s[p + "norm1"] = (W,)
        if layer.get("mlp") is not None:
            s[p + "norm2"] = (W,)
        H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        s[p + "mix.q"] = (H * (dn + dr), W)
        if m.get("kv_from") is None:
            s[p + "mix.dkv"] = (r + dr, W)
            s[p + "mix.dkv.norm"] = (r,)
        s[p + "mix.uk"] = (H * dn, r)
        s[p + "mix.uv"] = (H * dv, r)
        s[p + "mix.sink"] = (H,)
        s[p + "mix.o"] = (W, H * dv)
        if layer.get("mlp") is not None:
            ff, E = layer["mlp"]["expert"]["ff"], layer["mlp"]["router"]["experts"]
            for e in range(E):
                s[p + f"mlp.e{e}.up"] = (ff, W)
                s[p + f"mlp.e{e}.down"] = (W, ff)
            s[p + "mlp.router"] = (E, W)
            s[p + "mlp.correction"] = (E,)
    s["final.norm"] = (W,)
    s["head"] = (V, W)
    return s


def random_weights(cfg: dict, seed: int = 0) -> dict:
    """bf16-representable random weights sized so that activations stay O(1) through the layers."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("dkv.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif "norm" in name:
            t = 0.2 * torch.randn(shape, generator=g)
        elif name.endswith("sink"):
            t = torch.randn(shape, generator=g)
        elif name.endswith("correction"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif name.endswith("router"):
            t = torch.randn(shape, generator=g) * (2.0 / math.sqrt(shape[-1]))
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
