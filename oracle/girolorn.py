"""Oracle for the Girolorn design (a layer list of attention mixers and mixtures of experts): plain, slow float64
PyTorch, one function per mechanism.

TEST INFRASTRUCTURE.  Nothing here is shared with the product path.  Notation: x is the residual stream [T, D], t / j are
positions from 0, W matrices are [out, in] and act as h @ W.T, H query heads on G key/value heads of size dim.

  layer        x <- x + attention(ln(x, w1));   x <- x + moe(ln(x, w2))      ln: (x - mean) / sqrt(var + eps) * w
  rotary       f_i = base^(-2i / r), i < r / 2, on dimensions (2i, 2i + 1) of the first r of a head:
               (a, b) -> c (a cos(t f_i) - b sin(t f_i), b cos(t f_i) + a sin(t f_i))
               scaled frequencies: n(u) = r ln(orig / (2 pi u)) / (2 ln base); lo = max(floor(n(fast)), 0),
               hi = min(ceil(n(slow)), r - 1); g_i = clip((i - lo) / max(hi - lo, 1e-3), 0, 1);
               f_i <- g_i f_i / factor + (1 - g_i) f_i;  c = 1 + 0.1 ln(factor)   (c = 1 without scaling)
  attention    q = rms_all(h Wq) * nq, k = rms_all(h Wk) * nk over the full projection rows; v = h Wk (untouched);
               rotary on q and k;  s(t, j) = cap tanh(scale q_t.k_j / cap), j <= t;
               p(t, j) = exp(s(t, j)) / (exp(sink_head) + sum_j' exp(s(t, j')));  out = (p v) Wo
  expert       a = min(h Wg, L), b = clip(h Wu, -L, L);  (a sigmoid(1.702 a) (b + 1)) Wd
  moe          z = h Wr + br;  the `top` largest z choose experts, weights softmax over those z;
               out = sum_e weight_e expert_e(h) + sigmoid(h . wsg) shared(h)
  logits       ln with the final weight, head matrix, then cap tanh(. / cap)
"""
from __future__ import annotations

import math

import torch

from .hybrid import DT, save_model_dir  # noqa: F401  (file writer only: config.json + safetensors by hand)


def make_config(vocab=101, width=48, n_layers=3, *, heads=4, kv_heads=2, dim=12, rot_dims=8, base=5000.0, scaling=(4.0, 64, 16.0, 2.0),
                scale=0.3, softcap=7.0, experts=5, top=2, expert_ff=20, expert_limit=1.5, shared_ff=28, shared_limit=0.75, shared=True,
                mlps=None, weights_of=None, eps=1e-5, logit_softcap=11.0):
    """A config.json dict of the layout the product's loader reads.  scaling = (factor, original, fast, slow) or None;
    mlps[i] False drops layer i's feed-forward; weights_of = {layer: earlier layer} marks layers without tensors of their own."""
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    out = []
    for i in range(n_layers):
        f = {"expert": {"ff": expert_ff, "limit": expert_limit}, "kind": "moe", "router": {"experts": experts, "top": top}}
        if shared:
            f["shared"] = {"ff": shared_ff, "limit": shared_limit}
        if mlps is not None and not mlps[i]:
            f = None
        L = {"mixer": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": dict(rot), "scale": scale, "softcap": softcap, "vdim": dim},
             "mlp": f, "type": "attention"}
        if weights_of and i in weights_of:
            L["weights_of"] = weights_of[i]
        out.append(L)
    return {"architecture": "Girolorn", "layers": out, "logit_softcap": logit_softcap, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def tensor_shapes(cfg):
    D, V = cfg["width"], cfg["vocab"]
    sh = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    for i, L in enumerate(cfg["layers"]):
        if "weights_of" in L:
            continue
        p, m = f"l{i}.", L["mixer"]
        nq, nk = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
        sh.update({p + "norm1": (D,), p + "mix.q": (nq, D), p + "mix.k": (nk, D), p + "mix.q.norm": (nq,), p + "mix.k.norm": (nk,),
                   p + "mix.sink": (m["heads"],), p + "mix.o": (D, nq)})
        f = L["mlp"]
        if f:
            sh[p + "norm2"] = (D,)
            sh[p + "mlp.router"] = (f["router"]["experts"], D)
            sh[p + "mlp.router.b"] = (f["router"]["experts"],)
            for n in [f"e{x}" for x in range(f["router"]["experts"])] + (["shared"] if f.get("shared") else []):
                e = f["shared"]["ff"] if n == "shared" else f["expert"]["ff"]
                sh.update({f"{p}mlp.{n}.gate": (e, D), f"{p}mlp.{n}.up": (e, D), f"{p}mlp.{n}.down": (D, e)})
            if f.get("shared"):
                sh[p + "mlp.shared.sg"] = (1, D)
    return sh


def make_weights(cfg, seed=0):
    """Random bfloat16-representable weights (returned as float64), sized so that activations stay O(1) and the caps,
    the clamps and the sinks all bite."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last in ("norm1", "norm2") or name == "final.norm" or name.endswith(".norm"):
            t = 1.0 + 0.3 * torch.randn(shape, generator=g)
        elif last == "sink":
            t = 1.5 * torch.randn(shape, generator=g)
        elif last == "b":
            t = 0.5 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif last in ("q", "k"):
            t = torch.randn(shape, generator=g) * (3.0 / math.sqrt(shape[-1]))
        else:
            t = torch.randn(shape, generator=g) * (1.5 / math.sqrt(shape[-1]))
        W[name] = t.to(torch.bfloat16).to(DT)
    return W


# ------------------------------------------------------------------------------------------ mechanisms

def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = (x - mu).pow(2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_all(x, w, eps):
    """RMS norm over the whole last axis (all heads of a projection at once)."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def rotary_frequencies(rot):
    r, base = rot["dims"], rot["base"]
    i = torch.arange(r // 2, dtype=DT)
    f = base ** (-2.0 * i / r)
    c = 1.0
    sc = rot.get("scaling")
    if sc:
        def n(u):
            return r * math.log(sc["original"] / (2.0 * math.pi * u)) / (2.0 * math.log(base))
        lo, hi = max(math.floor(n(sc["fast"])), 0), min(math.ceil(n(sc["slow"])), r - 1)
        g = ((i - lo) / max(hi - lo, 1e-3)).clamp(0.0, 1.0)
        f = g * f / sc["factor"] + (1.0 - g) * f
        c = 1.0 + 0.1 * math.log(sc["factor"])
    return f, c


def rotary(x, positions, rot):
    """x [T, heads, dim]: pairs (2i, 2i + 1) of the first rot['dims'] dimensions turn by position * f_i."""
    r = rot["dims"]
    if r == 0:
        return x
    f, c = rotary_frequencies(rot)
    ang = positions.to(DT)[:, None] * f[None, :]
    cos, sin = (c * torch.cos(ang))[:, None, :], (c * torch.sin(ang))[:, None, :]
    a, b = x[..., 0:r:2], x[..., 1:r:2]
    turned = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).flatten(-2)
    return torch.cat([turned, x[..., r:]], dim=-1)


def sink_attention(h, P, m, eps, positions=None):
    T = h.shape[0]
    H, G, dim = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(T) if positions is None else positions
    q0, k0 = h @ P["q"].T, h @ P["k"].T
    v = k0.view(T, G, dim)
    q = rotary(rms_all(q0, P["q.norm"], eps).view(T, H, dim), pos, m["rot"])
    k = rotary(rms_all(k0, P["k.norm"], eps).view(T, G, dim), pos, m["rot"])
    out = torch.zeros(T, H, dim, dtype=DT)
    cap = m.get("softcap") or 0.0
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        for t in range(T):
            e = torch.exp(s[t, :t + 1])
            out[t, hd] = (e / (e.sum() + torch.exp(P["sink"][hd]))) @ v[:t + 1, g]
    return out.reshape(T, H * dim) @ P["o"].T


def clamped_expert(z, P, limit):
    a = (z @ P["gate"].T).clamp(max=limit)
    b = (z @ P["up"].T).clamp(-limit, limit)
    return (a * torch.sigmoid(1.702 * a) * (b + 1.0)) @ P["down"].T


def route(h, router, bias, top):
    """Per token: the chosen experts (largest logits first, ties to the lower index) and their weights."""
    z = h @ router.T + bias
    picks = []
    for t in range(h.shape[0]):
        order = sorted(range(z.shape[1]), key=lambda e: (-z[t, e].item(), e))[:top]
        w = torch.softmax(z[t, order], dim=0)
        picks.append((order, w))
    return picks


def route_margins(h, router, bias, top):
    """Per token: by how much the last chosen logit leads the first one left out (inf when every expert is chosen)."""
    z, _ = torch.sort(h @ router.T + bias, dim=-1, descending=True)
    if top >= z.shape[1]:
        return torch.full((h.shape[0],), math.inf, dtype=DT)
    return z[:, top - 1] - z[:, top]


def moe(h, W, prefix, f):
    out = torch.zeros_like(h)
    for t, (order, w) in enumerate(route(h, W[prefix + "router"], W[prefix + "router.b"], f["router"]["top"])):
        for e, we in zip(order, w):
            out[t] += we * clamped_expert(h[t], sub(W, f"{prefix}e{e}."), f["expert"]["limit"])
    if f.get("shared"):
        gate = torch.sigmoid(h @ W[prefix + "shared.sg"].T)
        out = out + gate * clamped_expert(h, sub(W, prefix + "shared."), f["shared"]["limit"])
    return out


def sub(W, prefix):
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def forward(cfg, W, tokens, return_layers=False, return_margins=False):
    """Logits [T, vocab] of one sequence (float64); optionally the residual stream after every layer, or per token the
    smallest routing margin over the layers (a 16-bit engine may choose another expert where it is tiny)."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)]
    layers = []
    margins = torch.full((len(tokens),), math.inf, dtype=DT)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{L.get('weights_of', i)}."
        x = x + sink_attention(layer_norm(x, W[p + "norm1"], eps), sub(W, p + "mix."), L["mixer"], eps)
        if L["mlp"]:
            h2 = layer_norm(x, W[p + "norm2"], eps)
            margins = torch.minimum(margins, route_margins(h2, W[p + "mlp.router"], W[p + "mlp.router.b"], L["mlp"]["router"]["top"]))
            x = x + moe(h2, W, p + "mlp.", L["mlp"])
        layers.append(x)
    z = layer_norm(x, W["final.norm"], eps) @ W["head"].T
    cap = cfg.get("logit_softcap") or 0.0
    logits = cap * torch.tanh(z / cap) if cap > 0 else z
    if return_margins:
        return logits, margins
    return (logits, layers) if return_layers else logits


def greedy(cfg, W, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]
