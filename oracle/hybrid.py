"""Oracle for layer-list models (the Safupel design): plain, slow float64 PyTorch, one function per mechanism.

TEST INFRASTRUCTURE.  Nothing here is shared with the product path.  Notation: x is the residual stream [T, D],
h its normalised copy, t / j are positions from 0, W matrices are [out, in] and act as h @ W.T.

  layer        h = rms(x) * (1 + g);   x <- x + (mixer(h) + ff(h))
  rglru        y = gelu_tanh(h Wy + by);  u = causal_conv(h Wx + bx);  per block b of the channels:
               r = sigmoid(Ra_b u_b + ra_b), i = sigmoid(Ri_b u_b + ri_b);  a = exp(-8 r softplus(lam));
               s_t = a s_(t-1) + sqrt(1 - a^2) i u,  s_(-1) = 0;   out = (s * y) Wo
  attention    score(t, j) = scale q_t.k_j - 2^(-8 (head+1) / heads) (t - j), keys j <= t of the same chunk
               (floor(t / c) == floor(j / c)), softmax, grouped key/value heads
  mlstm        log gates i~ = cap tanh(z_i / cap), f~ = logsigmoid(cap tanh(z_f / cap)); m_t = max(f~ + m_(t-1), i~), m_(-1) = 0;
               C_t = exp(f~ + m_(t-1) - m_t) C_(t-1) + exp(i~ - m_t) k v^T, n_t alike with k;  q scaled by dim^-0.5;
               o = C_t^T q / (max(|n_t.q|, exp(-m_t)) + 1e-6);  per head o / rms(o), times a weight, times sigmoid(h Wg), then Wo
  parallel     left_scale * attention + right_scale * mlstm
  dense ff     gelu_erf(h Wup) Wdown
  moe ff       p = sigmoid(h Wr); the `top` largest p choose experts; out = sum_e expert_e(p_e h) + shared(h),
               expert(z) = (silu(z Wg) * (z Wu)) Wd
  logits       rms-norm with the final weight, head matrix, times logit_scale
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch
import torch.nn.functional as F

DT = torch.float64


# ------------------------------------------------------------------------------------------ configs and weights

def make_config(vocab=97, width=64, layers=("parallel", "rglru"), mlps=("moe", "dense"), *, heads=4, kv_heads=2, dim=16, vdim=24,
                chunk=40, scale=0.21, m_heads=3, m_dim=8, m_vdim=16, gate_cap=9.0, left_scale=1.1, right_scale=0.8,
                r_width=96, r_blocks=3, r_conv=4, ff=72, experts=5, top=2, expert_ff=24, shared_ff=40, eps=1e-5, logit_scale=0.5):
    """A config.json dict of the layout the product's loader reads.  `layers` and `mlps` give each layer's mixer type and
    feed-forward kind ("dense", "moe", "moe-noshared" or None)."""
    out = []
    for mixer, mlp in zip(layers, mlps):
        if mixer == "rglru":
            m = {"blocks": r_blocks, "conv": r_conv, "width": r_width}
        else:
            m = {"left": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": chunk}, "scale": scale, "vdim": vdim},
                 "left_scale": left_scale, "right": {"dim": m_dim, "gate_cap": gate_cap, "heads": m_heads, "vdim": m_vdim},
                 "right_scale": right_scale}
        if mlp == "dense":
            f = {"ff": ff, "kind": "dense"}
        elif mlp in ("moe", "moe-noshared"):
            f = {"expert": {"ff": expert_ff}, "kind": "moe", "router": {"experts": experts, "top": top}}
            if mlp == "moe":
                f["shared"] = {"ff": shared_ff}
        else:
            f = None
        out.append({"mixer": m, "mlp": f, "type": mixer})
    return {"architecture": "Safupel", "layers": out, "logit_scale": logit_scale, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def tensor_shapes(cfg):
    D, V = cfg["width"], cfg["vocab"]
    sh = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        sh[p + "norm1"] = (D,)
        if L["type"] == "rglru":
            w, nb = m["width"], m["blocks"]
            bw = w // nb
            sh.update({p + "mix.y": (w, D), p + "mix.y.b": (w,), p + "mix.x": (w, D), p + "mix.x.b": (w,), p + "mix.conv": (w, m["conv"]),
                       p + "mix.conv.b": (w,), p + "mix.ra": (nb, bw, bw), p + "mix.ra.b": (nb, bw), p + "mix.ri": (nb, bw, bw),
                       p + "mix.ri.b": (nb, bw), p + "mix.lam": (w,), p + "mix.o": (D, w)})
        else:
            a, r = m["left"], m["right"]
            sh.update({p + "mix.left.q": (a["heads"] * a["dim"], D), p + "mix.left.k": (a["kv_heads"] * a["dim"], D),
                       p + "mix.left.v": (a["kv_heads"] * a["vdim"], D), p + "mix.left.o": (D, a["heads"] * a["vdim"]),
                       p + "mix.right.q": (r["heads"] * r["dim"], D), p + "mix.right.k": (r["heads"] * r["dim"], D),
                       p + "mix.right.v": (r["heads"] * r["vdim"], D), p + "mix.right.g": (r["heads"] * r["vdim"], D),
                       p + "mix.right.o": (D, r["heads"] * r["vdim"]), p + "mix.right.norm": (r["heads"] * r["vdim"],),
                       p + "mix.right.i": (r["heads"], D), p + "mix.right.i.b": (r["heads"],), p + "mix.right.f": (r["heads"], D),
                       p + "mix.right.f.b": (r["heads"],)})
        f = L["mlp"]
        if f and f["kind"] == "dense":
            sh.update({p + "mlp.up": (f["ff"], D), p + "mlp.down": (D, f["ff"])})
        elif f:
            sh[p + "mlp.router"] = (f["router"]["experts"], D)
            names = [f"e{x}" for x in range(f["router"]["experts"])] + (["shared"] if f.get("shared") else [])
            for n in names:
                e = f["shared"]["ff"] if n == "shared" else f["expert"]["ff"]
                sh.update({f"{p}mlp.{n}.gate": (e, D), f"{p}mlp.{n}.up": (e, D), f"{p}mlp.{n}.down": (D, e)})
    return sh


def make_weights(cfg, seed=0):
    """Random bfloat16-representable weights (returned as float64), sized so that activations stay O(1)."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if name.endswith("norm1") or name == "final.norm":
            t = 0.2 * torch.randn(shape, generator=g)
        elif name.endswith("right.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif last == "lam":
            t = torch.randn(shape, generator=g) - 1.5
        elif last == "conv":
            t = 0.5 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (1.5 / math.sqrt(shape[-1]))
        W[name] = t.to(torch.bfloat16).to(DT)
    return W


def save_model_dir(path, cfg, W):
    """config.json + model.safetensors (bfloat16), written by hand: 8-byte header length, JSON header, raw data."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    hdr, blobs, off = {}, [], 0
    for k, v in W.items():
        raw = v.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        hdr[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    js = json.dumps(hdr).encode()
    with open(os.path.join(path, "model.safetensors"), "wb") as fh:
        fh.write(struct.pack("<Q", len(js)) + js + b"".join(blobs))


# ------------------------------------------------------------------------------------------ mechanisms

def rms_norm_plus_one(x, g, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + g)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def causal_conv(x, w, b):
    """x [T, C]; w [C, taps] with the LAST tap on the current position; zeros before position 0."""
    T, taps = x.shape[0], w.shape[1]
    out = b.expand(T, -1).clone()
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                out[t] += w[:, j] * x[src]
    return out


def rglru(h, P, blocks):
    """P: dict with y, y.b, x, x.b, conv, conv.b, ra, ra.b, ri, ri.b, lam, o."""
    T = h.shape[0]
    y = gelu_tanh(h @ P["y"].T + P["y.b"])
    u = causal_conv(h @ P["x"].T + P["x.b"], P["conv"], P["conv.b"])
    bw = u.shape[1] // blocks
    r = torch.empty_like(u)
    i = torch.empty_like(u)
    for b in range(blocks):
        ub = u[:, b * bw:(b + 1) * bw]
        r[:, b * bw:(b + 1) * bw] = torch.sigmoid(ub @ P["ra"][b].T + P["ra.b"][b])
        i[:, b * bw:(b + 1) * bw] = torch.sigmoid(ub @ P["ri"][b].T + P["ri.b"][b])
    a = torch.exp(-8.0 * r * F.softplus(P["lam"]))
    s = torch.zeros(u.shape[1], dtype=DT)
    out = []
    for t in range(T):
        s = a[t] * s + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out.append(s * y[t])
    return torch.stack(out) @ P["o"].T


def chunked_biased_attention(h, P, heads, kv_heads, dim, vdim, scale, chunk):
    T = h.shape[0]
    q = (h @ P["q"].T).view(T, heads, dim)
    k = (h @ P["k"].T).view(T, kv_heads, dim)
    v = (h @ P["v"].T).view(T, kv_heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=DT)
    for hd in range(heads):
        g = hd // (heads // kv_heads)
        slope = 2.0 ** (-8.0 * (hd + 1) / heads)
        for t in range(T):
            lo = (t // chunk) * chunk if chunk > 0 else 0
            js = torch.arange(lo, t + 1)
            sc = (k[lo:t + 1, g] @ q[t, hd]) * scale - slope * (t - js).to(DT)
            out[t, hd] = torch.softmax(sc, 0) @ v[lo:t + 1, g]
    return out.reshape(T, heads * vdim) @ P["o"].T


def mlstm(h, P, heads, dim, vdim, cap, eps):
    T = h.shape[0]
    q = (h @ P["q"].T).view(T, heads, dim) * dim ** -0.5
    k = (h @ P["k"].T).view(T, heads, dim)
    v = (h @ P["v"].T).view(T, heads, vdim)
    li = cap * torch.tanh((h @ P["i"].T + P["i.b"]) / cap)
    lf = F.logsigmoid(cap * torch.tanh((h @ P["f"].T + P["f.b"]) / cap))
    out = torch.zeros(T, heads, vdim, dtype=DT)
    for hd in range(heads):
        C = torch.zeros(dim, vdim, dtype=DT)
        n = torch.zeros(dim, dtype=DT)
        m = torch.zeros((), dtype=DT)
        for t in range(T):
            m_new = torch.maximum(lf[t, hd] + m, li[t, hd])
            C = torch.exp(lf[t, hd] + m - m_new) * C + torch.exp(li[t, hd] - m_new) * torch.outer(k[t, hd], v[t, hd])
            n = torch.exp(lf[t, hd] + m - m_new) * n + torch.exp(li[t, hd] - m_new) * k[t, hd]
            m = m_new
            o = (C.T @ q[t, hd]) / (torch.maximum((n @ q[t, hd]).abs(), torch.exp(-m)) + 1e-6)
            out[t, hd] = o / torch.sqrt(o.pow(2).mean() + eps)
    return (out.reshape(T, heads * vdim) * P["norm"] * torch.sigmoid(h @ P["g"].T)) @ P["o"].T


def gated_expert(z, P):
    return (F.silu(z @ P["gate"].T) * (z @ P["up"].T)) @ P["down"].T


def moe(h, router, experts, shared, top):
    p = torch.sigmoid(h @ router.T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(p.shape[1]), key=lambda e: (-p[t, e].item(), e))[:top]
        for e in order:
            out[t] += gated_expert(p[t, e] * h[t], experts[e])
    if shared is not None:
        out = out + gated_expert(h, shared)
    return out


def sub(W, prefix):
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (float64), optionally the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)]
    layers = []
    for i, L in enumerate(cfg["layers"]):
        h = rms_norm_plus_one(x, W[f"l{i}.norm1"], eps)
        m = L["mixer"]
        if L["type"] == "rglru":
            mix = rglru(h, sub(W, f"l{i}.mix."), m["blocks"])
        else:
            a, r = m["left"], m["right"]
            mix = m["left_scale"] * chunked_biased_attention(h, sub(W, f"l{i}.mix.left."), a["heads"], a["kv_heads"], a["dim"], a["vdim"],
                                                             a["scale"], a["mask"]["size"]) \
                + m["right_scale"] * mlstm(h, sub(W, f"l{i}.mix.right."), r["heads"], r["dim"], r["vdim"], r["gate_cap"], eps)
        f = L["mlp"]
        if f is None:
            ff = torch.zeros_like(x)
        elif f["kind"] == "dense":
            ff = gelu_erf(h @ W[f"l{i}.mlp.up"].T) @ W[f"l{i}.mlp.down"].T
        else:
            ex = [sub(W, f"l{i}.mlp.e{e}.") for e in range(f["router"]["experts"])]
            ff = moe(h, W[f"l{i}.mlp.router"], ex, sub(W, f"l{i}.mlp.shared.") if f.get("shared") else None, f["router"]["top"])
        x = x + (mix + ff)
        layers.append(x)
    logits = (rms_norm_plus_one(x, W["final.norm"], eps) @ W["head"].T) * cfg["logit_scale"]
    return (logits, layers) if return_layers else logits


def greedy(cfg, W, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]
