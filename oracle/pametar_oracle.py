"""Oracle for the "Pametar" decoders (pipelinerl_b200/hybrid.py, `HybridConfig.from_pametar`): a plain, slow,
whole-sequence implementation.

TEST INFRASTRUCTURE (see oracle/__init__.py).  Torch float64 on CPU, one function per mechanism, every recurrence an
explicit loop over time, no cache, no chunks, no batching, no absorbed products, nothing shared with the product path.
The reference has no model code of its own (it serves through vLLM, pipelinerl/launch.py:191-247), so these functions
restate the design's equations and are the yardstick for the CUDA kernels.

Notation: T tokens, W the model width, h [T, W] a sublayer's input, weights stored [out, in] and applied as h @ M.T.
`wt` maps a checkpoint tensor name to a float64 tensor, `p` is the prefix of a sublayer's tensors, `cfg` the dict of
config.json.  `round_in`, when given, is applied to both operands of every matrix product (tests use it to measure the
least error a bf16 product can have).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def _mm(a, w, round_in=None):
    if round_in is not None:
        a, w = round_in(a), round_in(w)
    return a @ w.T


def rms_unit(x, eps):
    """x over its root mean square along the last axis (eps under the root)."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def tanh_norm(x, wt, name):
    """Dynamic-tanh "norm": no statistics, tanh(alpha x) * gain + shift."""
    return torch.tanh(wt[name + ".alpha"] * x) * wt[name] + wt[name + ".b"]


def silu(x):
    return x * torch.sigmoid(x)


def embed(tokens, wt, cfg):
    """Scaled token embedding plus a hashed embedding of the (previous, current) token pair; the first token of a
    sequence, which has no previous one, takes the table's extra last row."""
    e = cfg["embedding"]
    x = wt["embed"][torch.tensor(tokens)] * e["scale"]
    b = e.get("bigram")
    if b is not None:
        for t, tok in enumerate(tokens):
            row = b["buckets"] if t == 0 else (tokens[t - 1] * b["mul_prev"] + tok * b["mul_cur"]) % b["buckets"]
            x[t] = x[t] + wt["bigram"][row]
    return x


# ---- mixers ---------------------------------------------------------------------------------------------------------
def rotate_half(x, base, first_pos=0):
    """x [T, n]: channel i pairs with channel i + n/2; the pair turns by pos * base^(-2i/n)."""
    T, n = x.shape
    half = n // 2
    out = x.clone()
    for i in range(half):
        ang = (torch.arange(T, dtype=F64) + first_pos) * base ** (-2.0 * i / n)
        c, s = torch.cos(ang), torch.sin(ang)
        u, v = x[:, i], x[:, i + half]
        out[:, i] = u * c - v * s
        out[:, i + half] = v * c + u * s
    return out


def latent_attention(h, wt, p, m, eps, round_in=None):
    """Softmax attention whose keys and values are expanded from one normed low-rank latent per token, whose queries
    come through a normed latent of their own, with one rotated key part shared by all heads, and with a per-head
    "sink" logit that joins the softmax denominator only.  Everything is expanded here: per-head keys and values."""
    T = h.shape[0]
    H, d, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base = m["rot"]["base"]
    assert m["rot"]["dims"] == dr
    cq = rms_unit(_mm(h, wt[p + "dq"], round_in), eps) * wt[p + "dq.norm"]
    q = _mm(cq, wt[p + "uq"], round_in).view(T, H, d + dr)
    dkv = _mm(h, wt[p + "dkv"], round_in)
    c = rms_unit(dkv[:, :rk], eps) * wt[p + "dkv.norm"]
    k_rot = rotate_half(dkv[:, rk:], base)
    k = _mm(c, wt[p + "uk"], round_in).view(T, H, d)
    v = _mm(c, wt[p + "uv"], round_in).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        q_rot = rotate_half(q[:, head, d:], base)
        sink = float(wt[p + "sink"][head]) if p + "sink" in wt else -math.inf       # a checkpoint without sinks: plain softmax
        for t in range(T):
            s = (k[:t + 1, head] @ q[t, head, :d] + k_rot[:t + 1] @ q_rot[t]) * m["scale"]
            top = max(float(s.max()), sink)
            e = torch.exp(s - top)
            den = e.sum() + math.exp(sink - top)
            out[t, head] = (e / den) @ v[:t + 1, head]
    return _mm(out.reshape(T, H * dv), wt[p + "o"], round_in)


def general_delta(h, wt, p, m, eps, round_in=None):
    """Delta-rule memory with a decay and a removal rate per key channel:
    S <- diag(w) S - (a * u)(u^T S) + k v^T, o = S^T r, with u the key of unit length; both corrections read the old S."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = _mm(h, wt[p + "r"], round_in).view(T, H, d)
    k = _mm(h, wt[p + "k"], round_in).view(T, H, d)
    v = _mm(h, wt[p + "v"], round_in).view(T, H, d)
    low = torch.tanh(_mm(h, wt[p + "w1"], round_in))
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(_mm(low, wt[p + "w2"], round_in) + wt[p + "w0"])).view(T, H, d)
    a = torch.sigmoid(_mm(h, wt[p + "a"], round_in) + wt[p + "a.b"]).view(T, H, d)
    out = torch.zeros(T, H, d, dtype=F64)
    for head in range(H):
        S = torch.zeros(d, d, dtype=F64)
        for t in range(T):
            kt = k[t, head]
            u = kt / torch.sqrt(kt.pow(2).sum() + 1e-6)
            S = w[t, head][:, None] * S - torch.outer(a[t, head] * u, u @ S) + torch.outer(kt, v[t, head])
            out[t, head] = S.T @ r[t, head]
    y = rms_unit(out, eps).reshape(T, H * d) * wt[p + "norm"] * torch.sigmoid(_mm(h, wt[p + "g"], round_in))
    return _mm(y, wt[p + "o"], round_in)


# ---- feed-forward -----------------------------------------------------------------------------------------------------
def routed_experts(h, wt, p, f, round_in=None, margins=None):
    """Softmax over all experts; the `top` largest are taken; each taken expert's output is weighted by its softmax
    score times a constant (scores are not renormalised over the taken ones).  `margins`, a list, receives per token the
    gap between the last taken and the first left-out router logit (inf when all are taken)."""
    T, W = h.shape
    E, top, scale = f["router"]["experts"], f["router"]["top"], f["router"].get("scale", 1.0)
    z = _mm(h, wt[p + "router"], round_in)
    s = torch.softmax(z, dim=-1)
    out = torch.zeros(T, W, dtype=F64)
    for t in range(T):
        ranked = sorted(range(E), key=lambda e: (-float(s[t, e]), e))
        order = ranked[:top]
        if margins is not None:
            margins.append(float(z[t, ranked[top - 1]] - z[t, ranked[top]]) if top < E else math.inf)
        for e in order:
            q = f"{p}e{e}."
            a = silu(_mm(h[t:t + 1], wt[q + "gate"], round_in)) * _mm(h[t:t + 1], wt[q + "up"], round_in)
            out[t] += float(s[t, e]) * scale * _mm(a, wt[q + "down"], round_in)[0]
    return out


# ---- the layer arrangement --------------------------------------------------------------------------------------------
def sublayer(xs, fn, wt, layer, q, round_in=None):
    """One sublayer on the residual streams xs [S, T, W] (q = 1: mixer, 2: feed-forward).  The sublayer reads a
    weighted sum of the streams through the tanh norm; its result, scaled per channel and gated by a sigmoid of a
    projection of the same normed input, is added to every stream with that stream's weight after the streams have
    been mixed among themselves."""
    S = xs.shape[0]
    hc = f"{layer}.hc{q}."
    if hc + "in" in wt:
        u = sum(wt[hc + "in"][s] * xs[s] for s in range(S))
    else:
        assert S == 1
        u = xs[0]
    h = tanh_norm(u, wt, f"{layer}.norm{q}")
    y = fn(h)
    if f"{layer}.ls{q}" in wt:
        y = y * wt[f"{layer}.ls{q}"]
    if f"{layer}.rg{q}" in wt:
        y = y * torch.sigmoid(_mm(h, wt[f"{layer}.rg{q}"], round_in) + wt[f"{layer}.rg{q}.b"])
    new = torch.zeros_like(xs)
    for t in range(S):
        if hc + "in" in wt:
            new[t] = sum(wt[hc + "mix"][s, t] * xs[s] for s in range(S)) + wt[hc + "out"][t] * y
        else:
            new[t] = xs[t] + y
    return new


def layer_runs(cfg):
    """Indices of the layers in the order they run: the block [start, stop) repeats `times` times in a row."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, k = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * k + list(range(b, n))


def forward(tokens, wt, cfg, round_in=None, trace=None, margins=None):
    """Logits [T, vocab] of one sequence.  `trace`, a list, receives the sum of the streams after every layer run;
    `margins`, a list, one list of router gaps (see routed_experts) per routed feed-forward that runs."""
    eps = cfg["norm"]["eps"]
    x = embed(tokens, wt, cfg)
    S = int(cfg.get("streams", 1))
    xs = torch.stack([x.clone() for _ in range(S)])
    for i in layer_runs(cfg):
        L, name = cfg["layers"][i], f"l{i}"
        mixer = {"latent_attention": latent_attention, "general_delta": general_delta}[L["type"]]
        xs = sublayer(xs, lambda h: mixer(h, wt, name + ".mix.", L["mixer"], eps, round_in), wt, name, 1, round_in)
        if L.get("mlp") is not None:
            gaps = [] if margins is not None else None
            xs = sublayer(xs, lambda h: routed_experts(h, wt, name + ".mlp.", L["mlp"], round_in, gaps), wt, name, 2, round_in)
            if margins is not None:
                margins.append(gaps)
        if trace is not None:
            trace.append(xs.sum(0))
    return _mm(tanh_norm(xs.sum(0), wt, "final.norm"), wt["head"], round_in)


# ---- random checkpoints for the tests -----------------------------------------------------------------------------------
def tensor_shapes(cfg, layer_scale=True, gated=True, hyper=True, sink=True):
    """Checkpoint tensor names and shapes of a configuration; the four flags leave out optional parts of every layer."""
    W, S, out = cfg["width"], int(cfg.get("streams", 1)), {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        if L["type"] == "latent_attention":
            H, d, dr, dv, rk, rq = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out.update({p + "mix.dq": (rq, W), p + "mix.dq.norm": (rq,), p + "mix.uq": (H * (d + dr), rq),
                        p + "mix.dkv": (rk + dr, W), p + "mix.dkv.norm": (rk,), p + "mix.uk": (H * d, rk),
                        p + "mix.uv": (H * dv, rk), p + "mix.o": (W, H * dv)})
            if sink:
                out[p + "mix.sink"] = (H,)
        else:
            n, r = m["heads"] * m["dim"], m["rank"]
            for name in ("r", "k", "v", "g", "a"):
                out[p + "mix." + name] = (n, W)
            out.update({p + "mix.a.b": (n,), p + "mix.w1": (r, W), p + "mix.w2": (n, r), p + "mix.w0": (n,),
                        p + "mix.norm": (n,), p + "mix.o": (W, n)})
        for q in ("1", "2") if L.get("mlp") is not None else ("1",):
            out.update({f"{p}norm{q}": (W,), f"{p}norm{q}.b": (W,), f"{p}norm{q}.alpha": ()})
            if layer_scale:
                out[f"{p}ls{q}"] = (W,)
            if gated:
                out.update({f"{p}rg{q}": (W, W), f"{p}rg{q}.b": (W,)})
            if hyper:
                out.update({f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
        f = L.get("mlp")
        if f is not None:
            out[p + "mlp.router"] = (f["router"]["experts"], W)
            for e in range(f["router"]["experts"]):
                out.update({f"{p}mlp.e{e}.gate": (f["expert"]["ff"], W), f"{p}mlp.e{e}.up": (f["expert"]["ff"], W),
                            f"{p}mlp.e{e}.down": (W, f["expert"]["ff"])})
    out.update({"embed": (cfg["vocab"], W), "final.norm": (W,), "final.norm.b": (W,), "final.norm.alpha": (),
                "head": (cfg["vocab"], W)})
    if cfg["embedding"].get("bigram") is not None:
        out["bigram"] = (cfg["embedding"]["bigram"]["buckets"] + 1, W)
    return out


def random_weights(cfg, seed=0, dtype=torch.bfloat16, **parts):
    """Random tensors, rounded to `dtype` so that the engine and the oracle see the same numbers.  Matrices have unit
    row gain (std 1/sqrt(fan_in)); gains, stream weights and scales are spread around their neutral values."""
    g = torch.Generator().manual_seed(seed)
    S, wt = int(cfg.get("streams", 1)), {}
    for name, shape in tensor_shapes(cfg, **parts).items():
        leaf = name.split(".")[-1]
        rnd = lambda std=1.0: torch.randn(shape, generator=g) * std
        if ".hc" in name:
            t = {"in": 1.0 / S + rnd(0.2), "out": 1.0 + rnd(0.2), "mix": torch.eye(S) + rnd(0.15)}[leaf]
        elif leaf == "alpha":
            t = 0.4 + 0.2 * torch.rand(shape, generator=g)
        elif leaf in ("norm1", "norm2", "norm", "ls1", "ls2") or name == "final.norm":
            t = 1.0 + rnd(0.2)
        elif name in ("embed", "bigram"):
            t = rnd(0.7)
        elif leaf == "b":
            t = rnd(0.3)
        elif leaf in ("sink", "w0"):
            t = rnd(1.0)
        elif leaf == "router":
            t = rnd(4.0 / math.sqrt(shape[-1]))                             # well separated scores
        else:
            t = rnd(1.0 / math.sqrt(shape[-1]))
        wt[name] = t.to(dtype).to(F64)
    return wt
