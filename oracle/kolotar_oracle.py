"""Float64 oracle of the "Kolotar" decoder: one function per mechanism, whole sequences, no cache, no batching.

The model: every sublayer is normed AFTER the sum, x <- rmsnorm(alpha x + f(x)) * w, and reads x itself.  Mixers:

  attention         GQA with biased projections, RMS norm per head on q and k (one gain of head size for all heads),
                    rotate-half rotary on the leading channels with YaRN-scaled frequencies, values divided by their
                    RMS per head and blended with the values of the first such layer, sliding window, a per-head sink
                    logit in the softmax denominator, one sigmoid gate per head on the output
  latent attention  keys and values of all heads expanded from one normed latent per token, a rotated key part shared by
                    the heads (interleaved pairs), sliding window, plain softmax, element-wise sigmoid output gate
  parallel          left: attention WITHOUT softmax (weights sigmoid(score + b_h), RMS norm over the whole q / k
                    projection, a query temperature that grows with the logarithm of the position, tanh-capped scores,
                    the heads' weights mixed by a matrix);  right: gated delta rule (short causal convolutions + SiLU on
                    q, k, v, unit q and k, S <- g S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q, per-head RMS norm
                    times a SiLU gate);  result = a_l left + a_r right

Feed-forward: routed experts W_down(silu(W_gate h) * W_up h), the `top` largest router logits (with a bias), weights =
softmax over the chosen logits.  Logits = embed . rmsnorm(x) * w_final.

`forward(cfg, weights, tokens)` takes the parsed config.json (a dict), a {name: tensor} dict with the checkpoint's
tensor names and a list of token ids.  `round_inputs` rounds the inputs of every matrix product to bf16 (the least
rounding a bf16 engine can have); everything else stays float64.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def _bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float32).to(torch.bfloat16).to(F64)


class _Ctx:
    def __init__(self, weights: dict, round_inputs: bool):
        self.w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
        self.round = round_inputs

    def lin(self, x: torch.Tensor, name: str, bias: bool = False) -> torch.Tensor:
        """W x (+ b) for every row of x; W is stored [out, in]."""
        a = _bf16(x) if self.round else x
        y = a @ self.w[name].T
        if bias:
            y = y + self.w[name + ".b"]
        return y


# ---- norms ------------------------------------------------------------------------------------------------------------
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def unit_length(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


# ---- rotary positions -------------------------------------------------------------------------------------------------
def rotary_frequencies(dims: int, base: float, scaling: dict | None = None):
    """(frequency of pair i for i < dims / 2, factor on cos and sin).  With YaRN scaling the pairs that turn fast keep
    their frequency, the slow ones are divided by `factor`, with a linear ramp in between."""
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return torch.tensor(f, dtype=F64), 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate_half(x: torch.Tensor, pos: torch.Tensor, freq: torch.Tensor, mag: float, dims: int) -> torch.Tensor:
    """x [T, heads, d]: channel i < dims / 2 pairs with channel i + dims / 2; channels >= dims pass."""
    half = dims // 2
    a = pos.to(F64)[:, None, None] * freq[None, None, :]
    c, s = torch.cos(a) * mag, torch.sin(a) * mag
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], -1)


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, freq: torch.Tensor, dims: int) -> torch.Tensor:
    """x [T, heads, d]: channel 2i pairs with channel 2i + 1; channels >= dims pass."""
    half = dims // 2
    a = pos.to(F64)[:, None, None] * freq[None, None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
    out = x.clone()
    out[..., 0:2 * half:2] = u * c - v * s
    out[..., 1:2 * half:2] = v * c + u * s
    return out


# ---- masks ------------------------------------------------------------------------------------------------------------
def visible(T: int, window: int = 0) -> torch.Tensor:
    """[T, T] bool: query i sees key j when j <= i and (no window or i - j < window)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if window > 0:
        m = m & (i - j < window)
    return m


# ---- attention kinds --------------------------------------------------------------------------------------------------
def softmax_attention(q, k, v, scale: float, window: int, sink: torch.Tensor | None = None) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  Query head h reads key / value head h // (H / G).  `sink`
    [H]: a logit that joins the denominator only."""
    T, H, _ = q.shape
    G = k.shape[1]
    see = visible(T, window)
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~see, -math.inf)
        m = s.max(-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].reshape(1, 1))
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out[:, h] = (e / den) @ v[:, g]
    return out


def sigmoid_attention(q, k, v, scale: float, softcap: float, head_bias: torch.Tensor, talk: torch.Tensor) -> torch.Tensor:
    """Causal attention without a softmax: weight_h(i, j) = sigmoid(cap(score_h(i, j)) + b_h) for j <= i, never
    normalised over j; then weight_h <- sum_g talk[h, g] weight_g, applied to the values of head h's own value head."""
    T, H, _ = q.shape
    G = k.shape[1]
    see = visible(T)
    w = torch.zeros(H, T, T, dtype=F64)
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].T) * scale
        if softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        w[h] = torch.sigmoid(s + head_bias[h]) * see
    mixed = torch.einsum("hg,gij->hij", talk, w)
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for h in range(H):
        out[:, h] = mixed[h] @ v[:, h // (H // G)]
    return out


# ---- the gated delta rule ---------------------------------------------------------------------------------------------
def causal_conv_silu(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, n]: y_t = sum_j taps[:, n - 1 - j] x_(t - j) (zeros before the start), then SiLU."""
    T, C = x.shape
    n = taps.shape[1]
    y = torch.zeros(T, C, dtype=F64)
    for j in range(n):
        if j < T:
            y[j:] += x[:T - j] * taps[:, n - 1 - j]
    return y * torch.sigmoid(y)


def gated_delta_rule(q, k, v, beta, g) -> torch.Tensor:
    """q, k [T, Gk, dk], v [T, H, dv], beta, g [T, H] -> o [T, H, dv]; value head h uses q / k head h // (H / Gk).
    Token by token: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, H, dv = v.shape
    Gk, dk = k.shape[1], k.shape[2]
    rep = H // Gk
    S = torch.zeros(H, dk, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        kt = k[t].repeat_interleave(rep, 0)                  # [H, dk]
        qt = q[t].repeat_interleave(rep, 0)
        S = S * g[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, qt)
    return o


# ---- mixers -----------------------------------------------------------------------------------------------------------
def attention_mixer(c: _Ctx, p: str, m: dict, h: torch.Tensor, pos: torch.Tensor, eps: float, shared: dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])
    q = c.lin(h, p + "q", True).view(T, H, d)
    k = c.lin(h, p + "k", True).view(T, G, d)
    v = c.lin(h, p + "v", True).view(T, G, dv)
    q = rms_norm(q, c.w[p + "q.norm"], eps)
    k = rms_norm(k, c.w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot and int(rot.get("dims", 0)) > 0:
        freq, mag = rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        q = rotate_half(q, pos, freq, mag, int(rot["dims"]))
        k = rotate_half(k, pos, freq, mag, int(rot["dims"]))
    v = rms_unit(v, eps)
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = c.w[p + "vmix"]
            v = (1.0 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    window = int((m.get("mask") or {}).get("size", 0))
    sink = c.w.get(p + "sink")
    o = softmax_attention(q, k, v, float(m["scale"]), window, sink)
    if p + "g" in c.w:
        o = o * torch.sigmoid(c.lin(h, p + "g"))[:, :, None]
    return c.lin(o.reshape(T, H * dv), p + "o", True)


def latent_mixer(c: _Ctx, p: str, m: dict, h: torch.Tensor, pos: torch.Tensor, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dr, dv, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    q = c.lin(h, p + "q").view(T, H, d + dr)
    dkv = c.lin(h, p + "dkv")
    lat = rms_norm(dkv[:, :rank], c.w[p + "dkv.norm"], eps)
    k_rot = dkv[:, rank:].view(T, 1, dr)
    rot = m.get("rot") or {}
    freq, _ = rotary_frequencies(dr, float(rot.get("base", 10000.0)))
    q_rot = rotate_pairs(q[..., d:], pos, freq, dr)
    k_rot = rotate_pairs(k_rot, pos, freq, dr)
    k_plain = c.lin(lat, p + "uk").view(T, H, d)
    v = c.lin(lat, p + "uv").view(T, H, dv)
    qq = torch.cat([q[..., :d], q_rot], -1)
    kk = torch.cat([k_plain, k_rot.expand(T, H, dr)], -1)
    window = int((m.get("mask") or {}).get("size", 0))
    o = softmax_attention(qq, kk, v, float(m["scale"]), window).reshape(T, H * dv)
    o = o * torch.sigmoid(c.lin(h, p + "g"))
    return c.lin(o, p + "o")


def parallel_mixer(c: _Ctx, p: str, m: dict, h: torch.Tensor, pos: torch.Tensor, eps: float) -> torch.Tensor:
    T = h.shape[0]
    # left: sigmoid attention
    a, lp = m["left"], p + "left."
    H, G, d, dv = int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"]), int(a["vdim"])
    q = rms_norm(c.lin(h, lp + "q"), c.w[lp + "q.norm"], eps).view(T, H, d)
    k = rms_norm(c.lin(h, lp + "k"), c.w[lp + "k.norm"], eps).view(T, G, d)
    v = c.lin(h, lp + "v").view(T, G, dv)
    qt = a.get("q_temp")
    if qt:
        temp = 1.0 + float(qt["coef"]) * torch.log(torch.floor((pos.to(F64) + 1.0) / float(qt["every"])) + 1.0)
        q = q * temp[:, None, None]
    left = sigmoid_attention(q, k, v, float(a["scale"]), float(a.get("softcap", 0.0)), c.w[lp + "pb"], c.w[lp + "talk"])
    left = c.lin(left.reshape(T, H * dv), lp + "o")
    # right: gated delta rule
    r, rp = m["right"], p + "right."
    Hv, Gk, dk, dvr = int(r["heads"]), int(r.get("kv_heads", r["heads"])), int(r["dim"]), int(r["vdim"])
    rq = causal_conv_silu(c.lin(h, rp + "q"), c.w[rp + "q.conv"]).view(T, Gk, dk)
    rk = causal_conv_silu(c.lin(h, rp + "k"), c.w[rp + "k.conv"]).view(T, Gk, dk)
    rv = causal_conv_silu(c.lin(h, rp + "v"), c.w[rp + "v.conv"]).view(T, Hv, dvr)
    rq = unit_length(rq) * dk ** -0.5
    rk = unit_length(rk)
    beta = torch.sigmoid(c.lin(h, rp + "b"))
    g = torch.exp(-torch.exp(c.w[rp + "A_log"]) * torch.nn.functional.softplus(c.lin(h, rp + "a") + c.w[rp + "dt_bias"]))
    o = gated_delta_rule(rq, rk, rv, beta, g)
    o = rms_unit(o, eps) * c.w[rp + "norm"]
    gate = c.lin(h, rp + "g").view(T, Hv, dvr)
    o = o * (gate * torch.sigmoid(gate))
    right = c.lin(o.reshape(T, Hv * dvr), rp + "o")
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ---- feed-forward -----------------------------------------------------------------------------------------------------
def routed_experts(c: _Ctx, p: str, f: dict, h: torch.Tensor) -> torch.Tensor:
    E, top = int(f["router"]["experts"]), int(f["router"]["top"])
    z = c.lin(h, p + "router", True)
    val, idx = torch.topk(z, top, dim=-1)
    wt = torch.softmax(val, -1)
    out = torch.zeros_like(h)
    for e in range(E):
        rows, which = (idx == e).nonzero(as_tuple=True)
        if rows.numel() == 0:
            continue
        x = h[rows]
        gate = c.lin(x, f"{p}e{e}.gate")
        y = c.lin(gate * torch.sigmoid(gate) * c.lin(x, f"{p}e{e}.up"), f"{p}e{e}.down")
        out[rows] += wt[rows, which][:, None] * y
    return out


def router_margins(c: _Ctx, p: str, f: dict, h: torch.Tensor) -> torch.Tensor:
    """Per row: the gap between the last chosen and the first left-out router logit (a close call may flip in bf16)."""
    z = c.lin(h, p + "router", True)
    top = int(f["router"]["top"])
    if top >= z.shape[-1]:
        return torch.full((z.shape[0],), math.inf, dtype=F64)
    s = torch.sort(z, -1, descending=True).values
    return s[:, top - 1] - s[:, top]


# ---- the model --------------------------------------------------------------------------------------------------------
def forward(cfg: dict, weights: dict, tokens, round_inputs: bool = False, margins: list | None = None):
    """-> (logits [T, vocab], residual stream after every layer [layers, T, width]), float64."""
    c = _Ctx(weights, round_inputs)
    eps, alpha = float(cfg["norm"]["eps"]), float(cfg["postln_alpha"])
    tok = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(tok.numel())
    x = c.w["embed"][tok]
    shared: dict = {}
    trace = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        if L["type"] == "attention":
            y = attention_mixer(c, p + "mix.", L["mixer"], x, pos, eps, shared)
        elif L["type"] == "latent_attention":
            y = latent_mixer(c, p + "mix.", L["mixer"], x, pos, eps)
        elif L["type"] == "parallel":
            y = parallel_mixer(c, p + "mix.", L["mixer"], x, pos, eps)
        else:
            raise ValueError(f"layer {i}: unknown mixer {L['type']!r}")
        x = rms_norm(alpha * x + y, c.w[p + "norm1"], eps)
        f = L.get("mlp")
        if f is not None:
            if margins is not None:
                margins.append(router_margins(c, p + "mlp.", f, x))
            x = rms_norm(alpha * x + routed_experts(c, p + "mlp.", f, x), c.w[p + "norm2"], eps)
        trace.append(x.clone())
    xn = rms_norm(x, c.w["final.norm"], eps)
    logits = (_bf16(xn) if round_inputs else xn) @ c.w["embed"].T
    return logits, torch.stack(trace) if trace else torch.zeros(0, tok.numel(), x.shape[-1], dtype=F64)


# ---- random checkpoints for the tests ---------------------------------------------------------------------------------
def tensor_shapes(cfg: dict) -> dict:
    """{tensor name: shape} of a checkpoint of this config."""
    W, out = int(cfg["width"]), {"embed": (int(cfg["vocab"]), int(cfg["width"])), "final.norm": (int(cfg["width"]),)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", L["mixer"]
        if L["type"] == "attention":
            H, G, d, dv = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])
            for name, rows in (("q", H * d), ("k", G * d), ("v", G * dv), ("o", W)):
                out[p + name] = (rows, W if name != "o" else H * dv)
                out[p + name + ".b"] = (rows,)
            out.update({p + "q.norm": (d,), p + "k.norm": (d,), p + "vmix": (), p + "sink": (H,), p + "g": (H, W)})
        elif L["type"] == "latent_attention":
            H, d, dr, dv, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
            out.update({p + "q": (H * (d + dr), W), p + "dkv": (r + dr, W), p + "dkv.norm": (r,), p + "uk": (H * d, r),
                        p + "uv": (H * dv, r), p + "g": (H * dv, W), p + "o": (W, H * dv)})
        else:
            a, r = m["left"], m["right"]
            H, G, d, dv = int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"]), int(a["vdim"])
            out.update({p + "left.q": (H * d, W), p + "left.k": (G * d, W), p + "left.v": (G * dv, W), p + "left.q.norm": (H * d,),
                        p + "left.k.norm": (G * d,), p + "left.pb": (H,), p + "left.talk": (H, H), p + "left.o": (W, H * dv)})
            Hv, Gk, dk, dvr, taps = int(r["heads"]), int(r.get("kv_heads", r["heads"])), int(r["dim"]), int(r["vdim"]), int(r["conv"])
            out.update({p + "right.q": (Gk * dk, W), p + "right.q.conv": (Gk * dk, taps), p + "right.k": (Gk * dk, W),
                        p + "right.k.conv": (Gk * dk, taps), p + "right.v": (Hv * dvr, W), p + "right.v.conv": (Hv * dvr, taps),
                        p + "right.b": (Hv, W), p + "right.A_log": (Hv,), p + "right.norm": (dvr,), p + "right.a": (Hv, W),
                        p + "right.dt_bias": (Hv,), p + "right.g": (Hv * dvr, W), p + "right.o": (W, Hv * dvr)})
        out[f"l{i}.norm1"] = (W,)
        f = L.get("mlp")
        if f is not None:
            E, ff = int(f["router"]["experts"]), int(f["expert"]["ff"])
            for e in range(E):
                out.update({f"l{i}.mlp.e{e}.gate": (ff, W), f"l{i}.mlp.e{e}.up": (ff, W), f"l{i}.mlp.e{e}.down": (W, ff)})
            out.update({f"l{i}.mlp.router": (E, W), f"l{i}.mlp.router.b": (E,), f"l{i}.norm2": (W,)})
    return out


def random_weights(cfg: dict, seed: int = 0, dtype=torch.bfloat16) -> dict:
    """Random tensors rounded to `dtype`, so that the engine and the oracle see the same numbers.  Matrices have unit
    row gain, gains are spread around one, router rows are scaled so that the choice is rarely a close call."""
    g = torch.Generator().manual_seed(seed)
    wt = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        rnd = lambda std=1.0: torch.randn(shape, generator=g) * std
        if leaf in ("norm1", "norm2", "norm") or name == "final.norm":
            t = 1.0 + rnd(0.2)
        elif name == "embed":
            t = rnd(0.7)
        elif leaf == "vmix":
            t = 0.2 + 0.6 * torch.rand(shape, generator=g)
        elif leaf == "talk":
            t = torch.eye(shape[0]) + rnd(0.3)
        elif leaf == "A_log":
            t = torch.log(0.05 + 0.5 * torch.rand(shape, generator=g))
        elif leaf in ("sink", "pb", "dt_bias"):
            t = rnd(1.0)
        elif leaf == "b" and len(shape) == 1:
            t = rnd(0.3)
        elif leaf == "conv":
            t = rnd(0.6)
        elif leaf == "router":
            t = rnd(4.0 / math.sqrt(shape[-1]))
        else:
            t = rnd(1.0 / math.sqrt(shape[-1]))
        wt[name] = t.to(dtype).to(F64)
    return wt
