"""Hybrid decoders on the sampler engine: layers whose mixer is gated linear attention, or softmax attention running
in parallel with a state-space (Mamba-2 form) mixer, each sublayer normalised on its OUTPUT (x += norm(f(x))), with a
clamped gated feed-forward.  The reference serves any architecture its vLLM serves (pipelinerl/launch.py:191-247,
conf/base.yaml:59-73); this module is how such a family runs on `engine.EngineCore`: the core's slots, page pool,
scheduler, sampler and CUDA graph are shared with the Qwen2 engine, and this file adds only the layer program.

`HybridConfig` is a list of layer specs; every size and constant is a field, nothing is fixed to one model.  The
"Povurax" and "Belelorn" architectures are two parsers of that config (`HybridConfig.from_povurax`, `.from_belelorn`):
another design built from the same mixers needs a parser, not new kernels.  Belelorn adds: a matrix-memory LSTM mixer
(stabilised exponential gates), softmax attention whose values are its keys (per-head unit norms, tanh-capped scores,
a sliding window that keeps the first tokens) beside lightning attention (one fixed decay per head), every sublayer
normed on its input AND its output with gains kept as offsets from one, squared-ReLU and routed (mixture-of-experts)
feed-forwards, a block of layers that runs several times on the same weights with a cache and state per pass, and
sinusoidal positions added to the embedding.  "Pametar" (`.from_pametar`) adds: latent attention (keys and values of all
heads expanded from one cached low-rank latent, a rotated key part shared by the heads, a per-head sink logit in the
softmax denominator), a delta-rule matrix memory with per-channel decay and removal rate, a residual kept as several
parallel streams that every sublayer reads and writes through learned weights, a statistics-free tanh norm, per-channel
layer scale and a sigmoid gate on every sublayer's result, routed experts weighted by a softmax over all experts, and a
hashed token-pair table added to the embedding (the previous token is per-sequence state).

Numerics: the residual stream, every norm, softmax, router-like gate, decay, step size and recurrent state are fp32.
GEMM operands and the KV cache are bf16, or fp32 when the arena is fp32 (the true-fp32 mode: CUDA-core GEMMs with fp32
accumulation in a fixed order, no TF32).  One code path serves prompt chunks, single decoded tokens and mixtures of
both ("ragged rows"); a token's result depends only on its own sequence.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _lib
from .cache import PAGE_SIZE
from .engine import EngineCore


@dataclass(frozen=True)
class AttnSpec:
    heads: int
    kv_heads: int
    dim: int            # query / key size per head
    vdim: int           # value size per head
    rot_dims: int       # leading channels of each head that are rotated (interleaved pairs)
    rot_base: float
    scale: float        # score = (q . k) * scale
    # what follows is off / zero for a plain attention layer
    softcap: float = 0.0        # > 0: score <- softcap * tanh(score / softcap)
    window: int = 0             # > 0: a query sees only the last `window` positions (itself included) ...
    keep_first: int = 0         # ... and the first `keep_first` tokens of the sequence
    head_norm: bool = False     # q and k divided by their RMS per head, no gain (instead of one gained norm over all heads)
    bias: bool = False          # q and k projections have biases
    value_is_key: bool = False  # no value projection: the value is the key as projected (before its norm)
    gate: bool = True           # sigmoid output gate from its own projection
    # what follows belongs to the layers normed after the sum (HybridConfig.block == "post_ln")
    gate_per_head: bool = False  # the gate projection has one row per head instead of one per output channel
    head_gain: bool = False     # the per-head norms of q and k have a gain of head size shared by all heads (q.norm, k.norm)
    v_bias: bool = False        # the value projection has a bias
    o_bias: bool = False        # the output projection has a bias
    rot_half: bool = False      # rotated pairs are (i, i + rot_dims / 2) instead of (2i, 2i + 1)
    rot_scaling: tuple | None = None   # YaRN: (factor, original length, fast turns, slow turns)
    v_norm: bool = False        # every value head divided by its root mean square (no gain) before it is cached
    v_mix: int = 0              # 1: this layer's values are kept for later layers; 2: v <- (1 - l) v + l v_first, l = `vmix`
    v_mix_tensor: bool = False  # the checkpoint has a `vmix` scalar for this layer (used only when v_mix == 2)
    sink: bool = False          # a learned logit per head in the softmax denominator (no key, no value)
    weights: str = "softmax"    # "sigmoid": weight = sigmoid(score + pb[h]) for every visible key, not normalised
    q_temp: tuple = (0.0, 1.0)  # (coef, every): q times 1 + coef * ln(floor((pos + 1) / every) + 1)
    talking: bool = False       # the heads' weights are mixed by the matrix `talk` [heads, heads] before they meet the values


@dataclass(frozen=True)
class LightningSpec:
    """Linear attention S <- decay_h S + k v^T, o = S^T q, with SiLU on q, k, v and one fixed decay per head."""
    heads: int
    dim: int
    vdim: int
    decay: tuple


@dataclass(frozen=True)
class MlstmSpec:
    """Matrix-memory LSTM cell: exponential input gate, sigmoid forget gate, both soft-capped, running stabiliser."""
    heads: int
    dim: int
    vdim: int
    gate_cap: float
    den_eps: float = 1e-6


@dataclass(frozen=True)
class LatentAttnSpec:
    """Softmax attention over ONE cached latent per token: c = rmsnorm(W_dkv h)[:kv_rank], keys W_uk c and values W_uv c
    per head, plus `rot_dim` rotated key channels shared by all heads; queries through a normed latent of size q_rank."""
    heads: int
    dim: int            # unrotated query / key channels per head
    rot_dim: int        # rotated channels per head ("rotate half" pairs i, i + rot_dim / 2)
    vdim: int
    kv_rank: int
    q_rank: int
    rot_base: float
    scale: float
    sink: bool = True   # a learned logit per head in the softmax denominator (no key, no value)
    window: int = 0     # > 0: a query sees only the last `window` positions (itself included)
    interleaved: bool = False   # rotated pairs are (2i, 2i + 1) instead of (i, i + rot_dim / 2)
    gate: bool = False  # element-wise sigmoid gate on the concatenated heads, from its own projection `g`
    # q_rank == 0: the query comes straight from the layer's input (tensor `q`), without a latent


@dataclass(frozen=True)
class GatedDeltaSpec:
    """Gated delta rule S <- g S; d = beta (v - S^T k); S <- S + k d^T; o = S^T q: short causal convolutions + SiLU on
    q, k, v, unit q (times dim^-1/2) and k, beta = sigmoid(.), one decay g = exp(-exp(A_log) softplus(. + dt_bias)) per
    head, per-head RMS norm with a gain of size vdim times a SiLU gate.  `kv_heads` q / k heads serve `heads` value heads."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    unit_eps: float = 1e-6

    @property
    def conv_channels(self) -> int:
        return 2 * self.kv_heads * self.dim + self.heads * self.vdim

    @property
    def in_rows(self) -> int:   # [q | k | v | b | a | g]
        return self.conv_channels + 2 * self.heads + self.heads * self.vdim


@dataclass(frozen=True)
class DeltaSpec:
    """Delta-rule memory S <- diag(w) S - (a u)(u^T S) + k v^T, o = S^T r, u the unit key, w = exp(-decay_scale
    sigmoid(.)) from a rank-`rank` bottleneck, a = sigmoid(.); key and value size are both `dim`."""
    heads: int
    dim: int
    rank: int
    decay_scale: float = math.exp(-0.5)
    unit_eps: float = 1e-6


@dataclass(frozen=True)
class MoeSpec:
    experts: int
    top: int
    ff: int
    limit: float
    shared_ff: int = 0          # 0: no shared expert
    shared_limit: float = 0.0
    score: str = "sigmoid"      # "sigmoid" of the chosen logit | "softmax_all": softmax over ALL experts, not renormalised
                                # | "softmax_top": softmax over the chosen logits only
    router_bias: bool = False   # the router logits get a bias per expert (`router.b`) before the choice
    weight_on: str = "input"    # the score scales the expert's "input" (clamped unit) or its "output" (plain SiLU unit)
    weight_scale: float = 1.0   # constant factor on the scores


@dataclass(frozen=True)
class SsdSpec:
    heads: int
    vdim: int
    state: int          # N
    groups: int         # B / C groups
    conv: int           # taps of the causal convolution over x, B, C
    norm_groups: int    # the gated output is RMS-normed in this many equal parts

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state

    @property
    def in_rows(self) -> int:   # [z | x | B | C | dt]
        return 2 * self.inner + 2 * self.groups * self.state + self.heads


@dataclass(frozen=True)
class GlaSpec:
    heads: int
    dim: int
    vdim: int
    tau: float          # decay = sigmoid(z)^(1/tau)
    rank: int           # bottleneck of the decay projection


@dataclass(frozen=True)
class MlpSpec:
    ff: int
    limit: float
    beta: float = 1.702  # g * sigmoid(beta * g)
    kind: str = "glu"    # "glu": clamped gated unit | "relu2": W_down relu(W_up h)^2 | "moe": routed experts (+ a shared one)
    moe: MoeSpec | None = None


@dataclass(frozen=True)
class LayerSpec:
    kind: str                       # "gla" | "parallel" (attention || state space) | "parallel_lin" (attention || lightning) | "mlstm"
                                    # | "latent" (latent attention) | "delta" (delta-rule memory): the multi-stream program
                                    # | "attention" | "latent_attention" | "sigmoid_delta" (attention without a softmax ||
                                    #   gated delta rule): the layers normed after the sum
    weights_of: int                 # index of the layer whose tensors this layer uses (its own index if it has its own)
    gla: GlaSpec | None = None
    attn: AttnSpec | None = None
    ssd: SsdSpec | None = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    mlp: MlpSpec | None = None
    lin: LightningSpec | None = None
    mlstm: MlstmSpec | None = None
    sandwich: bool = False          # norms before AND after each sublayer (norm1, norm1b, norm2, norm2b) instead of after only
    opens_pass: int | None = None   # this run opens pass t of a repeated block: x <- W_loop [x; x0] + step[t] comes first
    latent: LatentAttnSpec | None = None
    delta: DeltaSpec | None = None
    layer_scale: bool = False       # sublayer results times a per-channel vector (ls1 / ls2)
    gated: bool = False             # sublayer results times sigmoid(W_rg h + b) of the sublayer's own input
    hyper: bool = False             # learned read / write / mixing weights over the residual streams (hc1.* / hc2.*)
    gdelta: GatedDeltaSpec | None = None


@dataclass(frozen=True)
class HybridConfig:
    vocab_size: int
    width: int
    eps: float
    embed_scale: float
    layers: tuple                   # one LayerSpec per layer RUN (a repeated block is unrolled; runs share tensors by weights_of)
    positions: str = "none"         # "sinusoid": sin / cos of position * 10000^(-2i/width) added to the embedding
    logit_scale: float = 1.0
    norm_offset: float = 0.0        # gains of the width norms are stored as offsets from this value
    loop_times: int = 0             # passes of the repeated block (rows of `loop.step`); 0: no such block
    norm_kind: str = "rms"          # "tanh": tanh(alpha x) * gain + shift, no statistics (tensors <name>, .b, .alpha)
    streams: int = 1                # parallel copies of the residual ("tanh" program only)
    pair_embed: tuple | None = None  # (buckets, mul_prev, mul_cur): hashed (previous, current) token table `bigram`
    block: str = "out_norm"         # "post_ln": x <- norm(skip_scale * x + f(x)) for every sublayer, f reads x itself
    skip_scale: float = 1.0
    tied_head: bool = False         # logits = embed . x: no separate `head` tensor

    @property
    def head_rows(self) -> int:
        return self.vocab_size

    @property
    def hidden_size(self) -> int:
        return self.width

    # ---- the "Povurax" reading of config.json ---------------------------------------------------------------------
    @staticmethod
    def from_povurax(d: dict, tensor_shapes: dict | None = None) -> "HybridConfig":
        """config.json of a Povurax checkpoint.  The rank of a GLA layer's decay bottleneck is not a config key: it is
        the row count of the layer's `mix.a1` tensor (tensor_shapes), or `mixer.rank` when building without a file."""
        layers = []
        n_layers = len(d["layers"])

        def owner(i: int) -> int:
            """The layer whose tensors layer i runs with: follow `weights_of` to a layer that has its own."""
            seen = set()
            while "weights_of" in d["layers"][i] and int(d["layers"][i]["weights_of"]) != i:
                if i in seen:
                    raise ValueError(f"layer {i}: weights_of runs in a circle")
                seen.add(i)
                i = int(d["layers"][i]["weights_of"])
                if not 0 <= i < n_layers:
                    raise ValueError(f"weights_of names layer {i}, which does not exist")
            return i
        for i, L in enumerate(d["layers"]):
            j = owner(i)
            if L["type"] != d["layers"][j]["type"]:
                raise ValueError(f"layer {i} ({L['type']}) cannot run with the tensors of layer {j} ({d['layers'][j]['type']})")
            m = L["mixer"]
            mlp = None
            if L.get("mlp") is not None:
                if L["mlp"].get("kind", "dense") != "dense":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {L['mlp'].get('kind')!r}")
                mlp = MlpSpec(ff=int(L["mlp"]["ff"]), limit=float(L["mlp"]["limit"]))
            if L["type"] == "gla":
                rank = m.get("rank")
                if rank is None and tensor_shapes is not None:
                    rank = tensor_shapes[f"l{j}.mix.a1"][0]
                if rank is None:
                    raise ValueError(f"layer {i}: the decay rank is neither in the config nor in a tensor shape")
                layers.append(LayerSpec("gla", j, gla=GlaSpec(int(m["heads"]), int(m["dim"]), int(m["vdim"]),
                                                              float(m["tau"]), int(rank)), mlp=mlp))
            elif L["type"] == "parallel":
                a, s = m["left"], m["right"]
                rot = a.get("rot") or {}                       # no rotary block: no dimension is rotated
                attn = AttnSpec(int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"]), int(a.get("vdim", a["dim"])),
                                int(rot.get("dims", 0)), float(rot.get("base", 10000.0)), float(a["scale"]))
                ssd = SsdSpec(int(s["heads"]), int(s["vdim"]), int(s["state"]), int(s["groups"]), int(s["conv"]),
                              int(s["norm_groups"]))
                layers.append(LayerSpec("parallel", j, attn=attn, ssd=ssd, left_scale=float(m["left_scale"]),
                                        right_scale=float(m["right_scale"]), mlp=mlp))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
        cfg = HybridConfig(int(d["vocab"]), int(d["width"]), float(d["norm"]["eps"]), float(d["embedding"]["scale"]),
                           tuple(layers))
        cfg.validate()
        return cfg

    # ---- the "Belelorn" reading of config.json ---------------------------------------------------------------------
    @staticmethod
    def from_belelorn(d: dict, tensor_shapes: dict | None = None) -> "HybridConfig":
        """config.json of a Belelorn checkpoint.  `loop` = {start, stop, times}: layers start .. stop-1 run `times` times
        in a row on the same tensors; every pass is a run of its own here (own cache and state)."""
        specs = []
        for i, L in enumerate(d["layers"]):
            m, mlp = L["mixer"], None
            f = L.get("mlp")
            if f is not None:
                kind = f.get("kind", "dense")
                if kind == "dense":
                    mlp = MlpSpec(ff=int(f["ff"]), limit=0.0, kind="relu2")
                elif kind == "moe":
                    sh = f.get("shared")
                    inf = float("inf")          # an expert without a limit is not clamped
                    moe = MoeSpec(int(f["router"]["experts"]), int(f["router"]["top"]), int(f["expert"]["ff"]),
                                  float(f["expert"].get("limit", inf)), int(sh["ff"]) if sh else 0,
                                  float(sh.get("limit", inf)) if sh else 0.0)
                    mlp = MlpSpec(ff=moe.shared_ff, limit=moe.shared_limit, kind="moe", moe=moe)
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")
            if L["type"] == "mlstm":
                specs.append(dict(kind="mlstm", mlp=mlp, mlstm=MlstmSpec(int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"])),
                                                                         float(m.get("gate_cap", 0.0)))))      # 0: gates not capped
            elif L["type"] == "parallel":
                a, r = m["left"], m["right"]
                mask = a.get("mask") or {}
                attn = AttnSpec(int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"]), int(a.get("vdim", a["dim"])),
                                0, 10000.0, float(a["scale"]), softcap=float(a.get("softcap", 0.0)),
                                window=int(mask.get("size", 0)), keep_first=int(mask.get("keep_first", 0)), head_norm=True,
                                bias=True, value_is_key=True, gate=False)
                decay = r["decay"] if isinstance(r["decay"], (list, tuple)) else [r["decay"]] * int(r["heads"])
                lin = LightningSpec(int(r["heads"]), int(r["dim"]), int(r.get("vdim", r["dim"])), tuple(float(v) for v in decay))
                specs.append(dict(kind="parallel_lin", mlp=mlp, attn=attn, lin=lin, left_scale=0.5, right_scale=0.5))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
        n, loop = len(specs), d.get("loop")
        runs = [(i, None) for i in range(n)]
        times = 0
        if loop:
            a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
            if not (0 <= a < b <= n and times >= 1):
                raise ValueError(f"bad loop {loop}")
            runs = [(i, None) for i in range(a)]
            for t in range(times):
                runs += [(i, t if i == a else None) for i in range(a, b)]
            runs += [(i, None) for i in range(b, n)]
        layers = tuple(LayerSpec(weights_of=i, sandwich=True, opens_pass=t, **specs[i]) for i, t in runs)
        cfg = HybridConfig(int(d["vocab"]), int(d["width"]), float(d["norm"]["eps"]), 1.0, layers, positions="sinusoid",
                           logit_scale=float(d.get("logit_scale", 1.0)), norm_offset=1.0, loop_times=times)
        cfg.validate()
        return cfg

    # ---- the "Pametar" reading of config.json ---------------------------------------------------------------------
    @staticmethod
    def from_pametar(d: dict, tensor_shapes: dict | None = None) -> "HybridConfig":
        """config.json of a Pametar checkpoint.  `loop` = {start, stop, times} repeats a block of layers on the same
        tensors (every pass is a run with its own cache and state; nothing happens between passes).  Which of layer
        scale, gate and stream weights a layer has is read off the tensor names when a file is at hand (all of them
        otherwise); the rank of the decay bottleneck is the row count of `mix.w1`."""
        shapes = tensor_shapes or {}
        specs = []
        for i, L in enumerate(d["layers"]):
            m, f, mlp = L["mixer"], L.get("mlp"), None
            if f is not None:
                if f.get("kind", "moe") != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
                r = f["router"]
                moe = MoeSpec(int(r["experts"]), int(r["top"]), int(f["expert"]["ff"]), 0.0, score="softmax_all",
                              weight_on="output", weight_scale=float(r.get("scale", 1.0)))
                mlp = MlpSpec(ff=0, limit=0.0, kind="moe", moe=moe)
            has = (lambda name: f"l{i}.{name}" in shapes) if shapes else (lambda name: True)
            flags = dict(layer_scale=has("ls1"), gated=has("rg1"), hyper=has("hc1.in"))
            if L["type"] == "latent_attention":
                rot = m.get("rot") or {}
                if int(rot.get("dims", m["rot_dim"])) != int(m["rot_dim"]):
                    raise ValueError(f"layer {i}: the rotated part has {m['rot_dim']} channels but rot.dims = {rot.get('dims')}")
                spec = LatentAttnSpec(int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"]),
                                      int(m["q_rank"]), float(rot.get("base", 10000.0)), float(m["scale"]),
                                      sink=has("mix.sink"))
                specs.append(dict(kind="latent", mlp=mlp, latent=spec, **flags))
            elif L["type"] == "general_delta":
                rank = m.get("rank")
                if f"l{i}.mix.w1" in shapes:
                    rank = shapes[f"l{i}.mix.w1"][0]
                if rank is None:
                    raise ValueError(f"layer {i}: the decay rank is neither in the config nor in a tensor shape")
                specs.append(dict(kind="delta", mlp=mlp, delta=DeltaSpec(int(m["heads"]), int(m["dim"]), int(rank)), **flags))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
        n, loop = len(specs), d.get("loop")
        runs = list(range(n))
        if loop:
            a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
            if not (0 <= a <= b <= n and times >= 1):
                raise ValueError(f"bad loop {loop}")
            runs = list(range(a)) + list(range(a, b)) * times + list(range(b, n))
        layers = tuple(LayerSpec(weights_of=i, **specs[i]) for i in runs)
        e = d["embedding"]
        pair = e.get("bigram")
        if shapes and "bigram" not in shapes:
            pair = None
        cfg = HybridConfig(int(d["vocab"]), int(d["width"]), float(d["norm"]["eps"]), float(e.get("scale", 1.0)), layers,
                           norm_kind="tanh", streams=int(d.get("streams", 1)),
                           pair_embed=(int(pair["buckets"]), int(pair["mul_prev"]), int(pair["mul_cur"])) if pair else None)
        cfg.validate()
        return cfg

    # ---- the "Kolotar" reading of config.json ---------------------------------------------------------------------
    @staticmethod
    def from_kolotar(d: dict, tensor_shapes: dict | None = None) -> "HybridConfig":
        """config.json of a Kolotar checkpoint: every sublayer normed after the sum with a weighted skip
        (`postln_alpha`), layers of three kinds in any order, routed experts everywhere, logits from the embedding
        table.  Which optional tensors a layer has (biases, sink, gate, router bias) is read off the tensor names when
        a file is at hand."""
        shapes = tensor_shapes or {}
        layers, first_vmix = [], None
        for i, L in enumerate(d["layers"]):
            m, f, mlp = L["mixer"], L.get("mlp"), None
            has = (lambda name: f"l{i}.{name}" in shapes) if shapes else (lambda name: True)
            if f is not None:
                if f.get("kind", "moe") != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
                r = f["router"]
                moe = MoeSpec(int(r["experts"]), int(r["top"]), int(f["expert"]["ff"]), 0.0, score="softmax_top",
                              weight_on="output", router_bias=has("mlp.router.b"))
                mlp = MlpSpec(ff=0, limit=0.0, kind="moe", moe=moe)
            if L["type"] == "attention":
                rot = m.get("rot") or {}
                sc = rot.get("scaling")
                mix = 0
                if m.get("v_mix"):
                    mix = 2 if first_vmix is not None else 1
                    first_vmix = i if first_vmix is None else first_vmix
                attn = AttnSpec(int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m.get("vdim", m["dim"])),
                                int(rot.get("dims", 0)), float(rot.get("base", 10000.0)), float(m["scale"]),
                                window=int((m.get("mask") or {}).get("size", 0)), head_norm=True, head_gain=True,
                                bias=has("mix.q.b"), v_bias=has("mix.v.b"), o_bias=has("mix.o.b"), gate=has("mix.g"),
                                gate_per_head=True, rot_half=True,
                                rot_scaling=(float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])) if sc else None,
                                v_norm=True, v_mix=mix, v_mix_tensor=has("mix.vmix") if shapes else mix == 2,
                                sink=has("mix.sink"))
                layers.append(LayerSpec("attention", i, attn=attn, mlp=mlp))
            elif L["type"] == "latent_attention":
                rot = m.get("rot") or {}
                if int(rot.get("dims", m["rot_dim"])) != int(m["rot_dim"]):
                    raise ValueError(f"layer {i}: the rotated part has {m['rot_dim']} channels but rot.dims = {rot.get('dims')}")
                lat = LatentAttnSpec(int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"]), 0,
                                     float(rot.get("base", 10000.0)), float(m["scale"]), sink=False,
                                     window=int((m.get("mask") or {}).get("size", 0)), interleaved=True, gate=has("mix.g"))
                layers.append(LayerSpec("latent_attention", i, latent=lat, mlp=mlp))
            elif L["type"] == "parallel":
                a, r = m["left"], m["right"]
                qt = a.get("q_temp") or {}
                attn = AttnSpec(int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"]), int(a.get("vdim", a["dim"])),
                                0, 10000.0, float(a["scale"]), softcap=float(a.get("softcap", 0.0)), gate=False,
                                weights="sigmoid", q_temp=(float(qt.get("coef", 0.0)), float(qt.get("every", 1.0))),
                                talking=has("mix.left.talk"))
                gd = GatedDeltaSpec(int(r["heads"]), int(r.get("kv_heads", r["heads"])), int(r["dim"]), int(r["vdim"]),
                                    int(r["conv"]))
                layers.append(LayerSpec("sigmoid_delta", i, attn=attn, gdelta=gd, left_scale=float(m["left_scale"]),
                                        right_scale=float(m["right_scale"]), mlp=mlp))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
        cfg = HybridConfig(int(d["vocab"]), int(d["width"]), float(d["norm"]["eps"]), 1.0, tuple(layers), block="post_ln",
                           skip_scale=float(d["postln_alpha"]), tied_head=True)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.norm_kind == "tanh":
            if not 1 <= self.streams <= 8 or any(L.kind not in ("latent", "delta") for L in self.layers):
                raise ValueError("the multi-stream program runs latent-attention and delta-rule layers over 1 to 8 streams")
            if self.pair_embed is not None and self.pair_embed[0] < 1:
                raise ValueError(f"bad token-pair table {self.pair_embed}")
        elif any(L.kind in ("latent", "delta") for L in self.layers):
            raise ValueError("latent-attention and delta-rule layers belong to the multi-stream program (norm_kind 'tanh')")
        post = ("attention", "latent_attention", "sigmoid_delta")
        if any((L.kind in post) != (self.block == "post_ln") for L in self.layers):
            raise ValueError(f"layers of the kinds {post} and no others run in the 'post_ln' block")
        mixing = [L.attn for L in self.layers if L.kind == "attention" and L.attn.v_mix]
        if mixing and (len({a.kv_heads * a.vdim for a in mixing}) != 1 or [a.v_mix for a in mixing] != [1] + [2] * (len(mixing) - 1)):
            raise ValueError("layers that blend their values have one value size; the first keeps its values, the others blend")
        for i, L in enumerate(self.layers):
            if L.kind in post:
                if L.mlp is not None and L.mlp.kind != "moe":
                    raise ValueError(f"layer run {i}: the 'post_ln' block has routed feed-forwards")
                if L.mlp is not None and not 1 <= L.mlp.moe.top <= L.mlp.moe.experts <= 1024:
                    raise ValueError(f"layer run {i}: bad router {L.mlp.moe}")
                if L.kind == "latent_attention":
                    a = L.latent
                    if (a.rot_dim % 2 or a.kv_rank > 512 or a.kv_rank + a.rot_dim > 1024 or min(a.heads, a.dim, a.vdim, a.kv_rank) < 1
                            or a.q_rank or a.window < 0):
                        raise ValueError(f"layer run {i}: bad latent-attention geometry {a} (kv_rank <= 512, even rot_dim)")
                    continue
                a = L.attn
                if a.heads % a.kv_heads or a.rot_dims % 2 or a.rot_dims > a.dim or a.dim > 1024 or a.vdim > 512 or a.window < 0:
                    raise ValueError(f"layer run {i}: bad attention geometry {a}")
                if L.kind == "sigmoid_delta":
                    g = L.gdelta
                    if g.heads % g.kv_heads or not 1 <= g.conv <= 16 or g.dim > 256 or min(g.dim, g.vdim) < 1:
                        raise ValueError(f"layer run {i}: bad gated-delta geometry {g}")
                continue
            if L.kind == "latent":
                a = L.latent
                if a.rot_dim % 2 or a.kv_rank > 512 or a.kv_rank + a.rot_dim > 1024 or min(a.heads, a.dim, a.vdim, a.q_rank) < 1:
                    raise ValueError(f"layer run {i}: bad latent-attention geometry {a} (kv_rank <= 512, even rot_dim)")
                if not L.hyper and self.streams != 1:
                    raise ValueError(f"layer run {i}: several streams need the layer's stream weights")
            elif L.kind == "delta":
                if L.delta.dim > 256 or L.delta.rank < 1:
                    raise ValueError(f"layer run {i}: bad delta-rule geometry {L.delta}")
                if not L.hyper and self.streams != 1:
                    raise ValueError(f"layer run {i}: several streams need the layer's stream weights")
            if L.kind == "mlstm":
                if L.mlstm.dim > 256 or L.mlstm.gate_cap < 0:
                    raise ValueError(f"layer run {i}: bad matrix-memory geometry {L.mlstm}")
            elif L.kind == "parallel_lin":
                a, r = L.attn, L.lin
                if a.heads % a.kv_heads or (a.value_is_key and a.vdim != a.dim) or a.dim > 512 or a.vdim > 256:
                    raise ValueError(f"layer run {i}: bad attention geometry {a}")
                if len(r.decay) != r.heads or r.dim > 256:
                    raise ValueError(f"layer run {i}: bad lightning-attention geometry {r}")
            if L.mlp is not None and L.mlp.kind == "moe" and not 1 <= L.mlp.moe.top <= L.mlp.moe.experts <= 1024:
                raise ValueError(f"layer run {i}: bad router {L.mlp.moe}")
            if L.kind in ("mlstm", "parallel_lin", "latent", "delta"):
                continue
            if L.kind == "parallel":
                a, s = L.attn, L.ssd
                if a.heads % a.kv_heads or a.rot_dims % 2 or a.rot_dims > a.dim:
                    raise ValueError(f"layer {i}: bad attention geometry {a}")
                if s.heads % s.groups or s.inner % s.norm_groups or s.conv < 1 or s.conv > 16:
                    raise ValueError(f"layer {i}: bad state-space geometry {s}")
                if a.dim > 512 or a.vdim > 256 or s.state > 256:
                    raise ValueError(f"layer {i}: head size beyond what the kernels are built for")
            elif L.gla.dim > 256:
                raise ValueError(f"layer {i}: key size beyond what the scan kernel is built for")

    # ---- the parameter arena: fused tensors in kernel order ---------------------------------------------------------
    def _own(self):
        """(tensor prefix index, spec) of every layer that has tensors of its own, in index order.  Runs that share
        tensors (weights_of) have the same sizes, so the first of them stands for all."""
        own: dict[int, LayerSpec] = {}
        for L in self.layers:
            own.setdefault(L.weights_of, L)
        return sorted(own.items())

    def fused_shapes(self) -> list[tuple[str, tuple[int, ...]]]:
        W, out = self.width, []
        for i, L in self._own():
            p = f"l{i}."
            if L.kind in ("latent", "delta"):
                out += [(name, shape) for name, shape, _ in self._stream_layer_tensors(i, L)]
                continue
            if self.block == "post_ln":
                out += [(name, shape) for name, shape, _ in self._postln_layer_tensors(i, L)]
                continue
            if L.kind == "gla":
                g = L.gla
                nq, nv = g.heads * g.dim, g.heads * g.vdim
                out += [(p + "mix.in", (2 * nq + 2 * nv + g.rank, W)), (p + "mix.a2", (nq, g.rank)),
                        (p + "mix.a2.b", (nq,)), (p + "mix.norm", (g.vdim,)), (p + "mix.o", (W, nv))]
            elif L.kind == "mlstm":
                m = L.mlstm
                nq, nv = m.heads * m.dim, m.heads * m.vdim
                out += [(p + "mix.in", (2 * nq + 2 * nv + 2 * m.heads, W)), (p + "mix.gate.b", (2 * m.heads,)),
                        (p + "mix.norm", (nv,)), (p + "mix.o", (W, nv))]
            elif L.kind == "parallel_lin":
                a, r = L.attn, L.lin
                nq, nk = a.heads * a.dim, a.kv_heads * a.dim
                rq, rv = r.heads * r.dim, r.heads * r.vdim
                out += [(p + "mix.in", (nq + nk + 2 * rq + 2 * rv, W)), (p + "mix.left.b", (nq + nk,)),
                        (p + "mix.left.o", (W, a.heads * a.vdim)), (p + "mix.right.norm", (rv,)),
                        (p + "mix.right.o", (W, rv)), (p + "mix.left.out", (W,)), (p + "mix.right.out", (W,))]
            else:
                a, s = L.attn, L.ssd
                nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
                ng = a.heads * a.vdim
                out += [(p + "mix.in", (nq + nk + nv + ng + s.in_rows, W)), (p + "mix.left.q.norm", (nq,)),
                        (p + "mix.left.k.norm", (nk,)), (p + "mix.left.o", (W, ng)),
                        (p + "mix.right.conv", (s.conv_channels, s.conv)), (p + "mix.right.conv.b", (s.conv_channels,)),
                        (p + "mix.right.dt_bias", (s.heads,)), (p + "mix.right.A_log", (s.heads,)),
                        (p + "mix.right.D", (s.heads,)), (p + "mix.right.norm", (s.inner,)),
                        (p + "mix.right.o", (W, s.inner))]
            out.append((p + "norm1", (W,)))
            if L.sandwich:
                out.append((p + "norm1b", (W,)))
            if L.mlp is not None:
                f = L.mlp
                if f.kind == "relu2":
                    out += [(p + "mlp.up", (f.ff, W)), (p + "mlp.down", (W, f.ff))]
                else:
                    if f.kind == "moe":
                        e = f.moe
                        out += [(p + "mlp.router", (e.experts, W)), (p + "mlp.experts.gate_up", (e.experts * 2 * e.ff, W)),
                                (p + "mlp.experts.down", (e.experts * W, e.ff))]
                    if f.ff > 0:
                        out += [(p + "mlp.gate_up", (2 * f.ff, W)), (p + "mlp.down", (W, f.ff))]
                out.append((p + "norm2", (W,)))
                if L.sandwich:
                    out.append((p + "norm2b", (W,)))
        if self.loop_times:
            out += [("loop.in", (W, 2 * W)), ("loop.step", (self.loop_times, W))]
        out += [("embed", (self.vocab_size, W)), ("final.norm", (W,))]
        if not self.tied_head:
            out.append(("head", (self.vocab_size, W)))
        if self.norm_kind == "tanh":
            out += [("final.norm.b", (W,)), ("final.norm.alpha", (1,))]
        if self.pair_embed is not None:
            out.append(("bigram", (self.pair_embed[0] + 1, W)))
        return out

    def _stream_layer_tensors(self, i: int, L: LayerSpec) -> list:
        """(fused tensor, shape, [(checkpoint tensor, rows)] in row order) of a latent-attention or delta-rule layer.
        The sublayer gate's projection rides in the mixer's input projection (one GEMM over the same input)."""
        W, S, p, out = self.width, self.streams, f"l{i}.", []
        one = lambda name, shape: out.append((p + name, shape, [(p + name, shape[0])]))
        gate = [(p + "rg1", W)] if L.gated else []
        if L.kind == "latent":
            a = L.latent
            parts = [(p + "mix.dq", a.q_rank), (p + "mix.dkv", a.kv_rank + a.rot_dim)] + gate
            out.append((p + "mix.in", (sum(n for _, n in parts), W), parts))
            one("mix.dq.norm", (a.q_rank,)); one("mix.dkv.norm", (a.kv_rank,))
            one("mix.uq", (a.heads * (a.dim + a.rot_dim), a.q_rank)); one("mix.uk", (a.heads * a.dim, a.kv_rank))
            one("mix.uv", (a.heads * a.vdim, a.kv_rank))
            if a.sink:
                one("mix.sink", (a.heads,))
            one("mix.o", (W, a.heads * a.vdim))
        else:
            c = L.delta
            nq = c.heads * c.dim
            parts = [(p + "mix.r", nq), (p + "mix.k", nq), (p + "mix.v", nq), (p + "mix.g", nq), (p + "mix.a", nq),
                     (p + "mix.w1", c.rank)] + gate
            out.append((p + "mix.in", (sum(n for _, n in parts), W), parts))
            one("mix.a.b", (nq,)); one("mix.w2", (nq, c.rank)); one("mix.w0", (nq,)); one("mix.norm", (nq,))
            one("mix.o", (W, nq))
        for q in ("1", "2") if L.mlp is not None else ("1",):
            one("norm" + q, (W,)); one(f"norm{q}.b", (W,)); one(f"norm{q}.alpha", (1,))
            if L.layer_scale:
                one("ls" + q, (W,))
            if L.gated:
                one(f"rg{q}.b", (W,))
            if L.hyper:
                one(f"hc{q}.in", (S,)); one(f"hc{q}.out", (S,)); one(f"hc{q}.mix", (S, S))
        if L.mlp is not None:
            e = L.mlp.moe
            one("mlp.router", (e.experts, W))
            out.append((p + "mlp.experts.gate_up", (e.experts * 2 * e.ff, W),
                        [(f"{p}mlp.e{k}.{part}", e.ff) for k in range(e.experts) for part in ("gate", "up")]))
            out.append((p + "mlp.experts.down", (e.experts * W, e.ff), [(f"{p}mlp.e{k}.down", W) for k in range(e.experts)]))
            if L.gated:
                one("rg2", (W, W))
        return out

    def _postln_layer_tensors(self, i: int, L: LayerSpec) -> list:
        """(fused tensor, shape, [(checkpoint tensor, rows)] in row order) of a layer of the 'post_ln' block.  All
        projections that read the layer's input are ONE fused tensor `mix.in` (both mixers of a parallel layer, gates
        included), the biases of its rows one vector."""
        W, p, out = self.width, f"l{i}.", []
        one = lambda name, shape: out.append((p + name, shape, [(p + name, shape[0])]))
        if L.kind == "attention":
            a = L.attn
            nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
            parts = [(p + "mix.q", nq), (p + "mix.k", nk), (p + "mix.v", nv)] + ([(p + "mix.g", a.heads)] if a.gate else [])
            out.append((p + "mix.in", (sum(n for _, n in parts), W), parts))
            if a.bias:
                out.append((p + "mix.qk.b", (nq + nk,), [(p + "mix.q.b", nq), (p + "mix.k.b", nk)]))
            if a.v_bias:
                one("mix.v.b", (nv,))
            if a.head_gain:
                one("mix.q.norm", (a.dim,)); one("mix.k.norm", (a.dim,))
            if a.v_mix_tensor or a.v_mix == 2:
                one("mix.vmix", (1,))
            if a.sink:
                one("mix.sink", (a.heads,))
            one("mix.o", (W, a.heads * a.vdim))
            if a.o_bias:
                one("mix.o.b", (W,))
        elif L.kind == "latent_attention":
            a = L.latent
            parts = [(p + "mix.q", a.heads * (a.dim + a.rot_dim)), (p + "mix.dkv", a.kv_rank + a.rot_dim)]
            parts += [(p + "mix.g", a.heads * a.vdim)] if a.gate else []
            out.append((p + "mix.in", (sum(n for _, n in parts), W), parts))
            one("mix.dkv.norm", (a.kv_rank,)); one("mix.uk", (a.heads * a.dim, a.kv_rank))
            one("mix.uv", (a.heads * a.vdim, a.kv_rank)); one("mix.o", (W, a.heads * a.vdim))
        else:
            a, g = L.attn, L.gdelta
            nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
            gq, gv = g.kv_heads * g.dim, g.heads * g.vdim
            parts = [(p + "mix.left.q", nq), (p + "mix.left.k", nk), (p + "mix.left.v", nv), (p + "mix.right.q", gq),
                     (p + "mix.right.k", gq), (p + "mix.right.v", gv), (p + "mix.right.b", g.heads), (p + "mix.right.a", g.heads),
                     (p + "mix.right.g", gv)]
            out.append((p + "mix.in", (sum(n for _, n in parts), W), parts))
            one("mix.left.q.norm", (nq,)); one("mix.left.k.norm", (nk,)); one("mix.left.pb", (a.heads,))
            if a.talking:
                one("mix.left.talk", (a.heads, a.heads))
            one("mix.left.o", (W, a.heads * a.vdim))
            out.append((p + "mix.right.conv", (g.conv_channels, g.conv),
                        [(p + "mix.right.q.conv", gq), (p + "mix.right.k.conv", gq), (p + "mix.right.v.conv", gv)]))
            one("mix.right.A_log", (g.heads,)); one("mix.right.dt_bias", (g.heads,)); one("mix.right.norm", (g.vdim,))
            one("mix.right.o", (W, gv))
        one("norm1", (W,))
        if L.mlp is not None:
            e = L.mlp.moe
            one("mlp.router", (e.experts, W))
            if e.router_bias:
                one("mlp.router.b", (e.experts,))
            out.append((p + "mlp.experts.gate_up", (e.experts * 2 * e.ff, W),
                        [(f"{p}mlp.e{k}.{part}", e.ff) for k in range(e.experts) for part in ("gate", "up")]))
            out.append((p + "mlp.experts.down", (e.experts * W, e.ff), [(f"{p}mlp.e{k}.down", W) for k in range(e.experts)]))
            one("norm2", (W,))
        return out

    def checkpoint_slices(self) -> dict[str, tuple[str, int, int]]:
        """checkpoint tensor name -> (fused tensor, first row, rows)."""
        m: dict[str, tuple[str, int, int]] = {}

        def rows(fused, parts):
            at = 0
            for name, n in parts:
                m[name] = (fused, at, n)
                at += n
        for i, L in self._own():
            p = f"l{i}."
            if L.kind in ("latent", "delta"):
                for fused, _, parts in self._stream_layer_tensors(i, L):
                    rows(fused, parts)
                continue
            if self.block == "post_ln":
                for fused, _, parts in self._postln_layer_tensors(i, L):
                    rows(fused, parts)
                continue
            if L.kind == "gla":
                g = L.gla
                nq, nv = g.heads * g.dim, g.heads * g.vdim
                rows(p + "mix.in", [(p + "mix.q", nq), (p + "mix.k", nq), (p + "mix.v", nv), (p + "mix.g", nv),
                                    (p + "mix.a1", g.rank)])
                for name, n in (("mix.a2", nq), ("mix.a2.b", nq), ("mix.norm", g.vdim), ("mix.o", self.width)):
                    m[p + name] = (p + name, 0, n)
            elif L.kind == "mlstm":
                c = L.mlstm
                nq, nv = c.heads * c.dim, c.heads * c.vdim
                rows(p + "mix.in", [(p + "mix.q", nq), (p + "mix.k", nq), (p + "mix.v", nv), (p + "mix.g", nv),
                                    (p + "mix.i", c.heads), (p + "mix.f", c.heads)])
                rows(p + "mix.gate.b", [(p + "mix.i.b", c.heads), (p + "mix.f.b", c.heads)])
                m[p + "mix.norm"] = (p + "mix.norm", 0, nv)
                m[p + "mix.o"] = (p + "mix.o", 0, self.width)
            elif L.kind == "parallel_lin":
                a, r = L.attn, L.lin
                nq, nk = a.heads * a.dim, a.kv_heads * a.dim
                rq, rv = r.heads * r.dim, r.heads * r.vdim
                rows(p + "mix.in", [(p + "mix.left.q", nq), (p + "mix.left.k", nk), (p + "mix.right.q", rq),
                                    (p + "mix.right.k", rq), (p + "mix.right.v", rv), (p + "mix.right.g", rv)])
                rows(p + "mix.left.b", [(p + "mix.left.q.b", nq), (p + "mix.left.k.b", nk)])
                for name, n in (("mix.left.o", self.width), ("mix.right.norm", rv), ("mix.right.o", self.width),
                                ("mix.left.out", self.width), ("mix.right.out", self.width)):
                    m[p + name] = (p + name, 0, n)
            else:
                a, s = L.attn, L.ssd
                nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
                rows(p + "mix.in", [(p + "mix.left.q", nq), (p + "mix.left.k", nk), (p + "mix.left.v", nv),
                                    (p + "mix.left.g", a.heads * a.vdim), (p + "mix.right.in", s.in_rows)])
                for name, n in (("mix.left.q.norm", nq), ("mix.left.k.norm", nk), ("mix.left.o", self.width),
                                ("mix.right.conv", s.conv_channels), ("mix.right.conv.b", s.conv_channels),
                                ("mix.right.dt_bias", s.heads), ("mix.right.A_log", s.heads), ("mix.right.D", s.heads),
                                ("mix.right.norm", s.inner), ("mix.right.o", self.width)):
                    m[p + name] = (p + name, 0, n)
            m[p + "norm1"] = (p + "norm1", 0, self.width)
            if L.sandwich:
                m[p + "norm1b"] = (p + "norm1b", 0, self.width)
            if L.mlp is not None:
                f = L.mlp
                if f.kind == "relu2":
                    m[p + "mlp.up"] = (p + "mlp.up", 0, f.ff)
                    m[p + "mlp.down"] = (p + "mlp.down", 0, self.width)
                elif f.kind == "moe":
                    e = f.moe
                    m[p + "mlp.router"] = (p + "mlp.router", 0, e.experts)
                    for k in range(e.experts):
                        m[f"{p}mlp.e{k}.gate"] = (p + "mlp.experts.gate_up", k * 2 * e.ff, e.ff)
                        m[f"{p}mlp.e{k}.up"] = (p + "mlp.experts.gate_up", k * 2 * e.ff + e.ff, e.ff)
                        m[f"{p}mlp.e{k}.down"] = (p + "mlp.experts.down", k * self.width, self.width)
                    if f.ff > 0:
                        rows(p + "mlp.gate_up", [(p + "mlp.shared.gate", f.ff), (p + "mlp.shared.up", f.ff)])
                        m[p + "mlp.shared.down"] = (p + "mlp.down", 0, self.width)
                else:
                    rows(p + "mlp.gate_up", [(p + "mlp.gate", f.ff), (p + "mlp.up", f.ff)])
                    m[p + "mlp.down"] = (p + "mlp.down", 0, self.width)
                m[p + "norm2"] = (p + "norm2", 0, self.width)
                if L.sandwich:
                    m[p + "norm2b"] = (p + "norm2b", 0, self.width)
        if self.loop_times:
            m["loop.in"] = ("loop.in", 0, self.width)
            m["loop.step"] = ("loop.step", 0, self.loop_times)
        m["embed"] = ("embed", 0, self.vocab_size)
        m["final.norm"] = ("final.norm", 0, self.width)
        if not self.tied_head:
            m["head"] = ("head", 0, self.vocab_size)
        if self.norm_kind == "tanh":
            m["final.norm.b"] = ("final.norm.b", 0, self.width)
            m["final.norm.alpha"] = ("final.norm.alpha", 0, 1)
        if self.pair_embed is not None:
            m["bigram"] = ("bigram", 0, self.pair_embed[0] + 1)
        return m

    def init_param(self, name: str, view: torch.Tensor, gen: torch.Generator) -> None:
        """Random initialisation for benches and tests: unit gains, small biases, weights of std 1/sqrt(fan_in)."""
        leaf = name.split(".")[-1]
        if ".hc1." in name or ".hc2." in name:        # read every stream equally, write to all, keep each stream
            view.copy_(torch.eye(self.streams) if leaf == "mix" else
                       torch.full(view.shape, 1.0 / self.streams if leaf == "in" else 1.0))
        elif leaf == "alpha":
            view.fill_(0.5)
        elif leaf == "vmix":
            view.fill_(0.5)
        elif leaf == "talk":
            view.copy_((torch.eye(view.shape[0], device=view.device)
                        + 0.1 * torch.randn(view.shape, generator=gen, device=view.device)).to(view.dtype))
        elif leaf in ("ls1", "ls2"):
            view.fill_(1.0)
        elif leaf in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm":
            view.fill_(1.0 - self.norm_offset)
        elif leaf in ("norm", "out"):
            view.fill_(1.0)
        elif name == "loop.step":
            view.copy_((torch.randn(view.shape, generator=gen, device=view.device) * 0.1).to(view.dtype))
        elif leaf == "A_log":
            view.copy_(torch.log(torch.linspace(1.0, 4.0, view.numel())).to(view.dtype))
        elif leaf in ("D",):
            view.fill_(1.0)
        elif leaf in ("b", "dt_bias"):
            view.copy_((torch.randn(view.shape, generator=gen, device=view.device) * 0.1).to(view.dtype))
        else:
            fan_in = view.shape[-1] if view.dim() > 1 else 1
            std = 0.02 if name == "embed" else 1.0 / math.sqrt(fan_in)
            flat = view.view(-1)
            step = 1 << 26
            for s in range(0, flat.numel(), step):
                n = min(step, flat.numel() - s)
                flat[s:s + n] = (torch.randn(n, generator=gen, device=view.device, dtype=torch.float32) * std).to(view.dtype)

    def num_params(self) -> int:
        n = 0
        for _, shape in self.fused_shapes():
            k = 1
            for s in shape:
                k *= s
            n += k
        return n


def rotary_table(dims: int, base: float, scaling: tuple | None = None):
    """(frequencies of the dims / 2 rotated pairs, factor on cos and sin).  Plain: base^(-2i/dims), factor 1.  With YaRN
    scaling (factor, original length, fast turns, slow turns): pairs that complete more than `fast` turns over the
    original length keep their frequency, those below `slow` turns are divided by `factor`, a linear ramp over the pair
    index in between; cos and sin are multiplied by 0.1 ln(factor) + 1."""
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling or not half:
        return f, 1.0
    factor, orig, fast, slow = scaling
    at = lambda turns: dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo, hi = max(math.floor(at(fast)), 0), min(math.ceil(at(slow)), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


class _Rows:
    """Activation buffers and ragged-row metadata for up to `n` rows."""

    def __init__(self, eng: "HybridEngine", n: int, pieces: bool = False):
        cfg, d, T = eng.cfg, eng.dev, eng.op_dtype
        W = cfg.width
        wide_p, wide_aux, wide_o, wide_o2, wide_q, wide_f = W, 1, 1, 1, 1, 1
        wide_gate, moe_pairs, moe_ff, moe_experts = 0, 0, 1, 1     # mLSTM gate heads; routed pairs per row, expert width
        wide_vfirst, wide_prep = 0, 0                               # values kept for later layers; gated-delta vectors
        for L in cfg.layers:
            if L.kind == "attention":
                a = L.attn
                nq = a.heads * a.dim
                wide_p = max(wide_p, nq + a.kv_heads * (a.dim + a.vdim) + a.heads)
                wide_q, wide_o = max(wide_q, nq), max(wide_o, a.heads * a.vdim)
                if a.v_mix:
                    wide_vfirst = max(wide_vfirst, a.kv_heads * a.vdim)
            elif L.kind == "latent_attention":
                a = L.latent               # buffer roles: see HybridEngine._latent_direct_mixer
                wide_p = max(wide_p, a.heads * (a.dim + a.rot_dim) + a.kv_rank + a.rot_dim + a.heads * a.vdim)
                wide_o = max(wide_o, a.heads * a.kv_rank, a.heads * a.vdim)
                wide_o2 = max(wide_o2, a.heads * a.dim, a.heads * a.vdim)
                wide_q = max(wide_q, a.heads * (a.kv_rank + a.rot_dim))
            elif L.kind == "sigmoid_delta":
                a, g = L.attn, L.gdelta
                nq = a.heads * a.dim
                wide_p = max(wide_p, nq + a.kv_heads * (a.dim + a.vdim) + g.in_rows)
                wide_q, wide_aux = max(wide_q, nq), max(wide_aux, g.conv_channels)
                wide_o = max(wide_o, a.heads * a.vdim, g.heads * g.vdim)
                wide_o2 = max(wide_o2, g.heads * g.vdim)
                wide_prep = max(wide_prep, 5 * g.heads * g.dim)
            elif L.kind == "gla":
                g = L.gla
                nq, nv = g.heads * g.dim, g.heads * g.vdim
                wide_p = max(wide_p, 2 * nq + 2 * nv + g.rank)
                wide_aux, wide_o = max(wide_aux, nq), max(wide_o, nv)
            elif L.kind == "mlstm":
                m = L.mlstm
                nq, nv = m.heads * m.dim, m.heads * m.vdim
                wide_p = max(wide_p, 2 * nq + 2 * nv + 2 * m.heads)
                wide_aux = max(wide_aux, m.heads * (m.vdim + 1))
                wide_o = max(wide_o, m.heads * (m.vdim + 1))
                wide_gate = max(wide_gate, m.heads)
            elif L.kind == "parallel_lin":
                a, r = L.attn, L.lin
                nq = a.heads * a.dim
                wide_p = max(wide_p, nq + a.kv_heads * a.dim + 2 * r.heads * (r.dim + r.vdim))
                wide_o, wide_q = max(wide_o, a.heads * a.vdim), max(wide_q, nq)
                wide_o2 = max(wide_o2, r.heads * r.vdim)
            elif L.kind == "latent":
                a = L.latent               # buffer roles: see HybridEngine._latent_mixer
                wide_p = max(wide_p, a.q_rank + a.kv_rank + a.rot_dim + (W if L.gated else 0))
                wide_aux = max(wide_aux, a.heads * (a.dim + a.rot_dim))
                wide_o = max(wide_o, a.heads * a.kv_rank, a.heads * a.vdim, a.q_rank)
                wide_o2 = max(wide_o2, a.heads * a.dim, a.heads * a.vdim)
                wide_q = max(wide_q, a.heads * (a.kv_rank + a.rot_dim))
            elif L.kind == "delta":
                c = L.delta
                nq = c.heads * c.dim
                wide_p = max(wide_p, 5 * nq + c.rank + (W if L.gated else 0))
                wide_aux, wide_o, wide_o2 = max(wide_aux, nq), max(wide_o, nq), max(wide_o2, nq)
            else:
                a, s = L.attn, L.ssd
                nq = a.heads * a.dim
                wide_p = max(wide_p, nq + a.kv_heads * (a.dim + a.vdim) + a.heads * a.vdim + s.in_rows)
                wide_aux, wide_o = max(wide_aux, s.conv_channels), max(wide_o, a.heads * a.vdim)
                wide_o2, wide_q = max(wide_o2, s.inner), max(wide_q, nq)
            if L.mlp is not None:
                wide_p, wide_f = max(wide_p, 2 * L.mlp.ff), max(wide_f, max(L.mlp.ff, 1))
                if L.mlp.kind == "moe":
                    e = L.mlp.moe
                    wide_p = max(wide_p, e.top * 2 * e.ff)
                    moe_pairs, moe_ff, moe_experts = max(moe_pairs, e.top), max(moe_ff, e.ff), max(moe_experts, e.experts)
        f32 = dict(dtype=torch.float32, device=d)
        i32 = dict(dtype=torch.int32, device=d)
        self.n = n
        self.x = torch.zeros(n * W, **f32)                      # the residual stream
        if cfg.norm_kind == "tanh":                             # ... or its parallel streams [row][stream][W]
            self.xs = torch.zeros(n * cfg.streams * W, **f32)
        self.xa = torch.zeros(n * W, dtype=T, device=d)         # its copy in the GEMM operand type
        self.P = torch.zeros(n * wide_p, **f32)                 # projection output of the current sublayer
        self.aux = torch.zeros(n * wide_aux, **f32)             # decay logits (GLA) / convolved x, B, C (state-space)
        self.o = torch.zeros(n * wide_o, **f32)                 # raw mixer output (GLA, attention)
        self.o2 = torch.zeros(n * wide_o2, **f32)               # raw state-space output
        self.ob = torch.zeros(n * wide_o if any(eng.tc_attn.values()) else 1, dtype=torch.bfloat16, device=d)  # tcgen05 attention out
        self.ya = torch.zeros(n * wide_o, dtype=T, device=d)    # gated / normed input of the output projection
        self.yb = torch.zeros(n * wide_o2, dtype=T, device=d)
        ny = max(n, 16 * min(n, 128)) * W                       # up to 16 split-K slices of a <= 128-row projection
        self.y0 = torch.zeros(ny, **f32)
        self.y1 = torch.zeros(ny, **f32)
        self.q = torch.zeros(n * wide_q, dtype=T, device=d)
        self.act = torch.zeros(n * wide_f, dtype=T, device=d)
        if wide_vfirst:                                         # the first value-blending layer's values of the batch's rows
            self.vfirst = torch.zeros(n * wide_vfirst, **f32)
        if wide_prep:                                           # u | a u | w | k | r of the gated delta rule
            self.dprep = torch.zeros(n * wide_prep, **f32)
        if cfg.loop_times:                                      # the embedding output and [x | x0], operand type
            self.x0a = torch.zeros(n * W, dtype=T, device=d)
            self.xcat = torch.zeros(n * 2 * W, dtype=T, device=d)
        if wide_gate:                                           # mLSTM: (keep, take) per head and token, exp(-m)
            self.gates = torch.zeros(n * 2 * wide_gate, **f32)
            self.minv = torch.zeros(n * wide_gate, **f32)
        if moe_pairs:                                           # routed feed-forward: pairs = choices x rows
            pairs = n * moe_pairs
            self.router = torch.zeros(n * moe_experts, **f32)
            self.sel = torch.zeros(pairs, **i32)
            self.wsel = torch.zeros(pairs, **f32)
            self.perm = torch.zeros(pairs, **i32)
            self.moe_meta = torch.zeros(4, **i32)
            self.moe_tiles = torch.zeros(3 * int(eng.lib.prl_moe_max_tiles(pairs, moe_experts)), **i32)
            self.moe_act = torch.zeros(pairs * moe_ff, dtype=T, device=d)
            self.moe_out = torch.zeros(pairs * W, **f32)        # [choice][row][W]: summed by the sublayer's closing kernel
        self.tokens = torch.zeros(n, **i32)
        self.row_pos = torch.zeros(n, **i32)
        self.row_slot = torch.zeros(n, **i32)
        self.row_back = torch.zeros(n, **i32)
        self.seg = torch.zeros(4, n, **i32)                     # seg_start, seg_len, seg_pos0, seg_slot
        self.want = torch.zeros(n, **i32)
        # side-by-side pieces of long segments (prompt portions only): piece tables, a scratch state and a decay
        # table per piece, sized for the largest recurrence of the model
        self.n_sub, self.max_sub = 0, 0
        if pieces:
            lib, st, dc = eng.lib, 1, 1
            for L in cfg.layers:
                for heads, dk, dv in eng.scan_geometry(L):
                    st = max(st, int(lib.prl_lin_scan_state_floats(heads, dk, dv)))
                    dc = max(dc, int(lib.prl_lin_scan_piece_decay_floats(heads, dk)))
            self.max_sub = n // eng.piece_tokens + 8
            self.scratch = torch.zeros(self.max_sub * st, **f32)
            self.cdec = torch.zeros(self.max_sub * dc, **f32)
            self.sub = torch.zeros(2, self.max_sub, **i32)          # sub_start, sub_len
            self.seg_sub = torch.zeros(2, n, **i32)                 # first piece, piece count of every segment


class HybridEngine(EngineCore):
    recurrent = True

    def __init__(self, cfg: HybridConfig, arena, **kw):
        self.f32 = arena.data.dtype == torch.float32
        self.op_dtype = arena.data.dtype
        if self.op_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("the hybrid engine runs bf16 or fp32 weights")
        self.force_plain_gemm = False      # tests: route every GEMM through the CUDA-core kernel
        self.unfused_glu = False           # tests: gate_up GEMM + activation kernel instead of the GEMM's gated epilogue
        self.force_plain_attn = False      # tests: the any-geometry attention kernel also where the tcgen05 ones fit
        self.unfused_router = False        # tests: router logits through the GEMM and a separate choice kernel
        # Long prompt portions run their recurrences as side-by-side pieces (prl_*_scan_split): same values up to fp32
        # rounding, many times the parallelism.  Off in the true-fp32 mode, whose results do not depend on the cut of
        # a prompt bit for bit.  A batch qualifies when its longest segment has split_min_rows rows.
        self.split_scan = not self.f32
        self.split_min_rows = 256
        self.piece_tokens = 64             # tokens per piece (tests lower it); at most prl_lin_scan_piece_tokens()
        self._rows: _Rows | None = None
        super().__init__(cfg, arena, **kw)

    # ---- caches, states, derived parameters ---------------------------------------------------------------------------
    def _alloc_model(self) -> None:
        cfg, d, lib = self.cfg, self.dev, self.lib
        self.k_pool, self.v_pool, self.conv_state, self.ssd_state, self.gla_state, self.rot_freq = {}, {}, {}, {}, {}, {}
        self.tc_attn: dict[int, bool] = {}
        self.lin_state, self.lin_decay, self.mlstm_state, self.mlstm_m = {}, {}, {}, {}
        self.lat_pool, self.delta_state = {}, {}
        self._head_tables: dict = {}
        if cfg.pair_embed is not None:                   # the last token of the sequence's previous portion
            self.prev_token = self.states.add("prev_token", (1,), dtype=torch.int32)
        self.rot_mag: dict[int, float] = {}
        for i, L in enumerate(cfg.layers):               # one cache / state per layer RUN, also where weights are shared
            if L.kind in ("attention", "sigmoid_delta"):
                a = L.attn
                self.k_pool[i] = torch.zeros(self.n_pages, a.kv_heads, PAGE_SIZE, a.dim, dtype=self.op_dtype, device=d)
                self.v_pool[i] = torch.zeros(self.n_pages, a.kv_heads, PAGE_SIZE, a.vdim, dtype=self.op_dtype, device=d)
                self.tc_attn[i] = False
                f, self.rot_mag[i] = rotary_table(a.rot_dims, a.rot_base, a.rot_scaling)
                self.rot_freq[i] = torch.tensor(f or [0.0], dtype=torch.float64, device=d)
                if L.kind == "sigmoid_delta":
                    g = L.gdelta
                    self.conv_state[i] = self.states.add(f"l{i}.conv", (g.conv_channels, max(g.conv - 1, 1)))
                    n = int(lib.prl_delta_state_floats(g.heads, g.dim, g.vdim))
                    self.delta_state[i] = self.states.add(f"l{i}.delta", (n,))
            elif L.kind in ("latent", "latent_attention"):
                a = L.latent                             # one row per token: [latent | rotated shared key part]
                self.lat_pool[i] = torch.zeros(self.n_pages, PAGE_SIZE, a.kv_rank + a.rot_dim, dtype=self.op_dtype, device=d)
                f = [a.rot_base ** (-2.0 * k / a.rot_dim) for k in range(a.rot_dim // 2)] or [0.0]
                self.rot_freq[i] = torch.tensor(f, dtype=torch.float64, device=d)
            elif L.kind == "delta":
                c = L.delta
                n = int(lib.prl_delta_state_floats(c.heads, c.dim, c.dim))
                self.delta_state[i] = self.states.add(f"l{i}.delta", (n,))
            elif L.kind == "gla":
                g = L.gla
                n = int(lib.prl_lin_scan_state_floats(g.heads, g.dim, g.vdim))
                self.gla_state[i] = self.states.add(f"l{i}.gla", (n,))
            elif L.kind == "mlstm":
                m = L.mlstm                              # matrix memory with the normaliser as one more value column, and m
                n = int(lib.prl_lin_scan_state_floats(m.heads, m.dim, m.vdim + 1))
                self.mlstm_state[i] = self.states.add(f"l{i}.mlstm", (n,))
                self.mlstm_m[i] = self.states.add(f"l{i}.mlstm.m", (m.heads,))
            elif L.kind == "parallel_lin":
                a, r = L.attn, L.lin
                pair = torch.zeros(2, self.n_pages, a.kv_heads, PAGE_SIZE, a.dim, dtype=self.op_dtype, device=d)
                if a.dim == a.vdim:
                    self.k_pool[i], self.v_pool[i] = pair[0], pair[1]
                else:
                    self.k_pool[i] = pair[0]
                    self.v_pool[i] = torch.zeros(self.n_pages, a.kv_heads, PAGE_SIZE, a.vdim, dtype=self.op_dtype, device=d)
                self.tc_attn[i] = False                  # window, kept first tokens and capped scores: the any-geometry kernel
                n = int(lib.prl_lin_scan_state_floats(r.heads, r.dim, r.vdim))
                self.lin_state[i] = self.states.add(f"l{i}.lin", (n,))
                self.lin_decay[i] = torch.tensor(r.decay, dtype=torch.float32, device=d)
            else:
                a, s = L.attn, L.ssd
                if a.dim == a.vdim:    # K and V pools adjacent: [2][page][kv head][64][d], the layout of the Qwen2 engine's pool
                    pair = torch.zeros(2, self.n_pages, a.kv_heads, PAGE_SIZE, a.dim, dtype=self.op_dtype, device=d)
                    self.k_pool[i], self.v_pool[i] = pair[0], pair[1]
                else:
                    self.k_pool[i] = torch.zeros(self.n_pages, a.kv_heads, PAGE_SIZE, a.dim, dtype=self.op_dtype, device=d)
                    self.v_pool[i] = torch.zeros(self.n_pages, a.kv_heads, PAGE_SIZE, a.vdim, dtype=self.op_dtype, device=d)
                # head size 128 in bf16 is what the tcgen05 chunked-prefill kernel and the TMA paged-decode kernel are built
                # for: such a layer runs the SAME attention kernels as the Qwen2 engine (with this layer's own scale)
                self.tc_attn[i] = (not self.f32 and a.dim == 128 and a.vdim == 128
                                   and a.heads // a.kv_heads in (1, 2, 4, 8, 16))
                self.conv_state[i] = self.states.add(f"l{i}.conv", (s.conv_channels, max(s.conv - 1, 1)))
                n = int(lib.prl_lin_scan_state_floats(s.heads, s.state, s.vdim))
                self.ssd_state[i] = self.states.add(f"l{i}.ssd", (n,))
                half = a.rot_dims // 2
                f = [a.rot_base ** (-2.0 * k / a.rot_dims) for k in range(half)] or [0.0]
                self.rot_freq[i] = torch.tensor(f, dtype=torch.float64, device=d)
        # fp32 copies of the small parameter vectors (gains, biases, taps, per-head constants): exact for bf16 weights
        self.vec: dict[str, torch.Tensor] = {}
        for name, shape in cfg.fused_shapes():
            if (len(shape) == 1 or name.endswith("mix.right.conv") or name.endswith("mix.left.talk") or name == "loop.step"
                    or name.endswith(".mix") and ".hc" in name):
                self.vec[name] = torch.zeros(shape, dtype=torch.float32, device=d)
        # per-head transposes W_uk,h^T [kv_rank, dim] of the latent layers' key expansion (operand type): the B operand
        # of the product that absorbs the expansion into the query.  Refreshed with the small vectors on a weight flip.
        self.uk_t = {L.weights_of: torch.zeros(L.latent.heads, L.latent.kv_rank, L.latent.dim, dtype=self.op_dtype, device=d)
                     for L in cfg.layers if L.latent is not None}
        if cfg.norm_kind == "tanh":                      # stream weights of layers without their own: the plain residual sum
            S = cfg.streams
            self.stream_ones = torch.ones(S, dtype=torch.float32, device=d)
            self.stream_eye = torch.eye(S, dtype=torch.float32, device=d)
        conv_ch = max([L.gdelta.conv_channels for L in cfg.layers if L.gdelta is not None], default=0)
        if conv_ch:                                      # the short convolutions of the gated delta rule have no bias
            self.zero_bias = torch.zeros(conv_ch, dtype=torch.float32, device=d)
        if cfg.positions == "sinusoid":
            W = cfg.width
            self.pos_freq = torch.tensor([10000.0 ** (-2.0 * k / W) for k in range((W + 1) // 2)], dtype=torch.float64, device=d)
        self._on_arena_change()
        B = self.B
        self.attn_splits, ws = {}, 0
        for i, on in self.tc_attn.items():
            if on:
                a = cfg.layers[i].attn
                self.attn_splits[i] = int(lib.prl_paged_attn_splits(B, a.kv_heads, self.max_seq_len))
                ws = max(ws, int(lib.prl_paged_attn_workspace_bytes(B, a.heads, self.attn_splits[i])))
        for L in cfg.layers:                              # latent attention: the key splits' shares of a batch of single tokens
            if L.latent is not None:
                for n_seg in range(1, max(B, 4) + 1):     # the split count falls as the batch grows; the product need not
                    ws = max(ws, int(lib.prl_attn_latent_workspace_bytes(n_seg, L.latent.heads, L.latent.kv_rank)))
            elif L.kind == "sigmoid_delta" and not self.f32:
                # attention without a softmax: the shares of CTAs that split a row tile's keys.  A decode step of up to B
                # single tokens; a packed batch never needs more than 8 shares of <= 16 rows per SM-filling unit
                a = L.attn
                for n_seg in range(1, max(B, 4) + 1):
                    ws = max(ws, int(lib.prl_attn_sigmoid_workspace_bytes(n_seg, n_seg, 1, a.heads, a.vdim)))
                ws = max(ws, 16 * 160 * a.heads * a.vdim * 4)
        self.attn_ws = torch.zeros(max(ws, 16), dtype=torch.uint8, device=d)
        self._dec = _Rows(self, B)
        i32 = dict(dtype=torch.int32, device=d)
        self._dec.seg[0].copy_(torch.arange(B, **i32))
        self._dec.seg[3].copy_(torch.arange(B, **i32))

    def _on_arena_change(self) -> None:
        cfg = self.cfg
        for name, t in self.vec.items():
            t.copy_(self.arena.view(name).float())
            if name == "final.norm" or name.split(".")[-1] in ("norm1", "norm1b", "norm2", "norm2b"):
                if cfg.norm_offset:
                    t.add_(cfg.norm_offset)              # gains stored as offsets
        if cfg.logit_scale != 1.0:
            self.vec["final.norm"].mul_(cfg.logit_scale)   # logits = head(norm(x)) * scale: folded into the last gain
        for j, t in self.uk_t.items():
            H, r, dm = t.shape
            t.copy_(self.arena.view(f"l{j}.mix.uk").view(H, dm, r).transpose(1, 2))

    @property
    def head_name(self) -> str:
        return "embed" if self.cfg.tied_head else "head"

    @staticmethod
    def scan_geometry(L) -> list:
        """(heads, key size, value columns) of every matrix-state recurrence of a layer."""
        if L.kind == "gla":
            return [(L.gla.heads, L.gla.dim, L.gla.vdim)]
        if L.kind == "mlstm":
            return [(L.mlstm.heads, L.mlstm.dim, L.mlstm.vdim + 1)]
        if L.kind == "parallel_lin":
            return [(L.lin.heads, L.lin.dim, L.lin.vdim)]
        if L.kind in ("latent", "delta", "attention", "latent_attention", "sigmoid_delta"):
            return []                      # the delta rules have a scan of their own (delta_scan.cu), walked token by token
        return [(L.ssd.heads, L.ssd.state, L.ssd.vdim)]

    def kv_bytes_per_token(self) -> int:
        e = 4 if self.f32 else 2
        return (sum(L.attn.kv_heads * (L.attn.dim + L.attn.vdim) * e for L in self.cfg.layers if L.attn is not None)
                + sum((L.latent.kv_rank + L.latent.rot_dim) * e for L in self.cfg.layers if L.latent is not None))

    # ---- GEMM dispatch ------------------------------------------------------------------------------------------------
    def _mm(self, src: torch.Tensor, K: int, w_name: str, N: int, out: torch.Tensor, n: int, split: bool = False) -> int:
        """out[n, N] (fp32) = src[n, K] @ W[N, K]^T.  bf16 with TMA-expressible sizes: the tcgen05 kernels (weight-
        streaming swap-AB for n <= 128 rows, persistent CTA-pair kernel above); otherwise the CUDA-core kernel.
        `split`: the consumer sums split-K slices (prl_postnorm_residual), so a small-N projection of a decode step may
        spread its K range over the SMs; returns the number of slices written ([slices][n][N])."""
        lib, st, wp = self.lib, self._st, self.arena.ptr(w_name)
        if self.f32 or self.force_plain_gemm or K % 8 or K < 64:
            _lib.check(lib.prl_gemm_any(src.data_ptr(), int(self.f32), K, wp, int(self.f32), K, n, N, K,
                                        out.data_ptr(), N, st))
        elif n <= 128:
            k = int(lib.prl_gemm_auto_split_k(n, N, K)) if split else 1
            _lib.check(lib.prl_gemm_bf16_splitk(wp, None, src.data_ptr(), n, N, K, k, out.data_ptr(), st))
            return k
        else:
            _lib.check(lib.prl_gemm_tn(src.data_ptr(), K, wp, K, n, N, K, out.data_ptr(), N, 1, 0, None, None, 0, 1.0, st))
        return 1

    # ---- the layer program over n ragged rows -------------------------------------------------------------------------
    def _layers(self, R: _Rows, n: int, ns: int, max_q: int, row_pos: torch.Tensor, seg_pos0: torch.Tensor,
                trace=None, decode: bool = False) -> None:
        cfg, lib, st, f32 = self.cfg, self.lib, self._st, int(self.f32)
        if cfg.norm_kind == "tanh":
            return self._stream_layers(R, n, ns, max_q, row_pos, seg_pos0, trace)
        if cfg.block == "post_ln":
            return self._postln_layers(R, n, ns, max_q, row_pos, seg_pos0, trace)
        W, eps, vec = cfg.width, cfg.eps, self.vec
        seg_start, seg_len, seg_slot = R.seg[0].data_ptr(), R.seg[1].data_ptr(), R.seg[3].data_ptr()
        P, x, xa = R.P.data_ptr(), R.x.data_ptr(), R.xa.data_ptr()
        n_sub = 0 if decode else R.n_sub
        if n_sub:
            pieces = (R.seg_sub[0].data_ptr(), R.seg_sub[1].data_ptr(), R.sub[0].data_ptr(), R.sub[1].data_ptr(), n_sub,
                      R.scratch.data_ptr(), R.cdec.data_ptr())
        segs = (seg_start, seg_len, seg_slot, ns)
        for i, L in enumerate(cfg.layers):
            w = f"l{L.weights_of}."
            if L.opens_pass is not None:
                # a pass of the repeated block opens: x <- W_loop [x; x0] + step[pass], then the first layer's input norm
                _lib.check(lib.prl_concat_rows(xa, R.x0a.data_ptr(), n, W, R.xcat.data_ptr(), f32, st))
                k0 = self._mm(R.xcat, 2 * W, "loop.in", W, R.y0, n, split=True)
                self._close(R, n, R.y0, k0, bias=vec["loop.step"][L.opens_pass], add=False, next_gain=self._pre_gain(i))
            elif i == 0 and L.sandwich:
                _lib.check(lib.prl_rmsnorm_rows(x, None, vec[w + "norm1"].data_ptr(), eps, n, W, xa, f32, st))
            if L.kind == "mlstm":
                self._mlstm_mixer(R, n, i, L, w, segs, pieces if n_sub else None)
            elif L.kind == "parallel_lin":
                self._attn_lightning_mixer(R, n, i, L, w, segs, pieces if n_sub else None, max_q, row_pos, seg_pos0)
            elif L.kind == "gla":
                g = L.gla
                nq, nv = g.heads * g.dim, g.heads * g.vdim
                ld = 2 * nq + 2 * nv + g.rank
                self._mm(R.xa, W, w + "mix.in", ld, R.P, n)                       # [q | k | v | g | a1]
                # decay logits z = W_a2 (W_a1 h): the bottleneck stays fp32 (A operand read from P as stored)
                _lib.check(lib.prl_gemm_any(P + 4 * (2 * nq + 2 * nv), 1, ld, self.arena.ptr(w + "mix.a2"), f32, g.rank,
                                            n, nq, g.rank, R.aux.data_ptr(), nq, st))
                _lib.check(lib.prl_gla_decay(R.aux.data_ptr(), nq, vec[w + "mix.a2.b"].data_ptr(), g.tau, n, nq, st))
                if n_sub:
                    _lib.check(lib.prl_gla_scan_split(P, ld, 0, nq, 2 * nq, g.dim ** -0.5, R.aux.data_ptr(), nq, g.heads, g.dim,
                                                      g.vdim, seg_slot, ns, *pieces, self.gla_state[i].data_ptr(),
                                                      R.o.data_ptr(), nv, st))
                else:
                    _lib.check(lib.prl_gla_scan(P, ld, 0, nq, 2 * nq, g.dim ** -0.5, R.aux.data_ptr(), nq, g.heads, g.dim,
                                                g.vdim, seg_start, seg_len, seg_slot, ns, self.gla_state[i].data_ptr(),
                                                R.o.data_ptr(), nv, st))
                _lib.check(lib.prl_gate_norm(R.o.data_ptr(), 1, nv, P + 4 * (2 * nq + nv), ld, vec[w + "mix.norm"].data_ptr(),
                                             g.vdim, g.vdim, n, nv, 0, 0, 1, eps, R.ya.data_ptr(), f32, st))
                k0 = self._mm(R.ya, nv, w + "mix.o", W, R.y0, n, split=True)
                _lib.check(lib.prl_postnorm_residual(R.y0.data_ptr(), W, 1.0, k0, None, 0, 0.0, 1, vec[w + "norm1"].data_ptr(),
                                                     eps, n, W, x, xa, f32, st))
            else:
                a, s = L.attn, L.ssd
                nq, nk, nvk, ng = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim, a.heads * a.vdim
                left = nq + nk + nvk + ng
                ld = left + s.in_rows
                self._mm(R.xa, W, w + "mix.in", ld, R.P, n)                       # [q | k | v | g || z | x B C | dt]
                # -- left: softmax attention over the paged cache
                _lib.check(lib.prl_qk_norm_rope_cache(P, ld, 0, nq, nq + nk, n, a.heads, a.kv_heads, a.dim, a.vdim,
                                                      a.rot_dims, self.rot_freq[i].data_ptr(),
                                                      vec[w + "mix.left.q.norm"].data_ptr(),
                                                      vec[w + "mix.left.k.norm"].data_ptr(), eps, row_pos.data_ptr(),
                                                      R.row_slot.data_ptr(), self.block_table.data_ptr(), self.max_blocks,
                                                      PAGE_SIZE, R.q.data_ptr(), self.k_pool[i].data_ptr(),
                                                      self.v_pool[i].data_ptr(), f32, st))
                if self.tc_attn[i] and not self.force_plain_attn:
                    kv = self.k_pool[i].data_ptr()       # K pool, V pool right behind it (one "layer" of the Qwen2 pool layout)
                    if decode:
                        _lib.check(lib.prl_paged_attn_decode(R.q.data_ptr(), kv, self.n_pages, 1, 0, self.block_table.data_ptr(),
                                                             self.max_blocks, self.seq_lens.data_ptr(), n, a.heads, a.kv_heads,
                                                             a.dim, PAGE_SIZE, self.attn_splits[i], a.scale, R.ob.data_ptr(),
                                                             self.attn_ws.data_ptr(), self.attn_ws.numel(), st))
                    else:
                        _lib.check(lib.prl_paged_attn_prefill_tc(R.q.data_ptr(), n, kv, self.n_pages, 1, 0,
                                                                 self.block_table.data_ptr(), self.max_blocks, seg_start,
                                                                 seg_len, seg_pos0.data_ptr(), seg_slot, ns, max_q, a.heads,
                                                                 a.kv_heads, a.dim, PAGE_SIZE, a.scale, R.ob.data_ptr(), st))
                    o_ptr, o_f32 = R.ob.data_ptr(), 0
                else:
                    _lib.check(lib.prl_attn_any(R.q.data_ptr(), self.k_pool[i].data_ptr(), self.v_pool[i].data_ptr(), f32,
                                                self.block_table.data_ptr(), self.max_blocks, PAGE_SIZE, seg_start, seg_len,
                                                seg_pos0.data_ptr(), seg_slot, ns, max_q, a.heads, a.kv_heads, a.dim, a.vdim,
                                                a.scale, R.o.data_ptr(), st))
                    o_ptr, o_f32 = R.o.data_ptr(), 1
                _lib.check(lib.prl_gate_norm(o_ptr, o_f32, ng, P + 4 * (nq + nk + nvk), ld, None, 1, ng, n, ng, 1, 0, 0,
                                             eps, R.ya.data_ptr(), f32, st))
                k0 = self._mm(R.ya, ng, w + "mix.left.o", W, R.y0, n, split=True)
                # -- right: state-space mixer
                inner, ch = s.inner, s.conv_channels
                conv_w, conv_b = vec[w + "mix.right.conv"].data_ptr(), vec[w + "mix.right.conv.b"].data_ptr()
                _lib.check(lib.prl_conv_silu(P, ld, left + inner, n, ch, s.conv, conv_w, conv_b, R.row_slot.data_ptr(),
                                             R.row_back.data_ptr(), self.conv_state[i].data_ptr(), R.aux.data_ptr(), st))
                _lib.check(lib.prl_conv_state_update(P, ld, left + inner, ch, s.conv, seg_start, seg_len, seg_slot, ns,
                                                     self.conv_state[i].data_ptr(), st))
                ssd_vec = (vec[w + "mix.right.dt_bias"].data_ptr(), vec[w + "mix.right.A_log"].data_ptr(),
                           vec[w + "mix.right.D"].data_ptr())
                if n_sub:
                    _lib.check(lib.prl_ssd_scan_split(P, ld, left + inner + ch, R.aux.data_ptr(), ch, *ssd_vec, s.heads,
                                                      s.groups, s.state, s.vdim, seg_slot, ns, *pieces,
                                                      self.ssd_state[i].data_ptr(), R.o2.data_ptr(), inner, st))
                else:
                    _lib.check(lib.prl_ssd_scan(P, ld, left + inner + ch, R.aux.data_ptr(), ch, *ssd_vec, s.heads, s.groups,
                                                s.state, s.vdim, seg_start, seg_len, seg_slot, ns,
                                                self.ssd_state[i].data_ptr(), R.o2.data_ptr(), inner, st))
                _lib.check(lib.prl_gate_norm(R.o2.data_ptr(), 1, inner, P + 4 * left, ld, vec[w + "mix.right.norm"].data_ptr(),
                                             inner, inner // s.norm_groups, n, inner, 0, 1, 1, eps, R.yb.data_ptr(), f32, st))
                k1 = self._mm(R.yb, inner, w + "mix.right.o", W, R.y1, n, split=True)
                _lib.check(lib.prl_postnorm_residual(R.y0.data_ptr(), W, L.left_scale, k0, R.y1.data_ptr(), W, L.right_scale, k1,
                                                     vec[w + "norm1"].data_ptr(), eps, n, W, x, xa, f32, st))
            if L.mlp is not None:
                f = L.mlp
                k0 = 0
                if f.kind == "relu2":
                    self._mm(R.xa, W, w + "mlp.up", f.ff, R.P, n)
                    _lib.check(lib.prl_act_store(P, f.ff, n, f.ff, 0, R.act.data_ptr(), f32, st))
                    k0 = self._mm(R.act, f.ff, w + "mlp.down", W, R.y0, n, split=True)
                elif f.ff > 0:
                    k0 = self._glu_ff(R, n, w, f)
                routed = self._routed_ff(R, n, w, f.moe, f.beta) if f.kind == "moe" else None
                if L.sandwich:
                    y, ky = (R.y0, k0) if k0 else (routed, f.moe.top)
                    y1, k1 = (routed, f.moe.top) if (k0 and routed is not None) else (None, 1)
                    self._close(R, n, y, ky, y1=y1, k1=k1, post_gain=vec[w + "norm2b"], next_gain=self._next_gain(i, False))
                else:
                    _lib.check(lib.prl_postnorm_residual(R.y0.data_ptr(), W, 1.0, k0, None, 0, 0.0, 1, vec[w + "norm2"].data_ptr(),
                                                         eps, n, W, x, xa, f32, st))
            if trace is not None:
                trace.append(R.x[:n * W].view(n, W).clone())

    # ---- pieces of the layer program shared by several layer kinds ------------------------------------------------------
    def _pre_gain(self, i: int):
        """Gain of the norm in front of run i's mixer (None: the mixer reads x as it is)."""
        L = self.cfg.layers[i]
        return self.vec[f"l{L.weights_of}.norm1"] if L.sandwich else None

    def _next_gain(self, i: int, after_mixer: bool):
        """Gain of the input norm of whatever reads x after this sublayer of run i: the run's feed-forward, the next
        run's mixer, or nothing (the opening of a pass and the model's last norm read x itself)."""
        L = self.cfg.layers[i]
        if after_mixer and L.mlp is not None:
            return self.vec[f"l{L.weights_of}.norm2"] if L.sandwich else None
        if i + 1 < len(self.cfg.layers) and self.cfg.layers[i + 1].opens_pass is None:
            return self._pre_gain(i + 1)
        return None

    def _close(self, R, n, y0, k0, gain0=None, s0=1.0, y1=None, k1=1, gain1=None, s1=1.0, post_gain=None, bias=None,
               add=True, next_gain=None) -> None:
        """prl_sublayer_close on the residual stream: branch norms, sum, output norm, residual, the next input norm."""
        W = self.cfg.width
        ptr = lambda t: None if t is None else t.data_ptr()
        _lib.check(self.lib.prl_sublayer_close(y0.data_ptr(), W, k0, ptr(gain0), s0, ptr(y1), W, k1, ptr(gain1), s1,
                                               ptr(post_gain), ptr(bias), int(add), ptr(next_gain), self.cfg.eps, n, W,
                                               R.x.data_ptr(), R.xa.data_ptr(), int(self.f32), self._st))

    def _glu_ff(self, R, n, w, f) -> int:
        """Clamped gated unit l<w>.mlp.gate_up / .down on xa; returns the number of split-K slices left in R.y0."""
        lib, st, W, F, f32 = self.lib, self._st, self.cfg.width, f.ff, int(self.f32)
        xa, P = R.xa.data_ptr(), R.P.data_ptr()
        tc = not (self.f32 or self.force_plain_gemm or W % 8 or W < 64 or self.unfused_glu)
        if tc and n <= 128 and F % 64 == 0:
            # the clamped gate in the gate_up GEMM's epilogue (the Qwen2 step's SwiGLU-epilogue kernel): no [n, 2F] tile
            _lib.check(lib.prl_gemm_glu_clamped_decode(self.arena.ptr(w + "mlp.gate_up"), xa, n, F, W, f.limit, f.beta,
                                                       R.act.data_ptr(), st))
        elif tc and n > 128 and F % 128 == 0:
            _lib.check(lib.prl_gemm_glu_clamped_f32(xa, W, self.arena.ptr(w + "mlp.gate_up"), W, n, F, W, f.limit, f.beta,
                                                    R.act.data_ptr(), F, st))
        else:
            self._mm(R.xa, W, w + "mlp.gate_up", 2 * F, R.P, n)
            _lib.check(lib.prl_glu_clamped(P, 2 * F, n, F, f.limit, f.beta, R.act.data_ptr(), f32, st))
        return self._mm(R.act, F, w + "mlp.down", W, R.y0, n, split=True)

    def _routed_ff(self, R, n, w, e, beta) -> torch.Tensor:
        """Routed experts on xa: fp32 router logits, top-k with sigmoid weights, pairs grouped by expert on the device,
        two grouped GEMMs around the gated activation.  Returns [top][n][W] fp32 (R.moe_out), to be summed by the caller."""
        lib, st, W, f32 = self.lib, self._st, self.cfg.width, int(self.f32)
        pairs = n * e.top
        route = (R.sel.data_ptr(), R.wsel.data_ptr(), R.perm.data_ptr(), R.moe_meta.data_ptr(), R.moe_tiles.data_ptr(), st)
        # weights: sigmoid of the chosen logit | softmax over the chosen | softmax over all experts
        mode = {"sigmoid": 0, "softmax_top": 1, "softmax_all": 2}[e.score]
        bias = self.vec[w + "mlp.router.b"].data_ptr() if e.router_bias else None
        if (W + e.experts) * 4 <= 160 * 1024 and not self.unfused_router:
            _lib.check(lib.prl_moe_router(R.xa.data_ptr(), f32, self.arena.ptr(w + "mlp.router"), f32, bias, n, W, e.experts, e.top,
                                          mode, *route))
        else:
            _lib.check(lib.prl_gemm_any(R.xa.data_ptr(), f32, W, self.arena.ptr(w + "mlp.router"), f32, W, n, e.experts, W,
                                        R.router.data_ptr(), e.experts, st))
            _lib.check(lib.prl_moe_route(R.router.data_ptr(), e.experts, bias, n, e.experts, e.top, mode, *route))
        tiles = int(lib.prl_moe_max_tiles(pairs, e.experts))
        table = (R.perm.data_ptr(), R.moe_meta.data_ptr(), R.moe_tiles.data_ptr(), tiles)
        _lib.check(lib.prl_moe_gemm(R.xa.data_ptr(), f32, W, n, self.arena.ptr(w + "mlp.experts.gate_up"), f32,
                                    2 * e.ff * W, W, *table, 2 * e.ff, W, R.P.data_ptr(), 2 * e.ff, 0, st))
        if e.weight_on == "output":      # plain SiLU unit, the score (times a constant) on the expert's output
            _lib.check(lib.prl_moe_glu_out(R.P.data_ptr(), 2 * e.ff, pairs, e.ff, R.perm.data_ptr(), R.wsel.data_ptr(),
                                           e.weight_scale, R.moe_act.data_ptr(), f32, st))
        else:
            _lib.check(lib.prl_moe_glu(R.P.data_ptr(), 2 * e.ff, pairs, e.ff, R.perm.data_ptr(), R.wsel.data_ptr(), e.limit, beta,
                                       R.moe_act.data_ptr(), f32, st))
        _lib.check(lib.prl_moe_gemm(R.moe_act.data_ptr(), f32, e.ff, 0, self.arena.ptr(w + "mlp.experts.down"), f32,
                                    W * e.ff, e.ff, *table, W, e.ff, R.moe_out.data_ptr(), W, 1, st))
        return R.moe_out

    def _mlstm_mixer(self, R, n, i, L, w, segs, pieces) -> None:
        """Matrix-memory LSTM: one projection [q | k | v | g | i | f]; the gates' running maximum is walked first (fp32),
        which turns the cell into S <- keep S + take k v^T, the recurrence prl_decay_scan runs; the normaliser rides along
        as one more value column (v with a one appended)."""
        c, lib, st, vec, f32, W = L.mlstm, self.lib, self._st, self.vec, int(self.f32), self.cfg.width
        H, nq, nv = c.heads, c.heads * c.dim, c.heads * c.vdim
        ld, P = 2 * nq + 2 * nv + 2 * H, R.P.data_ptr()
        seg_start, seg_len, seg_slot, ns = segs
        self._mm(R.xa, W, w + "mix.in", ld, R.P, n)
        gb = vec[w + "mix.gate.b"].data_ptr()
        _lib.check(lib.prl_mlstm_gates(P, ld, 2 * nq + 2 * nv, 2 * nq + 2 * nv + H, gb, gb + 4 * H, c.gate_cap, H, seg_start,
                                       seg_len, seg_slot, ns, self.mlstm_m[i].data_ptr(), R.gates.data_ptr(),
                                       R.minv.data_ptr(), st))
        _lib.check(lib.prl_append_one(P, ld, 2 * nq, n, H, c.vdim, R.aux.data_ptr(), st))
        dv = c.vdim + 1
        head = (P, ld, 0, nq, c.dim ** -0.5, R.aux.data_ptr(), H * dv, 0, R.gates.data_ptr(), 2 * H, 0, None, H, c.dim, dv)
        if pieces is not None:
            _lib.check(lib.prl_decay_scan_split(*head, seg_slot, ns, *pieces, self.mlstm_state[i].data_ptr(), R.o.data_ptr(),
                                                H * dv, st))
        else:
            _lib.check(lib.prl_decay_scan(*head, seg_start, seg_len, seg_slot, ns, self.mlstm_state[i].data_ptr(),
                                          R.o.data_ptr(), H * dv, st))
        _lib.check(lib.prl_mlstm_out(R.o.data_ptr(), n, H, c.vdim, R.minv.data_ptr(), c.den_eps, P + 4 * (2 * nq + nv), ld,
                                     vec[w + "mix.norm"].data_ptr(), self.cfg.eps, R.ya.data_ptr(), f32, st))
        k0 = self._mm(R.ya, nv, w + "mix.o", W, R.y0, n, split=True)
        self._close(R, n, R.y0, k0, post_gain=vec[w + "norm1b"] if L.sandwich else vec[w + "norm1"],
                    next_gain=self._next_gain(i, True))

    def _attn_lightning_mixer(self, R, n, i, L, w, segs, pieces, max_q, row_pos, seg_pos0) -> None:
        """Softmax attention (values = keys, per-head unit norms, capped scores, window + kept first tokens) beside
        lightning attention, both from ONE projection [q | k || q | k | v | g]; each branch is normed over the width
        with its own gain before the two are averaged."""
        a, r, lib, st, vec, f32, W = L.attn, L.lin, self.lib, self._st, self.vec, int(self.f32), self.cfg.width
        eps = self.cfg.eps
        nq, nk, no = a.heads * a.dim, a.kv_heads * a.dim, a.heads * a.vdim
        rq, rv = r.heads * r.dim, r.heads * r.vdim
        ld, P = nq + nk + 2 * rq + 2 * rv, R.P.data_ptr()
        seg_start, seg_len, seg_slot, ns = segs
        self._mm(R.xa, W, w + "mix.in", ld, R.P, n)
        # -- left
        qb = vec[w + "mix.left.b"].data_ptr()
        _lib.check(lib.prl_qk_headnorm_cache(P, ld, 0, nq, -1, n, a.heads, a.kv_heads, a.dim, a.vdim, qb, qb + 4 * nq, None,
                                             None, eps, row_pos.data_ptr(), R.row_slot.data_ptr(),
                                             self.block_table.data_ptr(), self.max_blocks, PAGE_SIZE, R.q.data_ptr(),
                                             self.k_pool[i].data_ptr(), self.v_pool[i].data_ptr(), f32, st))
        _lib.check(lib.prl_attn_any_masked(R.q.data_ptr(), self.k_pool[i].data_ptr(), self.v_pool[i].data_ptr(), f32,
                                           self.block_table.data_ptr(), self.max_blocks, PAGE_SIZE, seg_start, seg_len,
                                           seg_pos0.data_ptr(), seg_slot, ns, max_q, a.heads, a.kv_heads, a.dim, a.vdim,
                                           a.scale, a.window, a.keep_first, a.softcap, 1, R.ya.data_ptr(), st))
        k0 = self._mm(R.ya, no, w + "mix.left.o", W, R.y0, n, split=True)
        # -- right
        off = nq + nk
        _lib.check(lib.prl_act_cols(P, ld, off, n, 2 * rq + rv, 0, st))            # SiLU on q, k, v
        head = (P, ld, off, off + rq, 1.0, P, ld, off + 2 * rq, None, 0, 0, self.lin_decay[i].data_ptr(), r.heads, r.dim, r.vdim)
        if pieces is not None:
            _lib.check(lib.prl_decay_scan_split(*head, seg_slot, ns, *pieces, self.lin_state[i].data_ptr(), R.o2.data_ptr(),
                                                rv, st))
        else:
            _lib.check(lib.prl_decay_scan(*head, seg_start, seg_len, seg_slot, ns, self.lin_state[i].data_ptr(),
                                          R.o2.data_ptr(), rv, st))
        _lib.check(lib.prl_gate_norm(R.o2.data_ptr(), 1, rv, P + 4 * (off + 2 * rq + rv), ld, vec[w + "mix.right.norm"].data_ptr(),
                                     rv, rv, n, rv, 1, 0, 1, eps, R.yb.data_ptr(), f32, st))
        k1 = self._mm(R.yb, rv, w + "mix.right.o", W, R.y1, n, split=True)
        self._close(R, n, R.y0, k0, gain0=vec[w + "mix.left.out"], s0=L.left_scale, y1=R.y1, k1=k1,
                    gain1=vec[w + "mix.right.out"], s1=L.right_scale,
                    post_gain=vec[w + "norm1b"] if L.sandwich else vec[w + "norm1"], next_gain=self._next_gain(i, True))

    # ---- the 'post_ln' block: every sublayer is normed after the sum, x <- norm(skip_scale x + f(x)), f reads x ----------
    def _postln_close(self, R, n, w, q, y0, k0, s0=1.0, y1=None, k1=1, s1=1.0, bias=None) -> None:
        """x <- rmsnorm(skip_scale x + s0 y0 + s1 y1 + bias) * norm<q>, and its copy in the operand type."""
        cfg, ptr = self.cfg, (lambda t: None if t is None else t.data_ptr())
        _lib.check(self.lib.prl_postln_close(y0.data_ptr(), cfg.width, s0, k0, ptr(y1), cfg.width, s1, k1, ptr(bias),
                                             cfg.skip_scale, self.vec[w + "norm" + q].data_ptr(), cfg.eps, n, cfg.width,
                                             R.x.data_ptr(), R.xa.data_ptr(), int(self.f32), self._st))

    def _postln_layers(self, R, n, ns, max_q, row_pos, seg_pos0, trace=None) -> None:
        cfg, vec = self.cfg, self.vec
        segs = (R.seg[0].data_ptr(), R.seg[1].data_ptr(), R.seg[3].data_ptr(), ns)
        for i, L in enumerate(cfg.layers):
            w = f"l{L.weights_of}."
            if L.kind == "attention":
                k0 = self._window_attn_mixer(R, n, i, L, w, segs, max_q, row_pos, seg_pos0)
                self._postln_close(R, n, w, "1", R.y0, k0, bias=vec[w + "mix.o.b"] if L.attn.o_bias else None)
            elif L.kind == "latent_attention":
                k0 = self._latent_direct_mixer(R, n, i, L, w, segs, max_q, row_pos, seg_pos0)
                self._postln_close(R, n, w, "1", R.y0, k0)
            else:
                k0, k1 = self._sigmoid_delta_mixer(R, n, i, L, w, segs, max_q, row_pos, seg_pos0)
                self._postln_close(R, n, w, "1", R.y0, k0, s0=L.left_scale, y1=R.y1, k1=k1, s1=L.right_scale)
            if L.mlp is not None:
                y = self._routed_ff(R, n, w, L.mlp.moe, L.mlp.beta)
                self._postln_close(R, n, w, "2", y, L.mlp.moe.top)
            if trace is not None:
                trace.append(R.x[:n * cfg.width].view(n, cfg.width).clone())

    def _window_attn_mixer(self, R, n, i, L, w, segs, max_q, row_pos, seg_pos0) -> int:
        """Softmax attention with biased projections, per-head norms with a shared gain, scaled rotate-half rotary,
        unit-RMS values blended with an earlier layer's, a sliding window, a sink logit and one gate per head, from ONE
        projection [q | k | v | g].  Returns the number of split-K slices of the output projection left in R.y0."""
        a, lib, st, vec, f32, W = L.attn, self.lib, self._st, self.vec, int(self.f32), self.cfg.width
        seg_start, seg_len, seg_slot, ns = segs
        nq, nk, nv, no = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim, a.heads * a.vdim
        ld, P = nq + nk + nv + (a.heads if a.gate else 0), R.P.data_ptr()
        self._mm(R.xa, W, w + "mix.in", ld, R.P, n)
        qb = vec[w + "mix.qk.b"].data_ptr() if a.bias else None
        gain = (vec[w + "mix.q.norm"].data_ptr(), vec[w + "mix.k.norm"].data_ptr()) if a.head_gain else (None, None)
        _lib.check(lib.prl_attn_front(P, ld, 0, nq, nq + nk, n, a.heads, a.kv_heads, a.dim, a.vdim, qb,
                                      qb + 4 * nq if a.bias else None, vec[w + "mix.v.b"].data_ptr() if a.v_bias else None,
                                      int(a.head_norm), *gain, a.dim, self.cfg.eps, a.rot_dims, self.rot_freq[i].data_ptr(),
                                      self.rot_mag[i], int(a.v_norm), a.v_mix,
                                      vec[w + "mix.vmix"].data_ptr() if a.v_mix == 2 else None,
                                      R.vfirst.data_ptr() if a.v_mix else None, row_pos.data_ptr(), R.row_slot.data_ptr(),
                                      self.block_table.data_ptr(), self.max_blocks, PAGE_SIZE, R.q.data_ptr(),
                                      self.k_pool[i].data_ptr(), self.v_pool[i].data_ptr(), f32, st))
        sink = vec[w + "mix.sink"].data_ptr() if a.sink else None
        gated = a.gate and a.gate_per_head
        _lib.check(lib.prl_attn_any_sink(R.q.data_ptr(), self.k_pool[i].data_ptr(), self.v_pool[i].data_ptr(), a.vdim, f32,
                                         self.block_table.data_ptr(), self.max_blocks, PAGE_SIZE, seg_start, seg_len,
                                         seg_pos0.data_ptr(), seg_slot, ns, max_q, a.heads, a.kv_heads, a.dim, a.vdim, a.scale,
                                         a.window, 0, a.softcap, sink, 0 if gated else 1,
                                         R.o.data_ptr() if gated else R.ya.data_ptr(), st))
        if gated:
            _lib.check(lib.prl_gate_heads(R.o.data_ptr(), 1, no, P + 4 * (nq + nk + nv), ld, n, a.heads, a.vdim, R.ya.data_ptr(),
                                          f32, st))
        return self._mm(R.ya, no, w + "mix.o", W, R.y0, n, split=True)

    def _latent_direct_mixer(self, R, n, i, L, w, segs, max_q, row_pos, seg_pos0) -> int:
        """Latent attention whose query comes straight from the layer's input: ONE projection [q | dkv | g].  As in
        _latent_mixer the key expansion is absorbed into the query and the value expansion follows the attention, so
        the cache holds [latent | rotated shared key part] per token.  Buffers: yb = the heads' unrotated query parts,
        later the gated values (operand type); q = the attention query [n][H][kv_rank + rot_dim]; ya = the attention
        output over the latent (operand type); o = scratch of the per-head products, then the expanded values (fp32)."""
        a, lib, st, vec, f32, W = L.latent, self.lib, self._st, self.vec, int(self.f32), self.cfg.width
        seg_start, seg_len, seg_slot, ns = segs
        H, rk, dr, dv = a.heads, a.kv_rank, a.rot_dim, a.vdim
        hq, kd = H * (a.dim + dr), rk + dr
        ld, P = hq + kd + (H * dv if a.gate else 0), R.P.data_ptr()
        il = int(a.interleaved)
        self._mm(R.xa, W, w + "mix.in", ld, R.P, n)
        _lib.check(lib.prl_latent_prep(P, ld, 0, 0, hq, rk, dr, self.rot_freq[i].data_ptr(), None,
                                       vec[w + "mix.dkv.norm"].data_ptr(), self.cfg.eps, row_pos.data_ptr(),
                                       R.row_slot.data_ptr(), self.block_table.data_ptr(), self.max_blocks, PAGE_SIZE, n, il,
                                       None, self.lat_pool[i].data_ptr(), f32, st))
        _lib.check(lib.prl_latent_query(P, ld, n, H, a.dim, dr, rk, self.rot_freq[i].data_ptr(), row_pos.data_ptr(), il,
                                        R.yb.data_ptr(), R.q.data_ptr(), f32, st))
        self._mm_heads(R.yb, a.dim, self.uk_t[L.weights_of].data_ptr(), rk * a.dim, n, rk, R.o, H, R.q, kd)
        self._latent_attention(R, i, a, segs, max_q, seg_pos0, None)
        if a.gate:       # v[h] = W_uv,h o_lat[h] in fp32, times sigmoid(g) element by element
            self._mm_heads(R.ya, rk, self.arena.ptr(w + "mix.uv"), dv * rk, n, dv, R.o, H, None, 0, store=False)
            _lib.check(lib.prl_gate_norm(R.o.data_ptr(), 1, H * dv, P + 4 * (hq + kd), ld, None, 1, H * dv, n, H * dv, 1, 0, 0,
                                         self.cfg.eps, R.yb.data_ptr(), f32, st))
        else:
            self._mm_heads(R.ya, rk, self.arena.ptr(w + "mix.uv"), dv * rk, n, dv, R.o, H, R.yb, dv)
        return self._mm(R.yb, H * dv, w + "mix.o", W, R.y0, n, split=True)

    def _sigmoid_delta_mixer(self, R, n, i, L, w, segs, max_q, row_pos, seg_pos0):
        """Attention without a softmax beside the gated delta rule, both from ONE projection
        [q | k | v || q | k | v | b | a | g].  Returns the split-K slice counts of the two output projections
        (R.y0, R.y1); the caller's closing kernel adds them with the layer's two scales."""
        a, g, lib, st, vec, f32, W = L.attn, L.gdelta, self.lib, self._st, self.vec, int(self.f32), self.cfg.width
        seg_start, seg_len, seg_slot, ns = segs
        nq, nk, nv, no = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim, a.heads * a.vdim
        left = nq + nk + nv
        ld, P = left + g.in_rows, R.P.data_ptr()
        self._mm(R.xa, W, w + "mix.in", ld, R.P, n)
        # -- left: one RMS norm over all heads of q (and of k), no rotation; the temperature is folded into the score scale
        _lib.check(lib.prl_qk_norm_rope_cache(P, ld, 0, nq, nq + nk, n, a.heads, a.kv_heads, a.dim, a.vdim, 0,
                                              self.rot_freq[i].data_ptr(), vec[w + "mix.left.q.norm"].data_ptr(),
                                              vec[w + "mix.left.k.norm"].data_ptr(), self.cfg.eps, row_pos.data_ptr(),
                                              R.row_slot.data_ptr(), self.block_table.data_ptr(), self.max_blocks, PAGE_SIZE,
                                              R.q.data_ptr(), self.k_pool[i].data_ptr(), self.v_pool[i].data_ptr(), f32, st))
        _lib.check(lib.prl_attn_sigmoid(R.q.data_ptr(), self.k_pool[i].data_ptr(), self.v_pool[i].data_ptr(), f32,
                                        self.block_table.data_ptr(), self.max_blocks, PAGE_SIZE, seg_start, seg_len,
                                        seg_pos0.data_ptr(), seg_slot, ns, max_q, a.heads, a.kv_heads, a.dim, a.vdim, a.scale,
                                        a.softcap, a.q_temp[0], a.q_temp[1], vec[w + "mix.left.pb"].data_ptr(),
                                        vec[w + "mix.left.talk"].data_ptr() if a.talking else None, 1, R.ya.data_ptr(), n,
                                        int(not self.force_plain_attn), self.attn_ws.data_ptr(), self.attn_ws.numel(), st))
        k0 = self._mm(R.ya, no, w + "mix.left.o", W, R.y0, n, split=True)
        # -- right: convolutions + SiLU over [q | k | v], then the scan
        gq, gv, ch = g.kv_heads * g.dim, g.heads * g.vdim, g.conv_channels
        _lib.check(lib.prl_conv_silu(P, ld, left, n, ch, g.conv, vec[w + "mix.right.conv"].data_ptr(), self.zero_bias.data_ptr(),
                                     R.row_slot.data_ptr(), R.row_back.data_ptr(), self.conv_state[i].data_ptr(),
                                     R.aux.data_ptr(), st))
        _lib.check(lib.prl_conv_state_update(P, ld, left, ch, g.conv, seg_start, seg_len, seg_slot, ns,
                                             self.conv_state[i].data_ptr(), st))
        _lib.check(lib.prl_gated_delta_scan(R.aux.data_ptr(), ch, 0, gq, 2 * gq, P, ld, left + ch, left + ch + g.heads,
                                            vec[w + "mix.right.A_log"].data_ptr(), vec[w + "mix.right.dt_bias"].data_ptr(),
                                            g.unit_eps, g.heads, g.kv_heads, g.dim, g.vdim, n, R.dprep.data_ptr(), seg_start,
                                            seg_len, seg_slot, ns, max_q, self.delta_state[i].data_ptr(), R.o.data_ptr(), gv,
                                            st))
        _lib.check(lib.prl_gate_norm(R.o.data_ptr(), 1, gv, P + 4 * (left + ch + 2 * g.heads), ld,
                                     vec[w + "mix.right.norm"].data_ptr(), g.vdim, g.vdim, n, gv, 0, 0, 1, self.cfg.eps,
                                     R.yb.data_ptr(), f32, st))
        k1 = self._mm(R.yb, gv, w + "mix.right.o", W, R.y1, n, split=True)
        return k0, k1

    # ---- the multi-stream program: latent attention and delta-rule layers ------------------------------------------------
    def _stream_weights(self, i: int, q: str):
        """(read weights, write weights, mixing matrix) of sublayer q of run i; a layer without them sums plainly."""
        L = self.cfg.layers[i]
        if L.hyper:
            p = f"l{L.weights_of}.hc{q}."
            return self.vec[p + "in"], self.vec[p + "out"], self.vec[p + "mix"]
        return self.stream_ones, self.stream_ones, self.stream_eye

    def _tanh_norm(self, name: str):
        return self.vec[name + ".alpha"], self.vec[name], self.vec[name + ".b"]

    def _next_reader(self, i: int, after_mixer: bool):
        """(read weights, alpha, gain, shift) of whatever reads the streams after this sublayer of run i, or None at
        the end of the stack (the model's last norm gathers the wanted rows itself)."""
        L = self.cfg.layers[i]
        if after_mixer and L.mlp is not None:
            return (self._stream_weights(i, "2")[0], *self._tanh_norm(f"l{L.weights_of}.norm2"))
        if i + 1 < len(self.cfg.layers):
            return (self._stream_weights(i + 1, "1")[0], *self._tanh_norm(f"l{self.cfg.layers[i + 1].weights_of}.norm1"))
        return None

    def _stream_close(self, R, n, i, q, y, k, gate, ldg) -> None:
        """The sublayer's result (k slices [k][n][W]) back into the streams: layer scale, gate, stream update, and the
        next reader's normed input into R.xa (prl_streams_close)."""
        L, W = self.cfg.layers[i], self.cfg.width
        w = f"l{L.weights_of}."
        _, w_out, mix = self._stream_weights(i, q)
        nxt = self._next_reader(i, q == "1")
        ptr = lambda t: None if t is None else t.data_ptr()
        nx = [ptr(t) for t in nxt] if nxt is not None else [None] * 4
        _lib.check(self.lib.prl_streams_close(y.data_ptr(), W, k, n * W, ptr(self.vec.get(w + "ls" + q)) if L.layer_scale else None,
                                              gate, ldg, ptr(self.vec.get(f"{w}rg{q}.b")) if L.gated else None, mix.data_ptr(),
                                              w_out.data_ptr(), self.cfg.streams, n, W, R.xs.data_ptr(), *nx, R.xa.data_ptr(),
                                              int(self.f32), self._st))

    def _stream_layers(self, R, n, ns, max_q, row_pos, seg_pos0, trace=None) -> None:
        """Layer program of the "tanh" family.  On entry R.xa holds the first mixer's normed input (the embedding kernel
        wrote it); every closing kernel leaves the next sublayer's.  A sublayer's gate projection rides in its first GEMM
        (mixer) or is one more GEMM over the same input (feed-forward)."""
        cfg, W, S = self.cfg, self.cfg.width, self.cfg.streams
        segs = (R.seg[0].data_ptr(), R.seg[1].data_ptr(), R.seg[3].data_ptr(), ns)
        for i, L in enumerate(cfg.layers):
            w = f"l{L.weights_of}."
            if L.kind == "latent":
                y, k, gate, ldg = self._latent_mixer(R, n, i, L, w, segs, max_q, row_pos, seg_pos0)
            else:
                y, k, gate, ldg = self._delta_mixer(R, n, i, L, w, segs, max_q)
            self._stream_close(R, n, i, "1", y, k, gate, ldg)
            if L.mlp is not None:
                gate = None
                if L.gated:
                    self._mm(R.xa, W, w + "rg2", W, R.y1, n)
                    gate = R.y1.data_ptr()
                y = self._routed_ff(R, n, w, L.mlp.moe, L.mlp.beta)
                self._stream_close(R, n, i, "2", y, L.mlp.moe.top, gate, W)
            if trace is not None:
                trace.append(R.xs[:n * S * W].view(n, S, W).sum(1))

    def _latent_mixer(self, R, n, i, L, w, segs, max_q, row_pos, seg_pos0):
        """Latent attention with the key expansion absorbed into the query and the value expansion applied to the
        attention output, so that the cache holds one row [latent | rotated shared key part] per token and attention
        runs as one shared key head of size kv_rank + rot_dim whose values are the row's first kv_rank channels.
        Buffers: P = [dq | dkv | gate] (fp32); ya = the normed query latent, later the attention output (operand type);
        aux = W_uq cq (fp32); yb = the heads' unrotated query parts, later the expanded values (operand type); q = the
        attention query [n][H][kv_rank + rot_dim]; o = the absorbed query channels, later the expanded values (fp32)."""
        a, lib, st, vec, f32, W = L.latent, self.lib, self._st, self.vec, int(self.f32), self.cfg.width
        seg_start, seg_len, seg_slot, ns = segs
        H, rk, dr = a.heads, a.kv_rank, a.rot_dim
        kd = rk + dr
        ld = a.q_rank + kd + (W if L.gated else 0)
        P = R.P.data_ptr()
        self._mm(R.xa, W, w + "mix.in", ld, R.P, n)
        _lib.check(lib.prl_latent_prep(P, ld, 0, a.q_rank, a.q_rank, rk, dr, self.rot_freq[i].data_ptr(),
                                       vec[w + "mix.dq.norm"].data_ptr(), vec[w + "mix.dkv.norm"].data_ptr(), self.cfg.eps,
                                       row_pos.data_ptr(), R.row_slot.data_ptr(), self.block_table.data_ptr(), self.max_blocks,
                                       PAGE_SIZE, n, 0, R.ya.data_ptr(), self.lat_pool[i].data_ptr(), f32, st))
        hq = H * (a.dim + dr)
        self._mm(R.ya, a.q_rank, w + "mix.uq", hq, R.aux, n)
        _lib.check(lib.prl_latent_query(R.aux.data_ptr(), hq, n, H, a.dim, dr, rk, self.rot_freq[i].data_ptr(),
                                        row_pos.data_ptr(), 0, R.yb.data_ptr(), R.q.data_ptr(), f32, st))
        # q_lat[h] = W_uk,h^T q_h: per-head products over column blocks of the row buffers, into the attention query
        self._mm_heads(R.yb, a.dim, self.uk_t[L.weights_of].data_ptr(), rk * a.dim, n, rk, R.o, H, R.q, kd)
        sink = vec[w + "mix.sink"].data_ptr() if a.sink else None
        self._latent_attention(R, i, a, segs, max_q, seg_pos0, sink)
        # v[h] = W_uv,h o_lat[h], then the output projection over the concatenated heads
        self._mm_heads(R.ya, rk, self.arena.ptr(w + "mix.uv"), a.vdim * rk, n, a.vdim, R.o, H, R.yb, a.vdim)
        k0 = self._mm(R.yb, H * a.vdim, w + "mix.o", W, R.y0, n, split=True)
        return R.y0, k0, (P + 4 * (a.q_rank + kd)) if L.gated else None, ld

    def _latent_attention(self, R, i, a, segs, max_q, seg_pos0, sink=None) -> None:
        """Attention of the query R.q [n][H][kv_rank + rot_dim] over run i's latent cache, as ONE shared key head whose
        values are the rows' first kv_rank channels, into R.ya (operand type).  bf16 with sizes the tensor-core kernel
        is built for: the heads stacked into the M dimension of its products; else the any-geometry kernel."""
        lib, f32 = self.lib, int(self.f32)
        seg_start, seg_len, seg_slot, ns = segs
        H, rk, kd, pool = a.heads, a.kv_rank, a.kv_rank + a.rot_dim, self.lat_pool[i].data_ptr()
        if not self.f32 and not self.force_plain_attn and lib.prl_attn_latent_fits(kd, rk, PAGE_SIZE):
            _lib.check(lib.prl_attn_latent(R.q.data_ptr(), pool, self.block_table.data_ptr(), self.max_blocks, PAGE_SIZE,
                                           seg_start, seg_len, seg_pos0.data_ptr(), seg_slot, ns, max_q, H, kd, rk, a.scale,
                                           a.window, sink, R.ya.data_ptr(), self.attn_ws.data_ptr(), self.attn_ws.numel(),
                                           self._st))
        else:
            _lib.check(lib.prl_attn_any_sink(R.q.data_ptr(), pool, pool, kd, f32, self.block_table.data_ptr(), self.max_blocks,
                                             PAGE_SIZE, seg_start, seg_len, seg_pos0.data_ptr(), seg_slot, ns, max_q, H, 1, kd,
                                             rk, a.scale, a.window, 0, 0.0, sink, 1, R.ya.data_ptr(), self._st))

    def _head_table(self, n: int, heads: int):
        """Tile table of the grouped GEMM (csrc/moe_ops.cu) for per-head products over token-major buffers: the rows
        (token t, head h) = t * heads + h of a [n][heads][.] buffer, grouped by head.  Cached per (n, heads); built on
        the first use, which for the decode step is its eager run before the graph capture."""
        key = (n, heads)
        if key not in self._head_tables:
            i32 = dict(dtype=torch.int32, device=self.dev)
            perm = (torch.arange(n, dtype=torch.int32).view(1, n) * heads + torch.arange(heads, dtype=torch.int32).view(heads, 1)).reshape(-1)
            tiles = [(h, h * n + r0, min(64, n - r0)) for h in range(heads) for r0 in range(0, n, 64)]
            self._head_tables[key] = (perm.to(self.dev), torch.tensor([len(tiles), 0, 0, 0], **i32),
                                      torch.tensor(tiles, **i32).reshape(-1), len(tiles))
        return self._head_tables[key]

    def _mm_heads(self, src, K, w_ptr, w_step, n, N, tmp, heads, dst, dst_step, store: bool = True) -> None:
        """dst[t][h][:N] (operand type, rows dst_step apart) = src[t][h][:K] @ W_h[N, K]^T for every token t and head h
        (W_h = w_ptr + h * w_step elements, rows K apart): ONE grouped GEMM over the heads (tensor cores for bf16), the
        routed feed-forward's kernel with the head in the expert's place, into the fp32 buffer `tmp`, and a cast."""
        lib, st, f32 = self.lib, self._st, int(self.f32)
        perm, meta, tiles, n_tiles = self._head_table(n, heads)
        _lib.check(lib.prl_moe_gemm(src.data_ptr(), f32, K, n * heads, w_ptr, f32, w_step, K, perm.data_ptr(), meta.data_ptr(),
                                    tiles.data_ptr(), n_tiles, N, K, tmp.data_ptr(), N, 1, st))
        if store:                                        # else the caller consumes the fp32 rows [n][heads * N] in tmp
            _lib.check(lib.prl_store_groups(tmp.data_ptr(), heads * N, n, heads, N, dst.data_ptr(), dst_step, f32, st))

    def _delta_mixer(self, R, n, i, L, w, segs, max_q=0):
        """Delta-rule memory: one projection [r | k | v | g | a | w1 | gate]; the decay logits come through the tanh
        bottleneck in fp32; prl_delta_scan forms the unit key (into o2), decay and removal rate and walks the tokens."""
        c, lib, st, vec, f32, W = L.delta, self.lib, self._st, self.vec, int(self.f32), self.cfg.width
        seg_start, seg_len, seg_slot, ns = segs
        nq = c.heads * c.dim
        ld = 5 * nq + c.rank + (W if L.gated else 0)
        P = R.P.data_ptr()
        self._mm(R.xa, W, w + "mix.in", ld, R.P, n)
        _lib.check(lib.prl_act_cols(P, ld, 5 * nq, n, c.rank, 1, st))                 # tanh of the bottleneck
        _lib.check(lib.prl_gemm_any(P + 4 * 5 * nq, 1, ld, self.arena.ptr(w + "mix.w2"), f32, c.rank, n, nq, c.rank,
                                    R.aux.data_ptr(), nq, st))
        _lib.check(lib.prl_delta_scan(P, ld, 0, nq, 2 * nq, 4 * nq, R.aux.data_ptr(), nq, vec[w + "mix.w0"].data_ptr(),
                                      vec[w + "mix.a.b"].data_ptr(), c.decay_scale, c.unit_eps, c.heads, c.dim, c.dim, n,
                                      R.o2.data_ptr(), seg_start, seg_len, seg_slot, ns, max_q, self.delta_state[i].data_ptr(),
                                      R.o.data_ptr(), nq, st))
        _lib.check(lib.prl_gate_norm(R.o.data_ptr(), 1, nq, P + 4 * 3 * nq, ld, vec[w + "mix.norm"].data_ptr(), nq, c.dim, n,
                                     nq, 1, 0, 1, self.cfg.eps, R.ya.data_ptr(), f32, st))
        k0 = self._mm(R.ya, nq, w + "mix.o", W, R.y0, n, split=True)
        return R.y0, k0, (P + 4 * (5 * nq + c.rank)) if L.gated else None, ld

    def _embed(self, R, n, tokens, positions, ns=None) -> None:
        cfg, lib, st = self.cfg, self.lib, self._st
        if cfg.norm_kind == "tanh":
            # token (+ hashed token pair) embedding into every stream, and the first mixer's normed input
            pe = cfg.pair_embed
            w_in = self._stream_weights(0, "1")[0] if cfg.layers else self.stream_ones
            alpha, gain, shift = self._tanh_norm(f"l{cfg.layers[0].weights_of}.norm1" if cfg.layers else "final.norm")
            prev = self.prev_token.data_ptr() if pe else None
            _lib.check(lib.prl_embed_pair(tokens.data_ptr(), positions.data_ptr(), R.row_slot.data_ptr(), R.row_back.data_ptr(),
                                          prev, self.arena.ptr("embed"), self.arena.ptr("bigram") if pe else None, int(self.f32),
                                          cfg.embed_scale, *(pe or (0, 0, 0)), n, cfg.width, cfg.vocab_size, cfg.streams,
                                          w_in.data_ptr(), alpha.data_ptr(), gain.data_ptr(), shift.data_ptr(),
                                          R.xs.data_ptr(), R.xa.data_ptr(), st))
            if pe:
                _lib.check(lib.prl_last_token(tokens.data_ptr(), R.seg[0].data_ptr(), R.seg[1].data_ptr(), R.seg[3].data_ptr(),
                                              n if ns is None else ns, prev, st))
        elif cfg.positions == "sinusoid":
            x0a = R.x0a.data_ptr() if cfg.loop_times else None
            _lib.check(lib.prl_embed_sinusoid(tokens.data_ptr(), self.arena.ptr("embed"), int(self.f32), cfg.embed_scale,
                                              self.pos_freq.data_ptr(), positions.data_ptr(), n, cfg.width, cfg.vocab_size,
                                              R.x.data_ptr(), R.xa.data_ptr(), x0a, st))
        else:
            _lib.check(lib.prl_embed_scale(tokens.data_ptr(), self.arena.ptr("embed"), int(self.f32), cfg.embed_scale, n,
                                           cfg.width, cfg.vocab_size, R.x.data_ptr(), R.xa.data_ptr(), st))

    def _final_norm(self, R, rows, n_out) -> None:
        """R.xa[:n_out] = the model's last norm of the rows `rows` (None: the first n_out rows) of the residual."""
        cfg, lib, st = self.cfg, self.lib, self._st
        if cfg.norm_kind == "tanh":
            alpha, gain, shift = self._tanh_norm("final.norm")
            _lib.check(lib.prl_streams_open(R.xs.data_ptr(), rows, n_out, cfg.streams, cfg.width, self.stream_ones.data_ptr(),
                                            alpha.data_ptr(), gain.data_ptr(), shift.data_ptr(), R.xa.data_ptr(),
                                            int(self.f32), st))
        else:
            _lib.check(lib.prl_rmsnorm_rows(R.x.data_ptr(), rows, self.vec["final.norm"].data_ptr(), cfg.eps, n_out, cfg.width,
                                            R.xa.data_ptr(), int(self.f32), st))

    # ---- one token for every slot (captured into the engine's CUDA graph) ---------------------------------------------
    def _step_kernels(self) -> None:
        cfg, lib, R, B = self.cfg, self.lib, self._dec, self.B
        self._st = st = _lib.stream_ptr()
        _lib.check(lib.prl_decode_rows(self.active.data_ptr(), B, R.seg[1].data_ptr(), R.row_slot.data_ptr(), st))
        self._embed(R, B, self.tokens, self.positions)
        self._layers(R, B, B, 1, self.positions, self.positions, decode=True)
        self._final_norm(R, None, B)
        self._mm(R.xa, cfg.width, self.head_name, cfg.vocab_size, self.logits, B)

    # ---- a packed batch of prompt portions (prefill chunks, token streams) --------------------------------------------
    def _forward_rows(self, segs, want_rows, trace=None):
        cfg, lib = self.cfg, self.lib
        if self._rows is None:
            self._rows = _Rows(self, max(self.prefill_chunk, 1), pieces=True)
        R = self._rows
        n = sum(k for _, _, k in segs)
        if n > R.n:
            raise ValueError(f"{n} rows exceed the prefill chunk of {R.n}")
        toks, pos, slot, back, meta = [], [], [], [], [[], [], [], []]
        at = 0
        for req, s0, k in segs:
            toks += req.prompt_ids[s0:s0 + k]
            pos += range(s0, s0 + k)
            slot += [req.slot] * k
            back += range(k)
            meta[0].append(at); meta[1].append(k); meta[2].append(s0); meta[3].append(req.slot)
            at += k
        ns = len(segs)
        i32 = torch.int32
        R.n_sub = 0
        if self.split_scan and max(k for _, _, k in segs) >= self.split_min_rows:
            step = min(self.piece_tokens, int(lib.prl_lin_scan_piece_tokens()))
            sub, seg_sub = [[], []], [[], []]
            for start, k in zip(meta[0], meta[1]):
                seg_sub[0].append(len(sub[0]))
                seg_sub[1].append((k + step - 1) // step)
                sub[0] += range(start, start + k, step)
                sub[1] += [min(step, k - c) for c in range(0, k, step)]
            if len(sub[0]) <= R.max_sub:          # else: many short segments beside the long one, walk them token by token
                R.n_sub = len(sub[0])
                R.sub[:, :R.n_sub].copy_(torch.tensor(sub, dtype=i32), non_blocking=True)
                R.seg_sub[:, :ns].copy_(torch.tensor(seg_sub, dtype=i32), non_blocking=True)
        R.tokens[:n].copy_(torch.tensor(toks, dtype=i32), non_blocking=True)
        R.row_pos[:n].copy_(torch.tensor(pos, dtype=i32), non_blocking=True)
        R.row_slot[:n].copy_(torch.tensor(slot, dtype=i32), non_blocking=True)
        R.row_back[:n].copy_(torch.tensor(back, dtype=i32), non_blocking=True)
        R.seg[:, :ns].copy_(torch.tensor(meta, dtype=i32), non_blocking=True)
        self._st = st = _lib.stream_ptr()
        self._embed(R, n, R.tokens, R.row_pos, ns)
        self._layers(R, n, ns, max(k for _, _, k in segs), R.row_pos, R.seg[2], trace=trace)
        self.stats["prefill_tokens"] += n
        if not want_rows:
            return None
        nw = len(want_rows)
        R.want[:nw].copy_(torch.tensor(want_rows, dtype=i32), non_blocking=True)
        self._final_norm(R, R.want.data_ptr(), nw)
        out = torch.empty(nw, cfg.vocab_size, dtype=torch.float32, device=self.dev)
        self._mm(R.xa, cfg.width, self.head_name, cfg.vocab_size, out, nw)
        return out
