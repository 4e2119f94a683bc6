"""Small Kolotar configurations and helpers for the tests (random weights, sizes chosen to be awkward)."""
import copy

import torch

from oracle import kolotar_oracle as ko
from tests.belelorn_cases import rel_err, stream_logits, tokens_for, write_checkpoint  # noqa: F401  (model-independent helpers)
from tests.pametar_cases import bf16_round, stage_stream  # noqa: F401


def attention(heads=6, kv_heads=3, dim=12, vdim=10, window=40, rot_dims=8, base=50.0, scaling=(3.0, 64, 8.0, 1.0), v_mix=True,
              scale=None, mlp=None):
    rot = dict(base=base, dims=rot_dims)
    if scaling is not None:
        rot["scaling"] = dict(factor=scaling[0], original=scaling[1], fast=scaling[2], slow=scaling[3])
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot=rot, scale=scale if scale is not None else dim ** -0.5,
             v_mix=v_mix)
    if window:
        m["mask"] = dict(size=window)
    return dict(type="attention", mixer=m, mlp=mlp)


def latent(heads=3, dim=12, rot_dim=6, vdim=20, kv_rank=24, base=100.0, window=50, scale=None, mlp=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, rot=dict(base=base, dims=rot_dim),
             scale=scale if scale is not None else (dim + rot_dim) ** -0.5)
    if window:
        m["mask"] = dict(size=window)
    return dict(type="latent_attention", mixer=m, mlp=mlp)


def parallel(heads=4, kv_heads=2, dim=10, vdim=12, softcap=20.0, q_temp=(0.5, 16), scale=None, r_heads=4, r_kv_heads=2, r_dim=12,
             r_vdim=8, conv=3, left_scale=0.7, right_scale=0.6, mlp=None):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, softcap=softcap, scale=scale if scale is not None else dim ** -0.5)
    if q_temp is not None:
        left["q_temp"] = dict(coef=q_temp[0], every=q_temp[1])
    right = dict(heads=r_heads, kv_heads=r_kv_heads, dim=r_dim, vdim=r_vdim, conv=conv)
    return dict(type="parallel", mixer=dict(left=left, right=right, left_scale=left_scale, right_scale=right_scale), mlp=mlp)


def moe(experts=5, top=2, ff=24):
    return dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff))


def model(layers, vocab=96, width=72, eps=1e-5, alpha=2.5):
    return dict(architecture="Kolotar", vocab=vocab, width=width, norm=dict(eps=eps), postln_alpha=alpha,
                layers=copy.deepcopy(layers))


def weights(config, seed=0):
    return ko.random_weights(config, seed)


def build_engine(config, wt, dtype, device, **kw):
    from pipelinerl_b200.hybrid import HybridConfig, HybridEngine
    from pipelinerl_b200.model import ParamArena
    cfg = HybridConfig.from_kolotar(config, {k: tuple(v.shape) for k, v in wt.items()})
    arena = ParamArena(cfg, device, dtype=dtype)
    arena.load_hf_state_dict(wt)
    args = dict(max_batch=4, max_seq_len=512, max_new_tokens=32, prefill_chunk=256, use_cuda_graph=False, device=device)
    args.update(kw)
    return HybridEngine(cfg, arena, **args)


def oracle_logits(config, wt, tokens, **kw):
    return ko.forward(config, wt, tokens, **kw)[0]


def oracle_layers(config, wt, tokens):
    return ko.forward(config, wt, tokens)[1]
