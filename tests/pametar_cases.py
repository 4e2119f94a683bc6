"""Small Pametar configurations and helpers for the tests (random weights, sizes chosen to be awkward)."""
import copy

import torch

from oracle import pametar_oracle as po
from tests.belelorn_cases import rel_err, stream_logits, tokens_for, write_checkpoint  # noqa: F401  (model-independent helpers)


def latent(heads=3, dim=12, rot_dim=6, vdim=20, kv_rank=24, q_rank=40, base=100.0, scale=None, mlp=None):
    return dict(type="latent_attention", mlp=mlp,
                mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank,
                           rot=dict(base=base, dims=rot_dim), scale=scale if scale is not None else (dim + rot_dim) ** -0.5))


def delta(heads=3, dim=10, rank=5, mlp=None):
    return dict(type="general_delta", mixer=dict(heads=heads, dim=dim, rank=rank), mlp=mlp)


def moe(experts=5, top=2, ff=24, scale=1.5):
    return dict(kind="moe", router=dict(experts=experts, top=top, scale=scale), expert=dict(ff=ff))


def model(layers, vocab=96, width=72, eps=1e-5, loop=None, streams=2, embed_scale=3.0, pair=(53, 11, 5)):
    emb = dict(scale=embed_scale)
    if pair is not None:
        emb["bigram"] = dict(buckets=pair[0], mul_prev=pair[1], mul_cur=pair[2])
    cfg = dict(architecture="Pametar", vocab=vocab, width=width, norm=dict(eps=eps), streams=streams, embedding=emb,
               layers=copy.deepcopy(layers))
    if loop is not None:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return cfg


def weights(config, seed=0, **parts):
    return po.random_weights(config, seed, **parts)


def build_engine(config, wt, dtype, device, **kw):
    from pipelinerl_b200.hybrid import HybridConfig, HybridEngine
    from pipelinerl_b200.model import ParamArena
    cfg = HybridConfig.from_pametar(config, {k: tuple(v.shape) for k, v in wt.items()})
    arena = ParamArena(cfg, device, dtype=dtype)
    arena.load_hf_state_dict(wt)
    args = dict(max_batch=4, max_seq_len=512, max_new_tokens=32, prefill_chunk=256, use_cuda_graph=False, device=device)
    args.update(kw)
    return HybridEngine(cfg, arena, **args)


def oracle_logits(config, wt, tokens, **kw):
    return po.forward(tokens, wt, config, **kw)


def stage_stream(eng, tokens):
    """A stream holding `tokens` with its pages in the block table, for a direct call of the engine's row program."""
    s = eng.open_stream()
    s.prompt_ids.extend(tokens)
    need = -(-len(tokens) // 64)
    s.pages += eng._alloc_pages(need)
    eng.block_table[s.slot, :need].copy_(torch.tensor(s.pages, dtype=torch.int32))
    return s


def bf16_round(x):
    return x.to(torch.bfloat16).to(torch.float64)
