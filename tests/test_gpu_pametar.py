"""The Pametar decoders on the hybrid engine (pipelinerl_b200/hybrid.py and its kernels) against
oracle/pametar_oracle.py: each mechanism alone, whole prompts against token-by-token decoding, portions down to two
tokens, unequal batches against each request alone, pages and slots that are given back and taken again, keys far away
and at page borders made to stand out, the sink logit, far tokens in the delta-rule memory, the first tokens (the
token-pair table's extra row), long decoding, awkward sizes, the bf16 serving mode, greedy generation through the
engine's scheduler, and the trace runner."""
import copy
import json
import subprocess
import sys

import pytest
import torch

from oracle import pametar_oracle as po
from tests import pametar_cases as pc

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4      # fp32 kernels against the float64 oracle
BF16_TOL = 8e-2     # bf16 operands / cache: rounding of activations dominates


# ---- each mechanism alone ---------------------------------------------------------------------------------------
def _mechanisms():
    L, D, M = pc.latent, pc.delta, pc.moe
    return {
        "latent_attention": (pc.model([L()]), {}),
        "latent_one_head_wide_rotation": (pc.model([L(heads=1, dim=5, rot_dim=14, vdim=9, kv_rank=11, q_rank=7, base=7.0)]), {}),
        "latent_two_rotated_channels": (pc.model([L(heads=5, dim=16, rot_dim=2, vdim=8, kv_rank=40, q_rank=24)]), {}),
        "latent_without_sink": (pc.model([L()]), dict(sink=False)),
        "delta_rule": (pc.model([D()]), {}),
        "delta_one_head_rank_one": (pc.model([D(heads=1, dim=33, rank=1)]), {}),
        "delta_many_small_heads": (pc.model([D(heads=7, dim=4, rank=9)]), {}),
        "delta_wide_heads": (pc.model([D(heads=1, dim=128, rank=3), D(heads=1, dim=200, rank=2)], width=56), {}),
        "latent_wide_latent": (pc.model([L(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=300, q_rank=16)], width=48), {}),
        "odd_width_six_streams": (pc.model([L(mlp=M()), D(mlp=M(experts=2, top=1, ff=7))], vocab=61, width=50, streams=6), {}),
        "one_stream": (pc.model([L(mlp=M()), D()], streams=1), {}),
        "one_stream_plain_residual": (pc.model([D(mlp=M()), L()], streams=1), dict(hyper=False)),
        "four_streams": (pc.model([L(), D(mlp=M())], streams=4), {}),
        "no_layer_scale_no_gate": (pc.model([L(mlp=M()), D(mlp=M())]), dict(layer_scale=False, gated=False)),
        "no_pair_table": (pc.model([D(), L()], pair=None), {}),
        "pair_table_one_bucket": (pc.model([L()], pair=(1, 3, 2)), {}),
        "routed_top2": (pc.model([D(mlp=M())]), {}),
        "routed_top1_of_seven": (pc.model([L(mlp=M(experts=7, top=1, ff=10, scale=0.5))]), {}),
        "routed_all_experts": (pc.model([D(mlp=M(experts=3, top=3, ff=9, scale=1.0))]), {}),
        "repeated_block": (pc.model([L(mlp=M()), D(mlp=M(experts=4, top=3, ff=8))], loop=(0, 2, 3), streams=3), {}),
        "repeated_block_inside_once": (pc.model([D(), L(mlp=M()), D(mlp=M())], loop=(1, 2, 1)), {}),
        "repeated_single_layer": (pc.model([L(), D(mlp=M()), L(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=16, q_rank=16)],
                                           loop=(1, 2, 2)), {}),
    }


@pytest.mark.parametrize("name", sorted(_mechanisms()))
def test_each_mechanism_matches_the_oracle_fp32(cuda_device, name):
    config, parts = _mechanisms()[name]
    wt = pc.weights(config, seed=len(name), **parts)
    toks = pc.tokens_for(config, 150)
    ref = pc.oracle_logits(config, wt, toks)
    eng = pc.build_engine(config, wt, torch.float32, cuda_device)
    assert pc.rel_err(pc.stream_logits(eng, toks, [150]), ref) < F32_TOL
    assert pc.rel_err(pc.stream_logits(eng, toks, [2, 3, 61, 2, 7, 64, 2]), ref) < F32_TOL     # then one by one
    # the sum of the residual streams after every layer run of a whole prompt
    res = []
    pc.oracle_logits(config, wt, toks[:20], trace=res)
    s = pc.stage_stream(eng, toks[:20])
    got = []
    eng._forward_rows([(s, 0, 20)], [], trace=got)
    eng.close_stream(s)
    assert len(got) == len(res)
    for a, b in zip(got, res):
        assert (a.double().cpu() - b).abs().max().item() < 1e-4 * max(1.0, b.abs().max().item())


FULL = pc.model([pc.latent(mlp=pc.moe()), pc.delta(mlp=pc.moe(experts=6, top=3, ff=16, scale=2.0)),
                 pc.latent(heads=2, dim=16, rot_dim=8, vdim=12, kv_rank=32, q_rank=16), pc.delta(heads=2, dim=16, rank=3, mlp=pc.moe())],
                vocab=80, width=64, loop=(1, 3, 2), streams=3)


def test_prefill_against_token_by_token_decoding(cuda_device):
    wt = pc.weights(FULL, 3)
    toks = pc.tokens_for(FULL, 140, seed=5)
    ref = pc.oracle_logits(FULL, wt, toks)
    eng = pc.build_engine(FULL, wt, torch.float32, cuda_device)
    whole = pc.stream_logits(eng, toks, [140])
    single = pc.stream_logits(eng, toks, [])                                 # every token alone, through the cache / state
    assert pc.rel_err(whole, ref) < F32_TOL and pc.rel_err(single, ref) < F32_TOL
    assert pc.rel_err(whole, single) < 2e-5


@pytest.mark.parametrize("portions", [[2] * 40, [63, 2, 63, 2], [64, 64], [1, 65, 1, 2, 59], [129, 2]])
def test_portions_of_several_sizes(cuda_device, portions):
    wt = pc.weights(FULL, 4)
    toks = pc.tokens_for(FULL, 140, seed=6)
    ref = pc.oracle_logits(FULL, wt, toks)
    eng = pc.build_engine(FULL, wt, torch.float32, cuda_device, prefill_chunk=96)   # 129 is cut by the engine too
    assert pc.rel_err(pc.stream_logits(eng, toks, portions), ref) < F32_TOL


def test_unequal_batches_equal_each_request_alone(cuda_device):
    wt = pc.weights(FULL, 7)
    seqs = [pc.tokens_for(FULL, n, seed=10 + n) for n in (1, 37, 130, 66)]
    eng = pc.build_engine(FULL, wt, torch.float32, cuda_device)
    alone = [pc.stream_logits(eng, s, [len(s)]) for s in seqs]
    # together: every step brings a different mix of portion sizes; request 0 joins late, request 2 skips a step
    streams = [eng.open_stream() for _ in seqs]
    got = [[] for _ in seqs]
    at = [0] * len(seqs)
    plan = [{1: 5, 2: 64}, {0: 1, 1: 1, 2: 2, 3: 30}, {1: 31, 3: 36}, {2: 64, 3: 0}]
    for step in plan:
        entries, who = [], []
        for i, k in step.items():
            if k:
                entries.append((streams[i], seqs[i][at[i]:at[i] + k], list(range(k))))
                who.append((i, k))
                at[i] += k
        lg = eng.feed(entries).double().cpu()
        r = 0
        for i, k in who:
            got[i].append(lg[r:r + k])
            r += k
    assert at == [len(s) for s in seqs]
    for i, s in enumerate(streams):
        eng.close_stream(s)
        assert pc.rel_err(torch.cat(got[i]), alone[i]) < 2e-5, f"request {i} depends on its batch"
    assert pc.rel_err(alone[2], pc.oracle_logits(FULL, wt, seqs[2])) < F32_TOL


def test_pages_and_slots_are_reused(cuda_device):
    """Two slots and five pages for eight sequences: every later sequence runs in a slot whose delta-rule memories and
    previous token another one left, and on pages that held other latents."""
    wt = pc.weights(FULL, 8)
    eng = pc.build_engine(FULL, wt, torch.float32, cuda_device, max_batch=2, max_seq_len=192, n_pages=1 + 5)
    lens = [100, 70, 5, 128, 64, 1, 150, 65]
    for k, n in enumerate(lens):
        toks = pc.tokens_for(FULL, n, seed=40 + k)
        ref = pc.oracle_logits(FULL, wt, toks)
        held = eng.open_stream()
        eng.feed([(held, pc.tokens_for(FULL, 60 + k, seed=k), [])])          # a neighbour that dirties the other slot
        got = pc.stream_logits(eng, toks, [max(1, n // 2), 2])
        eng.close_stream(held)
        assert pc.rel_err(got, ref) < F32_TOL, f"sequence {k}"
        assert len(eng.free_pages) == 5 and len(eng.free_slots) == 2


# ---- keys made to stand out -------------------------------------------------------------------------------------------
def _standout(far_tok, ask_tok, sink=0.0, strength=6.0):
    """One latent-attention layer, no pair table, in which head 0 of every `ask_tok` query puts nearly all its weight on
    the key of `far_tok`, wherever that token sits: channel 0 of head 0's key expansion is aligned with far_tok's latent
    and channel 0 of its query expansion with ask_tok's query latent (a token's latents depend on the token alone
    here).  Head 0's value then decides the logits, so a far key that is lost, shifted or read from a wrong page, and a
    sink that is left out of the denominator, change them by O(1)."""
    config = pc.model([pc.latent(heads=2, dim=8, rot_dim=4, vdim=12, kv_rank=16, q_rank=12, scale=1.0)], vocab=48, width=40,
                      streams=2, pair=None)
    wt = pc.weights(config, 19)
    m, eps = config["layers"][0]["mixer"], config["norm"]["eps"]

    def latents(tok):
        x = po.embed([tok], wt, config)
        h = po.tanh_norm(sum(wt["l0.hc1.in"]) * x, wt, "l0.norm1")
        cq = po.rms_unit(h @ wt["l0.mix.dq"].T, eps) * wt["l0.mix.dq.norm"]
        c = po.rms_unit((h @ wt["l0.mix.dkv"].T)[:, :m["kv_rank"]], eps) * wt["l0.mix.dkv.norm"]
        return cq[0], c[0]
    cq, _ = latents(ask_tok)
    _, c = latents(far_tok)
    wt["l0.mix.uk"][0] = pc.bf16_round(strength * c / c.pow(2).sum())          # k[head 0][0] = strength for far_tok
    wt["l0.mix.uq"][0] = pc.bf16_round(strength * cq / cq.pow(2).sum())        # q[head 0][0] = strength for ask_tok
    wt["l0.mix.sink"] = torch.tensor([sink, -2.0], dtype=torch.float64)
    return config, wt


@pytest.mark.parametrize("far_at", [0, 5, 63, 64, 191])
def test_a_far_key_among_hundreds_and_the_sink(cuda_device, far_at):
    """330 tokens over five page borders; the key that matters sits at the very start, in the middle of a page or on
    either side of a page border, and is asked for from prompt portions and from single decoded tokens hundreds of
    positions later.  The sink logit is as large as the standing-out score, so it halves head 0's weights."""
    far_tok, ask_tok = 7, 11
    config, wt = _standout(far_tok, ask_tok, sink=36.0)
    toks = [t if t not in (far_tok, ask_tok) else 13 for t in pc.tokens_for(config, 330, seed=3)]
    toks[far_at] = far_tok
    for p in (far_at + 1, 200, 255, 256, 300, 329):
        if p > far_at:
            toks[p] = ask_tok
    asks = [p for p in range(330) if toks[p] == ask_tok]
    ref = pc.oracle_logits(config, wt, toks)
    # sharpness: without the far token, and without the sink, the asking positions are far outside the tolerance
    gone = list(toks)
    gone[far_at] = 13
    assert pc.rel_err(pc.oracle_logits(config, wt, gone)[asks], ref[asks]) > 100 * F32_TOL
    no_sink = dict(wt)
    no_sink["l0.mix.sink"] = torch.tensor([-1e4, -1e4], dtype=torch.float64)
    assert pc.rel_err(pc.oracle_logits(config, no_sink, toks)[asks], ref[asks]) > 100 * F32_TOL
    eng = pc.build_engine(config, wt, torch.float32, cuda_device)
    for portions in ([330], [63, 1, 1, 63, 2, 126], [64, 64, 64, 64], [199, 2, 54, 2], [250]):      # the rest one by one
        assert pc.rel_err(pc.stream_logits(eng, toks, portions), ref) < F32_TOL
    eng16 = pc.build_engine(config, wt, torch.bfloat16, cuda_device)
    assert pc.rel_err(pc.stream_logits(eng16, toks, [199, 2, 54, 2]), ref) < BF16_TOL


def test_rotation_follows_the_position(cuda_device):
    """Rotated channels only (two unrotated ones with their expansion silenced) and a fast rotation: a key or query turned
    by a neighbouring position's angle, in a portion or a decoded token, moves the scores by O(1)."""
    config = pc.model([pc.latent(heads=2, dim=2, rot_dim=12, vdim=10, kv_rank=12, q_rank=12, base=3.0, scale=1.5)], width=40)
    wt = pc.weights(config, 23)
    wt["l0.mix.uk"] = torch.zeros_like(wt["l0.mix.uk"])
    toks = pc.tokens_for(config, 200, seed=2)
    ref = pc.oracle_logits(config, wt, toks)
    other = copy.deepcopy(config)
    other["layers"][0]["mixer"]["rot"]["base"] = 3.3
    assert pc.rel_err(pc.oracle_logits(other, wt, toks), ref) > 100 * F32_TOL
    eng = pc.build_engine(config, wt, torch.float32, cuda_device)
    for portions in ([200], [1, 2, 62, 3, 64], [130]):
        assert pc.rel_err(pc.stream_logits(eng, toks, portions), ref) < F32_TOL


def test_far_tokens_in_the_delta_rule_memory(cuda_device):
    """Decays close to 1 and removal rates close to 0: the memory at token 300 still holds the first tokens, so a state
    that is lost, reset or not carried across portions shows at every later position.  A second model with strong decay
    and removal exercises both corrections."""
    config = pc.model([pc.delta(heads=2, dim=12, rank=4), pc.delta(heads=1, dim=20, rank=2)], streams=2)
    for shift_w, shift_a, far in ((-9.0, -5.0, True), (3.0, 4.0, False)):
        wt = pc.weights(config, 11)
        for i in (0, 1):
            wt[f"l{i}.mix.w0"] = pc.bf16_round(wt[f"l{i}.mix.w0"] + shift_w)
            wt[f"l{i}.mix.a.b"] = pc.bf16_round(wt[f"l{i}.mix.a.b"] + shift_a)
        toks = pc.tokens_for(config, 300, seed=4)
        ref = pc.oracle_logits(config, wt, toks)
        if far:
            other = [(toks[0] + 1) % config["vocab"]] + toks[1:]
            assert pc.rel_err(pc.oracle_logits(config, wt, other)[250:], ref[250:]) > 50 * F32_TOL   # token 0 still matters
        eng = pc.build_engine(config, wt, torch.float32, cuda_device)
        assert pc.rel_err(pc.stream_logits(eng, toks, [300]), ref) < F32_TOL
        assert pc.rel_err(pc.stream_logits(eng, toks, [7, 2, 120, 2, 9]), ref) < F32_TOL      # then 160 single tokens


def test_first_tokens_and_one_token_sequences(cuda_device):
    """The first token takes the pair table's extra row, the second one the first real pair; a portion that starts at
    token 1, 2 or 3 reads its previous token from the sequence's state."""
    wt = pc.weights(FULL, 12)
    eng = pc.build_engine(FULL, wt, torch.float32, cuda_device)
    for n in (1, 2, 3, 4):
        toks = pc.tokens_for(FULL, n, seed=70 + n)
        ref = pc.oracle_logits(FULL, wt, toks)
        assert pc.rel_err(pc.stream_logits(eng, toks, [n]), ref) < F32_TOL
        assert pc.rel_err(pc.stream_logits(eng, toks, []), ref) < F32_TOL
    # sharpness: the extra row is not row 0 and not "no pair": the oracle on a shifted table differs
    toks = pc.tokens_for(FULL, 3, seed=1)
    moved = dict(wt)
    moved["bigram"] = torch.roll(wt["bigram"], 1, 0)
    assert pc.rel_err(pc.oracle_logits(FULL, moved, toks), pc.oracle_logits(FULL, wt, toks)) > 100 * F32_TOL


def test_routing_follows_the_scores(cuda_device):
    """Router rows scaled so that the choice is never a close call, eleven experts of which three are taken: a wrong
    expert, weights renormalised over the taken ones or a forgotten constant shows at once."""
    config = pc.model([pc.delta(mlp=pc.moe(experts=11, top=3, ff=12, scale=2.5))], width=40)
    wt = pc.weights(config, 17)
    wt["l0.mlp.router"] = pc.bf16_round(wt["l0.mlp.router"] * 3.0)
    toks = pc.tokens_for(config, 120, seed=4)
    ref = pc.oracle_logits(config, wt, toks)
    other = copy.deepcopy(config)
    other["layers"][0]["mlp"]["router"]["scale"] = 2.0
    assert pc.rel_err(pc.oracle_logits(other, wt, toks), ref) > 50 * F32_TOL
    eng = pc.build_engine(config, wt, torch.float32, cuda_device)
    assert pc.rel_err(pc.stream_logits(eng, toks, [100, 2]), ref) < F32_TOL


BIG = pc.model([pc.latent(heads=4, dim=32, rot_dim=16, vdim=48, kv_rank=64, q_rank=96, mlp=pc.moe(experts=3, top=3, ff=64)),
                pc.delta(heads=2, dim=64, rank=8, mlp=pc.moe(experts=4, top=2, ff=96))], vocab=200, width=128, loop=(0, 1, 2), streams=3)


@pytest.mark.parametrize("plain_gemm", [False, True])
def test_bf16_serving_mode(cuda_device, plain_gemm):
    """bf16 operands and cache with the tensor-core GEMMs (and with the CUDA-core GEMM) against the float64 oracle.  Only
    the last layer run's router has a choice to make (the earlier ones take all their experts), so a token whose last-taken
    and first-left-out router logits are closer than bf16 rounding can tell apart touches only its own logits; the oracle
    reports the gaps and those positions are left out."""
    wt = pc.weights(BIG, 13)
    toks = pc.tokens_for(BIG, 300, seed=8)
    gaps = []
    ref = pc.oracle_logits(BIG, wt, toks, margins=gaps)
    assert len(gaps) == 3 and min(gaps[0] + gaps[1]) == float("inf")
    clear = torch.tensor(gaps[-1]) > 0.1
    assert clear.float().mean().item() > 0.8
    eng = pc.build_engine(BIG, wt, torch.bfloat16, cuda_device, prefill_chunk=512)
    eng.force_plain_gemm = plain_gemm
    whole = pc.stream_logits(eng, toks, [300])
    assert pc.rel_err(whole[clear], ref[clear]) < BF16_TOL
    assert pc.rel_err(pc.stream_logits(eng, toks, [100, 2, 30])[clear], ref[clear]) < BF16_TOL
    # the bf16 engine is about as close to the oracle as the oracle with only its matrix products' inputs rounded
    least = pc.rel_err(pc.oracle_logits(BIG, wt, toks, round_in=pc.bf16_round)[clear], ref[clear])
    assert pc.rel_err(whole[clear], ref[clear]) < 3 * least + 1e-3


@pytest.mark.parametrize("heads,dim,rot_dim,vdim,kv_rank", [(6, 16, 16, 24, 32), (16, 32, 32, 32, 128), (3, 8, 48, 8, 16), (20, 16, 16, 16, 240)])
def test_tensor_core_latent_attention(cuda_device, heads, dim, rot_dim, vdim, kv_rank):
    """bf16 with latent and rotated sizes that are multiples of 16: the heads of a token are stacked into the rows of
    mma.sync products over the shared key rows (a tile of sixteen stacked rows may span several tokens or a part of
    one), for prompt portions and for single decoded tokens.  Peaked scores and strong sinks, 330 tokens over five page
    borders; against the CUDA-core kernel on the same cache (they differ by the bf16 rounding of the softmax weights)
    and against the oracle."""
    config = pc.model([pc.latent(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=32, scale=0.6)], width=64)
    wt = pc.weights(config, 9)
    wt["l0.mix.sink"] = pc.bf16_round(wt["l0.mix.sink"] * 3.0 + 4.0)
    toks = pc.tokens_for(config, 330, seed=3)
    ref = pc.oracle_logits(config, wt, toks)
    eng = pc.build_engine(config, wt, torch.bfloat16, cuda_device, prefill_chunk=512)
    assert eng.lib.prl_attn_latent_fits(kv_rank + rot_dim, kv_rank, 64)
    plans = ([330], [63, 17, 16, 130, 65, 20, 3, 2], [300])                 # the rest one by one: the decode-shaped kernel
    fast = [pc.stream_logits(eng, toks, p) for p in plans]
    eng.force_plain_attn = True
    plain = [pc.stream_logits(eng, toks, p) for p in plans]
    for f, p in zip(fast, plain):
        assert pc.rel_err(f, p) < 0.25 * BF16_TOL
        assert pc.rel_err(f, ref) < BF16_TOL and pc.rel_err(p, ref) < BF16_TOL
    # a mixed batch: a portion beside single tokens of other sequences
    eng.force_plain_attn = False
    a, b, c = eng.open_stream(), eng.open_stream(), eng.open_stream()
    eng.feed([(b, toks[:70], []), (c, toks[:129], [])])
    got = eng.feed([(a, toks[:100], list(range(100))), (b, toks[70:71], [0]), (c, toks[129:130], [0])]).double().cpu()
    assert pc.rel_err(got[:100], ref[:100]) < BF16_TOL and pc.rel_err(got[100:101], ref[70:71]) < BF16_TOL
    assert pc.rel_err(got[101:], ref[129:130]) < BF16_TOL
    for s in (a, b, c):
        eng.close_stream(s)


def test_long_decoding(cuda_device):
    """A short prompt and 400 single tokens over six page borders, in fp32 against the oracle."""
    config = pc.model([pc.latent(mlp=pc.moe()), pc.delta()], loop=(0, 2, 2), streams=2)
    wt = pc.weights(config, 31)
    toks = pc.tokens_for(config, 420, seed=12)
    eng = pc.build_engine(config, wt, torch.float32, cuda_device)
    assert pc.rel_err(pc.stream_logits(eng, toks, [20]), pc.oracle_logits(config, wt, toks)) < F32_TOL


def test_greedy_generation_through_the_scheduler(cuda_device):
    """add_request / run_prefill / CUDA-graph token steps / harvest, five prompts on two slots (slots and pages are
    reused, idle slots ride along in the step), greedy ids against the oracle wherever its top-2 margin is not a
    rounding matter."""
    from pipelinerl_b200.engine import SamplingParams
    wt = pc.weights(FULL, 14)
    eng = pc.build_engine(FULL, wt, torch.float32, cuda_device, max_batch=2, max_seq_len=256, use_cuda_graph=True,
                          prefill_chunk=64)
    prompts = [pc.tokens_for(FULL, n, seed=90 + n) for n in (1, 5, 70, 130, 64)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=6, greedy=True, ignore_eos=True))
    assert len(eng.free_slots) == 2 and len(eng.free_pages) == eng.n_pages - 1
    for p, r in zip(prompts, outs):
        assert len(r.output_ids) == 6 and r.finish_reason == "length"
        seq = list(p)
        for tok, lp in zip(r.output_ids, r.output_logprobs):
            lg = pc.oracle_logits(FULL, wt, seq)[-1]
            top = torch.topk(lg, 2)
            if (top.values[0] - top.values[1]).item() > 1e-3:
                assert tok == top.indices[0].item()
            assert abs(lp - torch.log_softmax(lg, -1)[tok].item()) < 1e-3
            seq.append(tok)


def test_trace_runner_command_line(cuda_device, tmp_path):
    """bin/trace_run on a checkpoint folder: registry, safetensors loader, streams, output files, in both dtypes."""
    config = pc.model([pc.latent(mlp=pc.moe(experts=4, top=1, ff=8)), pc.delta(mlp=pc.moe(experts=3, top=2, ff=24))],
                      vocab=64, width=40, loop=(0, 1, 2), streams=2)
    wt = pc.weights(config, 15)
    pc.write_checkpoint(tmp_path, config, wt)
    a, b = pc.tokens_for(config, 90, seed=1), pc.tokens_for(config, 20, seed=2)
    steps = [
        dict(step=0, entries=[dict(id="a", tokens=a[:50], want=[0, 49])], end=[]),
        dict(step=1, entries=[dict(id="a", tokens=a[50:52], want=[]), dict(id="b", tokens=b[:19], want=[3])], end=[]),
        dict(step=2, entries=[dict(id="b", tokens=b[19:], want=[0]), dict(id="a", tokens=a[52:], want=[37])], end=["a", "b"]),
        dict(step=3, entries=[dict(id="c", tokens=b, want=[19])], end=["c"]),
    ]
    ra, rb = pc.oracle_logits(config, wt, a), pc.oracle_logits(config, wt, b)
    expect = {0: torch.stack([ra[0], ra[49]]), 1: rb[3:4], 2: torch.stack([rb[19], ra[89]]), 3: rb[19:20]}
    root = __import__("pathlib").Path(__file__).resolve().parent.parent
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        out = tmp_path / dtype
        p = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(tmp_path), "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=900)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(4)]
        import numpy as np
        for i, ref in expect.items():
            got = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4")).view(-1, config["vocab"])
            assert got.shape == ref.shape and pc.rel_err(got, ref) < tol
